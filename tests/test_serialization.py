import io
import struct

import pytest
import torch

import tensorplay_b200 as tp
from tensorplay_b200 import serialization as S


def _state():
    torch.manual_seed(0)
    return {"w": torch.randn(17, 5), "b": torch.arange(7, dtype=torch.int64), "h": torch.randn(3, 4).to(torch.bfloat16),
            "e": torch.empty(0, 3), "s": torch.tensor(3.5), "m": torch.tensor([True, False])}


def test_mega_roundtrip_flat_and_header_bytes(tmp_path):
    st = _state()
    p = tmp_path / "a.mega"
    tp.save(st, p)
    raw = p.read_bytes()
    magic, version, nt, nm = struct.unpack("<IIQQ", raw[:24])
    assert magic == 0x4147454D and version == 1 and nt == len(st) and nm >= 8
    doc = S.parse_mega(p)
    assert doc["data_start"] % 4096 == 0
    assert doc["metadata"]["tensorplay.container"] == "dict"
    # dims are stored reversed on disk but reported in logical order
    rec = {r["name"]: r for r in doc["tensors"]}
    assert rec["w"]["shape"] == [17, 5] and rec["w"]["dtype"] == "F32" and rec["h"]["dtype"] == "BF16"
    out = tp.load(p, verify_checksums=True)
    for k in st:
        assert out[k].dtype == st[k].dtype and torch.equal(out[k], st[k]), k
    info = tp.inspect_checkpoint(p)
    assert info["format"] == "mega" and info["tensors"]["b"]["shape"] == [7]


def test_mega_nested_tree_and_mmap(tmp_path):
    obj = {"model": {"l1": torch.ones(2, 2), "l2": [torch.zeros(3), (torch.ones(1), 5)]}, "step": 7, "name": "x",
           3: torch.ones(2)}
    p = tmp_path / "t.mega"
    tp.save(obj, p, checksum="sha256")
    out = tp.load(p, mmap=True, verify_checksums=True)
    assert out["step"] == 7 and out["name"] == "x"
    assert isinstance(out["model"]["l2"][1], tuple) and out["model"]["l2"][1][1] == 5
    assert torch.equal(out["model"]["l1"], torch.ones(2, 2)) and torch.equal(out[3], torch.ones(2))


def test_mega_checksum_detects_corruption(tmp_path):
    p = tmp_path / "c.mega"
    tp.save({"w": torch.arange(1000, dtype=torch.float32)}, p)
    raw = bytearray(p.read_bytes())
    raw[-5] ^= 0xFF
    p.write_bytes(bytes(raw))
    with pytest.raises(ValueError):
        tp.load(p, verify_checksums=True)


def test_crc32_matches_zlib():
    import zlib
    from tensorplay_b200.serialization.mega import _rt
    data = torch.randint(0, 255, (100003,), dtype=torch.uint8)
    assert _rt().tpb_crc32(data.data_ptr(), data.numel(), 0) == (zlib.crc32(data.numpy().tobytes()) & 0xFFFFFFFF)


def test_zip_and_safetensors_and_sniff(tmp_path):
    st = {k: v for k, v in _state().items() if k != "e"}
    pz, ps = tmp_path / "a.pt", tmp_path / "a.safetensors"
    tp.save(st, pz)
    tp.save(st, ps, metadata={"who": "test"})
    assert S.sniff_format(pz) == "zip" and S.sniff_format(ps) == "safetensors"
    assert torch.equal(torch.load(pz)["w"], st["w"])  # a torch-loadable archive
    for p in (pz, ps):
        out = tp.load(p)
        for k in st:
            assert torch.equal(out[k], st[k])
    assert tp.inspect_checkpoint(ps)["metadata"] == {"who": "test"}


def test_sharded_index(tmp_path):
    st = {f"p{i}": torch.randn(100) for i in range(10)}
    idx = S.save_sharded(st, tmp_path / "ck", max_shard_bytes=1000)
    out = tp.load(idx)
    assert set(out) == set(st) and all(torch.equal(out[k], st[k]) for k in st)
    assert torch.equal(tp.load(tmp_path / "ck")["p3"], st["p3"])


def test_mega_container_kinds_match_the_reference_writer(tmp_path):
    """Flat lists / tuples of tensors are stored as kind "list" / "tuple" with names "0", "1", ... and
    no layout (reference tensorplay/serialization/mega.py:393-398); nested structure is kind "tree";
    a tensor that occurs twice is stored once and comes back as one object."""
    import json

    from tensorplay_b200.serialization import mega
    a, b = torch.arange(6.).reshape(2, 3), torch.ones(4, dtype=torch.int32)
    for obj, kind in (([a, b], "list"), ((a, b), "tuple")):
        p = tmp_path / f"{kind}.mega"
        mega.save_mega(obj, p)
        meta = mega.parse_mega(p)
        assert meta["metadata"]["tensorplay.container"] == kind
        assert "tensorplay.layout" not in meta["metadata"]
        assert [r["name"] for r in meta["tensors"]] == ["0", "1"]
        back = mega.load_mega(p)
        assert type(back) is type(obj) and all(torch.equal(x, y) for x, y in zip(back, obj))
    # a header as the reference writes it for a nested tree with a tied tensor
    tree = {"w": a, "opt": [{"m": b, "tied": a}, (1, "s", None)], "__tensor__": {"x": 2.5}}
    p = tmp_path / "tree.mega"
    mega.save_mega(tree, p)
    meta = mega.parse_mega(p)["metadata"]
    assert meta["tensorplay.container"] == "tree"
    layout = json.loads(meta["tensorplay.layout"])
    assert layout["opt"][0]["tied"] == {"__tensor__": "w"}  # stored once, referenced by name
    assert sorted(r["name"] for r in mega.parse_mega(p)["tensors"]) == ["opt.0.m", "w"]
    back = mega.load_mega(p)
    assert back["opt"][0]["tied"] is back["w"]
    assert back["opt"][1] == (1, "s", None) and back["__tensor__"] == {"x": 2.5}
    # a dict whose only key is an escape marker is written in the escaped form
    p = tmp_path / "esc.mega"
    mega.save_mega({"outer": {"__tuple__": a}}, p)
    assert json.loads(mega.parse_mega(p)["metadata"]["tensorplay.layout"])["outer"] == \
        {"__dict__": [["__tuple__", {"__tensor__": "outer.__tuple__"}]]}
    assert torch.equal(mega.load_mega(p)["outer"]["__tuple__"], a)
    # colliding names get "#n"
    flat, kind, _ = mega.flatten_tree({"a": {"b": a}, "a.b": b, "z": [a]})
    assert kind == "tree" and set(flat) == {"a.b", "a.b#1"}
    # a bare tensor is stored under the name "0"
    flat, kind, layout = mega.flatten_tree(a)
    assert (list(flat), kind, layout) == (["0"], "tensor", None)
