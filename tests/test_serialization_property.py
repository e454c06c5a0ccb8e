"""Property tests of the checkpoint formats: arbitrary trees of tensors of every supported dtype and
shape (including empty and 0-d tensors and non-contiguous views) survive ``save`` / ``load`` bit for
bit in ``.mega``, torch zip and safetensors."""
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

import tensorplay_b200 as tp

DTYPES = [torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int8, torch.uint8, torch.int16,
          torch.int32, torch.int64, torch.bool]


@st.composite
def tensors(draw):
    dtype = draw(st.sampled_from(DTYPES))
    shape = tuple(draw(st.lists(st.integers(0, 5), min_size=0, max_size=3)))
    seed = draw(st.integers(0, 2 ** 16))
    g = torch.Generator().manual_seed(seed)
    n = 1
    for s in shape:
        n *= s
    if dtype == torch.bool:
        t = torch.rand(shape, generator=g) > 0.5
    elif dtype.is_floating_point:
        t = (torch.randn(shape, generator=g) * 100).to(dtype)
    else:
        info = torch.iinfo(dtype)
        t = torch.randint(max(info.min, -1000), min(info.max, 1000) + 1, shape, generator=g).to(dtype)
    if draw(st.booleans()) and t.dim() >= 2:
        t = t.transpose(0, 1)                              # a non-contiguous view
    return t


names = st.text(alphabet="abcdefghijklmnopqrstuvwxyz_0123456789.", min_size=1, max_size=12).filter(
    lambda s: not s.startswith(".") and not s.endswith(".") and ".." not in s)


def _same(a, b):
    assert a.dtype == b.dtype and a.shape == b.shape
    if a.numel():
        assert torch.equal(a.contiguous().reshape(-1).view(torch.uint8), b.contiguous().reshape(-1).view(torch.uint8))


@settings(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])
@given(state=st.dictionaries(names, tensors(), min_size=1, max_size=6), fmt=st.sampled_from(["mega", "zip", "safetensors"]))
def test_flat_state_roundtrip(tmp_path_factory, state, fmt):
    path = str(tmp_path_factory.mktemp("rt") / {"mega": "s.mega", "zip": "s.pt", "safetensors": "s.safetensors"}[fmt])
    tp.save(state, path)
    assert tp.serialization.sniff_format(path) == fmt
    back = tp.load(path)
    assert set(back) == set(state)
    for k in state:
        _same(back[k], state[k])


@settings(max_examples=25, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])
@given(leaves=st.lists(tensors(), min_size=1, max_size=5), meta=st.dictionaries(names, st.one_of(st.integers(0, 10 ** 6), st.text(max_size=8)),
                                                                               max_size=3))
def test_nested_tree_and_metadata_roundtrip_in_mega(tmp_path_factory, leaves, meta):
    tree = {"model": {f"w{i}": t for i, t in enumerate(leaves)}, "list": [leaves[0], {"inner": leaves[-1]}], "step": 7}
    path = str(tmp_path_factory.mktemp("tree") / "t.mega")
    tp.save(tree, path, metadata=meta)
    back = tp.load(path)
    assert back["step"] == 7 and set(back["model"]) == set(tree["model"])
    for k, t in tree["model"].items():
        _same(back["model"][k], t)
    _same(back["list"][1]["inner"], leaves[-1])
    info = tp.inspect_checkpoint(path, verify_checksums=True)
    assert info["format"] == "mega"
    for k, v in meta.items():
        assert info["metadata"].get(k) == v
