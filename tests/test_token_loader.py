"""Native token-file loader: coverage, rank partition, targets, determinism, epoch reshuffle."""
import numpy as np
import torch

from tensorplay_b200.utils.data import TokenFileLoader

SEQ, BATCH = 8, 3


def _file(tmp_path, n_samples=50, dtype=np.uint16):
    # token value = its position in the file, so a batch row identifies its sample
    n = n_samples * SEQ + 1
    arr = np.arange(n).astype(dtype)
    p = tmp_path / "tokens.bin"
    arr.tofile(p)
    return str(p)


def _epoch(loader):
    rows = []
    for tok, tgt in loader:
        assert torch.equal(tgt, tok + 1)                   # next-token targets
        assert bool((tok[:, 1:] == tok[:, :-1] + 1).all())   # contiguous window
        rows += [int(v) // SEQ for v in tok[:, 0]]
    return rows


def test_epoch_covers_each_sample_once_and_reshuffles(tmp_path):
    path = _file(tmp_path)
    ld = TokenFileLoader(path, SEQ, BATCH, seed=7, num_workers=3, depth=4)
    assert ld.num_samples == 50 and len(ld) == 50 // BATCH
    e0, e1 = _epoch(ld), _epoch(ld)
    assert len(e0) == 48 and len(set(e0)) == 48 and len(set(e1)) == 48
    assert e0 != e1 and e0 != sorted(e0)
    ld.close()
    ld2 = TokenFileLoader(path, SEQ, BATCH, seed=7, num_workers=1, depth=2)
    assert _epoch(ld2) == e0                               # same seed, same order, any worker count
    ld2.close()
    ld3 = TokenFileLoader(path, SEQ, BATCH, seed=7, shuffle=False)
    assert _epoch(ld3) == list(range(48))
    ld3.close()


def test_ranks_read_disjoint_samples(tmp_path):
    path = _file(tmp_path, n_samples=64, dtype=np.int32)
    seen = []
    for r in range(4):
        ld = TokenFileLoader(path, SEQ, 2, dtype=torch.int32, rank=r, world=4, seed=1)
        assert len(ld) == 8
        seen.append(_epoch(ld))
        ld.close()
    flat = [s for rows in seen for s in rows]
    assert len(flat) == 64 and len(set(flat)) == 64


def test_open_errors(tmp_path):
    import pytest
    with pytest.raises(RuntimeError):
        TokenFileLoader(str(tmp_path / "missing.bin"), SEQ, BATCH)
    p = tmp_path / "short.bin"
    np.arange(4).astype(np.uint16).tofile(p)
    with pytest.raises(RuntimeError):
        TokenFileLoader(str(p), SEQ, BATCH)
