"""The debug build of the kernel library (TPB_DEBUG=1 -> libtpb200_dbg.so): an index guard that only
skips the access in the release build reports its site through the status word, and the access is
still skipped (nothing out of range is read or written)."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import sys, torch
    sys.path.insert(0, %r)
    import tensorplay_b200.ops as O
    from tensorplay_b200.ops._common import lib, DeviceIndexError
    assert lib().tpb_debug_build() == 1
    dev = torch.device("cuda", 0)
    table = torch.randn(100, 64, device=dev, dtype=torch.bfloat16)
    ok = O.embedding(torch.tensor([[1, 5, 99]], device=dev), table)
    O.check_status()                                   # in range: nothing reported
    assert torch.equal(ok[0, 2], table[99])
    out = O.embedding(torch.tensor([[1, 100, 7]], device=dev), table)   # 100 is one past the end
    try:
        O.check_status()
        raise SystemExit("no report")
    except DeviceIndexError as e:
        assert "site 40" in str(e), str(e)
    assert float(out[0, 1].abs().sum()) == 0.0         # the row was skipped (zeros), not read out of range
    assert torch.equal(out[0, 2], table[7])
    # cross-entropy with a target outside the vocabulary: reported, and the row counts as ignored
    logits = torch.randn(4, 512, device=dev, dtype=torch.bfloat16)
    tgt = torch.tensor([1, 2, 512, 3], device=dev)
    loss = O.cross_entropy(logits, tgt, reduction="none")
    try:
        O.check_status()
        raise SystemExit("no report")
    except DeviceIndexError as e:
        assert "site 43" in str(e), str(e)
    assert float(loss[2]) == 0.0
    print("DEBUG_BUILD_OK")
""") % ROOT


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_debug_build_reports_skipped_indices():
    env = dict(os.environ, TPB_DEBUG="1")
    out = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0 and "DEBUG_BUILD_OK" in out.stdout, out.stdout + out.stderr
