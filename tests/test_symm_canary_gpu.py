"""Guard bytes behind symmetric-arena allocations (TPB_SYMM_CANARY=1) catch stores past the end of a
buffer; run in a child process because the arena is one per process."""
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
    from tensorplay_b200.parallel.symm import SymmArena
    torch.cuda.set_device(0)
    a = SymmArena(8 << 20)
    x = a.alloc(1000, torch.float32)
    y = a.alloc(64, torch.bfloat16)
    x.fill_(1.0); y.fill_(2.0)
    assert a.check_canaries() == [], a.check_canaries()
    # a store that runs 8 bytes past the end of x (through a view of the raw arena bytes)
    off = a.offset_of(x)
    a._raw_bytes(off, 4000 + 16)[4000:4008].fill_(7)
    bad = a.check_canaries()
    assert bad == [(off, 4000)], bad
    try:
        a.close()
    except RuntimeError as e:
        assert "guard bytes" in str(e)
        print("CANARY_OK")
""") % ROOT


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_guard_bytes_catch_overrun():
    env = dict(os.environ, TPB_SYMM_CANARY="1")
    out = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0 and "CANARY_OK" in out.stdout, out.stdout + out.stderr
