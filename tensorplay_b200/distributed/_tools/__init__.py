"""Memory / runtime estimation tools (tensorplay/distributed/_tools): torch's trackers plus a
per-unit memory plan of the sharded engine."""
from torch.distributed._tools import MemTracker  # noqa: F401

try:  # names differ across torch versions
    from torch.distributed._tools import FSDPMemTracker, RuntimeEstimator, SACEstimator  # noqa: F401
except ImportError:  # pragma: no cover
    pass


def engine_memory_plan(engine) -> dict:
    """Bytes per rank that ``FSDPEngine`` holds persistently (sharded fp32 master and moments, bf16
    shard) and transiently (rotating full-parameter and gradient buffers)."""
    esz = 2 if str(engine.param_dtype).endswith("bfloat16") or str(engine.param_dtype).endswith("float16") else 4
    shard = sum(u.shard_numel for u in engine.units)
    local = sum(u.local.padded for u in engine.units if u.local is not None)
    pools = (len(getattr(engine, "full_pool", [])) + len(getattr(engine, "grad_pool", []))) * engine.max_padded * esz
    return {"sharded_state_bytes": shard * (12 + esz), "expert_local_state_bytes": local * (12 + esz),
            "rotating_buffer_bytes": pools, "units": len(engine.units), "world": engine.world}
