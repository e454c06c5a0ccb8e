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


def activation_checkpoint_plan(cfg, seq_len: int, micro_batch: int = 1, act_bytes: int = 2) -> dict:
    """Per-policy estimate for a Llama-shaped decoder under ``FSDPEngine``'s activation
    checkpointing: bytes of activations kept across the forward, and forward FLOPs recomputed in
    backward (per rank, one micro-batch).

    * ``none``: every tensor autograd saves in a block stays alive until its backward.
    * ``selective``: the block input plus the outputs of its four GEMMs and of the attention
      (with its log-sum-exp); norms, RoPE and SwiGLU are recomputed (elementwise: no GEMM FLOPs).
    * ``full``: only the block input; the whole block forward runs again in backward.
    """
    t = seq_len * micro_batch
    h, f = cfg.hidden_size, cfg.ffn_size
    hq, hkv, d = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    qkv = (hq + 2 * hkv) * d
    gemm_flops = 2.0 * t * (h * qkv + hq * d * h + h * 2 * f + f * h)
    attn_flops = 2.0 * 2.0 * micro_batch * hq * seq_len * seq_len * d / 2   # causal: half the square
    kept_selective = t * (h + qkv + hq * d + h + 2 * f + h) * act_bytes + micro_batch * hq * seq_len * 4
    # plain autograd also keeps both norm outputs, the rotated q/k, the SwiGLU product and residual sums
    kept_none = kept_selective + t * (2 * h + (hq + hkv) * d + f + 2 * h) * act_bytes
    layers = cfg.num_layers
    return {
        "none": {"kept_bytes": layers * kept_none, "recompute_flops": 0.0},
        "selective": {"kept_bytes": layers * kept_selective, "recompute_flops": 0.0,
                      "recompute_elementwise_bytes": layers * t * (4 * h + 2 * (hq + hkv) * d + 3 * f) * act_bytes},
        "full": {"kept_bytes": layers * t * h * act_bytes, "recompute_flops": layers * (gemm_flops + attn_flops)},
        "forward_flops": layers * (gemm_flops + attn_flops),
    }


def __getattr__(name):
    """Other trackers and estimators (``MemoryTracker``, ``ModTracker``, SAC statistics ...) resolve to PyTorch's."""
    import importlib
    for mod in ("torch.distributed._tools", "torch.distributed._tools.memory_tracker", "torch.distributed._tools.mod_tracker",
                "torch.distributed._tools.sac_estimator", "torch.distributed._tools.sac_ilp", "torch.distributed._tools.ilp_utils"):
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
