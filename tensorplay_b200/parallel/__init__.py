"""B200-native parallel runtime: the flat-buffer sharded training engine and the
symmetric-memory (NVLink peer) communication layer with its fused compute+collective kernels."""
from .engine import AdamWConfig, FSDPEngine, ParamUnit

__all__ = ["AdamWConfig", "FSDPEngine", "ParamUnit"]
