"""KV caches for autoregressive decoding, in the reference's ``[B, H, T, D]`` layout.

API after tensorplay/nn/cache.py:51-457 (``Cache.update/get_seq_length``, Dynamic / Static /
SlidingWindow / Paged / Quantized caches, ``LinearStateCache``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
from torch import Tensor


class Cache:
    def update(self, key: Tensor, value: Tensor, layer_idx: int = 0) -> Tuple[Tensor, Tensor]:
        raise NotImplementedError

    def get_seq_length(self, layer_idx: int = 0) -> int:
        raise NotImplementedError


class DynamicCache(Cache):
    """Grows geometrically so that a decode step appends in place instead of re-copying the prefix."""

    def __init__(self) -> None:
        self._k: Dict[int, Tensor] = {}
        self._v: Dict[int, Tensor] = {}
        self._len: Dict[int, int] = {}

    def update(self, key, value, layer_idx: int = 0):
        n = self._len.get(layer_idx, 0)
        t = key.shape[2]
        buf = self._k.get(layer_idx)
        if buf is None or buf.shape[2] < n + t or buf.shape[0] != key.shape[0]:
            cap = max(2 * (n + t), 64)
            nk = key.new_empty(key.shape[0], key.shape[1], cap, key.shape[3])
            nv = value.new_empty(value.shape[0], value.shape[1], cap, value.shape[3])
            if buf is not None and n:
                nk[:, :, :n] = buf[:, :, :n]
                nv[:, :, :n] = self._v[layer_idx][:, :, :n]
            self._k[layer_idx], self._v[layer_idx] = nk, nv
        if key.is_cuda and key.dtype == torch.bfloat16:
            from ..ops import kv_append
            kv_append(self._k[layer_idx], key, n)
            kv_append(self._v[layer_idx], value, n)
        else:
            self._k[layer_idx][:, :, n:n + t] = key
            self._v[layer_idx][:, :, n:n + t] = value
        self._len[layer_idx] = n + t
        return self._k[layer_idx][:, :, :n + t], self._v[layer_idx][:, :, :n + t]

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._len.get(layer_idx, 0)


class StaticCache(Cache):
    """Preallocated ``max_seq_len`` slots per layer (CUDA-graph friendly: fixed addresses)."""

    def __init__(self, max_seq_len: int) -> None:
        self.max_seq_len = int(max_seq_len)
        self._k: Dict[int, Tensor] = {}
        self._v: Dict[int, Tensor] = {}
        self._len: Dict[int, int] = {}

    def update(self, key, value, layer_idx: int = 0):
        n = self._len.get(layer_idx, 0)
        t = key.shape[2]
        if n + t > self.max_seq_len:
            raise ValueError(f"StaticCache overflow: {n + t} > {self.max_seq_len}")
        if layer_idx not in self._k:
            shape = (key.shape[0], key.shape[1], self.max_seq_len, key.shape[3])
            self._k[layer_idx] = key.new_zeros(shape)
            self._v[layer_idx] = value.new_zeros(shape)
        if key.is_cuda and key.dtype == torch.bfloat16:
            from ..ops import kv_append
            kv_append(self._k[layer_idx], key, n)
            kv_append(self._v[layer_idx], value, n)
        else:
            self._k[layer_idx][:, :, n:n + t] = key
            self._v[layer_idx][:, :, n:n + t] = value
        self._len[layer_idx] = n + t
        return self._k[layer_idx][:, :, :n + t], self._v[layer_idx][:, :, :n + t]

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._len.get(layer_idx, 0)

    def reset(self) -> None:
        self._len.clear()


class SlidingWindowCache(Cache):
    """Keeps the last ``window_size`` positions; ``get_seq_length`` still counts all tokens seen."""

    def __init__(self, window_size: int) -> None:
        if window_size <= 0:
            raise ValueError("window_size must be positive")
        self.window_size = int(window_size)
        self._k: Dict[int, Tensor] = {}
        self._v: Dict[int, Tensor] = {}
        self._seen: Dict[int, int] = {}

    def update(self, key, value, layer_idx: int = 0):
        if layer_idx in self._k:
            key = torch.cat((self._k[layer_idx], key), dim=2)
            value = torch.cat((self._v[layer_idx], value), dim=2)
        self._seen[layer_idx] = self._seen.get(layer_idx, 0) + (key.shape[2] - (self._k[layer_idx].shape[2] if layer_idx in self._k else 0))
        self._k[layer_idx] = key[:, :, -self.window_size:]
        self._v[layer_idx] = value[:, :, -self.window_size:]
        return key, value

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._seen.get(layer_idx, 0)

    def get_window_length(self, layer_idx: int = 0) -> int:
        return self._k[layer_idx].shape[2] if layer_idx in self._k else 0


class PagedCache(Cache):
    """Block-table cache: storage is a pool of ``block_size``-token pages; sequences of a batch
    share the pool. ``update`` returns gathered dense views for attention."""

    def __init__(self, block_size: int = 16, num_blocks: Optional[int] = None) -> None:
        self.block_size = int(block_size)
        self.num_blocks = num_blocks
        self._pool_k: Dict[int, Tensor] = {}
        self._pool_v: Dict[int, Tensor] = {}
        self._tables: Dict[int, List[List[int]]] = {}
        self._free: Dict[int, List[int]] = {}
        self._len: Dict[int, int] = {}

    def _ensure(self, layer_idx, key, need_blocks):
        B, H, _, D = key.shape
        pool = self._pool_k.get(layer_idx)
        if pool is None:
            n = self.num_blocks or max(need_blocks * 2, 8)
            self._pool_k[layer_idx] = key.new_zeros(n, H, self.block_size, D)
            self._pool_v[layer_idx] = key.new_zeros(n, H, self.block_size, D)
            self._free[layer_idx] = list(range(n))[::-1]
            self._tables[layer_idx] = [[] for _ in range(B)]
        while len(self._free[layer_idx]) < need_blocks:
            if self.num_blocks is not None:
                raise RuntimeError("PagedCache: out of blocks")
            old = self._pool_k[layer_idx]
            n = old.shape[0]
            self._pool_k[layer_idx] = torch.cat((old, torch.zeros_like(old)), dim=0)
            self._pool_v[layer_idx] = torch.cat((self._pool_v[layer_idx], torch.zeros_like(old)), dim=0)
            self._free[layer_idx] = list(range(n, 2 * n))[::-1] + self._free[layer_idx]

    def update(self, key, value, layer_idx: int = 0):
        B, H, t, D = key.shape
        n = self._len.get(layer_idx, 0)
        bs = self.block_size
        have = (n + bs - 1) // bs
        need = (n + t + bs - 1) // bs
        self._ensure(layer_idx, key, (need - have) * B)
        tables = self._tables[layer_idx]
        for b in range(B):
            for _ in range(need - have):
                tables[b].append(self._free[layer_idx].pop())
        pk, pv = self._pool_k[layer_idx], self._pool_v[layer_idx]
        pos = torch.arange(n, n + t, device=key.device)
        tbl = torch.tensor(tables, device=key.device, dtype=torch.long)  # [B, need]
        blk = tbl[:, pos // bs]  # [B, t]
        off = (pos % bs).expand(B, t)
        if key.is_cuda and key.dtype == torch.bfloat16:
            from ..ops import kv_append
            kv_append(pk, key, n, block_table=tbl, block_size=bs)
            kv_append(pv, value, n, block_table=tbl, block_size=bs)
        else:
            pk[blk, :, off] = key.transpose(1, 2)
            pv[blk, :, off] = value.transpose(1, 2)
        self._len[layer_idx] = n + t
        kk = pk[tbl].permute(0, 2, 1, 3, 4).reshape(B, H, need * bs, D)[:, :, :n + t]
        vv = pv[tbl].permute(0, 2, 1, 3, 4).reshape(B, H, need * bs, D)[:, :, :n + t]
        return kk, vv

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._len.get(layer_idx, 0)

    def block_table(self, layer_idx: int = 0) -> List[List[int]]:
        return self._tables.get(layer_idx, [])


class QuantizedCache(Cache):
    """int8 per-token-per-head symmetric quantisation of K/V; dequantised on read."""

    def __init__(self) -> None:
        self._k: Dict[int, Tuple[Tensor, Tensor]] = {}
        self._v: Dict[int, Tuple[Tensor, Tensor]] = {}

    @staticmethod
    def _q(x):
        scale = x.float().abs().amax(dim=-1, keepdim=True).clamp_(min=1e-8) / 127.0
        return torch.clamp(torch.round(x.float() / scale), -127, 127).to(torch.int8), scale

    def update(self, key, value, layer_idx: int = 0):
        kq, ks = self._q(key)
        vq, vs = self._q(value)
        if layer_idx in self._k:
            kq = torch.cat((self._k[layer_idx][0], kq), dim=2)
            ks = torch.cat((self._k[layer_idx][1], ks), dim=2)
            vq = torch.cat((self._v[layer_idx][0], vq), dim=2)
            vs = torch.cat((self._v[layer_idx][1], vs), dim=2)
        self._k[layer_idx], self._v[layer_idx] = (kq, ks), (vq, vs)
        return (kq.float() * ks).to(key.dtype), (vq.float() * vs).to(value.dtype)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._k[layer_idx][0].shape[2] if layer_idx in self._k else 0


class LinearStateCache:
    """Per-layer conv window and recurrent state for linear-attention / state-space mixers."""

    def __init__(self) -> None:
        self.conv_states: Dict[int, Tensor] = {}
        self.recurrent_states: Dict[int, Tensor] = {}

    def update_conv_state(self, layer_idx: int, conv_state: Tensor, kernel_size: int) -> Tensor:
        prev = self.conv_states.get(layer_idx)
        full = conv_state if prev is None else torch.cat((prev, conv_state), dim=-1)
        self.conv_states[layer_idx] = full[..., -(kernel_size - 1):] if kernel_size > 1 else full[..., :0]
        return full

    def update_recurrent_state(self, layer_idx: int, state: Tensor) -> Tensor:
        self.recurrent_states[layer_idx] = state
        return state
