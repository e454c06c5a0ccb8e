"""Tensor-parallel Llama (Megatron-style TP with a sequence-parallel residual stream) for
inference and training on the fused kernels:

    x_local [rows/tp, H] --rmsnorm--> all-gather->GEMM (QKV shard) --> RoPE + flash attention over
    the local heads --> GEMM->reduce-scatter (o_proj shard) --> residual
    --rmsnorm--> all-gather->GEMM (gate/up shard) --> SwiGLU --> GEMM->reduce-scatter (down shard)

Every rank builds only its own weight shards (no rank ever holds the full model), keeps a KV
cache for its local KV heads in the token-major layout the attention kernel reads, and the LM
head is vocabulary-parallel (greedy decoding merges per-shard maxima).
The reference has no TP inference runner: users apply ``parallelize_module`` to a model and call
``generate`` on every rank (tensorplay/nn/generation.py:73-164).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor, nn

from .. import ops
from ..ops.attention import flash_attention, flash_fwd
from ..parallel.tp import TPContext
from .llama import LlamaConfig


class LlamaTPBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, tp: TPContext, layer_idx: int, device=None, dtype=None):
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        w = tp.world
        assert cfg.num_heads % w == 0 and cfg.num_kv_heads % w == 0 and cfg.ffn_size % w == 0
        self.cfg, self.tp, self.layer_idx = cfg, tp, layer_idx
        self.hq, self.hkv, self.ff = cfg.num_heads // w, cfg.num_kv_heads // w, cfg.ffn_size // w
        H, D = cfg.hidden_size, cfg.head_dim
        self.attn_norm = nn.Parameter(torch.ones(H, **kw))
        self.wqkv = nn.Parameter(torch.empty((self.hq + 2 * self.hkv) * D, H, **kw))
        self.wo = nn.Parameter(torch.empty(H, self.hq * D, **kw))
        self.ffn_norm = nn.Parameter(torch.ones(H, **kw))
        self.w_gate_up = nn.Parameter(torch.empty(2 * self.ff, H, **kw))
        self.w_down = nn.Parameter(torch.empty(H, self.ff, **kw))
        self.k_cache: Optional[Tensor] = None
        self.v_cache: Optional[Tensor] = None

    def reset_parameters(self, gen=None):
        for p in (self.wqkv, self.wo, self.w_gate_up, self.w_down):
            nn.init.normal_(p, std=self.cfg.init_std, generator=gen)

    def forward(self, x_local: Tensor, B: int, T: int, cos: Tensor, sin: Tensor, pos0: int = 0,
                use_cache: bool = False) -> Tensor:
        cfg, tp = self.cfg, self.tp
        D = cfg.head_dim
        h = ops.rms_norm(x_local, self.attn_norm, cfg.rms_eps)
        qkv = tp.all_gather_linear(h, self.wqkv)
        if not use_cache and pos0 == 0:
            # training: RoPE + attention on the packed projection, gradients written back packed
            o = ops.qkv_attention(qkv.view(B, T, -1), cos, sin, None, self.hq, self.hkv, D, causal=True)
            return self._after_attention(x_local, o.reshape(B * T, self.hq * D))
        qkv = qkv.view(B, T, self.hq + 2 * self.hkv, D)
        pos = None
        if pos0:
            pos = torch.arange(pos0, pos0 + T, device=qkv.device).expand(B, T)
        qk = ops.apply_rope(qkv[:, :, : self.hq + self.hkv], cos, sin, pos)
        q, k, v = qk[:, :, : self.hq], qk[:, :, self.hq:], qkv[:, :, self.hq + self.hkv:]
        if use_cache:
            self.k_cache[:B, pos0: pos0 + T] = k
            self.v_cache[:B, pos0: pos0 + T] = v
            k, v = self.k_cache[:B, : pos0 + T], self.v_cache[:B, : pos0 + T]
        if T == 1 and use_cache and self.hq % self.hkv == 0:
            # decode: the query heads of a KV group become the rows of one attention tile
            G = self.hq // self.hkv
            o = flash_attention(q.reshape(B, self.hkv, G, D).transpose(1, 2), k, v, causal=False)
            o = o.transpose(1, 2).reshape(B * T, self.hq * D)
        else:
            o = flash_attention(q, k, v, causal=True).reshape(B * T, self.hq * D)
        return self._after_attention(x_local, o)

    def _after_attention(self, x_local: Tensor, o: Tensor) -> Tensor:
        cfg, tp = self.cfg, self.tp
        x_local = x_local + tp.linear_reduce_scatter(o, self.wo)
        h = ops.rms_norm(x_local, self.ffn_norm, cfg.rms_eps)
        gu = tp.all_gather_linear(h, self.w_gate_up)
        a = ops.swiglu_packed(gu)
        return x_local + tp.linear_reduce_scatter(a, self.w_down)

    def decode(self, x_local: Tensor, B: int, cos: Tensor, sin: Tensor, pos64: Tensor, pos32: Tensor,
               kv_len: Tensor) -> Tensor:
        """One-token step with every position-dependent quantity read from device memory (``pos64``
        / ``pos32``: ``[B]`` write positions, ``kv_len``: int32 scalar = position + 1), so that the
        launch sequence is identical at every step and can be replayed from a CUDA graph."""
        cfg, tp = self.cfg, self.tp
        D = cfg.head_dim
        h = ops.rms_norm(x_local, self.attn_norm, cfg.rms_eps)
        qkv = tp.all_gather_linear(h, self.wqkv).view(B, 1, self.hq + 2 * self.hkv, D)
        qk = ops.apply_rope(qkv[:, :, : self.hq + self.hkv], cos, sin, pos64.view(B, 1))
        q, k, v = qk[:, :, : self.hq], qk[:, :, self.hq:], qkv[:, :, self.hq + self.hkv:]
        # caches are token-major [B, S, hkv, D]; the append kernel takes them head-major by strides
        ops.kv_append(self.k_cache[:B].permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), pos32)
        ops.kv_append(self.v_cache[:B].permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), pos32)
        G = self.hq // self.hkv
        # few CTAs per (sequence, kv head) would walk the whole cache serially: split the keys
        cap_blocks = (self.k_cache.shape[1] + 127) // 128
        n_splits = max(1, min(8, cap_blocks // 4, (2 * 148) // max(1, B * self.hkv)))
        o, _ = flash_fwd(q.reshape(B, self.hkv, G, D).transpose(1, 2), self.k_cache[:B], self.v_cache[:B],
                         False, 1.0 / math.sqrt(D), kv_len=kv_len, n_splits=n_splits)
        o = o.transpose(1, 2).reshape(B, self.hq * D)
        x_local = x_local + tp.linear_reduce_scatter(o, self.wo)
        h = ops.rms_norm(x_local, self.ffn_norm, cfg.rms_eps)
        a = ops.swiglu_packed(tp.all_gather_linear(h, self.w_gate_up))
        return x_local + tp.linear_reduce_scatter(a, self.w_down)


    def decode_replicated(self, x: Tensor, h: Tensor, B: int, cos: Tensor, sin: Tensor, pos64: Tensor, pos32: Tensor,
                          kv_len: Tensor, next_norm: Tensor) -> Tensor:
        """One-token step on REPLICATED activations: ``x [B, H]`` is the residual stream (the same on every
        rank, updated in place), ``h`` its normalised rows for this block's QKV projection. The column-parallel
        projections need no communication, each of the two row-parallel ones ends in one launch that sums the
        partials over the ranks (inside the switch), adds the residual and normalises for the next projection;
        returns the normalised rows for the next block (``next_norm``: its attention-norm weight, or the final
        norm's). Two rendezvous per layer instead of four, and none of them moves more than ``B x H`` values."""
        cfg, tp = self.cfg, self.tp
        D = cfg.head_dim
        qkv = ops.gemm(h, self.wqkv).view(B, self.hq + 2 * self.hkv, D)
        # rotation of q and k and both cache appends in one launch
        q = ops.decode_qkv_prep(qkv, cos, sin, pos32, self.hq, self.hkv, self.k_cache[:B], self.v_cache[:B])
        G = self.hq // self.hkv
        cap_blocks = (self.k_cache.shape[1] + 127) // 128
        n_splits = max(1, min(8, cap_blocks // 4, (2 * 148) // max(1, B * self.hkv)))
        # the kernel sees the G query heads of a KV head as G query rows; its output goes straight into the
        # [B, Hq * D] layout of the output projection (head = kv_head * G + g)
        o = torch.empty((B, self.hq * D), dtype=qkv.dtype, device=qkv.device)
        flash_fwd(q.view(B, self.hkv, G, D).transpose(1, 2), self.k_cache[:B], self.v_cache[:B],
                  False, 1.0 / math.sqrt(D), kv_len=kv_len, n_splits=n_splits,
                  out=o.view(B, self.hkv, G, D).transpose(1, 2))
        h2 = tp.linear_allreduce_add_norm(o, self.wo, x, self.ffn_norm, cfg.rms_eps)
        a = ops.swiglu_packed(ops.gemm(h2, self.w_gate_up))
        return tp.linear_allreduce_add_norm(a, self.w_down, x, next_norm, cfg.rms_eps)


class LlamaTP(nn.Module):
    def __init__(self, cfg: LlamaConfig, tp: TPContext, device=None, dtype=None):
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        self.cfg, self.tp = cfg, tp
        w = tp.world
        self.vshard = (cfg.vocab_size + w - 1) // w
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))  # replicated
        self.layers = nn.ModuleList([LlamaTPBlock(cfg, tp, i, **kw) for i in range(cfg.num_layers)])
        self.final_norm = nn.Parameter(torch.ones(cfg.hidden_size, **kw))
        self.lm_head = nn.Parameter(torch.empty(self.vshard, cfg.hidden_size, **kw))  # vocabulary shard
        self._rope = None
        self._graph = None  # captured decode step (see decode_step)

    def reset_parameters(self, seed: int = 0) -> None:
        dev = self.embed.device
        g_rep = torch.Generator(device=dev).manual_seed(seed)          # same on every rank
        g_loc = torch.Generator(device=dev).manual_seed(seed + 1 + self.tp.rank)  # per-rank shards
        nn.init.normal_(self.embed, std=self.cfg.init_std, generator=g_rep)
        nn.init.normal_(self.lm_head, std=self.cfg.init_std, generator=g_loc)
        for l in self.layers:
            l.reset_parameters(g_loc)

    def allocate_cache(self, batch: int, max_len: int) -> None:
        for l in self.layers:
            shape = (batch, max_len, l.hkv, self.cfg.head_dim)
            l.k_cache = torch.zeros(shape, dtype=self.embed.dtype, device=self.embed.device)
            l.v_cache = torch.zeros(shape, dtype=self.embed.dtype, device=self.embed.device)

    def rope_tables(self, n: int, device):
        if self._rope is None or self._rope[0].shape[0] < n:
            self._rope = ops.rope_tables(n, self.cfg.head_dim, self.cfg.rope_theta, device=device)
        return self._rope

    def _local_rows(self, tokens: Tensor) -> Tensor:
        """Embedding rows of this rank's slice of the flattened (batch, time) token list."""
        w, r = self.tp.world, self.tp.rank
        flat = tokens.reshape(-1)
        n = flat.numel() // w
        return self.embed.index_select(0, flat[r * n: (r + 1) * n])

    def hidden(self, tokens: Tensor, pos0: int = 0, use_cache: bool = False) -> Tensor:
        B, T = tokens.shape
        assert (B * T) % self.tp.world == 0
        cos, sin = self.rope_tables(max(pos0 + T, self.cfg.max_seq_len), tokens.device)
        x = self._local_rows(tokens)
        for l in self.layers:
            x = l(x, B, T, cos, sin, pos0, use_cache)
        return x  # [B*T / tp, H], rows of this rank

    def last_token_hidden(self, x_local: Tensor, B: int, T: int) -> Tensor:
        """``[B, H]`` hidden state of each sequence's last position, on every rank."""
        w, r = self.tp.world, self.tp.rank
        n = (B * T) // w
        rows = torch.arange(B, device=x_local.device) * T + (T - 1)
        mine = (rows >= r * n) & (rows < (r + 1) * n)
        out = torch.zeros(B, x_local.shape[1], dtype=torch.float32, device=x_local.device)
        out[mine] = x_local[(rows[mine] - r * n)].float()
        if w > 1:
            dist.all_reduce(out, group=self.tp.group)
        return out.to(x_local.dtype)

    def greedy_next(self, h_last: Tensor) -> Tensor:
        """Argmax over the vocabulary-parallel logits of ``h_last [B, H]``."""
        h = ops.rms_norm(h_last, self.final_norm, self.cfg.rms_eps)
        logits = ops.linear(h, self.lm_head).float()  # [B, V/tp]
        w, r = self.tp.world, self.tp.rank
        valid = min(self.vshard, self.cfg.vocab_size - r * self.vshard)
        if valid < self.vshard:
            logits[:, valid:] = float("-inf")
        m, idx = logits.max(dim=-1)
        idx = idx + r * self.vshard
        if w == 1:
            return idx
        pair = torch.stack((m, idx.float()), dim=-1)  # [B, 2]
        allp = [torch.empty_like(pair) for _ in range(w)]
        dist.all_gather(allp, pair, group=self.tp.group)
        allp = torch.stack(allp)  # [w, B, 2]
        best = allp[..., 0].argmax(dim=0)
        return allp[best, torch.arange(pair.shape[0], device=pair.device), 1].long()

    @torch.no_grad()
    def prefill(self, tokens: Tensor) -> Tensor:
        B, T = tokens.shape
        x = self.hidden(tokens, 0, use_cache=True)
        return self.greedy_next(self.last_token_hidden(x, B, T))

    @torch.no_grad()
    def decode_step(self, last_tokens: Tensor, pos: int, use_graph: bool = True) -> Tensor:
        """Greedy next token for ``last_tokens [B]`` written at cache position ``pos``.

        On CUDA the transformer body of the step is captured once into a CUDA graph and replayed:
        positions and the key length live in device memory and advance inside the graph, the fused
        collectives keep their epochs on the device, so a replay needs no host-side argument. The
        vocabulary-parallel head (an NCCL exchange of per-shard maxima) runs eagerly after it."""
        B = last_tokens.shape[0]
        if not (use_graph and last_tokens.is_cuda and self.cfg.num_heads % self.cfg.num_kv_heads == 0):
            x = self.hidden(last_tokens.view(B, 1), pos, use_cache=True)
            return self.greedy_next(self.last_token_hidden(x, B, 1))
        g = self._graph
        if g is None or g["B"] != B:
            # First step at this batch size: run the body eagerly (it is the real step, so every
            # kernel is configured and every plan buffer exists), then capture it for the next ones.
            assert B % self.tp.world == 0
            dev = last_tokens.device
            g = self._graph = {"B": B, "pos": pos + 1,
                               "tok": last_tokens.view(B, 1).clone(),
                               "pos64": torch.full((B,), pos, dtype=torch.long, device=dev),
                               "pos32": torch.full((B,), pos, dtype=torch.int32, device=dev),
                               "kv_len": torch.full((1,), pos + 1, dtype=torch.int32, device=dev)}
            out = self._decode_body(g)
            nxt = self.greedy_next(out if g.get("replicated") else self.last_token_hidden(out, B, 1))
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                g["out"] = self._decode_body(g)
            g["graph"] = graph
            return nxt
        if g["pos"] != pos:  # (re)position: plain copies outside the graph
            g["pos64"].fill_(pos)
            g["pos32"].fill_(pos)
            g["kv_len"].fill_(pos + 1)
        g["tok"].copy_(last_tokens.view(B, 1))
        g["graph"].replay()
        g["pos"] = pos + 1  # the graph advanced the device-side positions itself
        return self.greedy_next(g["out"] if g.get("replicated") else self.last_token_hidden(g["out"], B, 1))

    # "replicated": activations of the decode step are the same on every rank and the row-parallel projections
    # end in a one-launch all-reduce + residual + norm (2 rendezvous per layer); "sequence": the rows of the batch
    # are sharded over the ranks and every projection is a fused all-gather -> GEMM or GEMM -> reduce-scatter
    # (4 rendezvous per layer). Replicated is the default: at decode sizes a projection is bound by streaming its
    # weights and the collectives by their latency.
    decode_layout = "replicated"

    def _decode_body(self, g) -> Tensor:
        B = g["B"]
        cap = max(self.cfg.max_seq_len, self.layers[0].k_cache.shape[1])  # every cache position has a row
        cos, sin = self.rope_tables(cap, g["tok"].device)
        if self.decode_layout == "replicated" and self.tp.world > 1 and self.tp.arena is not None:
            x = self.embed.index_select(0, g["tok"].reshape(-1))      # [B, H] on every rank
            h = ops.rms_norm(x, self.layers[0].attn_norm, self.cfg.rms_eps)
            for i, l in enumerate(self.layers):
                nxt = self.layers[i + 1].attn_norm if i + 1 < len(self.layers) else None
                h = l.decode_replicated(x, h, B, cos, sin, g["pos64"], g["pos32"], g["kv_len"], nxt)
            g["pos64"] += 1
            g["pos32"] += 1
            g["kv_len"] += 1
            g["replicated"] = True   # x holds every sequence's hidden state on every rank
            return x
        x = self._local_rows(g["tok"])
        for l in self.layers:
            x = l.decode(x, B, cos, sin, g["pos64"], g["pos32"], g["kv_len"])
        g["pos64"] += 1
        g["pos32"] += 1
        g["kv_len"] += 1
        return x


class LlamaTPStage(nn.Module):
    """One pipeline stage of the tensor-parallel Llama for training: ``num_layers / num_stages``
    blocks, plus the embedding on the first stage and the final norm and LM head on the last.

    Activations between stages are this rank's rows ``[b * T / tp, H]`` of the sequence-parallel
    residual stream, so a stage talks only to the same tensor-parallel rank of the neighbouring
    stage. Embedding, norms and LM head are replicated over the tensor-parallel group and see only
    the local rows: their gradients are summed over that group by ``sync_replicated_grads`` after
    the backward passes. The last stage returns the logits of its local rows.
    """

    def __init__(self, cfg: LlamaConfig, tp: TPContext, stage_index: int, num_stages: int, micro_batch: int,
                 seq_len: int, device=None, dtype=None):
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        assert cfg.num_layers % num_stages == 0 and (micro_batch * seq_len) % tp.world == 0
        self.cfg, self.tp = cfg, tp
        self.first, self.last = stage_index == 0, stage_index == num_stages - 1
        self.b, self.T = micro_batch, seq_len
        per = cfg.num_layers // num_stages
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw)) if self.first else None
        self.layers = nn.ModuleList([LlamaTPBlock(cfg, tp, stage_index * per + i, **kw) for i in range(per)])
        if self.last:
            self.final_norm = nn.Parameter(torch.ones(cfg.hidden_size, **kw))
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        self._rope = None

    def reset_parameters(self, seed: int = 0) -> None:
        dev = self.layers[0].wqkv.device
        g_rep = torch.Generator(device=dev).manual_seed(seed)
        g_loc = torch.Generator(device=dev).manual_seed(seed + 1 + self.tp.rank + 64 * self.layers[0].layer_idx)
        if self.first:
            nn.init.normal_(self.embed, std=self.cfg.init_std, generator=g_rep)
        if self.last:
            nn.init.normal_(self.lm_head, std=self.cfg.init_std, generator=g_rep)
        for l in self.layers:
            l.reset_parameters(g_loc)

    def local_rows(self, t: Tensor) -> Tensor:
        """This rank's slice of a ``[b, T, ...]`` tensor flattened over (batch, time)."""
        flat = t.reshape(self.b * self.T, *t.shape[2:])
        n = flat.shape[0] // self.tp.world
        return flat[self.tp.rank * n: (self.tp.rank + 1) * n]

    def replicated_parameters(self):
        """Parameters that every tensor-parallel rank holds in full (by name)."""
        return [n for n, _ in self.named_parameters()
                if n.endswith("norm") or n in ("embed", "lm_head")]

    def forward(self, x: Tensor) -> Tensor:
        if self._rope is None:
            self._rope = ops.rope_tables(max(self.T, self.cfg.max_seq_len), self.cfg.head_dim, self.cfg.rope_theta,
                                         device=x.device)
        cos, sin = self._rope
        if self.first:
            x = ops.embedding(self.local_rows(x), self.embed)
        for l in self.layers:
            x = l(x, self.b, self.T, cos, sin)
        if self.last:
            x = ops.linear(ops.rms_norm(x, self.final_norm, self.cfg.rms_eps), self.lm_head)
        return x


def sync_replicated_grads(module: nn.Module, names, group) -> None:
    """Sum over the tensor-parallel group the gradients of the parameters ``names`` (those every
    rank of the group holds in full while seeing only its rows of the sequence): one flat
    all-reduce."""
    params = dict(module.named_parameters())
    grads = [params[n].grad for n in names if n in params and params[n].grad is not None]
    if not grads or dist.get_world_size(group) == 1:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=group)
    off = 0
    for g in grads:
        g.copy_(flat[off: off + g.numel()].view_as(g))
        off += g.numel()
