"""Interpretability tools for decoder language models (the reference's ``lumen/llm``:
logit_lens.py, patching.py, attention.py; ``_core/llm_attr.py``)."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch
from torch import Tensor, nn


def _block_outputs(model: nn.Module, layers: Sequence[nn.Module], run: Callable[[], Tensor]):
    acts: List[Tensor] = []
    hs = [l.register_forward_hook(lambda m, i, o: acts.append((o[0] if isinstance(o, tuple) else o).detach()))
          for l in layers]
    try:
        out = run()
    finally:
        for h in hs:
            h.remove()
    return out, acts


def logit_lens(model: nn.Module, tokens: Tensor, layers: Optional[Sequence[nn.Module]] = None,
               head: Optional[Callable[[Tensor], Tensor]] = None) -> Tensor:
    """Logits decoded from the residual stream after every block: ``[layers, B, T, V]``. ``head``
    maps hidden states to logits (default: the model's ``head`` method: final norm + LM head)."""
    layers = list(model.layers) if layers is None else list(layers)
    head = head or model.head
    with torch.no_grad():
        _, acts = _block_outputs(model, layers, lambda: model(tokens))
        return torch.stack([head(a) for a in acts])


def activation_patching(model: nn.Module, clean_tokens: Tensor, corrupt_tokens: Tensor,
                        metric: Callable[[Tensor], Tensor], layers: Optional[Sequence[nn.Module]] = None,
                        positions: Optional[Sequence[int]] = None) -> Tensor:
    """Causal tracing: run the corrupted prompt with one (layer, position) of the residual stream
    restored from the clean run; returns ``metric(logits)`` for every choice, ``[layers, positions]``."""
    layers = list(model.layers) if layers is None else list(layers)
    with torch.no_grad():
        _, clean = _block_outputs(model, layers, lambda: model(clean_tokens))
        T = clean_tokens.shape[1]
        positions = list(range(T)) if positions is None else list(positions)
        out = torch.zeros(len(layers), len(positions))
        for li, layer in enumerate(layers):
            for pi, pos in enumerate(positions):
                def hook(m, i, o, li=li, pos=pos):
                    t = (o[0] if isinstance(o, tuple) else o).clone()
                    t[:, pos] = clean[li][:, pos]
                    return (t,) + tuple(o[1:]) if isinstance(o, tuple) else t
                h = layer.register_forward_hook(hook)
                try:
                    out[li, pi] = float(metric(model(corrupt_tokens)))
                finally:
                    h.remove()
    return out


def attention_rollout(attentions: Sequence[Tensor], residual: bool = True) -> Tensor:
    """Product over layers of the head-averaged attention maps (with the identity mixed in for the
    residual connection): ``[B, T, T]`` token-to-token influence."""
    roll = None
    for a in attentions:
        m = a.mean(1)
        if residual:
            eye = torch.eye(m.shape[-1], dtype=m.dtype, device=m.device)
            m = 0.5 * m + 0.5 * eye
        m = m / m.sum(-1, keepdim=True)
        roll = m if roll is None else m @ roll
    return roll


class LLMGradientAttribution:
    """Token attribution of a continuation's log-probability by gradient x embedding."""

    def __init__(self, model: nn.Module, embed: Callable[[Tensor], Tensor], forward_embeds: Callable[[Tensor], Tensor]):
        self.model, self.embed, self.forward_embeds = model, embed, forward_embeds

    def attribute(self, prompt: Tensor, continuation: Tensor) -> Dict[str, Tensor]:
        toks = torch.cat((prompt, continuation), 1)
        with torch.enable_grad():
            e = self.embed(toks).detach().requires_grad_()
            logits = self.forward_embeds(e)
            lp = torch.log_softmax(logits.float(), -1)
            P = prompt.shape[1]
            sel = lp[:, P - 1: -1].gather(-1, continuation[..., None])[..., 0]   # log p of each continuation token
            total = sel.sum()
            g = torch.autograd.grad(total, e)[0]
        scores = (g * e).sum(-1).detach()
        return {"token_attr": scores, "log_prob": sel.detach(), "seq_attr": scores[:, :P]}


# ------------------------------------------------------------------------------------------- class spellings
class LogitLens:
    """Object form of :func:`logit_lens` (lumen/llm/logit_lens.py): ``LogitLens(model).attribute(tokens)`` returns the
    per-layer logits, ``top_tokens`` the ``k`` most likely next tokens per layer at one position."""

    def __init__(self, model: nn.Module, layers: Optional[Sequence[nn.Module]] = None,
                 head: Optional[Callable[[Tensor], Tensor]] = None):
        self.model, self.layers, self.head = model, layers, head

    def attribute(self, tokens: Tensor) -> Tensor:
        return logit_lens(self.model, tokens, self.layers, self.head)

    def top_tokens(self, tokens: Tensor, position: int = -1, k: int = 5) -> Tensor:
        return self.attribute(tokens)[:, :, position].topk(k, dim=-1).indices


class ActivationPatching:
    """Object form of :func:`activation_patching` (lumen/llm/patching.py)."""

    def __init__(self, model: nn.Module, layers: Optional[Sequence[nn.Module]] = None):
        self.model, self.layers = model, layers

    def attribute(self, clean_tokens: Tensor, corrupt_tokens: Tensor, metric: Callable[[Tensor], Tensor],
                  positions: Optional[Sequence[int]] = None) -> Tensor:
        return activation_patching(self.model, clean_tokens, corrupt_tokens, metric, self.layers, positions)


def collect_hidden_states(model: nn.Module, tokens: Tensor, layers: Optional[Sequence[nn.Module]] = None) -> List[Tensor]:
    """Residual stream after every block, ``[B, T, H]`` each (the training set of a sparse autoencoder)."""
    layers = list(model.layers) if layers is None else list(layers)
    with torch.no_grad():
        _, acts = _block_outputs(model, layers, lambda: model(tokens))
    return acts


def extract_attention(model: nn.Module, tokens: Tensor, attention_modules: Optional[Sequence[nn.Module]] = None) -> List[Tensor]:
    """Attention probabilities ``[B, heads, T, T]`` of every attention module, recomputed from the module's query and
    key projections as the causal softmax of ``q k^T / sqrt(d)`` (the fused kernels never materialise them). A module
    takes part if it exposes ``last_qk`` after a forward pass, or returns ``(output, probabilities)``."""
    mods = list(attention_modules) if attention_modules is not None else [
        m for m in model.modules() if hasattr(m, "last_qk") or getattr(m, "returns_attention", False)]
    got: List[Tensor] = []
    hooks = []
    for m in mods:
        def hook(mod, i, o):
            if isinstance(o, tuple) and len(o) > 1 and isinstance(o[1], Tensor) and o[1].dim() == 4:
                got.append(o[1].detach())
            elif getattr(mod, "last_qk", None) is not None:
                q, k = mod.last_qk                                        # [B, heads, T, d]
                s = (q.float() @ k.float().transpose(-1, -2)) / q.shape[-1] ** 0.5
                T = s.shape[-1]
                s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool, device=s.device), 1), float("-inf"))
                got.append(torch.softmax(s, dim=-1))
        hooks.append(m.register_forward_hook(hook))
    try:
        with torch.no_grad():
            model(tokens)
    finally:
        for h in hooks:
            h.remove()
    return got


def token_attention(attentions: Sequence[Tensor], query_position: int = -1, layer: Optional[int] = None,
                    head: Optional[int] = None) -> Tensor:
    """How much the token at ``query_position`` attends to every earlier token: ``[B, T]``, averaged over the layers and
    heads that are not fixed."""
    maps = [attentions[layer]] if layer is not None else list(attentions)
    rows = []
    for a in maps:
        a = a[:, head: head + 1] if head is not None else a
        rows.append(a[:, :, query_position].mean(1))
    return torch.stack(rows).mean(0)


class SparseAutoencoder(nn.Module):
    """Overcomplete dictionary of a hidden-state distribution (lumen/llm/sae.py): ``f = relu(W_e (x - b_d) + b_e)``,
    ``x_hat = W_d f + b_d``, decoder columns of unit norm, trained on reconstruction error plus an L1 penalty on ``f``."""

    def __init__(self, d_model: int, d_dict: int, l1_coeff: float = 1e-3):
        super().__init__()
        self.d_model, self.d_dict, self.l1_coeff = d_model, d_dict, l1_coeff
        self.encoder = nn.Linear(d_model, d_dict)
        self.decoder = nn.Linear(d_dict, d_model)
        with torch.no_grad():
            self.decoder.weight.copy_(torch.nn.functional.normalize(self.decoder.weight, dim=0))
            self.encoder.weight.copy_(self.decoder.weight.t())
            self.encoder.bias.zero_()
            self.decoder.bias.zero_()

    def encode(self, x: Tensor) -> Tensor:
        return torch.relu(self.encoder(x - self.decoder.bias))

    def decode(self, f: Tensor) -> Tensor:
        return self.decoder(f)

    def forward(self, x: Tensor):
        f = self.encode(x)
        return self.decode(f), f

    def loss(self, x: Tensor) -> Tensor:
        x_hat, f = self(x)
        return (x_hat - x).pow(2).sum(-1).mean() + self.l1_coeff * f.abs().sum(-1).mean()

    @torch.no_grad()
    def normalize_decoder(self) -> None:
        self.decoder.weight.copy_(torch.nn.functional.normalize(self.decoder.weight, dim=0))


def train_sae(sae: SparseAutoencoder, activations: Tensor, steps: int = 200, batch_size: int = 256, lr: float = 1e-3,
              seed: int = 0) -> List[float]:
    """Adam on random batches of ``activations`` ``[N, d_model]``; the decoder columns are renormalised after every
    step. Returns the loss curve."""
    x = activations.reshape(-1, activations.shape[-1]).float()
    opt = torch.optim.Adam(sae.parameters(), lr=lr)
    g = torch.Generator().manual_seed(seed)
    curve = []
    for _ in range(steps):
        idx = torch.randint(0, x.shape[0], (min(batch_size, x.shape[0]),), generator=g)
        loss = sae.loss(x[idx.to(x.device)])
        opt.zero_grad()
        loss.backward()
        opt.step()
        sae.normalize_decoder()
        curve.append(float(loss.detach()))
    return curve


@torch.no_grad()
def feature_frequency(sae: SparseAutoencoder, activations: Tensor, threshold: float = 0.0) -> Tensor:
    """Share of the inputs on which each dictionary feature fires: ``[d_dict]``."""
    f = sae.encode(activations.reshape(-1, activations.shape[-1]).float())
    return (f > threshold).float().mean(0)


@torch.no_grad()
def top_activating_indices(sae: SparseAutoencoder, activations: Tensor, feature: int, k: int = 10) -> Tensor:
    """Indices (into the flattened inputs) of the ``k`` inputs on which ``feature`` is largest."""
    f = sae.encode(activations.reshape(-1, activations.shape[-1]).float())[:, feature]
    return f.topk(min(k, f.numel())).indices


@torch.no_grad()
def reconstruction_error(sae: SparseAutoencoder, activations: Tensor) -> Tensor:
    """Fraction of the variance of ``activations`` that the reconstruction misses."""
    x = activations.reshape(-1, activations.shape[-1]).float()
    x_hat, _ = sae(x)
    return (x_hat - x).pow(2).sum() / (x - x.mean(0, keepdim=True)).pow(2).sum().clamp_min(1e-12)


# ------------------------------------------------------------------------------------------- cross-layer transcoder
def collect_component_updates(model: nn.Module, tokens: Tensor, layers: Optional[Sequence[nn.Module]] = None):
    """Per block: the residual stream that enters it and the update it adds (output minus input), both ``[B, T, H]``:
    the training pairs of a transcoder (lumen/llm/clt.py:111)."""
    layers = list(model.layers) if layers is None else list(layers)
    ins: List[Tensor] = []
    outs: List[Tensor] = []
    hooks = []
    for l in layers:
        hooks.append(l.register_forward_pre_hook(lambda m, a: ins.append(a[0].detach())))
        hooks.append(l.register_forward_hook(lambda m, a, o: outs.append((o[0] if isinstance(o, tuple) else o).detach())))
    try:
        with torch.no_grad():
            model(tokens)
    finally:
        for h in hooks:
            h.remove()
    return ins, [o - i for i, o in zip(ins, outs)]


class CrossLayerTranscoder(nn.Module):
    """Sparse features read from the residual stream at every layer and written to the updates of that layer and all
    later ones (lumen/llm/clt.py:20): ``f_l = relu(W_enc[l] x_l + b_enc[l])``, ``y_hat_m = sum_{l <= m} W_dec[l -> m] f_l +
    b_dec[m]``. A feature's effect on the output then runs through linear decoders only, which is what makes attribution
    between features exact."""

    def __init__(self, n_layers: int, d_model: int, d_dict: int, l1_coeff: float = 1e-3):
        super().__init__()
        self.n_layers, self.d_model, self.d_dict, self.l1_coeff = n_layers, d_model, d_dict, l1_coeff
        self.encoders = nn.ModuleList([nn.Linear(d_model, d_dict) for _ in range(n_layers)])
        # decoders[l][m - l]: features of layer l -> update of layer m >= l
        self.decoders = nn.ModuleList([nn.ModuleList([nn.Linear(d_dict, d_model, bias=False) for _ in range(n_layers - l)])
                                       for l in range(n_layers)])
        self.b_dec = nn.Parameter(torch.zeros(n_layers, d_model))
        with torch.no_grad():
            for l in range(n_layers):
                for dec in self.decoders[l]:
                    dec.weight.mul_(0.1)

    def encode(self, xs: Sequence[Tensor]) -> List[Tensor]:
        return [torch.relu(enc(x)) for enc, x in zip(self.encoders, xs)]

    def decode(self, feats: Sequence[Tensor]) -> List[Tensor]:
        out = []
        for m in range(self.n_layers):
            y = self.b_dec[m]
            for l in range(m + 1):
                y = y + self.decoders[l][m - l](feats[l])
            out.append(y)
        return out

    def forward(self, xs: Sequence[Tensor]):
        feats = self.encode(xs)
        return self.decode(feats), feats

    def loss(self, xs: Sequence[Tensor], ys: Sequence[Tensor]) -> Tensor:
        preds, feats = self(xs)
        rec = sum((p - y).pow(2).sum(-1).mean() for p, y in zip(preds, ys))
        return rec + self.l1_coeff * sum(f.abs().sum(-1).mean() for f in feats)


def train_clt(clt: CrossLayerTranscoder, inputs: Sequence[Tensor], updates: Sequence[Tensor], steps: int = 200,
              batch_size: int = 256, lr: float = 1e-3, seed: int = 0) -> List[float]:
    """Adam on random rows of the per-layer (input, update) pairs (``[N, d_model]`` each, or ``[B, T, d_model]``)."""
    xs = [x.reshape(-1, x.shape[-1]).float() for x in inputs]
    ys = [y.reshape(-1, y.shape[-1]).float() for y in updates]
    opt = torch.optim.Adam(clt.parameters(), lr=lr)
    g = torch.Generator().manual_seed(seed)
    curve = []
    for _ in range(steps):
        idx = torch.randint(0, xs[0].shape[0], (min(batch_size, xs[0].shape[0]),), generator=g)
        loss = clt.loss([x[idx] for x in xs], [y[idx] for y in ys])
        opt.zero_grad()
        loss.backward()
        opt.step()
        curve.append(float(loss.detach()))
    return curve


# ------------------------------------------------------------------------------------------- attention pictures
def _attention_grid(maps: Tensor):
    """``[rows, cols, T, T]`` maps -> one image array with a one-pixel gutter (values in [0, 1] per map)."""
    import numpy as np
    r, c, t, _ = maps.shape
    m = maps.detach().float().cpu()
    m = m / m.amax(dim=(-1, -2), keepdim=True).clamp_min(1e-12)
    img = np.ones((r * (t + 1) - 1, c * (t + 1) - 1), dtype=np.float32)
    for i in range(r):
        for j in range(c):
            img[i * (t + 1): i * (t + 1) + t, j * (t + 1): j * (t + 1) + t] = m[i, j].numpy()
    return img


def visualize_attention_heads(attention: Tensor, batch_index: int = 0, path: Optional[str] = None):
    """Every head of one layer's attention ``[B, heads, T, T]`` side by side as a grey-scale array (saved as PNG when
    ``path`` is given; no plotting library is needed)."""
    img = _attention_grid(attention[batch_index].unsqueeze(0))
    if path is not None:
        from .visualization import save_heat_map
        save_heat_map(path, torch.from_numpy(img))
    return img


def visualize_attention_multi_layer(attentions: Sequence[Tensor], batch_index: int = 0, path: Optional[str] = None):
    """Layers down, heads across."""
    img = _attention_grid(torch.stack([a[batch_index] for a in attentions]))
    if path is not None:
        from .visualization import save_heat_map
        save_heat_map(path, torch.from_numpy(img))
    return img


def visualize_token_attention(attentions: Sequence[Tensor], tokens: Sequence[str], query_position: int = -1,
                              batch_index: int = 0) -> str:
    """HTML line of the tokens shaded by how much the query position attends to each."""
    w = token_attention(attentions, query_position)[batch_index]
    w = (w / w.max().clamp_min(1e-12)).tolist()
    spans = [f'<span style="background-color: rgba(255, 120, 0, {a:.3f})">{t}</span>' for t, a in zip(tokens, w)]
    return "<div>" + " ".join(spans) + "</div>"


# ------------------------------------------------------------------------------------------- attribution graphs
from dataclasses import dataclass, field  # noqa: E402


@dataclass(frozen=True)
class GraphNode:
    layer: int
    feature: int
    activation: float


@dataclass(frozen=True)
class GraphEdge:
    src: int        # index into ``nodes``
    dst: int
    weight: float


@dataclass
class AttributionGraphData:
    nodes: List[GraphNode] = field(default_factory=list)
    edges: List[GraphEdge] = field(default_factory=list)

    def incoming(self, node: int) -> List[GraphEdge]:
        return [e for e in self.edges if e.dst == node]

    def outgoing(self, node: int) -> List[GraphEdge]:
        return [e for e in self.edges if e.src == node]


class AttributionGraph:
    """Direct effects between the active features of a cross-layer transcoder at one token (lumen/llm/attribution_graph.py).
    A feature ``(l, i)`` with activation ``a`` writes ``a * W_dec[l -> k][:, i]`` into the update of every layer ``k >= l``;
    a later feature ``(m, j)``, ``m > l``, reads the residual stream through ``W_enc[m][j]``. Its pre-activation therefore
    contains ``a * sum_{k = l}^{m - 1} W_enc[m][j] . W_dec[l -> k][:, i]``: the weight of the edge. Everything on the way is
    linear, so the edges into a node add up to the part of its pre-activation that the earlier features explain."""

    def __init__(self, clt: "CrossLayerTranscoder"):
        self.clt = clt

    @torch.no_grad()
    def build(self, xs: Sequence[Tensor], top_k: int = 8, min_weight: float = 0.0) -> AttributionGraphData:
        """``xs``: the residual stream entering every layer at ONE token, ``[d_model]`` each. Keeps the ``top_k`` most
        active features per layer."""
        clt = self.clt
        feats = clt.encode([x.reshape(1, -1).float() for x in xs])
        data = AttributionGraphData()
        per_layer: List[List[int]] = []
        for l, f in enumerate(feats):
            f = f[0]
            k = min(top_k, int((f > 0).sum()))
            idx = f.topk(k).indices.tolist() if k else []
            per_layer.append(list(range(len(data.nodes), len(data.nodes) + len(idx))))
            data.nodes += [GraphNode(l, i, float(f[i])) for i in idx]
        for l in range(clt.n_layers):
            for m in range(l + 1, clt.n_layers):
                if not per_layer[l] or not per_layer[m]:
                    continue
                src_f = [data.nodes[n].feature for n in per_layer[l]]
                dst_f = [data.nodes[n].feature for n in per_layer[m]]
                written = sum(clt.decoders[l][k - l].weight[:, src_f] for k in range(l, m))       # [d_model, |src|]
                w = clt.encoders[m].weight[dst_f] @ written                                      # [|dst|, |src|]
                acts = torch.tensor([data.nodes[n].activation for n in per_layer[l]])
                w = w * acts
                for bi, b in enumerate(per_layer[m]):
                    for ai, a in enumerate(per_layer[l]):
                        if abs(float(w[bi, ai])) > min_weight:
                            data.edges.append(GraphEdge(a, b, float(w[bi, ai])))
        return data


@dataclass(frozen=True)
class CircuitNode:
    layer: int
    feature: int
    score: float


@dataclass(frozen=True)
class CircuitEdge:
    src: int
    dst: int
    weight: float


@dataclass
class FeatureCircuitData:
    nodes: List[CircuitNode] = field(default_factory=list)
    edges: List[CircuitEdge] = field(default_factory=list)


class FeatureCircuit:
    """The part of an attribution graph that matters for one output direction (lumen/llm/feature_circuit.py): every
    feature is scored by its direct effect on ``direction`` (a vector in the residual stream, e.g. the difference of two
    unembedding rows) through all its decoders, the ``top_k`` features per layer are kept, and the edges between them
    are those of the attribution graph."""

    def __init__(self, clt: "CrossLayerTranscoder"):
        self.clt, self.graph = clt, AttributionGraph(clt)

    @torch.no_grad()
    def build(self, xs: Sequence[Tensor], direction: Tensor, top_k: int = 4) -> FeatureCircuitData:
        clt = self.clt
        feats = clt.encode([x.reshape(1, -1).float() for x in xs])
        keep: List[List[int]] = []
        out = FeatureCircuitData()
        for l, f in enumerate(feats):
            effect = sum(dec.weight.t() @ direction.float() for dec in clt.decoders[l]) * f[0]   # [d_dict]
            k = min(top_k, int((f[0] > 0).sum()))
            idx = effect.abs().topk(k).indices.tolist() if k else []
            keep.append(idx)
            out.nodes += [CircuitNode(l, i, float(effect[i])) for i in idx]
        full = self.graph.build(xs, top_k=clt.d_dict)
        pos = {(n.layer, n.feature): i for i, n in enumerate(out.nodes)}
        for e in full.edges:
            a, b = full.nodes[e.src], full.nodes[e.dst]
            if (a.layer, a.feature) in pos and (b.layer, b.feature) in pos:
                out.edges.append(CircuitEdge(pos[(a.layer, a.feature)], pos[(b.layer, b.feature)], e.weight))
        return out


@torch.no_grad()
def top_mlp_features(sae: "SparseAutoencoder", hidden: Tensor, k: int = 10) -> List[tuple]:
    """The ``k`` dictionary features most active on ``hidden`` (any leading shape), as ``(feature, mean activation)``."""
    f = sae.encode(hidden.reshape(-1, hidden.shape[-1]).float()).mean(0)
    top = f.topk(min(k, f.numel()))
    return [(int(i), float(v)) for i, v in zip(top.indices, top.values)]


def top_attention_heads(attentions: Sequence[Tensor], query_position: int = -1, key_position: int = 0, k: int = 5) -> List[tuple]:
    """The ``k`` (layer, head) pairs whose attention from ``query_position`` to ``key_position`` is largest (batch mean)."""
    scores = [(float(a[:, h, query_position, key_position].mean()), l, h)
              for l, a in enumerate(attentions) for h in range(a.shape[1])]
    return [(l, h, s) for s, l, h in sorted(scores, reverse=True)[:k]]


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
