"""Metrics defined on the features of a network: Fréchet / kernel inception distance, inception score,
LPIPS, CLIP score and CLIP-IQA, BERTScore. No pretrained weights ship with this package, so each
takes the network from the caller (any module or callable with the stated output); the
statistics on top of the features are computed here, in float64. Also the short-time objective
intelligibility measure, and the names of speech-quality scores whose models are external."""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence

import torch
from torch import Tensor

from . import Metric


def _features(net: Callable, x: Tensor) -> Tensor:
    if net is None:
        raise ValueError("pass the feature network (`feature=` module or callable): no pretrained weights are bundled")
    with torch.no_grad():
        f = net(x)
    return f.reshape(f.shape[0], -1).double()


class _RealFake(Metric):
    def __init__(self, feature: Optional[Callable] = None, normalize: bool = False, **kw) -> None:
        super().__init__()
        self.net, self.normalize = feature, normalize
        self.real: List[Tensor] = []
        self.fake: List[Tensor] = []

    def reset(self) -> None:
        self.real, self.fake = [], []

    def update(self, imgs: Tensor, real: bool) -> None:
        (self.real if real else self.fake).append(_features(self.net, imgs).cpu())


class FrechetInceptionDistance(_RealFake):
    """``|mu_r - mu_f|^2 + tr(S_r + S_f - 2 (S_r S_f)^(1/2))`` of the feature Gaussians; the trace of
    the matrix square root is the sum of the square roots of the eigenvalues of ``S_r S_f``."""

    def compute(self) -> Tensor:
        r, f = torch.cat(self.real), torch.cat(self.fake)
        if r.shape[0] < 2 or f.shape[0] < 2:
            raise RuntimeError("at least two real and two generated samples are needed")
        mu_r, mu_f = r.mean(0), f.mean(0)
        s_r, s_f = torch.cov(r.T), torch.cov(f.T)
        ev = torch.linalg.eigvals(s_r @ s_f).real.clamp(min=0)
        return (((mu_r - mu_f) ** 2).sum() + torch.trace(s_r) + torch.trace(s_f) - 2 * ev.sqrt().sum()).float()


class KernelInceptionDistance(_RealFake):
    """Unbiased MMD^2 with the polynomial kernel ``(gamma x.y + coef)^degree`` over random subsets;
    returns mean and standard deviation over the subsets."""

    def __init__(self, feature: Optional[Callable] = None, subsets: int = 100, subset_size: int = 1000, degree: int = 3,
                 gamma: Optional[float] = None, coef: float = 1.0, seed: int = 0, **kw) -> None:
        super().__init__(feature)
        self.subsets, self.subset_size, self.degree, self.gamma, self.coef, self.seed = subsets, subset_size, degree, gamma, coef, seed

    def _mmd(self, x: Tensor, y: Tensor) -> Tensor:
        g = self.gamma if self.gamma is not None else 1.0 / x.shape[1]
        k = lambda a, b: (g * a @ b.T + self.coef) ** self.degree   # noqa: E731
        m = x.shape[0]
        kxx, kyy, kxy = k(x, x), k(y, y), k(x, y)
        return ((kxx.sum() - kxx.diag().sum()) + (kyy.sum() - kyy.diag().sum())) / (m * (m - 1)) - 2 * kxy.sum() / (m * m)

    def compute(self):
        r, f = torch.cat(self.real), torch.cat(self.fake)
        if min(r.shape[0], f.shape[0]) < self.subset_size:
            raise ValueError("subset_size is larger than the number of samples")
        g = torch.Generator().manual_seed(self.seed)
        vals = torch.stack([self._mmd(r[torch.randperm(r.shape[0], generator=g)[: self.subset_size]],
                                      f[torch.randperm(f.shape[0], generator=g)[: self.subset_size]]) for _ in range(self.subsets)])
        return vals.mean().float(), vals.std(unbiased=False).float()


class InceptionScore(Metric):
    """``exp(E_x KL(p(y|x) || p(y)))`` over ``splits`` parts of the samples (mean, std); ``feature``
    returns class logits."""

    def __init__(self, feature: Optional[Callable] = None, splits: int = 10, seed: int = 0, **kw) -> None:
        super().__init__()
        self.net, self.splits, self.seed = feature, splits, seed
        self.logits: List[Tensor] = []

    def reset(self) -> None:
        self.logits = []

    def update(self, imgs: Tensor) -> None:
        self.logits.append(_features(self.net, imgs).cpu())

    def compute(self):
        x = torch.cat(self.logits)
        x = x[torch.randperm(x.shape[0], generator=torch.Generator().manual_seed(self.seed))]
        scores = []
        for part in x.chunk(self.splits):
            logp = torch.log_softmax(part, -1)
            p = logp.exp()
            marg = p.mean(0, keepdim=True).log()
            scores.append(((p * (logp - marg)).sum(-1).mean()).exp())
        s = torch.stack(scores)
        return s.mean().float(), s.std(unbiased=False).float()


class LearnedPerceptualImagePatchSimilarity(Metric):
    """Distance between the unit-normalised activations of a network's layers, averaged over space
    and summed over layers. ``net(img)`` returns the list of feature maps; ``weights`` (one vector
    per layer) are the learned channel weights, uniform ``1 / C`` when absent."""

    def __init__(self, net: Optional[Callable] = None, weights: Optional[Sequence[Tensor]] = None, reduction: str = "mean",
                 normalize: bool = False, net_type: Optional[str] = None, **kw) -> None:
        super().__init__()
        if net is None:
            raise ValueError(f"pass the feature network as `net=`: the pretrained {net_type or 'backbone'} weights are not bundled")
        self.net, self.weights, self.reduction, self.normalize = net, weights, reduction, normalize
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, img1: Tensor, img2: Tensor) -> None:
        if self.normalize:                       # [0, 1] inputs -> [-1, 1]
            img1, img2 = 2 * img1 - 1, 2 * img2 - 1
        with torch.no_grad():
            f1, f2 = self.net(img1), self.net(img2)
        d = torch.zeros(img1.shape[0], dtype=torch.float64)
        for i, (a, b) in enumerate(zip(f1, f2)):
            a = a.double() / a.double().norm(dim=1, keepdim=True).clamp(min=1e-10)
            b = b.double() / b.double().norm(dim=1, keepdim=True).clamp(min=1e-10)
            diff = (a - b) ** 2
            w = self.weights[i].double().reshape(1, -1, 1, 1) if self.weights is not None else 1.0 / a.shape[1]
            d += (diff * w).sum(1).flatten(1).mean(-1).cpu()
        self.total += d.sum()
        self.n += d.numel()

    def compute(self) -> Tensor:
        return (self.total if self.reduction == "sum" else self.total / self.n.clamp(min=1)).float()


class CLIPScore(Metric):
    """``100 * max(cos(E_img, E_txt), 0)`` averaged over pairs. ``model`` offers
    ``get_image_features(images)`` and ``get_text_features(texts)`` (or is a pair of callables)."""

    def __init__(self, model=None, **kw) -> None:
        super().__init__()
        if model is None or isinstance(model, str):
            raise ValueError("pass the image/text encoders as `model=`: pretrained CLIP weights are not bundled")
        self.img, self.txt = model if isinstance(model, (tuple, list)) else (model.get_image_features, model.get_text_features)
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, images, text) -> None:
        with torch.no_grad():
            a, b = self.img(images).double(), self.txt(text).double()
        cos = torch.nn.functional.cosine_similarity(a, b, dim=-1)
        self.total += (100 * cos.clamp(min=0)).sum().cpu()
        self.n += cos.numel()

    def compute(self) -> Tensor:
        return (self.total / self.n.clamp(min=1)).float()


class CLIPImageQualityAssessment(Metric):
    """Probability that an image is closer to the positive than to the negative prompt of each pair
    (softmax over the two scaled cosine similarities)."""

    _PROMPTS = {"quality": ("Good photo.", "Bad photo."), "brightness": ("Bright photo.", "Dark photo."),
                "noisiness": ("Clean photo.", "Noisy photo."), "colorfullness": ("Colorful photo.", "Dull photo."),
                "sharpness": ("Sharp photo.", "Blurry photo."), "contrast": ("High contrast photo.", "Low contrast photo."),
                "complexity": ("Complex photo.", "Simple photo."), "natural": ("Natural photo.", "Synthetic photo."),
                "happy": ("Happy photo.", "Sad photo."), "scary": ("Scary photo.", "Peaceful photo."),
                "new": ("New photo.", "Old photo."), "warm": ("Warm photo.", "Cold photo."),
                "real": ("Real photo.", "Abstract photo."), "beautiful": ("Beautiful photo.", "Ugly photo."),
                "lonely": ("Lonely photo.", "Sociable photo."), "relaxing": ("Relaxing photo.", "Stressful photo.")}

    def __init__(self, model=None, prompts=("quality",), logit_scale: float = 100.0, **kw) -> None:
        super().__init__()
        if model is None or isinstance(model, str):
            raise ValueError("pass the image/text encoders as `model=`: pretrained CLIP weights are not bundled")
        self.img, self.txt = model if isinstance(model, (tuple, list)) else (model.get_image_features, model.get_text_features)
        self.names = [p if isinstance(p, str) else f"user_defined_{i}" for i, p in enumerate(prompts)]
        self.pairs = [self._PROMPTS[p] if isinstance(p, str) else tuple(p) for p in prompts]
        self.scale = logit_scale
        self.probs: List[Tensor] = []

    def reset(self) -> None:
        self.probs = []

    def update(self, images) -> None:
        with torch.no_grad():
            a = torch.nn.functional.normalize(self.img(images).double(), dim=-1)
            t = torch.nn.functional.normalize(self.txt([s for pair in self.pairs for s in pair]).double(), dim=-1)
        logits = (self.scale * a @ t.T).reshape(a.shape[0], len(self.pairs), 2)
        self.probs.append(torch.softmax(logits, -1)[..., 0].cpu())

    def compute(self):
        p = torch.cat(self.probs).float()
        return p[:, 0] if len(self.pairs) == 1 else {n: p[:, i] for i, n in enumerate(self.names)}


class BERTScore(Metric):
    """Greedy matching of contextual token embeddings: precision = mean over candidate tokens of the
    best cosine similarity to a reference token, recall the converse, F1 their harmonic mean.
    ``model(sentences)`` returns one ``[tokens, dim]`` tensor per sentence; ``idf`` weights the
    tokens (``model`` then also returns the token ids: ``(embeddings, ids)`` per sentence)."""

    def __init__(self, model: Optional[Callable] = None, idf: bool = False, **kw) -> None:
        super().__init__()
        if model is None or isinstance(model, str):
            raise ValueError("pass the embedding model as `model=`: pretrained language-model weights are not bundled")
        self.model, self.idf = model, idf
        self.pairs: List = []

    def reset(self) -> None:
        self.pairs = []

    def update(self, preds: Sequence[str], target: Sequence[str]) -> None:
        preds, target = ([preds] if isinstance(preds, str) else list(preds)), ([target] if isinstance(target, str) else list(target))
        with torch.no_grad():
            self.pairs += list(zip(self.model(preds), self.model(target)))

    def compute(self):
        weights = None
        if self.idf:
            n = len(self.pairs)
            df = {}
            for _, (_, ids) in self.pairs:
                for t in set(ids.tolist()):
                    df[t] = df.get(t, 0) + 1
            weights = lambda ids: torch.tensor([math.log((n + 1) / (df.get(t, 0) + 1)) for t in ids.tolist()], dtype=torch.float64)  # noqa: E731
        P, R, F = [], [], []
        for c, r in self.pairs:
            (ce, ci), (re_, ri) = (c, r) if self.idf else ((c, None), (r, None))
            sim = torch.nn.functional.normalize(ce.double(), dim=-1) @ torch.nn.functional.normalize(re_.double(), dim=-1).T
            wc = weights(ci) if weights else torch.ones(sim.shape[0], dtype=torch.float64)
            wr = weights(ri) if weights else torch.ones(sim.shape[1], dtype=torch.float64)
            p = (sim.max(1).values * wc).sum() / wc.sum().clamp(min=1e-12)
            q = (sim.max(0).values * wr).sum() / wr.sum().clamp(min=1e-12)
            P.append(p)
            R.append(q)
            F.append(2 * p * q / (p + q).clamp(min=1e-12))
        return {"precision": torch.stack(P).float(), "recall": torch.stack(R).float(), "f1": torch.stack(F).float()}


# ----------------------------------------------------------------------------- speech intelligibility
def _third_octave_matrix(fs: int, nfft: int, bands: int, min_freq: float) -> Tensor:
    f = torch.linspace(0, fs, nfft + 1, dtype=torch.float64)[: nfft // 2 + 1]
    obm = torch.zeros(bands, f.numel(), dtype=torch.float64)
    for k in range(bands):
        lo, hi = min_freq * 2 ** ((2 * k - 1) / 6), min_freq * 2 ** ((2 * k + 1) / 6)
        obm[k, int((f - lo).abs().argmin()): int((f - hi).abs().argmin())] = 1
    return obm


def _frames(x: Tensor, size: int, hop: int) -> Tensor:
    return x.unfold(0, size, hop) if x.numel() >= size else x.new_zeros(0, size)


def short_time_objective_intelligibility(preds: Tensor, target: Tensor, fs: int, extended: bool = False) -> Tensor:
    """STOI of one degraded / clean pair (Taal et al. 2011): both are resampled to 10 kHz, frames more
    than 40 dB below the loudest clean frame are dropped, and the clipped, normalised one-third-
    octave envelopes are correlated over 384 ms segments. ``extended`` (Jensen & Taal 2016)
    normalises rows and columns of each segment instead of clipping."""
    FS, FRAME, NFFT, BANDS, SEG, BETA, DYN = 10000, 256, 512, 15, 30, -15.0, 40.0
    x, y = target.double().reshape(-1), preds.double().reshape(-1)
    if fs != FS:
        from scipy.signal import resample_poly
        g = math.gcd(FS, fs)
        x = torch.from_numpy(resample_poly(x.numpy(), FS // g, fs // g))
        y = torch.from_numpy(resample_poly(y.numpy(), FS // g, fs // g))
    w = torch.hann_window(FRAME + 2, periodic=False, dtype=torch.float64)[1:-1]
    hop = FRAME // 2
    xf, yf = _frames(x, FRAME, hop) * w, _frames(y, FRAME, hop) * w
    energy = 20 * torch.log10(xf.norm(dim=1) + 1e-12)
    keep = energy > energy.max() - DYN
    xf, yf = xf[keep], yf[keep]

    def overlap_add(fr: Tensor) -> Tensor:
        out = torch.zeros((fr.shape[0] - 1) * hop + FRAME, dtype=torch.float64)
        for i in range(fr.shape[0]):
            out[i * hop: i * hop + FRAME] += fr[i]
        return out
    x, y = overlap_add(xf), overlap_add(yf)
    obm = _third_octave_matrix(FS, NFFT, BANDS, 150.0)
    spec = lambda s: torch.fft.rfft(_frames(s, FRAME, hop) * w, NFFT).abs() ** 2   # noqa: E731
    X, Y = torch.sqrt(obm @ spec(x).T), torch.sqrt(obm @ spec(y).T)              # [bands, frames]
    if X.shape[1] < SEG:
        raise ValueError("not enough non-silent frames for one 384 ms segment")
    xs, ys = X.unfold(1, SEG, 1).permute(1, 0, 2), Y.unfold(1, SEG, 1).permute(1, 0, 2)   # [segments, bands, SEG]
    unit = lambda v, d: (v - v.mean(d, keepdim=True)) / (v - v.mean(d, keepdim=True)).norm(dim=d, keepdim=True).clamp(min=1e-12)  # noqa: E731
    if extended:
        xn, yn = unit(unit(xs, 2), 1), unit(unit(ys, 2), 1)
        return ((xn * yn).sum((1, 2)) / SEG).mean().float()
    scale = xs.norm(dim=2, keepdim=True) / ys.norm(dim=2, keepdim=True).clamp(min=1e-12)
    yc = torch.minimum(ys * scale, xs * (1 + 10 ** (-BETA / 20)))
    return (unit(xs, 2) * unit(yc, 2)).sum(2).mean().float()


class ShortTimeObjectiveIntelligibility(Metric):
    def __init__(self, fs: int, extended: bool = False, **kw) -> None:
        super().__init__()
        self.fs, self.extended = fs, extended
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, preds: Tensor, target: Tensor) -> None:
        p, t = preds.detach().cpu().reshape(-1, preds.shape[-1]), target.detach().cpu().reshape(-1, target.shape[-1])
        for a, b in zip(p, t):
            self.total += short_time_objective_intelligibility(a, b, self.fs, self.extended).double()
            self.n += 1

    def compute(self) -> Tensor:
        return (self.total / self.n.clamp(min=1)).float()


def _external(name: str, needs: str):
    class _External(Metric):
        __doc__ = f"{name}: {needs} is not part of this package; pass it as ``scorer=`` (a callable " \
                  f"``scorer(preds, target) -> Tensor`` or ``scorer(preds) -> Tensor``) and the class averages its values."

        def __init__(self, *a, scorer: Optional[Callable] = None, **kw) -> None:
            super().__init__()
            if scorer is None:
                raise RuntimeError(f"{name} needs {needs}, which is not bundled: pass an implementation as `scorer=`")
            self.scorer = scorer
            self.add_state("total", torch.zeros((), dtype=torch.float64))
            self.add_state("n", torch.zeros((), dtype=torch.float64))

        def update(self, *tensors) -> None:
            v = torch.as_tensor(self.scorer(*tensors)).double().reshape(-1)
            self.total += v.sum()
            self.n += v.numel()

        def compute(self) -> Tensor:
            return (self.total / self.n.clamp(min=1)).float()
    _External.__name__ = _External.__qualname__ = name
    return _External


PerceptualEvaluationSpeechQuality = _external("PerceptualEvaluationSpeechQuality", "an ITU-T P.862 implementation")
SpeechReverberationModulationEnergyRatio = _external("SpeechReverberationModulationEnergyRatio", "a gammatone filterbank implementation")
DeepNoiseSuppressionMeanOpinionScore = _external("DeepNoiseSuppressionMeanOpinionScore", "the pretrained DNSMOS networks")
NonIntrusiveSpeechQualityAssessment = _external("NonIntrusiveSpeechQualityAssessment", "the pretrained NISQA network")
InfoLM = _external("InfoLM", "a pretrained masked language model")

__all__ = ["FrechetInceptionDistance", "KernelInceptionDistance", "InceptionScore", "LearnedPerceptualImagePatchSimilarity",
           "CLIPScore", "CLIPImageQualityAssessment", "BERTScore", "ShortTimeObjectiveIntelligibility",
           "short_time_objective_intelligibility", "PerceptualEvaluationSpeechQuality",
           "SpeechReverberationModulationEnergyRatio", "DeepNoiseSuppressionMeanOpinionScore",
           "NonIntrusiveSpeechQualityAssessment", "InfoLM"]


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []


def __getattr__(name):
    """Names of this domain that live in another file of the pack (task wrappers, shared bases)."""
    if name.startswith("__"):
        raise AttributeError(name)
    import importlib
    pkg = importlib.import_module(__name__.rsplit(".", 1)[0])
    if name in pkg.__dict__:
        return pkg.__dict__[name]
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
