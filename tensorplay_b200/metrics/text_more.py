"""Machine-translation and question-answering scores that need their own tokenisation or alignment:
SacreBLEU, chrF / chrF++, translation edit rate, extended edit distance, SQuAD exact match / F1."""
from __future__ import annotations

import math
import re
import string
from collections import Counter
from typing import Dict, List, Sequence

import torch
from torch import Tensor

from . import Metric
from .domains import BLEUScore, _as_list, _ngrams, edit_distance


# ----------------------------------------------------------------------------- SacreBLEU
_13A = [(re.compile(r"([\{-\~\[-\` -\&\(-\+\:-\@\/])"), r" \1 "), (re.compile(r"([^0-9])([\.,])"), r"\1 \2 "),
        (re.compile(r"([\.,])([^0-9])"), r" \1 \2"), (re.compile(r"([0-9])(-)"), r"\1 \2 ")]


def _tokenize(line: str, scheme: str, lowercase: bool) -> str:
    if scheme == "13a":
        line = line.replace("<skipped>", "").replace("-\n", "").replace("\n", " ")
        line = line.replace("&quot;", '"').replace("&amp;", "&").replace("&lt;", "<").replace("&gt;", ">")
        line = f" {line} "
        for rx, sub in _13A:
            line = rx.sub(sub, line)
    elif scheme == "char":
        line = " ".join(ch for ch in line if not ch.isspace())
    elif scheme == "intl":
        line = re.sub(r"([^\w\s])", r" \1 ", line)
    elif scheme != "none":
        raise ValueError(f"unknown tokenizer {scheme!r} (none, 13a, intl, char)")
    line = " ".join(line.split())
    return line.lower() if lowercase else line


class SacreBLEUScore(BLEUScore):
    """BLEU on text that this class tokenises itself (``tokenize``: "13a", "intl", "char", "none"),
    so that scores of differently pre-processed systems are comparable."""

    def __init__(self, n_gram: int = 4, smooth: bool = False, tokenize: str = "13a", lowercase: bool = False, **kw) -> None:
        super().__init__(n_gram, smooth)
        self.scheme, self.lowercase = tokenize, lowercase

    def update(self, preds: Sequence[str], target: Sequence[Sequence[str]]) -> None:
        tok = lambda s: _tokenize(s, self.scheme, self.lowercase)   # noqa: E731
        super().update([tok(p) for p in _as_list(preds)], [[tok(r) for r in _as_list(refs)] for refs in target])


# ----------------------------------------------------------------------------- chrF
class CHRFScore(Metric):
    """chrF (``n_word_order = 0``) or chrF++ (``n_word_order = 2``): mean over the n-gram orders of the
    corpus-level F-beta of character (and word) n-grams; of several references the best one counts."""

    def __init__(self, n_char_order: int = 6, n_word_order: int = 2, beta: float = 2.0, lowercase: bool = False,
                 whitespace: bool = False, **kw) -> None:
        super().__init__()
        self.nc, self.nw, self.beta, self.lowercase, self.whitespace = n_char_order, n_word_order, beta, lowercase, whitespace
        n = n_char_order + n_word_order
        for name in ("match", "hyp", "ref"):
            self.add_state(name, torch.zeros(n, dtype=torch.float64))

    def _grams(self, s: str) -> List[Counter]:
        s = s.lower() if self.lowercase else s
        chars = s if self.whitespace else "".join(s.split())
        words = []
        for w in s.split():                       # punctuation at a word's edge is a word of its own
            if len(w) > 1 and w[-1] in string.punctuation:
                words += [w[:-1], w[-1]]
            elif len(w) > 1 and w[0] in string.punctuation:
                words += [w[0], w[1:]]
            else:
                words.append(w)
        return [_ngrams(list(chars), n) for n in range(1, self.nc + 1)] + [_ngrams(words, n) for n in range(1, self.nw + 1)]

    def _f(self, match, hyp, ref) -> float:
        b2, fs = self.beta ** 2, []
        for m, h, r in zip(match, hyp, ref):
            if h > 0 and r > 0:
                p, q = m / h, m / r
                fs.append((1 + b2) * p * q / (b2 * p + q) if p + q > 0 else 0.0)
        return sum(fs) / len(fs) if fs else 0.0

    def update(self, preds: Sequence[str], target: Sequence[Sequence[str]]) -> None:
        for p, refs in zip(_as_list(preds), target):
            pg = self._grams(p)
            hyp = [sum(c.values()) for c in pg]
            best = None
            for r in _as_list(refs):
                rg = self._grams(r)
                match = [sum((a & b).values()) for a, b in zip(pg, rg)]
                ref = [sum(c.values()) for c in rg]
                f = self._f(match, hyp, ref)
                if best is None or f > best[0]:
                    best = (f, match, ref)
            self.match += torch.tensor(best[1], dtype=torch.float64)
            self.hyp += torch.tensor(hyp, dtype=torch.float64)
            self.ref += torch.tensor(best[2], dtype=torch.float64)

    def compute(self) -> Tensor:
        return torch.tensor(self._f(self.match.tolist(), self.hyp.tolist(), self.ref.tolist()))


# ----------------------------------------------------------------------------- translation edit rate
_MAX_SHIFT = 10


def _ter_edits(hyp: List[str], ref: List[str]) -> int:
    """Word edits plus block shifts: greedily apply the shift of a hypothesis span (at most ten words,
    found verbatim elsewhere in the reference) that lowers the edit distance most, until none does."""
    cur, shifts = list(hyp), 0
    dist = edit_distance(cur, ref)
    while dist > 0:
        best = None
        for length in range(min(_MAX_SHIFT, len(cur)), 0, -1):
            for i in range(len(cur) - length + 1):
                span = cur[i: i + length]
                rest = cur[:i] + cur[i + length:]
                for j in range(len(ref) - length + 1):
                    if j == i or ref[j: j + length] != span:
                        continue
                    cand = rest[: min(j, len(rest))] + span + rest[min(j, len(rest)):]
                    d = edit_distance(cand, ref)
                    gain = dist - d
                    if gain > 1 and (best is None or gain > best[0]):      # a shift costs one edit itself
                        best = (gain, cand, d)
        if best is None:
            break
        _, cur, dist = best
        shifts += 1
    return dist + shifts


class TranslationEditRate(Metric):
    """TER: (word edits + block shifts) of the closest reference / mean reference length."""

    def __init__(self, normalize: bool = False, no_punctuation: bool = False, lowercase: bool = True,
                 return_sentence_level_score: bool = False, **kw) -> None:
        super().__init__()
        self.normalize, self.no_punct, self.lowercase = normalize, no_punctuation, lowercase
        self.sentence_level = return_sentence_level_score
        self.sentences: List[float] = []
        self.add_state("edits", torch.zeros((), dtype=torch.float64))
        self.add_state("length", torch.zeros((), dtype=torch.float64))

    def reset(self) -> None:
        super().reset()
        self.sentences = []

    def _prep(self, s: str) -> List[str]:
        s = s.lower() if self.lowercase else s
        if self.normalize:
            s = re.sub(r"([^\w\s])", r" \1 ", s)
        if self.no_punct:
            s = re.sub(r"[^\w\s]", "", s)
        return s.split()

    def update(self, preds: Sequence[str], target: Sequence[Sequence[str]]) -> None:
        for p, refs in zip(_as_list(preds), target):
            h = self._prep(p)
            rs = [self._prep(r) for r in _as_list(refs)]
            e = min(_ter_edits(h, r) for r in rs)
            avg = sum(len(r) for r in rs) / len(rs)
            self.edits += e
            self.length += avg
            self.sentences.append(e / avg if avg else float(e > 0))

    def compute(self):
        score = (self.edits / self.length.clamp(min=1e-12)).float()
        return (score, torch.tensor(self.sentences)) if self.sentence_level else score


# ----------------------------------------------------------------------------- extended edit distance
def _eed_sentence(hyp: str, ref: str, alpha: float, rho: float, deletion: float, insertion: float) -> float:
    """Character edit distance in which the hypothesis may jump at a blank of the reference for a cost
    of ``alpha``, plus a penalty ``rho`` for every hypothesis position visited a number of times
    other than once; normalised by reference length + penalty (Stanchev, Wang, Ney, WMT 2019)."""
    visits = [-1] * (len(hyp) + 1)
    row = [1.0] * (len(hyp) + 1)
    row[0] = 0.0
    for w in range(1, len(ref) + 1):
        nxt = [row[0] + 1.0] + [math.inf] * len(hyp)
        for i in range(1, len(hyp) + 1):
            nxt[i] = min(nxt[i - 1] + deletion, row[i - 1] + (0.0 if hyp[i - 1] == ref[w - 1] else 1.0), row[i] + insertion)
        k = min(range(len(nxt)), key=nxt.__getitem__)
        visits[k] += 1
        if ref[w - 1] == " ":
            jump = alpha + nxt[k]
            nxt = [min(x, jump) for x in nxt]
        row = nxt
    coverage = rho * sum(v if v >= 0 else 1 for v in visits)
    return min(1.0, (row[-1] + coverage) / (len(ref) + coverage))


class ExtendedEditDistance(Metric):
    def __init__(self, language: str = "en", return_sentence_level_score: bool = False, alpha: float = 2.0, rho: float = 0.3,
                 deletion: float = 0.2, insertion: float = 1.0, **kw) -> None:
        super().__init__()
        self.args = (alpha, rho, deletion, insertion)
        self.sentence_level = return_sentence_level_score
        self.scores: List[float] = []

    def reset(self) -> None:
        self.scores = []

    @staticmethod
    def _prep(s: str) -> str:
        s = re.sub(r"([\.,!\?:;])", r" \1", s.strip())         # punctuation becomes a token of its own
        return " " + " ".join(s.split()) + " "

    def update(self, preds: Sequence[str], target: Sequence[Sequence[str]]) -> None:
        for p, refs in zip(_as_list(preds), target):
            h = self._prep(p)
            self.scores.append(min(_eed_sentence(h, self._prep(r), *self.args) for r in _as_list(refs)))

    def compute(self):
        mean = torch.tensor(sum(self.scores) / max(1, len(self.scores)))
        return (mean, torch.tensor(self.scores)) if self.sentence_level else mean


# ----------------------------------------------------------------------------- SQuAD
def _squad_norm(s: str) -> List[str]:
    s = "".join(ch for ch in s.lower() if ch not in set(string.punctuation))
    return re.sub(r"\b(a|an|the)\b", " ", s).split()


class SQuAD(Metric):
    """Exact match and token F1 (percent) of predicted answers against the best of the gold answers;
    ``preds``: ``{"prediction_text", "id"}``, ``target``: ``{"answers": {"text": [...]}, "id"}``."""

    def __init__(self, **kw) -> None:
        super().__init__()
        for name in ("em", "f1", "n"):
            self.add_state(name, torch.zeros((), dtype=torch.float64))

    def update(self, preds, target) -> None:
        preds = [preds] if isinstance(preds, dict) else preds
        target = [target] if isinstance(target, dict) else target
        gold = {t["id"]: t["answers"]["text"] for t in target}
        for p in preds:
            if p["id"] not in gold:
                raise KeyError(f"no target with id {p['id']!r}")
            pt = _squad_norm(p["prediction_text"])
            em = f1 = 0.0
            for g in gold[p["id"]]:
                gt = _squad_norm(g)
                em = max(em, float(pt == gt))
                common = sum((Counter(pt) & Counter(gt)).values())
                if common:
                    pr, rc = common / len(pt), common / len(gt)
                    f1 = max(f1, 2 * pr * rc / (pr + rc))
                elif not pt and not gt:
                    f1 = 1.0
            self.em += em
            self.f1 += f1
            self.n += 1

    def compute(self) -> Dict[str, Tensor]:
        n = self.n.clamp(min=1)
        return {"exact_match": (100 * self.em / n).float(), "f1": (100 * self.f1 / n).float()}


__all__ = ["SacreBLEUScore", "CHRFScore", "TranslationEditRate", "ExtendedEditDistance", "SQuAD"]


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
