"""Interpretable inputs (text template, text tokens, image segments) and attribution of language
models over them, composable streaming statistics, baseline helpers, interpretable embedding layers.
Reference: tensorplay/lumen/_utils/interpretable_input.py, _utils/stat.py, _utils/baselines.py,
_utils/input_layer_wrapper.py, _core/llm_attr.py, _core/remote_provider.py."""
from __future__ import annotations

import abc
import random
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

import torch
from torch import Tensor, nn

# ----------------------------------------------------------------------------- statistics
StatValue = Union[Tensor, int, float]


class Stat:
    """One streaming statistic: ``update(x)`` with ``[batch, ...]`` tensors, ``get()`` the value.
    Statistics that build on others (variance on the mean ...) keep their own sufficient state,
    so every object is usable alone or inside :class:`SummarizerSingleTensor`."""

    def __init__(self, name: Optional[str] = None, **params) -> None:
        self.params, self._name = params, name
        self.init()

    @property
    def name(self) -> str:
        if self._name:
            return self._name
        shown = ", ".join(f"{k}={v}" for k, v in self.params.items() if v)      # default (falsy) parameters are not spelled
        return type(self).__name__.lower() + (f"({shown})" if shown else "")

    def init(self) -> None:
        pass

    def update(self, x: Tensor) -> None:
        raise NotImplementedError

    def get(self) -> Optional[StatValue]:
        raise NotImplementedError

    def __hash__(self):
        return hash((type(self), frozenset(self.params.items())))

    def __eq__(self, other):
        return type(self) is type(other) and self.params == other.params


class Count(Stat):
    def init(self):
        self.n = 0

    def update(self, x):
        self.n += x.shape[0]

    def get(self):
        return self.n or None


class Mean(Stat):
    def init(self):
        self.n, self.mean = 0, None

    def update(self, x):
        x = x.detach().double()
        n = x.shape[0]
        if self.mean is None:
            self.mean = torch.zeros_like(x[0])
        self.n += n
        self.mean = self.mean + (x.sum(0) - n * self.mean) / self.n

    def get(self):
        return self.mean


class MSE(Stat):
    """Sum of squared deviations from the running mean (Chan's pairwise update per batch)."""

    def init(self):
        self.n, self.mean, self.m2 = 0, None, None

    def update(self, x):
        x = x.detach().double()
        n = x.shape[0]
        bm = x.mean(0)
        bm2 = ((x - bm) ** 2).sum(0)
        if self.mean is None:
            self.n, self.mean, self.m2 = n, bm, bm2
            return
        d = bm - self.mean
        tot = self.n + n
        self.m2 = self.m2 + bm2 + d * d * self.n * n / tot
        self.mean = self.mean + d * n / tot
        self.n = tot

    def get(self):
        return self.m2


class Var(MSE):
    """Variance with ``order`` delta degrees of freedom (0: population, 1: sample)."""

    def __init__(self, name: Optional[str] = None, order: int = 0) -> None:
        super().__init__(name=name, order=order)

    def get(self):
        if self.m2 is None:
            return None
        if self.n - self.params["order"] <= 0:
            return torch.zeros_like(self.m2)
        return self.m2 / (self.n - self.params["order"])


class StdDev(Var):
    def get(self):
        v = super().get()
        return None if v is None else v.sqrt()


class GeneralAccumFn(Stat):
    def __init__(self, fn: Callable[[Tensor, Tensor], Tensor], name: Optional[str] = None) -> None:
        self.fn = fn
        super().__init__(name=name)

    def init(self):
        self.value = None

    def update(self, x):
        x = x.detach()
        for row in x:
            self.value = row.clone() if self.value is None else self.fn(self.value, row)

    def get(self):
        return self.value


class Min(GeneralAccumFn):
    def __init__(self, name: Optional[str] = None) -> None:
        super().__init__(torch.minimum, name)

    def update(self, x):
        m = x.detach().amin(0)
        self.value = m if self.value is None else torch.minimum(self.value, m)


class Max(GeneralAccumFn):
    def __init__(self, name: Optional[str] = None) -> None:
        super().__init__(torch.maximum, name)

    def update(self, x):
        m = x.detach().amax(0)
        self.value = m if self.value is None else torch.maximum(self.value, m)


class Sum(GeneralAccumFn):
    def __init__(self, name: Optional[str] = None) -> None:
        super().__init__(torch.add, name)

    def update(self, x):
        s = x.detach().sum(0)
        self.value = s if self.value is None else self.value + s


class SummarizerSingleTensor:
    """Updates a list of :class:`Stat` objects with every batch; ``summary`` maps the names of the
    chosen ones (``summary_stats_indices``; default all) to their values."""

    def __init__(self, stats: List[Stat], summary_stats_indices: Optional[List[int]] = None) -> None:
        self._stats = list(stats)
        idx = range(len(stats)) if summary_stats_indices is None else summary_stats_indices
        self._summary_stats = [self._stats[i] for i in idx]
        for s in self._stats:
            s.init()

    def update(self, x: Tensor) -> None:
        for s in self._stats:
            s.update(x)

    @property
    def summary(self) -> Dict[str, Optional[StatValue]]:
        return {s.name: s.get() for s in self._summary_stats}


# ----------------------------------------------------------------------------- baselines and embeddings
class ProductBaselines:
    """Callable baseline: every call draws one value per feature, independently, from that
    feature's list (``{"name": [...]}`` gives dicts, a list of lists gives lists; a tuple key spans
    several features that are drawn together)."""

    def __init__(self, baseline_values: Union[List[List[Any]], Dict[Union[str, tuple], List[Any]]], seed: Optional[int] = None) -> None:
        if isinstance(baseline_values, dict):
            self.keys, values = list(baseline_values.keys()), list(baseline_values.values())
        else:
            self.keys, values = None, baseline_values
        self.values = values
        self.rng = random.Random(seed)

    def sample(self):
        picks = [self.rng.choice(v) for v in self.values]
        if self.keys is None:
            return picks
        out = {}
        for k, p in zip(self.keys, picks):
            if isinstance(k, tuple):
                out.update(dict(zip(k, p)))
            else:
                out[k] = p
        return out

    __call__ = sample


class TokenReferenceBase:
    """Reference (baseline) token sequences: ``reference_token_idx`` repeated (usually PAD)."""

    def __init__(self, reference_token_idx: int = 0) -> None:
        self.reference_token_idx = reference_token_idx

    def generate_reference(self, sequence_length: int, device=None) -> Tensor:
        return torch.full((sequence_length,), self.reference_token_idx, dtype=torch.long, device=device)


class InterpretableEmbeddingBase(nn.Module):
    """Stands in for an embedding layer so that attribution can run on the embeddings: ``forward``
    passes its input through unchanged (the caller feeds precomputed embeddings),
    ``indices_to_embeddings`` applies the wrapped layer."""

    def __init__(self, embedding: nn.Module, full_name: str) -> None:
        super().__init__()
        self.embedding, self.full_name = embedding, full_name
        self.num_embeddings = getattr(embedding, "num_embeddings", None)
        self.embedding_dim = getattr(embedding, "embedding_dim", None)

    def forward(self, *inputs, **kwargs):
        return inputs[0] if inputs else next(iter(kwargs.values()))

    def indices_to_embeddings(self, *inputs, **kwargs) -> Tensor:
        return self.embedding(*inputs, **kwargs)


def _parent_and_leaf(model: nn.Module, name: str):
    parts = name.split(".")
    parent = model
    for p in parts[:-1]:
        parent = getattr(parent, p)
    return parent, parts[-1]


def configure_interpretable_embedding_layer(model: nn.Module, embedding_layer_name: str = "embedding") -> InterpretableEmbeddingBase:
    parent, leaf = _parent_and_leaf(model, embedding_layer_name)
    layer = getattr(parent, leaf)
    if isinstance(layer, InterpretableEmbeddingBase):
        raise AssertionError(f"{embedding_layer_name} is already an interpretable embedding layer")
    wrapped = InterpretableEmbeddingBase(layer, embedding_layer_name)
    setattr(parent, leaf, wrapped)
    return wrapped


def remove_interpretable_embedding_layer(model: nn.Module, interpretable_emb: InterpretableEmbeddingBase) -> None:
    parent, leaf = _parent_and_leaf(model, interpretable_emb.full_name)
    setattr(parent, leaf, interpretable_emb.embedding)


# ----------------------------------------------------------------------------- interpretable inputs
class InterpretableInput(abc.ABC):
    """An input seen as a few interpretable features: ``to_tensor`` gives their presence vector
    ``[1, n]`` (all ones), ``to_model_input(perturbed)`` builds what the model takes when some
    are absent (0), ``format_attr`` maps attributions of the interpretable features back onto
    ``values`` (features that share a mask id share their attribution)."""

    values: List[str]

    @abc.abstractmethod
    def to_tensor(self) -> Tensor: ...

    @abc.abstractmethod
    def to_model_input(self, perturbed_tensor: Optional[Tensor] = None) -> Any: ...

    def format_attr(self, itp_attr: Tensor) -> Tensor:
        return itp_attr


class TextTemplateInput(InterpretableInput):
    def __init__(self, template: Union[str, Callable[..., str]], values: Union[List[str], Dict[str, str]],
                 baselines: Union[List[str], Dict[str, str], Callable, None] = None,
                 mask: Union[List[int], Dict[str, int], None] = None) -> None:
        self.dict_keys = list(values.keys()) if isinstance(values, dict) else []
        self.values = [values[k] for k in self.dict_keys] if self.dict_keys else list(values)
        n = len(self.values)
        if baselines is not None and not callable(baselines):
            baselines = [baselines[k] for k in self.dict_keys] if isinstance(baselines, dict) else list(baselines)
            assert len(baselines) == n, "one baseline per value"
        self.baselines = baselines
        if mask is None:
            self.mask, self.n_itp_features = None, n
        else:
            mask = [mask[k] for k in self.dict_keys] if isinstance(mask, dict) else list(mask)
            ids = {m: i for i, m in enumerate(sorted(set(mask)))}
            self.mask = [ids[m] for m in mask]
            self.n_itp_features = len(ids)
        self.format_fn = template.format if isinstance(template, str) else template

    def to_tensor(self) -> Tensor:
        return torch.ones(1, self.n_itp_features)

    def to_model_input(self, perturbed_tensor: Optional[Tensor] = None) -> str:
        values = list(self.values)
        if perturbed_tensor is not None:
            base = self.baselines() if callable(self.baselines) else self.baselines
            if isinstance(base, dict):
                base = [base[k] for k in self.dict_keys]
            present = perturbed_tensor.reshape(-1)
            for i in range(len(values)):
                j = self.mask[i] if self.mask is not None else i
                if not bool(present[j]):
                    values[i] = base[i] if base is not None else ""
        if self.dict_keys:
            return self.format_fn(**dict(zip(self.dict_keys, values)))
        return self.format_fn(*values)

    def format_attr(self, itp_attr: Tensor) -> Tensor:
        if self.mask is None:
            return itp_attr
        return itp_attr[..., torch.tensor(self.mask, device=itp_attr.device)]


class TextTokenInput(InterpretableInput):
    """Every token of ``text`` is a feature, except ``skip_tokens`` (ids or token strings), which
    always stay; an absent token becomes ``baselines`` (an id or a token string, usually UNK)."""

    def __init__(self, text: str, tokenizer, baselines: Union[int, str] = 0, skip_tokens: Optional[Sequence] = None) -> None:
        ids = tokenizer.encode(text, return_tensors="pt")
        ids = torch.as_tensor(ids).reshape(1, -1)
        self.inp_tensor = ids
        if skip_tokens:
            skip = list(skip_tokens)
            if isinstance(skip[0], str):
                skip = tokenizer.convert_tokens_to_ids(skip)
            self.itp_mask = ~torch.isin(ids, torch.tensor(skip))
            itp_ids = ids[self.itp_mask][None]
        else:
            self.itp_mask, itp_ids = None, ids
        self.itp_tensor = itp_ids
        self.values = list(tokenizer.convert_ids_to_tokens(itp_ids[0].tolist()))
        self.tokenizer = tokenizer
        self.n_itp_features = len(self.values)
        self.baselines = baselines if isinstance(baselines, int) else tokenizer.convert_tokens_to_ids([baselines])[0]

    def to_tensor(self) -> Tensor:
        return torch.ones(1, self.n_itp_features)

    def to_model_input(self, perturbed_tensor: Optional[Tensor] = None) -> Tensor:
        if perturbed_tensor is None:
            return self.inp_tensor
        present = perturbed_tensor.reshape(1, -1).bool().to(self.inp_tensor.device)
        itp = torch.where(present, self.itp_tensor, torch.full_like(self.itp_tensor, self.baselines))
        if self.itp_mask is None:
            return itp
        out = self.inp_tensor.clone()
        out[self.itp_mask] = itp[0]
        return out


class ImageMaskInput(InterpretableInput):
    """Segments of an image as features: ``mask`` holds a segment id per pixel (``[H, W]``), or
    ``mask_list`` one boolean mask per segment (they may overlap); absent segments are painted
    with ``baseline`` before ``processor_fn`` turns the image into the model's input."""

    def __init__(self, image, mask: Optional[Tensor] = None, mask_list: Optional[List[Tensor]] = None,
                 baseline=(255, 255, 255), processor_fn: Callable = lambda x: x) -> None:
        self.image, self.baseline, self.processor_fn = image, baseline, processor_fn
        h, w = image.size[1], image.size[0]
        if mask_list is not None:
            for m in mask_list:
                assert tuple(m.shape) == (h, w), "every mask must have the image's height and width"
            self.mask_list = [m.bool() for m in mask_list]
        elif mask is not None:
            assert tuple(mask.shape) == (h, w), "mask must have the image's height and width"
            self.mask_list = [mask == i for i in mask.unique().tolist()]
        else:
            self.mask_list = [torch.ones(h, w, dtype=torch.bool)]
        self.values = [f"image_feature_{i}" for i in range(len(self.mask_list))]
        self.n_itp_features = len(self.mask_list)

    def to_tensor(self) -> Tensor:
        return torch.ones(1, self.n_itp_features)

    def get_mask_list(self) -> List[Tensor]:
        return self.mask_list

    def to_model_input(self, perturbed_tensor: Optional[Tensor] = None) -> Any:
        if perturbed_tensor is None:
            return self.processor_fn(self.image)
        import numpy as np
        from PIL import Image
        arr = np.array(self.image).copy()
        present = perturbed_tensor.reshape(-1)
        for i, m in enumerate(self.mask_list):
            if not bool(present[i]):
                arr[m.numpy()] = np.array(self.baseline[: arr.shape[-1]] if arr.ndim == 3 else self.baseline[0], dtype=arr.dtype)
        return self.processor_fn(Image.fromarray(arr))

    def format_pixel_attr(self, itp_attr: Tensor) -> Tensor:
        """Attribution per pixel ``[..., H, W]``: the sum of the attributions of the segments that cover it."""
        lead = itp_attr.shape[:-1]
        out = torch.zeros(*lead, *self.mask_list[0].shape, dtype=itp_attr.dtype)
        for i, m in enumerate(self.mask_list):
            out = out + itp_attr[..., i].reshape(*lead, 1, 1) * m.to(itp_attr.dtype)
        return out


# ----------------------------------------------------------------------------- language-model attribution
class LLMAttributionResult:
    """``seq_attr [n_input_features]`` (attribution to the whole target), ``token_attr
    [n_target_tokens, n_input_features]`` (None for the surrogate methods), the input feature
    names, the target tokens and their probabilities."""

    def __init__(self, *, input_tokens: List[str], output_tokens: List[str], seq_attr, token_attr=None, output_probs=None,
                 inp: Optional[InterpretableInput] = None) -> None:
        self.input_tokens, self.output_tokens, self.inp = input_tokens, output_tokens, inp
        self.seq_attr = torch.as_tensor(seq_attr)
        self.token_attr = None if token_attr is None else torch.as_tensor(token_attr)
        self.output_probs = None if output_probs is None else torch.as_tensor(output_probs)

    @property
    def seq_attr_dict(self) -> Dict[str, float]:
        return {k: float(v) for k, v in zip(self.input_tokens, self.seq_attr.tolist())}

    def _pyplot(self):
        try:
            import matplotlib.pyplot as plt
        except ImportError as e:
            raise ImportError("plotting attribution results needs matplotlib, which is not installed") from e
        return plt

    def plot_seq_attr(self, show: bool = False):
        plt = self._pyplot()
        fig, ax = plt.subplots()
        ax.bar(range(len(self.input_tokens)), self.seq_attr.tolist())
        ax.set_xticks(range(len(self.input_tokens)), self.input_tokens, rotation=45, ha="right")
        if show:
            plt.show()
            return None
        return fig, ax

    def plot_token_attr(self, show: bool = False):
        if self.token_attr is None:
            raise ValueError("this result has no per-token attribution (the method explains the whole sequence only)")
        plt = self._pyplot()
        fig, ax = plt.subplots()
        lim = float(self.token_attr.abs().max()) or 1.0
        ax.imshow(self.token_attr.numpy(), cmap="bwr", vmin=-lim, vmax=lim)
        ax.set_xticks(range(len(self.input_tokens)), self.input_tokens, rotation=45, ha="right")
        ax.set_yticks(range(len(self.output_tokens)), self.output_tokens)
        if show:
            plt.show()
            return None
        return fig, ax


class RemoteLLMProvider(abc.ABC):
    """A language model behind a service: text generation and log-probabilities of a given
    continuation, which is all that perturbation attribution needs."""

    api_url: str

    @abc.abstractmethod
    def generate(self, prompt: str, **gen_args: Any) -> str: ...

    @abc.abstractmethod
    def get_logprobs(self, input_prompt: str, target_str: str, tokenizer=None) -> List[float]: ...


class VLLMProvider(RemoteLLMProvider):
    """Client of a vLLM server's OpenAI-compatible completions endpoint (``api_url`` like
    ``http://host:8000``). Log-probabilities of the target come from a one-token completion of
    ``prompt + target`` with ``echo`` and ``logprobs`` on, of which the target's tokens are kept."""

    def __init__(self, api_url: str, model_name: Optional[str] = None, timeout: float = 60.0) -> None:
        if not api_url.strip():
            raise ValueError("api_url must not be empty")
        self.api_url, self.model_name, self.timeout = api_url.rstrip("/"), model_name, timeout

    def _post(self, payload: Dict[str, Any]) -> Dict[str, Any]:
        import requests
        if self.model_name is None:
            models = requests.get(self.api_url + "/v1/models", timeout=self.timeout).json()
            self.model_name = models["data"][0]["id"]
        r = requests.post(self.api_url + "/v1/completions", json={"model": self.model_name, **payload}, timeout=self.timeout)
        r.raise_for_status()
        return r.json()

    def generate(self, prompt: str, **gen_args: Any) -> str:
        if "max_new_tokens" in gen_args:
            gen_args["max_tokens"] = gen_args.pop("max_new_tokens")
        gen_args.pop("do_sample", None)
        out = self._post({"prompt": prompt, **gen_args})
        if not out.get("choices"):
            raise KeyError("the server's answer has no 'choices'")
        return out["choices"][0]["text"]

    def get_logprobs(self, input_prompt: str, target_str: str, tokenizer=None) -> List[float]:
        if tokenizer is None:
            raise ValueError("a tokenizer is needed to count the target's tokens")
        n = len(tokenizer.encode(target_str, add_special_tokens=False))
        out = self._post({"prompt": input_prompt + target_str, "max_tokens": 1, "temperature": 0.0, "echo": True, "logprobs": 0})
        lp = out["choices"][0]["logprobs"]["token_logprobs"]
        prompt_and_target = lp[:-1]                        # the last entry is the one generated token
        if len(prompt_and_target) < n:
            raise ValueError("the server returned fewer log-probabilities than the target has tokens")
        return [float(v) for v in prompt_and_target[-n:]]


class LLMAttribution:
    """Attribution of a causal language model's response to the interpretable features of its
    prompt. ``attr_method`` is a perturbation method built on the model (``FeatureAblation(model)``,
    ``ShapleyValueSampling``, ``ShapleyValues``, ``Lime``, ``KernelShap``); the model is called as
    ``model(input_ids)`` and returns logits ``[1, T, V]`` (or an object with ``.logits``), and offers
    ``generate(input_ids, **gen_args)`` when no target is given. One model call scores all target
    tokens of a perturbed prompt and is cached, so the per-token attributions re-use the calls made
    for the sequence attribution."""

    def __init__(self, attr_method, tokenizer, attr_target: str = "log_prob") -> None:
        if attr_target not in ("log_prob", "prob"):
            raise ValueError("attr_target is 'log_prob' or 'prob'")
        from .perturbation import Lime
        self.attr_method, self.tokenizer, self.attr_target = attr_method, tokenizer, attr_target
        self.model = attr_method.forward_func
        self.include_per_token_attr = not isinstance(attr_method, Lime)
        try:
            self.device = next(self.model.parameters()).device
        except (AttributeError, StopIteration):
            self.device = torch.device("cpu")

    # -- scoring of one perturbed prompt
    def _encode(self, model_input) -> Tensor:
        if isinstance(model_input, str):
            model_input = self.tokenizer.encode(model_input, return_tensors="pt")
        return torch.as_tensor(model_input).reshape(1, -1).to(self.device)

    def _target_log_probs(self, model_input, target_ids: Tensor) -> Tensor:
        ids = self._encode(model_input)
        with torch.no_grad():
            out = self.model(torch.cat((ids, target_ids[None].to(self.device)), 1))
        logits = getattr(out, "logits", out)
        logp = torch.log_softmax(logits[0, ids.shape[1] - 1: -1].float(), -1)
        return logp.gather(1, target_ids[:, None].to(logp.device))[:, 0].cpu()

    def _target_ids(self, inp: InterpretableInput, target, gen_args) -> Tensor:
        if target is None:
            ids = self._encode(inp.to_model_input())
            gen_args = {"max_new_tokens": 25, "do_sample": False, **(gen_args or {})}
            with torch.no_grad():
                out = self.model.generate(ids, **gen_args)
            return torch.as_tensor(out)[0, ids.shape[1]:].cpu()
        if isinstance(target, str):
            try:
                enc = self.tokenizer.encode(target, add_special_tokens=False)
            except TypeError:
                enc = self.tokenizer.encode(target)
            return torch.as_tensor(enc).reshape(-1)
        return torch.as_tensor(target).reshape(-1)

    def attribute(self, inp: InterpretableInput, target=None, num_trials: int = 1, gen_args: Optional[Dict[str, Any]] = None,
                  **kwargs) -> LLMAttributionResult:
        target_ids = self._target_ids(inp, target, gen_args)
        cache: Dict[tuple, Tensor] = {}

        def scores(z: Tensor) -> Tensor:
            rows = []
            for row in z.reshape(-1, z.shape[-1]):
                key = tuple(row.tolist())
                if key not in cache:
                    cache[key] = self._target_log_probs(inp.to_model_input(row[None]), target_ids)
                rows.append(cache[key])
            lp = torch.stack(rows)
            return lp if self.attr_target == "log_prob" else lp.exp()

        def seq_forward(z):
            s = scores(z)
            return s.sum(-1) if self.attr_target == "log_prob" else s.prod(-1)

        z0 = inp.to_tensor()
        saved = self.attr_method.forward_func
        try:
            seq = torch.zeros(inp.n_itp_features if hasattr(inp, "n_itp_features") else z0.shape[1])
            tok = torch.zeros(target_ids.numel(), seq.numel()) if self.include_per_token_attr else None
            for _ in range(num_trials):
                self.attr_method.forward_func = seq_forward
                seq = seq + self.attr_method.attribute(z0, **kwargs).reshape(-1).float()
                if tok is not None:
                    for t in range(target_ids.numel()):
                        self.attr_method.forward_func = lambda z, t=t: scores(z)[:, t]
                        tok[t] += self.attr_method.attribute(z0, **kwargs).reshape(-1).float()
        finally:
            self.attr_method.forward_func = saved
        seq = inp.format_attr(seq / num_trials)
        tok = None if tok is None else inp.format_attr(tok / num_trials)
        probs = scores(z0)[0] if self.attr_target == "prob" else scores(z0)[0].exp()
        return LLMAttributionResult(input_tokens=list(inp.values), seq_attr=seq, token_attr=tok, output_probs=probs, inp=inp,
                                    output_tokens=list(self.tokenizer.convert_ids_to_tokens(target_ids.tolist())))


class RemoteLLMAttribution(LLMAttribution):
    """The same over a :class:`RemoteLLMProvider`: the prompt goes out as text, the provider
    returns the target's log-probabilities; nothing runs locally but the perturbation loop."""

    def __init__(self, attr_method, tokenizer, provider: RemoteLLMProvider, attr_target: str = "log_prob") -> None:
        super().__init__(attr_method, tokenizer, attr_target)
        self.provider = provider
        self.device = torch.device("cpu")

    def _as_text(self, model_input) -> str:
        return model_input if isinstance(model_input, str) else self.tokenizer.decode(torch.as_tensor(model_input).reshape(-1).tolist())

    def _target_ids(self, inp, target, gen_args) -> Tensor:
        if target is None:
            target = self.provider.generate(self._as_text(inp.to_model_input()), **(gen_args or {}))
        return super()._target_ids(inp, target, gen_args)

    def _target_log_probs(self, model_input, target_ids: Tensor) -> Tensor:
        target_str = self.tokenizer.decode(target_ids.tolist())
        lp = self.provider.get_logprobs(self._as_text(model_input), target_str, self.tokenizer)
        if len(lp) != target_ids.numel():
            raise ValueError(f"the provider returned {len(lp)} log-probabilities for {target_ids.numel()} target tokens")
        return torch.tensor(lp, dtype=torch.float32)


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
