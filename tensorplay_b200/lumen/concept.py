"""Concept-based interpretation: concept activation vectors and TCAV scores
(tensorplay/lumen/concept/_core/{concept,cav,tcav}.py, concept/_utils/classifier.py).

A concept is a set of example inputs. Its activation vector (CAV) at a layer is the normal of a linear classifier
that separates the layer's activations on the concept's examples from those on another concept's (usually random
inputs). The TCAV score of a concept for a target is the share of inputs whose target output increases along the
CAV: the directional derivative of the output with respect to the layer's activation, projected on the CAV.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch
from torch import Tensor, nn

__all__ = ["Concept", "ConceptInterpreter", "Classifier", "DefaultClassifier", "CAV", "TCAV"]


class Concept:
    """``data_iter``: an iterable of input batches (tensors) that show the concept."""

    def __init__(self, id: int, name: str, data_iter: Optional[Iterable[Tensor]]):
        self.id, self.name, self.data_iter = id, name, data_iter

    @property
    def identifier(self) -> str:
        return f"{self.name}-{self.id}"

    def __repr__(self) -> str:
        return f"Concept({self.id}, {self.name!r})"


class ConceptInterpreter:
    """Base of the concept-based methods: holds the model, subclasses define ``interpret``."""

    def __init__(self, model: nn.Module):
        self.model = model

    def interpret(self, inputs, experimental_sets, target=None, **kwargs):
        raise NotImplementedError


class Classifier:
    """What CAV training needs from a linear classifier: ``train_and_eval`` on (activation, label) batches, then
    ``weights()`` ``[classes, features]`` and ``classes()``."""

    def train_and_eval(self, dataloader, **kwargs) -> Optional[Dict[str, Any]]:
        raise NotImplementedError

    def weights(self) -> Tensor:
        raise NotImplementedError

    def classes(self) -> List[int]:
        raise NotImplementedError


class DefaultClassifier(Classifier):
    """Multinomial logistic regression by full-batch L-BFGS on standardised activations, with a held-out third for the
    accuracy that ``train_and_eval`` reports."""

    def __init__(self, l2: float = 1e-3, max_iter: int = 100, test_split_ratio: float = 0.33, seed: int = 0):
        self.l2, self.max_iter, self.test_split_ratio, self.seed = l2, max_iter, test_split_ratio, seed
        self._w: Optional[Tensor] = None
        self._classes: List[int] = []

    def train_and_eval(self, dataloader, **kwargs) -> Dict[str, Any]:
        xs, ys = [], []
        for x, y in dataloader:
            xs.append(x.reshape(x.shape[0], -1).float())
            ys.append(y.reshape(-1).long())
        x, y = torch.cat(xs), torch.cat(ys)
        self._classes = sorted(set(y.tolist()))
        idx = torch.tensor([self._classes.index(int(v)) for v in y.tolist()])
        g = torch.Generator().manual_seed(self.seed)
        perm = torch.randperm(x.shape[0], generator=g)
        n_test = int(x.shape[0] * self.test_split_ratio)
        test, train = perm[:n_test], perm[n_test:]
        mu, sd = x[train].mean(0, keepdim=True), x[train].std(0, keepdim=True).clamp_min(1e-6)
        xn = (x - mu) / sd
        w = torch.zeros(len(self._classes), x.shape[1] + 1, requires_grad=True)
        opt = torch.optim.LBFGS([w], max_iter=self.max_iter, line_search_fn="strong_wolfe")
        xa = torch.cat((xn, torch.ones(x.shape[0], 1)), dim=1)

        def closure():
            opt.zero_grad()
            loss = torch.nn.functional.cross_entropy(xa[train] @ w.t(), idx[train]) + self.l2 * w[:, :-1].pow(2).sum()
            loss.backward()
            return loss
        opt.step(closure)
        with torch.no_grad():
            self._w = (w[:, :-1] / sd).detach()          # back to the scale of the raw activations
            acc = ((xa[test] @ w.t()).argmax(1) == idx[test]).float().mean() if n_test else torch.tensor(float("nan"))
        return {"accs": acc.detach()}

    def weights(self) -> Tensor:
        if self._w is None:
            raise RuntimeError("the classifier has not been trained")
        w = self._w
        # two classes: a softmax classifier's two rows are one direction and its negative up to a shift
        return torch.stack((w[0] - w[1], w[1] - w[0])) / 2 if w.shape[0] == 2 else w

    def classes(self) -> List[int]:
        return list(self._classes)


class CAV:
    """Activation vectors of the concepts of one experimental set at one layer, with the classifier's statistics."""

    def __init__(self, concepts: Sequence[Concept], layer: str, stats: Optional[Dict[str, Any]] = None):
        self.concepts, self.layer, self.stats = list(concepts), layer, stats

    def vector(self, concept: Concept) -> Tensor:
        i = self.stats["classes"].index(concept.id)
        return self.stats["weights"][i]


def _layer_of(model: nn.Module, name: str) -> nn.Module:
    return model.get_submodule(name)


def _activations(model: nn.Module, layer: nn.Module, x: Tensor) -> Tensor:
    got: List[Tensor] = []
    h = layer.register_forward_hook(lambda m, i, o: got.append(o[0] if isinstance(o, tuple) else o))
    try:
        with torch.no_grad():
            model(x)
    finally:
        h.remove()
    return got[0].detach()


class TCAV(ConceptInterpreter):
    def __init__(self, model: nn.Module, layers: Union[str, Sequence[str]], classifier: Optional[Classifier] = None,
                 **classifier_kwargs):
        super().__init__(model)
        self.layers = [layers] if isinstance(layers, str) else list(layers)
        self.classifier = classifier if classifier is not None else DefaultClassifier(**classifier_kwargs)
        self.cavs: Dict[str, Dict[str, CAV]] = {}      # experimental-set key -> layer -> CAV

    @staticmethod
    def _key(concepts: Sequence[Concept]) -> str:
        return "-".join(str(c.id) for c in concepts)

    def compute_cavs(self, experimental_sets: Sequence[Sequence[Concept]], force_train: bool = False):
        for concepts in experimental_sets:
            key = self._key(concepts)
            for lname in self.layers:
                if not force_train and key in self.cavs and lname in self.cavs[key]:
                    continue
                layer = _layer_of(self.model, lname)
                batches: List[Tuple[Tensor, Tensor]] = []
                for c in concepts:
                    for x in c.data_iter:
                        a = _activations(self.model, layer, x)
                        batches.append((a.reshape(a.shape[0], -1), torch.full((a.shape[0],), c.id)))
                stats = dict(self.classifier.train_and_eval(batches) or {})
                stats["weights"], stats["classes"] = self.classifier.weights().detach(), self.classifier.classes()
                self.cavs.setdefault(key, {})[lname] = CAV(concepts, lname, stats)
        return self.cavs

    def interpret(self, inputs: Tensor, experimental_sets: Sequence[Sequence[Concept]], target=None,
                  additional_forward_args=None, **kwargs) -> Dict[str, Dict[str, Dict[str, Tensor]]]:
        """``{set key: {layer: {"sign_count": [concepts], "magnitude": [concepts]}}}``: the share of inputs whose target
        output grows along each concept's vector, and the positive share of the summed sensitivities."""
        self.compute_cavs(experimental_sets)
        out: Dict[str, Dict[str, Dict[str, Tensor]]] = {}
        for lname in self.layers:
            layer = _layer_of(self.model, lname)
            kept: List[Tensor] = []

            def hook(m, i, o):
                t = o[0] if isinstance(o, tuple) else o
                t.retain_grad()
                kept.append(t)
            h = layer.register_forward_hook(hook)
            try:
                x = inputs.detach().requires_grad_(True) if inputs.is_floating_point() else inputs
                args = () if additional_forward_args is None else tuple(additional_forward_args)
                y = self.model(x, *args)
                y = y if target is None else (y[:, target] if isinstance(target, int) else y.gather(1, target.view(-1, 1))[:, 0])
                y.sum().backward()
            finally:
                h.remove()
            grad = kept[0].grad.reshape(kept[0].shape[0], -1)                  # [N, features]
            for concepts in experimental_sets:
                key = self._key(concepts)
                cav = self.cavs[key][lname]
                W = cav.stats["weights"].to(grad)                               # [classes, features]
                order = [cav.stats["classes"].index(c.id) for c in concepts]
                sens = grad @ W[order].t()                                      # [N, concepts]
                sign = (sens > 0).float().mean(0)
                mag = (sens * (sens > 0)).abs().sum(0) / sens.abs().sum(0).clamp_min(1e-12)
                out.setdefault(key, {})[lname] = {"sign_count": sign, "magnitude": mag}
        return out


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
