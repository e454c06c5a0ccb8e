"""Interpretable surrogate models for the perturbation methods (tensorplay/lumen/_models/{model,linear_model}.py):
a linear model as an ``nn.Module`` whose ``fit`` takes a loader of ``(inputs, targets, weights)`` batches, trained either
by mini-batch SGD here (lasso, ridge, plain regression) or by scikit-learn's solvers."""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch
from torch import Tensor, nn

__all__ = ["Model", "LinearModel", "SGDLinearModel", "SGDLasso", "SGDRidge", "SGDLinearRegression", "SkLearnLinearModel",
           "SkLearnLasso", "SkLearnRidge", "SkLearnLinearRegression", "sgd_train_linear_model", "sklearn_train_linear_model"]


class Model:
    """What a surrogate model offers: ``fit(train_data)``, ``representation()`` (the importance of every feature),
    ``__call__``."""

    def fit(self, train_data, **kwargs) -> Optional[Dict[str, float]]:
        raise NotImplementedError

    def representation(self) -> Tensor:
        raise NotImplementedError

    def __call__(self, x: Tensor) -> Tensor:
        raise NotImplementedError


def _collect(loader):
    xs, ys, ws = [], [], []
    for batch in loader:
        x, y = batch[0], batch[1]
        w = batch[2] if len(batch) > 2 else torch.ones(x.shape[0])
        xs.append(x.reshape(x.shape[0], -1).float())
        ys.append(y.reshape(x.shape[0], -1).float())
        ws.append(w.reshape(-1).float())
    return torch.cat(xs), torch.cat(ys), torch.cat(ws)


def sgd_train_linear_model(model: "LinearModel", dataloader, construct_kwargs: dict, max_epoch: int = 100,
                           reduce_lr: bool = True, initial_lr: float = 0.01, alpha: float = 1.0, reg_term: Optional[int] = 1,
                           patience: int = 10, threshold: float = 1e-4, seed: int = 0, **_ignored) -> Dict[str, float]:
    """Weighted least squares by Adam over the loader's batches, with an L1 (``reg_term=1``) or L2 (``2``) penalty of
    weight ``alpha``; stops when the epoch loss has not improved by ``threshold`` for ``patience`` epochs."""
    x0, y0, _ = _collect(dataloader)
    model._construct_model_params(in_features=x0.shape[1], out_features=y0.shape[1], **construct_kwargs)
    torch.manual_seed(seed)
    opt = torch.optim.Adam(model.linear.parameters(), lr=initial_lr)
    sched = torch.optim.lr_scheduler.ReduceLROnPlateau(opt, factor=0.5, patience=max(1, patience // 2)) if reduce_lr else None
    best, stale, loss_v = float("inf"), 0, float("nan")
    for _epoch in range(max_epoch):
        total, count = 0.0, 0
        for batch in dataloader:
            x, y = batch[0].reshape(batch[0].shape[0], -1).float(), batch[1].reshape(batch[0].shape[0], -1).float()
            w = batch[2].reshape(-1, 1).float() if len(batch) > 2 else torch.ones(x.shape[0], 1)
            loss = ((model(x) - y).pow(2) * w).sum() / w.sum().clamp_min(1e-12) / 2
            if reg_term is not None and alpha > 0:
                loss = loss + alpha * model.linear.weight.norm(p=reg_term) ** (reg_term if reg_term == 2 else 1)
            opt.zero_grad()
            loss.backward()
            opt.step()
            total, count = total + float(loss.detach()) * x.shape[0], count + x.shape[0]
        loss_v = total / max(count, 1)
        if sched is not None:
            sched.step(loss_v)
        if loss_v < best - threshold:
            best, stale = loss_v, 0
        else:
            stale += 1
            if stale >= patience:
                break
    return {"train_loss": loss_v}


def sklearn_train_linear_model(model: "LinearModel", dataloader, construct_kwargs: dict, sklearn_trainer: str = "Lasso",
                               **fit_kwargs) -> Dict[str, float]:
    """Fits ``sklearn.linear_model.<sklearn_trainer>`` on everything the loader yields (sample weights passed through)
    and copies coefficients and intercept into the module."""
    import sklearn.linear_model as lm
    x, y, w = _collect(dataloader)
    est = getattr(lm, sklearn_trainer)(**fit_kwargs)
    try:
        est.fit(x.numpy(), y.numpy(), sample_weight=w.numpy())
    except TypeError:                                        # a solver without sample weights: scale rows instead
        s = w.sqrt().unsqueeze(1)
        est.fit((x * s).numpy(), (y * s).numpy())
    coef = torch.as_tensor(est.coef_, dtype=torch.float32).reshape(y.shape[1], x.shape[1])
    icpt = torch.as_tensor(getattr(est, "intercept_", 0.0), dtype=torch.float32).reshape(-1)
    model._construct_model_params(in_features=x.shape[1], out_features=y.shape[1], weight_values=coef,
                                  bias_value=icpt if icpt.numel() == y.shape[1] else icpt.expand(y.shape[1]).clone(),
                                  **construct_kwargs)
    with torch.no_grad():
        return {"train_loss": float(((model(x) - y).pow(2) * w.unsqueeze(1)).sum() / w.sum().clamp_min(1e-12) / 2)}


class LinearModel(nn.Module, Model):
    def __init__(self, train_fn: Callable, **kwargs) -> None:
        super().__init__()
        self.train_fn, self.construct_kwargs = train_fn, kwargs
        self.norm: Optional[nn.Module] = None
        self.linear: Optional[nn.Linear] = None

    def _construct_model_params(self, in_features: Optional[int] = None, out_features: Optional[int] = None,
                                norm_type: Optional[str] = None, affine_norm: bool = False, bias: bool = True,
                                weight_values: Optional[Tensor] = None, bias_value: Optional[Tensor] = None,
                                classes: Optional[Tensor] = None) -> None:
        if norm_type == "batch_norm":
            self.norm = nn.BatchNorm1d(in_features, eps=1e-8, affine=affine_norm)
        elif norm_type == "layer_norm":
            self.norm = nn.LayerNorm(in_features, eps=1e-8, elementwise_affine=affine_norm)
        elif norm_type is not None:
            raise ValueError(f"{norm_type!r} is not a supported norm type: 'batch_norm' or 'layer_norm'")
        if weight_values is not None:
            out_features, in_features = weight_values.shape
        self.linear = nn.Linear(in_features, out_features, bias=bias)
        with torch.no_grad():
            if weight_values is not None:
                self.linear.weight.copy_(weight_values)
            if bias_value is not None and bias:
                self.linear.bias.copy_(bias_value)
        self._classes = classes

    def fit(self, train_data, **kwargs) -> Optional[Dict[str, float]]:
        return self.train_fn(self, dataloader=train_data, construct_kwargs=self.construct_kwargs, **kwargs)

    def forward(self, x: Tensor) -> Tensor:
        if self.linear is None:
            raise RuntimeError("the model has not been fitted")
        x = x.reshape(x.shape[0], -1).float()
        return self.linear(self.norm(x) if self.norm is not None else x)

    def representation(self) -> Tensor:
        return self.linear.weight.detach()

    def bias(self) -> Optional[Tensor]:
        return None if self.linear is None or self.linear.bias is None else self.linear.bias.detach()

    def classes(self) -> Optional[Tensor]:
        return getattr(self, "_classes", None)


class SGDLinearModel(LinearModel):
    def __init__(self, **kwargs) -> None:
        super().__init__(train_fn=sgd_train_linear_model, **kwargs)


class SGDLasso(SGDLinearModel):
    def fit(self, train_data, **kwargs):
        return super().fit(train_data, reg_term=1, **kwargs)


class SGDRidge(SGDLinearModel):
    def fit(self, train_data, **kwargs):
        return super().fit(train_data, reg_term=2, **kwargs)


class SGDLinearRegression(SGDLinearModel):
    def fit(self, train_data, **kwargs):
        return super().fit(train_data, reg_term=None, alpha=0.0, **kwargs)


class SkLearnLinearModel(LinearModel):
    def __init__(self, sklearn_module: str, **kwargs) -> None:
        """``sklearn_module``: ``"linear_model.Lasso"`` (the ``linear_model.`` prefix may be left out)."""
        self.sklearn_trainer = sklearn_module.split(".")[-1]
        self.fit_kwargs = kwargs
        super().__init__(train_fn=sklearn_train_linear_model)

    def fit(self, train_data, **kwargs):
        return super().fit(train_data, sklearn_trainer=self.sklearn_trainer, **{**self.fit_kwargs, **kwargs})


class SkLearnLasso(SkLearnLinearModel):
    def __init__(self, **kwargs) -> None:
        super().__init__("linear_model.Lasso", **kwargs)


class SkLearnRidge(SkLearnLinearModel):
    def __init__(self, **kwargs) -> None:
        super().__init__("linear_model.Ridge", **kwargs)


class SkLearnLinearRegression(SkLearnLinearModel):
    def __init__(self, **kwargs) -> None:
        super().__init__("linear_model.LinearRegression", **kwargs)


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
