"""Presentation of attributions without a plotting backend: normalisation by sign and outlier
percentile, a blended red / blue heat-map as an image array, and HTML for word importances.
The matplotlib figures of the reference (``visualize_image_attr`` ...) need matplotlib and say
so; ``heat_map`` / ``save_heat_map`` give the same overlays as arrays or PNG files.
Reference: tensorplay/lumen/_utils/visualization.py."""
from __future__ import annotations

import html
from enum import Enum
from typing import Iterable, List, Optional, Union

import numpy as np
import torch


class VisualizeSign(Enum):
    positive = 1
    absolute_value = 2
    negative = 3
    all = 4


class ImageVisualizationMethod(Enum):
    heat_map = 1
    blended_heat_map = 2
    original_image = 3
    masked_image = 4
    alpha_scaling = 5


def _np(x) -> np.ndarray:
    return x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x)


def _cumulative_sum_threshold(values: np.ndarray, percentile: float) -> float:
    flat = np.sort(values.reshape(-1))
    cum = np.cumsum(flat)
    idx = int(np.searchsorted(cum, cum[-1] * 0.01 * percentile))
    return float(flat[min(idx, flat.size - 1)])


def normalize_attr(attr, sign: Union[str, VisualizeSign] = "absolute_value", outlier_perc: float = 2.0,
                   reduction_axis: Optional[int] = None) -> np.ndarray:
    """Attribution scaled into [-1, 1] (or [0, 1]): channels summed over ``reduction_axis``, the sign
    selected, and the scale set where the cumulative mass reaches ``100 - outlier_perc`` percent."""
    a = _np(attr).astype(np.float64)
    if reduction_axis is not None:
        a = a.sum(axis=reduction_axis)
    sign = VisualizeSign[sign] if isinstance(sign, str) else sign
    if sign == VisualizeSign.all:
        scale = _cumulative_sum_threshold(np.abs(a), 100 - outlier_perc)
    elif sign == VisualizeSign.positive:
        a = np.maximum(a, 0)
        scale = _cumulative_sum_threshold(a, 100 - outlier_perc)
    elif sign == VisualizeSign.negative:
        a = np.minimum(a, 0)
        scale = -_cumulative_sum_threshold(-a, 100 - outlier_perc)
    else:
        a = np.abs(a)
        scale = _cumulative_sum_threshold(a, 100 - outlier_perc)
    if abs(scale) < 1e-5:
        return np.zeros_like(a)
    return np.clip(a / scale, -1, 1)


def heat_map(attr, original_image=None, sign: str = "all", outlier_perc: float = 2.0, alpha_overlay: float = 0.5) -> np.ndarray:
    """``[H, W, 3]`` uint8 image: positive attribution red, negative blue, over white, or blended with
    the grey-scale ``original_image`` (``[H, W, C]`` in 0..1 or 0..255). ``attr`` is ``[H, W, C]`` or ``[H, W]``."""
    a = _np(attr)
    n = normalize_attr(a, sign, outlier_perc, reduction_axis=2 if a.ndim == 3 else None)
    if sign in ("absolute_value", "positive"):
        n = np.abs(n)
    rgb = np.ones(n.shape + (3,))
    pos, neg = np.clip(n, 0, 1), np.clip(-n, 0, 1)
    rgb[..., 1] -= pos + neg
    rgb[..., 2] -= pos
    rgb[..., 0] -= neg
    rgb = np.clip(rgb, 0, 1)
    if original_image is not None:
        img = _np(original_image).astype(np.float64)
        img = img / 255.0 if img.max() > 1.0 else img
        grey = img.mean(-1, keepdims=True) if img.ndim == 3 else img[..., None]
        rgb = (1 - alpha_overlay) * np.repeat(grey, 3, -1) + alpha_overlay * rgb
    return (rgb * 255).round().astype(np.uint8)


def save_heat_map(path, attr, original_image=None, **kw) -> str:
    from PIL import Image
    Image.fromarray(heat_map(attr, original_image, **kw)).save(path)
    return str(path)


def _needs_matplotlib(name: str):
    def fn(*a, **kw):
        try:
            import matplotlib  # noqa: F401
        except ImportError as e:
            raise ImportError(f"{name} draws with matplotlib, which is not installed; heat_map / save_heat_map / "
                              "format_word_importances work without it") from e
        raise NotImplementedError(f"{name}: figures are not part of this package; use heat_map() and plot the array")
    fn.__name__ = name
    return fn


visualize_image_attr = _needs_matplotlib("visualize_image_attr")
visualize_image_attr_multiple = _needs_matplotlib("visualize_image_attr_multiple")
visualize_timeseries_attr = _needs_matplotlib("visualize_timeseries_attr")


# ----------------------------------------------------------------------------- text
class VisualizationDataRecord:
    """One explained example for :func:`visualize_text`."""

    def __init__(self, word_attributions, pred_prob, pred_class, true_class, attr_class, attr_score, raw_input_ids,
                 convergence_score=None) -> None:
        self.word_attributions, self.pred_prob, self.pred_class = word_attributions, pred_prob, pred_class
        self.true_class, self.attr_class, self.attr_score = true_class, attr_class, attr_score
        self.raw_input_ids, self.convergence_score = raw_input_ids, convergence_score


def _get_color(attr: float) -> str:
    attr = max(-1.0, min(1.0, float(attr)))
    if attr > 0:
        return f"hsl(120, 75%, {100 - int(50 * attr)}%)"
    return f"hsl(0, 75%, {100 - int(-40 * attr)}%)"


def format_classname(classname) -> str:
    return f'<td><text style="padding-right:2em"><b>{html.escape(str(classname))}</b></text></td>'


def format_special_tokens(token: str) -> str:
    return "#" + token.strip("<>") if token.startswith("<") and token.endswith(">") else token


def format_word_importances(words: Iterable[str], importances) -> str:
    """A table cell in which every word carries a green (positive) or red (negative) background."""
    words = list(words)
    imp = _np(importances).reshape(-1).tolist() if importances is not None else []
    if not imp:
        return "<td></td>"
    assert len(words) <= len(imp), "one importance per word is needed"
    spans = []
    for w, v in zip(words, imp):
        spans.append(f'<mark style="background-color: {_get_color(v)}; opacity:1.0; line-height:1.75">'
                     f'<font color="black"> {html.escape(format_special_tokens(w))} </font></mark>')
    return "<td>" + "".join(spans) + "</td>"


def visualize_text(datarecords: Iterable[VisualizationDataRecord], legend: bool = True) -> str:
    """HTML table (returned as a string; shown as well when IPython is running) of the records."""
    rows = ["<tr><th>True Label</th><th>Predicted Label</th><th>Attribution Label</th><th>Attribution Score</th>"
            "<th>Word Importance</th></tr>"]
    for r in datarecords:
        rows.append("<tr>" + format_classname(r.true_class) + format_classname(f"{r.pred_class} ({float(r.pred_prob):.2f})")
                    + format_classname(r.attr_class) + format_classname(f"{float(r.attr_score):.2f}")
                    + format_word_importances(r.raw_input_ids, r.word_attributions) + "</tr>")
    doc = '<table width="100%">' + "".join(rows) + "</table>"
    if legend:
        doc = ('<div style="border-top: 1px solid; margin-top: 5px; padding-top: 5px"><b>Legend: </b>'
               + "".join(f'<span style="display:inline-block;width:10px;height:10px;border:1px solid;background-color:'
                         f'{_get_color(v)}"></span> {label}  ' for v, label in ((-1, "Negative"), (0, "Neutral"), (1, "Positive")))
               + "</div>") + doc
    try:
        from IPython.display import HTML, display
        display(HTML(doc))
    except Exception:
        pass
    return doc


__all__ = ["VisualizeSign", "ImageVisualizationMethod", "normalize_attr", "heat_map", "save_heat_map", "visualize_image_attr",
           "visualize_image_attr_multiple", "visualize_timeseries_attr", "VisualizationDataRecord", "format_classname",
           "format_special_tokens", "format_word_importances", "visualize_text"]


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
