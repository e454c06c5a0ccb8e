"""Regression, divergence, aggregation metrics and wrappers against scikit-learn / scipy formulas."""
import numpy as np
import torch
from scipy import stats
from sklearn import metrics as skm

from tensorplay_b200 import metrics as M
from tensorplay_b200.metrics import regression as R


def _upd(m, p, t):
    h = len(p) // 2
    m.update(p[:h], t[:h])
    m.update(p[h:], t[h:])
    return float(m.compute())


def test_regression_metrics_match_sklearn():
    g = torch.Generator().manual_seed(0)
    t = torch.rand(200, generator=g).double() * 5 + 0.5
    p = (t + torch.randn(200, generator=g).double() * 0.5).clamp(min=0.05)
    tn, pn = t.numpy(), p.numpy()
    assert abs(_upd(R.MeanAbsolutePercentageError(), p, t) - skm.mean_absolute_percentage_error(tn, pn)) < 1e-6
    assert abs(_upd(R.MeanSquaredLogError(), p, t) - skm.mean_squared_log_error(tn, pn)) < 1e-6
    assert abs(_upd(R.ExplainedVariance(), p, t) - skm.explained_variance_score(tn, pn)) < 1e-6
    assert abs(_upd(R.SymmetricMeanAbsolutePercentageError(), p, t) - np.mean(2 * np.abs(pn - tn) / (np.abs(pn) + np.abs(tn)))) < 1e-6
    assert abs(_upd(R.WeightedMeanAbsolutePercentageError(), p, t) - np.abs(pn - tn).sum() / np.abs(tn).sum()) < 1e-6
    assert abs(_upd(R.LogCoshError(), p, t) - np.mean(np.log(np.cosh(pn - tn)))) < 1e-6
    assert abs(_upd(R.MinkowskiDistance(3.0), p, t) - (np.abs(pn - tn) ** 3).sum() ** (1 / 3)) < 1e-5
    assert abs(_upd(R.RelativeSquaredError(), p, t) - ((tn - pn) ** 2).sum() / ((tn - tn.mean()) ** 2).sum()) < 1e-6
    assert abs(_upd(R.NormalizedRootMeanSquaredError(), p, t) - np.sqrt(((tn - pn) ** 2).mean()) / tn.mean()) < 1e-6
    ccc = 2 * np.cov(pn, tn, bias=True)[0, 1] / (pn.var() + tn.var() + (pn.mean() - tn.mean()) ** 2)
    assert abs(_upd(R.ConcordanceCorrCoef(), p, t) - ccc) < 1e-6
    for power in (0.0, 1.0, 2.0, 1.5):
        assert abs(_upd(R.TweedieDevianceScore(power), p, t) - skm.mean_tweedie_deviance(tn, pn, power=power)) < 1e-5
    a, b = torch.rand(20, 6, generator=g).double(), torch.rand(20, 6, generator=g).double()
    cos = np.mean([1 - __import__("scipy.spatial.distance", fromlist=["cosine"]).cosine(x, y) for x, y in zip(a.numpy(), b.numpy())])
    assert abs(_upd(R.CosineSimilarity(), a, b) - cos) < 1e-6
    pa, pb = a / a.sum(-1, keepdim=True), b / b.sum(-1, keepdim=True)
    kl = np.mean([stats.entropy(x, y) for x, y in zip(pa.numpy(), pb.numpy())])
    assert abs(_upd(R.KLDivergence(), a, b) - kl) < 1e-6
    assert abs(_upd(R.KLDivergence(log_prob=True), pa.log(), pb.log()) - kl) < 1e-6
    from scipy.spatial.distance import jensenshannon
    js = np.mean([jensenshannon(x, y) ** 2 for x, y in zip(pa.numpy(), pb.numpy())])
    assert abs(_upd(R.JensenShannonDivergence(), a, b) - js) < 1e-6


def test_aggregation_and_wrappers():
    mx, mn, cat = R.MaxMetric(), R.MinMetric(), R.CatMetric()
    for v in (torch.tensor([1.0, 5.0]), torch.tensor([-2.0, 3.0])):
        mx.update(v)
        mn.update(v)
        cat.update(v)
    assert mx.compute() == 5 and mn.compute() == -2 and cat.compute().tolist() == [1.0, 5.0, -2.0, 3.0]
    rm = R.RunningMean(window=2)
    for v in (1.0, 2.0, 6.0):
        rm.update(torch.tensor(v))
    assert abs(float(rm.compute()) - 4.0) < 1e-6
    rs = R.RunningSum(window=2)
    for v in (1.0, 2.0, 6.0):
        rs.update(torch.tensor(v))
    assert float(rs.compute()) == 8.0
    tr = R.MetricTracker(M.MeanSquaredError(), maximize=False)
    for scale in (1.0, 0.1, 0.5):
        tr.increment()
        tr.update(torch.ones(4) * scale, torch.zeros(4))
    best, step = tr.best_metric(return_step=True)
    assert step == 1 and abs(best - 0.01) < 1e-6 and tr.compute_all().shape == (3,)
    mm = R.MinMaxMetric(M.MeanMetric())
    mm.update(torch.tensor(2.0))
    mm.compute()
    mm.update(torch.tensor(8.0))
    out = mm.compute()
    assert float(out["min"]) == 2.0 and float(out["max"]) == 5.0
    cw = R.ClasswiseWrapper(M.MulticlassRecall(num_classes=3, average="none"), labels=["a", "b", "c"], prefix="recall_")
    cw.update(torch.tensor([0, 1, 2, 2]), torch.tensor([0, 1, 1, 2]))
    res = cw.compute()
    assert set(res) == {"recall_a", "recall_b", "recall_c"} and float(res["recall_b"]) == 0.5
    mo = R.MultioutputWrapper(M.MeanSquaredError(), 2)
    mo.update(torch.tensor([[1.0, 0.0], [1.0, 0.0]]), torch.zeros(2, 2))
    assert mo.compute().tolist() == [1.0, 0.0]
    bs = R.BootStrapper(M.MeanSquaredError(), num_bootstraps=20, generator=torch.Generator().manual_seed(0))
    bs.update(torch.randn(500, generator=torch.Generator().manual_seed(1)), torch.zeros(500))
    out = bs.compute()
    assert 0.7 < float(out["mean"]) < 1.3 and 0 < float(out["std"]) < 0.3
    comp = R.CompositionalMetric(lambda a, b: a / b, M.MeanAbsoluteError(), 2.0)
    comp.update(torch.tensor([4.0]), torch.tensor([0.0]))
    assert float(comp.compute()) == 2.0
