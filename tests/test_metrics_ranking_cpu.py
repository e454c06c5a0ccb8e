"""Ranking / correlation / retrieval metrics against scipy and scikit-learn."""
import numpy as np
import torch
from scipy import stats
from sklearn import metrics as skm

from tensorplay_b200 import metrics as M
from tests.distutil import run_ranks

F = M.functional


def test_correlations_match_scipy_with_ties():
    g = torch.Generator().manual_seed(0)
    x = torch.randint(0, 12, (200,), generator=g).float()          # many ties
    y = x * 0.5 + torch.randn(200, generator=g)
    y[::7] = y[::7].round()
    x, y = x.double(), y.double()
    assert abs(F.pearson_corrcoef(x, y).item() - stats.pearsonr(x.numpy(), y.numpy())[0]) < 1e-10
    assert abs(F.spearman_corrcoef(x, y).item() - stats.spearmanr(x.numpy(), y.numpy())[0]) < 1e-10
    assert abs(F.kendall_tau(x, y).item() - stats.kendalltau(x.numpy(), y.numpy())[0]) < 1e-7
    m = M.KendallRankCorrCoef()
    m.update(x[:80], y[:80])
    m.update(x[80:], y[80:])
    assert abs(m.compute().item() - stats.kendalltau(x.numpy(), y.numpy())[0]) < 1e-7


def test_classification_curves_match_sklearn():
    g = torch.Generator().manual_seed(1)
    t = (torch.rand(300, generator=g) < 0.3).long()
    s = (t.float() * 0.8 + torch.randn(300, generator=g)).round(decimals=1).double()   # ties in the scores
    assert abs(F.binary_auroc(s, t).item() - skm.roc_auc_score(t.numpy(), s.numpy())) < 1e-10
    s2 = (t.float() + torch.randn(300, generator=g)).double()
    assert abs(F.binary_average_precision(s2, t).item() - skm.average_precision_score(t.numpy(), s2.numpy())) < 1e-10
    logits = torch.randn(64, 10, generator=g)
    y = torch.randint(0, 10, (64,), generator=g)
    ref = skm.top_k_accuracy_score(y.numpy(), logits.numpy(), k=3, labels=np.arange(10))
    assert abs(F.topk_accuracy(logits, y, 3).item() - ref) < 1e-12
    probs = torch.softmax(logits * 2, -1)
    ece = F.expected_calibration_error(probs, y, bins=10).item()
    assert 0 <= ece <= 1
    onehot = torch.nn.functional.one_hot(y, 10).float()
    assert F.expected_calibration_error(onehot, y).item() < 1e-12          # perfectly calibrated


def test_retrieval_metrics():
    g = torch.Generator().manual_seed(2)
    rel = torch.randint(0, 4, (8, 20), generator=g).double()
    sc = torch.randn(8, 20, generator=g).double()
    for k in (None, 5):
        ref = skm.ndcg_score(rel.numpy(), sc.numpy(), k=k)
        assert abs(F.ndcg(sc, rel, k).item() - ref) < 1e-10
    scores = torch.tensor([[0.9, 0.5, 0.1], [0.2, 0.8, 0.4], [0.3, 0.2, 0.1]])
    relevant = torch.tensor([[0, 1, 0], [0, 1, 0], [0, 0, 0]])
    assert abs(F.mean_reciprocal_rank(scores, relevant).item() - (0.5 + 1.0 + 0.0) / 3) < 1e-12


def _sync_worker(rank, world):
    g = torch.Generator().manual_seed(3)
    x, y = torch.randn(40, generator=g).double(), torch.randn(40, generator=g).double()
    m = M.SpearmanCorrCoef()
    m.update(x[rank * 20: (rank + 1) * 20], y[rank * 20: (rank + 1) * 20])
    m.sync()
    return abs(m.compute().item() - stats.spearmanr(x.numpy(), y.numpy())[0]) < 1e-10


def test_collecting_metric_syncs_samples_across_ranks():
    assert all(run_ranks(_sync_worker, 2))


def test_regression_metrics_native_reduction_matches_torch():
    from tensorplay_b200.metrics import _native_diff_sum
    g = torch.Generator().manual_seed(4)
    for n in (1, 7, 4096, 65537, 300001):
        a, b = torch.randn(n, generator=g), torch.randn(n, generator=g)
        sq, ab = _native_diff_sum(a, b, "sq"), _native_diff_sum(a, b, "abs")
        assert sq is not None and ab is not None
        assert abs(sq - ((a.double() - b.double()) ** 2).sum().item()) < 1e-6 * max(1.0, sq)
        assert abs(ab - (a.double() - b.double()).abs().sum().item()) < 1e-6 * max(1.0, ab)
    assert _native_diff_sum(a.double(), b.double(), "sq") is None           # other dtypes take the torch path
    m = M.MeanSquaredError(squared=False)
    m.update(a.view(-1, 1)[:, 0], b)
    torch.testing.assert_close(m.compute(), ((a - b) ** 2).mean().sqrt(), rtol=1e-5, atol=1e-6)
