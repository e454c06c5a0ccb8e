"""Task-specific classification metrics against scikit-learn."""
import numpy as np
import torch
from sklearn import metrics as skm

from tensorplay_b200.metrics import classification as C


def _two_updates(m, p, t):
    h = len(t) // 2
    m.update(p[:h], t[:h])
    m.update(p[h:], t[h:])
    return m.compute()


def test_binary_family():
    g = torch.Generator().manual_seed(0)
    t = (torch.rand(200, generator=g) < 0.4).long()
    s = (t.float() * 0.5 + torch.rand(200, generator=g) * 0.7).clamp(0, 1)
    yp = (s > 0.5).long().numpy()
    tn, fp, fn, tp = skm.confusion_matrix(t.numpy(), yp).ravel()
    checks = {"BinaryAccuracy": skm.accuracy_score(t, yp), "BinaryPrecision": skm.precision_score(t, yp),
              "BinaryRecall": skm.recall_score(t, yp), "BinaryF1Score": skm.f1_score(t, yp),
              "BinarySpecificity": tn / (tn + fp), "BinaryNegativePredictiveValue": tn / (tn + fn),
              "BinaryJaccardIndex": skm.jaccard_score(t, yp), "BinaryHammingDistance": skm.hamming_loss(t, yp),
              "BinaryCohenKappa": skm.cohen_kappa_score(t, yp), "BinaryMatthewsCorrCoef": skm.matthews_corrcoef(t, yp),
              "BinaryAUROC": skm.roc_auc_score(t, s.double()), "BinaryAveragePrecision": skm.average_precision_score(t, s.double())}
    for name, want in checks.items():
        got = _two_updates(getattr(C, name)(), s, t)
        assert abs(float(got) - want) < 1e-6, (name, float(got), want)
    assert abs(float(_two_updates(C.BinaryFBetaScore(beta=2.0), s, t)) - skm.fbeta_score(t, yp, beta=2.0)) < 1e-6
    assert _two_updates(C.BinaryStatScores(), s, t).tolist() == [tp, fp, tn, fn, tp + fn]
    assert torch.equal(_two_updates(C.BinaryConfusionMatrix(), s, t), torch.tensor([[tn, fp], [fn, tp]]))
    fpr, tpr, _ = _two_updates(C.BinaryROC(), s, t)
    rf, rt, _ = skm.roc_curve(t, s.double(), drop_intermediate=False)
    np.testing.assert_allclose(fpr.numpy(), rf, atol=1e-12)
    np.testing.assert_allclose(tpr.numpy(), rt, atol=1e-12)
    pr, rc, _ = _two_updates(C.BinaryPrecisionRecallCurve(), s, t)
    rp, rr, _ = skm.precision_recall_curve(t, s.double())
    np.testing.assert_allclose(pr.numpy()[-len(rp):], rp, atol=1e-12)
    np.testing.assert_allclose(rc.numpy()[-len(rr):], rr, atol=1e-12)
    margins = s * 4 - 2
    want = skm.hinge_loss(t.numpy() * 2 - 1, margins.numpy())
    assert abs(float(_two_updates(C.BinaryHingeLoss(), margins, t)) - want) < 1e-6
    assert 0 <= float(_two_updates(C.BinaryCalibrationError(n_bins=10), s, t)) <= 1


def test_multiclass_family():
    g = torch.Generator().manual_seed(1)
    n, k = 300, 5
    t = torch.randint(0, k, (n,), generator=g)
    logits = torch.randn(n, k, generator=g) + 2.0 * torch.nn.functional.one_hot(t, k)
    yp = logits.argmax(-1).numpy()
    for avg in ("macro", "micro", "weighted"):
        kw = dict(num_classes=k, average=avg)
        assert abs(float(_two_updates(C.MulticlassPrecision(**kw), logits, t)) - skm.precision_score(t, yp, average=avg)) < 1e-6
        assert abs(float(_two_updates(C.MulticlassRecall(**kw), logits, t)) - skm.recall_score(t, yp, average=avg)) < 1e-6
        assert abs(float(_two_updates(C.MulticlassF1Score(**kw), logits, t)) - skm.f1_score(t, yp, average=avg)) < 1e-6
        assert abs(float(_two_updates(C.MulticlassJaccardIndex(**kw), logits, t)) - skm.jaccard_score(t, yp, average=avg)) < 1e-6
    assert abs(float(_two_updates(C.MulticlassAccuracy(num_classes=k, average="micro"), logits, t)) - skm.accuracy_score(t, yp)) < 1e-6
    assert abs(float(_two_updates(C.MulticlassAccuracy(num_classes=k), logits, t)) - skm.balanced_accuracy_score(t, yp)) < 1e-6
    per = _two_updates(C.MulticlassRecall(num_classes=k, average="none"), logits, t)
    np.testing.assert_allclose(per.numpy(), skm.recall_score(t, yp, average=None), atol=1e-6)
    assert torch.equal(_two_updates(C.MulticlassConfusionMatrix(k), logits, t), torch.from_numpy(skm.confusion_matrix(t, yp)))
    assert abs(float(_two_updates(C.MulticlassCohenKappa(k), logits, t)) - skm.cohen_kappa_score(t, yp)) < 1e-6
    assert abs(float(_two_updates(C.MulticlassMatthewsCorrCoef(k), logits, t)) - skm.matthews_corrcoef(t, yp)) < 1e-6
    probs = torch.softmax(logits.double(), -1)
    assert abs(float(_two_updates(C.MulticlassAUROC(k), probs, t)) - skm.roc_auc_score(t, probs, multi_class="ovr")) < 1e-6
    top2 = _two_updates(C.MulticlassAccuracy(num_classes=k, average="micro", top_k=2), logits, t)
    assert abs(float(top2) - skm.top_k_accuracy_score(t, logits.numpy(), k=2)) < 1e-6
    assert abs(float(_two_updates(C.MulticlassHingeLoss(k), logits, t)) - skm.hinge_loss(t.numpy(), logits.numpy(), labels=np.arange(k))) < 1e-5
    assert C.FBetaScore(task="multiclass", num_classes=k, beta=0.5).__class__.__name__ == "MulticlassFBetaScore"


def test_multilabel_family():
    g = torch.Generator().manual_seed(2)
    t = (torch.rand(150, 4, generator=g) < 0.4).long()
    s = (t.float() * 0.4 + torch.rand(150, 4, generator=g) * 0.8).clamp(0, 1)
    yp = (s > 0.5).long().numpy()
    for avg in ("macro", "micro"):
        kw = dict(num_labels=4, average=avg)
        assert abs(float(_two_updates(C.MultilabelF1Score(**kw), s, t)) - skm.f1_score(t, yp, average=avg)) < 1e-6
        assert abs(float(_two_updates(C.MultilabelPrecision(**kw), s, t)) - skm.precision_score(t, yp, average=avg)) < 1e-6
    assert abs(float(_two_updates(C.MultilabelHammingDistance(num_labels=4, average="micro"), s, t)) - skm.hamming_loss(t, yp)) < 1e-6
    assert abs(float(_two_updates(C.ExactMatch(), s, t)) - skm.accuracy_score(t, yp)) < 1e-6
    cm = _two_updates(C.MultilabelConfusionMatrix(4), s, t)
    assert torch.equal(cm, torch.from_numpy(skm.multilabel_confusion_matrix(t, yp)))
    assert abs(float(_two_updates(C.MultilabelAUROC(4), s.double(), t)) - skm.roc_auc_score(t, s.double(), average="macro")) < 1e-6
    assert abs(float(_two_updates(C.MultilabelAveragePrecision(4), s.double(), t))
               - skm.average_precision_score(t, s.double(), average="macro")) < 1e-6
