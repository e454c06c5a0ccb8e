"""Text, audio, image and retrieval metrics against hand-computed values and library formulas."""
import math

import numpy as np
import torch
from sklearn import metrics as skm

from tensorplay_b200 import metrics as M


def test_text_metrics():
    assert M.edit_distance("kitten", "sitting") == 3
    preds, refs = ["this is the prediction", "there is an other sample"], ["this is the reference", "there is another one"]
    wer = M.WordErrorRate()
    wer.update(preds, refs)
    assert abs(float(wer.compute()) - 0.5) < 1e-6                  # (1 + 3) errors / 8 reference words
    cer = M.CharErrorRate()
    cer.update(["abcd"], ["abed"])
    assert abs(float(cer.compute()) - 0.25) < 1e-6
    mer = M.MatchErrorRate()
    mer.update(preds, refs)
    assert abs(float(mer.compute()) - 4 / 9) < 1e-6                # errors / (errors + hits)
    wip, wil = M.WordInfoPreserved(), M.WordInfoLost()
    for m in (wip, wil):
        m.update(preds, refs)
    assert abs(float(wip.compute()) + float(wil.compute()) - 1.0) < 1e-6
    ed = M.EditDistance()
    ed.update(["rain", "lnaguaeg"], ["shine", "language"])
    assert abs(float(ed.compute()) - 3.5) < 1e-6
    bleu = M.BLEUScore(n_gram=2)
    bleu.update(["the cat is on the mat"], [["there is a cat on the mat", "a cat is on the mat"]])
    # unigram precision 5/6, bigram 4/5, brevity 1 (closest reference has 6 words)
    assert abs(float(bleu.compute()) - math.sqrt(5 / 6 * 4 / 5)) < 1e-6
    perfect = M.BLEUScore()
    perfect.update(["a b c d e"], [["a b c d e"]])
    assert abs(float(perfect.compute()) - 1.0) < 1e-6
    rouge = M.ROUGEScore()
    rouge.update(["the cat sat on the mat"], ["the cat was on the mat"])
    out = rouge.compute()
    assert abs(float(out["rouge1_fmeasure"]) - 5 / 6) < 1e-6 and abs(float(out["rougeL_fmeasure"]) - 5 / 6) < 1e-6
    assert abs(float(out["rouge2_fmeasure"]) - 3 / 5) < 1e-6


def test_audio_and_image_metrics():
    g = torch.Generator().manual_seed(0)
    t = torch.randn(3, 1000, generator=g)
    p = t + 0.1 * torch.randn(3, 1000, generator=g)
    snr = M.SignalNoiseRatio()
    snr.update(p, t)
    want = np.mean([10 * np.log10((x ** 2).sum() / ((x - y) ** 2).sum()) for x, y in zip(t.numpy(), p.numpy())])
    assert abs(float(snr.compute()) - want) < 1e-4
    si = M.ScaleInvariantSignalDistortionRatio()
    si.update(3.0 * p, t)                                          # invariant to the prediction's scale
    si2 = M.ScaleInvariantSignalDistortionRatio()
    si2.update(p, t)
    assert abs(float(si.compute()) - float(si2.compute())) < 1e-4 and float(si2.compute()) > 15
    assert float(_once(M.ScaleInvariantSignalNoiseRatio(), p + 5.0, t)) > 15      # and to offsets
    img = torch.rand(2, 3, 32, 32, generator=g)
    noisy = (img + 0.05 * torch.randn(2, 3, 32, 32, generator=g)).clamp(0, 1)
    psnr = _once(M.PeakSignalNoiseRatio(data_range=1.0), noisy, img)
    assert abs(float(psnr) - 10 * math.log10(1.0 / float(((noisy - img) ** 2).mean()))) < 1e-4
    assert abs(float(_once(M.StructuralSimilarityIndexMeasure(), img, img)) - 1.0) < 1e-6
    s = float(_once(M.StructuralSimilarityIndexMeasure(), noisy, img))
    assert 0.5 < s < 1.0
    assert float(_once(M.UniversalImageQualityIndex(), img, img)) > 0.999
    tv = M.TotalVariation()
    tv.update(torch.tensor([[[[0.0, 1.0], [1.0, 0.0]]]]))
    assert float(tv.compute()) == 4.0


def _once(m, *a):
    m.update(*a)
    return m.compute()


def test_retrieval_metrics():
    scores = torch.tensor([0.9, 0.8, 0.7, 0.2, 0.6, 0.5, 0.4])
    rel = torch.tensor([1, 0, 1, 0, 0, 1, 1])
    q = torch.tensor([0, 0, 0, 0, 1, 1, 1])
    ap = [skm.average_precision_score(rel[q == i].numpy(), scores[q == i].numpy()) for i in (0, 1)]
    assert abs(float(_once(M.RetrievalMAP(), scores, rel, q)) - np.mean(ap)) < 1e-6
    assert abs(float(_once(M.RetrievalPrecision(top_k=2), scores, rel, q)) - (0.5 + 0.5) / 2) < 1e-6
    assert abs(float(_once(M.RetrievalRecall(top_k=2), scores, rel, q)) - (0.5 + 0.5) / 2) < 1e-6
    assert float(_once(M.RetrievalHitRate(top_k=1), scores, rel, q)) == 0.5
    assert abs(float(_once(M.RetrievalRPrecision(), scores, rel, q)) - (0.5 + 0.5) / 2) < 1e-6
    assert abs(float(_once(M.RetrievalFallOut(top_k=2), scores, rel, q)) - (0.5 + 1.0) / 2) < 1e-6
    auc = [skm.roc_auc_score(rel[q == i].numpy(), scores[q == i].numpy()) for i in (0, 1)]
    assert abs(float(_once(M.RetrievalAUROC(), scores, rel, q)) - np.mean(auc)) < 1e-6


def test_nominal_operating_point_and_spectral_metrics():
    from scipy import stats
    g = torch.Generator().manual_seed(3)
    a = torch.randint(0, 4, (400,), generator=g)
    b = (a + (torch.rand(400, generator=g) < 0.4).long() * torch.randint(0, 4, (400,), generator=g)) % 4
    table = skm.confusion_matrix(b.numpy(), a.numpy())
    chi2 = stats.chi2_contingency(table, correction=False)[0]
    assert abs(float(_once(M.CramersV(4), a, b)) - stats.contingency.association(table, method="cramer")) < 1e-6
    assert abs(float(_once(M.TschuprowsT(4), a, b)) - stats.contingency.association(table, method="tschuprow")) < 1e-6
    assert abs(float(_once(M.PearsonsContingencyCoefficient(4), a, b)) - math.sqrt(chi2 / (chi2 + 400))) < 1e-6
    u = float(_once(M.TheilsU(4), a, b))
    assert 0 < u < 1 and abs(float(_once(M.TheilsU(4), a, a)) - 1.0) < 1e-9
    # Fleiss' kappa on the textbook table (Fleiss 1971, 10 subjects x 5 categories, 14 raters): 0.210
    tbl = torch.tensor([[0, 0, 0, 0, 14], [0, 2, 6, 4, 2], [0, 0, 3, 5, 6], [0, 3, 9, 2, 0], [2, 2, 8, 1, 1],
                        [7, 7, 0, 0, 0], [3, 2, 6, 3, 0], [2, 5, 3, 2, 2], [6, 5, 2, 1, 0], [0, 2, 2, 3, 7]])
    assert abs(float(_once(M.FleissKappa(), tbl)) - 0.210) < 1e-3
    t = (torch.rand(300, generator=g) < 0.4).long()
    s = t * 0.6 + torch.rand(300, generator=g) * 0.8
    prec, thr = _once(M.BinaryPrecisionAtFixedRecall(min_value=0.8), s, t)
    p_curve, r_curve, _ = skm.precision_recall_curve(t.numpy(), s.numpy())
    assert abs(float(prec) - p_curve[r_curve >= 0.8].max()) < 1e-6
    sens, _ = _once(M.BinarySensitivityAtSpecificity(min_value=0.9), s, t)
    fpr, tpr, _ = skm.roc_curve(t.numpy(), s.numpy(), drop_intermediate=False)
    assert abs(float(sens) - tpr[(1 - fpr) >= 0.9].max()) < 1e-6
    csi = _once(M.CriticalSuccessIndex(0.5), torch.tensor([0.9, 0.2, 0.7, 0.1]), torch.tensor([0.8, 0.6, 0.1, 0.0]))
    assert abs(float(csi) - 1 / 3) < 1e-6
    curves = _once(M.ROC(task="multiclass", num_classes=3), torch.softmax(torch.randn(50, 3, generator=g), -1),
                   torch.randint(0, 3, (50,), generator=g))
    assert len(curves) == 3 and len(curves[0]) == 3
    mt = M.MultitaskWrapper({"cls": M.BinaryAccuracy(), "reg": M.MeanSquaredError()})
    mt.update({"cls": torch.tensor([0.9, 0.1]), "reg": torch.tensor([1.0, 2.0])}, {"cls": torch.tensor([1, 0]), "reg": torch.tensor([1.0, 4.0])})
    out = mt.compute()
    assert float(out["cls"]) == 1.0 and float(out["reg"]) == 2.0
    # permutation-invariant SI-SDR: swapping the estimated sources does not change the value
    src = torch.randn(2, 2, 400, generator=g)
    est = src + 0.05 * torch.randn(2, 2, 400, generator=g)

    def sisdr(p, t):
        alpha = (p * t).sum(-1, keepdim=True) / (t * t).sum(-1, keepdim=True)
        proj = alpha * t
        return 10 * torch.log10((proj ** 2).sum(-1) / ((proj - p) ** 2).sum(-1))
    v1 = float(_once(M.PermutationInvariantTraining(sisdr), est, src))
    v2 = float(_once(M.PermutationInvariantTraining(sisdr), est.flip(1), src))
    assert abs(v1 - v2) < 1e-4 and v1 > 20
    img = torch.rand(2, 4, 16, 16, generator=g) + 0.5
    assert float(_once(M.SpectralAngleMapper(), img, img * 1.7)) < 1e-3           # invariant to brightness
    assert float(_once(M.ErrorRelativeGlobalDimensionlessSynthesis(), img, img)) == 0.0
    assert float(_once(M.RelativeAverageSpectralError(), img * 1.1, img)) > 0
    assert float(_once(M.RootMeanSquaredErrorUsingSlidingWindow(4), img + 0.1, img)) - 0.1 < 1e-6
