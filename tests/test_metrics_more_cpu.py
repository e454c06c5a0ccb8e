"""Text, panoptic, feature-based and functional metrics: documented example values of the
reference's docstrings (tensorplay/metrics/text/{sacre_bleu,chrf,ter,eed}.py,
tensorplay/metrics/detection/panoptic_qualities.py), closed forms and scipy."""
import math

import numpy as np
import pytest
import torch

import tensorplay_b200.metrics as M

P = ["the cat is on the mat"]
T = [["there is a cat on the mat", "a cat is on the mat"]]


def _once(metric, *args):
    metric.update(*args)
    return metric.compute()


def test_translation_scores_match_the_documented_examples():
    assert abs(float(_once(M.SacreBLEUScore(), P, T)) - 0.7598) < 1e-4
    assert abs(float(_once(M.CHRFScore(), P, T)) - 0.8640) < 1e-4
    assert abs(float(_once(M.TranslationEditRate(), P, T)) - 0.1538) < 1e-4
    eed = _once(M.ExtendedEditDistance(), ["this is the prediction", "here is an other sample"],
                [["this is the reference"], ["here is another one"]])
    assert abs(float(eed) - 0.3078) < 1e-4
    # a block shift costs one edit: "c d a b" -> "a b c d"
    assert abs(float(_once(M.TranslationEditRate(), ["c d a b"], [["a b c d"]])) - 0.25) < 1e-6
    assert float(_once(M.CHRFScore(), ["same text"], [["same text"]])) == 1.0
    from tensorplay_b200.metrics.text_more import _tokenize
    assert _tokenize("Hello, world! It's 3.5 km (approx).", "13a", False) == "Hello , world ! It's 3.5 km ( approx ) ."
    sq = _once(M.SQuAD(), [{"prediction_text": "1976", "id": "a"}, {"prediction_text": "the big cat", "id": "b"}],
               [{"answers": {"text": ["1976"]}, "id": "a"}, {"answers": {"text": ["a big dog", "cat"]}, "id": "b"}])
    assert float(sq["exact_match"]) == 50.0 and abs(float(sq["f1"]) - 100 * (1 + 2 / 3) / 2) < 1e-4


def test_panoptic_quality_matches_the_documented_examples():
    preds = torch.tensor([[[[6, 0], [0, 0], [6, 0], [6, 0]], [[0, 0], [0, 0], [6, 0], [0, 1]], [[0, 0], [0, 0], [6, 0], [0, 1]],
                           [[0, 0], [7, 0], [6, 0], [1, 0]], [[0, 0], [7, 0], [7, 0], [7, 0]]]])
    target = torch.tensor([[[[6, 0], [0, 1], [6, 0], [0, 1]], [[0, 1], [0, 1], [6, 0], [0, 1]], [[0, 1], [0, 1], [6, 0], [1, 0]],
                            [[0, 1], [7, 0], [1, 0], [1, 0]], [[0, 1], [7, 0], [7, 0], [7, 0]]]])
    assert abs(float(_once(M.PanopticQuality({0, 1}, {6, 7}), preds, target)) - 0.5463) < 1e-4
    three = _once(M.PanopticQuality({0, 1}, {6, 7}, return_sq_and_rq=True), preds, target)
    assert torch.allclose(three, torch.tensor([0.5463, 0.6111, 0.6667], dtype=torch.float64), atol=1e-4)
    per = _once(M.PanopticQuality({0, 1}, {6, 7}, return_per_class=True), preds, target)
    assert torch.allclose(per, torch.tensor([[0.5185, 0.0, 0.6667, 1.0]], dtype=torch.float64), atol=1e-4)
    mod = _once(M.ModifiedPanopticQuality({0, 1}, {6, 7}), torch.tensor([[[0, 0], [0, 1], [6, 0], [7, 0], [0, 2], [1, 0]]]),
                torch.tensor([[[0, 1], [0, 0], [6, 0], [7, 0], [6, 0], [255, 0]]]))
    assert abs(float(mod) - 0.7667) < 1e-4
    with pytest.raises(ValueError):
        M.PanopticQuality({0, 1}, {1, 2})
    with pytest.raises(ValueError):
        _once(M.PanopticQuality({0}, {6}), torch.tensor([[[9, 0]]]), torch.tensor([[[0, 0]]]))


def test_feature_statistics_against_scipy():
    import scipy.linalg
    g = torch.Generator().manual_seed(0)
    torch.manual_seed(0)                       # the layer's initial weights
    net = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(48, 8)).double()
    real = torch.randn(200, 3, 4, 4, generator=g).double()
    fake = (torch.randn(200, 3, 4, 4, generator=g) * 1.3 + 0.2).double()
    fid = M.FrechetInceptionDistance(feature=net)
    fid.update(real, True)
    fid.update(fake, False)
    fr, ff = net(real).detach().numpy(), net(fake).detach().numpy()
    sr, sf = np.cov(fr.T), np.cov(ff.T)
    want = ((fr.mean(0) - ff.mean(0)) ** 2).sum() + np.trace(sr + sf - 2 * scipy.linalg.sqrtm(sr @ sf).real)
    assert abs(float(fid.compute()) - want) < 1e-5 * max(1.0, want)
    far = (torch.randn(200, 3, 4, 4, generator=g) * 2.0 + 1.0).double()
    kid = M.KernelInceptionDistance(feature=net, subsets=5, subset_size=100)
    kid.update(real, True)
    kid.update(far, False)
    same = M.KernelInceptionDistance(feature=net, subsets=5, subset_size=100)
    same.update(real, True)
    same.update(real.flip(0), False)
    assert float(kid.compute()[0]) > 10 * abs(float(same.compute()[0]))
    # inception score: uniform predictions -> 1, confident and balanced over k classes -> k
    onehot = lambda x: 50.0 * torch.nn.functional.one_hot(x.reshape(-1).long() % 4, 4).double()   # noqa: E731
    conf = M.InceptionScore(feature=onehot, splits=2)
    conf.update(torch.arange(400))
    assert abs(float(conf.compute()[0]) - 4.0) < 0.05     # the random halves are not exactly balanced
    flat = M.InceptionScore(feature=lambda x: torch.zeros(x.shape[0], 4), splits=2)
    flat.update(torch.arange(40))
    assert abs(float(flat.compute()[0]) - 1.0) < 1e-6
    with pytest.raises(ValueError):
        M.FrechetInceptionDistance().update(real, True)


def test_embedding_metrics_with_caller_networks():
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(1)
    conv = torch.nn.Conv2d(3, 6, 3).double()
    feats = lambda x: [conv(x.double()), torch.nn.functional.avg_pool2d(conv(x.double()), 2)]   # noqa: E731
    img = torch.rand(2, 3, 12, 12, generator=g)
    lp = M.LearnedPerceptualImagePatchSimilarity(net=feats)
    assert float(_once(lp, img, img)) == 0.0
    assert float(_once(M.LearnedPerceptualImagePatchSimilarity(net=feats), img, img.flip(-1))) > 0
    table = {"a photo of a cat": torch.tensor([1.0, 0.0]), "a photo of a dog": torch.tensor([0.0, 1.0])}
    text = lambda ts: torch.stack([table.get(t, torch.tensor([0.7, -0.7])) for t in ts])           # noqa: E731
    image = lambda x: x                                                                            # noqa: E731
    score = _once(M.CLIPScore(model=(image, text)), torch.tensor([[2.0, 0.0], [1.0, 1.0]]), ["a photo of a cat", "a photo of a dog"])
    assert abs(float(score) - 100 * (1 + math.sqrt(0.5)) / 2) < 1e-4
    iqa = M.CLIPImageQualityAssessment(model=(image, lambda ts: torch.tensor([[1.0, 0.0], [0.0, 1.0]])), prompts=("quality",))
    p = _once(iqa, torch.tensor([[1.0, 0.0], [0.0, 1.0]]))
    assert float(p[0]) > 0.99 and float(p[1]) < 0.01
    vocab = {}
    emb = torch.randn(50, 8, generator=g)

    def embed(sentences):
        out = []
        for s in sentences:
            ids = torch.tensor([vocab.setdefault(w, len(vocab)) for w in s.split()])
            out.append(emb[ids])
        return out
    bs = _once(M.BERTScore(model=embed), ["the cat sat", "a dog"], ["the cat sat", "the cat"])
    assert abs(float(bs["f1"][0]) - 1.0) < 1e-6 and float(bs["f1"][1]) < 0.9
    with pytest.raises(ValueError):
        M.CLIPScore()
    with pytest.raises(RuntimeError):
        M.PerceptualEvaluationSpeechQuality(16000, "wb")
    ext = M.PerceptualEvaluationSpeechQuality(16000, "wb", scorer=lambda p, t: torch.tensor([2.0, 4.0]))
    assert float(_once(ext, torch.zeros(2, 4), torch.zeros(2, 4))) == 3.0


def test_audio_and_image_additions():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(2, 4000, generator=g)
    h = torch.tensor([0.5, 0.3, -0.2, 0.1])
    y = torch.nn.functional.conv1d(x[:, None], h.flip(0)[None, None], padding=3)[:, 0, :4000]
    # a filtered copy of the reference is no distortion for SDR, while it is for plain SNR
    sdr = M.more.signal_distortion_ratio(y, x, filter_length=16)
    snr = 10 * torch.log10((x ** 2).sum(-1) / ((x - y) ** 2).sum(-1))
    assert float(sdr.min()) > 30 and float(snr.max()) < 5
    noisy = x + 0.1 * torch.randn(2, 4000, generator=g)
    assert abs(float(_once(M.SignalDistortionRatio(filter_length=16), noisy, x)) - 20.0) < 0.5
    sa = _once(M.SourceAggregatedSignalDistortionRatio(scale_invariant=False), noisy[None], x[None])
    assert abs(float(sa) - 20.0) < 0.5
    # intelligibility falls as noise is added to amplitude-modulated broadband noise
    t = torch.arange(32000) / 16000.0
    clean = torch.randn(32000, generator=g) * (0.55 + 0.45 * torch.sin(2 * math.pi * 4 * t))
    vals = [float(M.short_time_objective_intelligibility(clean + torch.randn(32000, generator=g) * 10 ** (-snr_db / 20), clean, 16000))
            for snr_db in (60, 10, 0, -10)]
    assert vals[0] > 0.99 and vals[0] > vals[1] > vals[2] > vals[3]
    assert float(_once(M.ShortTimeObjectiveIntelligibility(16000, extended=True), clean[None], clean[None])) > 0.99
    img = torch.rand(2, 3, 192, 192, generator=g)
    assert abs(float(_once(M.MultiScaleStructuralSimilarityIndexMeasure(), img, img)) - 1.0) < 1e-6
    worse = [float(_once(M.MultiScaleStructuralSimilarityIndexMeasure(), (img + s * torch.randn(img.shape, generator=g)).clamp(0, 1), img))
             for s in (0.05, 0.2)]
    assert 1 > worse[0] > worse[1] > 0
    ms = torch.rand(2, 4, 16, 16, generator=g)
    fused = torch.nn.functional.interpolate(ms, scale_factor=2, mode="bilinear")
    assert float(_once(M.SpectralDistortionIndex(), ms, ms)) == 0.0
    assert float(_once(M.SpectralDistortionIndex(), fused + 0.2 * torch.rand(fused.shape, generator=g), ms)) > 0
    pan = fused.mean(1, keepdim=True)
    d_s = _once(M.SpatialDistortionIndex(), fused, {"ms": ms, "pan": pan})
    assert 0 <= float(d_s) < 0.5
    lve = _once(M.LipVertexError([0, 2]), torch.tensor([[[0.0, 0, 0], [9, 9, 9], [1, 0, 0]]]), torch.zeros(1, 3, 3))
    assert float(lve) == 1.0


def test_classification_and_retrieval_additions():
    from sklearn import metrics as skm
    g = torch.Generator().manual_seed(3)
    t = (torch.rand(4000, generator=g) < 0.3).long()
    s = torch.rand(4000, generator=g)
    # random scores: tpr = fpr, so the area over log10(fpr) in (0.001, 0.1) is (0.1 - 0.001) / (2 ln 10)
    assert abs(float(_once(M.BinaryLogAUC(), s, t)) - 0.099 / (2 * math.log(10))) < 0.01
    assert abs(float(_once(M.BinaryLogAUC(), t + 0.01 * s, t)) - 1.0) < 1e-6
    p = (torch.rand(300, 4, generator=g) < 0.5)
    y = torch.where(torch.rand(300, 4, generator=g) < 0.8, p, ~p)
    want = skm.matthews_corrcoef(y.reshape(-1).numpy(), p.reshape(-1).numpy())
    assert abs(float(_once(M.MultilabelMatthewsCorrCoef(4), p.float(), y.long())) - want) < 1e-6
    assert type(M.HingeLoss(task="multiclass", num_classes=3)).__name__ == "MulticlassHingeLoss"
    prec, rec, ks = _once(M.RetrievalPrecisionRecallCurve(max_k=2), torch.tensor([0.2, 0.3, 0.5]), torch.tensor([1, 0, 1]),
                          torch.tensor([0, 0, 0]))
    assert prec.tolist() == [1.0, 0.5] and rec.tolist() == [0.5, 0.5] and ks.tolist() == [1, 2]
    r, k = _once(M.RetrievalRecallAtFixedPrecision(min_precision=0.8), torch.tensor([0.9, 0.8, 0.7, 0.1]), torch.tensor([1, 0, 1, 1]),
                 torch.zeros(4, dtype=torch.long))
    assert abs(float(r) - 1 / 3) < 1e-6 and int(k) == 1      # precision at k = 1..4: 1, 1/2, 2/3, 3/4
    sc = torch.softmax(torch.randn(100, 3, generator=g), -1)
    tc = torch.randint(0, 3, (100,), generator=g)
    v, thr = _once(M.MulticlassPrecisionAtFixedRecall(num_classes=3, min_value=0.5), sc, tc)
    one, _ = _once(M.BinaryPrecisionAtFixedRecall(min_value=0.5), sc[:, 1], (tc == 1).long())
    assert v.shape == (3,) and abs(float(v[1]) - float(one)) < 1e-7
    assert float(_once(M.MulticlassExactMatch(num_classes=2), torch.tensor([[0, 1], [1, 1]]), torch.tensor([[0, 1], [1, 0]]))) == 0.5
    assert _once(M.MultilabelExactMatch(num_labels=2, multidim_average="samplewise"), torch.tensor([[0.9, 0.1], [0.9, 0.9]]),
                 torch.tensor([[1, 0], [1, 0]])).tolist() == [1.0, 0.0]


def test_functional_spellings_and_domain_views():
    import tensorplay_b200.metrics.functional as F
    from tensorplay_b200.metrics.detection import PanopticQuality
    from tensorplay_b200.metrics.text import CHRFScore
    from tensorplay_b200.metrics.utilities import class_reduce, dim_zero_cat
    assert PanopticQuality is M.PanopticQuality and CHRFScore is M.CHRFScore
    assert float(F.mean_squared_error(torch.tensor([1.0, 2.0]), torch.tensor([1.0, 4.0]))) == 2.0
    assert abs(float(F.multiclass_accuracy(torch.tensor([0, 1, 2]), torch.tensor([0, 1, 1]), num_classes=3, average="micro")) - 2 / 3) < 1e-6
    assert abs(float(F.chrf_score(P, T)) - 0.8640) < 1e-4
    assert abs(float(F.word_information_lost(["a b c"], ["a b d"])) - 5 / 9) < 1e-6
    g = torch.Generator().manual_seed(4)
    mat = torch.randint(0, 3, (200, 3), generator=g)
    mat[:, 2] = mat[:, 0]
    cv = F.cramers_v_matrix(mat)
    assert abs(float(cv[0, 2]) - 1.0) < 1e-6 and torch.allclose(cv, cv.T) and float(cv[0, 1]) < 0.3
    src = torch.randn(2, 2, 5, generator=g)
    assert torch.equal(F.pit_permutate(src, torch.tensor([[1, 0], [0, 1]]))[0], src[0].flip(0))
    assert dim_zero_cat([torch.tensor(1.0), torch.tensor([2.0, 3.0])]).tolist() == [1.0, 2.0, 3.0]
    got = class_reduce(torch.tensor([1.0, 0.0, 2.0]), torch.tensor([2.0, 0.0, 2.0]), torch.tensor([2.0, 0.0, 2.0]), "weighted")
    assert abs(float(got) - 0.75) < 1e-6
    with pytest.raises(AttributeError):
        F.no_such_metric


def test_every_metric_name_of_the_reference_resolves():
    """The names below are the public list of tensorplay/metrics/__init__.py that are not covered by
    the value tests of the other metric test files."""
    names = """Accuracy AUROC AveragePrecision BERTScore BLEUScore BootStrapper CalibrationError CatMetric CharErrorRate CHRFScore
    ClasswiseWrapper CLIPImageQualityAssessment CLIPScore CohenKappa ConcordanceCorrCoef ConfusionMatrix CosineSimilarity CramersV
    CriticalSuccessIndex DeepNoiseSuppressionMeanOpinionScore EditDistance ErrorRelativeGlobalDimensionlessSynthesis ExactMatch
    ExplainedVariance ExtendedEditDistance F1Score FBetaScore FleissKappa FrechetInceptionDistance HammingDistance HingeLoss
    InceptionScore InfoLM JaccardIndex KendallRankCorrCoef KernelInceptionDistance KLDivergence LearnedPerceptualImagePatchSimilarity
    LipVertexError LogAUC LogCoshError MatchErrorRate MatthewsCorrCoef MaxMetric MeanAbsoluteError MeanAbsolutePercentageError
    MeanMetric MeanSquaredError MeanSquaredLogError MetricCollection MetricTracker MinkowskiDistance MinMaxMetric MinMetric
    ModifiedPanopticQuality MultioutputWrapper MultiScaleStructuralSimilarityIndexMeasure MultitaskWrapper
    NonIntrusiveSpeechQualityAssessment PanopticQuality PeakSignalNoiseRatio PearsonCorrCoef PearsonsContingencyCoefficient
    PerceptualEvaluationSpeechQuality PermutationInvariantTraining Perplexity Precision PrecisionAtFixedRecall PrecisionRecallCurve
    R2Score Recall RecallAtFixedPrecision RelativeAverageSpectralError RelativeSquaredError RetrievalFallOut RetrievalHitRate
    RetrievalMAP RetrievalMRR RetrievalNormalizedDCG RetrievalPrecision RetrievalPrecisionRecallCurve RetrievalRecall
    RetrievalRecallAtFixedPrecision RetrievalRPrecision ROC ROUGEScore RootMeanSquaredErrorUsingSlidingWindow RunningMean RunningSum
    SacreBLEUScore ScaleInvariantSignalDistortionRatio ScaleInvariantSignalNoiseRatio SensitivityAtSpecificity
    ShortTimeObjectiveIntelligibility SignalDistortionRatio SignalNoiseRatio SourceAggregatedSignalDistortionRatio
    SpatialDistortionIndex SpearmanCorrCoef Specificity SpecificityAtSensitivity SpectralAngleMapper SpectralDistortionIndex
    SpeechReverberationModulationEnergyRatio SQuAD StatScores StructuralSimilarityIndexMeasure SumMetric
    SymmetricMeanAbsolutePercentageError TheilsU TotalVariation TranslationEditRate TschuprowsT TweedieDevianceScore
    UniversalImageQualityIndex WeightedMeanAbsolutePercentageError WordErrorRate WordInfoLost WordInfoPreserved""".split()
    missing = [n for n in names if not hasattr(M, n)]
    assert not missing, missing
