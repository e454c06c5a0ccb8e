"""Attribution algorithms on models whose attributions are known in closed form."""
import torch
from torch import nn

from tensorplay_b200 import lumen


def _linear():
    torch.manual_seed(0)
    m = nn.Linear(6, 3)
    return m, torch.randn(4, 6)


def test_gradient_methods_on_a_linear_model():
    m, x = _linear()
    w = m.weight[1]
    torch.testing.assert_close(lumen.Saliency(m).attribute(x, target=1), w.abs().expand(4, 6))
    torch.testing.assert_close(lumen.InputXGradient(m).attribute(x, target=1), (x * w).detach())
    ig, delta = lumen.IntegratedGradients(m).attribute(x, target=1, n_steps=8, return_convergence_delta=True)
    torch.testing.assert_close(ig, (x * w).detach(), atol=1e-5, rtol=1e-5)
    assert delta.abs().max() < 1e-5
    # per-example targets
    t = torch.tensor([0, 1, 2, 1])
    ig = lumen.IntegratedGradients(m).attribute(x, target=t, n_steps=4)
    torch.testing.assert_close(ig, (x * m.weight[t]).detach(), atol=1e-5, rtol=1e-5)


def test_integrated_gradients_completeness_on_a_nonlinear_model():
    torch.manual_seed(1)
    m = nn.Sequential(nn.Linear(5, 16), nn.Tanh(), nn.Linear(16, 2))
    x, b = torch.randn(3, 5), torch.randn(1, 5)
    attr, delta = lumen.IntegratedGradients(m).attribute(x, baselines=b, target=0, n_steps=64,
                                                         return_convergence_delta=True)
    assert delta.abs().max() < 1e-4
    with torch.no_grad():
        torch.testing.assert_close(attr.sum(1), m(x)[:, 0] - m(b)[:, 0].expand(3), atol=1e-4, rtol=1e-4)


def test_deeplift_sums_to_output_difference_on_relu_net():
    torch.manual_seed(2)
    m = nn.Sequential(nn.Linear(5, 12), nn.ReLU(), nn.Linear(12, 12), nn.ReLU(), nn.Linear(12, 1))
    x = torch.randn(4, 5)
    attr, delta = lumen.DeepLift(m).attribute(x, return_convergence_delta=True)
    assert delta.abs().max() < 1e-5
    gb = lumen.GuidedBackprop(m).attribute(x)
    dc = lumen.Deconvolution(m).attribute(x)
    assert gb.shape == x.shape and dc.shape == x.shape and not torch.equal(gb, dc)


def test_perturbation_methods_on_an_additive_model():
    m, x = _linear()
    w = m.weight[2]
    exact = (x * w).detach()
    torch.testing.assert_close(lumen.FeatureAblation(m).attribute(x, target=2, perturbations_per_eval=3), exact,
                               atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(lumen.Occlusion(m).attribute(x, (1,), target=2), exact, atol=1e-5, rtol=1e-5)
    g = torch.Generator().manual_seed(0)
    torch.testing.assert_close(lumen.ShapleyValueSampling(m).attribute(x, target=2, n_samples=3, generator=g), exact,
                               atol=1e-5, rtol=1e-5)
    mask = torch.tensor([[0, 0, 1, 1, 2, 2]])
    sv = lumen.ShapleyValues(m).attribute(x, target=2, feature_mask=mask)
    torch.testing.assert_close(sv[:, 0], exact[:, 0] + exact[:, 1], atol=1e-5, rtol=1e-5)
    ks = lumen.KernelShap(m).attribute(x[:1], target=2, n_samples=200, generator=g)
    torch.testing.assert_close(ks, exact[:1], atol=1e-3, rtol=1e-3)
    li = lumen.Lime(m).attribute(x[:1], target=2, n_samples=200, generator=g)
    torch.testing.assert_close(li, exact[:1], atol=1e-3, rtol=1e-3)
    fp = lumen.FeaturePermutation(m).attribute(x, target=2, generator=g)
    assert fp.shape == x.shape


def test_shapley_values_exact_on_an_interaction():
    # f = x0 * x1 + x2: the product's value is shared equally by x0 and x1
    f = lambda x: x[:, 0] * x[:, 1] + x[:, 2]   # noqa: E731
    x = torch.tensor([[2.0, 3.0, 5.0]])
    sv = lumen.ShapleyValues(f).attribute(x)
    torch.testing.assert_close(sv, torch.tensor([[3.0, 3.0, 5.0]]))


def test_noise_tunnel_and_gradient_shap():
    m, x = _linear()
    g = torch.Generator().manual_seed(0)
    sg = lumen.NoiseTunnel(lumen.Saliency(m)).attribute(x, nt_samples=3, stdevs=0.1, generator=g, target=0, abs=False)
    torch.testing.assert_close(sg, m.weight[0].expand(4, 6).detach())          # constant gradient
    vg = lumen.NoiseTunnel(lumen.Saliency(m)).attribute(x, nt_type="vargrad", nt_samples=3, generator=g, target=0)
    assert vg.abs().max() < 1e-6
    gs = lumen.GradientShap(m).attribute(x, torch.zeros(2, 6), target=0, n_samples=4, generator=g)
    torch.testing.assert_close(gs, (x * m.weight[0]).detach(), atol=1e-5, rtol=1e-5)


def test_layer_methods():
    torch.manual_seed(3)
    conv = nn.Conv2d(2, 4, 3, padding=1)
    m = nn.Sequential(conv, nn.ReLU(), nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(4, 3))
    x = torch.randn(2, 2, 5, 5)
    act = lumen.LayerActivation(m, conv).attribute(x)
    torch.testing.assert_close(act, conv(x).detach())
    cam = lumen.LayerGradCam(m, conv).attribute(x, target=1)
    assert cam.shape == (2, 1, 5, 5)
    ga = lumen.LayerGradientXActivation(m, conv).attribute(x, target=1)
    assert ga.shape == act.shape
    # conductance of a layer sums to the output difference (completeness through the layer)
    mlp = nn.Sequential(nn.Linear(4, 8), nn.Tanh(), nn.Linear(8, 1))
    xi = torch.randn(3, 4)
    cond = lumen.LayerConductance(mlp, mlp[1]).attribute(xi, n_steps=200)
    with torch.no_grad():
        torch.testing.assert_close(cond.sum(1), (mlp(xi) - mlp(torch.zeros(3, 4)))[:, 0], atol=1e-3, rtol=1e-3)
    lig, delta = lumen.LayerIntegratedGradients(mlp, mlp[0]).attribute(xi, n_steps=32, return_convergence_delta=True)
    assert lig.shape == (3, 8) and delta.abs().max() < 1e-4
    assert lumen.InternalInfluence(mlp, mlp[1]).attribute(xi, n_steps=8).shape == (3, 8)
    assert lumen.NeuronConductance(mlp, mlp[1]).attribute(xi, 2, n_steps=8).shape == (3,)


def test_llm_tools_on_the_tiny_llama():
    from tensorplay_b200.models.llama import Llama, LlamaConfig
    cfg = LlamaConfig.tiny(hidden_size=32, num_heads=4, num_kv_heads=2, head_dim=8, ffn_size=48, vocab_size=50,
                           num_layers=3, max_seq_len=16)
    m = Llama(cfg)
    m.reset_parameters(0)
    toks = torch.randint(0, 50, (2, 7), generator=torch.Generator().manual_seed(0))
    lens = lumen.logit_lens(m, toks)
    assert lens.shape == (3, 2, 7, 50)
    with torch.no_grad():
        torch.testing.assert_close(lens[-1], m(toks))       # the last block's lens is the model's output
    other = toks.clone()
    other[:, 6] = (other[:, 6] + 1) % 50      # last position: under the causal mask only it differs
    metric = lambda logits: logits[0, -1, 3]   # noqa: E731
    patch = lumen.activation_patching(m, toks, other, metric)
    assert patch.shape == (3, 7)
    with torch.no_grad():
        clean_val = float(metric(m(toks)))
    # restoring the corrupted position after the first block restores the clean run exactly
    assert abs(float(patch[0, 6]) - clean_val) < 1e-5 and abs(float(patch[0, 2]) - clean_val) > 1e-6
    att = [torch.softmax(torch.randn(2, 4, 7, 7), -1) for _ in range(3)]
    roll = lumen.attention_rollout(att)
    torch.testing.assert_close(roll.sum(-1), torch.ones(2, 7))

    def fwd_embeds(e):
        cos, sin = m.rope_tables(e.shape[1], e.device)
        x = e
        for l in m.layers:
            x = l(x, cos, sin)
        return m.head(x)
    res = lumen.LLMGradientAttribution(m, m.embed_tokens, fwd_embeds).attribute(toks[:, :5], toks[:, 5:])
    assert res["token_attr"].shape == (2, 7) and res["log_prob"].shape == (2, 2)


def test_lrp_conserves_relevance_and_matches_input_x_gradient_on_relu_nets():
    torch.manual_seed(4)
    m = nn.Sequential(nn.Linear(6, 10, bias=False), nn.ReLU(), nn.Linear(10, 3, bias=False))
    x = torch.randn(5, 6)
    rel, delta = lumen.LRP(m).attribute(x, target=1, return_convergence_delta=True)
    assert delta.abs().max() < 1e-5                        # bias-free: relevance sums to the output
    # epsilon-LRP on bias-free ReLU networks equals gradient x input
    torch.testing.assert_close(rel, lumen.InputXGradient(m).attribute(x, target=1), rtol=1e-4, atol=1e-6)
    at_hidden = lumen.LayerLRP(m, m[1]).attribute(x, target=1)
    assert at_hidden.shape == (5, 10)
    with torch.no_grad():
        torch.testing.assert_close(at_hidden.sum(1), m(x)[:, 1], rtol=1e-4, atol=1e-5)


def test_combined_layer_and_neuron_variants():
    torch.manual_seed(5)
    mlp = nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.Linear(8, 2))
    x = torch.randn(3, 4)
    base = torch.randn(6, 4) * 0.1
    dls = lumen.DeepLiftShap(mlp).attribute(x, base, target=0)
    with torch.no_grad():
        want = mlp(x)[:, 0] - mlp(base)[:, 0].mean()
    torch.testing.assert_close(dls.sum(1), want, rtol=1e-4, atol=1e-5)      # completeness against the mean baseline output
    # layer variants: attribution of the hidden layer's units
    fa = lumen.LayerFeatureAblation(mlp, mlp[1]).attribute(x, target=0)
    with torch.no_grad():
        h = torch.relu(mlp[0](x))
        exact = h * mlp[2].weight[0]                       # the tail is linear in the hidden units
    torch.testing.assert_close(fa, exact, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(lumen.LayerDeepLift(mlp, mlp[1]).attribute(x, target=0), exact - 0 * exact + (
        -torch.relu(mlp[0](torch.zeros(3, 4))).detach() * mlp[2].weight[0].detach()), rtol=1e-3, atol=1e-4)
    gs = lumen.LayerGradientShap(mlp, mlp[1]).attribute(x, torch.zeros(3, 4), target=0, n_samples=3,
                                                        generator=torch.Generator().manual_seed(0))
    assert gs.shape == (3, 8)
    assert lumen.LayerFeaturePermutation(mlp, mlp[1]).attribute(x, target=0, generator=torch.Generator().manual_seed(0)).shape == (3, 8)
    # neuron variants: hidden unit 2 is relu(w_2 . x + b_2)
    ng = lumen.NeuronGradient(mlp, mlp[0]).attribute(x, 2)
    torch.testing.assert_close(ng, mlp[0].weight[2].detach().expand(3, 4))
    nig = lumen.NeuronIntegratedGradients(mlp, mlp[0]).attribute(x, 2, n_steps=8)
    torch.testing.assert_close(nig, (x * mlp[0].weight[2]).detach(), rtol=1e-4, atol=1e-5)
    nfa = lumen.NeuronFeatureAblation(mlp, mlp[0]).attribute(x, 2)
    torch.testing.assert_close(nfa, (x * mlp[0].weight[2]).detach(), rtol=1e-4, atol=1e-5)
    assert lumen.NeuronGuidedBackprop(mlp, mlp[1]).attribute(x, 2).shape == x.shape
    assert lumen.NeuronDeconvolution(mlp, mlp[1]).attribute(x, 2).shape == x.shape
    # guided Grad-CAM on a small conv net
    conv = nn.Conv2d(1, 3, 3, padding=1)
    net = nn.Sequential(conv, nn.ReLU(), nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(3, 2))
    img = torch.randn(2, 1, 6, 6)
    assert lumen.GuidedGradCam(net, conv).attribute(img, target=1).shape == img.shape
    # summarizers
    s = lumen.Summarizer()
    data = torch.randn(50, 4, generator=torch.Generator().manual_seed(1))
    s.update(data[:20])
    s.update(data[20:])
    torch.testing.assert_close(s.summary["mean"].float(), data.mean(0), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(s.summary["var"].float(), data.var(0, unbiased=False), rtol=1e-5, atol=1e-6)
    cs = lumen.ClassSummarizer(["mean"])
    cs.update(data, torch.arange(50) % 2)
    torch.testing.assert_close(cs.class_summaries[1]["mean"].float(), data[1::2].mean(0), rtol=1e-5, atol=1e-6)


def test_tcav_finds_the_direction_a_model_uses():
    """A model whose output is driven by one hidden direction: the concept whose examples move the hidden state along
    that direction gets a TCAV score near 1, its opposite near 0, and the classifier separates the two."""
    import torch
    from torch import nn
    from tensorplay_b200.lumen import TCAV, Concept
    torch.manual_seed(0)
    d = 12
    body = nn.Linear(d, d, bias=False)
    with torch.no_grad():
        body.weight.copy_(torch.eye(d))
    direction = torch.zeros(d)
    direction[3] = 1.0

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.body = body

        def forward(self, x):
            h = self.body(x)
            return torch.stack((h @ direction, -(h @ direction)), dim=1)

    net = Net()
    plus = Concept(0, "along", [torch.randn(64, d) + 3 * direction for _ in range(2)])
    rand = Concept(1, "random", [torch.randn(64, d) for _ in range(2)])
    tcav = TCAV(net, "body")
    scores = tcav.interpret(torch.randn(40, d), [[plus, rand]], target=0)
    s = scores["0-1"]["body"]
    assert s["sign_count"][0] > 0.95 and s["sign_count"][1] < 0.05 and s["magnitude"][0] > 0.95
    cav = tcav.cavs["0-1"]["body"]
    assert float(cav.stats["accs"]) > 0.9
    v = cav.vector(plus)
    assert v[3] / v.norm() > 0.9                     # the learnt vector points along the planted direction
    # target 1 is the negated read-out: the scores swap
    s1 = tcav.interpret(torch.randn(40, d), [[plus, rand]], target=1)["0-1"]["body"]
    assert s1["sign_count"][0] < 0.05


def test_sparse_autoencoder_recovers_a_planted_dictionary():
    import torch
    from tensorplay_b200.lumen import (SparseAutoencoder, feature_frequency, reconstruction_error,
                                       top_activating_indices, train_sae)
    torch.manual_seed(0)
    d, k, n = 16, 6, 4096
    atoms = torch.nn.functional.normalize(torch.randn(k, d), dim=1)
    codes = (torch.rand(n, k) < 0.15).float() * (torch.rand(n, k) + 0.5)
    x = codes @ atoms
    sae = SparseAutoencoder(d, 24, l1_coeff=3e-2)
    before = float(reconstruction_error(sae, x))
    curve = train_sae(sae, x, steps=1500, batch_size=512, lr=3e-3)
    after = float(reconstruction_error(sae, x))
    assert curve[-1] < curve[0] and after < 0.1 < before
    # every planted atom has a dictionary column pointing its way
    cols = torch.nn.functional.normalize(sae.decoder.weight.t(), dim=1)            # [dict, d]
    assert (atoms @ cols.t()).max(dim=1).values.min() > 0.9
    freq = feature_frequency(sae, x)
    assert freq.shape == (24,) and 0 < freq.max() < 0.6
    best = int(freq.argmax())
    top = top_activating_indices(sae, x, best, k=5)
    assert sae.encode(x[top])[:, best].min() >= sae.encode(x)[:, best].median()


def test_llm_wrappers_and_attention_helpers():
    import torch
    from tensorplay_b200.lumen import LogitLens, collect_hidden_states, token_attention
    from tensorplay_b200.models.llama import Llama, LlamaConfig
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(max_seq_len=16)
    model = Llama(cfg)
    model.reset_parameters(0)
    toks = torch.randint(0, cfg.vocab_size, (2, 8))
    lens = LogitLens(model)
    out = lens.attribute(toks)
    assert out.shape[:3] == (cfg.num_layers, 2, 8) and lens.top_tokens(toks, k=3).shape == (cfg.num_layers, 2, 3)
    hs = collect_hidden_states(model, toks)
    assert len(hs) == cfg.num_layers and hs[0].shape == (2, 8, cfg.hidden_size)
    att = [torch.softmax(torch.randn(2, 4, 8, 8), -1) for _ in range(3)]
    ta = token_attention(att, query_position=-1)
    assert ta.shape == (2, 8) and torch.allclose(ta.sum(-1), torch.ones(2), atol=1e-5)
    assert torch.allclose(token_attention(att, -1, layer=1, head=2), att[1][:, 2, -1])


def test_surrogate_linear_models_recover_planted_weights():
    import torch
    from tensorplay_b200 import lumen as L
    torch.manual_seed(0)
    n, d = 512, 6
    x = torch.randn(n, d)
    w_true = torch.tensor([2.0, -1.0, 0.0, 0.0, 0.5, 0.0])
    y = x @ w_true + 0.3
    loader = [(x[i: i + 128], y[i: i + 128], torch.ones(128)) for i in range(0, n, 128)]
    for cls, kw, tol in ((L.SkLearnLinearRegression, {}, 1e-4), (L.SkLearnRidge, {"alpha": 1e-3}, 1e-3),
                         (L.SkLearnLasso, {"alpha": 1e-3}, 2e-2)):
        m = cls(**kw)
        stats = m.fit(loader)
        assert (m.representation()[0] - w_true).abs().max() < tol and abs(float(m.bias()) - 0.3) < tol and stats["train_loss"] < 1e-3
    m = L.SGDLinearRegression()
    m.fit(loader, max_epoch=300, initial_lr=0.05)
    assert (m.representation()[0] - w_true).abs().max() < 0.05
    lasso = L.SGDLasso()
    lasso.fit(loader, max_epoch=300, initial_lr=0.05, alpha=0.05)
    rep = lasso.representation()[0]
    assert rep[[2, 3, 5]].abs().max() < 0.05 < rep[[0, 1, 4]].abs().min()          # the penalty zeroes the unused features
    # sample weights: rows with weight zero do not count
    y_bad = y.clone()
    y_bad[:256] += 100.0
    wts = torch.cat((torch.zeros(256), torch.ones(256)))
    m = L.SkLearnLinearRegression()
    m.fit([(x, y_bad, wts)])
    assert (m.representation()[0] - w_true).abs().max() < 1e-3
    g = L.compute_gradients(lambda a: (a * a).sum(1, keepdim=True), x[:4], target_ind=0)
    assert torch.allclose(g, 2 * x[:4])


def test_cross_layer_transcoder_learns_the_blocks_updates():
    import torch
    from tensorplay_b200.lumen import (CrossLayerTranscoder, collect_component_updates, train_clt,
                                       visualize_attention_heads, visualize_attention_multi_layer, visualize_token_attention)
    from tensorplay_b200.models.llama import Llama, LlamaConfig
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(max_seq_len=16)
    model = Llama(cfg)
    model.reset_parameters(0)
    toks = torch.randint(0, cfg.vocab_size, (16, 16))
    ins, ups = collect_component_updates(model, toks)
    assert len(ins) == len(ups) == cfg.num_layers and ins[0].shape == ups[0].shape == (16, 16, cfg.hidden_size)
    # the update of block l is its output minus its input: the residual stream entering block l + 1
    assert torch.allclose(ins[0] + ups[0], ins[1], atol=1e-5)
    clt = CrossLayerTranscoder(cfg.num_layers, cfg.hidden_size, 4 * cfg.hidden_size, l1_coeff=1e-4)
    curve = train_clt(clt, ins, ups, steps=150, batch_size=128, lr=3e-3)
    assert curve[-1] < 0.5 * curve[0]
    preds, feats = clt([x.reshape(-1, cfg.hidden_size) for x in ins])
    assert len(preds) == cfg.num_layers and feats[0].shape[-1] == 4 * cfg.hidden_size and (feats[0] >= 0).all()
    att = [torch.softmax(torch.randn(2, 3, 6, 6), -1) for _ in range(2)]
    assert visualize_attention_heads(att[0]).shape == (6, 3 * 7 - 1)
    assert visualize_attention_multi_layer(att).shape == (2 * 7 - 1, 3 * 7 - 1)
    html = visualize_token_attention(att, list("abcdef"))
    assert html.count("<span") == 6 and "rgba(255, 120, 0, 1.000)" in html


def test_attribution_graph_edges_sum_to_the_explained_preactivation():
    """With zero encoder biases and inputs that are exactly what the earlier features wrote, the edges into a node add up
    to its pre-activation: the linearity the graph relies on."""
    import torch
    from tensorplay_b200.lumen import AttributionGraph, CrossLayerTranscoder, FeatureCircuit, top_attention_heads
    torch.manual_seed(0)
    L, d, D = 3, 8, 12
    clt = CrossLayerTranscoder(L, d, D)
    with torch.no_grad():
        for enc in clt.encoders:
            enc.bias.zero_()
        clt.b_dec.zero_()
        for l in range(L):
            for dec in clt.decoders[l]:
                dec.weight.copy_(torch.randn(d, D) * 0.3)
    # build a residual stream that the transcoder itself explains: x_0 random, x_{m} = sum of updates written for layers < m
    x0 = torch.randn(d)
    xs = [x0]
    feats = []
    for m in range(1, L + 1):
        feats.append(torch.relu(clt.encoders[m - 1](xs[m - 1])))
        if m < L:
            xs.append(sum(clt.decoders[l][k - l](feats[l]) for l in range(m) for k in range(l, m)))
    g = AttributionGraph(clt).build(xs, top_k=D)
    assert all(e.src != e.dst and g.nodes[e.src].layer < g.nodes[e.dst].layer for e in g.edges)
    for i, n in enumerate(g.nodes):
        if n.layer == 0:
            continue
        incoming = sum(e.weight for e in g.incoming(i))
        pre = float((clt.encoders[n.layer].weight[n.feature] @ xs[n.layer]).detach())
        assert abs(incoming - pre) < 1e-4 * max(1.0, abs(pre)) and abs(pre - n.activation) < 1e-5   # active: relu is the identity
    direction = torch.randn(d)
    circ = FeatureCircuit(clt).build(xs, direction, top_k=2)
    assert len(circ.nodes) <= 2 * L and all(abs(e.weight) >= 0 for e in circ.edges)
    att = [torch.zeros(1, 2, 4, 4) for _ in range(2)]
    att[1][0, 1, -1, 0] = 0.9
    att[0][0, 0, -1, 0] = 0.4
    assert [(l, h) for l, h, _ in top_attention_heads(att, k=2)] == [(1, 1), (0, 0)]
