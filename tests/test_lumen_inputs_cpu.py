"""Interpretable inputs, language-model attribution over them, streaming statistics, generic LIME,
data-loader attribution, graph-mode guided backprop and the presentation helpers."""
import numpy as np
import pytest
import torch
from torch import nn

import tensorplay_b200.lumen as L


class _Tok:
    """Whitespace tokenizer over a growing vocabulary (ids from 1; 0 = <unk>)."""

    def __init__(self):
        self.vocab = {"<unk>": 0}

    def _id(self, w):
        return self.vocab.setdefault(w, len(self.vocab))

    def encode(self, text, return_tensors=None, add_special_tokens=True):
        ids = [self._id(w) for w in text.split()]
        return torch.tensor([ids]) if return_tensors == "pt" else ids

    def decode(self, ids):
        inv = {v: k for k, v in self.vocab.items()}
        return " ".join(inv[int(i)] for i in ids)

    def convert_ids_to_tokens(self, ids):
        inv = {v: k for k, v in self.vocab.items()}
        return [inv[int(i)] for i in ids]

    def convert_tokens_to_ids(self, toks):
        return [self._id(t) for t in toks]


class _KeywordLM(nn.Module):
    """Next-token logits favour token ``yes`` in proportion to how many ``good`` tokens the prefix holds."""

    def __init__(self, good_id, yes_id, vocab=32):
        super().__init__()
        self.good, self.yes, self.vocab = good_id, yes_id, vocab
        self.dummy = nn.Parameter(torch.zeros(1))

    def forward(self, ids):
        count = torch.cumsum((ids == self.good).float(), 1)
        logits = torch.zeros(ids.shape[0], ids.shape[1], self.vocab)
        logits[..., self.yes] = 2.0 * count
        return logits

    def generate(self, ids, max_new_tokens=2, **kw):
        for _ in range(max_new_tokens):
            ids = torch.cat((ids, self.forward(ids)[:, -1].argmax(-1, keepdim=True)), 1)
        return ids


def test_text_inputs_build_perturbed_prompts():
    t = L.TextTemplateInput("{} lives in {} and works as {}", ["Ann", "Oslo", "a pilot"], baselines=["Someone", "a city", "a worker"],
                            mask=[0, 1, 1])
    assert t.to_tensor().shape == (1, 2)
    assert t.to_model_input() == "Ann lives in Oslo and works as a pilot"
    assert t.to_model_input(torch.tensor([[1, 0]])) == "Ann lives in a city and works as a worker"
    assert t.format_attr(torch.tensor([0.5, 2.0])).tolist() == [0.5, 2.0, 2.0]
    d = L.TextTemplateInput(lambda name, city: f"{name}@{city}", {"name": "Ann", "city": "Oslo"})
    assert d.to_model_input(torch.tensor([[0, 1]])) == "@Oslo"
    tok = _Tok()
    ti = L.TextTokenInput("the good good film .", tok, baselines=0, skip_tokens=["."])
    assert ti.values == ["the", "good", "good", "film"] and ti.to_tensor().shape == (1, 4)
    out = ti.to_model_input(torch.tensor([[1, 0, 1, 1]]))
    assert out.tolist() == [[tok.vocab["the"], 0, tok.vocab["good"], tok.vocab["film"], tok.vocab["."]]]
    pb = L.ProductBaselines({"name": ["A", "B"], ("city", "country"): [("Oslo", "NO"), ("Rome", "IT")]}, seed=0)
    s = pb()
    assert s["name"] in "AB" and (s["city"], s["country"]) in (("Oslo", "NO"), ("Rome", "IT"))
    assert L.TokenReferenceBase(7).generate_reference(3).tolist() == [7, 7, 7]


def test_llm_attribution_finds_the_tokens_that_drive_the_answer():
    tok = _Tok()
    ti = L.TextTokenInput("the good good film", tok)
    yes = tok.convert_tokens_to_ids(["yes"])[0]
    model = _KeywordLM(tok.vocab["good"], yes)
    res = L.LLMAttribution(L.FeatureAblation(model), tok).attribute(ti, target="yes yes")
    assert res.input_tokens == ["the", "good", "good", "film"] and res.output_tokens == ["yes", "yes"]
    assert res.token_attr.shape == (2, 4) and res.output_probs.shape == (2,)
    s = res.seq_attr
    assert s[1] > 0.1 and s[2] > 0.1 and abs(float(s[0])) < 1e-6 and abs(float(s[3])) < 1e-6
    assert torch.allclose(res.token_attr.sum(0), s, atol=1e-5)          # log-probabilities add over the target tokens
    assert list(res.seq_attr_dict) == ["the", "good", "film"] or len(res.seq_attr_dict) == 3   # duplicate words share a key
    # no target: the model's own continuation is explained
    gen = L.LLMAttribution(L.FeatureAblation(model), tok).attribute(ti, gen_args={"max_new_tokens": 2})
    assert gen.output_tokens == ["yes", "yes"]
    # a surrogate method explains the sequence only
    lime = L.LLMAttribution(L.Lime(model), tok).attribute(ti, target="yes", n_samples=40, generator=torch.Generator().manual_seed(0))
    assert lime.token_attr is None and lime.seq_attr[1] > abs(lime.seq_attr[0])
    with pytest.raises(ImportError):
        res.plot_seq_attr()

    class Fake(L.RemoteLLMProvider):
        api_url = "fake"

        def generate(self, prompt, **kw):
            return "yes"

        def get_logprobs(self, input_prompt, target_str, tokenizer=None):
            n = len(target_str.split())
            return [-1.0 / (1 + input_prompt.split().count("good"))] * n
    remote = L.RemoteLLMAttribution(L.FeatureAblation(lambda *a: 0), tok, Fake()).attribute(ti)
    assert remote.output_tokens == ["yes"] and remote.seq_attr[1] > 0 and float(remote.seq_attr[0]) == 0.0
    with pytest.raises(ValueError):
        L.VLLMProvider("  ")


def test_image_mask_input_paints_absent_segments():
    from PIL import Image
    img = Image.fromarray(np.full((4, 6, 3), 100, dtype=np.uint8))
    mask = torch.zeros(4, 6, dtype=torch.long)
    mask[:, 3:] = 1
    inp = L.ImageMaskInput(img, mask=mask, processor_fn=lambda im: torch.from_numpy(np.array(im)))
    assert inp.to_tensor().shape == (1, 2) and inp.values == ["image_feature_0", "image_feature_1"]
    out = inp.to_model_input(torch.tensor([[1, 0]]))
    assert out[:, :3].unique().tolist() == [100] and out[:, 3:].unique().tolist() == [255]
    px = inp.format_pixel_attr(torch.tensor([[1.0, -2.0]]))
    assert px.shape == (1, 4, 6) and float(px[0, 0, 0]) == 1.0 and float(px[0, 0, 5]) == -2.0


def test_stats_embedding_wrapper_and_generic_lime():
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(50, 3, generator=g).double()
    s = L.SummarizerSingleTensor([L.Mean(), L.Var(), L.Var(order=1), L.StdDev(), L.Min(), L.Max(), L.Sum(), L.Count(), L.MSE()])
    for part in x.split(7):
        s.update(part)
    got = s.summary
    assert torch.allclose(got["mean"], x.mean(0)) and torch.allclose(got["var"], x.var(0, unbiased=False))
    assert torch.allclose(got["var(order=1)"], x.var(0)) and torch.allclose(got["stddev"], x.std(0, unbiased=False))
    assert torch.equal(got["min"], x.amin(0)) and torch.equal(got["max"], x.amax(0)) and got["count"] == 50
    assert torch.allclose(got["sum"], x.sum(0)) and torch.allclose(got["mse"], ((x - x.mean(0)) ** 2).sum(0))

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(10, 4)
            self.head = nn.Linear(4, 2)

        def forward(self, ids_or_emb):
            return self.head(self.emb(ids_or_emb).mean(1))
    net = Net()
    ids = torch.tensor([[1, 2, 3]])
    want = net(ids)
    wrapper = L.configure_interpretable_embedding_layer(net, "emb")
    emb = wrapper.indices_to_embeddings(ids)
    assert torch.allclose(net(emb), want)
    attr = L.IntegratedGradients(net).attribute(emb, target=1, n_steps=16)
    assert attr.shape == emb.shape
    L.remove_interpretable_embedding_layer(net, wrapper)
    assert isinstance(net.emb, nn.Embedding) and torch.allclose(net(ids), want)

    # generic LIME recovers the weights of a linear model over binary features
    w = torch.tensor([2.0, -1.0, 0.5, 0.0])
    lime = L.LimeBase(lambda z: (z * w).sum(-1), lambda a, y, wt: torch.linalg.lstsq(torch.cat((a, torch.ones(len(a), 1, dtype=a.dtype)), 1)
                                                                                    * wt[:, None].sqrt(), (y * wt.sqrt())[:, None]).solution[:-1, 0],
                      similarity_func=lambda inp, pert, interp, **kw: 1.0,
                      perturb_func=lambda inp, **kw: (torch.rand(1, 4, generator=g) < 0.5).float(),
                      perturb_interpretable_space=True, from_interp_rep_transform=lambda z, inp, **kw: z, to_interp_rep_transform=None)
    coef = lime.attribute(torch.ones(1, 4), n_samples=60)
    assert torch.allclose(coef[0], w, atol=1e-4)


def test_dataloader_attribution_and_deeplift_shap_variants():
    torch.manual_seed(0)                         # initial weights of the small networks
    g = torch.Generator().manual_seed(1)
    x = torch.randn(12, 3, generator=g)
    w = torch.tensor([1.0, -2.0, 0.0])
    y = (x * w).sum(-1)
    loader = [(x[i: i + 4], y[i: i + 4]) for i in range(0, 12, 4)]
    model = lambda inp: (inp * w).sum(-1)          # noqa: E731
    dl = L.DataLoaderAttribution(L.FeatureAblation(model))
    attr = dl.attribute(loader, input_roles=[0, 2], reduce=lambda acc, out, batch: ((out - batch[1]) ** 2).sum() + (0 if acc is None else acc),
                        to_metric=lambda acc: -acc / 12)
    # ablating feature k (to 0) raises the squared error by w_k^2 * mean(x_k^2); the unused feature gets 0
    want = (w ** 2) * (x ** 2).mean(0)
    assert torch.allclose(attr.reshape(-1), want, atol=1e-5)

    net = nn.Sequential(nn.Linear(3, 5), nn.ReLU(), nn.Linear(5, 2))
    inp, base = torch.randn(2, 3, generator=g), torch.randn(4, 3, generator=g)
    a = L.LayerDeepLiftShap(net, net[1]).attribute(inp, base, target=0)
    assert a.shape == (2, 5)
    # completeness at the layer: attributions sum to the output difference to the mean baseline output
    diff = net(inp)[:, 0] - net(base)[:, 0].mean()
    assert torch.allclose(a.sum(-1), diff, atol=1e-3)
    n = L.NeuronDeepLiftShap(net, net[0]).attribute(inp, 2, baselines=base)
    lin = net[0]
    assert torch.allclose(n, lin.weight[2][None] * (inp - base.mean(0)), atol=1e-5)   # a linear neuron: w * (x - E[b])


def test_graph_mode_and_presentation():
    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(4, 6), nn.ReLU(), nn.Linear(6, 3))
    names = L.node_names(net)
    assert names[0] == "input_1" or names[0].startswith("input") and names[-1] == "output"
    x = torch.randn(2, 4, generator=torch.Generator().manual_seed(2))
    (g,) = L.graph_gradient_func(net, x.clone().requires_grad_(), 1)
    (want,) = torch.autograd.grad(net(x.requires_grad_())[:, 1].sum(), x)
    assert torch.allclose(g, want, atol=1e-6)
    hooked = L.GuidedBackprop(net).attribute(x.detach().clone(), target=1)
    graph = L.GraphGuidedBackprop(net).attribute(x.detach().clone(), target=1)
    assert torch.allclose(hooked, graph, atol=1e-6)
    assert torch.allclose(L.Deconvolution(net).attribute(x.detach().clone(), target=1),
                          L.GraphDeconvolution(net).attribute(x.detach().clone(), target=1), atol=1e-6)

    class Branchy(nn.Module):
        def forward(self, x):
            return x if x.sum() > 0 else -x
    b = Branchy()
    assert L.trace(b) is b                                    # not traceable: returned as it is

    V = L.visualization
    attr = np.zeros((4, 4, 3))
    attr[0, 0] = 1.0
    attr[3, 3] = -1.0
    hm = V.heat_map(attr, sign="all", outlier_perc=0)
    assert hm.shape == (4, 4, 3) and hm[0, 0].tolist() == [255, 0, 0] and hm[3, 3].tolist() == [0, 0, 255] and hm[1, 1].tolist() == [255] * 3
    n = V.normalize_attr(torch.tensor([[0.0, 2.0], [-4.0, 1.0]]), "positive", outlier_perc=0)
    assert n.max() == 1.0 and n.min() == 0.0
    cell = V.format_word_importances(["good", "<pad>"], [0.8, -0.5])
    assert "hsl(120" in cell and "hsl(0" in cell and "#pad" in cell
    rec = V.VisualizationDataRecord([0.8, -0.5], 0.9, "pos", "pos", "pos", 0.3, ["good", "bad"])
    page = V.visualize_text([rec])
    assert "<table" in page and "Legend" in page and "good" in page
    with pytest.raises(ImportError):
        V.visualize_image_attr(attr)
