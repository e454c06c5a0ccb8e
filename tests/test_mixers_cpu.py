"""Latent attention and gated delta rule: closed-form checks and cache consistency."""
import torch

import tensorplay_b200 as tp
from tensorplay_b200.nn import DynamicCache, GatedDeltaNet, LinearStateCache, MultiheadLatentAttention, gated_delta_rule


def test_latent_attention_cache_matches_full_forward_and_formula():
    torch.manual_seed(0)
    m = MultiheadLatentAttention(embed_dim=64, num_heads=4, kv_lora_rank=24, qk_nope_head_dim=16,
                                 qk_rope_head_dim=8, v_head_dim=16, q_lora_rank=32).eval()
    x = torch.randn(2, 10, 64)
    full = m(x)
    assert full.shape == x.shape
    # prefill 6 tokens, then 4 single-token steps through the compressed cache
    cache = DynamicCache()
    outs = [m(x[:, :6], past_key_values=cache)]
    for t in range(6, 10):
        outs.append(m(x[:, t:t + 1], past_key_values=cache))
    torch.testing.assert_close(torch.cat(outs, 1), full, rtol=1e-4, atol=1e-5)
    # the cache holds one latent and one rotary key per token, not per-head keys / values
    lat, rot = cache.update(torch.empty(2, 1, 0, 24), torch.empty(2, 1, 0, 8), 0)
    assert lat.shape == (2, 1, 10, 24) and rot.shape == (2, 1, 10, 8)
    # causality: the output at position t does not depend on later tokens
    x2 = x.clone()
    x2[:, 7:] += 1.0
    torch.testing.assert_close(m(x2)[:, :7], full[:, :7], rtol=1e-4, atol=1e-5)


def test_gated_delta_rule_matches_explicit_state_update():
    torch.manual_seed(1)
    B, T, H, Dk, Dv = 2, 5, 3, 4, 6
    q, k = torch.randn(B, T, H, Dk), torch.nn.functional.normalize(torch.randn(B, T, H, Dk), dim=-1)
    v, g, beta = torch.randn(B, T, H, Dv), -torch.rand(B, T, H), torch.rand(B, T, H)
    o, S = gated_delta_rule(q, k, v, g, beta)
    # explicit matrices, one (batch, head) at a time
    for b in range(B):
        for h in range(H):
            St = torch.zeros(Dk, Dv)
            for t in range(T):
                kt = k[b, t, h].unsqueeze(1)
                St = torch.exp(g[b, t, h]) * St
                St = (torch.eye(Dk) - beta[b, t, h] * kt @ kt.t()) @ St + beta[b, t, h] * kt @ v[b, t, h].unsqueeze(0)
                torch.testing.assert_close(o[b, t, h], St.t() @ q[b, t, h], rtol=1e-4, atol=1e-5)
            torch.testing.assert_close(S[b, h], St, rtol=1e-4, atol=1e-5)
    # a second call continuing from the state equals one long call
    o1, S1 = gated_delta_rule(q[:, :3], k[:, :3], v[:, :3], g[:, :3], beta[:, :3])
    o2, S2 = gated_delta_rule(q[:, 3:], k[:, 3:], v[:, 3:], g[:, 3:], beta[:, 3:], S1)
    torch.testing.assert_close(torch.cat((o1, o2), 1), o)


def test_gated_delta_net_streaming_equals_full_sequence_and_trains():
    torch.manual_seed(2)
    m = GatedDeltaNet(embed_dim=32, num_heads=2, head_dim=8, conv_size=4)
    x = torch.randn(2, 9, 32)
    full = m(x)
    cache = LinearStateCache()
    parts = [m(x[:, :4], past_key_values=cache)] + [m(x[:, t:t + 1], past_key_values=cache) for t in range(4, 9)]
    torch.testing.assert_close(torch.cat(parts, 1), full, rtol=1e-4, atol=1e-5)
    full.pow(2).mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.parameters())
    assert tp.nn.GatedDeltaNet is GatedDeltaNet


def test_chunked_delta_rule_equals_token_recurrence():
    from tensorplay_b200.nn import chunk_gated_delta_rule
    torch.manual_seed(3)
    B, T, H, Dk, Dv = 2, 37, 2, 8, 5
    q, k = torch.randn(B, T, H, Dk), torch.nn.functional.normalize(torch.randn(B, T, H, Dk), dim=-1)
    v, g, beta = torch.randn(B, T, H, Dv), -0.3 * torch.rand(B, T, H), torch.rand(B, T, H)
    s0 = torch.randn(B, H, Dk, Dv)
    o_ref, s_ref = gated_delta_rule(q, k, v, g, beta, s0)
    for chunk in (8, 16, 64):
        o, s = chunk_gated_delta_rule(q, k, v, g, beta, s0, chunk=chunk)
        torch.testing.assert_close(o, o_ref, rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(s, s_ref, rtol=1e-4, atol=1e-4)


def test_kimi_delta_attention_streaming_and_per_channel_decay():
    from tensorplay_b200.nn import KimiDeltaAttention
    torch.manual_seed(4)
    m = KimiDeltaAttention(embed_dim=32, num_heads=2, head_dim=8, gate_rank=4)
    x = torch.randn(2, 7, 32)
    full = m(x)
    cache = LinearStateCache()
    parts = [m(x[:, :3], past_key_values=cache)] + [m(x[:, t:t + 1], past_key_values=cache) for t in range(3, 7)]
    torch.testing.assert_close(torch.cat(parts, 1), full, rtol=1e-4, atol=1e-5)
    # with a decay that is constant over the channels the fine-grained rule equals the head-scalar one
    B, T, H, Dk, Dv = 1, 6, 2, 4, 3
    q, k = torch.randn(B, T, H, Dk), torch.nn.functional.normalize(torch.randn(B, T, H, Dk), dim=-1)
    v, g, beta = torch.randn(B, T, H, Dv), -torch.rand(B, T, H), torch.rand(B, T, H)
    o1, _ = gated_delta_rule(q, k, v, g, beta)
    o2, _ = gated_delta_rule(q, k, v, g.unsqueeze(-1).expand(B, T, H, Dk), beta)
    torch.testing.assert_close(o1, o2)


def test_causal_encoder_decoder_shapes_mixers_and_gradients():
    from tensorplay_b200.nn import CausalEncoderDecoder
    torch.manual_seed(6)
    m = CausalEncoderDecoder(hidden_size=32, num_heads=4, n_encoder_layers=2, n_decoder_layers=2, num_kv_heads=2)
    x = torch.randn(2, 6, 32)
    y = m(x)
    assert y.shape == x.shape
    y.pow(2).mean().backward()
    assert all(p.grad is not None for p in m.parameters())
    # the mixer is swappable per layer: a linear-time mixer in both stacks
    m2 = CausalEncoderDecoder(32, 4, 1, 1, mixer_factory=lambda w, i: GatedDeltaNet(w, 2, head_dim=8, layer_idx=i))
    assert m2(x).shape == x.shape


def test_compressed_sparse_attention_causality_and_tiers():
    from tensorplay_b200.nn import CompressedSparseAttention
    torch.manual_seed(7)
    m = CompressedSparseAttention(hidden_size=32, num_heads=4, head_dim=8, q_lora_rank=16, compress_rate=4,
                                  window_size=6, index_n_heads=2, index_head_dim=8, index_topk=2).eval()
    x = torch.randn(2, 24, 32)
    y = m(x)
    assert y.shape == x.shape
    # causal: outputs before position 13 do not depend on tokens from 13 on (also through the
    # compressed entries: an entry is visible only when all of its source tokens are in the past)
    x2 = x.clone()
    x2[:, 13:] += 1.0
    torch.testing.assert_close(m(x2)[:, :13], y[:, :13], rtol=1e-4, atol=1e-5)
    # the compressed tier matters: beyond the window, distant tokens still influence the output
    x3 = x.clone()
    x3[:, 0:4] += 1.0           # far outside the 6-token window of position 23, inside entry 0
    assert (m(x3)[:, 23] - y[:, 23]).abs().max() > 1e-6
    y.pow(2).mean().backward()
    assert m.sinks.grad is not None and m.compress_gate.weight.grad is not None


def test_reference_spellings_of_the_delta_rules_and_gated_norm():
    """Per-channel decay: the chunked form (factorised decay, float64 chunk matrices) equals the token-by-token form,
    with an initial state and over a ragged last chunk; the head-scalar recurrent spelling equals the chunked one."""
    import torch
    from tensorplay_b200 import nn
    torch.manual_seed(0)
    B, T, H, Dk, Dv = 2, 150, 3, 16, 8
    q, k, v = torch.randn(B, T, H, Dk), torch.randn(B, T, H, Dk), torch.randn(B, T, H, Dv)
    beta, s0 = torch.rand(B, T, H), torch.randn(B, H, Dk, Dv) * 0.1
    g = -torch.rand(B, T, H, Dk) * 0.3
    o1, s1 = nn.recurrent_kimi_delta_rule(q, k, v, g, beta, s0, True, True)
    o2, s2 = nn.chunk_kimi_delta_rule(q, k, v, g, beta, 64, s0, True, True)
    assert (o1 - o2).abs().max() < 1e-5 and (s1 - s2).abs().max() < 1e-5
    assert nn.chunk_kimi_delta_rule(q, k, v, g, beta)[1] is None
    gs = -torch.rand(B, T, H) * 0.3
    o3, s3 = nn.recurrent_gated_delta_rule(q, k, v, gs, beta, None, True, True)
    kn = torch.nn.functional.normalize(k, dim=-1)
    qn = torch.nn.functional.normalize(q, dim=-1) * Dk ** -0.5
    o4, s4 = nn.chunk_gated_delta_rule(qn, kn, v, gs, beta)
    assert (o3 - o4).abs().max() < 1e-5 and (s3 - s4).abs().max() < 1e-5
    norm = nn.GatedRMSNorm(8, activation="sigmoid")
    x, gate = torch.randn(4, 8), torch.randn(4, 8)
    want = torch.nn.functional.rms_norm(x, (8,), eps=1e-6) * torch.sigmoid(gate)
    assert torch.allclose(norm(x, gate), want, atol=1e-6)
    conv = nn.DepthwiseConv2d(4, 8, 3, padding=1)
    assert conv.groups == 4 and conv(torch.randn(1, 4, 9, 9)).shape == (1, 8, 9, 9)
