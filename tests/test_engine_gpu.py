"""Single-GPU sharded engine on the sm_100a kernels against an fp32 PyTorch run of the same model."""
import copy

import pytest
import torch

import tensorplay_b200.ops as O
from tensorplay_b200.models.llama import Llama, LlamaConfig
from tensorplay_b200.parallel import AdamWConfig, FSDPEngine

pytestmark = pytest.mark.gpu


def test_engine_llama_bf16_tracks_fp32_reference():
    torch.manual_seed(0)
    dev = torch.device("cuda")
    cfg = LlamaConfig.tiny(hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64, ffn_size=512,
                           vocab_size=512, num_layers=2)
    model = Llama(cfg, device=dev, dtype=torch.bfloat16)
    model.reset_parameters(seed=0)
    ref = copy.deepcopy(model).float().cpu()
    tok = torch.randint(0, cfg.vocab_size, (2, 128), device=dev)
    tgt = torch.randint(0, cfg.vocab_size, (2, 128), device=dev)
    ocfg = AdamWConfig(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    eng = FSDPEngine(model, ocfg, activation_checkpointing=True)
    losses = [float(eng.step(tok, tgt)) for _ in range(6)]
    O.check_status()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref_losses = []
    for _ in range(6):
        opt.zero_grad()
        loss = ref(tok.cpu(), tgt.cpu())
        loss.backward()
        opt.step()
        ref_losses.append(float(loss))
    assert losses[-1] < losses[0]
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 0.05, (losses, ref_losses)
