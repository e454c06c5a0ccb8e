"""Looking inside a decoder language model with ``tensorplay_b200.lumen``: logit lens, activation patching, a sparse
autoencoder on the residual stream and a cross-layer transcoder with its attribution graph - on a tiny random-init Llama,
so it runs in seconds on CPU (with a trained checkpoint the same calls give meaningful pictures).

    python examples/interpret_llm.py [--steps 200]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tensorplay_b200 import lumen  # noqa: E402
from tensorplay_b200.models.llama import Llama, LlamaConfig  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    a = ap.parse_args()
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(max_seq_len=32)
    model = Llama(cfg)
    model.reset_parameters(0)
    tokens = torch.randint(0, cfg.vocab_size, (8, 24))

    lens = lumen.LogitLens(model)
    top = lens.top_tokens(tokens, position=-1, k=3)
    print(f"logit lens: top-3 next tokens per layer for sequence 0: {top[:, 0].tolist()}")

    corrupt = tokens.clone()
    corrupt[:, 5] = (corrupt[:, 5] + 1) % cfg.vocab_size
    target = int(model(tokens)[0, -1].argmax())
    effect = lumen.ActivationPatching(model).attribute(tokens[:1], corrupt[:1], lambda logits: logits[0, -1, target],
                                                        positions=[4, 5, 6])
    print(f"activation patching: restoring position 5 moves the target logit most at layer "
          f"{int(effect[:, 1].abs().argmax())} (effects {effect[:, 1].tolist()})")

    hidden = lumen.collect_hidden_states(model, tokens)[-1]
    sae = lumen.SparseAutoencoder(cfg.hidden_size, 4 * cfg.hidden_size, l1_coeff=1e-3)
    before = float(lumen.reconstruction_error(sae, hidden))
    lumen.train_sae(sae, hidden, steps=a.steps, batch_size=128, lr=3e-3)
    after = float(lumen.reconstruction_error(sae, hidden))
    print(f"sparse autoencoder: unexplained variance {before:.3f} -> {after:.3f}; most frequent feature fires on "
          f"{float(lumen.feature_frequency(sae, hidden).max()):.2f} of the tokens")

    ins, ups = lumen.collect_component_updates(model, tokens)
    clt = lumen.CrossLayerTranscoder(cfg.num_layers, cfg.hidden_size, 2 * cfg.hidden_size, l1_coeff=1e-4)
    curve = lumen.train_clt(clt, ins, ups, steps=a.steps, batch_size=128, lr=3e-3)
    graph = lumen.AttributionGraph(clt).build([x[0, -1] for x in ins], top_k=4)
    strongest = max(graph.edges, key=lambda e: abs(e.weight)) if graph.edges else None
    print(f"cross-layer transcoder: loss {curve[0]:.3f} -> {curve[-1]:.3f}; attribution graph with {len(graph.nodes)} nodes "
          f"and {len(graph.edges)} edges" + (f", strongest edge layer {graph.nodes[strongest.src].layer} -> "
                                             f"{graph.nodes[strongest.dst].layer} ({strongest.weight:+.3f})" if strongest else ""))
    if not (after < before and curve[-1] < curve[0]):
        sys.exit(1)


if __name__ == "__main__":
    main()
