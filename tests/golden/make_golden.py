"""Compares the plain implementation (tests/plain_qwen2.py) ONCE with the reference's own model
code on tiny random models, and stores the reference's outputs beside this script.

    python tests/golden/make_golden.py /path/to/TuringServe

It imports ``turingserve`` from the given checkout (CPU, float32, ``get_ops("reference")``), builds
each tiny model folder with this repository's random-weights writer, runs the reference's
``Qwen2Model.forward_dense`` / paged ``forward`` / ``generate_greedy`` on it, checks that the plain
implementation agrees, and writes ``tiny_<name>.npz``: token ids, logits at every position, the
hidden states of every layer, a greedy continuation and fingerprints of the weights (so that a
change of the random writer shows up as a fingerprint mismatch, not as a numerics failure).

Tiny B has a separate output head, which the reference's loader refuses
(turingserve/model/loader.py:99-100): its ``Weights`` are built by hand and the head is applied
outside.  The windowed configuration has no counterpart in the reference and is not stored.
"""

from __future__ import annotations

import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if len(sys.argv) < 2:
    raise SystemExit("usage: python tests/golden/make_golden.py /path/to/TuringServe")
REF = sys.argv[1]
sys.path.insert(0, REF)
sys.path.insert(0, ROOT)              # this repository's ``tests`` package wins over the reference's

from tests import plain_qwen2 as plain  # noqa: E402
from tests import tiny  # noqa: E402
from turingserve.model.layers import LayerWeights, LinearWeight, Weights  # noqa: E402
from turingserve.model.qwen2 import Qwen2Model  # noqa: E402
from turingserve.model.qwen2_config import Qwen2Config  # noqa: E402
from turingserve.ops import get_ops  # noqa: E402
from turingserve.runner.contiguous_cache import ContiguousCache  # noqa: E402
from turingserve.simple_generate import generate_greedy  # noqa: E402


def reference_model(cfg: dict, w: dict):
    rc = Qwen2Config.from_dict({**cfg, "tie_word_embeddings": True})
    layers = []
    for i in range(rc.num_layers):
        p = f"model.layers.{i}."
        cat = lambda names, kind: torch.cat([w[p + n + kind] for n in names], dim=0)  # noqa: E731
        layers.append(LayerWeights(
            w_in=w[p + "input_layernorm.weight"],
            qkv=LinearWeight(cat(["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"], ".weight"),
                             cat(["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"], ".bias")),
            o=LinearWeight(w[p + "self_attn.o_proj.weight"]), w_post=w[p + "post_attention_layernorm.weight"],
            gu=LinearWeight(cat(["mlp.gate_proj", "mlp.up_proj"], ".weight")),
            down=LinearWeight(w[p + "mlp.down_proj.weight"])))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    weights = Weights(embed=w["model.embed_tokens.weight"], layers=layers, w_norm=w["model.norm.weight"])
    model = Qwen2Model(rc, weights, get_ops("reference"), torch.device("cpu"), torch.float32,
                       cfg["max_position_embeddings"])
    return model, head


def main() -> None:
    for name, n_tokens in (("A", 33), ("B", 70)):
        with tempfile.TemporaryDirectory() as tmp:
            folder = tiny.make_tiny_folder(name, tmp)
            cfg, w = plain.read_folder(folder)
        ids = tiny.random_ids(n_tokens, cfg["vocab_size"], 5)
        model, head = reference_model(cfg, w)
        t = torch.tensor(ids)
        with torch.inference_mode():
            x, hiddens = model.forward_dense(t, torch.arange(n_tokens), return_hidden=True)
            ref_logits = (x @ head.T).float()
            cache = ContiguousCache(model.cfg, n_tokens, "cpu", torch.float32)
            xc = model.forward_contiguous(t[:20], torch.arange(20), cache, 0)
            xc2 = model.forward_contiguous(t[20:], torch.arange(20, n_tokens), cache, 20)
            chunked = (torch.cat([xc, xc2]) @ head.T).float()
        mine, my_hidden = plain.forward(cfg, w, ids, return_hidden=True)
        err = (mine - ref_logits).abs().max().item()
        herr = max((a - b).abs().max().item() for a, b in zip(my_hidden, hiddens))
        cerr = (chunked - ref_logits).abs().max().item()
        print(f"tiny {name}: plain vs reference logits {err:.2e}, hidden states {herr:.2e}; "
              f"reference chunked vs dense {cerr:.2e}")
        assert err < 1e-5 and herr < 1e-5
        greedy = None
        if cfg.get("tie_word_embeddings"):
            greedy = generate_greedy(model, ids[:9], 8)
            assert greedy == plain.greedy(cfg, w, ids[:9], 8), (greedy, plain.greedy(cfg, w, ids[:9], 8))
        fp = {k: float(v.double().abs().sum()) for k, v in w.items()
              if k in ("model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.bias",
                       f"model.layers.{cfg['num_hidden_layers'] - 1}.mlp.down_proj.weight")}
        np.savez_compressed(
            os.path.join(HERE, f"tiny_{name}.npz"), ids=np.array(ids), logits=ref_logits.numpy(),
            hidden=np.stack([h.numpy() for h in hiddens]), greedy=np.array(greedy if greedy else []),
            fingerprint_names=np.array(sorted(fp)), fingerprint=np.array([fp[k] for k in sorted(fp)]))


if __name__ == "__main__":
    main()
