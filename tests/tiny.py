"""The tiny configurations of the test-suite.  They differ in every size and option: layers, width,
heads and groups, head size, feed-forward width, vocabulary, rope base, norm eps, tied or separate
head, window, cache page size and seed."""

from __future__ import annotations

import os

import numpy as np

from turingserve_b200.models.qwen2 import make_config
from turingserve_b200.weights.random_init import write_random_model

# name -> (config arguments, seed, cache page size, weight std)
TINY = {
    # BASELINE "Tiny Qwen2 A"
    "A": (dict(hidden_size=64, intermediate_size=128, num_layers=2, num_heads=4, num_kv_heads=2,
               vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
               max_position_embeddings=128), 0, 16, 0.02),
    # BASELINE "Tiny Qwen2 B"
    "B": (dict(hidden_size=96, intermediate_size=224, num_layers=3, num_heads=3, num_kv_heads=1,
               vocab_size=320, rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False,
               max_position_embeddings=256), 1, 8, 0.02),
    # a third one with a window on its later layers, sizes that are no power of two, larger weights
    "W": (dict(hidden_size=80, intermediate_size=176, num_layers=3, num_heads=5, num_kv_heads=5,
               head_dim=48, vocab_size=301, rope_theta=50000.0, rms_norm_eps=3e-6,
               tie_word_embeddings=False, max_position_embeddings=512, sliding_window=24,
               max_window_layers=1), 2, 16, 0.08),
    # two with the head sizes and pages the tensor-core and TMA attention kernels take (the three
    # above go to the any-size kernel): 128 with groups of two, 64 with groups of three and a window
    "K": (dict(hidden_size=192, intermediate_size=320, num_layers=2, num_heads=4, num_kv_heads=2,
               head_dim=128, vocab_size=300, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True,
               max_position_embeddings=512), 3, 16, 0.03),
    "L": (dict(hidden_size=160, intermediate_size=272, num_layers=3, num_heads=9, num_kv_heads=3,
               head_dim=64, vocab_size=333, rope_theta=20000.0, rms_norm_eps=2e-6, tie_word_embeddings=False,
               max_position_embeddings=512, sliding_window=70, max_window_layers=1), 4, 32, 0.03),
    # sizes in steps of 16 that nothing else has: heads of 80, a width, a feed-forward width and a
    # vocabulary that are odd multiples, more key/value heads than groups
    "X": (dict(hidden_size=208, intermediate_size=136, num_layers=2, num_heads=6, num_kv_heads=3,
               head_dim=80, vocab_size=1001, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
               max_position_embeddings=256), 5, 32, 0.04),
}


def tiny_config(name: str):
    return make_config(**TINY[name][0])


def make_tiny_folder(name: str, base: str, std: float | None = None) -> str:
    kw, seed, _, default_std = TINY[name]
    folder = os.path.join(str(base), f"tiny_{name}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        write_random_model(folder, make_config(**kw), seed, std=default_std if std is None else std)
    return folder


def page_size(name: str) -> int:
    return TINY[name][2]


def random_ids(n: int, vocab: int, seed: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
