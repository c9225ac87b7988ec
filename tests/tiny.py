"""The tiny configurations the tests use, and helpers to write them as model folders.

A and B differ in every size and option: layers, width, heads and head size,
inner width (B's is not four times the width), vocabulary, positions, the
norms' epsilon, the activation, whether norm scales and biases are trivial,
and the cache page size the tests pair them with.
"""
from __future__ import annotations

import os

from rosellm_b200.config import GPT2Config
from rosellm_b200.weights import write_model_folder

TINY_A = dict(
    config=GPT2Config(n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512, n_positions=128,
                      layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    seed=0, norm_affine="identity", page_size=16, std=0.02,
)
TINY_B = dict(
    config=GPT2Config(n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000, n_positions=256,
                      layer_norm_epsilon=1e-6, activation_function="gelu"),
    seed=1, norm_affine="random", page_size=8, std=0.02,
)
# Weights ten times larger make attention far from uniform, so that a wrong or missing key
# changes the logits by much more than the tolerance.
TINY_A_SHARP = dict(TINY_A, seed=2, std=0.2)
TINY_B_SHARP = dict(TINY_B, seed=3, std=0.2)

# One layer, heads of 16, an inner width that is no multiple of 8 (the feed-forward fills it up
# with idle units), an odd vocabulary, pages of 64.
TINY_C_SHARP = dict(
    config=GPT2Config(n_layer=1, n_embd=48, n_head=3, n_inner=100, vocab_size=777, n_positions=192,
                      layer_norm_epsilon=1e-4, activation_function="gelu_new"),
    seed=4, norm_affine="random", page_size=64, std=0.2,
)

TINY = {"A": TINY_A, "B": TINY_B, "A_sharp": TINY_A_SHARP, "B_sharp": TINY_B_SHARP, "C_sharp": TINY_C_SHARP}


def write_tiny(name: str, root: str) -> str:
    t = TINY[name]
    out = os.path.join(root, f"tiny_{name}")
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        write_model_folder(t["config"], t["seed"], out, std=t["std"], norm_affine=t["norm_affine"])
    return out
