"""The plain implementation against the reference's own model code (stored outputs), and
against itself where two of its functions must agree."""
import hashlib
import os

import numpy as np
import pytest
import torch

import plain_gpt2 as P
from tiny import write_tiny

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_the_reference_model(tmp_path, name):
    """tests/golden/tiny_*.npz hold logits of rosellm.rosetrainer.model.GPTModel on the CPU
    (made by tests/golden/make_golden.py) for the same random-weight folders."""
    gold = np.load(os.path.join(GOLDEN, f"tiny_{name}.npz"))
    folder = write_tiny(name, str(tmp_path))
    cfg, t32 = P.load_folder(folder, torch.float32)
    h = hashlib.sha256()
    for k in sorted(t32):
        h.update(k.encode())
        h.update(t32[k].numpy().tobytes())
    assert h.hexdigest() == str(gold["weights_sha256"]), "the random-weights mode no longer writes the stored model"
    cfg, t = P.load_folder(folder)
    mine = P.forward(cfg, t, gold["ids"]).numpy()
    assert np.abs(mine - gold["logits"]).max() < 5e-6


def test_causality_and_window():
    torch.manual_seed(0)
    T, D, H = 12, 32, 2
    h = torch.randn(T, D, dtype=torch.float64)
    w = [torch.randn(D, 3 * D, dtype=torch.float64) * 0.2, torch.randn(3 * D, dtype=torch.float64),
         torch.randn(D, D, dtype=torch.float64) * 0.2, torch.randn(D, dtype=torch.float64)]
    full = P.attention(h, *w, H)
    h2 = h.clone()
    h2[8:] += 1.0
    assert torch.allclose(P.attention(h2, *w, H)[:8], full[:8])  # later tokens change nothing earlier
    win = P.attention(h, *w, H, window=3)
    assert torch.allclose(win[:3], full[:3]) and not torch.allclose(win[5:], full[5:])
    h3 = h.clone()
    h3[0] += 5.0
    assert torch.allclose(P.attention(h3, *w, H, window=3)[3:], win[3:])  # out of the window: unseen


def test_gelu_forms():
    u = torch.linspace(-4, 4, 101, dtype=torch.float64)
    assert torch.allclose(P.gelu_erf(u), torch.nn.functional.gelu(u))
    assert torch.allclose(P.gelu_tanh(u), torch.nn.functional.gelu(u, approximate="tanh"))
    assert (P.gelu_tanh(u) - P.gelu_erf(u)).abs().max() > 1e-4


def test_filters_follow_the_reference_rules():
    x = torch.tensor([2.0, 1.0, 0.0, -1.0, 3.0])
    assert torch.isinf(P.top_k_filter(x, 2)).tolist() == [False, True, True, True, False]
    assert P.top_k_filter(x, 0) is x and P.top_k_filter(x, 9) is x
    p = torch.softmax(x, -1)  # sorted: 3, 2, 1, 0, -1 -> cumulative .636, .870, .956, ...
    assert torch.isinf(P.top_p_filter(x, 0.9)).tolist() == [False, True, True, True, False]
    assert torch.isinf(P.top_p_filter(x, 0.5)).tolist() == [True, True, True, True, False]  # the first stays
    assert P.top_p_filter(x, 1.0) is x
    assert float(p[4] + p[0]) < 0.9 < float(p[4] + p[0] + p[1])


def test_gumbel_draw_is_a_function_of_seed_counter_and_index():
    a = P.gumbel_noise(5, 2, 50)
    assert np.array_equal(a, P.gumbel_noise(5, 2, 50)) and np.array_equal(a[:20], P.gumbel_noise(5, 2, 20))
    assert not np.array_equal(a, P.gumbel_noise(5, 3, 50)) and not np.array_equal(a, P.gumbel_noise(6, 2, 50))
    logits = torch.tensor([1.0, 0.0, -1.0, 2.0])
    counts = np.zeros(4)
    for c in range(4000):
        counts[P.gumbel_sample(logits, 1.0, 0, 1.0, 9, c)[0]] += 1
    assert np.abs(counts / 4000 - torch.softmax(logits, -1).numpy()).max() < 0.03
