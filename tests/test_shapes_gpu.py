"""The published GPT-2 widths (124M, 355M, 1.5B: head size 64 with 12, 16 and 25 heads, the
full vocabulary of 50,257) with two layers of random weights: 32-bit logits against the plain
implementation under every way of cutting the work, bfloat16 within its rounding noise."""
import numpy as np
import pytest

import replay_util as R
from rosellm_b200.config import GPT2Config
from rosellm_b200.weights import write_model_folder

pytestmark = pytest.mark.gpu

SHAPES = {
    "124M": dict(n_embd=768, n_head=12, n_inner=3072),
    "355M": dict(n_embd=1024, n_head=16, n_inner=4096),
    "1.5B": dict(n_embd=1600, n_head=25, n_inner=6400),
}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("shapes")
    out = {}
    for name, sizes in SHAPES.items():
        cfg = GPT2Config(n_layer=2, vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5,
                         activation_function="gelu_new", **sizes)
        out[name] = write_model_folder(cfg, 7, str(root / name), std=0.02)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SHAPES))
def test_published_widths_in_all_cutting_modes(folders, tmp_path, name, dtype):
    rng = np.random.default_rng(11)
    reqs = {f"r{i}": rng.integers(0, 50257, n).tolist() for i, n in enumerate([70, 33, 5])}
    last = {rid: [len(t) - 1] for rid, t in reqs.items()}
    # whole prompts (logits of three places each), the tail token by token, portions, and mixed
    whole = R.Trace()
    for rid, toks in reqs.items():
        whole.add([(rid, toks, [0, len(toks) // 2, len(toks) - 1])], end=[rid])
    traces = {
        "whole": whole,
        "tail": R.tail_decoded(reqs, tail=6),
        "portions": R.portions({k: v for k, v in list(reqs.items())[:2]}, sizes=(17, 2, 40, 3)),
        "mixed": R.mixed(reqs, {rid: len(t) - 4 for rid, t in reqs.items()}, max_live=3, sizes=(16, 2, 30), seed=2),
    }
    atol = 1e-4 if dtype == "float32" else 2e-2
    factor = None if dtype == "float32" else 3.0
    for label, tr in traces.items():
        got = R.replay(folders[name], dtype, tr, str(tmp_path / label), page_size=16)
        R.check(folders[name], reqs, tr, got, atol, factor)


def test_long_prompts_take_the_tcgen05_attention(folders, tmp_path):
    """Contexts of 512 tokens and more at head size 64 run the prompt attention on tcgen05: a
    prompt whole, the same prompt in portions that end inside its tiles of 128, and a prompt
    beside a decoded token of another request, against the plain implementation."""
    from rosellm_b200.parts.standard import TC_ATTENTION_MIN_CONTEXT

    rng = np.random.default_rng(5)
    reqs = {"long": rng.integers(0, 50257, 700).tolist(), "other": rng.integers(0, 50257, 530).tolist()}
    assert min(len(t) for t in reqs.values()) >= TC_ATTENTION_MIN_CONTEXT
    whole = R.Trace()
    whole.add([("long", reqs["long"], [0, 127, 128, 511, 699])], end=["long"])
    cut = R.Trace()
    cut.add([("long", reqs["long"][:300], [299]), ("other", reqs["other"][:529], [])])
    cut.add([("long", reqs["long"][300:645], [0, 344]), ("other", reqs["other"][529:], [0])], end=["other"])
    cut.add([("long", reqs["long"][645:], [54])], end=["long"])
    for label, tr in (("whole", whole), ("cut", cut)):
        got = R.replay(folders["124M"], "bfloat16", tr, str(tmp_path / label), page_size=16)
        R.check(folders["124M"], reqs, tr, got, 2e-2, 3.0)
