"""Trace replay through the engine's own step function, cache and kernels, in 32-bit and in
bfloat16, compared with the plain implementation: whole requests; the last 32 tokens one by
one; portions of changing size; mixed batches with so few pages that they are used again."""
import os

import numpy as np
import pytest

import replay_util as R
from tiny import TINY, write_tiny

pytestmark = pytest.mark.gpu

# Largest |logit difference| allowed.  float32: the bound the project states for the 32-bit
# path.  bfloat16: activations between products and the cache carry 8 bits of mantissa.  How
# much that alone moves the logits depends on the model (the "sharp" models, with weights ten
# times larger, have attention scores in the tens and are far more sensitive), so the
# bfloat16 bound is tied to it: three times the change that rounding the plain
# implementation's activations to bfloat16 at the same places causes on the same tokens
# (the engine also rounds partial results inside attention and orders sums differently),
# and never below 2e-2.
ATOL = {"float32": 1e-4, "bfloat16": 2e-2}
NOISE_FACTOR = {"float32": None, "bfloat16": 3.0}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("models"))
    return {name: write_tiny(name, root) for name in TINY}


def requests_for(name: str, lens, seed: int) -> dict[str, list[int]]:
    vocab = TINY[name]["config"].vocab_size
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, vocab, size=n).tolist() for i, n in enumerate(lens)}


LENS = {"A": [5, 17, 32, 100, 128], "B": [1, 40, 97, 150, 256], "A_sharp": [48, 128, 33], "B_sharp": [150, 256, 64],
        "C_sharp": [192, 65, 130]}


def atol_for(name, dtype):
    return ATOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_whole_requests(folders, tmp_path, name, dtype):
    reqs = requests_for(name, LENS[name], 1)
    tr = R.whole(reqs)
    got = R.replay(folders[name], dtype, tr, str(tmp_path), page_size=TINY[name]["page_size"])
    R.check(folders[name], reqs, tr, got, atol_for(name, dtype), NOISE_FACTOR[dtype])


@pytest.mark.parametrize("graphs", [False, True], ids=["walked", "graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_last_32_tokens_one_by_one(folders, tmp_path, name, dtype, graphs):
    """With ``graphs`` the single-token steps are replays of a CUDA graph captured for their
    batch-size bucket (padding rows, a workspace of its own, a decode plan fixed at capture):
    the path generation takes."""
    reqs = requests_for(name, LENS[name], 2)
    tr = R.tail_decoded(reqs)
    stats = {}
    got = R.replay(folders[name], dtype, tr, str(tmp_path), page_size=TINY[name]["page_size"], cuda_graphs=graphs,
                   stats=stats)
    R.check(folders[name], reqs, tr, got, atol_for(name, dtype), NOISE_FACTOR[dtype])
    single = sum(1 for s in tr.steps if s["entries"] and all(len(e["tokens"]) == 1 for e in s["entries"]))
    assert stats["graph_replays"] == (single if graphs else 0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_portions_of_changing_size(folders, tmp_path, name, dtype):
    reqs = requests_for(name, LENS[name], 3)
    tr = R.portions(reqs)
    got = R.replay(folders[name], dtype, tr, str(tmp_path), page_size=TINY[name]["page_size"])
    R.check(folders[name], reqs, tr, got, atol_for(name, dtype), NOISE_FACTOR[dtype])


@pytest.mark.parametrize("graphs", [False, True], ids=["walked", "graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_mixed_with_reused_pages(folders, tmp_path, name, dtype, graphs):
    """With ``graphs`` the steps in which every live request brings one token are graph replays
    (three live requests in the bucket of four, with a padding row), between walked steps that
    mix portions and single tokens over the same pages."""
    npos = TINY[name]["config"].n_positions
    lens = [npos // 2, 9, npos, 33, npos // 3, 2, npos - 7, 64, 20, npos // 2 + 1]
    reqs = requests_for(name, lens, 4)
    prompt_lens = {rid: max(1, len(t) - (8 if i % 2 else 40)) for i, (rid, t) in enumerate(reqs.items())}
    tr = R.mixed(reqs, prompt_lens, max_live=4, seed=5)
    peak = R.peak_tokens(tr)
    assert sum(-(-len(t) // 64) * 64 for t in reqs.values()) > 1.5 * peak  # pages must come round again
    stats = {}
    got = R.replay(folders[name], dtype, tr, str(tmp_path), max_tokens=peak, page_size=TINY[name]["page_size"],
                   cuda_graphs=graphs, stats=stats)
    R.check(folders[name], reqs, tr, got, atol_for(name, dtype), NOISE_FACTOR[dtype])
    if graphs:
        assert 0 < stats["graph_replays"] < stats["steps"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_as_a_program(folders, tmp_path, dtype):
    """bin/trace_run itself, as a child process reading its steps from standard input."""
    reqs = requests_for("B", [40, 150, 3], 6)
    tr = R.mixed(reqs, {rid: len(t) - 5 for rid, t in reqs.items()}, max_live=2, seed=1)
    got = R.replay(folders["B"], dtype, tr, str(tmp_path), subprocess_mode=True, page_size=8)
    R.check(folders["B"], reqs, tr, got, ATOL[dtype], NOISE_FACTOR[dtype])


@pytest.mark.parametrize("graphs", [False, True], ids=["walked", "graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A_sharp", "B_sharp"])
def test_long_decoding(folders, tmp_path, name, dtype, graphs):
    """Three prompt tokens, then every further token up to the model's limit one by one."""
    npos = TINY[name]["config"].n_positions
    reqs = requests_for(name, [npos], 8)
    tr = R.tail_decoded(reqs, tail=npos - 3)
    got = R.replay(folders[name], dtype, tr, str(tmp_path), page_size=TINY[name]["page_size"], cuda_graphs=graphs)
    R.check(folders[name], reqs, tr, got, atol_for(name, dtype), NOISE_FACTOR[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A_sharp", "B_sharp"])
def test_first_tokens_of_a_sequence(folders, tmp_path, name, dtype):
    """Sequences of one to four tokens: whole, and token by token from the very first."""
    reqs = requests_for(name, [1, 2, 3, 4], 9)
    for tr in (R.whole(reqs), R.tail_decoded(reqs, tail=10), R.portions(reqs, sizes=(2, 1))):
        got = R.replay(folders[name], dtype, tr, str(tmp_path / str(id(tr))), page_size=TINY[name]["page_size"])
        R.check(folders[name], reqs, tr, got, atol_for(name, dtype), NOISE_FACTOR[dtype])
