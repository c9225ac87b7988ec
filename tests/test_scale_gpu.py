"""The compositions that the benchmarks time, row by row against the plain implementation.

GPT-2 124M with all of its twelve layers, and the width of the 1.5B model (25 heads, two
layers), with the full vocabulary: 8 and 64 requests are prefilled to the benchmarks' context
lengths through ``ModelRunner.step`` and then decoded for a few steps that are replays of the
CUDA graph of their batch-size bucket (blocks of sixteen warps at 8 requests, of four warps at
64; products of 8 and 64 rows; the decode plan fixed when the graph was captured); and a whole
prompt of 1,024 tokens.  The plain implementation runs in float64 on the same GPU.
"""
import numpy as np
import pytest
import torch

import plain_gpt2 as P
from rosellm_b200.config import EngineConfig, GPT2Config
from rosellm_b200.engine.runner import ModelRunner, StepEntry
from rosellm_b200.weights import write_model_folder

pytestmark = pytest.mark.gpu

MODELS = {
    "124M": dict(n_layer=12, n_embd=768, n_head=12, n_inner=3072),
    "1.5B-width": dict(n_layer=2, n_embd=1600, n_head=25, n_inner=6400),
}
VOCAB = 50257


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("scale")
    out = {}
    for name, sizes in MODELS.items():
        cfg = GPT2Config(vocab_size=VOCAB, n_positions=1024, layer_norm_epsilon=1e-5,
                         activation_function="gelu_new", **sizes)
        folder = write_model_folder(cfg, 21, str(root / name), std=0.02)
        out[name] = (folder, P.load_folder(folder, device="cuda"))
    yield out
    out.clear()
    torch.cuda.empty_cache()


def plain_rows(plain, toks, rows, rounding=None):
    cfg, t = plain
    if rounding is None:
        return P.forward(cfg, t, toks, rows=rows)
    return P.forward(cfg, t, toks, rounding=rounding, rows=rows)


def compare(plain, dtype, toks, rows, got, what):
    """``got`` [len(rows), vocab] against the plain logits of ``toks`` at ``rows``: 1e-4 in
    32-bit; in bfloat16 three times what rounding the plain implementation's activations to
    bfloat16 moves these rows, and at least 2e-2."""
    ref = plain_rows(plain, toks, rows)
    diff = float((got.double() - ref).abs().max())
    limit = 1e-4
    if dtype == "bfloat16":
        noise = float((plain_rows(plain, toks, rows, P.to_bfloat16_and_back) - ref).abs().max())
        limit = max(2e-2, 3.0 * noise)
    assert np.isfinite(diff) and diff <= limit, f"{what}: |logits - plain| = {diff:.3e} > {limit:.1e}"
    return diff


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,batch,context", [("124M", 8, 512), ("124M", 64, 512),
                                                ("1.5B-width", 8, 896), ("1.5B-width", 64, 896)])
def test_graph_replayed_decode_at_benchmark_sizes(models, name, batch, context, dtype):
    folder, plain = models[name]
    steps = 3
    runner = ModelRunner.from_folder(folder, EngineConfig(
        dtype=dtype, page_size=16, kv_cache_tokens=batch * (context + 16), max_num_seqs=batch,
        max_num_batched_tokens=2048, cuda_graphs=True, capture_graphs_at_start=False))
    rng = np.random.default_rng(batch + context)
    seqs = rng.integers(0, VOCAB, size=(batch, context + steps + 1)).tolist()
    slots = [runner.cache.new_request() for _ in range(batch)]
    # prompts in portions of 512 tokens, as many requests a step as the token budget takes;
    # the logits of each prompt's last token are checked for the first request of every step
    at = [0] * batch
    first_rows = {}
    while min(at) < context:
        entries, budget = [], 2048
        for r in range(batch):
            n = min(512, context - at[r], budget)
            if n <= 0:
                continue
            last = at[r] + n == context
            entries.append((r, StepEntry(slots[r], seqs[r][at[r]:at[r] + n], [n - 1] if last else [])))
            at[r] += n
            budget -= n
        logits = runner.step([e for _, e in entries])
        row = 0
        for r, e in entries:
            if e.want:
                if not first_rows or r % 16 == 5:
                    first_rows[r] = logits[row].clone()
                row += 1
    for r, got in first_rows.items():
        compare(plain, dtype, seqs[r][:context], [context - 1], got[None], f"prompt of request {r}")
    before = runner.graph_replays
    got = []
    for s in range(steps):
        logits = runner.step([StepEntry(slots[r], [seqs[r][context + s]], [0]) for r in range(batch)])
        got.append(logits.clone())
    runner.check_status()
    assert runner.graph_replays - before == steps
    rows = list(range(context, context + steps))
    worst = 0.0
    for r in range(batch):
        mine = torch.stack([g[r] for g in got])
        worst = max(worst, compare(plain, dtype, seqs[r], rows, mine, f"request {r} of {batch}, decoded rows"))
    print(f"{name} batch {batch} context {context} {dtype}: worst difference {worst:.2e}")
    if not runner.samples_in_head(batch):
        return
    # one more step, through the graph whose head chooses the tokens itself (the weight-streaming
    # product at 8 rows, tcgen05 tiles at 64): each token is the plain arg-max, or as near to it
    # as two logits may be apart
    from rosellm_b200.ops import kernels as K

    tokens = torch.full((batch,), -1, dtype=torch.int32, device=runner.device)
    none = runner.step([StepEntry(slots[r], [seqs[r][context + steps]], [0]) for r in range(batch)],
                       sample_into=K.SampleInto(tokens))
    runner.check_status()
    assert none is None and runner.graph_replays - before == steps + 1
    tokens = tokens.cpu().tolist()
    for r in range(0, batch, 8):
        ref = plain_rows(plain, seqs[r], [context + steps])[0]
        noise = float((plain_rows(plain, seqs[r], [context + steps], P.to_bfloat16_and_back)[0] - ref).abs().max())
        gap = float(ref.max() - ref[tokens[r]])
        assert 0 <= tokens[r] < VOCAB and gap <= 2 * max(2e-2, 3.0 * noise), \
            f"request {r}: token {tokens[r]} lies {gap:.3e} under the plain maximum"


@pytest.mark.parametrize("name", list(MODELS))
def test_a_whole_prompt_of_1024_tokens_in_32_bit(models, name):
    folder, plain = models[name]
    runner = ModelRunner.from_folder(folder, EngineConfig(
        dtype="float32", page_size=16, kv_cache_tokens=1024, max_num_seqs=2, max_num_batched_tokens=1024,
        cuda_graphs=False))
    toks = np.random.default_rng(3).integers(0, VOCAB, size=1024).tolist()
    rows = [0, 1, 63, 64, 511, 777, 1022, 1023]
    slot = runner.cache.new_request()
    logits = runner.step([StepEntry(slot, toks, rows)])
    runner.check_status()
    compare(plain, "float32", toks, rows, logits, f"{name}, 1,024 tokens whole")
