"""Generation through the Python entry point against the plain implementation."""
import numpy as np
import pytest
import torch

import plain_gpt2 as P
from tiny import TINY, write_tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("models"))
    return {name: write_tiny(name, root) for name in TINY}


def engine(folder, dtype, **kw):
    from rosellm_b200.engine.llm import InferenceEngine

    return InferenceEngine(folder, dtype=dtype, **kw)


def greedy_tolerance(cfg, t, ids, ref, dtype) -> float:
    """How far below the plain maximum the plain logit of a chosen token may lie: twice the
    error allowed on a logit (the chosen and the largest may both be off), which is 1e-4 in
    32-bit and, in bfloat16, three times what rounding the plain implementation's activations
    to bfloat16 moves the logits of these very tokens (at least 2e-2), as in the replay tests."""
    if dtype == "float32":
        return 2e-4
    noise = float((P.forward(cfg, t, ids, rounding=P.to_bfloat16_and_back)[-1] - ref).abs().max())
    return 2 * max(2e-2, 3.0 * noise)


def check_greedy(folder, prompt, out, dtype):
    """Every generated token is, given the tokens before it, the plain arg-max or within the
    precision's tolerance of it."""
    cfg, t = P.load_folder(folder)
    ids = list(prompt)
    for i, tok in enumerate(out):
        ref = P.forward(cfg, t, ids)[-1]
        gap = float(ref.max() - ref[tok])
        if gap > 0:
            tol = greedy_tolerance(cfg, t, ids, ref, dtype)
            assert gap <= tol, f"token {i} of {out}: plain logit is {gap:.3e} below the plain maximum (allowed {tol:.1e})"
        ids.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_config_a(folders, dtype):
    """Three prompts of 5, 17 and 32 ids, 16 greedy tokens each, pages of 16."""
    name = "A_sharp"
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 512, n).tolist() for n in (5, 17, 32)]
    eng = engine(folders[name], dtype, page_size=16, max_batch_size=4, kv_cache_max_tokens=512)
    outs = eng.generate_batch(prompts, max_new_tokens=16, stop_on_eos=False)
    assert [len(o) for o in outs] == [16, 16, 16]
    for p, o in zip(prompts, outs):
        check_greedy(folders[name], p, o, dtype)
    if dtype == "float32":
        cfg, t = P.load_folder(folders[name])
        assert outs[0] == P.greedy(cfg, t, prompts[0], 16)
    assert eng.runner.cache.num_free_pages == eng.runner.cache.num_pages  # everything was given back


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sampled_generation_config_b(folders, dtype):
    """Prompts of 1, 40, 97 and 150 ids, portions of 16 beside decoding, 24 tokens at
    temperature 0.8 from seeded requests, pages of 8."""
    name = "B_sharp"
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 1000, n).tolist() for n in (1, 40, 97, 150)]
    eng = engine(folders[name], dtype, page_size=8, max_batch_size=4, prefill_chunk_size=16,
                 max_num_batched_tokens=40, kv_cache_max_tokens=1024)
    rids = [eng.add_request(prompt_token_ids=p, max_new_tokens=24, temperature=0.8, do_sample=True,
                            stop_on_eos=False, seed=100 + i) for i, p in enumerate(prompts)]
    while eng.has_unfinished():
        eng.step()
    outs = [eng.pop_response(r) for r in rids]
    cfg, t = P.load_folder(folders[name])
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert len(o.token_ids) == 24 and o.finish_reason == "length"
        ids = list(p)
        for c, tok in enumerate(o.token_ids):
            ref = P.forward(cfg, t, ids)[-1]
            _, scores = P.gumbel_sample(ref, 0.8, 0, 1.0, 100 + i, c)
            gap = scores.max() - scores[tok]
            if gap > 0:
                assert gap <= greedy_tolerance(cfg, t, ids, ref, dtype) / 0.8 + 1e-3, f"request {i} token {c}"
            ids.append(tok)


def test_a_request_samples_the_same_alone_and_in_company(folders):
    name = "B_sharp"
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, 1000, n).tolist() for n in (30, 7, 64, 19)]
    kw = dict(max_new_tokens=12, temperature=0.9, do_sample=True, top_k=50, top_p=0.9, stop_on_eos=False)
    eng = engine(folders[name], "float32", page_size=8, max_batch_size=4, prefill_chunk_size=16, kv_cache_max_tokens=1024)
    alone = []
    for i, p in enumerate(prompts):
        rid = eng.add_request(prompt_token_ids=p, seed=7 + i, **kw)
        while eng.has_unfinished():
            eng.step()
        alone.append(eng.pop_response(rid).token_ids)
    rids = [eng.add_request(prompt_token_ids=p, seed=7 + i, **kw) for i, p in enumerate(prompts)]
    while eng.has_unfinished():
        eng.step()
    together = [eng.pop_response(r).token_ids for r in rids]
    assert together == alone
    rid = eng.add_request(prompt_token_ids=prompts[0], seed=999, **kw)
    while eng.has_unfinished():
        eng.step()
    assert eng.pop_response(rid).token_ids != alone[0]  # another seed, another continuation


def test_preemption_changes_no_token(folders):
    """With pages for barely more than one request, requests are preempted and recomputed;
    greedy tokens equal those of a roomy cache."""
    name = "A_sharp"
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, 512, n).tolist() for n in (20, 25, 18, 30)]
    roomy = engine(folders[name], "float32", page_size=4, max_batch_size=4, kv_cache_max_tokens=1024)
    want = roomy.generate_batch(prompts, max_new_tokens=40, stop_on_eos=False)
    tight = engine(folders[name], "float32", page_size=4, max_batch_size=4, kv_cache_max_tokens=120)
    got = tight.generate_batch(prompts, max_new_tokens=40, stop_on_eos=False)
    assert tight.num_preemptions > 0 and roomy.num_preemptions == 0
    assert got == want
    assert tight.runner.cache.num_free_pages == tight.runner.cache.num_pages
    tight.runner.cache.check()


def test_stream_and_stop_on_eos(folders):
    name = "A_sharp"
    eng = engine(folders[name], "float32", max_batch_size=2, kv_cache_max_tokens=256)
    prompt = [1, 2, 3, 4]
    full = eng.generate(prompt, max_new_tokens=10, stop_on_eos=False)
    assert list(eng.stream_generate(prompt, max_new_tokens=10, stop_on_eos=False)) == full
    eng.scheduler.eos_token_id = full[3]
    rid = eng.add_request(prompt_token_ids=prompt, max_new_tokens=10)
    while eng.has_unfinished():
        eng.step()
    out = eng.pop_response(rid)
    assert out.token_ids == full[: full.index(full[3]) + 1] and out.finish_reason == "stop"
    with pytest.raises(ValueError, match="tokenizer"):
        eng.generate("text prompt")


def test_llm_entry_point(folders):
    from rosellm_b200 import LLM, SamplingParams

    llm = LLM(folders["A_sharp"], dtype="float32", max_batch_size=4, kv_cache_max_tokens=512)
    outs = llm.generate([[1, 2, 3], [9, 8, 7, 6, 5]], SamplingParams(max_new_tokens=5, stop_on_eos=False))
    assert [len(o.token_ids) for o in outs] == [5, 5] and outs[0].prompt_token_ids == [1, 2, 3]
    check_greedy(folders["A_sharp"], [1, 2, 3], outs[0].token_ids, "float32")


def test_no_cpu_path():
    from rosellm_b200.config import EngineConfig
    from rosellm_b200.engine.runner import ModelRunner

    with pytest.raises(RuntimeError, match="CUDA device only"):
        ModelRunner(TINY["A"]["config"], {}, EngineConfig(device="cpu"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlapped_scheduling_changes_no_token(folders, dtype):
    """Launching a step before the host has read the previous step's tokens (they are fed from
    device memory) gives the same tokens as reading them first: sampled and greedy requests, a
    prompt fed in portions, an early stop on the end-of-sequence token, and a cache so small
    that requests are preempted."""
    name = "B_sharp"
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, 1000, n).tolist() for n in (30, 7, 64, 19, 3)]

    def run(overlap, kv_tokens, eos=None):
        eng = engine(folders[name], dtype, page_size=8, max_batch_size=4, prefill_chunk_size=16,
                     max_num_batched_tokens=48, kv_cache_max_tokens=kv_tokens, overlap_schedule=overlap)
        eng.scheduler.eos_token_id = eos
        rids = [eng.add_request(prompt_token_ids=p, max_new_tokens=20 + i, temperature=0.9, do_sample=i % 2 == 0,
                                top_k=40 if i == 2 else 0, seed=50 + i) for i, p in enumerate(prompts)]
        seen = {r: [] for r in rids}
        while eng.has_unfinished():
            for rid, tok in eng.step().items():
                seen[rid].append(tok)
        outs = [eng.pop_response(r) for r in rids]
        for r, o in zip(rids, outs):
            assert seen[r] == o.token_ids  # step() reported every token once, in order
        assert eng.runner.cache.num_free_pages == eng.runner.cache.num_pages
        return [(o.token_ids, o.finish_reason) for o in outs], eng.num_preemptions

    base, _ = run(False, 1024)
    eos = base[1][0][5]  # a token the second request generates: it must stop there
    for kv_tokens in (1024, 160):
        want, p0 = run(False, kv_tokens, eos)
        got, p1 = run(True, kv_tokens, eos)
        assert got == want
        assert want[1][1] == "stop" and len(want[1][0]) <= 6
        if kv_tokens == 160:
            assert p0 > 0 and p1 > 0


def test_graphs_are_captured_when_the_engine_is_built(folders):
    """Every batch-size bucket has its decode graph before the first request (captured on
    padding rows), generation through them equals generation without graphs, and a new
    feedback buffer drops them (they hold the old one's address)."""
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, TINY["A"]["config"].vocab_size, n).tolist() for n in (9, 33, 2)]
    eng = engine(folders["A"], "bfloat16", max_batch_size=8)
    # the head of these graphs chooses the tokens itself, into the sampler's buffers
    assert sorted(eng.runner._graphs) == [(b, id(eng.sampler.target)) for b in (1, 2, 4, 8)]
    logits_only = engine(folders["A"], "bfloat16", max_batch_size=8, sample_in_head=False)
    assert sorted(logits_only.runner._graphs) == [1, 2, 4, 8]
    lazy = engine(folders["A"], "bfloat16", max_batch_size=8, capture_graphs_at_start=False)
    assert not lazy.runner._graphs
    plain = engine(folders["A"], "bfloat16", max_batch_size=8, cuda_graphs=False)
    want = plain.generate_batch(prompts, max_new_tokens=12)
    assert eng.generate_batch(prompts, max_new_tokens=12) == want
    assert lazy.generate_batch(prompts, max_new_tokens=12) == want and lazy.runner._graphs
    eng.runner.token_feedback = torch.zeros(8, dtype=torch.int32, device=eng.device)
    assert not eng.runner._graphs


@pytest.mark.parametrize("graphs", [True, False])
def test_tokens_chosen_by_the_head_are_those_sampled_from_logits(folders, graphs):
    """Steps of few rows without top-k or top-p get their tokens from the head's own product
    (no logits written); the same requests through an engine that writes logits and samples
    from them give the same tokens: greedy and temperature rows side by side, prompts that end
    in different steps, a request with top-k joining later (its steps fall back to logits)."""
    rng = np.random.default_rng(5)
    vocab = TINY["A"]["config"].vocab_size
    prompts = [rng.integers(0, vocab, n).tolist() for n in (3, 21, 40, 9, 2)]

    def run(sample_in_head):
        eng = engine(folders["A"], "bfloat16", max_batch_size=8, prefill_chunk_size=16, max_num_batched_tokens=24,
                     cuda_graphs=graphs, sample_in_head=sample_in_head)
        rids = [eng.add_request(prompt_token_ids=p, max_new_tokens=14 + i, temperature=0.7 + 0.1 * i,
                                do_sample=i % 2 == 1, stop_on_eos=False, seed=100 + i) for i, p in enumerate(prompts)]
        steps = 0
        while eng.has_unfinished():
            eng.step()
            steps += 1
            if steps == 6:
                rids.append(eng.add_request(prompt_token_ids=prompts[0], max_new_tokens=5, temperature=0.9, top_k=7,
                                            do_sample=True, stop_on_eos=False, seed=3))
        return [eng.pop_response(r).token_ids for r in rids], eng

    want, plain = run(False)
    got, eng = run(True)
    assert got == want
    assert [len(o) for o in got] == [14, 15, 16, 17, 18, 5]
    if graphs:
        assert any(isinstance(k, tuple) for k in eng.runner._graphs)      # graphs whose head samples
        assert all(not isinstance(k, tuple) for k in plain.runner._graphs)


@pytest.mark.parametrize("name", ["A_sharp", "B_sharp"])
def test_forty_requests_at_once_decode_as_each_alone(folders, name):
    """Batch sizes beyond the few requests of the replay tests take other kernels (products of 17
    to 64 rows, decode attention in blocks of four warps without a split, graph buckets up to
    64): forty requests generated together give the tokens each of them gives alone (32-bit, so
    that rounding decides no arg-max)."""
    vocab = TINY[name.split("_")[0]]["config"].vocab_size
    rng = np.random.default_rng(40)
    prompts = [rng.integers(0, vocab, int(n)).tolist() for n in rng.integers(1, 40, 40)]
    eng = engine(folders[name], "float32", page_size=8, max_batch_size=64, prefill_chunk_size=32,
                 max_num_batched_tokens=128, kv_cache_max_tokens=4096)
    together = eng.generate_batch(prompts, max_new_tokens=10, stop_on_eos=False)
    assert max(eng.runner._graphs) == 64
    for i in (0, 7, 19, 39):
        assert eng.generate_batch([prompts[i]], max_new_tokens=10, stop_on_eos=False)[0] == together[i]
    half = engine(folders[name], "bfloat16", page_size=8, max_batch_size=64, prefill_chunk_size=32,
                  max_num_batched_tokens=128, kv_cache_max_tokens=4096)
    outs = half.generate_batch(prompts, max_new_tokens=10, stop_on_eos=False)
    for i in (3, 21, 38):
        check_greedy(folders[name], prompts[i], outs[i], "bfloat16")


def test_a_late_table_upload_carries_the_table_of_its_own_step():
    """The block table's copy to the device runs when the stream reaches it; the host may by
    then have ended the request and given the slot to another.  The copy carries the rows as
    they were when the step was put together (made visible by a stream that is kept busy)."""
    from rosellm_b200.cache import CacheManager
    from rosellm_b200.parts import KVCacheSpec

    spec = KVCacheSpec(num_kv_heads=1, head_dim=16, window=None)
    for n_slots in (2, 12):  # few rows go one by one, more than eight as the whole table
        cm = CacheManager({0: spec}, {}, page_size=4, num_pages=64, max_slots=12, max_seq_len=32,
                          dtype=torch.float32, device="cuda")
        slots = [cm.new_request() for _ in range(n_slots)]
        for s in slots:
            assert cm.reserve(s, 9)
            cm.commit(s, 9)
        want = cm.groups[0].table.copy()
        torch.cuda._sleep(200_000_000)  # about a tenth of a second before the stream gets to the copy
        cm.sync_to_device()
        for s in slots:
            cm.release(s)
        again = cm.new_request()
        assert cm.reserve(again, 30)
        torch.cuda.synchronize()
        assert np.array_equal(cm.groups[0].device_table.cpu().numpy(), want)
        cm.sync_to_device()
        torch.cuda.synchronize()
        assert np.array_equal(cm.groups[0].device_table.cpu().numpy(), cm.groups[0].table)


@pytest.mark.parametrize("seed", [0, 1])
def test_random_arrivals_small_cache_and_discards_change_no_token(folders, seed):
    """Thirty requests arrive at random steps with lengths, token counts and sampling options of
    their own, in a cache that holds a fraction of them (so some are preempted and recomputed),
    a few are discarded on the way, and the host runs a step ahead of the device: every
    request that stays gets the tokens it gets alone in a roomy engine that waits for each step
    (32-bit, so that rounding decides nothing)."""
    name = "B_sharp"
    vocab = TINY["B"]["config"].vocab_size
    rng = np.random.default_rng(100 + seed)
    n = 30
    prompts = [rng.integers(0, vocab, int(k)).tolist() for k in rng.integers(1, 70, n)]
    kws = []
    for i in range(n):
        kind = int(rng.integers(0, 4))
        kws.append(dict(max_new_tokens=int(rng.integers(1, 30)), stop_on_eos=False, seed=1000 + i,
                        do_sample=kind > 0, temperature=float(rng.uniform(0.6, 1.3)),
                        top_k=int(rng.integers(2, 60)) if kind == 2 else 0,
                        top_p=float(rng.uniform(0.5, 0.95)) if kind == 3 else 1.0))
    arrive = np.sort(rng.integers(0, 30, n))
    drop_at = {int(i): int(arrive[i] + rng.integers(1, 12)) for i in rng.choice(n, 5, replace=False)}

    roomy = engine(folders[name], "float32", page_size=8, max_batch_size=4, kv_cache_max_tokens=1024,
                   overlap_schedule=False)
    alone = []
    for p, kw in zip(prompts, kws):
        rid = roomy.add_request(prompt_token_ids=p, **kw)
        while roomy.has_unfinished():
            roomy.step()
        alone.append(roomy.pop_response(rid).token_ids)

    eng = engine(folders[name], "float32", page_size=8, max_batch_size=16, prefill_chunk_size=24,
                 max_num_batched_tokens=64, kv_cache_max_tokens=208, overlap_schedule=True)
    rids, dropped, step = {}, set(), 0
    while len(rids) < n or eng.has_unfinished():
        for i in range(n):
            if i not in rids and arrive[i] <= step:
                rids[i] = eng.add_request(prompt_token_ids=prompts[i], **kws[i])
        for i, at in drop_at.items():
            if at == step and i in rids and i not in dropped:
                eng.discard_request(rids[i])
                dropped.add(i)
        if eng.has_unfinished():
            eng.step()
        step += 1
        assert step < 5000
    eng.runner.check_status()
    assert eng.num_preemptions > 0
    for i in range(n):
        if i not in dropped:
            out = eng.pop_response(rids[i])
            assert out.token_ids == alone[i], f"request {i} (preempted {out.num_preemptions} times)"
    assert eng.runner.cache.num_free_pages == eng.runner.cache.num_pages
    eng.runner.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_noted_launches_give_the_logits_of_a_walk_through_the_parts(folders, dtype):
    """Steps of sizes seen before issue the noted library calls again.  The same steps (prompt
    portions beside decoded tokens, other tokens, other slots, other positions and pages each
    time, contexts on both sides of the length from which decoded requests are split) give
    bit-equal logits in a runner that walks through the parts every time.  (The fused kernels
    of few rows are switched off for this comparison: they sum with atomic additions, whose
    order, and so whose last bits, differ between any two runs; a second comparison with them
    on allows what that moves.)"""
    from rosellm_b200.config import EngineConfig
    from rosellm_b200.engine.runner import ModelRunner, StepEntry
    from rosellm_b200.ops import kernels as K

    name = "B_sharp"
    vocab = TINY["B"]["config"].vocab_size

    def run(reuse):
        r = ModelRunner.from_folder(folders[name], EngineConfig(
            dtype=dtype, page_size=8, max_num_seqs=6, max_num_batched_tokens=96, kv_cache_tokens=2048,
            cuda_graphs=False, reuse_launch_lists=reuse))
        rng = np.random.default_rng(9)
        out = []
        for round_ in range(4):
            slots = [r.cache.new_request() for _ in range(3)]
            if round_ % 2:
                slots.reverse()
            first = [int(n) for n in (40, 17, 30)]
            ids = lambda n: rng.integers(0, vocab, n).tolist()
            out.append(r.step([StepEntry(s, ids(n), [n - 1]) for s, n in zip(slots, first)]).clone())
            for _ in range(3):  # two decoded requests beside a portion of the third, then all decoded
                out.append(r.step([StepEntry(slots[0], ids(1), [0]), StepEntry(slots[1], ids(1), [0]),
                                   StepEntry(slots[2], ids(20), [3, 19])]).clone())
            for _ in range(2):
                out.append(r.step([StepEntry(s, ids(1), [0]) for s in slots]).clone())
            for s in slots:
                r.cache.release(s)
        r.check_status()
        return out, r.launch_list_replays

    try:
        K.FUSED_ROWS = False
        want, none = run(False)
        got, replays = run(True)
    finally:
        K.FUSED_ROWS = True
    assert none == 0 and replays >= 12  # of 24 steps; the first of each kind note their launches
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    fused, replays = run(True)
    assert replays >= 12
    for a, b in zip(fused, want):
        torch.testing.assert_close(a, b, atol=1e-4 if dtype == "float32" else 5e-2, rtol=0)
