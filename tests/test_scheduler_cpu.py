"""The scheduler's decisions, driven by a fake step that 'samples' a function of the tokens."""
import pytest

from rosellm_b200.cache import CacheManager
from rosellm_b200.engine.scheduler import FINISHED, RUNNING, WAITING, Scheduler
from rosellm_b200.parts import KVCacheSpec
from rosellm_b200.sampling import SamplingParams


def make(pages=64, page=4, seqs=4, budget=32, chunk=16, max_len=64, eos=None, **kw):
    cache = CacheManager({0: KVCacheSpec(1, 16)}, {}, page_size=page, num_pages=pages, max_slots=seqs,
                         max_seq_len=max_len, device="cpu", allocate_pools=False)
    return Scheduler(cache, max_num_seqs=seqs, max_num_batched_tokens=budget, prefill_chunk_size=chunk,
                     max_model_len=max_len, eos_token_id=eos, **kw), cache


def fake_token(req) -> int:
    """Depends only on the request's own tokens, like a model would."""
    return (sum(req.all_ids) * 31 + len(req.all_ids)) % 97 + 1


def run_step(s, cache):
    plan = s.schedule()
    for it in plan.items:  # what ModelRunner.step does to the cache
        assert int(cache.num_tokens[it.request.slot]) == it.start == it.request.num_computed
        cache.commit(it.request.slot, it.count)
    done = s.update(plan, [fake_token(it.request) for it in plan.items if it.samples])
    cache.check()
    return plan, done


def run_all(s, cache, limit=10_000):
    plans = []
    while s.has_unfinished():
        plans.append(run_step(s, cache)[0])
        assert len(plans) < limit
    return plans


def test_prompt_is_cut_into_portions_under_the_budget():
    s, cache = make(budget=20, chunk=8)
    a = s.add_request(list(range(1, 20)), SamplingParams(max_new_tokens=3))
    b = s.add_request(list(range(1, 6)), SamplingParams(max_new_tokens=2))
    p1, _ = run_step(s, cache)
    assert [(i.request is a, i.start, i.count, i.samples) for i in p1.items] == [(True, 0, 8, False), (False, 0, 5, True)]
    assert len(b.output_ids) == 1
    p2, _ = run_step(s, cache)
    # the single token of b first, then a's next portion
    assert [(i.request is b, i.count, i.samples) for i in p2.items] == [(True, 1, True), (False, 8, False)]
    assert b.status == FINISHED and b.finish_reason == "length"
    p3, _ = run_step(s, cache)
    assert [(i.start, i.count, i.samples) for i in p3.items] == [(16, 3, True)]
    run_all(s, cache)
    assert a.status == FINISHED and len(a.output_ids) == 3
    assert cache.num_free_pages == 64 and cache.num_free_slots == 4


def test_token_budget_limits_a_step():
    s, cache = make(budget=10, chunk=16, seqs=4)
    reqs = [s.add_request([1] * 7, SamplingParams(max_new_tokens=4)) for _ in range(3)]
    p1, _ = run_step(s, cache)
    assert [i.count for i in p1.items] == [7, 3] and p1.num_tokens == 10
    p2, _ = run_step(s, cache)
    assert [(i.request is reqs[0], i.count) for i in p2.items][0] == (True, 1)
    assert p2.num_tokens <= 10
    run_all(s, cache)
    assert all(r.status == FINISHED and len(r.output_ids) == 4 for r in reqs)


def test_max_num_seqs_caps_admission_and_order_is_fifo():
    s, cache = make(seqs=2, budget=64)
    reqs = [s.add_request([i + 1] * 3, SamplingParams(max_new_tokens=2 + i)) for i in range(4)]
    p1, _ = run_step(s, cache)
    assert [i.request for i in p1.items] == reqs[:2] and reqs[2].status == WAITING
    run_step(s, cache)  # the first finishes (2 tokens) and frees its slot
    assert reqs[0].status == FINISHED
    p3, _ = run_step(s, cache)
    assert reqs[2] in [i.request for i in p3.items] and reqs[3].status == WAITING
    run_all(s, cache)
    assert [len(r.output_ids) for r in reqs] == [2, 3, 4, 5]


def test_finish_on_eos_and_on_context_end():
    s, cache = make(eos=5, max_len=12)
    r = s.add_request([1, 2], SamplingParams(max_new_tokens=50))
    assert r.max_new_tokens == 10  # cut to the room left in the context
    plan = s.schedule()
    cache.commit(r.slot, 2)
    s.update(plan, [5])
    assert r.status == FINISHED and r.finish_reason == "stop" and r.output_ids == [5]
    r2 = s.add_request([1, 2], SamplingParams(max_new_tokens=50, stop_on_eos=False))
    plan = s.schedule()
    cache.commit(r2.slot, 2)
    s.update(plan, [5])
    assert r2.status == RUNNING
    run_all(s, cache)
    assert r2.finish_reason == "length" and r2.num_tokens == 12
    full = s.add_request(list(range(12)), SamplingParams())
    assert full.status == FINISHED and full.finish_reason == "length" and full.output_ids == []
    assert s.add_request([], SamplingParams(max_new_tokens=1)).prompt_ids == [5]  # empty prompt: the eos token


def test_prompts_that_do_not_fit():
    s, _ = make(max_len=16, pages=2)
    with pytest.raises(ValueError, match="exceeds the context"):
        s.add_request([1] * 17, SamplingParams())
    with pytest.raises(ValueError, match="can never fit"):
        s.add_request([1] * 9, SamplingParams(max_new_tokens=1))  # 9 tokens need 3 pages of 4
    s2, _ = make(max_len=16, truncate_prompt=True)
    assert s2.add_request(list(range(20)), SamplingParams()).prompt_ids == list(range(4, 20))
    s3, _ = make()
    with pytest.raises(ValueError, match="empty prompt"):
        s3.add_request([], SamplingParams())


def test_no_admission_while_the_first_portion_does_not_fit():
    s, cache = make(pages=6, page=4, budget=64, chunk=64, max_len=24)
    a = s.add_request([1] * 16, SamplingParams(max_new_tokens=4))
    b = s.add_request([2] * 12, SamplingParams(max_new_tokens=2))
    p1, _ = run_step(s, cache)
    assert [i.request for i in p1.items] == [a] and b.status == WAITING  # 4 + 3 pages > 6
    run_all(s, cache)
    assert a.status == b.status == FINISHED and a.num_preemptions == b.num_preemptions == 0


def test_youngest_request_is_preempted_and_recomputed_when_pages_run_out():
    # 5 pages of 4: two requests of 7 prompt tokens take 2 pages each and both need a third
    s, cache = make(pages=5, page=4, budget=64, chunk=64, max_len=20)
    a = s.add_request([1] * 7, SamplingParams(max_new_tokens=8))
    b = s.add_request([2] * 7, SamplingParams(max_new_tokens=8))
    seen_preempt = False
    outputs_before = None
    steps = 0
    while s.has_unfinished():
        plan, _ = run_step(s, cache)
        steps += 1
        if plan.preempted:
            assert plan.preempted == [b] and not seen_preempt  # the one admitted last
            seen_preempt = True
            outputs_before = list(b.output_ids)
            assert b.status == WAITING and b.slot is None and b.num_computed == 0
            assert s.waiting[0] is b and a in [i.request for i in plan.items]
            assert all(i.request is not b for i in plan.items)  # no admission in the step that preempted
        assert steps < 100
    assert seen_preempt and b.num_preemptions == 1 and a.num_preemptions == 0
    assert b.output_ids[: len(outputs_before)] == outputs_before and len(b.output_ids) == 8
    # the same requests with room for both give the same tokens: preemption changes no result
    s2, cache2 = make(pages=64, page=4, budget=64, chunk=64, max_len=20)
    a2 = s2.add_request([1] * 7, SamplingParams(max_new_tokens=8))
    b2 = s2.add_request([2] * 7, SamplingParams(max_new_tokens=8))
    run_all(s2, cache2)
    assert (a2.output_ids, b2.output_ids) == (a.output_ids, b.output_ids)
    assert cache.num_free_pages == 5 and cache.num_free_slots == 4


def test_abort_gives_everything_back():
    s, cache = make()
    a = s.add_request([1] * 9, SamplingParams(max_new_tokens=5))
    b = s.add_request([1] * 3, SamplingParams(max_new_tokens=5))
    run_step(s, cache)
    s.abort(a)
    assert a.finish_reason == "abort" and cache.num_free_slots == 3
    run_all(s, cache)
    assert b.status == FINISHED and cache.num_free_pages == 64


def test_seeds_default_per_request_and_greedy_rule():
    s, _ = make()
    r1 = s.add_request([1], SamplingParams(seed=11))
    r2 = s.add_request([1], SamplingParams())
    assert r1.seed == 11 and isinstance(r2.seed, int)
    # a default seed is a checksum, not Python's salted hash: the same in every process, and another
    # for another id, prompt length or engine seed
    assert len({s.default_seed("req-a", 3), s.default_seed("req-b", 3), s.default_seed("req-a", 4),
                s.default_seed(7, 3), s.default_seed("7", 3), make(seed=1)[0].default_seed("req-a", 3)}) == 6
    import subprocess
    import sys
    code = ("from rosellm_b200.engine.scheduler import Scheduler; "
            "print(Scheduler.default_seed(type('S', (), {'seed': 0})(), 'req-a', 3))")
    outs = {subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, check=True,
                           env={"PYTHONHASHSEED": h, "PYTHONPATH": ":".join(sys.path)}).stdout for h in ("1", "2")}
    assert outs == {f"{s.default_seed('req-a', 3)}\n"}
    assert SamplingParams(temperature=0.7).greedy  # not asked to sample: arg-max whatever the temperature
    assert SamplingParams(temperature=0.0, do_sample=True).greedy
    assert not SamplingParams(temperature=0.7, do_sample=True).greedy
    with pytest.raises(ValueError):
        SamplingParams(max_new_tokens=0)


def run_overlapped(s, cache, limit=10_000):
    """Drives the scheduler as the engine does with overlap: the step is planned and 'launched'
    (advance) before the tokens of the step before it are known (resolve)."""
    inflight = None
    steps = 0
    while s.has_unfinished() or inflight is not None:
        launched = None
        if s.has_unfinished():
            plan = s.schedule()
            if plan.items:
                for it in plan.items:
                    assert int(cache.num_tokens[it.request.slot]) == it.start
                    cache.commit(it.request.slot, it.count)
                s.advance(plan)
                launched = plan
        if inflight is not None:
            # the device knows the tokens of the step before; the fake model reads the resolved prefix
            toks = []
            for it in inflight.items:
                if it.samples:
                    r = it.request
                    prefix = r.prompt_ids + [t for t in r.output_ids[: it.out_index]]
                    assert all(t >= 0 for t in prefix)
                    toks.append((sum(prefix) * 31 + len(prefix)) % 97 + 1)
            s.resolve(inflight, toks)
        inflight = launched
        cache.check()
        steps += 1
        assert steps < limit
    return steps


@pytest.mark.parametrize("pages", [64, 5])
def test_launching_before_reading_gives_the_same_tokens(pages):
    """Overlapped driving equals step-by-step driving, with room and with preemptions, with
    requests ending on their token count and on an end-of-sequence token that is only known
    after the next step has been launched."""
    def requests(s):
        return [s.add_request([1] * 7, SamplingParams(max_new_tokens=8)),
                s.add_request([2] * 7, SamplingParams(max_new_tokens=5)),
                s.add_request([3, 4], SamplingParams(max_new_tokens=9))]

    s1, c1 = make(pages=pages, page=4, budget=64, chunk=64, max_len=20, eos=None)
    r1 = requests(s1)
    run_all(s1, c1)
    eos = r1[2].output_ids[3]  # make the third request stop early on a token it will produce
    outs = {}
    for mode in ("sync", "overlap"):
        s, c = make(pages=pages, page=4, budget=64, chunk=64, max_len=20, eos=eos)
        rs = requests(s)
        run_all(s, c) if mode == "sync" else run_overlapped(s, c)
        assert all(r.status == FINISHED for r in rs)
        assert all(t >= 0 for r in rs for t in r.output_ids)
        outs[mode] = [(r.output_ids, r.finish_reason) for r in rs]
        assert c.num_free_pages == pages and c.num_free_slots == 4
    assert outs["sync"] == outs["overlap"]
    assert outs["sync"][2][1] == "stop" and outs["sync"][2][0][-1] == eos


@pytest.mark.parametrize("seed", range(8))
def test_random_workloads_keep_every_rule(seed):
    """Random limits, arrivals, lengths and aborts, driven step by step: no step exceeds the
    token budget, the request limit or a portion's length; portions follow one another without a
    gap; a prompt's portions precede its decoded tokens; everything ends and gives back what it
    held; and each request's tokens are those it gets alone in a cache with room (the fake
    model's token depends on the request's own tokens only)."""
    import random

    rnd = random.Random(seed)
    page = rnd.choice([1, 4, 8])
    max_len = rnd.choice([24, 40, 64])
    seqs = rnd.randint(1, 6)
    budget = rnd.randint(4, 48)
    chunk = rnd.randint(2, 24)
    # room for the longest request at least; often little more, so that requests are preempted
    pages = -(-max_len // page) + rnd.randint(0, 2 * max_len // page)
    n = 14
    jobs = []
    for i in range(n):
        plen = rnd.randint(1, max_len - 2)
        jobs.append(dict(prompt=[rnd.randint(1, 90) for _ in range(plen)],
                         new=rnd.randint(1, max_len - plen), at=rnd.randint(0, 25),
                         abort_at=rnd.randint(3, 40) if rnd.random() < 0.2 else None))

    def alone(job):
        s, c = make(pages=max_len, page=page, seqs=1, budget=max_len, chunk=max_len, max_len=max_len)
        r = s.add_request(job["prompt"], SamplingParams(max_new_tokens=job["new"], stop_on_eos=False))
        run_all(s, c)
        return r.output_ids

    want = [alone(j) for j in jobs]
    s, cache = make(pages=pages, page=page, seqs=seqs, budget=budget, chunk=chunk, max_len=max_len)
    reqs, aborted, step = {}, set(), 0
    while len(reqs) < n or s.has_unfinished():
        for i, j in enumerate(jobs):
            if i not in reqs and j["at"] <= step:
                reqs[i] = s.add_request(j["prompt"], SamplingParams(max_new_tokens=j["new"], stop_on_eos=False))
        for i, j in enumerate(jobs):
            if j["abort_at"] == step and i in reqs and reqs[i].status != FINISHED:
                s.abort(reqs[i])
                aborted.add(i)
        if s.has_unfinished():
            plan, _ = run_step(s, cache)
            assert sum(it.count for it in plan.items) <= budget
            assert len(plan.items) <= seqs and len({id(it.request) for it in plan.items}) == len(plan.items)
            for it in plan.items:
                assert 1 <= it.count <= chunk
                known = len(it.request.prompt_ids) + len(it.request.output_ids)  # after this step's token
                if it.samples:  # the portion brought the last token known before the step
                    assert it.start + it.count == known - 1
                else:
                    assert it.start + it.count < known
        step += 1
        assert step < 5000
    for i in range(n):
        if i not in aborted:
            assert reqs[i].status == FINISHED and reqs[i].output_ids == want[i], i
    assert cache.num_free_pages == pages and cache.num_free_slots == seqs
    cache.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_launched_ahead_equal_step_by_step(seed):
    """The same random requests under random limits, driven with each step launched before the
    tokens of the step before are read, and driven step by step: the same tokens and reasons,
    with an end-of-sequence token that some requests produce on their way."""
    import random

    rnd = random.Random(100 + seed)
    page, max_len = rnd.choice([2, 4, 8]), rnd.choice([24, 48])
    limits = dict(pages=-(-max_len // page) + rnd.randint(0, max_len // page), page=page, seqs=rnd.randint(1, 5),
                  budget=rnd.randint(4, 40), chunk=rnd.randint(2, 16), max_len=max_len)
    jobs = []
    for _ in range(10):
        plen = rnd.randint(1, max_len - 2)
        jobs.append(([rnd.randint(1, 90) for _ in range(plen)], rnd.randint(1, max_len - plen)))

    def drive(overlapped, eos):
        s, c = make(eos=eos, **limits)
        rs = [s.add_request(p, SamplingParams(max_new_tokens=n)) for p, n in jobs]
        run_overlapped(s, c) if overlapped else run_all(s, c)
        assert all(r.status == FINISHED for r in rs)
        assert c.num_free_pages == limits["pages"] and c.num_free_slots == limits["seqs"]
        return [(r.output_ids, r.finish_reason) for r in rs]

    free = drive(False, None)
    produced = [t for out, _ in free for t in out[1:-1]]
    eos = produced[len(produced) // 2] if produced else None  # a token from the middle of some output
    want = drive(False, eos)
    assert drive(True, eos) == want
    if eos is not None:
        assert any(reason == "stop" for _, reason in want)
