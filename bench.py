"""Decode and prefill throughput of the engine on one B200, GPT-2 shapes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--workloads all|none]

Prints one JSON line.  A step is one decode step of ``--batch`` requests (default 8) that
each hold ``--context`` cached tokens (default 512) of the 124M model; ``value`` is decoded tokens
per second timed on the device over exactly K steps (``regions`` gives the median, least and
largest step time of five consecutive parts of them), ``e2e`` the same through
``InferenceEngine.add_request`` / ``step`` with token ids going in and coming out on the host.
``prefill`` is one step of 2 x 1024 prompt tokens, ``points`` decode at batch 1 and 64 (device
time, and wall clock through the entry point as ``*_e2e``), ``roofline`` the bytes a decode step
has to read (every weight once, the cache of the live requests) over its time.  ``workloads``
holds the two other workloads: 64 requests of 16 to 1023 prompt tokens and 128 new tokens through
continuous batching with portions of 512 tokens on the 355M model, and decode at batch 1 / 8 /
64 with 896 cached tokens plus a 2 x 1024 prefill on the 1.5B model.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {
    "124M": dict(n_layer=12, n_embd=768, n_head=12, n_inner=3072),
    "355M": dict(n_layer=24, n_embd=1024, n_head=16, n_inner=4096),
    "1.5B": dict(n_layer=48, n_embd=1600, n_head=25, n_inner=6400),
}
COMMON = dict(vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new")
MODEL = dict(MODELS["124M"], **COMMON)
METRIC = "decode tok/s at batch 8, 512 cached tokens (GPT-2 124M)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
REGIONS = 5  # consecutive parts the K timed steps are cut into, each between its own pair of events


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=128)
    p.add_argument("--warmup", type=int, default=16)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=512)
    p.add_argument("--layers", type=int, default=MODEL["n_layer"], help="fewer layers than the model has (named in config)")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--no-points", action="store_true", help="skip prefill and the batch 1 / 64 points")
    p.add_argument("--no-graphs", action="store_true")
    p.add_argument("--logits-then-sample", action="store_true",
                   help="write logits and sample from them in a kernel of its own, also where the head's product "
                        "could choose the tokens (for comparisons)")
    p.add_argument("--workloads", default="all", choices=["all", "none", "355M", "1.5B"],
                   help="the other two workloads (355M continuous batching, 1.5B decode and prefill)")
    return p.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            out["source"] = "measured"
        except (OSError, ValueError):
            pass
    return out


class Clocks:
    """Samples nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def decode_bytes(engine, batch, ctx_tokens, elem):
    """Bytes one decode step has to read: every weight once (the tied table once) and the
    keys and values of the live requests."""
    cfg = engine.config
    weights = engine.runner.model.weight_bytes() - cfg.n_positions * cfg.n_embd * elem  # position table: one row per token
    kv = batch * ctx_tokens * 2 * cfg.n_layer * cfg.n_embd * elem
    return weights + kv


def prefill_flops(cfg, layers, n_seqs, seq_len, rows):
    D, F, V = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    n = n_seqs * seq_len
    gemm = 2 * n * layers * (D * 3 * D + D * D + 2 * D * F)
    attn = layers * n_seqs * (4 * seq_len * seq_len * D // 2)
    head = 2 * rows * D * V
    return gemm + attn + head


class Harness:
    """An engine of one model with the measurements the bench takes of it."""

    def __init__(self, cfg: dict, dtype: str, max_batch: int, graphs: bool = True, seed: int = 0, **engine_options):
        import numpy as np

        from rosellm_b200.config import GPT2Config
        from rosellm_b200.engine.llm import InferenceEngine

        self.cfg = cfg
        self.config = GPT2Config(**cfg)
        self.dtype = dtype
        self.elem = 2 if dtype == "bfloat16" else 4
        options = dict(max_num_batched_tokens=2048, prefill_chunk_size=1024,
                       kv_cache_max_tokens=max_batch * self.config.n_positions)
        options.update(engine_options)
        self.eng = InferenceEngine(config=self.config, seed=seed, dtype=dtype, max_batch_size=max_batch,
                                   cuda_graphs=graphs, **options)
        self.runner = self.eng.runner
        self.rng = np.random.default_rng(0)
        self.vocab = self.config.vocab_size

    def close(self):
        import gc

        import torch

        self.eng = self.runner = None
        gc.collect()
        torch.cuda.empty_cache()

    def fill(self, batch, ctx):
        from rosellm_b200.engine.runner import StepEntry

        slots = [self.runner.cache.new_request() for _ in range(batch)]
        per_step = max(1, 2048 // ctx)  # prompts go in as many at a time as 2,048 tokens take
        for i in range(0, batch, per_step):
            group = slots[i:i + per_step]
            self.runner.step([StepEntry(s, self.rng.integers(0, self.vocab, ctx).tolist(), []) for s in group])
        return slots

    def device_decode(self, batch, ctx, steps, warmup):
        """(ms a step over exactly ``steps`` steps, launches, ms of the captured step alone, the
        step times of the REGIONS consecutive parts) with CUDA events on the launching stream."""
        import torch

        from rosellm_b200.engine.runner import StepEntry
        from rosellm_b200.ops import kernels as K

        runner = self.runner
        slots = self.fill(batch, ctx)
        out = torch.zeros(batch, dtype=torch.int32, device=runner.device)
        toks = self.rng.integers(0, self.vocab, (steps + warmup, batch)).tolist()

        # as the engine does it: where the head's product can choose the tokens itself, no logits
        into = K.SampleInto(out) if self.eng.sample_in_head and runner.samples_in_head(batch) else None

        def one(i):
            logits = runner.step([StepEntry(s, [toks[i][j]], [0]) for j, s in enumerate(slots)], sample_into=into)
            if into is None:
                K.sample(logits, None, None, None, None, None, out)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        l0 = K.launches() + runner.graph_launches
        n_regions = min(REGIONS, steps)
        cuts = [warmup + steps * r // n_regions for r in range(n_regions + 1)]
        events = [torch.cuda.Event(enable_timing=True) for _ in cuts]
        events[0].record()
        for r in range(n_regions):
            for i in range(cuts[r], cuts[r + 1]):
                one(i)
            events[r + 1].record()
        torch.cuda.synchronize()
        ms = events[0].elapsed_time(events[-1]) / steps
        parts = [events[r].elapsed_time(events[r + 1]) / (cuts[r + 1] - cuts[r]) for r in range(n_regions)]
        launches = K.launches() + runner.graph_launches - l0
        runner.check_status()
        # the captured step alone: the same graph replayed back to back, no host work between
        gms = None
        entry = runner._graphs.get(runner._graph_key(runner._bucket(batch), into)) if runner._graph_ok_for(batch) else None
        if entry is not None:
            g = entry[0]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(steps):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            gms = e0.elapsed_time(e1) / steps
        for s in slots:
            runner.cache.release(s)
        return ms, launches, gms, parts

    def e2e_decode(self, batch, ctx, steps, warmup):
        """Tokens a second by the wall clock through ``InferenceEngine.add_request`` / ``step``:
        token ids go in on the host and come out on the host every step."""
        import torch

        eng, runner = self.eng, self.runner
        for j in range(batch):
            # no request ends inside the timed steps (results lag a step under overlapped scheduling)
            eng.add_request(prompt_token_ids=self.rng.integers(0, self.vocab, ctx).tolist(),
                            max_new_tokens=warmup + steps + 8, stop_on_eos=False, request_id=f"b{j}")
        while any(len(eng.get_generated_ids(f"b{j}")) == 0 for j in range(batch)):
            eng.step()
        for _ in range(warmup - 1):
            eng.step()
        torch.cuda.synchronize()
        hb0 = runner.h2d_bytes + eng.sampler.h2d_bytes + runner.cache.h2d_bytes
        db0 = eng.sampler.d2h_bytes
        t0 = time.perf_counter()
        n_tok = 0
        for _ in range(steps):
            n_tok += len(eng.step())
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        h2d = (runner.h2d_bytes + eng.sampler.h2d_bytes + runner.cache.h2d_bytes - hb0) / steps
        d2h = (eng.sampler.d2h_bytes - db0) / steps
        for j in range(batch):
            eng.discard_request(f"b{j}")
        eng.pop_finished_ids()
        return n_tok / dt, h2d, d2h  # (d2h: a copy after the sampling kernel, or the ids that the head's kernel writes into pinned host memory itself)

    def prefill(self, n_seqs=2, seq_len=1024, reps=5):
        import torch

        from rosellm_b200.engine.runner import StepEntry

        runner = self.runner
        times = []
        for r in range(reps + 3):
            slots = [runner.cache.new_request() for _ in range(n_seqs)]
            # int32 arrays, as the engine hands a prompt's portions to the step function
            entries = [StepEntry(s, self.rng.integers(0, self.vocab, seq_len).astype("int32"), [seq_len - 1])
                       for s in slots]
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.step(entries)
            e1.record()
            torch.cuda.synchronize()
            if r >= 3:
                times.append(e0.elapsed_time(e1))
            for s in slots:
                runner.cache.release(s)
        return statistics.median(times)

    def continuous_batching(self, n_requests=64, new_tokens=128, lo=16, hi=1024, seed=1):
        """``n_requests`` prompts of ``lo`` to ``hi - 1`` uniform random tokens, ``new_tokens`` greedy
        tokens each (fewer where the context ends first), all added at once and run to the end
        through the scheduler (the reference's offline workload,
        benchmarks/serving/offline_compare.py:404-421, metrics of
        rosellm/roseinfer/benchmark_scheduler.py:228-234), by the wall clock."""
        import numpy as np
        import torch

        eng = self.eng
        rng = np.random.default_rng(seed)
        lens = rng.integers(lo, hi, n_requests).tolist()
        prompts = [rng.integers(0, self.vocab, n).tolist() for n in lens]
        torch.cuda.synchronize()
        steps0 = eng.num_steps
        t0 = time.perf_counter()
        rids = [eng.add_request(prompt_token_ids=p, max_new_tokens=new_tokens, stop_on_eos=False) for p in prompts]
        while eng.has_unfinished():
            eng.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        eng.pop_finished_ids()
        done = [eng.pop_response(r) for r in rids]
        completion = sum(len(o.token_ids) for o in done)
        steps = eng.num_steps - steps0
        return {"requests": n_requests, "prompt_tokens": int(sum(lens)), "completion_tokens": int(completion),
                "seconds": round(dt, 4), "steps": int(steps),
                "output_tok_s": round(completion / dt, 1), "total_tok_s": round((sum(lens) + completion) / dt, 1),
                "mean_tokens_per_step": round((sum(lens) + completion) / max(1, steps), 1),
                "preemptions": int(eng.num_preemptions)}


def workload_355m(args, pk):
    """64 requests, prompts of 16 to 1,023 tokens, 128 new tokens, continuous batching with
    portions of 512 tokens, GPT-2 355M shape."""
    h = Harness(dict(MODELS["355M"], **COMMON), args.dtype, 64, graphs=not args.no_graphs, prefill_chunk_size=512)
    try:
        h.continuous_batching(n_requests=8, new_tokens=8, seed=7)  # warm-up: graphs of the small buckets, launch lists
        rec = h.continuous_batching()
        rec["model"] = "gpt2-355M"
        rec["prefill_chunk_size"] = 512
        rec["max_num_batched_tokens"] = 2048
        return rec
    finally:
        h.close()


def workload_1_5b(args, pk):
    """Decode at batch 1 / 8 / 64 with 896 cached tokens and a prefill of 2 x 1024 tokens, GPT-2 1.5B shape."""
    cfg = dict(MODELS["1.5B"], **COMMON)
    h = Harness(cfg, args.dtype, 64, graphs=not args.no_graphs)
    try:
        rec = {"model": "gpt2-1.5B", "context_cached_tokens": 896}
        steps, warmup = 24, 4
        for b in (1, 8, 64):
            ms, _, gms, _ = h.device_decode(b, 896, steps, warmup)
            nbytes = decode_bytes(h.eng, b, 896 + warmup + steps // 2, h.elem)
            rec[f"decode_b{b}"] = round(b / (ms * 1e-3), 1)
            rec[f"ms_b{b}"] = round(ms, 4)
            rec[f"hbm_frac_b{b}"] = round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        pms = h.prefill()
        fl = prefill_flops(cfg, cfg["n_layer"], 2, 1024, 2)
        peak_fl = pk["bf16_tflops"] if args.dtype == "bfloat16" else 75.0
        rec["prefill_ms"] = round(pms, 4)
        rec["prefill_tok_s"] = round(2048 / (pms * 1e-3), 1)
        rec["prefill_frac"] = round(fl / (pms * 1e-3) / 1e12 / peak_fl, 4)
        return rec
    finally:
        h.close()


def run_ours(args):
    cfg = dict(MODEL, n_layer=args.layers)
    pk = peaks()
    h = Harness(cfg, args.dtype, max(64, args.batch), graphs=not args.no_graphs,
                sample_in_head=not args.logits_then_sample)
    eng = h.eng
    clocks = Clocks()
    clocks.start()
    ms, launches, graph_ms, parts = h.device_decode(args.batch, args.context, args.steps, args.warmup)
    clock_rec = clocks.stop()
    value = args.batch / (ms * 1e-3)
    e2e_value, h2d, d2h = h.e2e_decode(args.batch, args.context, args.steps, args.warmup)
    ctx_mid = args.context + args.warmup + args.steps // 2
    nbytes = decode_bytes(eng, args.batch, ctx_mid, h.elem)
    achieved = nbytes / (ms * 1e-3) / 1e9
    rec = {
        "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids", "impl": "ours",
        "config": config_record(args, page_size=eng.engine_config.page_size, cuda_graphs=not args.no_graphs,
                                peaks=pk["source"],
                                tokens_chosen="in the head's product" if eng.sample_in_head and h.runner.samples_in_head(args.batch)
                                else "by a sampling kernel from logits"),
        "regions": {"n": len(parts), "ms_median": round(statistics.median(parts), 4), "ms_min": round(min(parts), 4),
                    "ms_max": round(max(parts), 4)},
        "clocks": clock_rec,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(nbytes)},
    }
    if not args.no_points:
        pms = h.prefill()
        fl = prefill_flops(cfg, args.layers, 2, 1024, 2)
        peak_fl = pk["bf16_tflops"] if args.dtype == "bfloat16" else 75.0
        rec["prefill"] = {"value": round(2048 / (pms * 1e-3), 1), "tokens": 2048, "ms": round(pms, 4),
                          "frac": round(fl / (pms * 1e-3) / 1e12 / peak_fl, 4)}
        points = {"timing": "decode_b*: CUDA events on the device; decode_b*_e2e: wall clock through the entry point"}
        for b in (1, 64):
            st, wu = max(16, args.steps // 2), max(4, args.warmup // 2)
            pm, _, gm, _ = h.device_decode(b, args.context, st, wu)
            points[f"decode_b{b}"] = round(b / (pm * 1e-3), 1)
            if gm is not None:
                points[f"graph_ms_b{b}"] = round(gm, 4)
            points[f"hbm_frac_b{b}"] = round(decode_bytes(eng, b, args.context + wu + st // 2, h.elem) / (pm * 1e-3) / 1e9
                                             / pk["hbm_gbs"], 4)
            points[f"decode_b{b}_e2e"] = round(h.e2e_decode(b, args.context, st, wu)[0], 1)
        points[f"decode_b{args.batch}"] = round(value, 1)
        points[f"decode_b{args.batch}_e2e"] = round(e2e_value, 1)
        if graph_ms is not None:
            points[f"graph_ms_b{args.batch}"] = round(graph_ms, 4)
        rec["points"] = points
    h.close()
    if args.workloads != "none" and not args.no_points:
        rec["workloads"] = {}
        for key, fn in (("355M", workload_355m), ("1.5B", workload_1_5b)):
            if args.workloads in ("all", key):
                try:
                    rec["workloads"][key] = fn(args, pk)
                except Exception as e:  # the headline stands whatever happens to a further workload
                    rec["workloads"][key] = {"failed": f"{type(e).__name__}: {str(e)[:200]}"}
    print(json.dumps(rec))


def config_record(args, **more):
    """The sizes of the run, flat, the same keys for both arms."""
    rec = {"model": "gpt2-124M", "n_layer": args.layers, "n_layer_of_model": MODEL["n_layer"],
           "n_embd": MODEL["n_embd"], "n_head": MODEL["n_head"], "n_inner": MODEL["n_inner"],
           "vocab_size": MODEL["vocab_size"], "n_positions": MODEL["n_positions"], "global_batch": args.batch,
           "seq_len": args.context, "context_cached_tokens": args.context, "parallelism": "single GPU",
           "l2": "inputs larger than L2 (weights + cache read per step exceed 126 MB)"}
    rec.update(more)
    return rec


def run_reference(args):
    """The unmodified reference through its own public API: GPTModel with its own random
    initialisation, InferenceEngine and its schedulers with token-id prompts."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "rosellm")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"}))
        return
    sys.path.insert(0, ref)
    try:
        import gc

        import numpy as np
        import torch
        from rosellm.roseinfer.engine import ChunkedOnlineScheduler, InferenceEngine, OnlineRequest, OnlineScheduler
        from rosellm.roseinfer.simple_tokenizer import ByteTokenizer
        from rosellm.rosetrainer.config import GPTConfig
        from rosellm.rosetrainer.model import GPTModel

        rng = np.random.default_rng(0)
        vocab = COMMON["vocab_size"]

        def engine_of(sizes, layers, concurrency):
            torch.manual_seed(0)
            cfg = GPTConfig(vocab_size=vocab, max_position_embeddings=COMMON["n_positions"], n_layers=layers,
                            n_heads=sizes["n_head"], d_model=sizes["n_embd"], d_ff=sizes["n_inner"], dropout=0.0,
                            activation="gelu_new")
            model = GPTModel(cfg).to(device="cuda", dtype=torch.bfloat16).eval()
            return InferenceEngine(model=model, config=cfg, tokenizer=ByteTokenizer(256), tokenizer_name="bytes",
                                   device="cuda", use_amp=True, bf16=True, kv_cache_max_concurrency=concurrency,
                                   prefix_cache_max_entries=0)

        def decode_rate(eng, batch, ctx, steps, warmup):
            sched = OnlineScheduler(eng, max_batch_size=batch, use_prefix_cache=False)
            total = warmup + steps + 2
            reqs = [OnlineRequest(prompt="", prompt_token_ids=rng.integers(0, vocab, ctx).tolist(),
                                  max_new_tokens=total, stop_on_eos=False, request_id=i) for i in range(batch)]
            sched.add_requests(reqs)
            for _ in range(warmup):
                sched.step()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                sched.step()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            for i in range(batch):
                sched.discard_request(i)
            return batch * steps / dt, dt

        def prefill_ms(eng):
            # 2 x 1023 tokens (1024 leaves no room to generate): admission runs the prompts in one padded forward pass
            times = []
            for rep in range(5):
                sched = OnlineScheduler(eng, max_batch_size=2, use_prefix_cache=False)
                reqs = [OnlineRequest(prompt="", prompt_token_ids=rng.integers(0, vocab, 1023).tolist(),
                                      max_new_tokens=1, stop_on_eos=False, request_id=i) for i in range(2)]
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                sched.add_requests(reqs)
                torch.cuda.synchronize()
                times.append(time.perf_counter() - t0)
            return statistics.median(times[2:]) * 1e3

        def continuous(eng, n_requests=64, new_tokens=128, seed=1):
            """The 355M workload through the reference's chunked scheduler (portions of 512), or,
            where that refuses to run here, its scheduler that prefills at admission."""
            r2 = np.random.default_rng(seed)
            lens = r2.integers(16, 1024, n_requests).tolist()
            prompts = [r2.integers(0, vocab, n).tolist() for n in lens]

            def go(make, label):
                sched = make()
                reqs = [OnlineRequest(prompt="", prompt_token_ids=p, max_new_tokens=new_tokens, stop_on_eos=False,
                                      request_id=i) for i, p in enumerate(prompts)]
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                sched.add_requests(reqs)
                steps = 0
                while sched.has_unfinished():
                    sched.step()
                    steps += 1
                torch.cuda.synchronize()
                dt = time.perf_counter() - t0
                completion = sum(len(sched.get_generated_ids(i)) for i in range(n_requests))
                for i in range(n_requests):
                    sched.discard_request(i)
                return {"requests": n_requests, "prompt_tokens": int(sum(lens)), "completion_tokens": int(completion),
                        "seconds": round(dt, 4), "steps": steps, "output_tok_s": round(completion / dt, 1),
                        "total_tok_s": round((sum(lens) + completion) / dt, 1), "path": label}

            try:
                return go(lambda: ChunkedOnlineScheduler(eng, max_batch_size=64, prefill_chunk_size=512,
                                                         use_prefix_cache=False), "ChunkedOnlineScheduler, portions of 512")
            except Exception as e:
                first = f"{type(e).__name__}: {str(e)[:120]}"
                out = go(lambda: OnlineScheduler(eng, max_batch_size=64, use_prefix_cache=False),
                         "OnlineScheduler (prompts prefilled at admission)")
                out["chunked_scheduler"] = first
                return out

        eng = engine_of(MODELS["124M"], args.layers, max(64, args.batch))
        clocks = Clocks()
        clocks.start()
        value, dt = decode_rate(eng, args.batch, args.context, args.steps, args.warmup)
        clock_rec = clocks.stop()
        rec = {
            "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: the reference's own random initialisation, uniform random token ids",
            "impl": "reference",
            "config": config_record(args, page_size=64, cuda_graphs=True, peaks=peaks()["source"],
                                    tokens_chosen="by the reference's own sampling"),
            "path": "OnlineScheduler.step (paged decode, CUDA graphs, overlap schedule)",
            "clocks": clock_rec,
            "e2e": {"value": round(value, 1), "unit": "tokens/s", "note": "wall clock around OnlineScheduler.step"},
        }
        if not args.no_points:
            points = {"timing": "wall clock around OnlineScheduler.step"}
            for b in (1, 64):
                try:
                    rate = decode_rate(eng, b, args.context, max(16, args.steps // 2), max(4, args.warmup // 2))[0]
                    points[f"decode_b{b}"] = points[f"decode_b{b}_e2e"] = round(rate, 1)
                except Exception as e:
                    points[f"decode_b{b}"] = f"{type(e).__name__}: {str(e)[:120]}"
            points[f"decode_b{args.batch}"] = points[f"decode_b{args.batch}_e2e"] = round(value, 1)
            rec["points"] = points
            try:
                ms = prefill_ms(eng)
                rec["prefill"] = {"value": round(2046 / (ms * 1e-3), 1), "tokens": 2046, "ms": round(ms, 4),
                                  "note": "wall clock around OnlineScheduler.add_requests (2 x 1023 tokens; 1024 leaves no room to generate)"}
            except Exception as e:
                rec["prefill"] = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
        del eng
        gc.collect()
        torch.cuda.empty_cache()
        if args.workloads != "none" and not args.no_points:
            rec["workloads"] = {}
            if args.workloads in ("all", "355M"):
                try:
                    eng = engine_of(MODELS["355M"], MODELS["355M"]["n_layer"], 64)
                    continuous(eng, n_requests=8, new_tokens=8, seed=7)
                    rec["workloads"]["355M"] = dict(continuous(eng), model="gpt2-355M")
                except Exception as e:
                    rec["workloads"]["355M"] = {"failed": f"{type(e).__name__}: {str(e)[:200]}"}
                eng = None
                gc.collect()
                torch.cuda.empty_cache()
            if args.workloads in ("all", "1.5B"):
                try:
                    eng = engine_of(MODELS["1.5B"], MODELS["1.5B"]["n_layer"], 128)
                    w = {"model": "gpt2-1.5B", "context_cached_tokens": 896}
                    for b in (1, 8, 64):
                        w[f"decode_b{b}"] = round(decode_rate(eng, b, 896, 24, 4)[0], 1)
                    ms = prefill_ms(eng)
                    w["prefill_ms"] = round(ms, 4)
                    w["prefill_tok_s"] = round(2046 / (ms * 1e-3), 1)
                    rec["workloads"]["1.5B"] = w
                except Exception as e:
                    rec["workloads"]["1.5B"] = {"failed": f"{type(e).__name__}: {str(e)[:200]}"}
                eng = None
                gc.collect()
                torch.cuda.empty_cache()
        print(json.dumps(rec))
    except Exception as e:  # the reference's own failure is reported, not hidden
        print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}))


def main():
    args = parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        sys.exit(2)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
