"""Decode and prefill throughput of the engine on one B200, GPT-2 124M shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  A step is one decode step of ``--batch`` requests (default 8) that
each hold ``--context`` cached tokens (default 512); ``value`` is decoded tokens per second
timed on the device over K steps, ``e2e`` the same through ``InferenceEngine.add_request`` /
``step`` with token ids going in and coming out on the host.  ``prefill`` is one step of
2 x 1024 prompt tokens, ``points`` decode at batch 1 and 64, ``roofline`` the bytes a decode
step has to read (every weight once, the cache of the live requests) over its time.
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

MODEL = dict(n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257, n_positions=1024,
             layer_norm_epsilon=1e-5, activation_function="gelu_new")
METRIC = "decode tok/s at batch 8, 512 cached tokens (GPT-2 124M)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


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


def model_numbers(cfg, layers):
    D, F, V, H = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"], cfg["n_head"]
    layer_params = D * 3 * D + D * D + 2 * D * F
    return dict(layer_matrix_params=layers * layer_params, D=D, F=F, V=V, L=layers)


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


def run_ours(args):
    import numpy as np
    import torch

    from rosellm_b200.config import GPT2Config
    from rosellm_b200.engine.llm import InferenceEngine
    from rosellm_b200.engine.runner import StepEntry
    from rosellm_b200.ops import kernels as K

    cfg = dict(MODEL, n_layer=args.layers)
    config = GPT2Config(**cfg)
    max_b = max(64, args.batch)
    eng = InferenceEngine(config=config, seed=0, dtype=args.dtype, max_batch_size=max_b,
                          max_num_batched_tokens=2048, prefill_chunk_size=1024,
                          kv_cache_max_tokens=max_b * config.n_positions, cuda_graphs=not args.no_graphs)
    runner = eng.runner
    rng = np.random.default_rng(0)
    vocab = config.vocab_size
    elem = 2 if args.dtype == "bfloat16" else 4
    pk = peaks()

    def fill(batch, ctx):
        slots = []
        for _ in range(batch):
            s = runner.cache.new_request()
            slots.append(s)
        # prompts go in two at a time, 1024 tokens a step at most
        for i in range(0, batch, max(1, 2048 // ctx)):
            group = slots[i:i + max(1, 2048 // ctx)]
            runner.step([StepEntry(s, rng.integers(0, vocab, ctx).tolist(), []) for s in group])
        return slots

    def device_decode(batch, ctx, steps, warmup):
        slots = fill(batch, ctx)
        out = torch.zeros(batch, dtype=torch.int32, device=runner.device)
        toks = rng.integers(0, vocab, (steps + warmup, batch)).tolist()

        def one(i):
            logits = runner.step([StepEntry(s, [toks[i][j]], [0]) for j, s in enumerate(slots)])
            K.sample(logits, None, None, None, None, None, out)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        l0 = K.launches() + runner.graph_launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(warmup, warmup + steps):
            one(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = K.launches() + runner.graph_launches - l0
        runner.check_status()
        # the captured step alone: the same graph replayed back to back, no host work between
        gms = None
        entry = runner._graphs.get(runner._bucket(batch)) if runner._graph_ok_for(batch) else None
        if entry is not None:
            g = entry[0]
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
        return ms, launches, gms

    def e2e_decode(batch, ctx, steps, warmup):
        h0 = runner.h2d_bytes + eng.sampler.h2d_bytes
        for j in range(batch):
            # no request ends inside the timed steps (results lag a step under overlapped scheduling)
            eng.add_request(prompt_token_ids=rng.integers(0, vocab, ctx).tolist(), max_new_tokens=warmup + steps + 8,
                            stop_on_eos=False, request_id=f"b{j}")
        while any(len(eng.get_generated_ids(f"b{j}")) == 0 for j in range(batch)):
            eng.step()
        for _ in range(warmup - 1):
            eng.step()
        torch.cuda.synchronize()
        hb0 = runner.h2d_bytes + eng.sampler.h2d_bytes
        db0 = eng.sampler.d2h_bytes
        t0 = time.perf_counter()
        n_tok = 0
        for _ in range(steps):
            n_tok += len(eng.step())
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        h2d = (runner.h2d_bytes + eng.sampler.h2d_bytes - hb0) / steps
        d2h = (eng.sampler.d2h_bytes - db0) / steps
        for j in range(batch):
            eng.discard_request(f"b{j}")
        eng.pop_finished_ids()
        return n_tok / dt, h2d, d2h

    def prefill(n_seqs=2, seq_len=1024, reps=5):
        times = []
        for r in range(reps + 3):
            slots = [runner.cache.new_request() for _ in range(n_seqs)]
            entries = [StepEntry(s, rng.integers(0, vocab, seq_len).tolist(), [seq_len - 1]) for s in slots]
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

    clocks = Clocks()
    clocks.start()
    ms, launches, graph_ms = device_decode(args.batch, args.context, args.steps, args.warmup)
    clock_rec = clocks.stop()
    value = args.batch / (ms * 1e-3)
    e2e_value, h2d, d2h = e2e_decode(args.batch, args.context, args.steps, args.warmup)
    ctx_mid = args.context + args.warmup + args.steps // 2
    nbytes = decode_bytes(eng, args.batch, ctx_mid, elem)
    achieved = nbytes / (ms * 1e-3) / 1e9
    rec = {
        "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids", "impl": "ours",
        "config": {"model": "gpt2-124M", "n_layer": args.layers, "n_layer_of_model": MODEL["n_layer"],
                   "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "n_inner": cfg["n_inner"],
                   "vocab_size": cfg["vocab_size"], "n_positions": cfg["n_positions"], "global_batch": args.batch,
                   "seq_len": args.context, "context_cached_tokens": args.context, "parallelism": "single GPU",
                   "page_size": eng.engine_config.page_size, "cuda_graphs": not args.no_graphs,
                   "l2": "inputs larger than L2 (weights + cache read per step exceed 126 MB)",
                   "peaks": pk["source"]},
        "clocks": clock_rec,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(nbytes)},
    }
    if not args.no_points:
        pms = prefill()
        fl = prefill_flops(cfg, args.layers, 2, 1024, 2)
        peak_fl = pk["bf16_tflops"] if args.dtype == "bfloat16" else 75.0
        rec["prefill"] = {"value": round(2048 / (pms * 1e-3), 1), "tokens": 2048, "ms": round(pms, 4),
                          "frac": round(fl / (pms * 1e-3) / 1e12 / peak_fl, 4)}
        points = {}
        for b in (1, 64):
            pm, _, gm = device_decode(b, args.context, max(16, args.steps // 2), max(4, args.warmup // 2))
            points[f"decode_b{b}"] = round(b / (pm * 1e-3), 1)
            if gm is not None:
                points[f"graph_ms_b{b}"] = round(gm, 4)
        points[f"decode_b{args.batch}"] = round(value, 1)
        if graph_ms is not None:
            points[f"graph_ms_b{args.batch}"] = round(graph_ms, 4)
        rec["points"] = points
    print(json.dumps(rec))


def run_reference(args):
    """The unmodified reference through its own public API: GPTModel with its own random
    initialisation, InferenceEngine and OnlineScheduler with token-id prompts."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "rosellm")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"}))
        return
    sys.path.insert(0, ref)
    try:
        import torch
        from rosellm.roseinfer.engine import InferenceEngine, OnlineRequest, OnlineScheduler
        from rosellm.roseinfer.simple_tokenizer import ByteTokenizer
        from rosellm.rosetrainer.config import GPTConfig
        from rosellm.rosetrainer.model import GPTModel

        import numpy as np

        torch.manual_seed(0)
        cfg = GPTConfig(vocab_size=MODEL["vocab_size"], max_position_embeddings=MODEL["n_positions"],
                        n_layers=args.layers, n_heads=MODEL["n_head"], d_model=MODEL["n_embd"],
                        d_ff=MODEL["n_inner"], dropout=0.0, activation="gelu_new")
        model = GPTModel(cfg).to(device="cuda", dtype=torch.bfloat16).eval()
        eng = InferenceEngine(model=model, config=cfg, tokenizer=ByteTokenizer(256), tokenizer_name="bytes",
                              device="cuda", use_amp=True, bf16=True, kv_cache_max_concurrency=max(64, args.batch),
                              prefix_cache_max_entries=0)
        rng = np.random.default_rng(0)

        def decode_rate(batch, steps, warmup):
            sched = OnlineScheduler(eng, max_batch_size=batch, use_prefix_cache=False)
            total = warmup + steps + 2
            reqs = [OnlineRequest(prompt="", prompt_token_ids=rng.integers(0, cfg.vocab_size, args.context).tolist(),
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

        clocks = Clocks()
        clocks.start()
        value, dt = decode_rate(args.batch, args.steps, args.warmup)
        clock_rec = clocks.stop()
        rec = {
            "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: the reference's own random initialisation, uniform random token ids",
            "impl": "reference",
            "config": {"model": "gpt2-124M", "n_layer": args.layers, "n_layer_of_model": MODEL["n_layer"],
                       "global_batch": args.batch, "seq_len": args.context, "parallelism": "single GPU",
                       "path": "OnlineScheduler.step (paged decode, CUDA graphs, overlap schedule)"},
            "clocks": clock_rec,
            "e2e": {"value": round(value, 1), "unit": "tokens/s", "note": "wall clock around OnlineScheduler.step"},
        }
        if not args.no_points:
            points = {}
            for b in (1, 64):
                try:
                    points[f"decode_b{b}"] = round(decode_rate(b, max(16, args.steps // 2), max(4, args.warmup // 2))[0], 1)
                except Exception as e:
                    points[f"decode_b{b}"] = f"{type(e).__name__}: {str(e)[:120]}"
            rec["points"] = points
            try:
                # prefill of 2 x 1024 tokens: admission runs the prompts in one padded forward pass
                times = []
                for rep in range(5):
                    sched = OnlineScheduler(eng, max_batch_size=2, use_prefix_cache=False)
                    reqs = [OnlineRequest(prompt="", prompt_token_ids=rng.integers(0, cfg.vocab_size, 1023).tolist(),
                                          max_new_tokens=1, stop_on_eos=False, request_id=i) for i in range(2)]
                    torch.cuda.synchronize()
                    t0 = time.perf_counter()
                    sched.add_requests(reqs)
                    torch.cuda.synchronize()
                    times.append(time.perf_counter() - t0)
                ms = statistics.median(times[2:]) * 1e3
                rec["prefill"] = {"value": round(2046 / (ms * 1e-3), 1), "tokens": 2046, "ms": round(ms, 4),
                                  "note": "wall clock around OnlineScheduler.add_requests (2 x 1023 tokens; 1024 leaves no room to generate)"}
            except Exception as e:
                rec["prefill"] = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
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
