"""Trace replay: feed given token ids through a model step by step and write logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Reads one JSON object per line from standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

runs each step's entries as one batch through ``ModelRunner.step`` (the same
model, step function, cache and kernels that generation uses; nothing is
sampled), writes ``DIR/<step>.f32`` with the logits at the wanted places as
little-endian float32 ``[wanted, vocab]`` when a step wants any, and prints
``done <step>`` after every step.  Requests named in ``end`` give back what
they hold after the step.  The cache pool is made for ``--max-tokens`` tokens
(each request's count rounded up to a whole page), so pages are used again.

The reference has no such tool; its nearest are the greedy-id comparisons of
rosellm/roseinfer/verify_paged_attention.py:55-111.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="tokens the live requests hold at most, each rounded up to a multiple of 64")
    p.add_argument("--page-size", type=int, default=16, help="tokens per cache page (divides 64)")
    p.add_argument("--max-requests", type=int, default=8, help="requests live at once")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--cuda-graphs", action="store_true",
                   help="replay steps in which every request brings one token and wants its logits from "
                        "CUDA graphs, as generation does (off: every step walks through the parts)")
    return p.parse_args(argv)


def main(argv=None) -> int:
    return run(parse_args(argv), sys.stdin)


def run(args: argparse.Namespace, lines, stats: dict | None = None) -> int:
    """Replay ``lines`` (an iterable of JSON lines) with the options of ``parse_args``.
    ``stats`` (a dict) receives counters of the run: steps, and how many of them were graph replays."""
    if args.max_tokens <= 0:
        print("trace_run: --max-tokens must be positive", file=sys.stderr)
        return 2
    if 64 % args.page_size != 0:
        print("trace_run: --page-size must divide 64", file=sys.stderr)
        return 2
    os.makedirs(args.out, exist_ok=True)

    from ..config.engine import EngineConfig
    from .runner import ModelRunner, StepEntry

    pool_tokens = -(-args.max_tokens // 64) * 64
    runner = ModelRunner.from_folder(
        args.model,
        EngineConfig(
            dtype=args.dtype,
            page_size=args.page_size,
            kv_cache_tokens=pool_tokens,
            max_num_seqs=args.max_requests,
            max_num_batched_tokens=max(pool_tokens, 64),
            cuda_graphs=args.cuda_graphs,
            capture_graphs_at_start=False,
            device=args.device,
        ),
    )
    slots: dict[str, int] = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for ent in rec.get("entries", []):
            rid = str(ent["id"])
            if rid not in slots:
                slot = runner.cache.new_request()
                if slot is None:
                    raise RuntimeError(f"step {step}: more than {args.max_requests} requests live")
                slots[rid] = slot
            entries.append(StepEntry(slots[rid], [int(t) for t in ent["tokens"]],
                                     [int(w) for w in ent.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(args.out, f"{step}.f32"))
            runner.check_status()
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                runner.cache.release(slots.pop(rid))
        print(f"done {step}", flush=True)
    if stats is not None:
        stats["steps"] = runner.steps_run
        stats["graph_replays"] = runner.graph_replays
        stats["launch_list_replays"] = runner.launch_list_replays
    return 0


if __name__ == "__main__":
    sys.exit(main())
