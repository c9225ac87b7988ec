"""Builds replay traces (whole, tail decoded, portions, mixed) and checks their logits
against the plain implementation."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import torch

import plain_gpt2 as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Trace:
    def __init__(self):
        self.steps: list[dict] = []
        self.wanted: list[list[tuple[str, int]]] = []  # per step: (request, absolute position)
        self._at: dict[str, int] = {}

    def add(self, entries: list[tuple[str, list[int], list[int]]], end=()):
        """entries: (request id, tokens, wanted places among them)."""
        rec = {"step": len(self.steps), "entries": [], "end": list(end)}
        want = []
        for rid, toks, places in entries:
            base = self._at.get(rid, 0)
            rec["entries"].append({"id": rid, "tokens": list(map(int, toks)), "want": list(places)})
            want.extend((rid, base + p) for p in places)
            self._at[rid] = base + len(toks)
        for rid in end:
            self._at.pop(rid, None)
        self.steps.append(rec)
        self.wanted.append(want)

    def lines(self):
        return [json.dumps(s) for s in self.steps]


def whole(reqs: dict[str, list[int]]) -> Trace:
    t = Trace()
    for rid, toks in reqs.items():
        t.add([(rid, toks, list(range(len(toks))))], end=[rid])
    return t


def tail_decoded(reqs: dict[str, list[int]], tail: int = 32) -> Trace:
    t = Trace()
    for rid, toks in reqs.items():
        head = max(1, len(toks) - tail)
        t.add([(rid, toks[:head], [head - 1])])
        for i in range(head, len(toks)):
            t.add([(rid, [toks[i]], [0])], end=[rid] if i == len(toks) - 1 else [])
        if head == len(toks):
            t.add([], end=[rid])
    return t


def portions(reqs: dict[str, list[int]], sizes=(7, 2, 16, 3, 2, 5, 33, 2, 1, 17)) -> Trace:
    t = Trace()
    k = 0
    for rid, toks in reqs.items():
        at = 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            last = at + n == len(toks)
            t.add([(rid, toks[at:at + n], list(range(n)))], end=[rid] if last else [])
            at += n
    return t


def mixed(reqs: dict[str, list[int]], prompt_lens: dict[str, int], max_live: int = 4,
          sizes=(5, 2, 9, 16, 3, 2, 11), seed: int = 0) -> Trace:
    """Up to ``max_live`` requests at once: prompts go in as portions of changing size beside
    other requests' single (given) tokens; a request now and then sits a step out."""
    rng = np.random.default_rng(seed)
    t = Trace()
    waiting = list(reqs)
    live: dict[str, int] = {}
    k = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        entries, ended = [], []
        for rid in list(live):
            at, toks = live[rid], reqs[rid]
            if len(live) > 1 and rng.random() < 0.15:
                continue  # left out of this step, goes on later
            if at < prompt_lens[rid]:
                n = min(sizes[k % len(sizes)], prompt_lens[rid] - at)
                k += 1
            else:
                n = 1
            places = list(range(n)) if n > 1 else [0]
            entries.append((rid, toks[at:at + n], places))
            live[rid] = at + n
            if live[rid] == len(toks):
                ended.append(rid)
                del live[rid]
        t.add(entries, end=ended)
    return t


def peak_tokens(trace: Trace, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: dict[str, int] = {}
    peak = 0
    for s in trace.steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def replay(model_dir: str, dtype: str, trace: Trace, out_dir: str, *, max_tokens: int | None = None,
           page_size: int = 16, subprocess_mode: bool = False, cuda_graphs: bool = False,
           stats: dict | None = None) -> dict[int, np.ndarray]:
    max_tokens = max_tokens or peak_tokens(trace)
    os.makedirs(out_dir, exist_ok=True)
    argv = ["--model", model_dir, "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens),
            "--page-size", str(page_size)] + (["--cuda-graphs"] if cuda_graphs else [])
    if subprocess_mode:
        res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), *argv],
                             input="\n".join(trace.lines()) + "\n", text=True, capture_output=True, timeout=900)
        assert res.returncode == 0, res.stderr[-3000:]
        done = [l for l in res.stdout.splitlines() if l.startswith("done ")]
        assert done == [f"done {s['step']}" for s in trace.steps]
    else:
        from rosellm_b200.engine import trace as T

        assert T.run(T.parse_args(argv), trace.lines(), stats) == 0
    out = {}
    for s, want in zip(trace.steps, trace.wanted):
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if want:
            out[s["step"]] = np.fromfile(path, dtype="<f4")
        else:
            assert not os.path.exists(path)
    return out


_plain_cache: dict = {}


def plain_logits(model_dir: str, toks: list[int]) -> torch.Tensor:
    key = (model_dir, tuple(toks))
    if key not in _plain_cache:
        if model_dir not in _plain_cache:
            _plain_cache[model_dir] = P.load_folder(model_dir)
        cfg, t = _plain_cache[model_dir]
        _plain_cache[key] = P.forward(cfg, t, toks)
    return _plain_cache[key]


def bfloat16_noise(model_dir: str, toks: list[int]) -> float:
    """The largest change of a logit of this sequence when the plain implementation rounds its
    activations to bfloat16 where a 16-bit engine stores them: the size of error that 16-bit
    storage alone explains, to which the tests tie the bfloat16 tolerance."""
    key = ("noise", model_dir, tuple(toks))
    if key not in _plain_cache:
        cfg, t = _plain_cache[model_dir]
        rounded = P.forward(cfg, t, toks, rounding=P.to_bfloat16_and_back)
        _plain_cache[key] = float((rounded - plain_logits(model_dir, toks)).abs().max())
    return _plain_cache[key]


def check(model_dir: str, reqs: dict[str, list[int]], trace: Trace, got: dict[int, np.ndarray], atol: float,
          noise_factor: float | None = None) -> float:
    """Every wanted row against the plain implementation; returns the largest difference.

    With ``noise_factor`` (bfloat16 runs) a request's tolerance is that many times the error
    that rounding the plain implementation's activations to bfloat16 causes on the same
    tokens, and at least ``atol``."""
    worst = 0.0
    for s, want in zip(trace.steps, trace.wanted):
        if not want:
            continue
        arr = got[s["step"]]
        vocab = arr.size // len(want)
        arr = torch.from_numpy(arr.reshape(len(want), vocab).astype(np.float64))
        for row, (rid, pos) in enumerate(want):
            ref = plain_logits(model_dir, reqs[rid])[pos]
            diff = float((arr[row] - ref).abs().max())
            limit = atol if noise_factor is None else max(atol, noise_factor * bfloat16_noise(model_dir, reqs[rid]))
            assert np.isfinite(diff) and diff <= limit, (
                f"step {s['step']}: request {rid} position {pos}: |logits - plain| = {diff:.3e} > {limit:.1e} "
                f"(first wrong place of the trace; entries of the step: "
                f"{[(e['id'], len(e['tokens'])) for e in s['entries']]})"
            )
            worst = max(worst, diff)
    return worst
