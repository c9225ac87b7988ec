"""Times one kernel of the library by itself, with CUDA events, after warm-up.

    python -m rosellm_b200.ops.microbench --op linear --rows 8 --n 2304 --k 768
    python -m rosellm_b200.ops.microbench --op attention-decode --batch 64 --context 512
    python -m rosellm_b200.ops.microbench --op attention-prefill --batch 2 --context 1024
    python -m rosellm_b200.ops.microbench --op layernorm --rows 8 --k 768
    python -m rosellm_b200.ops.microbench --op sample --rows 8 --n 50257
    python -m rosellm_b200.ops.microbench --op decode-layer --batch 64 --context 512 --k 768 --n 3072
    python -m rosellm_b200.ops.microbench --op prefill-layer --batch 2 --context 1024 --k 768 --n 3072
    python -m rosellm_b200.ops.microbench --op mlp --rows 8 --k 768 --n 3072 [--unfused] [--slice 32]

The two layer operations run the engine's own parts (``PreNormBlock.forward`` over attention,
feed-forward and norms bound to random weights), so what they time is the engine's order and
choice of kernels by construction.

Every timed launch works on operands other than the launch before it (a ring of copies
larger than the 126 MB L2), so weights and cache come from memory as they do inside a step.
Prints one JSON line with the time per launch and the achieved bytes/s and flop/s.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..engine.context import build_host_batch
from . import kernels as K

L2_BYTES = 126 * 1024 * 1024


def _ring(make, nbytes: int) -> list:
    """Enough copies of an operand that a pass over them exceeds L2."""
    n = max(2, min(64, -(-2 * L2_BYTES // max(nbytes, 1))))
    return [make() for _ in range(n)]


def _time(fn, reps: int, warmup: int = 5, graph: bool = True) -> float:
    """Microseconds per launch.  With ``graph`` the launches are captured once and replayed,
    as the engine replays a decode step: the host's launch cost is then not in the number."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(reps):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
    else:
        e0.record()
        for i in range(reps):
            fn(i)
        e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def _decode_plan(a, n_decode: int, heads: int, head_dim: int) -> tuple[int, bool]:
    """(parts of a request's keys, wide blocks): as given by --splits and --wide, else as the
    attention part plans a decode step of this many requests and this context."""
    if a.splits or a.wide:
        return max(1, a.splits), a.wide
    from ..parts.standard import CausalSelfAttention

    return CausalSelfAttention(heads * head_dim, heads, head_dim).decode_plan_for(n_decode, a.context)


ATTENTION_PHASES = ["start", "copies issued", "kernels ahead done", "rows normalised", "weights arrived", "qkv product",
                    "bias, cache write, to peers", "cluster barrier 1", "attention", "warps' parts written",
                    "block's parts to peers", "cluster barrier 2", "cluster's parts merged", "output product",
                    "all blocks have read", "added"]
MLP_PHASES = ["start", "copies issued", "kernels ahead done", "rows normalised", "weights arrived", "first product",
              "bias, activation", "second product", "all blocks have read", "added"]


GEMM_PHASES = ["start", "barriers, tensor memory", "kernels ahead done", "first copy issued", "a tile's copies issued",
               "a tile's products issued", "accumulator complete", "tile written", "end", "-"] + \
              [f"K block {i} arrived" for i in range(16)] + \
              ["every block has its sums", "pieces sent to their owners", "every block has sent"]


PROMPT_ATTENTION_PHASES = ["start", "barriers, tensor memory", "kernels ahead done", "tile 0's copies issued",
                           "tile 1's copies issued", "tile 2's copies issued", "queries and tile 0 arrived",
                           "last P V taken", "end", "-"] + \
                          [f"probabilities of tile {t} ready" for t in range(6)] + \
                          [f"tile {t}: {what}" for t in range(4)
                           for what in ("scores arrived", "row maximum agreed", "probabilities handed over", "P V before taken")]


def _print_phases() -> None:
    """The phases of the last launch of each fused decode kernel (one block's thread 0), in ns at 1.9 GHz."""
    import ctypes

    for title, names, reader in (("attention half", ATTENTION_PHASES, "rl_attn_block_fused_phase_times"),
                                 ("feed-forward", MLP_PHASES, "rl_mlp_fused_phase_times"),
                                 ("tcgen05 product", GEMM_PHASES, "rl_gemm_tc_phase_times"),
                                 ("tcgen05 prompt attention", PROMPT_ATTENTION_PHASES, "rl_attention_phase_times")):
        buf = (ctypes.c_longlong * 32)()
        fn = getattr(K._lib(), reader)
        fn.argtypes = [ctypes.c_void_p, ctypes.c_int]
        fn(ctypes.cast(buf, ctypes.c_void_p), len(names))
        v = list(buf)[:len(names)]
        if not any(v):
            continue
        print(title)
        for i in range(1, len(names)):
            if v[i]:
                print(f"  {names[i]:>24}: +{(v[i] - v[i - 1]) / 1.9:7.0f} ns   (at {(v[i] - v[0]) / 1.9:7.0f})")


class _RingCache:
    """Pages and one block table for a ring of layers, with the face of the cache manager that
    the parts use."""

    def __init__(self, pools: list, table, max_seq_len: int, device) -> None:
        self.pools, self.table, self.max_seq_len, self.device = pools, table, max_seq_len, device

    def kv_pool(self, key):
        return self.pools[key]

    def block_table(self, key):
        return self.table

    def state(self, key):
        raise KeyError(key)


def _layer_ring(a, dev, dt, entries):
    """A ring of pre-norm layers of the engine's own parts, more than L2 holds, with a step
    context over ``entries`` (as ``build_host_batch`` takes them); request r uses slot r and
    the pages r * pages-per-sequence onwards."""
    from ..engine.context import standalone_context
    from ..models.model import Layer
    from ..parts.spec import RunEntry
    from ..parts.standard import CausalSelfAttention, DenseMLP, LayerNorm, NoPositions, PreNormBlock

    h, dh, ps, hid, inner = a.heads, a.head_dim, a.page_size, a.k, a.n
    hk = a.kv_heads or h
    el = 2 if dt == torch.bfloat16 else 4
    n_req = len(entries)
    longest = max(e[1] + len(e[2]) for e in entries)
    per_seq = -(-longest // ps)
    n_pages = n_req * per_seq
    layer_bytes = ((h + 2 * hk) * dh * hid + hid * hid + 2 * hid * inner) * el + n_pages * 2 * hk * ps * dh * el
    n_layers = max(2, min(64, -(-2 * L2_BYTES // layer_bytes)))
    w = lambda *shape: (torch.randn(*shape, device=dev) * 0.02).to(dt)
    vec = lambda n: torch.randn(n, device=dev) * 0.02
    ring, pools = [], []
    for i in range(n_layers):
        mixer = CausalSelfAttention(hid, h, dh, hk)
        mixer.bind({"qkv_weight": w((h + 2 * hk) * dh, hid), "qkv_bias": vec((h + 2 * hk) * dh),
                    "out_weight": w(hid, h * dh), "out_bias": vec(hid)})
        ff = DenseMLP(hid, inner, "gelu_tanh")
        ff.bind({"in_weight": w(inner, hid), "in_bias": vec(inner), "out_weight": w(hid, inner), "out_bias": vec(hid)})
        norms = []
        for _ in range(2):
            n = LayerNorm(hid, 1e-5)
            n.bind({"weight": 1 + vec(hid), "bias": vec(hid)})
            norms.append(n)
        parts = {"mixer": mixer, "feed_forward": ff, "norm_mixer": norms[0], "norm_feed_forward": norms[1]}
        ring.append((RunEntry(i), Layer(PreNormBlock(), parts, {})))
        pools.append(torch.randn(n_pages, 2, hk, ps, dh, device=dev).to(dt))
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(n_req, per_seq)
    cache = _RingCache(pools, table, per_seq * ps, dev)
    ctx = standalone_context(cache, entries, dt)
    ctx.position = NoPositions()
    x = torch.randn(len(ctx.host.token_ids), hid, device=dev)
    return ring, ctx, x, layer_bytes


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--op", required=True, choices=["linear", "attention-decode", "attention-prefill", "layernorm", "sample", "head", "decode-layer", "prefill-layer", "mlp"])
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--rows", type=int, default=8)
    p.add_argument("--n", type=int, default=2304)
    p.add_argument("--k", type=int, default=768)
    p.add_argument("--path", default=None, choices=["rows", "tile", "mma", "tc", "tcr", "smem", "library"],
                   help="linear: the kernel to force; 'library' times torch.mm on the same shape (no bias, no "
                        "activation) as a yardstick of what the shape allows")
    p.add_argument("--act", default="none", choices=sorted(K.ACTIVATIONS))
    p.add_argument("--residual", action="store_true")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=512)
    p.add_argument("--heads", type=int, default=12)
    p.add_argument("--kv-heads", type=int, default=None)
    p.add_argument("--head-dim", type=int, default=64)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--splits", type=int, default=0, help="0: as the engine chooses (with --wide: 1)")
    p.add_argument("--wide", action="store_true", help="decode attention: blocks of sixteen warps instead of four")
    p.add_argument("--reps", type=int, default=50)
    p.add_argument("--temperature", type=float, default=0.0, help="sample: 0 takes the largest logit")
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--slice", type=int, default=0, help="mlp: slice of the inner width a block takes (0: as the library chooses)")
    p.add_argument("--unfused", action="store_true",
                   help="decode-layer: the fused kernels of few rows switched off (every product a kernel of its own)")
    p.add_argument("--phases", action="store_true",
                   help="print the clock stamps of the fused decode kernels' phases (a library built with "
                        "ROSELLM_B200_NVCC_EXTRA=-DRL_PHASE_TIMING; all zero otherwise)")
    p.add_argument("--tile-width", type=int, default=0, help="linear on tcgen05 tiles: the columns of a tile (0: chosen)")
    p.add_argument("--k-parts", type=int, default=0, help="linear on tcgen05 tiles: the parts of the inner size (0: chosen)")
    p.add_argument("--eager", action="store_true", help="launch from the host each time instead of replaying a graph")
    p.add_argument("--no-bulk-copies", action="store_true",
                   help="heads of few rows on the weight-streaming kernel instead of the one fed by bulk copies")
    a = p.parse_args(argv)
    dev = torch.device("cuda:0")
    if a.no_bulk_copies:
        K.rows_bulk_kernel(False)
    dt = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    el = 2 if dt == torch.bfloat16 else 4
    rec: dict = {"op": a.op, "dtype": a.dtype}
    if a.op == "linear":
        m, n, k = a.rows, a.n, a.k
        ws = _ring(lambda: torch.randn(n, k, device=dev).to(dt), n * k * el)
        x = torch.randn(m, k, device=dev).to(dt)
        bias = torch.zeros(n, device=dev)
        out = torch.zeros(m, n, device=dev, dtype=torch.float32 if a.residual else dt)
        act = K.ACTIVATIONS[a.act]
        if a.path == "library":
            lib_out = torch.empty(m, n, device=dev, dtype=dt)
            us = _time(lambda i: torch.mm(x, ws[i % len(ws)].t(), out=lib_out), a.reps, graph=not a.eager)
        else:
            us = _time(lambda i: K.linear(x, ws[i % len(ws)], bias, out, act=act, residual=a.residual, path=a.path,
                                            tile_width=a.tile_width, splits=a.k_parts), a.reps, graph=not a.eager)
        nbytes = n * k * el + m * k * el + m * n * (4 if a.residual else el) * (2 if a.residual else 1)
        rec.update(rows=m, n=n, k=k, path=a.path or "auto", us=round(us, 2), gbytes_per_s=round(nbytes / us / 1e3, 1),
                   tflops=round(2 * m * n * k / us / 1e6, 2))
    elif a.op == "mlp":
        # the feed-forward of few rows: LayerNorm, product, activation, product, += residual;
        # one fused kernel, or (--unfused) the two products
        m, hid, inner = a.rows, a.k, a.n
        width = a.slice or K.mlp_fused_slice(m, hid, inner, True, dt)

        def mk():
            w1, w2 = (torch.randn(inner, hid, device=dev) * 0.02).to(dt), (torch.randn(hid, inner, device=dev) * 0.02).to(dt)
            return w1, w2, (K.mlp_pack_out_weight(w2, width) if width and not a.unfused else None)

        ws = _ring(mk, 2 * hid * inner * el)
        x = torch.randn(m, hid, device=dev)
        g, b = torch.ones(hid, device=dev), torch.zeros(hid, device=dev)
        b1, b2 = torch.zeros(inner, device=dev), torch.zeros(hid, device=dev)
        mid = torch.empty(m, inner, device=dev, dtype=dt)
        act = K.ACT_GELU_TANH

        def run(i):
            w1, w2, w2p = ws[i % len(ws)]
            if a.unfused or not width:
                K.linear(K.NormInput(x, g, b, 1e-5), w1, b1, mid, act=act)
                K.linear(mid, w2, b2, x, residual=True)
            else:
                K.mlp_fused(x, K.NormInput(x, g, b, 1e-5), w1, b1, w2p, b2, act=act, slice_width=width)

        us = _time(run, a.reps, graph=not a.eager)
        rec.update(rows=m, hidden=hid, inner=inner, slice=0 if a.unfused else width, us=round(us, 2),
                   gbytes_per_s=round(2 * hid * inner * el / us / 1e3, 1))
    elif a.op == "layernorm":
        x = torch.randn(a.rows, a.k, device=dev)
        g, b = torch.ones(a.k, device=dev), torch.zeros(a.k, device=dev)
        out = torch.empty(a.rows, a.k, device=dev, dtype=dt)
        us = _time(lambda i: K.layernorm(x, g, b, 1e-5, out), a.reps, graph=not a.eager)
        rec.update(rows=a.rows, k=a.k, us=round(us, 2), gbytes_per_s=round(a.rows * a.k * (4 + el) / us / 1e3, 1))
    elif a.op == "sample":
        ls = _ring(lambda: torch.randn(a.rows, a.n, device=dev), a.rows * a.n * 4)
        ids = torch.empty(a.rows, dtype=torch.int32, device=dev)
        if a.temperature > 0:
            f = lambda v, t: torch.full((a.rows,), v, dtype=t, device=dev)
            par = (f(a.temperature, torch.float32), f(a.top_k, torch.int32), f(a.top_p, torch.float32),
                   torch.arange(a.rows, dtype=torch.int64, device=dev), f(0, torch.int32))
        else:
            par = (None,) * 5
        us = _time(lambda i: K.sample(ls[i % len(ls)], *par, ids), a.reps, graph=not a.eager)
        rec.update(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p)
        rec.update(rows=a.rows, n=a.n, us=round(us, 2), gbytes_per_s=round(a.rows * a.n * 4 / us / 1e3, 1))
    elif a.op == "head":
        # a head's product and the choice of the next tokens: logits written and read back by the
        # sampling kernel (--unfused), or the choice inside the product; --n is the vocabulary
        ws = _ring(lambda: torch.randn(a.n, a.k, device=dev).to(dt), a.n * a.k * el)
        x = torch.randn(a.rows, a.k, device=dev).to(dt)
        ids = torch.empty(a.rows, dtype=torch.int32, device=dev)
        logits = torch.empty(a.rows, a.n, device=dev)
        par = (None,) * 3
        if a.temperature > 0:
            par = (torch.full((a.rows,), a.temperature, device=dev), torch.arange(a.rows, dtype=torch.int64, device=dev),
                   torch.zeros(a.rows, dtype=torch.int32, device=dev))
        into = K.SampleInto(ids, *par)

        def run(i):
            if a.unfused:
                K.linear(x, ws[i % len(ws)], None, logits)
                K.sample(logits, par[0], None, None, par[1], par[2], ids)
            else:
                K.linear_sample(x, ws[i % len(ws)], None, into)

        us = _time(run, a.reps, graph=not a.eager)
        rec.update(rows=a.rows, n=a.n, k=a.k, temperature=a.temperature, in_product=not a.unfused, us=round(us, 2),
                   gbytes_per_s=round(a.n * a.k * el / us / 1e3, 1))
    elif a.op == "prefill-layer":
        # one layer of a prompt step run by the engine's own parts: --batch prompts of --context tokens
        h, dh, hid, inner = a.heads, a.head_dim, a.k, a.n
        rows = a.batch * a.context
        assert h * dh == hid
        ring, ctx, x, _ = _layer_ring(a, dev, dt, [(r, 0, [0] * a.context, []) for r in range(a.batch)])

        def layer(i):
            run, parts = ring[i % len(ring)]
            parts.block.forward(ctx, run, parts, x)

        us = _time(layer, a.reps, graph=not a.eager)
        flops = 2 * rows * (4 * hid * hid + 2 * hid * inner) + 4 * a.batch * h * dh * a.context * a.context // 2
        rec.update(batch=a.batch, context=a.context, hidden=hid, inner=inner, us=round(us, 2),
                   tflops=round(flops / us / 1e6, 1))
    elif a.op == "decode-layer":
        # one layer of a decode step, run by the engine's own parts (``PreNormBlock.forward`` over
        # attention, feed-forward and norms bound to random weights): the order and choice of
        # kernels is the engine's by construction.  Hidden size --k, inner size --n, --batch
        # requests at --context cached tokens; every timed layer has weights and pages of its own.
        h, dh, hid, inner, rows = a.heads, a.head_dim, a.k, a.n, a.batch
        assert h * dh == hid
        ring, ctx, x, layer_bytes = _layer_ring(a, dev, dt, [(r, a.context - 1, [0], []) for r in range(rows)])
        K.FUSED_ROWS = not a.unfused
        if a.splits or a.wide:
            ctx.extras["decode_plan"] = (max(1, a.splits), a.wide)

        def layer(i):
            run, parts = ring[i % len(ring)]
            parts.block.forward(ctx, run, parts, x)

        us = _time(layer, a.reps, graph=not a.eager)
        rec.update(batch=rows, context=a.context, hidden=hid, inner=inner, fused=not a.unfused,
                   plan=ctx.extras.get("decode_plan"), us=round(us, 2), gbytes_per_s=round(layer_bytes / us / 1e3, 1))
    else:
        h, hk, dh, ps = a.heads, a.kv_heads or a.heads, a.head_dim, a.page_size
        decode = a.op == "attention-decode"
        q_len = 1 if decode else a.context
        per_seq = -(-a.context // ps)
        n_pages = a.batch * per_seq
        pools = _ring(lambda: torch.randn(n_pages, 2, hk, ps, dh, device=dev).to(dt), n_pages * 2 * hk * ps * dh * el)
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(a.batch, per_seq)
        hb = build_host_batch([(r, a.context - q_len, [0] * q_len, []) for r in range(a.batch)])
        i32 = lambda arr: torch.as_tensor(arr, dtype=torch.int32).contiguous().to(dev)
        n_tok = a.batch * q_len
        q = torch.randn(n_tok, h * dh, device=dev).to(dt)
        out = torch.empty_like(q)
        splits, wide = _decode_plan(a, a.batch, h, dh) if decode else (1, False)
        po = torch.empty(max(1, a.batch * h * splits * dh), device=dev)
        pm = torch.empty(max(1, a.batch * h * splits * 2), device=dev)
        args = dict(n_heads=h, scale=dh ** -0.5, window=None, tiles=i32(hb.tiles.reshape(-1)), n_tiles=len(hb.tiles),
                    decode_reqs=i32(hb.decode_reqs), n_decode=len(hb.decode_reqs), n_splits=splits, part_o=po,
                    part_ml=pm, tiles_wide=i32(hb.tiles_wide.reshape(-1)), n_tiles_wide=len(hb.tiles_wide),
                    decode_wide=wide, old_keys_settled=True)  # as inside the engine: the cache is of earlier steps
        qs, kl, sl = i32(hb.q_start), i32(hb.kv_len), i32(hb.slots)
        us = _time(lambda i: K.attention(q, pools[i % len(pools)], table, qs, kl, sl, out, **args), a.reps, graph=not a.eager)
        kv_bytes = a.batch * a.context * 2 * hk * dh * el
        flops = 4 * a.batch * h * dh * (a.context if decode else a.context * a.context // 2)
        rec.update(batch=a.batch, context=a.context, heads=h, kv_heads=hk, head_dim=dh, splits=splits, us=round(us, 2),
                   gbytes_per_s=round(kv_bytes / us / 1e3, 1), tflops=round(flops / us / 1e6, 2))
    K.check_status(dev)
    print(json.dumps(rec))
    if a.phases:
        _print_phases()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
