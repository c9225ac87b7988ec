"""rl_attention_decode_noalloc, the decode attention for callers that cannot allocate device
memory (see rosellm_b200/csrc/attention_noalloc.h), called through its exported C symbol.

Such callers (a plug-in inside a process whose allocator it must leave alone, a runtime that
owns the whole device heap, a loop that cannot afford cudaMalloc's synchronisation) get the
same result as callers of the ordinary entry point, which is handed scratch from outside.
Two calls in a row share the library's scratch array; the second must not be disturbed by
what the first left there.  The results are also checked against a float64 reference, and the
device's free memory is the same after the second call as before it.  This file sorts last so that a run that stops at the first
failure has already run every other test.
"""
import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def c_entry():
    from rosellm_b200.ops import build

    lib = ctypes.CDLL(build.build())
    fn = lib.rl_attention_decode_noalloc
    P, I, L, F = c_void_p, c_int, c_long, c_float
    fn.argtypes = [I, P, L, P, P, I, P, P, P, P, L, I, I, I, I, I, F, P, I, I, P, P]
    fn.restype = I
    lib.rl_attention_decode_noalloc_error.argtypes = [I]
    lib.rl_attention_decode_noalloc_error.restype = ctypes.c_char_p
    return fn, lib.rl_attention_decode_noalloc_error


def case(dtype, lens_kv, n_heads, n_kv, dh, page, seed, window=None):
    g = torch.Generator().manual_seed(seed)
    n_req = len(lens_kv)
    max_pages = max(-(-l // page) for l in lens_kv)
    n_pages = sum(-(-l // page) for l in lens_kv) + 3
    pool = torch.randn(n_pages, 2, n_kv, page, dh, generator=g).to(dtype).to(DEV)
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n_req, max_pages), -1, dtype=torch.int32)
    for r, l in enumerate(lens_kv):
        for p in range(-(-l // page)):
            table[r, p] = perm.pop()
    q = torch.randn(n_req, n_heads * dh, generator=g).to(dtype).to(DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    # float64 reference: softmax(q.k / sqrt(dh)) v over the request's keys, gathered from its pages
    ref = torch.zeros(n_req, n_heads, dh, dtype=torch.float64)
    grp = n_heads // n_kv
    pool64, q64 = pool.double().cpu(), q.double().cpu().view(n_req, n_heads, dh)
    for r, l in enumerate(lens_kv):
        pages = table[r, : -(-l // page)].long()
        k = pool64[pages, 0].permute(0, 2, 1, 3).reshape(-1, n_kv, dh)[:l].repeat_interleave(grp, dim=1)
        v = pool64[pages, 1].permute(0, 2, 1, 3).reshape(-1, n_kv, dh)[:l].repeat_interleave(grp, dim=1)
        lo = 0 if window is None else max(0, l - window)
        sc = torch.einsum("hd,thd->ht", q64[r], k[lo:]) * dh ** -0.5
        ref[r] = torch.einsum("ht,thd->hd", torch.softmax(sc, dim=-1), v[lo:])
    return dict(ref=ref.view(n_req, n_heads * dh), q=q, pool=pool, table=table.to(DEV), q_start=i32(list(range(n_req + 1))), kv_len=i32(lens_kv),
                slots=i32(list(range(n_req))), decode_reqs=i32(list(range(n_req))), n_heads=n_heads, n_kv=n_kv,
                dh=dh, page=page)


def ordinary(c, n_splits, window):
    """The existing entry point, with scratch allocated by the caller (torch)."""
    from rosellm_b200.ops import kernels as K

    n = c["q"].shape[0]
    out = torch.zeros_like(c["q"])
    part_o = torch.empty(n * c["n_heads"] * n_splits * c["dh"], device=DEV)
    part_ml = torch.empty(n * c["n_heads"] * n_splits * 2, device=DEV)
    K.attention(c["q"], c["pool"], c["table"], c["q_start"], c["kv_len"], c["slots"], out, n_heads=c["n_heads"],
                scale=c["dh"] ** -0.5, window=window, tiles=None, n_tiles=0, decode_reqs=c["decode_reqs"],
                n_decode=n, n_splits=n_splits, part_o=part_o, part_ml=part_ml)
    return out


def no_alloc(fn, c, n_splits, window, status, out=None):
    n = c["q"].shape[0]
    out = torch.zeros_like(c["q"]) if out is None else out
    code = 0 if c["q"].dtype == torch.float32 else 1
    rc = fn(code, c["q"].data_ptr(), c["q"].stride(0), c["pool"].data_ptr(), c["table"].data_ptr(),
            c["table"].stride(0), c["q_start"].data_ptr(), c["kv_len"].data_ptr(), c["slots"].data_ptr(),
            out.data_ptr(), out.stride(0), c["n_heads"], c["n_kv"], c["dh"], c["page"], window or 0,
            c["dh"] ** -0.5, c["decode_reqs"].data_ptr(), n, n_splits, None if status is None else status.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    return rc, out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_calls_in_a_row_match_the_ordinary_entry_point(dtype):
    fn, _ = c_entry()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    first = case(dtype, [700, 33, 129, 1], 6, 2, 64, 16, seed=1)
    second = case(dtype, [64, 300], 4, 4, 32, 8, seed=2, window=100)  # other sizes over the first call's leftovers
    wants = [ordinary(c, splits, window) for c, splits, window in ((first, 5, None), (second, 8, 100))]
    torch.cuda.synchronize()
    free_before = None
    for i, (c, splits, window) in enumerate(((first, 5, None), (second, 8, 100))):
        out = torch.zeros_like(c["q"])  # the caller's output, made before free memory is read
        if i == 1:
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
        rc, got = no_alloc(fn, c, splits, window, status, out)
        assert rc == 0
        torch.cuda.synchronize()
        if i == 1:  # the second call took no device memory (the first looked up the scratch's address)
            assert torch.cuda.mem_get_info()[0] == free_before
        assert int(status.item()) == 0
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float(), wants[i].float(), **tol)
        torch.testing.assert_close(got.double().cpu(), c["ref"], **tol)


def test_sizes_beyond_the_scratch_are_refused_with_a_reason():
    fn, why = c_entry()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    c = case(torch.float32, [40] * 8, 64, 64, 128, 16, seed=3)
    rc, out = no_alloc(fn, c, 32, None, status)  # 8 * 64 * 32 * 130 floats > 2^20
    assert rc == -5 and b"scratch" in why(rc)
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0  # nothing was launched
    rc, _ = no_alloc(fn, dict(c, dh=24), 1, None, status)
    assert rc == -2 and b"multiple of 16" in why(rc)
    rc, _ = no_alloc(fn, c, 70000, None, status)
    assert rc == -4 and b"65535" in why(rc)
    rc, out = no_alloc(fn, c, 2, None, None)  # no status word: refused, not dereferenced
    assert rc == -7 and b"status" in why(rc)
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0


def test_one_split_needs_no_scratch_however_large_the_batch():
    """256 requests x 64 heads x 128: far beyond the scratch if it were used, but a single split
    writes straight to the output."""
    fn, _ = c_entry()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    c = case(torch.bfloat16, [33] * 256, 64, 8, 128, 16, seed=4)
    assert 256 * 64 * 130 > (1 << 20)
    rc, got = no_alloc(fn, c, 1, None, status)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    torch.testing.assert_close(got.double().cpu(), c["ref"], atol=2e-2, rtol=2e-2)
