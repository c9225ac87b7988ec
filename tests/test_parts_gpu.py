"""Each shipped part alone, built from its own parameters at sizes no model here uses,
against the plain functions."""
import numpy as np
import pytest
import torch

import plain_gpt2 as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def tol(dtype):
    return dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)


def bind_random(part, dtype, seed=0, scale=0.3):
    """Random tensors for every declared role, as the loader would hand them over."""
    from rosellm_b200.weights.loader import to_device_tensor

    g = torch.Generator().manual_seed(seed)
    files = {}
    for spec in part.param_specs():
        t = torch.randn(spec.shape, generator=g) * scale
        if spec.init == "ones":
            t = t + 1.0
        t = t.to(torch.bfloat16).float() if spec.kind == "matrix" else t
        files[spec.role] = t
    part.bind({s.role: to_device_tensor(files[s.role], s, dtype, DEV) for s in part.param_specs()})
    return {k: v.double() for k, v in files.items()}


def make_cache(kv_specs, page=8, pages=64, slots=4, seq=256, dtype=torch.float32, state=None):
    from rosellm_b200.cache import CacheManager

    return CacheManager(kv_specs, state or {}, page_size=page, num_pages=pages, max_slots=slots, max_seq_len=seq,
                        dtype=dtype, device=DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_and_without_positions(dtype):
    from rosellm_b200.engine.context import standalone_context
    from rosellm_b200.parts.standard import LearnedAbsolutePositions, NoPositions, TokenEmbedding

    emb, pos = TokenEmbedding(vocab_size=77, hidden_size=48), LearnedAbsolutePositions(max_positions=40, hidden_size=48)
    we, wp = bind_random(emb, dtype, 1), bind_random(pos, dtype, 2)
    cache = make_cache({})
    s0, s1 = cache.new_request(), cache.new_request()
    ctx = standalone_context(cache, [(s0, 5, [3, 76, 0], []), (s1, 0, [10], [])], dtype)
    x = emb.forward(ctx, pos).double().cpu()
    ids, where = torch.tensor([3, 76, 0, 10]), torch.tensor([5, 6, 7, 0])
    torch.testing.assert_close(x, we["weight"][ids] + wp["weight"][where], atol=1e-6, rtol=0)
    x2 = emb.forward(ctx, NoPositions()).double().cpu()
    torch.testing.assert_close(x2, we["weight"][ids], atol=1e-6, rtol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_part(dtype):
    from rosellm_b200.engine.context import standalone_context
    from rosellm_b200.parts.standard import LayerNorm

    norm = LayerNorm(hidden_size=80, eps=3e-4)
    w = bind_random(norm, dtype, 3)
    cache = make_cache({})
    ctx = standalone_context(cache, [(cache.new_request(), 0, [0] * 11, [])], dtype)
    x = torch.randn(11, 80, generator=torch.Generator().manual_seed(4)) * 2 + 1
    h = norm.forward(ctx, x.to(DEV)).double().cpu()
    torch.testing.assert_close(h, P.layer_norm(x.double(), w["weight"], w["bias"], 3e-4), **tol(dtype))
    nobias = LayerNorm(hidden_size=80, eps=3e-4, bias=False)
    w2 = bind_random(nobias, dtype, 5)
    h2 = nobias.forward(ctx, x.to(DEV)).double().cpu()
    torch.testing.assert_close(h2, P.layer_norm(x.double(), w2["weight"], torch.zeros(80, dtype=torch.float64), 3e-4), **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("activation,fn", [("gelu_tanh", P.gelu_tanh), ("gelu_erf", P.gelu_erf)])
@pytest.mark.parametrize("in_out", [True, False])
@pytest.mark.parametrize("inner", [136, 77])  # 77: no multiple of 8, filled up with idle units
def test_dense_mlp_part(dtype, activation, fn, in_out, inner):
    from rosellm_b200.engine.context import standalone_context
    from rosellm_b200.parts.standard import DenseMLP

    mlp = DenseMLP(hidden_size=48, inner_size=inner, activation=activation, weights_in_out=in_out)
    w = bind_random(mlp, dtype, 6)
    cache = make_cache({})
    ctx = standalone_context(cache, [(cache.new_request(), 0, [0] * 70, [])], dtype)
    g = torch.Generator().manual_seed(7)
    h = torch.randn(70, 48, generator=g).to(dtype)
    x = torch.randn(70, 48, generator=g)
    xd = x.to(DEV)
    mlp.forward(ctx, h.to(DEV), xd)
    wi, wo = (w["in_weight"], w["out_weight"]) if in_out else (w["in_weight"].t(), w["out_weight"].t())
    want = x.double() + P.mlp(h.double(), wi, w["in_bias"], wo, w["out_bias"], fn)
    torch.testing.assert_close(xd.double().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dh,window", [(3, 3, 32, None), (6, 2, 16, None), (4, 1, 48, 9)])
def test_attention_part_in_portions_against_whole(dtype, heads, kv_heads, dh, window):
    """The mixer over a cache it fills in three steps (a portion, a single token, a portion)
    equals plain attention over the whole sequence."""
    from rosellm_b200.engine.context import standalone_context
    from rosellm_b200.parts.spec import RunEntry
    from rosellm_b200.parts.standard import CausalSelfAttention, NoPositions

    hidden = 40
    att = CausalSelfAttention(hidden_size=hidden, num_heads=heads, head_dim=dh, num_kv_heads=kv_heads, window=window)
    # weights of this size give attention scores of order one; with much larger ones the scores
    # themselves (tens) lose whole units to bfloat16 rounding of queries and keys
    w = bind_random(att, dtype, 8, scale=0.15)
    cache = make_cache({0: att.cache_spec()}, page=8, dtype=dtype)
    slot = cache.new_request()
    T = 45
    g = torch.Generator().manual_seed(9)
    h_all = torch.randn(T, hidden, generator=g).to(dtype)
    x_all = torch.zeros(T, hidden)
    got = []
    at = 0
    for n in (20, 1, 24):
        assert cache.reserve(slot, n)
        cache.sync_to_device()
        ctx = standalone_context(cache, [(slot, at, [0] * n, [])], dtype)
        ctx.position = NoPositions()
        x = torch.zeros(n, hidden, device=DEV)
        att.forward(ctx, RunEntry(0), h_all[at:at + n].to(DEV), x)
        got.append(x.double().cpu())
        cache.commit(slot, n)
        at += n
    # plain: grouped heads spelled out
    hd = h_all.double()
    qkv = hd @ w["qkv_weight"].t() + w["qkv_bias"]
    q, k, v = qkv.split([heads * dh, kv_heads * dh, kv_heads * dh], dim=-1)
    q = q.view(T, heads, dh)
    k = k.view(T, kv_heads, dh).repeat_interleave(heads // kv_heads, dim=1)
    v = v.view(T, kv_heads, dh).repeat_interleave(heads // kv_heads, dim=1)
    s = torch.einsum("thd,shd->hts", q, k) * dh ** -0.5
    i = torch.arange(T)
    vis = i[None, :] <= i[:, None]
    if window is not None:
        vis &= i[None, :] > i[:, None] - window
    o = torch.einsum("hts,shd->thd", torch.softmax(s.masked_fill(~vis, float("-inf")), -1), v).reshape(T, heads * dh)
    want = o @ w["out_weight"].t() + w["out_bias"]
    # the largest error against the largest output: bfloat16 rounds the queries, keys, values
    # and the merged heads to 8 bits of mantissa (relative step 2^-8) before the last product
    err, size = float((torch.cat(got) - want).abs().max()), float(want.abs().max())
    assert err <= (2.0 ** -7 if dtype == torch.bfloat16 else 1e-5) * size, f"error {err:.3e} on outputs up to {size:.3f}"
    if window is not None:
        assert len(cache.pages_of(slot)) <= -(-window // 8) + 1  # pages behind the window went back


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_heads_tied_and_linear(dtype):
    from rosellm_b200.engine.context import standalone_context
    from rosellm_b200.parts.standard import LinearHead, TiedHead, TokenEmbedding

    emb = TokenEmbedding(vocab_size=203, hidden_size=48)
    we = bind_random(emb, dtype, 10)
    tied = TiedHead(vocab_size=203, hidden_size=48)
    tied.weight = emb.weight
    own = LinearHead(vocab_size=203, hidden_size=48)
    wo = bind_random(own, dtype, 11)
    cache = make_cache({})
    ctx = standalone_context(cache, [(cache.new_request(), 0, [0] * 5, [])], dtype)
    h = torch.randn(5, 48, generator=torch.Generator().manual_seed(12)).to(dtype)
    t32 = dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=2e-3, rtol=2e-3)
    out = tied.forward(ctx, h.to(DEV))
    assert out.dtype == torch.float32
    torch.testing.assert_close(out.double().cpu(), h.double() @ we["weight"].t(), **t32)
    torch.testing.assert_close(own.forward(ctx, h.to(DEV)).double().cpu(), h.double() @ wo["weight"].t(), **t32)


def test_parts_refuse_sizes_the_kernels_cannot_take():
    from rosellm_b200.parts.standard import CausalSelfAttention, DenseMLP

    with pytest.raises(ValueError, match="multiples of 16"):
        CausalSelfAttention(hidden_size=40, num_heads=2, head_dim=20)
    with pytest.raises(ValueError, match="multiple"):
        CausalSelfAttention(hidden_size=64, num_heads=4, head_dim=16, num_kv_heads=3)
    with pytest.raises(ValueError, match="activation"):
        DenseMLP(hidden_size=8, inner_size=8, activation="relu")


@pytest.mark.parametrize("hidden,heads,dh,page", [(64, 4, 16, 16), (96, 3, 32, 8), (768, 12, 64, 16), (256, 2, 128, 32),
                                                   (1024, 16, 64, 64), (128, 2, 64, 4)])
@pytest.mark.parametrize("lens", [[0], [511, 64, 1], [5, 0, 17, 33, 100, 7, 64, 65], [3] * 16, [300, 40, 129, 16, 15]])
def test_decode_step_of_few_requests_in_one_kernel(hidden, heads, dh, page, lens):
    """A step in which every request brings one token runs norm, qkv product, cache write,
    attention and output product of the layer in one kernel (bfloat16, up to 16 requests).
    Requests with 0 to 511 cached keys (shares of keys that end inside a tile, a first token with
    nothing cached), a padding row, pages that are used again: against float64, and the keys and
    values it wrote against those the separate kernels write."""
    from rosellm_b200.engine.context import standalone_context
    from rosellm_b200.ops import kernels as K
    from rosellm_b200.parts.spec import RunEntry
    from rosellm_b200.parts.standard import CausalSelfAttention, LayerNorm, NoPositions

    dtype = torch.bfloat16
    att = CausalSelfAttention(hidden_size=hidden, num_heads=heads, head_dim=dh)
    norm = LayerNorm(hidden_size=hidden, eps=1e-5)
    w = bind_random(att, dtype, 8, scale=0.6 / hidden ** 0.5)
    wn = bind_random(norm, dtype, 9, scale=0.2)
    n_req = len(lens)
    if not K.attn_block_fused_fits(n_req, hidden, heads, dh, dtype):
        # the blocks of the kernel wait for one another, so all of its clusters (one a head) must
        # run at once; sixteen clusters of eight are more than this device holds
        assert (hidden, heads) == (1024, 16)
        pytest.skip("the device does not hold a cluster for every head at once")
    cache = make_cache({0: att.cache_spec()}, page=page, pages=-(-sum(lens) // page) + 2 * n_req + 2, slots=n_req + 1,
                       seq=640, dtype=dtype)
    g = torch.Generator().manual_seed(sum(lens) + hidden)
    xs = [torch.randn(n + 1, hidden, generator=g) * 1.5 + 0.3 for n in lens]  # the residual rows of every token
    slots = [cache.new_request() for _ in lens]
    # the cached keys and values: each request's earlier tokens as one portion through the separate kernels
    for r, n in enumerate(lens):
        if n == 0:
            continue
        assert cache.reserve(slots[r], n)
        cache.sync_to_device()
        ctx = standalone_context(cache, [(slots[r], 0, [0] * n, [])], dtype)
        ctx.position = NoPositions()
        x = xs[r][:n].to(DEV)
        att.forward(ctx, RunEntry(0), norm.forward(ctx, x), x)
        cache.commit(slots[r], n)
    for r in range(n_req):
        assert cache.reserve(slots[r], 1)
    cache.sync_to_device()
    entries = [(slots[r], lens[r], [0], []) for r in range(n_req)]
    pad = n_req < 16 and n_req > 1
    if pad:
        entries.insert(1, (-1, 0, [0], []))  # a padding row of a fixed-size batch
    rows = torch.stack([xs[r][-1] for r in range(n_req)])
    if pad:
        rows = torch.cat([rows[:1], torch.randn(1, hidden, generator=g), rows[1:]])
    calls = []
    real = K.attn_block_fused
    K.attn_block_fused = lambda *a, **k: (calls.append(1), real(*a, **k))[1]
    try:
        results = []
        for fused in (False, True):
            K.FUSED_ROWS = fused
            pool_before = cache.kv_pool(0).clone()
            ctx = standalone_context(cache, entries, dtype)
            ctx.position = NoPositions()
            x = rows.clone().to(DEV)
            att.forward(ctx, RunEntry(0), norm.forward(ctx, x, defer=True), x)
            K.check_status(DEV)
            results.append((x.double().cpu(), cache.kv_pool(0).clone()))
            untouched = cache.kv_pool(0) == pool_before  # (of the second run: compared below)
            cache.kv_pool(0).copy_(pool_before)
    finally:
        K.attn_block_fused = real
        K.FUSED_ROWS = True
    assert len(calls) == 1  # the second run took the one kernel
    (x_sep, pool_sep), (x_one, pool_one) = results
    # the same keys and values in the same places (the two paths sum over the width in different
    # orders, so a value may round to the neighbouring bfloat16), nothing else touched
    changed = pool_sep != pool_before
    assert int(changed.sum()) > 0 and bool((untouched | changed).all())
    torch.testing.assert_close(pool_one.float(), pool_sep.float(), atol=1e-3, rtol=2.0 ** -7)
    # float64: the layer over each whole sequence, with bfloat16 rounding where both paths store
    rnd = P.to_bfloat16_and_back
    keep = [i for i in range(len(entries)) if entries[i][0] >= 0]
    for i, r in zip(keep, range(n_req)):
        hs = rnd(P.layer_norm(xs[r].double(), wn["weight"], wn["bias"], 1e-5))
        qkv = rnd(hs @ w["qkv_weight"].t() + w["qkv_bias"])
        q, k, v = (t.view(-1, heads, dh) for t in qkv.split(hidden, dim=-1))
        s = torch.einsum("hd,shd->hs", q[-1], k) * dh ** -0.5
        o = rnd(torch.einsum("hs,shd->hd", torch.softmax(s, -1), v).reshape(hidden))
        want = xs[r][-1].double() + o @ w["out_weight"].t() + w["out_bias"]
        for got, name in ((x_one[i], "one kernel"), (x_sep[i], "separate kernels")):
            err = float((got - want).abs().max())
            assert err <= 2.0 ** -7 * float(want.abs().max()), f"{name}, request {r} ({lens[r]} cached): error {err:.3e}"
