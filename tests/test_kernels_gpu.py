"""Each CUDA kernel alone against a plain PyTorch float64 reference of the same op,
at sizes other than the engine's tiny configurations."""
import math

import numpy as np
import pytest
import torch

import plain_gpt2 as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def K():
    from rosellm_b200.ops import kernels

    kernels._lib()
    return kernels


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,hidden,vocab,npos", [(1, 16, 11, 3), (37, 80, 1000, 50), (300, 1600, 777, 300)])
def test_embed(K, dtype, n, hidden, vocab, npos):
    g = torch.Generator().manual_seed(n)
    table = torch.randn(vocab, hidden, generator=g).to(dtype).to(DEV)
    pos_table = torch.randn(npos, hidden, generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, vocab, (n,), generator=g, dtype=torch.int32).to(DEV)
    pos = torch.randint(0, npos, (n,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.full((n, hidden), float("nan"), device=DEV)
    K.embed(ids, pos, table, pos_table, out)
    ref = table.float()[ids.long()] + pos_table.float()[pos.long()]
    torch.testing.assert_close(out, ref, atol=0, rtol=0)
    out2 = torch.empty_like(out)
    K.embed(ids, None, table, None, out2)
    torch.testing.assert_close(out2, table.float()[ids.long()], atol=0, rtol=0)
    K.check_status(torch.device(DEV))


def test_embed_flags_bad_token(K):
    table = torch.zeros(4, 16, device=DEV)
    ids = torch.tensor([1, 9], dtype=torch.int32, device=DEV)
    out = torch.empty(2, 16, device=DEV)
    K.embed(ids, None, table, None, out)
    with pytest.raises(K.KernelError, match="token id"):
        K.check_status(torch.device(DEV))
    K.check_status(torch.device(DEV))  # the word is cleared


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,hidden,eps", [(1, 16, 1e-5), (19, 80, 1e-6), (130, 1600, 1e-3), (5, 12000, 1e-5), (7, 2048, 1e-5),
                                          (3, 1028, 1e-5), (2, 2052, 1e-5)])
def test_layernorm(K, out_dtype, n, hidden, eps):
    g = torch.Generator().manual_seed(hidden)
    x = (torch.randn(n, hidden, generator=g) * 3 + 5).to(DEV)  # a large mean tests the variance
    gamma = torch.randn(hidden, generator=g).to(DEV)
    beta = torch.randn(hidden, generator=g).to(DEV)
    out = torch.empty(n, hidden, dtype=out_dtype, device=DEV)
    K.layernorm(x, gamma, beta, eps, out)
    ref = P.layer_norm(x.double().cpu(), gamma.double().cpu(), beta.double().cpu(), eps)
    torch.testing.assert_close(out.double().cpu(), ref, **tol(out_dtype))
    rows = torch.tensor([n - 1, 0, n // 2], dtype=torch.int32, device=DEV)
    out3 = torch.empty(3, hidden, dtype=out_dtype, device=DEV)
    K.layernorm(x, gamma, None, eps, out3, rows)
    ref3 = P.layer_norm(x.double().cpu()[rows.long().cpu()], gamma.double().cpu(), torch.zeros(hidden, dtype=torch.float64), eps)
    torch.testing.assert_close(out3.double().cpu(), ref3, **tol(out_dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 2, 3, 7, 8, 17, 64, 65, 130, 257])
@pytest.mark.parametrize("n,k", [(50, 40), (257, 96), (1000, 1600)])
def test_linear(K, dtype, m, n, k):
    g = torch.Generator().manual_seed(m * 1000 + n)
    a = (torch.randn(m, k, generator=g)).to(dtype).to(DEV)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(dtype).to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    ad, wd, bd = a.double().cpu(), w.double().cpu(), b.double().cpu()
    base = ad @ wd.t() + bd
    t = dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    out = torch.empty(m, n, dtype=dtype, device=DEV)
    K.linear(a, w, b, out)
    torch.testing.assert_close(out.double().cpu(), base, **t)
    for act, fn in ((K.ACT_GELU_TANH, P.gelu_tanh), (K.ACT_GELU_ERF, P.gelu_erf)):
        K.linear(a, w, b, out, act=act)
        torch.testing.assert_close(out.double().cpu(), fn(base), **t)
    x = torch.randn(m, n, generator=g).to(DEV)
    x0 = x.double().cpu()
    K.linear(a, w, b, x, residual=True)
    t32 = dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(x.double().cpu(), x0 + base, **t32)
    # float32 logits from either input type, no bias
    lo = torch.empty(m, n, dtype=torch.float32, device=DEV)
    K.linear(a, w, None, lo)
    torch.testing.assert_close(lo.double().cpu(), ad @ wd.t(), **t32)


@pytest.mark.parametrize("m,n,k", [(65, 50, 40), (128, 64, 64), (130, 257, 96), (257, 1000, 1600), (2048, 768, 768),
                                   (300, 2304, 768), (1024, 768, 3072), (200, 5003, 768),
                                   (17, 768, 3072), (64, 768, 768), (64, 2304, 768), (33, 3072, 768), (100, 257, 1600),
                                   (2048, 3072, 768), (2048, 2304, 768), (4096, 768, 768), (1000, 1024, 512), (129, 300, 96)])
def test_linear_tensor_cores(K, m, n, k):
    """The tcgen05 path against float64 on the same bfloat16 inputs: float32 accumulation, so the
    float32 outputs agree far more closely than bfloat16 rounding would explain."""
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    ad, wd, bd = a.double().cpu(), w.double().cpu(), b.double().cpu()
    base = ad @ wd.t()
    lo = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    K.linear(a, w, None, lo, path="tc")
    K.check_status(torch.device(DEV))
    torch.testing.assert_close(lo.double().cpu(), base, atol=2e-5, rtol=2e-5)
    x = torch.randn(m, n, generator=g).to(DEV)
    x0 = x.double().cpu()
    K.linear(a, w, b, x, residual=True, path="tc")
    torch.testing.assert_close(x.double().cpu(), x0 + base + bd, atol=3e-5, rtol=3e-5)
    for act, fn in ((K.ACT_GELU_TANH, P.gelu_tanh), (K.ACT_GELU_ERF, P.gelu_erf), (K.ACT_NONE, lambda u: u)):
        ob = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        K.linear(a, w, b, ob, act=act, path="tc")
        torch.testing.assert_close(ob.double().cpu(), fn(base + bd), atol=2e-2, rtol=2e-2)
    # and a strided input, as the merged attention heads are
    wide = torch.zeros(m, k + 24, dtype=torch.bfloat16, device=DEV)
    wide[:, 8:8 + k] = a
    lo2 = torch.empty_like(lo)
    K.linear(wide[:, 8:8 + k], w, None, lo2, path="tc")
    K.check_status(torch.device(DEV))
    assert torch.equal(lo2, lo)


@pytest.mark.parametrize("width", [32, 64, 96, 160, 192, 224, 256])
@pytest.mark.parametrize("m,n,k", [(300, 1000, 136), (129, 72, 64), (520, 776, 200)])
def test_linear_tensor_core_tile_widths(K, width, m, n, k):
    """Every tile width of the tcgen05 kernel (the kernel chooses one by the output's shape):
    stores and additions through the output's tensor map, edges inside a 32-column piece."""
    g = torch.Generator().manual_seed(width + m)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    base = a.double().cpu() @ w.double().cpu().t()
    bd = b.double().cpu()
    lo = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    K.linear(a, w, None, lo, path="tc", tile_width=width)
    K.check_status(torch.device(DEV))
    torch.testing.assert_close(lo.double().cpu(), base, atol=2e-5, rtol=2e-5)
    x = torch.randn(m, n, generator=g).to(DEV)
    x0 = x.double().cpu()
    K.linear(a, w, b, x, residual=True, path="tc", tile_width=width)
    K.linear(a, w, b, x, residual=True, path="tc", tile_width=width)  # twice: an addition, not a store
    torch.testing.assert_close(x.double().cpu(), x0 + 2 * (base + bd), atol=5e-5, rtol=5e-5)
    ob = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.linear(a, w, b, ob, act=K.ACT_GELU_TANH, path="tc", tile_width=width)
    K.check_status(torch.device(DEV))
    torch.testing.assert_close(ob.double().cpu(), P.gelu_tanh(base + bd), atol=2e-2, rtol=2e-2)
    with pytest.raises(K.KernelError):
        K.linear(a, w, None, lo, path="tc", tile_width=width + 8)


@pytest.mark.parametrize("m,n,k,width,parts", [(300, 1000, 1024, 256, 2), (2048, 768, 3072, 256, 3), (129, 72, 512, 64, 4),
                                               (520, 776, 1544, 160, 3), (2048, 768, 3072, 0, 0), (640, 200, 2048, 128, 8),
                                               (300, 2304, 768, 256, 6), (2048, 1024, 4096, 0, 0)])
def test_linear_tensor_cores_inner_size_in_parts(K, m, n, k, width, parts):
    """The tcgen05 kernel with the inner size cut into parts, one a block of a cluster, whose
    sums meet through distributed shared memory in a fixed order: the same bits every time."""
    g = torch.Generator().manual_seed(m + parts)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    base = a.double().cpu() @ w.double().cpu().t()
    bd = b.double().cpu()
    x0 = torch.randn(m, n, generator=g).to(DEV)
    results = []
    for _ in range(3):
        x = x0.clone()
        K.linear(a, w, b, x, residual=True, path="tc", tile_width=width, splits=parts)
        results.append(x)
    K.check_status(torch.device(DEV))
    torch.testing.assert_close(results[0].double().cpu(), x0.double().cpu() + base + bd, atol=5e-5, rtol=5e-5)
    assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])
    ob = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.linear(a, w, b, ob, act=K.ACT_GELU_TANH, path="tc", tile_width=width, splits=parts)
    K.check_status(torch.device(DEV))
    torch.testing.assert_close(ob.double().cpu(), P.gelu_tanh(base + bd), atol=2e-2, rtol=2e-2)


def test_linear_strided_input_and_refusals(K):
    a_full = torch.randn(9, 48, device=DEV)
    a = a_full[:, 16:32]
    w = torch.randn(5, 16, device=DEV)
    out = torch.empty(9, 5, device=DEV)
    K.linear(a, w, None, out)
    torch.testing.assert_close(out.cpu().double(), a.cpu().double() @ w.cpu().double().t(), atol=3e-5, rtol=3e-5)
    with pytest.raises(K.KernelError, match="multiple of 8"):
        K.linear(torch.randn(2, 12, device=DEV), torch.randn(3, 12, device=DEV), None, torch.empty(2, 3, device=DEV))
    with pytest.raises(K.KernelError, match="CUDA tensor"):
        K.linear(torch.randn(2, 16), torch.randn(3, 16), None, torch.empty(2, 3))


@pytest.mark.parametrize("m", [1, 2, 5, 8, 9, 16, 17, 31, 33, 64])
@pytest.mark.parametrize("n,k", [(50, 40), (257, 96), (2304, 768), (768, 3072), (5003, 1600)])
def test_linear_mma_rows(K, m, n, k):
    """The weight-streaming mma kernel (bfloat16, up to 64 rows) against float64 on the same
    inputs; float32 outputs agree to float32-accumulation accuracy."""
    g = torch.Generator().manual_seed(m * 7 + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    ad, wd, bd = a.double().cpu(), w.double().cpu(), b.double().cpu()
    base = ad @ wd.t()
    lo = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    K.linear(a, w, None, lo, path="mma")
    torch.testing.assert_close(lo.double().cpu(), base, atol=2e-5, rtol=2e-5)
    x = torch.randn(m, n, generator=g).to(DEV)
    x0 = x.double().cpu()
    K.linear(a, w, b, x, residual=True, path="mma")
    torch.testing.assert_close(x.double().cpu(), x0 + base + bd, atol=3e-5, rtol=3e-5)
    ob = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.linear(a, w, b, ob, act=K.ACT_GELU_ERF, path="mma")
    torch.testing.assert_close(ob.double().cpu(), P.gelu_erf(base + bd), atol=2e-2, rtol=2e-2)
    with pytest.raises(K.KernelError, match="at most 64 rows"):
        K.linear(torch.zeros(65, k, dtype=torch.bfloat16, device=DEV), w, None, torch.empty(65, n, device=DEV), path="mma")


@pytest.mark.parametrize("m,n,k", [(1, 40001, 768), (8, 50257, 768), (13, 40001, 136), (16, 45007, 768), (5, 16001, 1600),
                                   (16, 30011, 1600)])
def test_linear_rows_with_weights_copied_by_the_copy_engine(K, m, n, k):
    """Very wide float32 outputs of few rows (heads) run on the kernel whose warps get their
    weight rows by bulk copies into shared memory, two groups of eight columns ahead: against
    float64 on the same inputs, with the last group cut short by an odd width, with a bias, with
    the LayerNorm inside, and against the weight-streaming kernel that it stands in for."""
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    base = (a.double() @ w.double().t()).cpu()
    for bias in (None, b):
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
        K.linear(a, w, bias, out, path="mma")
        want = base + (b.double().cpu() if bias is not None else 0.0)
        torch.testing.assert_close(out.double().cpu(), want, atol=2e-5, rtol=2e-5)
    K.rows_bulk_kernel(False)
    try:
        old = torch.empty_like(out)
        K.linear(a, w, b, old, path="mma")
    finally:
        K.rows_bulk_kernel(True)
    torch.testing.assert_close(out, old, atol=2e-5, rtol=2e-5)  # (the same sums in the same order where K is not split)
    if k <= 1024 and k % 4 == 0:
        x = torch.randn(m, k, generator=g).to(DEV) * 2 + 0.5
        gamma, beta = torch.randn(k, generator=g).to(DEV), torch.randn(k, generator=g).to(DEV)
        h = P.layer_norm(x.double().cpu(), gamma.double().cpu(), beta.double().cpu(), 1e-5).to(torch.bfloat16).double()
        K.linear(K.NormInput(x, gamma, beta, 1e-5), w, None, out)
        torch.testing.assert_close(out.double().cpu(), h @ w.double().cpu().t(), atol=3e-2, rtol=3e-2)
    K.check_status(torch.device(DEV))


@pytest.mark.parametrize("m,n,k", [(17, 50, 40), (33, 3072, 768), (64, 2304, 768), (64, 768, 3072), (48, 1000, 1000),
                                   (20, 136, 72), (64, 768, 768), (1, 64, 64), (40, 1024, 4096), (32, 96, 2056),
                                   (49, 770, 1024), (8, 257, 1600), (16, 6400, 1600), (3, 1001, 776),
                                   (16, 88, 6400)])
def test_linear_rows_in_shared_memory(K, m, n, k):
    """The kernel that keeps both operands in shared memory (inner sizes too long for it cut over
    blocks that add into the float32 output; blocks of 8 to 32 columns; an odd output width)
    against float64 on the same inputs."""
    g = torch.Generator().manual_seed(m * 5 + n + k)
    a_full = torch.randn(m + 1, k + 8, generator=g).to(torch.bfloat16).to(DEV)
    a = a_full[1:, :k]  # rows with a stride
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    ad, wd, bd = a.double().cpu(), w.double().cpu(), b.double().cpu()
    base = ad @ wd.t()
    x = torch.randn(m, n, generator=g).to(DEV)
    x0 = x.double().cpu()
    K.linear(a, w, b, x, residual=True, path="smem")
    torch.testing.assert_close(x.double().cpu(), x0 + base + bd, atol=3e-5, rtol=3e-5)
    assert K.bf16_path(m, n, k, residual=True, out_f32=True) == ("smem" if m > 16 else "mma")
    if K._lib().rl_gemm_rows_smem_fits(m, n, k, 0, 0, 0, 0):
        lo = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
        K.linear(a, w, None, lo, path="smem")
        torch.testing.assert_close(lo.double().cpu(), base, atol=2e-5, rtol=2e-5)
        for act, fn in ((K.ACT_GELU_ERF, P.gelu_erf), (K.ACT_GELU_TANH, P.gelu_tanh)):
            ob = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
            K.linear(a, w, b, ob, act=act, path="smem")
            torch.testing.assert_close(ob.double().cpu(), fn(base + bd), atol=2e-2, rtol=2e-2)
    else:  # a long inner size is taken only where the parts can be added into the output
        with pytest.raises(K.KernelError, match="at most 64 rows"):
            K.linear(a, w, b, torch.empty(m, n, dtype=torch.bfloat16, device=DEV), path="smem")
        assert K.bf16_path(m, n, k) != "smem"
    K.check_status(torch.device(DEV))
    with pytest.raises(K.KernelError, match="at most 64 rows"):
        K.linear(torch.zeros(65, k, dtype=torch.bfloat16, device=DEV), w, None, torch.empty(65, n, device=DEV), path="smem")


@pytest.mark.parametrize("m,n,k", [(17, 50, 40), (24, 257, 96), (64, 2304, 768), (64, 768, 3072), (33, 3072, 768),
                                   (128, 768, 768), (100, 300, 1032), (1, 136, 64), (64, 1000, 2000), (48, 50257, 768)])
def test_linear_clustered_tensor_cores(K, m, n, k):
    """The tcgen05 kernel for 17 to 128 rows (K split over a cluster, sums through distributed
    shared memory) against float64 on the same inputs, run twice: the result is the same bits."""
    g = torch.Generator().manual_seed(m * 7 + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    ad, wd, bd = a.double().cpu(), w.double().cpu(), b.double().cpu()
    base = ad @ wd.t()
    lo = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    K.linear(a, w, None, lo, path="tcr")
    torch.testing.assert_close(lo.double().cpu(), base, atol=2e-5, rtol=2e-5)
    again = torch.full_like(lo, float("nan"))
    K.linear(a, w, None, again, path="tcr")
    assert torch.equal(lo, again)
    x = torch.randn(m, n, generator=g).to(DEV)
    x0 = x.double().cpu()
    K.linear(a, w, b, x, residual=True, path="tcr")
    torch.testing.assert_close(x.double().cpu(), x0 + base + bd, atol=3e-5, rtol=3e-5)
    ob = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.linear(a, w, b, ob, act=K.ACT_GELU_ERF, path="tcr")
    torch.testing.assert_close(ob.double().cpu(), P.gelu_erf(base + bd), atol=2e-2, rtol=2e-2)
    wide = torch.randn(m, k + 16, generator=g).to(torch.bfloat16).to(DEV)  # rows with a stride
    lo2 = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    K.linear(wide[:, 8:8 + k], w, None, lo2, path="tcr")
    torch.testing.assert_close(lo2.double().cpu(), wide[:, 8:8 + k].double().cpu() @ wd.t(), atol=2e-5, rtol=2e-5)
    K.check_status(torch.device(DEV))


def test_linear_clustered_tensor_cores_refuses_what_does_not_fit(K):
    w = torch.zeros(64, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(K.KernelError, match="at most 128 rows"):
        K.linear(torch.zeros(129, 64, dtype=torch.bfloat16, device=DEV), w, None, torch.empty(129, 64, device=DEV), path="tcr")
    w = torch.zeros(64, 16384, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(K.KernelError, match="fits the shared memory"):
        K.linear(torch.zeros(64, 16384, dtype=torch.bfloat16, device=DEV), w, None, torch.empty(64, 64, device=DEV), path="tcr")


@pytest.mark.parametrize("m,n,k", [(1, 50, 40), (3, 257, 96), (8, 2304, 768), (16, 3072, 768), (5, 300, 1024), (8, 768, 64)])
def test_linear_with_fused_layernorm(K, m, n, k):
    """The mma row product normalising its own input equals LayerNorm followed by the product."""
    g = torch.Generator().manual_seed(m + n + k)
    x = (torch.randn(m + 2, k + 4, generator=g) * 2 + 0.5).to(DEV)[1:m + 1, :k]  # rows with a stride
    gamma, beta = (torch.randn(k, generator=g) * 0.2 + 1).to(DEV), (torch.randn(k, generator=g) * 0.2).to(DEV)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    h = torch.empty(m, k, dtype=torch.bfloat16, device=DEV)
    K.layernorm(x.contiguous(), gamma, beta, 1e-5, h)
    for bt in (beta, None):
        if bt is None:
            K.layernorm(x.contiguous(), gamma, None, 1e-5, h)
        want = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
        K.linear(h, w, b, want, act=K.ACT_GELU_TANH)
        got = torch.full_like(want, float("nan"))
        K.linear(K.NormInput(x, gamma, bt, 1e-5), w, b, got, act=K.ACT_GELU_TANH)
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    with pytest.raises(K.KernelError, match="at most 16 rows"):
        K.linear(K.NormInput(torch.zeros(17, k, device=DEV), gamma, beta, 1e-5), w, b, torch.empty(17, n, dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("m,hidden,inner,act", [
    (1, 64, 256, "gelu_tanh"), (3, 96, 320, "gelu_erf"), (8, 768, 3072, "gelu_tanh"), (16, 768, 3072, "gelu_tanh"),
    (5, 48, 104, "gelu_tanh"), (13, 1024, 4096, "gelu_erf"), (16, 72, 40, "gelu_tanh"), (9, 200, 1000, "gelu_erf"),
])
def test_fused_feed_forward_of_few_rows(K, m, hidden, inner, act):
    """x += act(in W_in^T + b) W_out^T + b in one kernel, the input being LayerNorm(x) or given
    rows, against float64: widths that are no multiple of 16, inner widths that no slice width
    divides, every slice width the kernel takes, with and without biases."""
    g = torch.Generator().manual_seed(m + hidden + inner)
    big = (torch.randn(m + 2, hidden + 4, generator=g) * 2 + 0.5).to(DEV)
    x0 = big[1:m + 1, :hidden]  # rows with a stride
    gamma, beta = (torch.randn(hidden, generator=g) * 0.2 + 1).to(DEV), (torch.randn(hidden, generator=g) * 0.2).to(DEV)
    w_in = (torch.randn(inner, hidden, generator=g) / math.sqrt(hidden)).to(torch.bfloat16).to(DEV)
    w_out = (torch.randn(hidden, inner, generator=g) / math.sqrt(inner)).to(torch.bfloat16).to(DEV)
    b_in, b_out = torch.randn(inner, generator=g).to(DEV), torch.randn(hidden, generator=g).to(DEV)
    fn = P.gelu_tanh if act == "gelu_tanh" else P.gelu_erf
    chosen = K.mlp_fused_slice(m, hidden, inner, True, torch.bfloat16)
    assert chosen in (16, 32)
    assert K.mlp_fused_slice(17, hidden, inner, True, torch.bfloat16) == 0  # more rows: the separate products
    assert K.mlp_fused_slice(m, hidden, inner, True, torch.float32) == 0
    for normed in (True, False):
        for biases in (True, False):
            bt = beta if biases else None
            if normed:
                h64 = P.layer_norm(x0.double().cpu(), gamma.double().cpu(), (bt if bt is not None else beta * 0).double().cpu(), 1e-5)
                h64 = h64.to(torch.bfloat16).double()  # the kernel rounds the normalised rows to bfloat16
            else:
                h = (torch.randn(m, hidden, generator=g)).to(torch.bfloat16).to(DEV)
                h64 = h.double().cpu()
            bi, bo = (b_in, b_out) if biases else (None, None)
            u = fn(h64 @ w_in.double().cpu().t() + (bi.double().cpu() if biases else 0.0)).to(torch.bfloat16).double()
            want = x0.double().cpu() + u @ w_out.double().cpu().t() + (bo.double().cpu() if biases else 0.0)
            for width in sorted({chosen, 16, 32}):
                x = big.clone()[1:m + 1, :hidden]
                try:
                    K.mlp_fused(x, K.NormInput(x, gamma, bt, 1e-5) if normed else h, w_in, bi,
                                K.mlp_pack_out_weight(w_out, width), bo, act=K.ACTIVATIONS[act], slice_width=width)
                except K.KernelError:
                    assert width != chosen  # a wider slice than shared memory holds at this width is refused
                    continue
                torch.testing.assert_close(x.double().cpu(), want, atol=2e-2, rtol=2e-2)
    with pytest.raises(K.KernelError, match="sizes not taken"):
        K.mlp_fused(torch.zeros(17, hidden, device=DEV), torch.zeros(17, hidden, dtype=torch.bfloat16, device=DEV), w_in,
                    None, K.mlp_pack_out_weight(w_out, 16), None, act=K.ACT_GELU_TANH, slice_width=16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_scatters_keys_and_values_into_pages(K, dtype):
    """The qkv product writing its key and value columns straight into the cache equals the
    product followed by the separate cache write; padding rows (slot -1) write nothing."""
    from rosellm_b200.engine.context import build_host_batch

    heads, n_kv, dh, page, hidden = 6, 2, 48, 8, 96
    q_w, kv_w = heads * dh, n_kv * dh
    hb = build_host_batch([(4, 3, [0] * 5, []), (0, 16, [0], []), (2, 0, [0] * 6, [])])
    m = 12
    g = torch.Generator().manual_seed(1)
    a = torch.randn(m, hidden, generator=g).to(dtype).to(DEV)
    w = (torch.randn(q_w + 2 * kv_w, hidden, generator=g) * 0.1).to(dtype).to(DEV)
    b = torch.randn(q_w + 2 * kv_w, generator=g).to(DEV)
    table = torch.full((6, 4), -1, dtype=torch.int32)
    table[4, :1] = torch.tensor([7]); table[0, :3] = torch.tensor([1, 9, 3]); table[2, :1] = torch.tensor([11])
    table = table.to(DEV)
    dev = lambda arr: torch.as_tensor(arr, dtype=torch.int32).to(DEV)
    pos, rot, slots = dev(hb.positions), dev(hb.req_of_token), dev(hb.slots)
    slots_padded = slots.clone()
    slots_padded[1] = -1
    for sl in (slots, slots_padded):
        qkv = torch.zeros(m, q_w + 2 * kv_w, dtype=dtype, device=DEV)
        K.linear(a, w, b, qkv)  # float32: the row kernel; bfloat16: the mma row kernel
        want = torch.zeros(12, 2, n_kv, page, dh, dtype=dtype, device=DEV)
        K.kv_write(qkv[:, q_w:q_w + kv_w], qkv[:, q_w + kv_w:], want, table, pos, rot, sl, 32)
        pool = torch.zeros_like(want)
        out = torch.zeros_like(qkv)
        K.linear(a, w, b, out, kv=K.KvTarget(pool, table, pos, rot, sl, q_w, 32))
        K.check_status(torch.device(DEV))
        assert torch.equal(pool, want) and float(pool.float().abs().sum()) > 0
        assert torch.equal(out[:, :q_w], qkv[:, :q_w]) and float(out[:, q_w:].float().abs().sum()) == 0.0
        if dtype == torch.bfloat16:  # the clustered tcgen05 kernel writes the same pages
            for forced in ("tcr", "tc", "smem"):  # and so do the persistent one and the shared-memory row kernel
                pool2, out2 = torch.zeros_like(want), torch.zeros_like(qkv)
                K.linear(a, w, b, out2, kv=K.KvTarget(pool2, table, pos, rot, sl, q_w, 32), path=forced)
                K.check_status(torch.device(DEV))
                assert float((pool2 == 0).logical_xor(want == 0).sum()) == 0  # the same places are written
                torch.testing.assert_close(pool2.float(), want.float(), atol=2e-2, rtol=2e-2)
                torch.testing.assert_close(out2[:, :q_w].float(), qkv[:, :q_w].float(), atol=2e-2, rtol=2e-2)
                assert float(out2[:, q_w:].float().abs().sum()) == 0.0


@pytest.mark.parametrize("heads,n_kv,dh,page", [(6, 2, 48, 8), (12, 12, 64, 16), (5, 5, 16, 64)])
def test_tcgen05_product_scatters_keys_and_values_of_long_portions(K, heads, n_kv, dh, page):
    """Several row tiles, column tiles that straddle the queries, keys, values and the end of the
    output, requests that start inside a page, a padding request: the pages equal those that
    the separate cache-write kernel fills from the same product."""
    from rosellm_b200.engine.context import build_host_batch

    hidden = 96
    q_w, kv_w = heads * dh, n_kv * dh
    lens = [(3, 13, 150), (0, 0, 1), (5, 40, 131), (1, 7, 2)]  # (slot, cached, new)
    hb = build_host_batch([(s, c, [0] * n, []) for s, c, n in lens])
    m = len(hb.token_ids)
    g = torch.Generator().manual_seed(5)
    a = torch.randn(m, hidden, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(q_w + 2 * kv_w, hidden, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    b = torch.randn(q_w + 2 * kv_w, generator=g).to(DEV)
    per_seq = -(-256 // page)
    perm = torch.randperm(6 * per_seq, generator=g).to(torch.int32).view(6, per_seq)
    table = perm.to(DEV)
    dev = lambda arr: torch.as_tensor(arr, dtype=torch.int32).to(DEV)
    pos, rot, slots = dev(hb.positions), dev(hb.req_of_token), dev(hb.slots)
    slots[3] = -1  # the last request is padding: nothing of it is written
    qkv = torch.zeros(m, q_w + 2 * kv_w, dtype=torch.bfloat16, device=DEV)
    K.linear(a, w, b, qkv, path="tc")
    want = torch.zeros(6 * per_seq, 2, n_kv, page, dh, dtype=torch.bfloat16, device=DEV)
    K.kv_write(qkv[:, q_w:q_w + kv_w], qkv[:, q_w + kv_w:], want, table, pos, rot, slots, 256)
    pool, out = torch.zeros_like(want), torch.zeros_like(qkv)
    K.linear(a, w, b, out, kv=K.KvTarget(pool, table, pos, rot, slots, q_w, 256), path="tc")
    K.check_status(torch.device(DEV))
    assert torch.equal(pool, want) and float(pool.float().abs().sum()) > 0
    assert torch.equal(out[:, :q_w], qkv[:, :q_w]) and float(out[:, q_w:].float().abs().sum()) == 0.0


def make_paged_case(dtype, lens_q, lens_kv, n_heads, n_kv, dh, page, window, seed, sharp=False):
    """Random queries and a paged cache with shuffled, poisoned pages; returns tensors and the reference."""
    g = torch.Generator().manual_seed(seed)
    n_req = len(lens_q)
    max_pages = max(-(-l // page) for l in lens_kv) + 1
    n_pages = sum(-(-l // page) for l in lens_kv) + 5
    pool = torch.full((n_pages, 2, n_kv, page, dh), float("nan"))
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n_req + 2, max_pages), -1, dtype=torch.int32)
    slots = torch.randperm(n_req + 2, generator=g)[:n_req].to(torch.int32)
    keys, vals = [], []
    for r in range(n_req):
        k = torch.randn(lens_kv[r], n_kv, dh, generator=g)
        v = torch.randn(lens_kv[r], n_kv, dh, generator=g)
        keys.append(k)
        vals.append(v)
    total_q = sum(lens_q)
    q = torch.randn(total_q, n_heads, dh, generator=g)
    if sharp:
        # one far key of each request matches its last query: that score stands out
        at = 0
        for r in range(n_req):
            far = 1 if window is None else max(0, lens_kv[r] - window)
            far = min(far, lens_kv[r] - 1)
            qlast = q[at + lens_q[r] - 1]
            grp = n_heads // n_kv
            keys[r][far] = qlast.view(n_kv, grp, dh)[:, 0, :] * 4.0
            at += lens_q[r]
    q = q.to(dtype)
    for r in range(n_req):
        keys[r] = keys[r].to(dtype)
        vals[r] = vals[r].to(dtype)
        first_page = 0
        if window is not None:
            first_page = max(0, lens_kv[r] - lens_q[r] - window + 1) // page
        for p in range(first_page, -(-lens_kv[r] // page)):
            pid = perm.pop()
            table[slots[r], p] = pid
            lo, hi = p * page, min((p + 1) * page, lens_kv[r])
            pool[pid, 0, :, : hi - lo] = keys[r][lo:hi].float().transpose(0, 1)
            pool[pid, 1, :, : hi - lo] = vals[r][lo:hi].float().transpose(0, 1)
    # reference
    ref = torch.zeros(total_q, n_heads, dh, dtype=torch.float64)
    at = 0
    grp = n_heads // n_kv
    for r in range(n_req):
        kd = keys[r].double().repeat_interleave(grp, dim=1)
        vd = vals[r].double().repeat_interleave(grp, dim=1)
        for i in range(lens_q[r]):
            pos = lens_kv[r] - lens_q[r] + i
            lo = 0 if window is None else max(0, pos - window + 1)
            s = torch.einsum("hd,thd->ht", q[at + i].double(), kd[lo:pos + 1]) * dh ** -0.5
            ref[at + i] = torch.einsum("ht,thd->hd", torch.softmax(s, dim=-1), vd[lo:pos + 1])
        at += lens_q[r]
    return q, pool.to(dtype), table, slots, ref


def run_attention(K, dtype, lens_q, lens_kv, n_heads, n_kv, dh, page, window, seed, sharp=False, splits=None, use_wide=True,
                  decode_wide=False, prefill_path=None):
    from rosellm_b200.engine.context import build_host_batch

    q, pool, table, slots, ref = make_paged_case(dtype, lens_q, lens_kv, n_heads, n_kv, dh, page, window, seed, sharp)
    hb = build_host_batch([(int(slots[r]), lens_kv[r] - lens_q[r], [0] * lens_q[r], []) for r in range(len(lens_q))])
    dev = lambda a: torch.as_tensor(a, dtype=torch.int32).contiguous().to(DEV)
    total_q = sum(lens_q)
    # queries sit inside a wider buffer, as they do in the packed qkv activations
    wide = torch.zeros(total_q, n_heads * dh + 32, dtype=dtype, device=DEV)
    wide[:, 16:16 + n_heads * dh] = q.view(total_q, -1).to(DEV)
    qv = wide[:, 16:16 + n_heads * dh]
    out = torch.full((total_q, n_heads * dh), float("nan"), dtype=dtype, device=DEV)
    n_dec = len(hb.decode_reqs)
    n_splits = splits or 1
    part_o = torch.empty(max(1, n_dec * n_heads * n_splits * dh), device=DEV)
    part_ml = torch.empty(max(1, n_dec * n_heads * n_splits * 2), device=DEV)
    K.attention(qv, pool.to(DEV), table.to(DEV), dev(hb.q_start), dev(hb.kv_len), dev(hb.slots), out,
                n_heads=n_heads, scale=dh ** -0.5, window=window, tiles=dev(hb.tiles.reshape(-1)),
                n_tiles=len(hb.tiles), decode_reqs=dev(hb.decode_reqs), n_decode=n_dec,
                n_splits=n_splits, part_o=part_o, part_ml=part_ml,
                tiles_wide=dev(hb.tiles_wide.reshape(-1)) if use_wide else None, n_tiles_wide=len(hb.tiles_wide),
                decode_wide=decode_wide, prefill_path=prefill_path)
    K.check_status(torch.device(DEV))
    got = out.double().cpu().view(total_q, n_heads, dh)
    assert torch.isfinite(got).all(), "attention read a poisoned (unused) part of the cache"
    t = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(got, ref, **t)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decode_right_after_the_cache_write_with_no_copy_between(K, dtype):
    """A caller outside the engine writes a whole prompt's keys and values and attends over
    them with the very next launch on the stream, no copy in between.  Without the promise
    ``old_keys_settled`` the decode kernel reads nothing before it has waited for the kernel
    ahead of it, so it sees every key (repeated a few times: what is at stake is an overlap of
    two launches)."""
    n_heads, n_kv, dh, page = 6, 2, 64, 16
    lens = [700, 130, 64, 1]
    q, pool, table, slots, ref = make_paged_case(dtype, [1] * len(lens), lens, n_heads, n_kv, dh, page, None, seed=77)
    pool_dev, table_dev = pool.to(DEV), table.to(DEV)
    # the keys and values as the rows a packed qkv product would have left, token after token
    rows_k, rows_v, pos, req_of = [], [], [], []
    for r, l in enumerate(lens):
        pages = table[slots[r], : -(-l // page)].long()
        rows_k.append(pool[pages, 0].permute(0, 2, 1, 3).reshape(-1, n_kv * dh)[:l])
        rows_v.append(pool[pages, 1].permute(0, 2, 1, 3).reshape(-1, n_kv * dh)[:l])
        pos += list(range(l))
        req_of += [r] * l
    dev = lambda a: torch.as_tensor(a, dtype=torch.int32).contiguous().to(DEV)
    k_rows, v_rows = torch.cat(rows_k).to(DEV).contiguous(), torch.cat(rows_v).to(DEV).contiguous()
    pos, req_of, slots_dev = dev(pos), dev(req_of), dev(slots)
    n = len(lens)
    q_start, kv_len, decode_reqs = dev(list(range(n + 1))), dev(lens), dev(list(range(n)))
    qv = q.view(n, -1).to(DEV).contiguous()
    part_o = torch.empty(n * n_heads * 4 * dh, device=DEV)
    part_ml = torch.empty(n * n_heads * 4 * 2, device=DEV)
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    for splits, wide in ((1, False), (4, False), (1, True)) * 3:
        fresh = torch.full_like(pool_dev, float("nan"))  # nothing is in the cache yet
        out = torch.full((n, n_heads * dh), float("nan"), dtype=dtype, device=DEV)
        torch.cuda.synchronize()
        K.kv_write(k_rows, v_rows, fresh, table_dev, pos, req_of, slots_dev, 1024)
        K.attention(qv, fresh, table_dev, q_start, kv_len, slots_dev, out, n_heads=n_heads, scale=dh ** -0.5,
                    window=None, tiles=None, n_tiles=0, decode_reqs=decode_reqs, n_decode=n, n_splits=splits,
                    part_o=part_o, part_ml=part_ml, decode_wide=wide)
        K.check_status(torch.device(DEV))
        got = out.double().cpu().view(n, n_heads, dh)
        assert torch.isfinite(got).all(), "the decode kernel read keys before the write ahead of it had finished"
        torch.testing.assert_close(got, ref, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_heads,n_kv,dh,page,window", [
    (4, 4, 16, 16, None), (3, 3, 32, 8, None), (6, 2, 48, 4, None), (5, 1, 80, 32, None),
    (2, 2, 128, 64, None), (1, 1, 256, 16, None), (6, 3, 64, 16, 20), (4, 4, 16, 8, 5),
])
def test_attention_mixed_batch(K, dtype, n_heads, n_kv, dh, page, window):
    lens_q = [1, 17, 1, 2, 33, 1, 16]
    lens_kv = [1, 17, 70, 41, 100, 300, 16]
    run_attention(K, dtype, lens_q, lens_kv, n_heads, n_kv, dh, page, window, seed=dh + page)


@pytest.mark.parametrize("dh", [16, 32, 48, 64, 80, 96, 112, 128])
@pytest.mark.parametrize("window", [None, 70])
def test_attention_prompt_portions_on_tensor_cores(K, dh, window):
    """Long and short portions, with and without earlier context, through the mma kernel
    (64-query tiles) and, for comparison, the CUDA-core kernel (16-query tiles)."""
    lens_q = [200, 3, 64, 65, 130, 17]
    lens_kv = [200, 90, 64, 300, 131, 401]
    for use_wide in (True, False):
        run_attention(K, torch.bfloat16, lens_q, lens_kv, 4, 2, dh, 16, window, seed=dh, use_wide=use_wide)
    run_attention(K, torch.bfloat16, [150, 70], [400, 333], 3, 3, dh, 8, window, seed=dh + 1, sharp=True)


@pytest.mark.parametrize("page", [8, 16, 64])
def test_attention_prompt_portions_on_tcgen05(K, page):
    """The tcgen05 kernel for prompt portions (head size 64, no window): whole prompts, portions
    that start anywhere in a request, lengths that are no multiple of its tiles, grouped heads,
    a far key that stands out, beside decoded requests of the same step."""
    for path in ("tc", "mma"):
        run_attention(K, torch.bfloat16, [130], [130], 2, 1, 64, page, None, seed=1, prefill_path=path)
        run_attention(K, torch.bfloat16, [5, 1, 300, 64, 129], [5, 77, 300, 200, 1000], 4, 2, 64, page, None, seed=2,
                      prefill_path=path)
        run_attention(K, torch.bfloat16, [150, 70, 1], [400, 333, 9], 3, 3, 64, page, None, seed=3, sharp=True,
                      prefill_path=path)
        # five and three pieces of 128 queries: blocks that take two pieces (the last with the
        # first, ...) and the middle piece alone, a portion that starts inside its request
        run_attention(K, torch.bfloat16, [520, 257], [700, 257], 2, 2, 64, page, None, seed=5, prefill_path=path)
    with pytest.raises(K.KernelError, match="head size 64"):
        run_attention(K, torch.bfloat16, [20], [20], 2, 1, 32, page, None, seed=4, prefill_path="tc")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("splits", [1, 2, 5, 32])
@pytest.mark.parametrize("decode_wide", [False, True])
def test_attention_decode_splits(K, dtype, splits, decode_wide):
    """Both forms of the decode kernel (four and sixteen warps a block), keys split over blocks."""
    run_attention(K, dtype, [1, 1, 1, 1], [700, 1, 33, 129], 6, 2, 64, 16, None, seed=splits, splits=splits,
                  decode_wide=decode_wide)
    run_attention(K, dtype, [1, 1, 1], [700, 5, 64], 4, 4, 32, 8, 100, seed=splits, splits=splits,
                  decode_wide=decode_wide)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dh", [16, 48, 128, 256])
def test_attention_decode_wide_blocks_head_sizes(K, dtype, dh):
    run_attention(K, dtype, [1, 1, 1], [1100, 17, 300], 4, 2, dh, 16, None, seed=dh, splits=1, decode_wide=True, sharp=True)
    run_attention(K, dtype, [1, 1], [640, 90], 2, 1, dh, 8, 200, seed=dh + 1, splits=2, decode_wide=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 64])
def test_attention_far_key_stands_out(K, dtype, window):
    # the last query of each request matches one key hundreds of positions back (at the
    # window's far edge when there is a window): dropping that key changes the result wholly
    run_attention(K, dtype, [1, 40, 1], [600, 500, 65], 4, 2, 64, 16, window, seed=7, sharp=True, splits=4)
    run_attention(K, dtype, [1, 40, 1], [600, 500, 65], 4, 2, 64, 16, window, seed=8, sharp=True, splits=1, decode_wide=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kv_write(K, dtype):
    n_kv, dh, page = 3, 48, 8
    lens_new, cached = [5, 1, 20], [3, 16, 0]
    from rosellm_b200.engine.context import build_host_batch

    hb = build_host_batch([(s, c, [0] * n, []) for s, c, n in zip([4, 0, 2], cached, lens_new)])
    n = sum(lens_new)
    g = torch.Generator().manual_seed(0)
    buf = torch.randn(n, 3 * n_kv * dh, generator=g).to(dtype).to(DEV)
    k, v = buf[:, n_kv * dh: 2 * n_kv * dh], buf[:, 2 * n_kv * dh:]
    n_pages = 12
    pool = torch.zeros(n_pages, 2, n_kv, page, dh, dtype=dtype, device=DEV)
    table = torch.full((6, 4), -1, dtype=torch.int32)
    table[4, :1] = torch.tensor([7]); table[0, :3] = torch.tensor([1, 9, 3]); table[2, :3] = torch.tensor([11, 0, 5])
    dev = lambda a: torch.as_tensor(a, dtype=torch.int32).to(DEV)
    K.kv_write(k, v, pool, table.to(DEV), dev(hb.positions), dev(hb.req_of_token), dev(hb.slots), 32)
    K.check_status(torch.device(DEV))
    expect = torch.zeros_like(pool).cpu()
    for i in range(n):
        slot = int(hb.slots[hb.req_of_token[i]]); pos = int(hb.positions[i])
        pid = int(table[slot, pos // page])
        expect[pid, 0, :, pos % page] = k[i].cpu().view(n_kv, dh)
        expect[pid, 1, :, pos % page] = v[i].cpu().view(n_kv, dh)
    assert torch.equal(pool.cpu(), expect)


def test_kv_write_flags_missing_page(K):
    pool = torch.zeros(2, 2, 1, 4, 16, device=DEV)
    table = torch.full((1, 2), -1, dtype=torch.int32, device=DEV)
    kv = torch.randn(1, 16, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.kv_write(kv, kv, pool, table, z, z, z, 8)
    with pytest.raises(K.KernelError, match="block table"):
        K.check_status(torch.device(DEV))
    assert float(pool.abs().sum()) == 0.0


@pytest.mark.parametrize("vocab", [1000, 50257, 100003, 140000, 300001])
def test_sample_greedy_and_filters(K, vocab):
    """Small vocabularies and very large ones take one block a row; between, a row is spread
    over a cluster of eight blocks with 8, 16 or 32 entries a thread."""
    g = torch.Generator().manual_seed(vocab)
    rows = 12
    logits = (torch.randn(rows, vocab, generator=g) * 3).to(DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    K.sample(logits, None, None, None, None, None, out)
    assert out.cpu().tolist() == logits.cpu().argmax(-1).tolist()
    temps = torch.tensor([0.0, 0.7, 1.0, 1.3, 0.8, 0.8, 0.8, 2.0, 1.0, 0.5, 1.0, 1.0])
    top_k = torch.tensor([0, 0, 5, 0, 50, 1, 2000, 3, 0, 10, 0, 999], dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 1.0, 0.9, 0.5, 0.3, 0.95, 0.01, 0.0, 0.7, 0.999, 0.6])
    seeds = torch.arange(rows, dtype=torch.int64) * 7919 + (1 << 40)
    counters = torch.arange(rows, dtype=torch.int32) * 3
    kept = torch.empty(rows, dtype=torch.int32, device=DEV)
    K.sample(logits, temps.to(DEV), top_k.to(DEV), top_p.to(DEV), seeds.to(DEV), counters.to(DEV), out, kept)
    got, kept = out.cpu().tolist(), kept.cpu().tolist()
    for r in range(rows):
        row = logits[r].cpu()
        if temps[r] <= 0:
            assert got[r] == int(row.argmax())
            continue
        tok, scores = P.gumbel_sample(row, float(temps[r]), int(top_k[r]), float(top_p[r]), int(seeds[r]), int(counters[r]))
        n_keep = int(np.isfinite(scores).sum())
        assert kept[r] == n_keep, f"row {r}: kernel kept {kept[r]} tokens, the sort-based filter {n_keep}"
        assert np.isfinite(scores[got[r]]), f"row {r}: sampled a filtered token"
        assert scores[got[r]] >= scores.max() - 1e-4, f"row {r}: token {got[r]} vs {tok}"


@pytest.mark.parametrize("rows,vocab,k", [(1, 50257, 768), (8, 50257, 768), (16, 5003, 1600), (3, 301, 136), (5, 77, 40),
                                          (12, 30011, 1600),
                                          (17, 50257, 768), (64, 50257, 768), (100, 50257, 1600), (150, 20011, 136),
                                          (40, 301, 1600), (64, 5003, 1600)])
def test_product_that_chooses_the_tokens_itself(K, rows, vocab, k):
    """The head's product with the choice of the next token in its epilogue gives, row by row,
    the token that the sampling kernel chooses from the logits of the ordinary product:
    greedy rows and rows with a temperature, again and again (its scratch is left zero), an
    exact tie going to the lower index, and the LayerNorm inside the product for one or two rows."""
    g = torch.Generator().manual_seed(rows * 1000 + vocab)
    a = torch.randn(rows, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(vocab, k, generator=g) / math.sqrt(k)).to(torch.bfloat16)
    w[vocab - 1] = w[vocab // 3]  # two entries with the same logit in every row
    a[0] = (w[vocab // 3] * 8).to(DEV)  # ... which in row 0 is the largest
    w = w.to(DEV)
    bias = torch.randn(vocab, generator=g).mul(0.1).to(DEV)
    bias[vocab - 1] = bias[vocab // 3]
    logits = torch.empty(rows, vocab, device=DEV)
    want, got = (torch.empty(rows, dtype=torch.int32, device=DEV) for _ in range(2))
    path = K.bf16_path(rows, vocab, k, out_f32=True)  # up to 16 rows the weight-streaming kernel, tcgen05 tiles beyond
    # (17 to 64 rows of a narrow output and a long inner size: none of the kernels between takes them,
    # so weight-streaming too, with two and four tiles of 16 rows)
    assert path == ("mma" if rows <= 16 or (rows <= 64 and vocab < 9000) else "tc")
    for b in (None, bias):
        K.linear(a, w, b, logits, path=path)
        K.sample(logits, None, None, None, None, None, want)
        assert int(want[0]) == vocab // 3
        for _ in range(3):
            got.fill_(-7)
            K.linear_sample(a, w, b, K.SampleInto(got))
            assert got.cpu().tolist() == want.cpu().tolist()
        temps = torch.tensor([0.0, 0.7, 1.0, 1.3, 0.8, 2.0, 0.0, 0.5] * 20)[:rows].to(DEV)
        seeds = (torch.arange(rows, dtype=torch.int64) * 7919 + (1 << 40)).to(DEV)
        for step in range(3):
            counters = (torch.arange(rows, dtype=torch.int32) * 3 + step).to(DEV)
            K.sample(logits, temps, None, None, seeds, counters, want)
            K.linear_sample(a, w, b, K.SampleInto(got, temps, seeds, counters))
            assert got.cpu().tolist() == want.cpu().tolist()
    if rows <= 2 and k % 4 == 0 and k <= 1024:
        x = torch.randn(rows, k, generator=g).to(DEV)
        gamma, beta = torch.randn(k, generator=g).to(DEV), torch.randn(k, generator=g).to(DEV)
        K.linear(K.NormInput(x, gamma, beta, 1e-5), w, None, logits)
        K.sample(logits, None, None, None, None, None, want)
        K.linear_sample(K.NormInput(x, gamma, beta, 1e-5), w, None, K.SampleInto(got))
        assert got.cpu().tolist() == want.cpu().tolist()
    with pytest.raises(K.KernelError):
        K.linear_sample(a, w, None, K.SampleInto(got, temps, None, None))


@pytest.mark.parametrize("rows,vocab,k", [(8, 50257, 768), (3, 301, 136), (40, 50257, 768)])
def test_chosen_tokens_reach_the_host_without_a_copy(K, rows, vocab, k):
    """With a ring of pinned host slots in its ``SampleInto`` the kernel that chooses the tokens
    writes them there too, launch number n into slot n % SAMPLE_RING, and counts its launches on
    the device (the three kernels that have the epilogue: bulk-fed, weight-streaming, tcgen05)."""
    g = torch.Generator().manual_seed(rows + vocab)
    w = (torch.randn(vocab, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    ring = torch.full((K.SAMPLE_RING, 64), -1, dtype=torch.int32).pin_memory()
    step = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = torch.empty(rows, dtype=torch.int32, device=DEV)
    into = K.SampleInto(got, host_ring=ring, ring_step=step)
    logits, want = torch.empty(rows, vocab, device=DEV), torch.empty(rows, dtype=torch.int32, device=DEV)
    history = []
    for n in range(K.SAMPLE_RING + 2):
        a = torch.randn(rows, k, generator=g).to(torch.bfloat16).to(DEV)
        K.linear(a, w, None, logits)
        K.sample(logits, None, None, None, None, None, want)
        K.linear_sample(a, w, None, into)
        torch.cuda.synchronize()
        history.append(want.cpu().tolist())
        assert got.cpu().tolist() == history[-1]
        assert ring[n % K.SAMPLE_RING, :rows].tolist() == history[-1]
        assert int(step) == n + 1
        for back in range(1, min(n, K.SAMPLE_RING - 1) + 1):  # the slots of the launches before are untouched
            assert ring[(n - back) % K.SAMPLE_RING, :rows].tolist() == history[-1 - back]
    assert ring[:, rows:].eq(-1).all()
    with pytest.raises(K.KernelError):
        K.SampleInto(got, host_ring=torch.zeros(K.SAMPLE_RING, 8, dtype=torch.int32), ring_step=step)  # not pinned
    short = K.SampleInto(got, host_ring=torch.zeros(K.SAMPLE_RING, 2, dtype=torch.int32).pin_memory(), ring_step=step)
    with pytest.raises(K.KernelError):
        K.linear_sample(torch.zeros(3, k, dtype=torch.bfloat16, device=DEV), w, None, short)


def test_product_that_chooses_the_tokens_refuses_what_it_cannot_take(K):
    """Between 17 and 64 rows a narrow output runs on the kernel that keeps both operands in
    shared memory, which has no such epilogue: the call says so, and so does the query."""
    w = torch.zeros(2304, 768, dtype=torch.bfloat16, device=DEV)
    a = torch.zeros(40, 768, dtype=torch.bfloat16, device=DEV)
    assert K.bf16_path(40, 2304, 768, out_f32=True) == "smem"
    assert not K.sampling_product_possible(40, 2304, 768, torch.bfloat16)
    assert not K.sampling_product_possible(8, 50257, 768, torch.float32)
    assert K.sampling_product_possible(40, 50257, 768, torch.bfloat16)
    with pytest.raises(K.KernelError):
        K.linear_sample(a, w, None, K.SampleInto(torch.empty(40, dtype=torch.int32, device=DEV)))


def test_sample_follows_the_softmax(K):
    vocab, n = 8, 20000
    row = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, -2.0, 1.5, -0.5])
    logits = row.repeat(n, 1).to(DEV)
    temp = 0.8
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    K.sample(logits, torch.full((n,), temp, device=DEV), None, None,
             torch.arange(n, dtype=torch.int64, device=DEV), torch.zeros(n, dtype=torch.int32, device=DEV), out)
    freq = torch.bincount(out.cpu().long(), minlength=vocab).double() / n
    p = torch.softmax(row.double() / temp, -1)
    assert (freq - p).abs().max() < 4 * math.sqrt(0.25 / n) + 1e-3
    # the same (seed, counter) gives the same token whatever row it sits in
    out2 = torch.empty(5, dtype=torch.int32, device=DEV)
    K.sample(logits[:5], torch.full((5,), temp, device=DEV), None, None,
             torch.tensor([9, 3, 9, 9, 3], dtype=torch.int64, device=DEV),
             torch.tensor([1, 1, 1, 2, 1], dtype=torch.int32, device=DEV), out2)
    o = out2.cpu().tolist()
    assert o[0] == o[2] and o[1] == o[4]
