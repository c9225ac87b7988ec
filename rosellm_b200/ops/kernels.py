"""Python faces of the CUDA kernels: argument checks, then one call into the library.

Every function takes CUDA tensors, launches on torch's current stream and
returns nothing the host has to wait for.  There is no CPU or library
fallback: without a GPU, or without the built library, a call raises.
Sizes a kernel cannot take are refused here with an error that says why.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from . import build

F32, BF16 = 0, 1
ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2
ACTIVATIONS = {"none": ACT_NONE, "gelu_tanh": ACT_GELU_TANH, "gelu_erf": ACT_GELU_ERF}

STATUS_BITS = {
    1: "a token id outside the embedding table",
    2: "a position outside the position table or the sequence limit",
    4: "a block table without a page where the step reads or writes",
    8: "a bounded wait inside a kernel gave up",
}

# Rows up to which a matrix product streams the weights once per group of rows
# instead of tiling: float32 products up to 64 rows (csrc/gemm_simt.cu), then 64x64 tiles in
# IEEE arithmetic on the CUDA cores; bfloat16 products up to 16 rows the weight-streaming mma
# kernel (csrc/gemm_rows_mma.cu), and up to 64 rows too unless the output is wide; otherwise
# tcgen05, clustered (csrc/gemm_tc_rows.cu) or with 128-row tiles (csrc/gemm_tc.cu): bf16_path.
ROWS_STREAMING_LIMIT = 64


class KernelError(RuntimeError):
    pass


_signatures_set = False
_status: dict[int, torch.Tensor] = {}
_launches = 0


def launches() -> int:
    """How many kernels of this library have been launched by this process."""
    return _launches


_loaded = None
_recorder = None  # a LaunchList being filled (see ``recording``)


class LaunchList:
    """The library calls of one step, with their arguments, in order.

    What a step launches depends on its sizes, not on its contents (those lie in device
    buffers whose addresses stay): a step of sizes seen before can issue the recorded calls
    again instead of walking through the parts and the checked wrappers a second time.
    """

    def __init__(self) -> None:
        self.calls: list[tuple] = []  # (library function, arguments without the stream)
        self.launches = 0             # kernels these calls launch
        self.result = None            # whatever the recorded code returned (set by the caller)

    def replay(self) -> None:
        global _launches
        stream = _stream()
        for fn, args in self.calls:
            rc = fn(*args, stream)
            if rc != 0:
                raise KernelError(f"{fn.__name__}: code {rc} when a recorded launch was issued again")
        _launches += self.launches


class _RecordingLib:
    """Stands for the library while a ``LaunchList`` is filled: every launch is made and noted."""

    def __init__(self, lib, into: LaunchList) -> None:
        self._lib, self._into = lib, into

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if name in _QUERIES:
            return fn

        def call(*args):
            self._into.calls.append((fn, args[:-1]))  # the stream is every launch's last argument
            return fn(*args)

        return call


_QUERIES = ("rl_gemm_tc_rows_fits", "rl_gemm_rows_smem_fits", "rl_mlp_fused_slice", "rl_attn_block_fused_fits", "rl_attn_block_fused_cluster",
            "rl_host_memory_on_device")  # library functions that launch nothing


class recording:
    """``with recording() as launches:`` notes every library launch made inside."""

    def __enter__(self) -> LaunchList:
        global _recorder
        if _recorder is not None:
            raise KernelError("launches are being recorded already")
        self._list = LaunchList()
        self._before = _launches
        _recorder = _RecordingLib(_lib(), self._list)
        return self._list

    def __exit__(self, *exc) -> None:
        global _recorder
        _recorder = None
        self._list.launches = _launches - self._before


def _lib() -> ctypes.CDLL:
    global _signatures_set, _loaded
    if _recorder is not None:
        return _recorder
    if _loaded is not None:
        return _loaded
    lib = build.load()
    if not _signatures_set:
        P, I, L, F = c_void_p, c_int, c_long, c_float
        lib.rl_embed.argtypes = [I, P, P, P, P, P, I, I, I, I, P, P, I, P]
        lib.rl_layernorm.argtypes = [I, P, P, P, P, P, I, I, F, P]
        lib.rl_gemm_simt.argtypes = [I, I, P, L, P, P, P, L, I, I, I, I, I, I, P, P, I, P, P, P,
                                     I, I, I, I, I, I, P, P]
        lib.rl_gemm_rows_bf16.argtypes = [I, P, L, P, P, P, L, I, I, I, I, I, P, L, P, P, F, P, P, I, P, P, P,
                                          I, I, I, I, I, I, P, P]
        lib.rl_gemm_rows_bf16_sample.argtypes = [P, L, P, P, I, I, I, P, L, P, P, F, P, P, P, P, P, P, P, I, P, P, P]
        lib.rl_host_memory_on_device.argtypes = [P]
        lib.rl_host_memory_on_device.restype = ctypes.c_ulonglong
        lib.rl_gemm_rows_bulk_enable.argtypes = [I]
        lib.rl_gemm_rows_bulk_enable.restype = None
        lib.rl_gemm_tc.argtypes = [I, P, L, P, P, P, L, I, I, I, I, I, P, P, I, P, P, P, I, I, I, I, I, I, P, P]
        lib.rl_gemm_tc_sample.argtypes = [P, L, P, P, I, I, I, P, P, P, P, P, P, P, I, P, P, P]
        lib.rl_gemm_tc_cut.argtypes = [I, P, L, P, P, P, L, I, I, I, I, I, P, P, I, P, P, P, I, I, I, I, I, I, P, I, I, P]
        lib.rl_gemm_tc_rows.argtypes = [I, P, L, P, P, P, L, I, I, I, I, I, P, P, I, P, P, P, I, I, I, I, I, I, P, P]
        lib.rl_gemm_tc_rows_fits.argtypes = [I, I, I]
        lib.rl_gemm_rows_smem.argtypes = [I, P, L, P, P, P, L, I, I, I, I, I, P, P, I, P, P, P, I, I, I, I, I, I, P, P]
        lib.rl_gemm_rows_smem_fits.argtypes = [I, I, I, I, I, I, I]
        lib.rl_copy_to_device.argtypes = [P, P, L, P]
        lib.rl_event_record.argtypes = [P, P]
        lib.rl_attention.argtypes = [I, P, L, P, P, I, P, P, P, P, L, I, I, I, I, I, F, P, I, P, I, P, I, I, I, P, P, I, L, I, I, P, P]
        lib.rl_kv_write.argtypes = [I, P, P, L, P, P, I, P, P, P, I, I, I, I, I, P, P]
        lib.rl_sample.argtypes = [P, L, I, I, P, P, P, P, P, P, P, I, P, P, I, P]
        lib.rl_mlp_fused_slice.argtypes = [I, I, I, I]
        lib.rl_attn_block_fused_fits.argtypes = [I, I, I, I]
        lib.rl_attn_block_fused_cluster.argtypes = [I, I, I]
        lib.rl_attn_block_fused.argtypes = [P, L, P, P, F, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, P, P]
        lib.rl_mlp_fused.argtypes = [P, L, P, L, P, P, F, P, P, P, P, I, I, I, I, I, P, P]
        for name in ("rl_copy_to_device", "rl_event_record", "rl_embed", "rl_layernorm", "rl_gemm_simt", "rl_gemm_tc", "rl_gemm_tc_sample", "rl_gemm_tc_cut", "rl_gemm_tc_rows", "rl_gemm_tc_rows_fits",
                     "rl_gemm_rows_smem", "rl_gemm_rows_smem_fits",
                     "rl_gemm_rows_bf16", "rl_gemm_rows_bf16_sample", "rl_attention", "rl_kv_write", "rl_sample", "rl_mlp_fused_slice", "rl_mlp_fused",
                     "rl_attn_block_fused_fits", "rl_attn_block_fused_cluster", "rl_attn_block_fused"):
            getattr(lib, name).restype = I
        _signatures_set = True
    _loaded = lib
    return lib


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {t.dtype}; float32 or bfloat16")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle (asked for at every launch: the raw call costs a
    tenth of a microsecond, ``torch.cuda.current_stream()`` several)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, name: str, dtype: torch.dtype | None = None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _ok(rc: int, what: str) -> None:
    global _launches
    _launches += 1
    if rc != 0:
        if rc > 0:
            raise KernelError(f"{what}: CUDA error {rc} at launch")
        raise KernelError(f"{what}: refused its arguments (code {rc})")


def status_word(device: torch.device) -> torch.Tensor:
    """The int32 word kernels OR error bits into (one per device)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device: torch.device) -> None:
    """Read the status word (waits for the stream) and raise if a kernel flagged its inputs."""
    word = status_word(device)
    bits = int(word.item())
    if bits:
        word.zero_()
        why = "; ".join(text for bit, text in STATUS_BITS.items() if bits & bit)
        raise KernelError(f"a kernel refused part of its input: {why}")


def copy_to_device(dst: torch.Tensor, src: torch.Tensor, n: int, offset: int = 0) -> None:
    """dst[offset:offset + n] = src[offset:offset + n] for a device tensor and a pinned host tensor
    of the same element type (both contiguous), ordered on the current stream; the host side must
    stay as it is until the stream has passed the copy."""
    if not dst.is_cuda or src.is_cuda or not src.is_pinned() or dst.dtype != src.dtype:
        raise KernelError("copy_to_device: a device tensor and a pinned host tensor of one element type are needed")
    if offset < 0 or n < 0 or offset + n > min(dst.numel(), src.numel()):
        raise KernelError("copy_to_device: the range lies outside the tensors")
    size = dst.element_size()
    rc = _lib().rl_copy_to_device(dst.data_ptr() + offset * size, src.data_ptr() + offset * size, n * size, _stream())
    if rc != 0:  # not a kernel: it does not count as a launch
        raise KernelError(f"copy_to_device: CUDA error {rc}")


def copy_to_device_raw(dst_ptr: int, src_ptr: int, n_bytes: int) -> None:
    """The same for addresses the caller has checked once (buffers it keeps for the purpose):
    nothing is looked up or checked here, a step makes two such copies."""
    rc = _lib().rl_copy_to_device(dst_ptr, src_ptr, n_bytes, _stream())
    if rc != 0:
        raise KernelError(f"copy_to_device: CUDA error {rc}")


def record_event(event: "torch.cuda.Event") -> None:
    """``event.record()`` on the current stream; after the event's first use, by the plain runtime
    call on its handle (the framework's own call looks the stream object up each time)."""
    handle = event.cuda_event
    if not handle:
        event.record()
        return
    rc = _lib().rl_event_record(handle, _stream())
    if rc != 0:
        raise KernelError(f"record_event: CUDA error {rc}")


def embed(token_ids, positions, table, pos_table, out, feedback=None) -> None:
    """out[n] = table[token_ids[n]] (+ pos_table[positions[n]]), float32 [tokens, hidden].
    With ``feedback`` (int32), an id -(r+1) is replaced on the device by ``feedback[r]``."""
    _need(token_ids, "token_ids", torch.int32)
    _need(table, "table")
    _need(out, "out", torch.float32)
    n, hidden = out.shape
    if table.shape[1] != hidden:
        raise KernelError("table width differs from out")
    n_pos = 0
    if pos_table is not None:
        _need(pos_table, "pos_table", table.dtype)
        _need(positions, "positions", torch.int32)
        n_pos = pos_table.shape[0]
    rc = _lib().rl_embed(_code(table), _ptr(token_ids), _ptr(positions), _ptr(table), _ptr(pos_table),
                         _ptr(out), n, hidden, table.shape[0], n_pos, _ptr(status_word(out.device)),
                         _ptr(feedback), 0 if feedback is None else feedback.numel(), _stream())
    _ok(rc, "embed")


def layernorm(x, gamma, beta, eps: float, out, rows=None) -> None:
    """out[i] = LayerNorm(x[rows[i]] or x[i]) * gamma + beta; x float32, out float32 or bfloat16."""
    _need(x, "x", torch.float32)
    _need(gamma, "gamma", torch.float32)
    if beta is not None:
        _need(beta, "beta", torch.float32)
    _need(out, "out")
    hidden = x.shape[1]
    n_out = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() < n_out:
            raise KernelError("rows shorter than out")
    elif x.shape[0] < n_out:
        raise KernelError("x has fewer rows than out")
    if out.shape[1] != hidden or gamma.numel() != hidden:
        raise KernelError("layernorm: widths differ")
    rc = _lib().rl_layernorm(_code(out), _ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out),
                             n_out, hidden, float(eps), _stream())
    if rc == -2:
        raise KernelError(f"layernorm: a row of {hidden} floats does not fit in shared memory")
    _ok(rc, "layernorm")


_device_facts: dict[int, tuple[int, int]] = {}
device_facts_given: tuple[int, int] | None = None  # set by tests that plan for a device they do not have


def device_facts(device: torch.device | None = None) -> tuple[int, int]:
    """(SMs, bytes of shared memory an SM has) of the device the kernels run on, asked once."""
    if device_facts_given is not None:
        return device_facts_given
    key = torch.cuda.current_device() if device is None or device.index is None else device.index
    have = _device_facts.get(key)
    if have is None:
        props = torch.cuda.get_device_properties(key)
        have = _device_facts[key] = (int(props.multi_processor_count), int(props.shared_memory_per_multiprocessor))
    return have


def sm_count(device: torch.device | None = None) -> int:
    return device_facts(device)[0]


def bf16_path(rows: int, n_out: int, k: int, *, residual: bool = False, out_f32: bool = False, act: int = ACT_NONE,
              to_cache: bool = False) -> str:
    """Which kernel a bfloat16 product of these sizes runs on (measured on B200 at the widths of
    GPT-2): up to 16 rows the weight-streaming mma kernel; 17 to 64 rows the kernel that keeps
    both operands in shared memory, unless the output alone has tiles enough to fill the SMs (the
    head: tcgen05 tiles) or its sizes do not fit (then the weight-streaming kernel, or for a long
    inner size the clustered tcgen05 kernel); up to 128 rows the clustered kernel when the output
    is too narrow to give the tiled kernel work; beyond, tcgen05 tiles."""
    if rows < 17:
        return "mma"
    if rows <= 64:
        if -(-n_out // 64) >= sm_count():
            return "tc"
        if ROWS_IN_SHARED_MEMORY and _lib().rl_gemm_rows_smem_fits(rows, n_out, k, int(residual), int(out_f32), act,
                                                                   int(to_cache)):
            return "smem"
        if rows > 32 and k >= 2048 and _lib().rl_gemm_tc_rows_fits(rows, n_out, k):
            return "tcr"
        return "mma"
    if rows <= 128 and n_out <= 1024 and _lib().rl_gemm_tc_rows_fits(rows, n_out, k):
        return "tcr"
    return "tc"


# The kernel of 17 to 64 rows that stages both operands in shared memory (csrc/gemm_rows_smem.cu);
# switched off, those products run as they did without it (for comparisons).
ROWS_IN_SHARED_MEMORY = True


def product_writes_cache(rows: int, dtype: torch.dtype, n_out: int = 0, k: int = 0) -> bool:
    """Whether ``linear`` on this many rows (``n_out`` output columns, inner size ``k``) runs a
    kernel into which the cache write after it can be fused."""
    if dtype == torch.float32:
        return rows <= ROWS_STREAMING_LIMIT
    return True  # every bfloat16 product kernel can scatter keys and values


# Most rows, and longest rows, for which a LayerNorm is computed inside the product that
# consumes it (csrc/gemm_rows_mma.cu).
FUSED_NORM_MAX_ROWS = 16
FUSED_NORM_MAX_WIDTH = 1024


class NormInput:
    """The input of a bfloat16 product given as "LayerNorm of these float32 rows": the row
    kernel normalises them itself (``linear(NormInput(...), ...)``)."""

    def __init__(self, x, gamma, beta, eps: float) -> None:
        self.x, self.gamma, self.beta, self.eps = x, gamma, beta, float(eps)

    @staticmethod
    def possible(rows: int, width: int, dtype: torch.dtype) -> bool:
        return dtype == torch.bfloat16 and rows <= FUSED_NORM_MAX_ROWS and width <= FUSED_NORM_MAX_WIDTH and width % 4 == 0


class KvTarget:
    """Where the key and value columns of a packed qkv product go instead of the output buffer."""

    def __init__(self, pool, block_table, positions, req_of_token, slots, q_width: int, max_pos: int) -> None:
        self.pool, self.block_table = pool, block_table
        self.positions, self.req_of_token, self.slots = positions, req_of_token, slots
        self.q_width, self.max_pos = q_width, max_pos


def linear(a, weight, bias, out, *, act: int = ACT_NONE, residual: bool = False, path: str | None = None,
           kv: KvTarget | None = None, tile_width: int = 0, splits: int = 0) -> None:
    """out = act(a @ weight.T + bias), or out += ... when residual (out float32).

    ``a`` may be a ``NormInput``: the product then normalises float32 rows itself (bfloat16,
    at most 16 rows).  Otherwise
    a [rows, k] (row stride a multiple of 8), weight [n, k] contiguous, both float32 or both
    bfloat16; out [rows, n] of a's dtype or float32.  Which kernel runs: float32 up to 64 rows
    the row kernel, above it 64x64 tiles (both IEEE FFMA); bfloat16 up to 16 rows the
    weight-streaming mma kernel (for a very wide float32 output, a head, its form that is fed by
    bulk copies: the library chooses), above it as ``bf16_path`` says.  ``path`` (for tests) forces
    ``"rows"``, ``"tile"``, ``"mma"``, ``"smem"``, ``"tc"`` or ``"tcr"``.  ``kv``: output columns from
    ``kv.q_width`` on are written into cache pages, not ``out`` (not with ``"tile"``).
    ``tile_width`` and ``splits`` (for tests and measurements, ``"tc"`` only): the columns of an
    output tile, a multiple of 32 up to 256, and the parts the inner size is cut into (1, 2, 3, 4, 6
    or 8: the blocks of a cluster take one each), instead of what the kernel would choose.
    """
    norm = a if isinstance(a, NormInput) else None
    _need(weight, "weight")
    _need(out, "out", contiguous=False)
    if norm is not None:
        _need(norm.x, "norm.x", torch.float32, contiguous=False)
        _need(norm.gamma, "norm.gamma", torch.float32)
        m, k = norm.x.shape
        if weight.dtype != torch.bfloat16 or not NormInput.possible(m, k, torch.bfloat16) or norm.x.stride(1) != 1 \
                or norm.x.stride(0) % 4 or norm.gamma.numel() != k or path not in (None, "mma"):
            raise KernelError("linear: a LayerNorm is fused only into bfloat16 row products of at most "
                              f"{FUSED_NORM_MAX_ROWS} rows of at most {FUSED_NORM_MAX_WIDTH} elements")
        a_dtype, a_ptr, lda = torch.bfloat16, None, 0
        path = "mma"
    else:
        _need(a, "a", weight.dtype, contiguous=False)
        m, k = a.shape
        if a.stride(1) != 1:
            raise KernelError("linear: rows of a must be contiguous")
        if a.stride(0) % 8 != 0 or a.data_ptr() % 16:
            raise KernelError(f"linear: the row stride {a.stride(0)} must be a multiple of 8 and a start on a 16-byte boundary")
        a_dtype, a_ptr, lda = a.dtype, a.data_ptr(), a.stride(0)
    n = weight.shape[0]
    if weight.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise KernelError(f"linear: shapes do not fit: input [{m}, {k}], weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if out.stride(1) != 1:
        raise KernelError("linear: rows of out must be contiguous")
    if k % 8 != 0:
        raise KernelError(f"linear: the inner size {k} must be a multiple of 8")
    if weight.data_ptr() % 16:
        raise KernelError("linear: operands must start on 16-byte boundaries")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != n:
            raise KernelError("linear: bias length differs from the output width")
    if residual and out.dtype != torch.float32:
        raise KernelError("linear: the residual stream is float32")
    if a_dtype == torch.float32 and out.dtype != torch.float32:
        raise KernelError("linear: float32 inputs give float32 outputs")
    bf16 = a_dtype == torch.bfloat16
    if path is None:
        if bf16:
            path = bf16_path(m, n, k, residual=residual, out_f32=out.dtype == torch.float32, act=act, to_cache=kv is not None)
        else:
            path = "rows" if m <= ROWS_STREAMING_LIMIT else "tile"
    if path in ("mma", "tc", "tcr", "smem") and not bf16:
        raise KernelError("linear: the tensor-core kernels take bfloat16 inputs")
    if path == "mma" and m > 64:
        raise KernelError("linear: the mma row kernel takes at most 64 rows")
    if path == "tcr" and not _lib().rl_gemm_tc_rows_fits(m, n, k):
        raise KernelError("linear: the clustered tcgen05 kernel takes at most 128 rows and an inner size that "
                          "fits the shared memory of eight blocks")
    if kv is not None and path == "tile":
        raise KernelError("linear: the 32-bit tile kernel does not write into the cache")
    if kv is not None and (act != ACT_NONE or residual):
        raise KernelError("linear: a product that writes keys and values has no activation and no residual")
    status = _ptr(status_word(out.device))
    kx = (None, None, 0, None, None, None, 0, 0, 0, 0, 0, 0)
    if kv is not None:
        _need(kv.pool, "kv.pool", a_dtype)
        _, two, n_kv, page_size, dh = kv.pool.shape
        if kv.q_width + 2 * n_kv * dh != n:
            raise KernelError("linear: the packed qkv width does not fit the cache's heads")
        kx = (kv.pool.data_ptr(), kv.block_table.data_ptr(), kv.block_table.stride(0), kv.positions.data_ptr(),
              kv.req_of_token.data_ptr(), kv.slots.data_ptr(), kv.q_width, n_kv * dh, dh, page_size, n_kv, kv.max_pos)
    if path == "smem":
        rc = _lib().rl_gemm_rows_smem(_code(out), a_ptr, lda, _ptr(weight), _ptr(bias), _ptr(out),
                                      out.stride(0), m, n, k, act, int(residual), *kx, status, _stream())
        if rc == -2:
            raise KernelError("linear: the shared-memory row kernel takes at most 64 rows, an even output width, and an "
                              "inner size of at most 1024 (longer only for out += ... into float32)")
        _ok(rc, "linear (rows in shared memory)")
    elif path == "tc":
        rc = _lib().rl_gemm_tc_cut(_code(out), a_ptr, lda, _ptr(weight), _ptr(bias), _ptr(out),
                                   out.stride(0), m, n, k, act, int(residual), *kx, status, tile_width, splits, _stream())
        if rc in (-10, -11):
            raise KernelError("linear: the driver refused to encode a TMA tensor map for these operands")
        _ok(rc, "linear (tcgen05)")
    elif path == "tcr":
        rc = _lib().rl_gemm_tc_rows(_code(out), a_ptr, lda, _ptr(weight), _ptr(bias), _ptr(out),
                                    out.stride(0), m, n, k, act, int(residual), *kx, status, _stream())
        if rc in (-10, -11):
            raise KernelError("linear: the driver refused to encode a TMA tensor map for these operands")
        _ok(rc, "linear (tcgen05 rows)")
    elif path == "mma":
        nx = (None, 0, None, None, 0.0)
        if norm is not None:
            nx = (norm.x.data_ptr(), norm.x.stride(0), norm.gamma.data_ptr(), _ptr(norm.beta), norm.eps)
        rc = _lib().rl_gemm_rows_bf16(_code(out), a_ptr, lda, _ptr(weight), _ptr(bias), _ptr(out),
                                      out.stride(0), m, n, k, act, int(residual), *nx, *kx, status, _stream())
        if rc == -6:
            raise KernelError("linear: the rows to normalise must be 16-byte aligned float32")
        _ok(rc, "linear (mma rows)")
    else:
        rows_limit = (1 << 30) if path == "rows" else 0
        rc = _lib().rl_gemm_simt(_code(weight), _code(out), a_ptr, lda, _ptr(weight), _ptr(bias), _ptr(out),
                                 out.stride(0), m, n, k, act, int(residual), rows_limit, *kx, status, _stream())
        _ok(rc, "linear")


class SampleInto:
    """Where a step's next tokens go when the head's product chooses them itself, and the rows'
    sampling options: device tensors whose addresses stay (captured graphs hold them).
    ``out_ids`` int32; ``temperature`` float32 (<= 0: arg-max), ``seeds`` int64, ``counters``
    int32, one entry a row, or all three ``None`` when every row takes the arg-max.
    ``host_ring`` (optional): pinned int32 host memory of ``SAMPLE_RING`` slots of ``ring_stride``
    ids that the kernel writes the ids to as well, with ``ring_step`` (device, one uint32-sized
    int32) counting the launches that have: launch number n (from 0) fills slot
    ``n % SAMPLE_RING``, so that the host needs no copy of its own to see the tokens."""

    def __init__(self, out_ids, temperature=None, seeds=None, counters=None, host_ring=None, ring_step=None) -> None:
        self.out_ids, self.temperature, self.seeds, self.counters = out_ids, temperature, seeds, counters
        self.host_ring, self.ring_step = host_ring, ring_step
        self.ring_address, self.ring_stride = 0, 0
        if host_ring is not None:
            if ring_step is None or not host_ring.is_pinned() or host_ring.dtype != torch.int32 \
                    or host_ring.numel() % SAMPLE_RING or not host_ring.is_contiguous():
                raise KernelError("SampleInto: the host ring is pinned int32 memory of SAMPLE_RING equal slots, "
                                  "with a device counter beside it")
            _need(ring_step, "ring_step", torch.int32)
            self.ring_address = host_memory_on_device(host_ring)
            self.ring_stride = host_ring.numel() // SAMPLE_RING
            if not self.ring_address:
                raise KernelError("SampleInto: the device cannot write to this host memory")


SAMPLE_RING = 4  # slots of a SampleInto's host ring (csrc/gemm_epilogue.cuh)


def host_memory_on_device(t: torch.Tensor) -> int:
    """The address under which kernels reach the pinned host tensor ``t`` (0: they cannot)."""
    if t.is_cuda or not t.is_pinned():
        return 0
    return int(_lib().rl_host_memory_on_device(t.data_ptr()))


# A head's product chooses the tokens in its epilogue where it runs on the weight-streaming
# kernel (up to 16 rows) or on tcgen05 tiles (more rows and an output wide enough to fill the
# SMs: ``bf16_path``); the kernels between them have no such epilogue.
SAMPLING_PRODUCT_MAX_ROWS = 1024  # words of scratch
_sampling_product_bufs: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}


def sampling_product_possible(rows: int, n_out: int, k: int, dtype: torch.dtype, with_temperature: bool = False) -> bool:
    """Whether ``linear_sample`` takes these sizes, and is the faster way: on tcgen05 tiles the
    few epilogue threads of a block are slower at the noise of rows with a temperature than the
    sampling kernel after an ordinary product (64 x 50257: 64 against 46 us; the arg-max alone:
    24 against 33), so such batches are left to that."""
    if dtype != torch.bfloat16 or not 0 < rows <= SAMPLING_PRODUCT_MAX_ROWS or k % 8:
        return False
    path = bf16_path(rows, n_out, k, out_f32=True)
    return path == "mma" or (path == "tc" and not with_temperature)


def linear_sample(a, weight, bias, into: SampleInto) -> None:
    """``into.out_ids[r]`` = the token ``sample`` would choose from row r of ``a @ weight.T + bias``
    (arg-max, or with a temperature the arg-max of logit / temperature + Gumbel noise), without
    the logits being written anywhere.  bfloat16, where ``sampling_product_possible``;
    ``a`` may be a ``NormInput`` as for ``linear``.  Rows with top-k or top-p need their logits:
    they are not for this call."""
    norm = a if isinstance(a, NormInput) else None
    _need(weight, "weight", torch.bfloat16)
    n, k = weight.shape
    if norm is not None:
        _need(norm.x, "norm.x", torch.float32, contiguous=False)
        _need(norm.gamma, "norm.gamma", torch.float32)
        m = norm.x.shape[0]
        if not NormInput.possible(m, k, torch.bfloat16) or norm.x.shape[1] != k or norm.x.stride(1) != 1 \
                or norm.x.stride(0) % 4 or norm.gamma.numel() != k:
            raise KernelError("linear_sample: a LayerNorm is fused only into bfloat16 row products of at most "
                              f"{FUSED_NORM_MAX_ROWS} rows of at most {FUSED_NORM_MAX_WIDTH} elements")
        a_ptr, lda = None, 0
        nx = (norm.x.data_ptr(), norm.x.stride(0), norm.gamma.data_ptr(), _ptr(norm.beta), norm.eps)
    else:
        _need(a, "a", torch.bfloat16, contiguous=False)
        m = a.shape[0]
        if a.shape[1] != k or a.stride(1) != 1 or a.stride(0) % 8 or a.data_ptr() % 16:
            raise KernelError("linear_sample: a must be [rows, k] with contiguous rows, a row stride that is a "
                              "multiple of 8 and a start on a 16-byte boundary")
        a_ptr, lda = a.data_ptr(), a.stride(0)
        nx = (None, 0, None, None, 0.0)
    if not sampling_product_possible(m, n, k, torch.bfloat16) or weight.data_ptr() % 16:
        raise KernelError("linear_sample: rows and an output width that the weight-streaming or the tcgen05 product "
                          "takes, an inner size that is a multiple of 8 and weights on a 16-byte boundary")
    path = bf16_path(m, n, k, out_f32=True)
    if norm is not None and path != "mma":
        raise KernelError("linear_sample: a LayerNorm is fused only into the weight-streaming product")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != n:
            raise KernelError("linear_sample: bias length differs from the output width")
    _need(into.out_ids, "out_ids", torch.int32)
    if into.out_ids.numel() < m:
        raise KernelError("linear_sample: out_ids is shorter than the number of rows")
    given = [t is not None for t in (into.temperature, into.seeds, into.counters)]
    if any(given) and not all(given):
        raise KernelError("linear_sample: temperature, seeds and counters come together")
    for t, name, dt in ((into.temperature, "temperature", torch.float32), (into.seeds, "seeds", torch.int64),
                        (into.counters, "counters", torch.int32)):
        if t is not None:
            _need(t, name, dt)
            if t.numel() < m:
                raise KernelError(f"linear_sample: {name} is shorter than the number of rows")
    key = weight.device.index if weight.device.index is not None else torch.cuda.current_device()
    bufs = _sampling_product_bufs.get(key)
    if bufs is None:  # best words and ticket: zero between launches
        bufs = _sampling_product_bufs[key] = (
            torch.zeros(SAMPLING_PRODUCT_MAX_ROWS, dtype=torch.int64, device=weight.device),
            torch.zeros(1, dtype=torch.int32, device=weight.device))
    if into.ring_address and into.ring_stride < m:
        raise KernelError("linear_sample: the host ring's slots are shorter than the number of rows")
    ring = (into.ring_address or None, into.ring_stride, _ptr(into.ring_step) if into.ring_address else None)
    if path == "tc":
        rc = _lib().rl_gemm_tc_sample(a_ptr, lda, _ptr(weight), _ptr(bias), m, n, k, _ptr(into.temperature),
                                      _ptr(into.seeds), _ptr(into.counters), _ptr(into.out_ids), _ptr(bufs[0]),
                                      _ptr(bufs[1]), *ring, _ptr(status_word(weight.device)), _stream())
        if rc in (-10, -11):
            raise KernelError("linear_sample: the driver refused to encode a TMA tensor map for these operands")
        _ok(rc, "linear_sample (tcgen05)")
        return
    rc = _lib().rl_gemm_rows_bf16_sample(a_ptr, lda, _ptr(weight), _ptr(bias), m, n, k, *nx, _ptr(into.temperature),
                                         _ptr(into.seeds), _ptr(into.counters), _ptr(into.out_ids), _ptr(bufs[0]),
                                         _ptr(bufs[1]), *ring, _ptr(status_word(weight.device)), _stream())
    _ok(rc, "linear_sample")


def rows_bulk_kernel(on: bool) -> None:
    """Heads of few rows on the kernel that has their weights copied into shared memory by the
    copy engine (the default), or on the weight-streaming kernel as every other product of few
    rows (for comparisons and measurements)."""
    build.load().rl_gemm_rows_bulk_enable(int(on))


# The fused kernels of a decode layer (csrc/mlp_fused.cu) are taken where their sizes fit;
# switched off, every layer runs as separate products (for comparisons and measurements).
FUSED_ROWS = True
_mlp_slices: dict[tuple, int] = {}


def mlp_fused_slice(rows: int, hidden: int, inner: int, norm: bool, dtype: torch.dtype) -> int:
    """How wide a slice of the inner width a block of the fused feed-forward kernel takes for
    these sizes; 0 when that kernel does not take them (more than 16 rows, a 32-bit model, a
    width whose slices do not fit shared memory) or is switched off."""
    if not FUSED_ROWS or dtype != torch.bfloat16 or rows > 16:
        return 0
    key = (rows, hidden, inner, norm)
    got = _mlp_slices.get(key)
    if got is None:
        got = _mlp_slices[key] = int(_lib().rl_mlp_fused_slice(rows, hidden, inner, int(norm)))
    return got


def mlp_pack_out_weight(w_out: torch.Tensor, slice_width: int) -> torch.Tensor:
    """``w_out`` [hidden, inner] as the fused feed-forward kernel reads it: [slices, hidden,
    slice_width + 8], slice s holding ``w_out[:, s*slice_width : (s+1)*slice_width]`` followed by
    eight zero columns (the padding its rows have in shared memory), units beyond ``inner`` zero.
    A block then fetches its slice with one copy instead of one per row."""
    hidden, inner = w_out.shape
    n = -(-inner // slice_width)
    wide = torch.zeros(hidden, n * slice_width, dtype=w_out.dtype, device=w_out.device)
    wide[:, :inner] = w_out
    packed = torch.zeros(n, hidden, slice_width + 8, dtype=w_out.dtype, device=w_out.device)
    packed[:, :, :slice_width] = wide.view(hidden, n, slice_width).permute(1, 0, 2)
    return packed.contiguous()


def mlp_fused(x, h, w_in, b_in, w_out_packed, b_out, *, act: int, slice_width: int) -> None:
    """x += act(h @ w_in.T + b_in) @ w_out.T + b_out for at most 16 rows, in one kernel.

    x float32 [rows, hidden] (the residual stream); ``h`` the bfloat16 input rows, or a
    ``NormInput`` over ``x`` itself (the kernel then normalises the rows); w_in [inner, hidden]
    bfloat16; ``w_out_packed``: ``mlp_pack_out_weight(w_out, slice_width)``; biases float32 or
    ``None``.  ``slice_width``: what ``mlp_fused_slice`` returned.  The sum over slices of the inner width is taken with
    float32 atomic additions: its order, and so its last bits, may differ from run to run.
    """
    _need(x, "x", torch.float32, contiguous=False)
    _need(w_in, "w_in", torch.bfloat16)
    _need(w_out_packed, "w_out_packed", torch.bfloat16)
    rows, hidden = x.shape
    inner = w_in.shape[0]
    if w_in.shape[1] != hidden or slice_width <= 0 \
            or tuple(w_out_packed.shape) != (-(-inner // slice_width), hidden, slice_width + 8):
        raise KernelError(f"mlp_fused: weights {tuple(w_in.shape)} and (packed) {tuple(w_out_packed.shape)} do not fit "
                          f"rows of {hidden} and slices of {slice_width}")
    norm = h if isinstance(h, NormInput) else None
    if norm is not None:
        if norm.x.data_ptr() != x.data_ptr() or norm.x.stride(0) != x.stride(0):
            raise KernelError("mlp_fused: the fused norm reads the residual stream it adds to")
        a_ptr, lda, gamma, beta, eps = None, 0, norm.gamma.data_ptr(), _ptr(norm.beta), norm.eps
    else:
        _need(h, "h", torch.bfloat16, contiguous=False)
        if tuple(h.shape) != (rows, hidden) or h.stride(1) != 1:
            raise KernelError("mlp_fused: input rows do not fit the residual stream")
        a_ptr, lda, gamma, beta, eps = h.data_ptr(), h.stride(0), None, None, 0.0
    for b, n, name in ((b_in, inner, "b_in"), (b_out, hidden, "b_out")):
        if b is not None:
            _need(b, name, torch.float32)
            if b.numel() != n:
                raise KernelError(f"mlp_fused: {name} has {b.numel()} entries, not {n}")
    rc = _lib().rl_mlp_fused(x.data_ptr(), x.stride(0), a_ptr, lda, gamma, beta, eps, w_in.data_ptr(), _ptr(b_in),
                             w_out_packed.data_ptr(), _ptr(b_out), rows, hidden, inner, slice_width, act,
                             _ptr(status_word(x.device)), _stream())
    if rc == -2:
        raise KernelError(f"mlp_fused: sizes not taken (rows {rows}, hidden {hidden}, inner {inner}, slice {slice_width})")
    _ok(rc, "mlp_fused")


_attn_block_fits: dict[tuple, bool] = {}


def attn_block_fused_fits(rows: int, hidden: int, n_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the fused attention kernel of a decode step (csrc/attn_block_fused.cu) takes these
    sizes: bfloat16, at most 16 rows, hidden = heads x head size up to 1024, head size 16, 32, 64
    or 128, and a grid (heads x up to 8 blocks) that the device holds at once."""
    if not FUSED_ROWS or dtype != torch.bfloat16 or rows > 16:
        return False
    key = (rows, hidden, n_heads, head_dim)
    got = _attn_block_fits.get(key)
    if got is None:
        got = _attn_block_fits[key] = bool(_lib().rl_attn_block_fused_fits(rows, hidden, n_heads, head_dim))
    return got


def attn_block_fused_cluster(hidden: int, n_heads: int, head_dim: int, dtype: torch.dtype) -> int:
    """Blocks that share a head in the fused attention kernel at these sizes (0: not taken)."""
    if dtype != torch.bfloat16:
        return 0
    return int(_lib().rl_attn_block_fused_cluster(hidden, n_heads, head_dim))


def attn_pack_out_weight(w_out: torch.Tensor, n_heads: int, head_dim: int, cluster: int) -> torch.Tensor:
    """``w_out`` [hidden, hidden] as the fused attention kernel reads it: [heads, cluster, NO,
    head_dim + 8] with NO = hidden / cluster rounded up to a multiple of 8; slice (h, c) holds
    ``w_out[c*NO : (c+1)*NO, h*head_dim : (h+1)*head_dim]`` (rows beyond hidden zero) followed by
    eight zero columns, the padding its rows have in shared memory."""
    hidden = w_out.shape[0]
    no = -(-(hidden // 8) // cluster) * 8
    tall = torch.zeros(cluster * no, hidden, dtype=w_out.dtype, device=w_out.device)
    tall[:hidden] = w_out
    packed = torch.zeros(n_heads, cluster, no, head_dim + 8, dtype=w_out.dtype, device=w_out.device)
    packed[..., :head_dim] = tall.view(cluster, no, n_heads, head_dim).permute(2, 0, 1, 3)
    return packed.contiguous()


def attn_block_fused(x, norm: NormInput, w_qkv, b_qkv, w_out_packed, b_out, pool, block_table, positions, slots, *,
                     n_heads: int, scale: float, max_pos: int) -> None:
    """x += (attention of LayerNorm(x) over the cache) @ w_out.T + b_out, for a step in which every
    row is the new token of a decoded request (row r: request r, at ``positions[r]``, block-table
    row ``slots[r]``; a negative slot marks a padding row).  The new keys and values are written
    to their pages.  One kernel; the keys below each request's new position must be of earlier
    steps, and the sum over heads is taken with float32 atomic additions, in no fixed order.
    ``w_out_packed``: ``attn_pack_out_weight(w_out, ...)``."""
    _need(x, "x", torch.float32, contiguous=False)
    _need(w_qkv, "w_qkv", torch.bfloat16)
    _need(w_out_packed, "w_out_packed", torch.bfloat16)
    _need(pool, "pool", torch.bfloat16)
    rows, hidden = x.shape
    _, two, n_kv, page_size, dh = pool.shape
    if norm.x.data_ptr() != x.data_ptr() or norm.x.stride(0) != x.stride(0):
        raise KernelError("attn_block_fused: the fused norm reads the residual stream it adds to")
    if n_kv != n_heads or n_heads * dh != hidden or tuple(w_qkv.shape) != (3 * hidden, hidden):
        raise KernelError("attn_block_fused: as many key/value heads as heads, hidden = heads x head size")
    cluster = attn_block_fused_cluster(hidden, n_heads, dh, torch.bfloat16)
    if cluster == 0 or tuple(w_out_packed.shape) != (n_heads, cluster, -(-(hidden // 8) // cluster) * 8, dh + 8):
        raise KernelError("attn_block_fused: the output matrix is not laid out for these sizes (attn_pack_out_weight)")
    for b, n, name in ((b_qkv, 3 * hidden, "b_qkv"), (b_out, hidden, "b_out")):
        if b is not None:
            _need(b, name, torch.float32)
            if b.numel() != n:
                raise KernelError(f"attn_block_fused: {name} has {b.numel()} entries, not {n}")
    _need(positions, "positions", torch.int32)
    _need(slots, "slots", torch.int32)
    if positions.numel() < rows or slots.numel() < rows:
        raise KernelError("attn_block_fused: a position and a slot for every row")
    rc = _lib().rl_attn_block_fused(x.data_ptr(), x.stride(0), norm.gamma.data_ptr(), _ptr(norm.beta), norm.eps,
                                    w_qkv.data_ptr(), _ptr(b_qkv), w_out_packed.data_ptr(), _ptr(b_out), pool.data_ptr(),
                                    block_table.data_ptr(), block_table.stride(0), positions.data_ptr(),
                                    slots.data_ptr(), rows, hidden, n_heads, dh, page_size, max_pos, float(scale),
                                    _ptr(status_word(x.device)), _stream())
    if rc == -2:
        raise KernelError(f"attn_block_fused: sizes not taken (rows {rows}, hidden {hidden}, heads {n_heads} of {dh})")
    _ok(rc, "attn_block_fused")


def kv_write(k, v, pool, block_table, positions, req_of_token, slots, max_pos: int) -> None:
    """Copy the step's keys and values [tokens, kv heads*head dim] (views with a row stride)
    into the pages ``block_table[slots[req_of_token[n]]][positions[n] // page]``."""
    _need(k, "k", contiguous=False)
    _need(v, "v", k.dtype, contiguous=False)
    _need(pool, "pool", k.dtype)
    _need(block_table, "block_table", torch.int32)
    n_tokens = k.shape[0]
    _, two, n_kv, page_size, dh = pool.shape
    if two != 2 or k.shape[1] != n_kv * dh or k.stride(1) != 1 or v.stride(1) != 1 or k.stride(0) != v.stride(0):
        raise KernelError("kv_write: keys/values do not fit the pool")
    if dh % 16 != 0:
        raise KernelError(f"kv_write: head size {dh} is not a multiple of 16")
    if k.data_ptr() % 16 or v.data_ptr() % 16 or k.stride(0) % 8:
        raise KernelError("kv_write: key and value rows must start on 16-byte boundaries")
    rc = _lib().rl_kv_write(_code(k), _ptr(k), _ptr(v), k.stride(0), _ptr(pool), _ptr(block_table),
                            block_table.stride(0), _ptr(positions), _ptr(req_of_token), _ptr(slots),
                            n_tokens, n_kv, dh, page_size, block_table.shape[1] * page_size,
                            _ptr(status_word(k.device)), _stream())
    _ok(rc, "kv_write")


def attention(q, pool, block_table, q_start, kv_len, slots, out, *, n_heads: int, scale: float,
              window: int | None, tiles, n_tiles: int, decode_reqs, n_decode: int,
              n_splits: int = 1, part_o=None, part_ml=None, tiles_wide=None, n_tiles_wide: int = 0,
              decode_wide: bool = False, prefill_path: str | None = None, old_keys_settled: bool = False) -> None:
    """Causal attention of the step's queries over the paged cache (see csrc/attention.cu).

    q [tokens, heads*head dim] (a view with a row stride), out the same shape; ``tiles``
    int32 [n_tiles, 2] lists (request, first query) of 16-query tiles of prompt portions,
    ``decode_reqs`` int32 [n_decode] the requests with one query.  ``tiles_wide``: the
    portions again as 64-query tiles, used instead of ``tiles`` by the tensor-core kernel
    (bfloat16, head size up to 128).  ``decode_wide``: the blocks of decoded requests have
    sixteen warps instead of four (few requests, so that their keys need no split).
    ``prefill_path`` (for tests): ``"tc"`` or ``"mma"`` forces the kernel of the prompt portions.
    ``old_keys_settled``: the caller promises that the block table and the keys and values below
    each decoded request's last position were written by work that was over before the kernel
    preceding this call on the stream began (true inside the engine, whose steps are separated
    by a copy to the device); the decode kernel then fetches them before it waits for the
    kernels ahead of it.  Off, it reads nothing before that wait, and a cache write issued just
    before this call is seen.
    """
    _need(q, "q", contiguous=False)
    _need(pool, "pool", q.dtype)
    _need(out, "out", q.dtype, contiguous=False)
    _, two, n_kv, page_size, dh = pool.shape
    if dh % 16 != 0 or dh > 256:
        raise KernelError(f"attention: head size {dh} must be a multiple of 16, at most 256")
    if n_heads % n_kv != 0:
        raise KernelError(f"attention: {n_heads} heads are not a multiple of {n_kv} key/value heads")
    if q.shape[1] != n_heads * dh or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention: q does not fit heads * head size")
    if n_splits > 1:
        need = n_decode * n_heads * n_splits
        if part_o is None or part_ml is None or part_o.numel() < need * dh or part_ml.numel() < need * 2:
            raise KernelError("attention: scratch for the split partial results is too small")
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
    rc = _lib().rl_attention(_code(q), _ptr(q), q.stride(0), _ptr(pool), _ptr(block_table), block_table.stride(0),
                             _ptr(q_start), _ptr(kv_len), _ptr(slots), _ptr(out), out.stride(0),
                             n_heads, n_kv, dh, page_size, int(window or 0), float(scale),
                             _ptr(tiles), n_tiles, _ptr(tiles_wide), n_tiles_wide if tiles_wide is not None else 0,
                             _ptr(decode_reqs), n_decode, n_splits, int(decode_wide),
                             _ptr(part_o), _ptr(part_ml), q.shape[0], pool.shape[0],
                             {None: 0, "mma": 1, "tc": 2}[prefill_path], int(old_keys_settled),
                             _ptr(status_word(q.device)), _stream())
    if rc == -5:
        raise KernelError("attention: the tcgen05 kernel takes bfloat16, head size 64, no window and pages of "
                          "8 to 128 tokens that divide 128")
    _ok(rc, "attention")
    global _launches
    _launches += (1 if n_tiles and n_decode else 0) + (1 if n_decode and n_splits > 1 else 0)


def sample(logits, temperature, top_k, top_p, seeds, counters, out_ids, kept=None, filtered: bool | None = None) -> None:
    """One token per row of float32 logits.  Rows with temperature <= 0 take the arg-max.

    temperature float32, top_k int32 (0: off), top_p float32 (>= 1: off), seeds int64,
    counters int32 (index of the generated token within its request), out_ids int32.
    ``filtered``: whether any row has top-k or top-p switched on (``None``: not known; the
    kernel for such rows is then launched whenever ``top_k`` or ``top_p`` is given).
    """
    _need(logits, "logits", torch.float32, contiguous=False)
    if logits.stride(1) != 1:
        raise KernelError("sample: rows of logits must be contiguous")
    n, vocab = logits.shape
    for t, name, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                        (top_p, "top_p", torch.float32), (seeds, "seeds", torch.int64),
                        (counters, "counters", torch.int32)):
        if t is not None:
            _need(t, name, dt)
            if t.numel() < n:
                raise KernelError(f"sample: {name} is shorter than the number of rows")
    if temperature is not None and (seeds is None or counters is None):
        raise KernelError("sample: sampling rows need seeds and counters")
    _need(out_ids, "out_ids", torch.int32)
    n_chunks = SAMPLE_CHUNKS if vocab >= 4096 else 1
    part = tickets = None
    if n_chunks > 1:
        part, tickets = _sample_scratch(logits.device, n)
    rc = _lib().rl_sample(_ptr(logits), logits.stride(0), n, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p),
                          _ptr(seeds), _ptr(counters), _ptr(out_ids), _ptr(kept), n_chunks, _ptr(part),
                          _ptr(tickets), int(filtered is None or bool(filtered)), _stream())
    _ok(rc, "sample")


# Blocks that share a row of a large vocabulary in the sampling kernel.
SAMPLE_CHUNKS = 32
_sample_bufs: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}


def _sample_scratch(device: torch.device, rows: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Partial winners and tickets of the sampling kernel; the tickets are zero between calls."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    have = _sample_bufs.get(key)
    if have is None or have[1].numel() < rows:
        cap = max(256, rows)
        have = (torch.empty(cap * SAMPLE_CHUNKS * 2, dtype=torch.float32, device=device),
                torch.zeros(cap, dtype=torch.int32, device=device))
        _sample_bufs[key] = have
    return have
