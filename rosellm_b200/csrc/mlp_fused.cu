// The feed-forward of a layer for at most 16 rows (decoded tokens, short portions) in ONE kernel:
//   x += act(LN(x) W_in^T + b_in) W_out^T + b_out        (rosellm/rosetrainer/model.py:331-349, 419-428)
// where the unfused path runs two weight-streaming products with the inner activations [rows, F]
// going through global memory in between.
//
// Such a step is bound by latency, not by bytes: each product of a decode step waits for the
// kernel ahead of it, then for its weights, then sums over K.  Here a block owns a slice of the
// inner width F.  Its two weight slices (rows [f0, f0+fs) of W_in, columns [f0, f0+fs) of W_out)
// are weights, which no kernel writes, so their copies into shared memory are issued BEFORE the
// block waits for the kernels ahead (programmatic dependent launch): they travel while the
// kernel ahead still runs.  After the wait the block normalises the rows (float32 statistics,
// as csrc/gemm_rows_mma.cu does), multiplies them by its slice of W_in on mma.sync m16n8k16,
// applies bias and activation, multiplies the [16, fs] result by its slice of W_out and adds the
// [rows, hidden] partial result into the float32 residual stream with red.global.add: the sum
// over the slices of F is taken by the memory system, in whatever order the blocks arrive.
// (tcgen05 is for many rows; with 16 rows a 128-lane tile would be seven eighths padding.)
//
// Sums of float32 in an order that differs from run to run differ by rounding (1e-7 relative),
// which is four orders below what bfloat16 activations carry; the 32-bit mode never takes this
// kernel.
//
// The rows that are normalised and the rows that are added to are the same memory, so no block
// may add before every block has taken its copy of the rows.  A seventeenth warp of each block
// does that talking while the sixteen others compute: it announces (one atomic on a counter)
// that the block's rows have been read as soon as they have, then watches for the last block's
// announcement; the computing warps ask it just before their additions, two products and an
// activation later.  All blocks of the grid must therefore run at once; the entry point refuses
// grids that the device does not hold in one wave.
#include "gemm_epilogue.cuh"
#include "tc_common.cuh"

namespace rl {
namespace mlpf {

constexpr int WARPS = 16;              // warps that compute
constexpr int CTHREADS = 32 * WARPS;
constexpr int THREADS = CTHREADS + 32;  // and one that talks to the other blocks meanwhile
constexpr int MAX_K4 = 8;   // float4 pieces of a row a lane keeps while normalising: K <= 32 * 4 * 8 = 1024
constexpr int MAX_FS = 32;  // widest slice of the inner width a block takes: 16 rows x 32 units, a thread each
constexpr int MAX_PAIRS = 16;  // (tile of eight columns, part of K) pairs of the first product

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four 8x8 matrices of 16-bit elements from shared memory, one row address a lane: lanes 0-7
// give the rows of the first matrix, 8-15 of the second, and so on.
__device__ __forceinline__ void ldmatrix4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr)
               : "memory");
}
__device__ __forceinline__ void ldmatrix2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr) : "memory");
}

// A run of bytes from global to shared memory by the copy engine; its arrival is counted on `bar`.
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void red_add2(float* addr, float a, float b) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(a), "f"(b) : "memory");
}

// Row strides in shared memory (elements): a multiple of 8 (16-byte rows) that is an odd
// number of 16-byte pieces, so that the eight rows an ldmatrix reads fall into distinct banks.
__host__ __device__ inline int padded(int k) {
  const int k16 = (k + 15) / 16 * 16;  // the MMA steps over K in sixteens; the tail is zero
  return k16 + 8;
}

// Arrival counter and generation of the "every block has read the rows" barrier.  One per
// device and library: launches that use it must not overlap (the engine issues everything on
// one stream, and a launch reads the generation only after the kernels ahead have completed).
__device__ unsigned int rows_taken_count = 0;
__device__ unsigned int rows_taken_generation = 0;

__device__ __forceinline__ unsigned int load_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// This block has taken what it needs of memory that other blocks will overwrite.
__device__ __forceinline__ void rows_taken_arrive() {
  __threadfence();
  const unsigned int ticket = atomicAdd(&rows_taken_count, 1u);
  if (ticket == gridDim.x * gridDim.y - 1) {
    rows_taken_count = 0;  // everyone has arrived; nobody touches the counter before the next launch
    __threadfence();
    atomicAdd(&rows_taken_generation, 1u);
  }
}

// Have all blocks arrived since `generation` was read?  Waits about 50 ms at most.
__device__ __forceinline__ bool rows_taken_wait(unsigned int generation, int* status) {
  const long long t0 = clock64();
  while (load_acquire(&rows_taken_generation) == generation) {
    if (clock64() - t0 > 100000000LL) {
      atomicOr(status, RL_STATUS_WAIT_TIMEOUT);
      return false;
    }
  }
  return true;
}

// Named barriers of a block: 1 = the rows have been read (computing warps arrive, the talking
// warp waits), 2 = every block has read its rows (the talking warp arrives, the others wait),
// 3 = the computing warps among themselves.
__device__ __forceinline__ void bar_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void compute_sync() { bar_sync(3, CTHREADS); }

struct Args {
  float* x;             // [M, hidden] float32 residual stream: read (normalised) and added to
  long ldx;
  const __nv_bfloat16* a;  // the input rows when no norm is fused (gamma == nullptr), [M, hidden]
  long lda;
  const float* gamma;   // LayerNorm scale (nullptr: `a` is the input as it is)
  const float* beta;    // may be nullptr
  float eps;
  const __nv_bfloat16* w_in;   // [F, hidden]
  const float* b_in;           // [F] or nullptr
  const __nv_bfloat16* w_out;  // [slices][hidden][fs + 8]: W_out[:, slice] as it lies in shared memory (padding and missing units zero)
  const float* b_out;          // [hidden] or nullptr
  int M, hidden, F, fs, act;
  int* status;
};

// Shared memory: barriers | a_s [16][lds] | win_s [fs][lds] | wout_s [hidden][fs + 8] | part_s
// [pairs][16][8] float | u_s [16][fs + 8] | gamma, beta [hidden] float each.
template <bool NORM>
__global__ __launch_bounds__(THREADS) void mlp_rows_fused_kernel(Args p) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = p.hidden, fs = p.fs;
  const int lds = padded(K), ldo = fs + 8;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);       // [0]: norm scale and shift, [1]: weights
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 16);
  __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(smem + 32);
  __nv_bfloat16* win_s = a_s + 16 * lds;
  __nv_bfloat16* wout_s = win_s + (size_t)fs * lds;
  float* part_s = reinterpret_cast<float*>(wout_s + (size_t)K * ldo);
  __nv_bfloat16* u_s = reinterpret_cast<__nv_bfloat16*>(part_s + MAX_PAIRS * 16 * 8);
  float* gb_s = reinterpret_cast<float*>(u_s + 16 * ldo);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int f0 = blockIdx.x * fs;
  const int f_here = min(fs, p.F - f0);  // the last slice may be short: its missing units are zero
  const uint32_t bar_g = tc::smem_u32(&bars[0]), bar_w = tc::smem_u32(&bars[1]);

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  RL_PHASE(0);
  // ---- before the wait for the kernels ahead: the weight slices start travelling ----
  if (tid == 0) {
    tc::mbar_init(bar_g, 1);
    tc::mbar_init(bar_w, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (tid == 0) {
    if (NORM) tc::mbar_expect_tx(bar_g, (uint32_t)(K * 4 * (p.beta != nullptr ? 2 : 1)));
    tc::mbar_expect_tx(bar_w, (uint32_t)(f_here * K * 2 + K * ldo * 2));
    // this block's slice of W_out was laid out for it when the weights were bound: one copy
    bulk_copy(tc::smem_u32(wout_s), p.w_out + (size_t)blockIdx.x * K * ldo, (uint32_t)(K * ldo * 2), bar_w);
    if (NORM) {
      bulk_copy(tc::smem_u32(gb_s), p.gamma, (uint32_t)K * 4, bar_g);
      if (p.beta != nullptr) bulk_copy(tc::smem_u32(gb_s + K), p.beta, (uint32_t)K * 4, bar_g);
    }
  }
  if (tid < f_here)  // a row of W_in is one run of K elements
    bulk_copy(tc::smem_u32(win_s + (size_t)tid * lds), p.w_in + (size_t)(f0 + tid) * K, (uint32_t)K * 2, bar_w);
  // the biases of this block's outputs are weights too: fetched now, used at the end
  const int u_row = tid / fs, u_col = tid - u_row * fs;  // the element of the inner activations this thread finishes
  float bias_in = 0.f;
  if (p.b_in != nullptr && tid < 16 * fs && f0 + u_col < p.F) bias_in = p.b_in[f0 + u_col];
  {
    // what the copies do not fill must be zero: the tail of K up to a multiple of 16, and the
    // units of a short last slice
    const __nv_bfloat16 z = __float2bfloat16_rn(0.f);
    const int kt = lds - 8 - K;  // 0 or 8 columns between K and the next multiple of 16
    if (kt > 0) {
      for (int i = tid; i < (16 + fs) * kt; i += THREADS) {
        const int r = i / kt, c = K + (i - r * kt);
        (r < 16 ? a_s + (size_t)r * lds : win_s + (size_t)(r - 16) * lds)[c] = z;
      }
    }
    if (f_here < fs) {
      for (int i = tid; i < (fs - f_here) * (lds - 8); i += THREADS) {
        const int r = f_here + i / (lds - 8), c = i % (lds - 8);
        win_s[(size_t)r * lds + c] = z;
      }
    }
  }
  RL_PHASE(1);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  RL_PHASE(2);
  if (warp == WARPS) {
    // ---- the talking warp ----
    unsigned int generation = 0;
    if (lane == 0) generation = load_acquire(&rows_taken_generation);  // the launches ahead are over: it is stable now
    bar_sync(1, THREADS);  // the computing warps hold their rows
    if (lane == 0) {
      rows_taken_arrive();
      if (!rows_taken_wait(generation, p.status)) *abort_flag = 1;
    }
    __syncwarp();
    bar_arrive(2, THREADS);
    return;
  }

  // ---- the rows: normalised from the residual stream (a warp a row), or copied as they are ----
  bool ok = true;
  if constexpr (NORM) {
    const int n4 = K >> 2;
    const int row = warp;  // sixteen warps, sixteen rows
    __nv_bfloat16* dst = a_s + (size_t)row * lds;
    float4 r[MAX_K4];
    if (row < p.M) {
      const float4* xr = reinterpret_cast<const float4*>(p.x + (size_t)row * p.ldx);
#pragma unroll
      for (int q = 0; q < MAX_K4; ++q) {
        const int d = lane + 32 * q;
        r[q] = xr[d < n4 ? d : 0];
      }
    }
    float sum = 0.f;
    if (row < p.M) {
      const int n4r = K >> 2;
#pragma unroll
      for (int q = 0; q < MAX_K4; ++q) {
        if (lane + 32 * q >= n4r) r[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        sum += (r[q].x + r[q].y) + (r[q].z + r[q].w);
      }
      sum = warp_sum(sum);  // every lane's loads have returned: the row is in registers
    }
    bar_arrive(1, THREADS);
    ok = tc::mbar_wait(bar_g, 0, abort_flag, p.status);  // the scale and shift have arrived long ago
    if (row >= p.M || !ok) {
      for (int d = lane; d < n4; d += 32) *reinterpret_cast<uint2*>(dst + 4 * d) = make_uint2(0u, 0u);
    } else {
      const float4* g4 = reinterpret_cast<const float4*>(gb_s);
      const float4* b4 = reinterpret_cast<const float4*>(gb_s + K);
      const float mean = sum / (float)K;
      float sq = 0.f;
#pragma unroll
      for (int q = 0; q < MAX_K4; ++q) {
        if (lane + 32 * q < n4) {
          const float a = r[q].x - mean, b = r[q].y - mean, c = r[q].z - mean, d = r[q].w - mean;
          sq += (a * a + b * b) + (c * c + d * d);
        }
      }
      const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)K + p.eps);
#pragma unroll
      for (int q = 0; q < MAX_K4; ++q) {
        const int d = lane + 32 * q;
        if (d < n4) {
          const float4 gm = g4[d];
          const float4 bt = p.beta != nullptr ? b4[d] : make_float4(0.f, 0.f, 0.f, 0.f);
          const float4 v = r[q];
          const __nv_bfloat162 lo = __floats2bfloat162_rn((v.x - mean) * rstd * gm.x + bt.x, (v.y - mean) * rstd * gm.y + bt.y);
          const __nv_bfloat162 hi = __floats2bfloat162_rn((v.z - mean) * rstd * gm.z + bt.z, (v.w - mean) * rstd * gm.w + bt.w);
          *reinterpret_cast<uint2*>(dst + 4 * d) =
              make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        }
      }
    }
  } else {
    bar_arrive(1, THREADS);  // nothing of the residual stream is read here
    const int k8 = K / 8;
    for (int i = tid; i < 16 * k8; i += CTHREADS) {
      const int r = i / k8, c = i - r * k8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < p.M) v = *reinterpret_cast<const uint4*>(p.a + (size_t)r * p.lda + 8 * c);
      *reinterpret_cast<uint4*>(a_s + (size_t)r * lds + 8 * c) = v;
    }
  }
  RL_PHASE(3);
  ok = tc::mbar_wait(bar_w, 0, abort_flag, p.status) && ok;
  compute_sync();
  RL_PHASE(4);  // rows and weights are in shared memory (or a wait gave up: then every thread knows below)
  if (*abort_flag) {  // the status word says why; nothing is added to the residual stream
    tc::mbar_wait_quiet(bar_w, 0);  // copies still in flight land before the block's memory is given up
    return;
  }

  // ---- first product: [16, K] x W_in[f0 : f0 + fs, :]^T; a warp takes eight columns and a part of K ----
  const int g = lane >> 2, j = lane & 3;
  const int ntiles = fs / 8;           // fs is 16 or 32: 2 or 4 tiles
  const int ksteps = (lds - 8) / 16;
  const int kparts = WARPS / ntiles;   // 8 or 4 parts of K
  if (warp < ntiles * kparts) {
    const int nt = warp % ntiles, kp = warp / ntiles;
    const int per = (ksteps + kparts - 1) / kparts;
    const int k_lo = kp * per, k_hi = min(ksteps, k_lo + per);
    float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};  // two chains of products
    // ldmatrix row addresses: A 16x16 tile = four 8x8 matrices (rows 0-7 / 8-15, columns 0-7 / 8-15)
    const uint32_t a_addr = tc::smem_u32(a_s + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * lds + (lane >> 4) * 8);
    // B: eight rows of W_in, columns k..k+7 and k+8..k+15 (lanes 16-31 repeat valid addresses)
    const uint32_t b_addr = tc::smem_u32(win_s + (size_t)(nt * 8 + (lane & 7)) * lds + ((lane >> 3) & 1) * 8);
    int ks = k_lo;
#pragma unroll 2
    for (; ks + 1 < k_hi; ks += 2) {
      uint32_t af[4], bf[2], af2[4], bf2[2];
      ldmatrix4(af, a_addr + ks * 32);
      ldmatrix2(bf, b_addr + ks * 32);
      ldmatrix4(af2, a_addr + ks * 32 + 32);
      ldmatrix2(bf2, b_addr + ks * 32 + 32);
      mma_16816(c, af, bf[0], bf[1]);
      mma_16816(c2, af2, bf2[0], bf2[1]);
    }
    if (ks < k_hi) {
      uint32_t af[4], bf[2];
      ldmatrix4(af, a_addr + ks * 32);
      ldmatrix2(bf, b_addr + ks * 32);
      mma_16816(c, af, bf[0], bf[1]);
    }
    float* ps = part_s + (size_t)(kp * ntiles + nt) * 16 * 8;
    *reinterpret_cast<float2*>(ps + g * 8 + 2 * j) = make_float2(c[0] + c2[0], c[1] + c2[1]);
    *reinterpret_cast<float2*>(ps + (g + 8) * 8 + 2 * j) = make_float2(c[2] + c2[2], c[3] + c2[3]);
  }
  compute_sync();
  RL_PHASE(5);
  if (tid < 16 * fs) {  // bias, activation, rounding: the inner activations of this slice, [16][fs]
    const int nt = u_col >> 3, cc = u_col & 7;
    float acc = 0.f;
    for (int kp = 0; kp < kparts; ++kp) acc += part_s[((size_t)(kp * ntiles + nt) * 16 + u_row) * 8 + cc];
    const float v = f0 + u_col < p.F ? tc::act_fn(acc + bias_in, p.act) : 0.f;
    u_s[(size_t)u_row * ldo + u_col] = __float2bfloat16_rn(v);
  }
  compute_sync();
  RL_PHASE(6);

  // ---- second product: [16, fs] x W_out[:, f0 : f0 + fs]^T, added into the residual stream ----
  {
    const int out_tiles = K / 8;  // the hidden size is a multiple of 8
    const int k2 = fs / 16;       // 1 to 4 steps
    uint32_t af[MAX_FS / 16][4];
    const uint32_t a_addr = tc::smem_u32(u_s + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * ldo + (lane >> 4) * 8);
#pragma unroll
    for (int ks = 0; ks < MAX_FS / 16; ++ks)
      if (ks < k2) ldmatrix4(af[ks], a_addr + ks * 32);
    const bool first = blockIdx.x == 0 && p.b_out != nullptr;
    // the warp's tiles of eight output columns: all computed, then (once every block has read
    // its rows, which the talking warp reports) added
    constexpr int MAX_TILES = (32 * 4 * MAX_K4 / 8 + WARPS - 1) / WARPS;
    float c[MAX_TILES][4];
#pragma unroll
    for (int t = 0; t < MAX_TILES; ++t) {
      const int nt = warp + t * WARPS;
      c[t][0] = c[t][1] = c[t][2] = c[t][3] = 0.f;
      if (nt < out_tiles) {
        const uint32_t b_addr = tc::smem_u32(wout_s + (size_t)(nt * 8 + (lane & 7)) * ldo + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int ks = 0; ks < MAX_FS / 16; ++ks) {
          if (ks < k2) {
            uint32_t bf[2];
            ldmatrix2(bf, b_addr + ks * 32);
            mma_16816(c[t], af[ks], bf[0], bf[1]);
          }
        }
        if (first) {
          const int n = nt * 8 + 2 * j;
          const float b0 = p.b_out[n], b1 = p.b_out[n + 1];
          c[t][0] += b0; c[t][1] += b1; c[t][2] += b0; c[t][3] += b1;
        }
      }
    }
    RL_PHASE(7);
    bar_sync(2, THREADS);
    RL_PHASE(8);
    if (*abort_flag) return;
#pragma unroll
    for (int t = 0; t < MAX_TILES; ++t) {
      const int nt = warp + t * WARPS;
      if (nt < out_tiles) {
        const int n = nt * 8 + 2 * j;
        if (g < p.M) red_add2(p.x + (size_t)g * p.ldx + n, c[t][0], c[t][1]);
        if (g + 8 < p.M) red_add2(p.x + (size_t)(g + 8) * p.ldx + n, c[t][2], c[t][3]);
      }
    }
    RL_PHASE(9);
  }
}

static size_t smem_bytes(int hidden, int fs, bool norm) {
  const int lds = padded(hidden), ldo = fs + 8;
  size_t b = 32 + (size_t)(16 + fs) * lds * 2 + (size_t)hidden * ldo * 2 + (size_t)MAX_PAIRS * 16 * 8 * 4 + (size_t)16 * ldo * 2;
  if (norm) b += 2 * (size_t)hidden * 4;
  return b;
}

}  // namespace mlpf
}  // namespace rl

// How wide a slice of the inner width a block takes for these sizes, or 0 when the kernel does
// not take them.  Two blocks should fit an SM (their weight copies then run under the kernel
// ahead), and there should be about as many blocks as the device runs at once.
RL_EXPORT int rl_mlp_fused_slice(int M, int hidden, int F, int norm) {
  if (M < 1 || M > 16 || hidden % 8 != 0 || hidden > 32 * 4 * rl::mlpf::MAX_K4 || F % 8 != 0 || F < 16) return 0;
  static int n_sms = 0, smem_sm = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
  }
  // The widest slice first: fewer blocks add into each element of the residual stream (the
  // additions to one address queue up), and 64-byte runs of W_out use whole memory bursts.
  // All blocks must run at once (they wait for one another before they add).
  for (int fs = rl::mlpf::MAX_FS; fs >= 16; fs -= 16) {
    const size_t need = rl::mlpf::smem_bytes(hidden, fs, norm != 0);
    const int blocks = (F + fs - 1) / fs;
    const int per_sm = need + 1024 > (size_t)smem_sm ? 0 : (int)((size_t)smem_sm / (need + 1024));
    if (need <= 200 * 1024 && blocks <= n_sms * (per_sm > 2 ? 2 : per_sm)) return fs;
  }
  return 0;
}

// x [M <= 16, hidden] float32 += act(in W_in^T + b_in) W_out^T + b_out, where in = LayerNorm(x)
// (gamma != nullptr) or the bfloat16 rows `a`.  w_out is not the matrix [hidden, F] but its slices
// as the blocks keep them: [ceil(F / fs)][hidden][fs + 8] bfloat16, slice s holding W_out[:, s*fs :
// (s+1)*fs] with eight zero columns after it (and zeros for units beyond F), so that a block
// fetches its slice with one copy.  fs: as rl_mlp_fused_slice says (or any multiple of
// 16 up to 32 that fits shared memory).  status: the word a wait that gave up is recorded in.  Returns -2 for sizes the kernel does not take.
RL_EXPORT int rl_mlp_fused(float* x, long ldx, const void* a, long lda, const float* gamma, const float* beta, float eps,
                           const void* w_in, const float* b_in, const void* w_out, const float* b_out, int M,
                           int hidden, int F, int fs, int act, int* status, cudaStream_t stream) {
  using namespace rl::mlpf;
  if (M <= 0) return 0;
  const bool norm = gamma != nullptr;
  if (M > 16 || hidden % 8 != 0 || F % 8 != 0 || fs < 16 || fs > MAX_FS || fs % 16 != 0 || ldx % 4 != 0 ||
      ((uintptr_t)x % 16) != 0 || status == nullptr)
    return -2;
  if (norm && hidden > 32 * 4 * MAX_K4) return -2;
  if (!norm && (a == nullptr || lda % 8 != 0 || ((uintptr_t)a % 16) != 0)) return -2;
  if (((uintptr_t)w_in % 16) != 0 || ((uintptr_t)w_out % 16) != 0) return -2;
  if (norm && (((uintptr_t)gamma % 16) != 0 || (beta != nullptr && ((uintptr_t)beta % 16) != 0))) return -2;
  const size_t smem = smem_bytes(hidden, fs, norm);
  if (smem > 200 * 1024) return -2;
  Args p{x, ldx, (const __nv_bfloat16*)a, lda, gamma, beta, eps, (const __nv_bfloat16*)w_in, b_in,
         (const __nv_bfloat16*)w_out, b_out, M, hidden, F, fs, act, status};
  const int blocks = (F + fs - 1) / fs;
  {
    // the blocks wait for one another: all of them must be resident at once
    static int n_sms = 0, smem_sm = 0;
    if (n_sms == 0) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
      cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
    }
    const int per_sm = (int)((size_t)smem_sm / (smem + 1024));
    if (blocks > n_sms * (per_sm > 2 ? 2 : per_sm)) return -2;
  }
  static bool attr_set[2] = {false, false};
  if (!attr_set[norm]) {
    // all of an SM's memory as shared memory, as the other fused kernel of a decode layer asks:
    // where two kernels in a row want different splits the SM has to run empty in between
    if (norm) {
      rl::note_launch(cudaFuncSetAttribute(mlp_rows_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      rl::note_launch(cudaFuncSetAttribute(mlp_rows_fused_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                           cudaSharedmemCarveoutMaxShared));
    } else {
      rl::note_launch(cudaFuncSetAttribute(mlp_rows_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      rl::note_launch(cudaFuncSetAttribute(mlp_rows_fused_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                           cudaSharedmemCarveoutMaxShared));
    }
    attr_set[norm] = true;
  }
  if (norm)
    rl::launch_pdl_split(false, mlp_rows_fused_kernel<true>, dim3(blocks), dim3(THREADS), smem, stream, p);
  else
    rl::launch_pdl_split(false, mlp_rows_fused_kernel<false>, dim3(blocks), dim3(THREADS), smem, stream, p);
  RL_CHECK_LAUNCH();
  return 0;
}

RL_PHASE_READER(rl_mlp_fused_phase_times)
