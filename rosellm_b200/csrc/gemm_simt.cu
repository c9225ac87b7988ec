// Matrix products on the CUDA cores: out[M,N] = A[M,K] * W[N,K]^T, with the epilogues the
// model needs fused in: + bias[N]; GELU; and accumulation into a float32 residual stream.
//
// This is the whole matrix path of the 32-bit mode (IEEE float32 FMA, no tensor-core mode of
// reduced precision), and the small-batch path of the bfloat16 mode, where a product streams
// the weights once and is bound by memory, not arithmetic.  The formulas fused here:
//   y = a W + b                           rosellm/rosetrainer/model.py:95, 220, 334-337
//   gelu_tanh(u) = 0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3)))   model.py:274-277,
//                                                                    fused_mlp.py:79-89
//   gelu_erf(u)  = 0.5 u (1 + erf(u / sqrt 2))                       model.py:345-346 (F.gelu)
//   x = x + y (residual)                  model.py:412-413, 424-428; fused_mlp.py:91-113
#include "common.cuh"
#include "gemm_vec.cuh"

#define RL_ACT_NONE 0
#define RL_ACT_GELU_TANH 1
#define RL_ACT_GELU_ERF 2

namespace rl {

__device__ __forceinline__ float apply_act(float u, int act) {
  if (act == RL_ACT_GELU_TANH) {
    const float c = 0.7978845608028654f;  // sqrt(2/pi)
    return 0.5f * u * (1.0f + tanhf(c * (u + 0.044715f * u * u * u)));
  }
  if (act == RL_ACT_GELU_ERF) return 0.5f * u * (1.0f + erff(u * 0.7071067811865476f));
  return u;
}

template <typename TOut>
__device__ __forceinline__ void store_out(TOut* out, size_t idx, float v, int residual) {
  out[idx] = from_f32<TOut>(v);
}
template <>
__device__ __forceinline__ void store_out<float>(float* out, size_t idx, float v, int residual) {
  out[idx] = residual ? out[idx] + v : v;
}

// 64x64 output tile per block of 256 threads, 4x4 outputs per thread, K in steps of 16.
// Each output's sum runs over k in ascending order whatever M is, so a row's result does
// not depend on which other rows share the launch.
template <typename TIn, typename TOut>
__global__ __launch_bounds__(256) void gemm_tile_kernel(
    const TIn* __restrict__ A, long lda, const TIn* __restrict__ W, const float* __restrict__ bias,
    TOut* __restrict__ out, long ldo, int M, int N, int K, int act, int residual) {
  constexpr int BM = 64, BN = 64, BK = 16;
  pdl_begin();
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  float ra[4], rw[4];
  auto fetch = [&](int k0) {
    const int k = k0 + lk;
    const int m = m0 + lrow, n = n0 + lrow;
    if (m < M && k < K) load4(A + (size_t)m * lda + k, ra);
    else { ra[0] = ra[1] = ra[2] = ra[3] = 0.f; }
    if (n < N && k < K) load4(W + (size_t)n * K + k, rw);
    else { rw[0] = rw[1] = rw[2] = rw[3] = 0.f; }
  };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[lk + i][lrow] = ra[i];
      Ws[lk + i][lrow] = rw[i];
    }
    __syncthreads();
    if (k0 + BK < K) fetch(k0 + BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w};
      const float b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias != nullptr) v += bias[n];
      v = apply_act(v, act);
      store_out<TOut>(out, (size_t)m * ldo + n, v, residual);
    }
  }
}

// What the row kernel may do besides the product ------------------------------------------------

// LayerNorm of the float32 residual rows as the product's input (x == nullptr: off):
// a = (x - mean) * rsqrt(var + eps) * gamma + beta, statistics in float32 in two passes
// (rosellm/rosetrainer/fused_layernorm.py:99-120), rounded to the input type as the separate
// kernel would have stored it.
struct NormArgs {
  const float* x;
  long ldx;
  const float* gamma;
  const float* beta;
  float eps;
};

// Output columns from q_width on are keys, then values, of kv heads: instead of the output
// buffer they go to the page of the row's position (pool == nullptr: off).  The reference
// appends keys and values in a kernel of its own (rosellm/roseinfer/kv_append_triton.py:28-165)
// or inside its decode attention (rosellm/rosetrainer/paged_attention.py:179-204).
struct KvScatter {
  void* pool;
  const int* block_table;
  int bt_stride;
  const int* positions;
  const int* req_of_token;
  const int* slots;
  int q_width, kv_width, head_dim, page_size, n_kv_heads, max_pos;
  int* status;
};

template <typename T>
__device__ __forceinline__ bool scatter_kv(const KvScatter& kv, int m, int n, float v) {
  if (kv.pool == nullptr || n < kv.q_width) return false;
  const int c = n - kv.q_width;
  const int which = c / kv.kv_width;
  const int r = c - which * kv.kv_width;
  const int head = r / kv.head_dim, d = r - head * kv.head_dim;
  const int slot = kv.slots[kv.req_of_token[m]];
  if (slot < 0) return true;  // padding row of a fixed-size batch
  const int pos = kv.positions[m];
  if (pos < 0 || pos >= kv.max_pos) {
    atomicOr(kv.status, RL_STATUS_BAD_POSITION);
    return true;
  }
  const int page = kv.block_table[(size_t)slot * kv.bt_stride + pos / kv.page_size];
  if (page < 0) {
    atomicOr(kv.status, RL_STATUS_BAD_PAGE);
    return true;
  }
  T* dst = (T*)kv.pool +
           ((((size_t)page * 2 + which) * kv.n_kv_heads + head) * kv.page_size + pos % kv.page_size) * kv.head_dim + d;
  *dst = from_f32<T>(v);
  return true;
}

// Few rows (decoded tokens).  A block of four warps computes 4 / KSPLIT output columns for all
// rows: KSPLIT warps share a column, each taking a contiguous part of K, and their partial
// sums meet in shared memory in a fixed order.  Lanes split a warp's part of K in 16-byte
// pieces and four pieces of the weight row are in flight per lane before any is used, so that
// a weight matrix is streamed from memory once, with enough loads outstanding to keep the
// memory system busy even when the matrix has few rows of its own.
template <typename TIn, typename TOut, int MB, int KSPLIT>
__global__ __launch_bounds__(128) void gemm_rows_kernel(
    const TIn* __restrict__ A, long lda, NormArgs norm, const TIn* __restrict__ W,
    const float* __restrict__ bias, TOut* __restrict__ out, long ldo, int M, int N, int K, int act,
    int residual, KvScatter kv) {
  constexpr int VEC = Vec16<TIn>::N;
  constexpr int U = 4;
  constexpr int COLS = 4 / KSPLIT;
  extern __shared__ __align__(16) uint8_t rows_smem[];
  float* part_s = reinterpret_cast<float*>(rows_smem);          // [4][MB]
  TIn* a_s = reinterpret_cast<TIn*>(rows_smem + 4 * MB * sizeof(float));  // [M][K] when normalising
  pdl_begin();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (norm.x != nullptr) {
    constexpr int RPL = 32;  // row elements a lane keeps in registers between the passes
    const bool cached = K <= 32 * RPL;
    for (int row = warp; row < M; row += 4) {
      const float* xr = norm.x + (size_t)row * norm.ldx;
      float r[RPL];
      float sum = 0.f;
      if (cached) {
#pragma unroll
        for (int j = 0; j < RPL; ++j) {
          const int idx = lane + 32 * j;
          r[j] = idx < K ? xr[idx] : 0.f;
          sum += r[j];
        }
      } else {
        for (int idx = lane; idx < K; idx += 32) sum += xr[idx];
      }
      const float mean = warp_sum(sum) / (float)K;
      float sq = 0.f;
      if (cached) {
#pragma unroll
        for (int j = 0; j < RPL; ++j) {
          const float d = lane + 32 * j < K ? r[j] - mean : 0.f;
          sq += d * d;
        }
      } else {
        for (int idx = lane; idx < K; idx += 32) {
          const float d = xr[idx] - mean;
          sq += d * d;
        }
      }
      const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)K + norm.eps);
      if (cached) {
#pragma unroll
        for (int j = 0; j < RPL; ++j) {
          const int idx = lane + 32 * j;
          if (idx < K) {
            float v = (r[j] - mean) * rstd * norm.gamma[idx];
            if (norm.beta != nullptr) v += norm.beta[idx];
            a_s[(size_t)row * K + idx] = from_f32<TIn>(v);
          }
        }
      } else {
        for (int idx = lane; idx < K; idx += 32) {
          float v = (xr[idx] - mean) * rstd * norm.gamma[idx];
          if (norm.beta != nullptr) v += norm.beta[idx];
          a_s[(size_t)row * K + idx] = from_f32<TIn>(v);
        }
      }
    }
    __syncthreads();
    A = a_s;
    lda = K;
  }
  const int n = blockIdx.x * COLS + warp / KSPLIT;
  const int part = warp % KSPLIT;
  const int k_part = ((K + KSPLIT - 1) / KSPLIT + 32 * VEC - 1) / (32 * VEC) * (32 * VEC);
  const int k_begin = part * k_part;
  const int k_end = min(K, k_begin + k_part);
  const bool active = n < N;
  const TIn* w = W + (size_t)(active ? n : 0) * K;
  const float b = (bias != nullptr && active) ? bias[n] : 0.f;
  for (int m0 = 0; m0 < M; m0 += MB) {
    float acc[MB];
#pragma unroll
    for (int i = 0; i < MB; ++i) acc[i] = 0.f;
    if (active) {
      for (int k0 = k_begin + lane * VEC; k0 < k_end; k0 += 32 * VEC * U) {
        float wv[U][VEC];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int k = k0 + u * 32 * VEC;
          if (k < k_end) {
            Vec16<TIn>::load(w + k, wv[u]);
          } else {
#pragma unroll
            for (int v = 0; v < VEC; ++v) wv[u][v] = 0.f;
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int k = k0 + u * 32 * VEC;
          if (k >= k_end) break;
#pragma unroll
          for (int i = 0; i < MB; ++i) {
            if (m0 + i < M) {
              float av[VEC];
              Vec16<TIn>::load(A + (size_t)(m0 + i) * lda + k, av);
#pragma unroll
              for (int v = 0; v < VEC; ++v) acc[i] = fmaf(av[v], wv[u][v], acc[i]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < MB; ++i) acc[i] = warp_sum(acc[i]);
    if (KSPLIT > 1) {
      __syncthreads();  // part_s may still be read for the previous group of rows
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < MB; ++i) part_s[warp * MB + i] = acc[i];
      }
      __syncthreads();
      if (lane == 0 && part == 0) {
#pragma unroll
        for (int i = 0; i < MB; ++i) {
          float t = 0.f;
#pragma unroll
          for (int q = 0; q < KSPLIT; ++q) t += part_s[(warp + q) * MB + i];
          acc[i] = t;
        }
      }
    }
    if (lane == 0 && part == 0 && active) {
#pragma unroll
      for (int i = 0; i < MB; ++i) {
        if (m0 + i < M) {
          const float v = apply_act(acc[i] + b, act);
          if (!scatter_kv<TIn>(kv, m0 + i, n, v)) store_out<TOut>(out, (size_t)(m0 + i) * ldo + n, v, residual);
        }
      }
    }
  }
}

template <typename TIn, typename TOut, int MB>
static void launch_rows(const TIn* a, long lda, const NormArgs& norm, const TIn* w, const float* bias, TOut* o,
                        long ldo, int M, int N, int K, int act, int residual, const KvScatter& kv,
                        cudaStream_t stream) {
  // enough warps to keep loads in flight on every SM: split K among warps while columns are few
  constexpr int VEC = Vec16<TIn>::N;
  int ks = 1;
  while (ks < 4 && (long)N * ks < 3000 && K / (ks * 2) >= 32 * VEC) ks *= 2;
  const size_t smem = 4 * MB * sizeof(float) + (norm.x != nullptr ? (size_t)M * K * sizeof(TIn) : 0);
  const int cols = 4 / ks;
  const int blocks = (N + cols - 1) / cols;
#define RL_ROWS(KS)                                                                                       \
  do {                                                                                                    \
    if (smem > 48 * 1024)                                                                                 \
      cudaFuncSetAttribute(gemm_rows_kernel<TIn, TOut, MB, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)smem);                                                                    \
    launch_pdl(gemm_rows_kernel<TIn, TOut, MB, KS>, blocks, 128, smem, stream, a, lda, norm, w, bias, o, ldo, \
               M, N, K, act, residual, kv);                                                               \
  } while (0)
  if (ks == 1) RL_ROWS(1);
  else if (ks == 2) RL_ROWS(2);
  else RL_ROWS(4);
#undef RL_ROWS
}

template <typename TIn, typename TOut>
static int launch_gemm(const void* A, long lda, const NormArgs& norm, const void* W, const float* bias, void* out,
                       long ldo, int M, int N, int K, int act, int residual, int rows_limit,
                       const KvScatter& kv, cudaStream_t stream) {
  const TIn* a = (const TIn*)A;
  const TIn* w = (const TIn*)W;
  TOut* o = (TOut*)out;
  if (M <= rows_limit) {
    if (M == 1) launch_rows<TIn, TOut, 1>(a, lda, norm, w, bias, o, ldo, M, N, K, act, residual, kv, stream);
    else if (M == 2) launch_rows<TIn, TOut, 2>(a, lda, norm, w, bias, o, ldo, M, N, K, act, residual, kv, stream);
    else if (M <= 4) launch_rows<TIn, TOut, 4>(a, lda, norm, w, bias, o, ldo, M, N, K, act, residual, kv, stream);
    else launch_rows<TIn, TOut, 8>(a, lda, norm, w, bias, o, ldo, M, N, K, act, residual, kv, stream);
  } else {
    if (norm.x != nullptr || kv.pool != nullptr) return -5;  // fused only in the row kernel
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    launch_pdl(gemm_tile_kernel<TIn, TOut>, grid, 256, 0, stream, a, lda, w, bias, o, ldo, M, N, K, act, residual);
  }
  return 0;
}

}  // namespace rl

// in_dtype / out_dtype: RL_F32 or RL_BF16; out may be float32 with bfloat16 inputs.
// residual != 0: out (float32) += result.  rows_limit: up to this many rows the streaming
// kernel runs, above it the tiled one.  norm_x != nullptr (streaming kernel, at most 16 rows):
// the input is LayerNorm(norm_x) and A is ignored.  kv_pool != nullptr (streaming kernel):
// output columns from kv_q_width on are scattered into cache pages as keys and values.
RL_EXPORT int rl_gemm_simt(int in_dtype, int out_dtype, const void* A, long lda, const void* W,
                           const float* bias, void* out, long ldo, int M, int N, int K, int act,
                           int residual, int rows_limit, const float* norm_x, long norm_ldx,
                           const float* norm_gamma, const float* norm_beta, float norm_eps, void* kv_pool,
                           const int* kv_block_table, int kv_bt_stride, const int* kv_positions,
                           const int* kv_req_of_token, const int* kv_slots, int kv_q_width, int kv_width,
                           int kv_head_dim, int kv_page_size, int kv_heads, int kv_max_pos, int* status,
                           cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0 || (norm_x == nullptr && lda % 8 != 0)) return -2;
  if (residual && out_dtype != RL_F32) return -3;
  if (norm_x != nullptr && (M > 16 || M > rows_limit)) return -5;
  rl::NormArgs norm{norm_x, norm_ldx, norm_gamma, norm_beta, norm_eps};
  rl::KvScatter kv{kv_pool, kv_block_table, kv_bt_stride, kv_positions, kv_req_of_token, kv_slots,
                   kv_q_width, kv_width, kv_head_dim, kv_page_size, kv_heads, kv_max_pos, status};
  int rc;
  if (in_dtype == RL_F32 && out_dtype == RL_F32)
    rc = rl::launch_gemm<float, float>(A, lda, norm, W, bias, out, ldo, M, N, K, act, residual, rows_limit, kv, stream);
  else if (in_dtype == RL_BF16 && out_dtype == RL_BF16)
    rc = rl::launch_gemm<__nv_bfloat16, __nv_bfloat16>(A, lda, norm, W, bias, out, ldo, M, N, K, act, residual, rows_limit, kv, stream);
  else if (in_dtype == RL_BF16 && out_dtype == RL_F32)
    rc = rl::launch_gemm<__nv_bfloat16, float>(A, lda, norm, W, bias, out, ldo, M, N, K, act, residual, rows_limit, kv, stream);
  else
    return -4;
  if (rc != 0) return rc;
  RL_CHECK_LAUNCH();
  return 0;
}
