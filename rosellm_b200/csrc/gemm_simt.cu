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
#include "gemm_epilogue.cuh"

namespace rl {

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

// Few rows (decoded tokens).  A block of four warps computes 4 / KSPLIT output columns for all
// rows: KSPLIT warps share a column, each taking a contiguous part of K, and their partial
// sums meet in shared memory in a fixed order.  Lanes split a warp's part of K in 16-byte
// pieces and four pieces of the weight row are in flight per lane before any is used, so that
// a weight matrix is streamed from memory once, with enough loads outstanding to keep the
// memory system busy even when the matrix has few rows of its own.
template <typename TIn, typename TOut, int MB, int KSPLIT>
__global__ __launch_bounds__(128) void gemm_rows_kernel(
    const TIn* __restrict__ A, long lda, const TIn* __restrict__ W,
    const float* __restrict__ bias, TOut* __restrict__ out, long ldo, int M, int N, int K, int act,
    int residual, KvScatter kv) {
  constexpr int VEC = Vec16<TIn>::N;
  constexpr int U = 4;
  constexpr int COLS = 4 / KSPLIT;
  extern __shared__ __align__(16) uint8_t rows_smem[];
  float* part_s = reinterpret_cast<float*>(rows_smem);          // [4][MB]
  pdl_begin();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * COLS + warp / KSPLIT;
  const int part = warp % KSPLIT;
  const int k_part = ((K + KSPLIT - 1) / KSPLIT + VEC - 1) / VEC * VEC;
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
static void launch_rows(const TIn* a, long lda, const TIn* w, const float* bias, TOut* o,
                        long ldo, int M, int N, int K, int act, int residual, const KvScatter& kv,
                        cudaStream_t stream) {
  // enough warps to keep loads in flight on every SM: split K among warps while columns are few
  constexpr int VEC = Vec16<TIn>::N;
  int ks = 1;
  while (ks < 4 && (long)N * ks < 3000 && K / (ks * 2) >= 32 * VEC && (M <= 4 || N <= 1024)) ks *= 2;
  const size_t smem = 4 * MB * sizeof(float);
  const int cols = 4 / ks;
  const int blocks = (N + cols - 1) / cols;
#define RL_ROWS(KS)                                                                                       \
  do {                                                                                                    \
    if (smem > 48 * 1024)                                                                                 \
      cudaFuncSetAttribute(gemm_rows_kernel<TIn, TOut, MB, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)smem);                                                                    \
    launch_pdl(gemm_rows_kernel<TIn, TOut, MB, KS>, blocks, 128, smem, stream, a, lda, w, bias, o, ldo, \
               M, N, K, act, residual, kv);                                                               \
  } while (0)
  if (ks == 1) RL_ROWS(1);
  else if (ks == 2) RL_ROWS(2);
  else RL_ROWS(4);
#undef RL_ROWS
}

template <typename TIn, typename TOut>
static int launch_gemm(const void* A, long lda, const void* W, const float* bias, void* out,
                       long ldo, int M, int N, int K, int act, int residual, int rows_limit,
                       const KvScatter& kv, cudaStream_t stream) {
  const TIn* a = (const TIn*)A;
  const TIn* w = (const TIn*)W;
  TOut* o = (TOut*)out;
  if (M <= rows_limit) {
    if (M == 1) launch_rows<TIn, TOut, 1>(a, lda, w, bias, o, ldo, M, N, K, act, residual, kv, stream);
    else if (M == 2) launch_rows<TIn, TOut, 2>(a, lda, w, bias, o, ldo, M, N, K, act, residual, kv, stream);
    else if (M <= 4) launch_rows<TIn, TOut, 4>(a, lda, w, bias, o, ldo, M, N, K, act, residual, kv, stream);
    else launch_rows<TIn, TOut, 8>(a, lda, w, bias, o, ldo, M, N, K, act, residual, kv, stream);
  } else {
    if (kv.pool != nullptr) return -5;  // the cache scatter is fused only into the row kernel
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    launch_pdl(gemm_tile_kernel<TIn, TOut>, grid, 256, 0, stream, a, lda, w, bias, o, ldo, M, N, K, act, residual);
  }
  return 0;
}

}  // namespace rl

// in_dtype / out_dtype: RL_F32 or RL_BF16; out may be float32 with bfloat16 inputs.
// residual != 0: out (float32) += result.  rows_limit: up to this many rows the streaming
// kernel runs, above it the tiled one.  kv_pool != nullptr (streaming kernel): output columns
// from kv_q_width on are scattered into cache pages as keys and values.
RL_EXPORT int rl_gemm_simt(int in_dtype, int out_dtype, const void* A, long lda, const void* W,
                           const float* bias, void* out, long ldo, int M, int N, int K, int act,
                           int residual, int rows_limit, void* kv_pool,
                           const int* kv_block_table, int kv_bt_stride, const int* kv_positions,
                           const int* kv_req_of_token, const int* kv_slots, int kv_q_width, int kv_width,
                           int kv_head_dim, int kv_page_size, int kv_heads, int kv_max_pos, int* status,
                           cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0 || lda % 8 != 0) return -2;
  if (residual && out_dtype != RL_F32) return -3;
  rl::KvScatter kv{kv_pool, kv_block_table, kv_bt_stride, kv_positions, kv_req_of_token, kv_slots,
                   kv_q_width, kv_width, kv_head_dim, kv_page_size, kv_heads, kv_max_pos, status};
  int rc;
  if (in_dtype == RL_F32 && out_dtype == RL_F32)
    rc = rl::launch_gemm<float, float>(A, lda, W, bias, out, ldo, M, N, K, act, residual, rows_limit, kv, stream);
  else if (in_dtype == RL_BF16 && out_dtype == RL_BF16)
    rc = rl::launch_gemm<__nv_bfloat16, __nv_bfloat16>(A, lda, W, bias, out, ldo, M, N, K, act, residual, rows_limit, kv, stream);
  else if (in_dtype == RL_BF16 && out_dtype == RL_F32)
    rc = rl::launch_gemm<__nv_bfloat16, float>(A, lda, W, bias, out, ldo, M, N, K, act, residual, rows_limit, kv, stream);
  else
    return -4;
  if (rc != 0) return rc;
  RL_CHECK_LAUNCH();
  return 0;
}
