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

// Few rows: one warp per output column streams that column's weights once per group of MB
// rows; lanes split K in 16-byte pieces, four pieces of the weight row are in flight per lane
// before any is used, and the partial sums meet in a shuffle tree.
template <typename TIn, typename TOut, int MB>
__global__ __launch_bounds__(128) void gemm_rows_kernel(
    const TIn* __restrict__ A, long lda, const TIn* __restrict__ W, const float* __restrict__ bias,
    TOut* __restrict__ out, long ldo, int M, int N, int K, int act, int residual) {
  constexpr int VEC = Vec16<TIn>::N;
  constexpr int U = 4;
  const int lane = threadIdx.x & 31;
  const int n = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  if (n >= N) return;
  const TIn* w = W + (size_t)n * K;
  const float b = bias != nullptr ? bias[n] : 0.f;
  for (int m0 = 0; m0 < M; m0 += MB) {
    float acc[MB];
#pragma unroll
    for (int i = 0; i < MB; ++i) acc[i] = 0.f;
    for (int k0 = lane * VEC; k0 < K; k0 += 32 * VEC * U) {
      float wv[U][VEC];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = k0 + u * 32 * VEC;
        if (k < K) {
          Vec16<TIn>::load(w + k, wv[u]);
        } else {
#pragma unroll
          for (int v = 0; v < VEC; ++v) wv[u][v] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = k0 + u * 32 * VEC;
        if (k >= K) break;
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
#pragma unroll
    for (int i = 0; i < MB; ++i) acc[i] = warp_sum(acc[i]);
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < MB; ++i) {
        if (m0 + i < M) {
          const float v = apply_act(acc[i] + b, act);
          store_out<TOut>(out, (size_t)(m0 + i) * ldo + n, v, residual);
        }
      }
    }
  }
}

template <typename TIn, typename TOut>
static int launch_gemm(const void* A, long lda, const void* W, const float* bias, void* out,
                       long ldo, int M, int N, int K, int act, int residual, int rows_limit,
                       cudaStream_t stream) {
  const TIn* a = (const TIn*)A;
  const TIn* w = (const TIn*)W;
  TOut* o = (TOut*)out;
  if (M <= rows_limit) {
    const int threads = 128;
    const int blocks = (N + (threads / 32) - 1) / (threads / 32);
    if (M == 1)
      gemm_rows_kernel<TIn, TOut, 1><<<blocks, threads, 0, stream>>>(a, lda, w, bias, o, ldo, M, N, K, act, residual);
    else if (M == 2)
      gemm_rows_kernel<TIn, TOut, 2><<<blocks, threads, 0, stream>>>(a, lda, w, bias, o, ldo, M, N, K, act, residual);
    else if (M <= 4)
      gemm_rows_kernel<TIn, TOut, 4><<<blocks, threads, 0, stream>>>(a, lda, w, bias, o, ldo, M, N, K, act, residual);
    else
      gemm_rows_kernel<TIn, TOut, 8><<<blocks, threads, 0, stream>>>(a, lda, w, bias, o, ldo, M, N, K, act, residual);
  } else {
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    gemm_tile_kernel<TIn, TOut><<<grid, 256, 0, stream>>>(a, lda, w, bias, o, ldo, M, N, K, act, residual);
  }
  return 0;
}

}  // namespace rl

// in_dtype / out_dtype: RL_F32 or RL_BF16; out may be float32 with bfloat16 inputs.
// residual != 0: out (float32) += result.  rows_limit: up to this many rows the streaming
// kernel runs, above it the tiled one.
RL_EXPORT int rl_gemm_simt(int in_dtype, int out_dtype, const void* A, long lda, const void* W,
                           const float* bias, void* out, long ldo, int M, int N, int K, int act,
                           int residual, int rows_limit, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0 || lda % 8 != 0) return -2;
  if (residual && out_dtype != RL_F32) return -3;
  if (in_dtype == RL_F32 && out_dtype == RL_F32)
    rl::launch_gemm<float, float>(A, lda, W, bias, out, ldo, M, N, K, act, residual, rows_limit, stream);
  else if (in_dtype == RL_BF16 && out_dtype == RL_BF16)
    rl::launch_gemm<__nv_bfloat16, __nv_bfloat16>(A, lda, W, bias, out, ldo, M, N, K, act, residual, rows_limit, stream);
  else if (in_dtype == RL_BF16 && out_dtype == RL_F32)
    rl::launch_gemm<__nv_bfloat16, float>(A, lda, W, bias, out, ldo, M, N, K, act, residual, rows_limit, stream);
  else
    return -4;
  RL_CHECK_LAUNCH();
  return 0;
}
