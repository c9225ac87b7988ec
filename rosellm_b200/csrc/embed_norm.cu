// Token embedding (+ learned position table) and LayerNorm.
//
// embed: x[n,:] = table[id_n,:] + pos_table[pos_n,:]      (rosellm/rosetrainer/model.py:543-562)
// layernorm: y = (x - mean) * rsqrt(var + eps) * gamma + beta, biased variance over the last
// dimension, statistics in float32 (rosellm/rosetrainer/fused_layernorm.py:99-120; the variance
// here is the mean of squared deviations, computed in a second pass over the row held in shared
// memory, rather than E[x^2] - mean^2).
#include "common.cuh"

namespace rl {

template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ pos,
                             const T* __restrict__ table, const T* __restrict__ pos_table,
                             float* __restrict__ out, int n_tokens, int hidden, int vocab,
                             int n_positions, int* __restrict__ status) {
  pdl_begin();
  const int n = blockIdx.x;
  if (n >= n_tokens) return;
  const int id = ids[n];
  float* o = out + (size_t)n * hidden;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, RL_STATUS_BAD_TOKEN);
    for (int d = threadIdx.x; d < hidden; d += blockDim.x) o[d] = 0.f;
    return;
  }
  const T* e = table + (size_t)id * hidden;
  const T* p = nullptr;
  if (pos_table != nullptr) {
    const int ps = pos[n];
    if (ps < 0 || ps >= n_positions) {
      if (threadIdx.x == 0) atomicOr(status, RL_STATUS_BAD_POSITION);
      for (int d = threadIdx.x; d < hidden; d += blockDim.x) o[d] = 0.f;
      return;
    }
    p = pos_table + (size_t)ps * hidden;
  }
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    float v = to_f32(e[d]);
    if (p != nullptr) v += to_f32(p[d]);
    o[d] = v;
  }
}

// One block per output row.  rows == nullptr: row i of x; else row rows[i] of x.
template <typename T>
__global__ void layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 T* __restrict__ out, int n_out, int hidden, float eps) {
  extern __shared__ float smem[];
  float* row = smem;            // hidden floats
  float* scratch = smem + hidden;  // 33 floats
  pdl_begin();
  const int i = blockIdx.x;
  if (i >= n_out) return;
  const int src = rows != nullptr ? rows[i] : i;
  const float* xr = x + (size_t)src * hidden;
  float s = 0.f;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    const float v = xr[d];
    row[d] = v;
    s += v;
  }
  const float mean = block_sum(s, scratch) / (float)hidden;
  float q = 0.f;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    const float c = row[d] - mean;
    q += c * c;
  }
  const float var = block_sum(q, scratch) / (float)hidden;
  const float rstd = 1.0f / sqrtf(var + eps);
  T* o = out + (size_t)i * hidden;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    float v = (row[d] - mean) * rstd * gamma[d];
    if (beta != nullptr) v += beta[d];
    o[d] = from_f32<T>(v);
  }
}

// The same for rows of at most 1024 elements: one warp per row, the row in registers between
// the passes, no block-wide barrier.  Rows of a decode step are few and short, and what this
// kernel costs is the latency of its dependent steps, which this form has the fewest of.
template <typename T>
__global__ __launch_bounds__(128) void layernorm_warp_kernel(const float* __restrict__ x,
                                                             const int* __restrict__ rows,
                                                             const float* __restrict__ gamma,
                                                             const float* __restrict__ beta, T* __restrict__ out,
                                                             int n_out, int hidden, float eps) {
  constexpr int PER_LANE = 32;
  pdl_begin();
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (i >= n_out) return;
  const int src = rows != nullptr ? rows[i] : i;
  const float* xr = x + (size_t)src * hidden;
  // every load is unconditional (a clamped address) so that all are issued before the first is
  // used; a load under a condition would wait for the one before it
  float r[PER_LANE];
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int d = lane + 32 * j;
    r[j] = xr[d < hidden ? d : 0];
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    if (lane + 32 * j >= hidden) r[j] = 0.f;
    s += r[j];
  }
  const float mean = warp_sum(s) / (float)hidden;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const float c = lane + 32 * j < hidden ? r[j] - mean : 0.f;
    q += c * c;
  }
  const float rstd = 1.0f / sqrtf(warp_sum(q) / (float)hidden + eps);
  T* o = out + (size_t)i * hidden;
  float gm[PER_LANE], bt[PER_LANE];
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int d = lane + 32 * j;
    gm[j] = gamma[d < hidden ? d : 0];
    bt[j] = beta != nullptr ? beta[d < hidden ? d : 0] : 0.f;
  }
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int d = lane + 32 * j;
    if (d < hidden) o[d] = from_f32<T>((r[j] - mean) * rstd * gm[j] + bt[j]);
  }
}

}  // namespace rl

RL_EXPORT int rl_embed(int dtype, const int* ids, const int* pos, const void* table,
                       const void* pos_table, float* out, int n_tokens, int hidden, int vocab,
                       int n_positions, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int threads = hidden >= 512 ? 256 : 128;
  if (dtype == RL_F32)
    rl::launch_pdl(rl::embed_kernel<float>, n_tokens, threads, 0, stream, ids, pos, (const float*)table,
                   (const float*)pos_table, out, n_tokens, hidden, vocab, n_positions, status);
  else
    rl::launch_pdl(rl::embed_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, ids, pos,
                   (const __nv_bfloat16*)table, (const __nv_bfloat16*)pos_table, out, n_tokens, hidden, vocab,
                   n_positions, status);
  RL_CHECK_LAUNCH();
  return 0;
}

RL_EXPORT int rl_layernorm(int out_dtype, const float* x, const int* rows, const float* gamma,
                           const float* beta, void* out, int n_out, int hidden, float eps,
                           cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (hidden <= 1024) {
    const int blocks = (n_out + 3) / 4;
    if (out_dtype == RL_F32)
      rl::launch_pdl(rl::layernorm_warp_kernel<float>, blocks, 128, 0, stream, x, rows, gamma, beta, (float*)out,
                     n_out, hidden, eps);
    else
      rl::launch_pdl(rl::layernorm_warp_kernel<__nv_bfloat16>, blocks, 128, 0, stream, x, rows, gamma, beta,
                     (__nv_bfloat16*)out, n_out, hidden, eps);
    RL_CHECK_LAUNCH();
    return 0;
  }
  const size_t smem = (size_t)(hidden + 33) * sizeof(float);
  if (smem > 200 * 1024) return -2;  // a row must fit in shared memory
  const int threads = hidden >= 1024 ? 256 : 128;
  if (out_dtype == RL_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(rl::layernorm_kernel<float>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rl::launch_pdl(rl::layernorm_kernel<float>, n_out, threads, smem, stream, x, rows, gamma, beta,
                   (float*)out, n_out, hidden, eps);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(rl::layernorm_kernel<__nv_bfloat16>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rl::launch_pdl(rl::layernorm_kernel<__nv_bfloat16>, n_out, threads, smem, stream, x, rows, gamma, beta,
                   (__nv_bfloat16*)out, n_out, hidden, eps);
  }
  RL_CHECK_LAUNCH();
  return 0;
}
