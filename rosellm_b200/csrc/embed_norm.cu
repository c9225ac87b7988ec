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
                             int n_positions, int* __restrict__ status,
                             const int* __restrict__ feedback, int n_feedback) {
  pdl_begin();
  const int n = blockIdx.x;
  if (n >= n_tokens) return;
  int id = ids[n];
  // a negative id -(r+1) stands for "the token row r of the previous step's sampling wrote":
  // the step was launched before the host had read that token
  if (id < 0 && feedback != nullptr && -id - 1 < n_feedback) id = feedback[-id - 1];
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

// The same for rows of at most 2048 elements (a multiple of 4): one warp per row, the row in
// registers between the passes as PIECES (8: up to 1024 elements; 16: up to 2048) 16-byte pieces
// per lane, no block-wide barrier.  Every
// load is unconditional (a clamped address), so that all are issued before the first is used;
// a load under a condition would wait for the one before it.
template <typename T, int PIECES>
__global__ __launch_bounds__(128) void layernorm_warp_kernel(const float* __restrict__ x,
                                                             const int* __restrict__ rows,
                                                             const float* __restrict__ gamma,
                                                             const float* __restrict__ beta, T* __restrict__ out,
                                                             int n_out, int hidden, float eps) {
  pdl_begin();
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (i >= n_out) return;
  const int src = rows != nullptr ? rows[i] : i;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * hidden);
  const int n4 = hidden >> 2;
  float4 r[PIECES];
#pragma unroll
  for (int j = 0; j < PIECES; ++j) {
    const int d = lane + 32 * j;
    r[j] = xr[d < n4 ? d : 0];
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < PIECES; ++j) {
    if (lane + 32 * j >= n4) r[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    s += (r[j].x + r[j].y) + (r[j].z + r[j].w);
  }
  const float mean = warp_sum(s) / (float)hidden;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < PIECES; ++j) {
    if (lane + 32 * j < n4) {
      const float a = r[j].x - mean, b = r[j].y - mean, c = r[j].z - mean, d = r[j].w - mean;
      q += (a * a + b * b) + (c * c + d * d);
    }
  }
  const float rstd = 1.0f / sqrtf(warp_sum(q) / (float)hidden + eps);
  const float4* g4 = reinterpret_cast<const float4*>(gamma);
  const float4* b4 = reinterpret_cast<const float4*>(beta);
  T* o = out + (size_t)i * hidden;
#pragma unroll
  for (int j = 0; j < PIECES; ++j) {
    const int d = lane + 32 * j;
    const int dc = d < n4 ? d : 0;
    const float4 gm = g4[dc];
    const float4 bt = beta != nullptr ? b4[dc] : make_float4(0.f, 0.f, 0.f, 0.f);
    if (d < n4) {
      const float v0 = (r[j].x - mean) * rstd * gm.x + bt.x, v1 = (r[j].y - mean) * rstd * gm.y + bt.y;
      const float v2 = (r[j].z - mean) * rstd * gm.z + bt.z, v3 = (r[j].w - mean) * rstd * gm.w + bt.w;
      if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(o + 4 * d) = make_float4(v0, v1, v2, v3);
      } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v0, v1), hi = __floats2bfloat162_rn(v2, v3);
        *reinterpret_cast<uint2*>(o + 4 * d) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
      }
    }
  }
}

}  // namespace rl

// A copy from pinned host memory to the device, ordered on the stream (a step's description,
// changed rows of a block table): the plain runtime call, without a framework's dispatch around it.
RL_EXPORT int rl_copy_to_device(void* dst, const void* src, long bytes, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  return (int)cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, stream);
}

// Records an event (the handle a framework's event object holds) on the stream.
RL_EXPORT int rl_event_record(cudaEvent_t event, cudaStream_t stream) { return (int)cudaEventRecord(event, stream); }

RL_EXPORT int rl_embed(int dtype, const int* ids, const int* pos, const void* table,
                       const void* pos_table, float* out, int n_tokens, int hidden, int vocab,
                       int n_positions, int* status, const int* feedback, int n_feedback,
                       cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int threads = hidden >= 512 ? 256 : 128;
  if (dtype == RL_F32)
    rl::launch_pdl(rl::embed_kernel<float>, n_tokens, threads, 0, stream, ids, pos, (const float*)table,
                   (const float*)pos_table, out, n_tokens, hidden, vocab, n_positions, status, feedback, n_feedback);
  else
    rl::launch_pdl(rl::embed_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, ids, pos,
                   (const __nv_bfloat16*)table, (const __nv_bfloat16*)pos_table, out, n_tokens, hidden, vocab,
                   n_positions, status, feedback, n_feedback);
  RL_CHECK_LAUNCH();
  return 0;
}

namespace rl {

// The same for few rows (a decode step of a wide model, a norm before 17 to 64 rows' products):
// a block per row, so that a row's latency is not one warp's walk through it: every thread holds
// two 16-byte pieces (one, where the row is short), the statistics meet through shared memory, and gamma and beta (no
// kernel writes them) are asked for before the wait for the kernels ahead.  Rows of at most 2048
// elements, a multiple of 4.
template <typename T>
__global__ __launch_bounds__(256) void layernorm_block_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                                              const float* __restrict__ gamma,
                                                              const float* __restrict__ beta, T* __restrict__ out,
                                                              int n_out, int hidden, float eps) {
  __shared__ float red_s[2][8];
  const int n4 = hidden >> 2;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
  const int d0 = tid, d1 = tid + blockDim.x;
  const bool has0 = d0 < n4, has1 = d1 < n4;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4* g4 = reinterpret_cast<const float4*>(gamma);
  const float4* b4 = reinterpret_cast<const float4*>(beta);
  const float4 ga = g4[has0 ? d0 : 0], gb = g4[has1 ? d1 : 0];
  const float4 ba = beta != nullptr ? b4[has0 ? d0 : 0] : zero, bb = beta != nullptr ? b4[has1 ? d1 : 0] : zero;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int i = blockIdx.x;
  const int src = rows != nullptr ? rows[i] : i;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * hidden);
  float4 va = xr[has0 ? d0 : 0], vb = xr[has1 ? d1 : 0];
  if (!has0) va = zero;
  if (!has1) vb = zero;
  float s = ((va.x + va.y) + (va.z + va.w)) + ((vb.x + vb.y) + (vb.z + vb.w));
  s = warp_sum(s);
  if (lane == 0) red_s[0][warp] = s;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < n_warps; ++w) total += red_s[0][w];
  const float mean = total / (float)hidden;
  float q = 0.f;
  if (has0) {
    const float a = va.x - mean, b = va.y - mean, c = va.z - mean, d = va.w - mean;
    q += (a * a + b * b) + (c * c + d * d);
  }
  if (has1) {
    const float a = vb.x - mean, b = vb.y - mean, c = vb.z - mean, d = vb.w - mean;
    q += (a * a + b * b) + (c * c + d * d);
  }
  q = warp_sum(q);
  if (lane == 0) red_s[1][warp] = q;
  __syncthreads();
  float var = 0.f;
  for (int w = 0; w < n_warps; ++w) var += red_s[1][w];
  const float rstd = 1.0f / sqrtf(var / (float)hidden + eps);
  T* o = out + (size_t)i * hidden;
  auto put = [&](int d, const float4& v, const float4& gm, const float4& bt) {
    const float y0 = (v.x - mean) * rstd * gm.x + bt.x, y1 = (v.y - mean) * rstd * gm.y + bt.y;
    const float y2 = (v.z - mean) * rstd * gm.z + bt.z, y3 = (v.w - mean) * rstd * gm.w + bt.w;
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(o + 4 * d) = make_float4(y0, y1, y2, y3);
    } else {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
      *reinterpret_cast<uint2*>(o + 4 * d) =
          make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
  };
  if (has0) put(d0, va, ga, ba);
  if (has1) put(d1, vb, gb, bb);
}

}  // namespace rl

// Rows up to which a LayerNorm runs a block a row (beyond: a warp a row, four rows a block).
#define RL_LAYERNORM_BLOCK_ROWS 512

RL_EXPORT int rl_layernorm(int out_dtype, const float* x, const int* rows, const float* gamma,
                           const float* beta, void* out, int n_out, int hidden, float eps,
                           cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (hidden <= 2048 && hidden % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)out % 8) == 0 &&
      ((uintptr_t)gamma % 16) == 0 && (beta == nullptr || ((uintptr_t)beta % 16) == 0)) {
    if (n_out <= RL_LAYERNORM_BLOCK_ROWS && hidden >= 256 && (out_dtype != RL_F32 || ((uintptr_t)out % 16) == 0)) {
      // threads enough for a row's 16-byte pieces, two a thread at most
      const int n4 = hidden / 4;
      const int threads = ((n4 + 1) / 2 + 31) / 32 * 32;
      if (out_dtype == RL_F32)
        rl::launch_pdl(rl::layernorm_block_kernel<float>, n_out, threads, 0, stream, x, rows, gamma, beta, (float*)out,
                       n_out, hidden, eps);
      else
        rl::launch_pdl(rl::layernorm_block_kernel<__nv_bfloat16>, n_out, threads, 0, stream, x, rows, gamma, beta,
                       (__nv_bfloat16*)out, n_out, hidden, eps);
      RL_CHECK_LAUNCH();
      return 0;
    }
    const int blocks = (n_out + 3) / 4;
    const bool wide = hidden > 1024;
    if (out_dtype == RL_F32) {
      if (wide)
        rl::launch_pdl(rl::layernorm_warp_kernel<float, 16>, blocks, 128, 0, stream, x, rows, gamma, beta, (float*)out,
                       n_out, hidden, eps);
      else
        rl::launch_pdl(rl::layernorm_warp_kernel<float, 8>, blocks, 128, 0, stream, x, rows, gamma, beta, (float*)out,
                       n_out, hidden, eps);
    } else {
      if (wide)
        rl::launch_pdl(rl::layernorm_warp_kernel<__nv_bfloat16, 16>, blocks, 128, 0, stream, x, rows, gamma, beta,
                       (__nv_bfloat16*)out, n_out, hidden, eps);
      else
        rl::launch_pdl(rl::layernorm_warp_kernel<__nv_bfloat16, 8>, blocks, 128, 0, stream, x, rows, gamma, beta,
                       (__nv_bfloat16*)out, n_out, hidden, eps);
    }
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

// The address under which kernels of the current device reach pinned host memory `host` (0 when
// they cannot: the memory is not pinned, or not mapped into the device's address space).
RL_EXPORT unsigned long long rl_host_memory_on_device(void* host) {
  void* dev = nullptr;
  if (cudaHostGetDevicePointer(&dev, host, 0) != cudaSuccess) {
    cudaGetLastError();
    return 0ull;
  }
  return (unsigned long long)(uintptr_t)dev;
}

