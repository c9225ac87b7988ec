// bfloat16 products with at most 64 rows (decoded tokens): out[M,N] = A[M,K] * W[N,K]^T with the
// same epilogues as the other matrix kernels (rosellm/rosetrainer/model.py:95, 220, 334-337).
//
// Such a product reads every weight once and does almost no arithmetic per byte, so the kernel
// is built around the weight stream: a warp owns eight output columns and a contiguous part of
// K; each lane fetches 16 bytes of one weight row per 32-wide step of K, four steps in flight
// before the first is used, and feeds them to mma.sync m16n8k16 (bfloat16 in, float32
// accumulators) against the matching 16 bytes of two rows of A per 16-row tile (one, two or four
// tiles for up to 16, 32 or 64 rows; rows beyond M are zero), so the weights are read once
// whatever M is.  Along K
// the elements are taken in a permuted order (a lane's eight consecutive elements serve two
// MMA steps), which a dot product does not mind as long as A and W are permuted alike.
// Warps that share columns (KSPLIT parts of K) add their accumulators in shared memory in a
// fixed order.  tcgen05 is the tool for many rows (gemm_tc.cu); here its 128-row tiles and
// shared-memory staging would only add latency.
#include "gemm_epilogue.cuh"
#include "sampling_key.cuh"

namespace rl {

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// LayerNorm of float32 rows as the product's input (x == nullptr: off; K <= 1024, M <= 16):
// a = (x - mean) * rsqrt(var + eps) * gamma + beta with two-pass float32 statistics
// (rosellm/rosetrainer/fused_layernorm.py:99-120), rounded to bfloat16 as the separate kernel
// stores it.  Every block normalises the few rows itself, into shared memory, after it has
// issued its first weight loads: that costs less than a kernel of its own between two products.
struct NormArgs {
  const float* x;
  long ldx;
  const float* gamma;
  const float* beta;
  float eps;
};

// LayerNorm of the float32 rows `norm.x` [M, K] into shared memory as bfloat16 (row stride
// a_stride elements), a warp a row at a time; g4 / b4: gamma and beta in shared memory.
// Two-pass float32 statistics (rosellm/rosetrainer/fused_layernorm.py:99-120), rounded to
// bfloat16 as the separate kernel stores it.  K <= 1024.
__device__ __forceinline__ void normalise_rows_to_shared(const NormArgs& norm, int M, int K, __nv_bfloat16* a_s,
                                                         int a_stride, const float4* g4, const float4* b4, int warp,
                                                         int n_warps, int lane) {
  const int n4 = K >> 2;
  for (int row = warp; row < M; row += n_warps) {
    const float4* xr = reinterpret_cast<const float4*>(norm.x + (size_t)row * norm.ldx);
    float4 r[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int d = lane + 32 * q;
      r[q] = xr[d < n4 ? d : 0];
    }
    float sum = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (lane + 32 * q >= n4) r[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      sum += (r[q].x + r[q].y) + (r[q].z + r[q].w);
    }
    const float mean = warp_sum(sum) / (float)K;
    float sq = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (lane + 32 * q < n4) {
        const float a = r[q].x - mean, b = r[q].y - mean, cc = r[q].z - mean, dd = r[q].w - mean;
        sq += (a * a + b * b) + (cc * cc + dd * dd);
      }
    }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)K + norm.eps);
#pragma unroll
    for (int q0 = 0; q0 < 8; q0 += 4) {  // scale and shift, four pieces at a time: loads, then uses
      float4 gm[4], bt[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int d = lane + 32 * (q0 + q);
        const int dc = d < n4 ? d : 0;
        gm[q] = g4[dc];
        bt[q] = norm.beta != nullptr ? b4[dc] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int d = lane + 32 * (q0 + q);
        const float4 v = r[q0 + q];
        if (d < n4) {
          const __nv_bfloat162 lo = __floats2bfloat162_rn((v.x - mean) * rstd * gm[q].x + bt[q].x,
                                                          (v.y - mean) * rstd * gm[q].y + bt[q].y);
          const __nv_bfloat162 hi = __floats2bfloat162_rn((v.z - mean) * rstd * gm[q].z + bt[q].z,
                                                          (v.w - mean) * rstd * gm[q].w + bt[q].w);
          *reinterpret_cast<uint2*>(a_s + (size_t)row * a_stride + 4 * d) =
              make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        }
      }
    }
  }
}

static int rows_sm_count() {
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    if (n_sms <= 0) n_sms = 1;
  }
  return n_sms;
}

}  // namespace rl

#include "gemm_rows_bulk.cuh"

namespace rl {

// MT: 16-row tiles (M <= 16 * MT).  KSPLIT warps share eight columns, each on a part of K;
// a block holds GROUPS such column groups, so that small K splits still make blocks of
// several warps (an SM takes at most 32 blocks).
template <typename TOut, int MT, int KSPLIT, int GROUPS, bool NORM>
__global__ __launch_bounds__(32 * KSPLIT * GROUPS) void gemm_rows_mma_kernel(
    const __nv_bfloat16* __restrict__ A, long lda, NormArgs norm, const __nv_bfloat16* __restrict__ W,
    const float* __restrict__ bias, TOut* __restrict__ out, long ldo, int M, int N, int K, int act, int residual,
    KvScatter kv, SampleArgs sample) {
  constexpr int U = MT <= 2 ? 4 : 2;  // K steps in flight: fewer when the rows need more registers
  __shared__ float part_s[GROUPS][KSPLIT > 1 ? KSPLIT : 1][MT][32][4];
  extern __shared__ __align__(16) uint8_t norm_smem[];  // [M][K] bfloat16, then gamma and beta [K] float32, when normalising
  if constexpr (NORM) {
    // gamma and beta are weights: no kernel writes them, so their copy into shared memory
    // starts before the wait for the kernels ahead and costs no round trip after it
    float* gb_s = reinterpret_cast<float*>(norm_smem + (size_t)M * K * sizeof(__nv_bfloat16));
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(gb_s);
    for (int i = threadIdx.x; i < K / 4; i += blockDim.x) {
      asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst + 16 * i), "l"(norm.gamma + 4 * i) : "memory");
      if (norm.beta != nullptr)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst + 4 * K + 16 * i), "l"(norm.beta + 4 * i)
                     : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  // The block's rows of W are weights too: they are asked into L2 before the wait for the kernels
  // ahead (no register waits for them, unlike a load), so that the loads below find them there.
  {
    const int n_first = blockIdx.x * GROUPS * 8;
    const int rows_here = min(GROUPS * 8, N - n_first);
    if (threadIdx.x == 0 && rows_here > 0) {
      const size_t bytes = (size_t)rows_here * K * sizeof(__nv_bfloat16);  // K is a multiple of 8: of 16 bytes
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(W + (size_t)n_first * K), "r"((uint32_t)bytes) : "memory");
    }
  }
  pdl_begin();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = warp / KSPLIT, part = warp % KSPLIT;
  const int g = lane >> 2, j = lane & 3;
  const int n0 = (blockIdx.x * GROUPS + group) * 8;
  const int chunks = (K + 31) / 32;
  // gridDim.y blocks share a group's K between them (only `out += ...` products, whose parts meet
  // by additions in memory): the warps of block y take parts y * KSPLIT ... of gridDim.y * KSPLIT
  const int n_parts = KSPLIT * (int)gridDim.y;
  const int per_part = (chunks + n_parts - 1) / n_parts;
  const int k_begin = min(K, ((int)blockIdx.y * KSPLIT + part) * per_part * 32);
  const int k_end = min(K, k_begin + per_part * 32);
  const bool col_ok = n0 + g < N;
  const __nv_bfloat16* wrow = W + (size_t)(col_ok ? n0 + g : 0) * K;
  const __nv_bfloat16* arow[MT][2];
  bool row_ok[MT][2];
#pragma unroll
  for (int t = 0; t < MT; ++t) {
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      const int m = t * 16 + hlf * 8 + g;
      row_ok[t][hlf] = m < M;
      arow[t][hlf] = A + (size_t)(row_ok[t][hlf] ? m : 0) * lda;
    }
  }
  float c[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) c[t][0] = c[t][1] = c[t][2] = c[t][3] = 0.f;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  uint4 w_first[NORM ? U : 1];  // the first round of weight loads, in flight while the rows are normalised
  if constexpr (NORM) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = k_begin + 32 * u + 8 * j;
      // a part that lies wholly beyond K (K not a multiple of the parts) reads the row's start
      w_first[u] = *reinterpret_cast<const uint4*>(wrow + (k < k_end ? k : (k_begin < k_end ? k_begin : 0)));
    }
    __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(norm_smem);
    const int n_warps = KSPLIT * GROUPS;
    const float* gb_s = reinterpret_cast<const float*>(norm_smem + (size_t)M * K * sizeof(__nv_bfloat16));
    const float4* g4 = reinterpret_cast<const float4*>(gb_s);
    const float4* b4 = reinterpret_cast<const float4*>(gb_s + K);
    // gamma and beta have long arrived: every thread waits for its own copies, then all meet
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    normalise_rows_to_shared(norm, M, K, a_s, K, g4, b4, warp, n_warps, lane);
    __syncthreads();
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        const int m = t * 16 + hlf * 8 + g;
        arow[t][hlf] = a_s + (size_t)(row_ok[t][hlf] ? m : 0) * K;
      }
  }
  // Where the keys and values of the lane's rows go.  The page of each row is looked up
  // all rows at once per level of indirection; with few rows this is done before the main
  // loop, so that the three dependent loads run under the weight stream.
  int kv_pos[MT][2], kv_page[MT][2];
  bool kv_ok[MT][2];
  const bool to_cache = kv.pool != nullptr && n0 >= kv.q_width;
  auto find_pages = [&]() {
    int req[MT][2], slot[MT][2];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        const int m = t * 16 + hlf * 8 + g;
        kv_ok[t][hlf] = m < M;
        const int mc = kv_ok[t][hlf] ? m : 0;
        req[t][hlf] = kv.req_of_token[mc];
        kv_pos[t][hlf] = kv.positions[mc];
      }
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) slot[t][hlf] = kv.slots[req[t][hlf]];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        const int p = kv_pos[t][hlf];
        if (kv_ok[t][hlf] && slot[t][hlf] >= 0 && (p < 0 || p >= kv.max_pos)) {
          atomicOr(kv.status, RL_STATUS_BAD_POSITION);
          kv_ok[t][hlf] = false;
        }
        kv_ok[t][hlf] = kv_ok[t][hlf] && slot[t][hlf] >= 0;  // slot -1: padding of a fixed-size batch
        const int sc = kv_ok[t][hlf] ? slot[t][hlf] : 0, pc = kv_ok[t][hlf] ? p : 0;
        kv_page[t][hlf] = kv.block_table[(size_t)sc * kv.bt_stride + pc / kv.page_size];
      }
  };
  constexpr bool EARLY_PAGES = MT <= 2;  // more rows: the registers are needed for the pieces of A
  if (EARLY_PAGES && to_cache) find_pages();
  // the temperatures of the lane's rows, for a product that samples: asked for under the weight stream too
  float temp_of[MT][2];
#pragma unroll
  for (int t = 0; t < MT; ++t) temp_of[t][0] = temp_of[t][1] = 0.f;
  auto find_temperatures = [&]() {
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        const int m = t * 16 + hlf * 8 + g;
        temp_of[t][hlf] = sample.temperature[m < M ? m : 0];
      }
  };
  const bool sampled_rows = sizeof(TOut) == 4 && sample.out_ids != nullptr && sample.temperature != nullptr;
  if (EARLY_PAGES && sampled_rows) find_temperatures();
  for (int k0 = k_begin; k0 < k_end; k0 += 32 * U) {
    // The weight loads are unconditional (an offset outside the part is replaced by the part's
    // first, which is always valid) and what they brought is zeroed afterwards: a load under a
    // condition would not be issued before the one ahead of it has returned.
    uint4 wv[U];
    int ke[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = k0 + 32 * u + 8 * j;
      ok[u] = k < k_end;
      ke[u] = ok[u] ? k : k_begin;
    }
    if (NORM && k0 == k_begin) {
#pragma unroll
      for (int u = 0; u < U; ++u) wv[u] = w_first[u];
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) wv[u] = *reinterpret_cast<const uint4*>(wrow + ke[u]);
    }
    {
      // the pieces of A are fetched with the weights, all before anything is used
      // (instructions issue in order: a use between two loads would hold the second back)
      uint4 av[U][MT][2];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          av[u][t][0] = *reinterpret_cast<const uint4*>(arow[t][0] + ke[u]);
          av[u][t][1] = *reinterpret_cast<const uint4*>(arow[t][1] + ke[u]);
        }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!(ok[u] && col_ok)) wv[u] = zero;  // a zero weight makes the matching piece of A irrelevant
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          if (!row_ok[t][0]) av[u][t][0] = zero;
          if (!row_ok[t][1]) av[u][t][1] = zero;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (k0 + 32 * u >= k_end) break;
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          mma_bf16_16816(c[t], av[u][t][0].x, av[u][t][1].x, av[u][t][0].y, av[u][t][1].y, wv[u].x, wv[u].y);
          mma_bf16_16816(c[t], av[u][t][0].z, av[u][t][1].z, av[u][t][0].w, av[u][t][1].w, wv[u].z, wv[u].w);
        }
      }
    }
  }
  if (KSPLIT > 1) {
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) part_s[group][part][t][lane][i] = c[t][i];
    __syncthreads();
    if (part != 0) return;
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float acc = 0.f;
#pragma unroll
        for (int q = 0; q < KSPLIT; ++q) acc += part_s[group][q][t][lane][i];
        c[t][i] = acc;
      }
  }
  // accumulator layout: c0, c1 = row g, columns 2j, 2j+1; c2, c3 = row g+8, the same columns
  const int n = n0 + 2 * j;
  const float bias0 = (bias != nullptr && blockIdx.y == 0 && n < N) ? bias[n] : 0.f;
  const float bias1 = (bias != nullptr && blockIdx.y == 0 && n + 1 < N) ? bias[n + 1] : 0.f;
  if constexpr (sizeof(TOut) == 4) {
    if (gridDim.y > 1) {
      // K over several blocks: each adds its part into the residual stream (in no fixed order)
#pragma unroll
      for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int m = t * 16 + g + (i >> 1) * 8, nn = n + (i & 1);
          if (m < M && nn < N) atomicAdd(reinterpret_cast<float*>(out) + (size_t)m * ldo + nn, c[t][i] + ((i & 1) ? bias1 : bias0));
        }
      return;
    }
    if (sample.out_ids != nullptr) {
      if (!EARLY_PAGES && sampled_rows) find_temperatures();
      bool offered = false;
#pragma unroll
      for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          const int m = t * 16 + hlf * 8 + g;
          const int mc = m < M ? m : 0;  // every lane takes part in the exchanges below
          const float temp = temp_of[t][hlf];
          float s0 = apply_act(c[t][2 * hlf] + bias0, act), s1 = apply_act(c[t][2 * hlf + 1] + bias1, act);
          if (temp > 0.f) {
            const uint64_t seed = (uint64_t)sample.seeds[mc];
            const uint32_t counter = (uint32_t)sample.counters[mc];
            const float inv_t = 1.0f / temp;
            s0 = sample_key(s0, inv_t, seed, counter, (uint32_t)n);
            s1 = sample_key(s1, inv_t, seed, counter, (uint32_t)(n + 1));
          }
          ArgMax best{-CUDART_INF_F, 0x7fffffff};
          if (n < N) best = ArgMax{s0, n};
          if (n + 1 < N) best = better(best, ArgMax{s1, n + 1});
#pragma unroll
          for (int o = 1; o <= 2; o <<= 1) {
            const ArgMax b{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
            best = better(best, b);
          }
          if (j == 0 && m < M && best.i != 0x7fffffff) {
            const unsigned long long word =
                ((unsigned long long)ordered_bits(best.v) << 32) | (unsigned long long)(~(uint32_t)best.i);
            if (word > __ldcg(sample.best + m)) {
              atomicMax(sample.best + m, word);
              offered = true;
            }
          }
        }
      if (offered) __threadfence();  // the offer is in place before the ticket is taken
      __syncwarp();
      int last = 0;
      if (lane == 0) last = atomicAdd(sample.ticket, 1) == (int)(gridDim.x * GROUPS) - 1;
      last = __shfl_sync(0xffffffffu, last, 0);
      if (last) sample_finish(sample, M, lane);
      return;
    }
  }
  if (to_cache) {
    // The eight columns of the group are keys or values of one head (the query width and the
    // head size are multiples of 16): they go to the page of the row's position.
    if (!EARLY_PAGES) find_pages();
    const int cidx = n - kv.q_width;
    const int which = cidx / kv.kv_width;
    const int rem = cidx - which * kv.kv_width;
    const int head = rem / kv.head_dim, d = rem - head * kv.head_dim;
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        if (!kv_ok[t][hlf] || n >= N) continue;
        if (kv_page[t][hlf] < 0) {
          atomicOr(kv.status, RL_STATUS_BAD_PAGE);
          continue;
        }
        const float v0 = apply_act(c[t][2 * hlf] + bias0, act), v1 = apply_act(c[t][2 * hlf + 1] + bias1, act);
        __nv_bfloat16* dst = (__nv_bfloat16*)kv.pool +
                             ((((size_t)kv_page[t][hlf] * 2 + which) * kv.n_kv_heads + head) * kv.page_size +
                              kv_pos[t][hlf] % kv.page_size) * kv.head_dim + d;
        const __nv_bfloat162 pr = __floats2bfloat162_rn(v0, v1);
        *reinterpret_cast<__nv_bfloat162*>(dst) = pr;  // d is even: the pair is 4-byte aligned
      }
    return;
  }
  // What the residual stream holds is fetched for all of the lane's outputs before the first
  // store (from a valid place where the output lies outside): a load behind a store to the
  // same array would wait for it.
  float old[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) old[t][i] = 0.f;
  if constexpr (sizeof(TOut) == 4) {
    if (residual) {
#pragma unroll
      for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int m = min(t * 16 + g + (i >> 1) * 8, M - 1);
          const int nn = min(n + (i & 1), N - 1);
          old[t][i] = to_f32(out[(size_t)m * ldo + nn]);
        }
    }
  }
#pragma unroll
  for (int t = 0; t < MT; ++t) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = t * 16 + g + (i >> 1) * 8;
      const int nn = n + (i & 1);
      if (m < M && nn < N) {
        const float v = apply_act(c[t][i] + ((i & 1) ? bias1 : bias0), act);
        out[(size_t)m * ldo + nn] = from_f32<TOut>(v + old[t][i]);
      }
    }
  }
}

// How many blocks of one form of the kernel an SM holds (registers and shared memory decide).
template <typename TOut, int MT, int KS>
static int rows_mma_blocks_per_sm() {
  static int nb = -1;
  if (nb < 0) {
    int v = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, gemm_rows_mma_kernel<TOut, MT, KS, 1, false>, 32 * KS, 0) !=
            cudaSuccess || v < 1)
      v = 1;
    nb = v;
  }
  return nb;
}

static bool k_blocks_allowed = true;  // (off: for comparisons)

template <typename TOut, int MT>
static void launch_rows_mma(const __nv_bfloat16* a, long lda, const NormArgs& norm, const __nv_bfloat16* w,
                            const float* bias, TOut* o, long ldo, int M, int N, int K, int act, int residual,
                            const KvScatter& kv, cudaStream_t stream, const SampleArgs& sample = SampleArgs{}) {
  const int groups = (N + 7) / 8;
  const int chunks = (K + 31) / 32;
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  // warps enough to have the whole matrix, or some thousands of loads, in flight at once ...
  int ks = 1;
  while (ks < 16 && groups * ks < 2400 && chunks / (ks * 2) >= 2) ks *= 2;
  // ... but no more than are resident at once, or a quarter more: a second, mostly empty round of
  // blocks costs more than longer parts of K per warp, a short one less (6400 x 1600 at 8 rows:
  // 800 groups on 740 places, 9.7 us with K in four parts against 12.4 in two)
  auto fits = [&](int k) {
    int nb = 1;
    switch (k) {
      case 2: nb = rows_mma_blocks_per_sm<TOut, MT, 2>(); break;
      case 4: nb = rows_mma_blocks_per_sm<TOut, MT, 4>(); break;
      case 8: nb = rows_mma_blocks_per_sm<TOut, MT, 8>(); break;
      case 16: nb = rows_mma_blocks_per_sm<TOut, MT, 16>(); break;
      default: return true;
    }
    return groups * 4 <= n_sms * nb * 5;
  };
  while (ks > 1 && !fits(ks)) ks /= 2;
  // An `out += ...` into float32 whose blocks leave the SMs short of warps (a narrow output with a
  // long inner size: 1600 x 6400 gives 200 blocks of eight warps, eleven warps an SM, 22 KB of
  // weights on the way per SM) has its K shared between two blocks a group.
  int k_blocks = 1;
  if (sizeof(TOut) == 4 && residual && act == RL_ACT_NONE && kv.pool == nullptr && sample.out_ids == nullptr &&
      norm.x == nullptr && k_blocks_allowed && (long)groups * ks < (long)n_sms * 16 && chunks / (ks * 2) >= 2)
    k_blocks = 2;
  const size_t smem = norm.x != nullptr ? (size_t)M * K * sizeof(__nv_bfloat16) + 2 * (size_t)K * sizeof(float) : 0;
#define RL_MMA(KS, GR)                                                                                        \
  do {                                                                                                        \
    if constexpr (MT == 1) {                                                                                  \
      if (norm.x != nullptr) {                                                                                \
        launch_pdl(gemm_rows_mma_kernel<TOut, MT, KS, GR, true>, (groups + GR - 1) / GR, 32 * KS * GR, smem,   \
                   stream, a, lda, norm, w, bias, o, ldo, M, N, K, act, residual, kv, sample);                \
        break;                                                                                                \
      }                                                                                                       \
    }                                                                                                         \
    launch_pdl(gemm_rows_mma_kernel<TOut, MT, KS, GR, false>, dim3((groups + GR - 1) / GR, k_blocks), 32 * KS * GR, 0, stream,  \
               a, lda, norm, w, bias, o, ldo, M, N, K, act, residual, kv, sample);                            \
  } while (0)
  switch (ks) {
    case 1: RL_MMA(1, 1); break;
    case 2: RL_MMA(2, 1); break;
    case 4: RL_MMA(4, 1); break;
    case 8: RL_MMA(8, 1); break;
    default: RL_MMA(16, 1); break;
  }
#undef RL_MMA
}

}  // namespace rl

// bfloat16 A [M <= 64, K] (row stride lda) and W [N, K]; out bfloat16 or float32 [M, N].
// residual != 0: out (float32) += result.  norm_x != nullptr: the input is LayerNorm(norm_x)
// (float32 rows, at most 16 of at most 1024 elements) and A is ignored.  kv_pool != nullptr:
// output columns from kv_q_width on are written into cache pages as keys and values, not out.
RL_EXPORT int rl_gemm_rows_bf16(int out_dtype, const void* A, long lda, const void* W, const float* bias,
                                void* out, long ldo, int M, int N, int K, int act, int residual,
                                const float* norm_x, long norm_ldx, const float* norm_gamma,
                                const float* norm_beta, float norm_eps, void* kv_pool,
                                const int* kv_block_table, int kv_bt_stride, const int* kv_positions,
                                const int* kv_req_of_token, const int* kv_slots, int kv_q_width, int kv_width,
                                int kv_head_dim, int kv_page_size, int kv_heads, int kv_max_pos, int* status,
                                cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64) return -5;
  if (K % 8 != 0 || ((uintptr_t)W % 16) != 0) return -2;
  if (norm_x == nullptr && (lda % 8 != 0 || ((uintptr_t)A % 16) != 0)) return -2;
  if (norm_x != nullptr && (M > 16 || K > 1024 || norm_ldx % 4 != 0 || ((uintptr_t)norm_x % 16) != 0 ||
                            ((uintptr_t)norm_gamma % 16) != 0 || (norm_beta != nullptr && ((uintptr_t)norm_beta % 16) != 0)))
    return -6;
  if (residual && out_dtype != RL_F32) return -3;
  const rl::NormArgs norm{norm_x, norm_ldx, norm_gamma, norm_beta, norm_eps};
  rl::KvScatter kv{kv_pool, kv_block_table, kv_bt_stride, kv_positions, kv_req_of_token, kv_slots,
                   kv_q_width, kv_width, kv_head_dim, kv_page_size, kv_heads, kv_max_pos, status};
  const __nv_bfloat16* a = (const __nv_bfloat16*)A;
  const __nv_bfloat16* w = (const __nv_bfloat16*)W;
  // a very wide float32 output of few rows (a head): the weights by bulk copies into shared memory
  if (out_dtype == RL_F32 && !residual && act == RL_ACT_NONE && kv_pool == nullptr && status != nullptr) {
    const int warps = rl::bulk::plan_warps(M, N, K, norm_x != nullptr, rl::rows_sm_count());
    if (warps > 0) {
      const cudaError_t e = norm_x != nullptr
          ? rl::bulk::launch<true>(warps, rl::rows_sm_count(), a, lda, norm, w, bias, (float*)out, ldo, M, N, K,
                                   rl::SampleArgs{}, status, stream)
          : rl::bulk::launch<false>(warps, rl::rows_sm_count(), a, lda, norm, w, bias, (float*)out, ldo, M, N, K,
                                    rl::SampleArgs{}, status, stream);
      return e == cudaSuccess ? 0 : (int)e;
    }
  }
#define RL_ROWS_MT(MT)                                                                                        \
  do {                                                                                                        \
    if (out_dtype == RL_F32)                                                                                  \
      rl::launch_rows_mma<float, MT>(a, lda, norm, w, bias, (float*)out, ldo, M, N, K, act, residual, kv, stream);   \
    else                                                                                                      \
      rl::launch_rows_mma<__nv_bfloat16, MT>(a, lda, norm, w, bias, (__nv_bfloat16*)out, ldo, M, N, K, act,    \
                                             residual, kv, stream);                                                     \
  } while (0)
  if (out_dtype != RL_F32 && out_dtype != RL_BF16) return -4;
  if (M <= 16) RL_ROWS_MT(1);
  else if (M <= 32) RL_ROWS_MT(2);
  else RL_ROWS_MT(4);
#undef RL_ROWS_MT
  RL_CHECK_LAUNCH();
  return 0;
}

// The product above with the next token of each row chosen in its epilogue and no logits
// written: out_ids[m] is what rl_sample would choose from row m of A W^T (+ bias) with the same
// temperature, seed and counter (rows with top-k or top-p are not for this entry point).
// best [M] and ticket [1] are scratch that is zero before the call and zero again after it.
// host_ring != nullptr: the ids are also written to that pinned host memory (see SampleArgs).
RL_EXPORT int rl_gemm_rows_bf16_sample(const void* A, long lda, const void* W, const float* bias, int M, int N, int K,
                                       const float* norm_x, long norm_ldx, const float* norm_gamma,
                                       const float* norm_beta, float norm_eps, const float* temperature,
                                       const long long* seeds, const int* counters, int* out_ids,
                                       unsigned long long* best, int* ticket, int* host_ring, int ring_stride,
                                       unsigned int* ring_step, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64) return -5;
  if (out_ids == nullptr || best == nullptr || ticket == nullptr) return -7;
  if (temperature != nullptr && (seeds == nullptr || counters == nullptr)) return -7;
  if (K % 8 != 0 || ((uintptr_t)W % 16) != 0) return -2;
  if (norm_x == nullptr && (lda % 8 != 0 || ((uintptr_t)A % 16) != 0)) return -2;
  if (norm_x != nullptr && (M > 16 || K > 1024 || norm_ldx % 4 != 0 || ((uintptr_t)norm_x % 16) != 0 ||
                            ((uintptr_t)norm_gamma % 16) != 0 || (norm_beta != nullptr && ((uintptr_t)norm_beta % 16) != 0)))
    return -6;
  const rl::NormArgs norm{norm_x, norm_ldx, norm_gamma, norm_beta, norm_eps};
  const rl::KvScatter kv{};
  if (host_ring != nullptr && (ring_step == nullptr || ring_stride < M)) return -7;
  const rl::SampleArgs sample{out_ids, temperature, seeds, counters, best, ticket, host_ring, ring_stride, ring_step};
  const __nv_bfloat16* a = (const __nv_bfloat16*)A;
  const __nv_bfloat16* w = (const __nv_bfloat16*)W;
  if (status != nullptr) {
    const int warps = rl::bulk::plan_warps(M, N, K, norm_x != nullptr, rl::rows_sm_count());
    if (warps > 0) {
      const cudaError_t e = norm_x != nullptr
          ? rl::bulk::launch<true>(warps, rl::rows_sm_count(), a, lda, norm, w, bias, nullptr, 0, M, N, K, sample, status, stream)
          : rl::bulk::launch<false>(warps, rl::rows_sm_count(), a, lda, norm, w, bias, nullptr, 0, M, N, K, sample, status, stream);
      return e == cudaSuccess ? 0 : (int)e;
    }
  }
  if (M <= 16)
    rl::launch_rows_mma<float, 1>(a, lda, norm, w, bias, nullptr, 0, M, N, K, RL_ACT_NONE, 0, kv, stream, sample);
  else if (M <= 32)
    rl::launch_rows_mma<float, 2>(a, lda, norm, w, bias, nullptr, 0, M, N, K, RL_ACT_NONE, 0, kv, stream, sample);
  else
    rl::launch_rows_mma<float, 4>(a, lda, norm, w, bias, nullptr, 0, M, N, K, RL_ACT_NONE, 0, kv, stream, sample);
  RL_CHECK_LAUNCH();
  return 0;
}

// The kernel of gemm_rows_bulk.cuh on or off (on by default; off, heads of few rows run on the
// kernel above, for comparisons).
RL_EXPORT void rl_gemm_rows_bulk_enable(int on) {
  rl::bulk::enabled = on != 0;
  rl::k_blocks_allowed = on != 0;  // the same switch takes the newer forms of the register-fed kernel off
}

