// bfloat16 products of at most 16 rows with a very wide output (a head: 768 -> 50257), float32
// out or the next tokens chosen in the epilogue: the weight-streaming product of
// gemm_rows_mma.cu with the stream taken off the registers.
//
// There a warp's weights travel through its registers, four loads of 16 bytes a lane in flight,
// and the registers they occupy limit an SM to 24 warps: 48 KB on the way per SM, hardly what
// the memory's latency times its bandwidth asks for, and none while a warp computes (a head of
// 77 MB took 20.5 us, 0.58 of the copy bandwidth).  Here one block per SM stays for the whole
// product; each of its warps takes every (blocks x warps)-th group of eight output columns,
// whose weight rows lie one behind the other in memory, and has them copied by the copy engine
// (one cp.async.bulk of 16 K bytes, completion counted on an mbarrier) into one of its two
// buffers in shared memory while it works on the other: 100 to 200 KB are on the way per SM
// whatever the registers hold.  The first two groups of every warp are asked for before the wait
// for the kernels ahead (weights are written by none of them), so that in a decode step the head's
// table starts to arrive while the final norm still runs.  The rows of A (or their LayerNorm)
// are put into shared memory once a block, in rows 64 bytes longer than K elements, so that the
// eight lanes of a 16-byte access phase (two rows, four pieces each) hit different banks; the
// weight rows stay as they lie in memory (a copy a row into padded rows measured no faster).
// A warp's MMAs go to two sets of accumulators in turn: each waits for the one before it on its
// set, and eight warps an SM hide little.  Included by gemm_rows_mma.cu, whose NormArgs,
// SampleArgs and MMA wrapper it uses.
#pragma once

namespace rl {
namespace bulk {

constexpr int MAX_WARPS = 8;
constexpr int ROW_PAD = 64;                 // bytes
constexpr int SMEM_LIMIT = 220 * 1024;

__device__ __forceinline__ uint32_t shared_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool barrier_passed(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// Waits for the phase, for about two seconds at most; false (and the status bit set) when it gave up.
__device__ __forceinline__ bool barrier_wait(uint32_t bar, uint32_t parity, int* status) {
  if (barrier_passed(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 0;; ++it) {
    if (barrier_passed(bar, parity)) return true;
    if ((it & 0xffu) == 0xffu && clock64() - t0 > 4000000000LL) {
      atomicOr(status, RL_STATUS_WAIT_TIMEOUT);
      return false;
    }
  }
}

__host__ __device__ inline int row_bytes(int K) { return 2 * K + ROW_PAD; }
// Shared memory: rows of A | gamma and beta (when normalising) | two buffers of eight weight rows a warp | barriers
__host__ __device__ inline size_t smem_bytes(int a_rows, int K, bool norm, int warps) {
  return (size_t)a_rows * row_bytes(K) + (norm ? 2 * (size_t)K * 4 : 0) + (size_t)warps * 2 * 8 * 2 * K +
         (size_t)warps * 2 * 8 + 16;
}

template <bool NORM>
__global__ __launch_bounds__(32 * MAX_WARPS) void gemm_rows_bulk_kernel(
    const __nv_bfloat16* __restrict__ A, long lda, NormArgs norm, const __nv_bfloat16* __restrict__ W,
    const float* __restrict__ bias, float* __restrict__ out, long ldo, int M, int N, int K, SampleArgs sample,
    int* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int g = lane >> 2, j = lane & 3;
  const int rb = row_bytes(K);
  const int a_rows = M <= 8 ? 8 : 16;
  uint8_t* a_s = smem;
  float* gb_s = reinterpret_cast<float*>(smem + (size_t)a_rows * rb);
  const int wb = 8 * 2 * K;  // a buffer: a group's eight weight rows as they lie in memory
  uint8_t* w_s = reinterpret_cast<uint8_t*>(gb_s) + (NORM ? 2 * (size_t)K * 4 : 0) + (size_t)warp * 2 * wb;
  const uint32_t bar0 = shared_u32(smem + (size_t)a_rows * rb + (NORM ? 2 * (size_t)K * 4 : 0) + (size_t)n_warps * 2 * wb) +
                        (uint32_t)warp * 16u;
  const int n_groups = (N + 7) / 8;
  const int first = (int)blockIdx.x * n_warps + warp, stride = (int)gridDim.x * n_warps;
  // the copies of a group's weight rows into buffer `stage` of this warp (one lane issues them)
  auto fetch = [&](int group, int stage) {
    const int rows = min(8, N - 8 * group);
    const uint32_t bar = bar0 + 8u * stage;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)(rows * 2 * K)) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     shared_u32(w_s + (size_t)stage * wb)),
                 "l"(W + (size_t)group * 8 * K), "r"((uint32_t)(rows * 2 * K)), "r"(bar)
                 : "memory");
  };
  if (lane == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + 8u));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (first < n_groups) fetch(first, 0);
    if (first + stride < n_groups) fetch(first + stride, 1);
  }
  if constexpr (NORM) {
    // gamma and beta are weights too: on their way before the wait
    const uint32_t dst = shared_u32(gb_s);
    for (int i = threadIdx.x; i < K / 4; i += blockDim.x) {
      asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst + 16 * i), "l"(norm.gamma + 4 * i) : "memory");
      if (norm.beta != nullptr)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst + 4 * K + 16 * i), "l"(norm.beta + 4 * i)
                     : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  pdl_begin();
  // the rows of A into shared memory (rows from M on are zero), or their LayerNorm
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  if constexpr (NORM) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    for (int i = threadIdx.x; i < (a_rows - M) * (rb / 16); i += blockDim.x)
      *reinterpret_cast<uint4*>(a_s + (size_t)M * rb + 16 * (size_t)i) = zero;
    __syncthreads();
    normalise_rows_to_shared(norm, M, K, reinterpret_cast<__nv_bfloat16*>(a_s), rb / 2,
                             reinterpret_cast<const float4*>(gb_s), reinterpret_cast<const float4*>(gb_s + K), warp,
                             n_warps, lane);
  } else {
    const int per_row = K / 8;  // 16-byte pieces of a row
    for (int i = threadIdx.x; i < a_rows * per_row; i += blockDim.x) {
      const int row = i / per_row, piece = i - row * per_row;
      *reinterpret_cast<uint4*>(a_s + (size_t)row * rb + 16 * piece) =
          row < M ? *reinterpret_cast<const uint4*>(A + (size_t)row * lda + 8 * piece) : zero;
    }
  }
  __syncthreads();
  const uint8_t* a_lo = a_s + (size_t)g * rb + 16 * j;           // row g
  const uint8_t* a_hi = a_s + (size_t)(g + 8) * rb + 16 * j;     // row g + 8 (there when a_rows is 16)
  const bool two_halves = a_rows == 16;
  const bool sampling = sample.out_ids != nullptr;
  // the sampling options of the lane's two rows
  float temp2[2] = {0.f, 0.f};
  uint64_t seed2[2] = {0, 0};
  uint32_t counter2[2] = {0, 0};
  if (sampling && sample.temperature != nullptr) {
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      const int m = hlf * 8 + g;
      const int mc = m < M ? m : 0;
      temp2[hlf] = sample.temperature[mc];
      if (temp2[hlf] > 0.f) {
        seed2[hlf] = (uint64_t)sample.seeds[mc];
        counter2[hlf] = (uint32_t)sample.counters[mc];
      }
    }
  }
  ArgMax best_lo{-CUDART_INF_F, 0x7fffffff}, best_hi{-CUDART_INF_F, 0x7fffffff};
  bool ok = true;
  int it = 0;
  for (int group = first; group < n_groups; group += stride, ++it) {
    const int stage = it & 1;
    ok = barrier_wait(bar0 + 8u * stage, (uint32_t)(it >> 1) & 1u, status);
    if (!ok) break;
    const uint8_t* w_row = w_s + (size_t)stage * wb + (size_t)g * 2 * K + 16 * j;
    // Two sets of accumulators, taken in turn: every MMA waits for the one before it on the same
    // set, and a warp has few others to hide that behind (eight warps an SM).  A lane's eight
    // consecutive elements of K serve two MMA steps (A and W permuted alike).
    float c[4] = {0.f, 0.f, 0.f, 0.f}, d[4] = {0.f, 0.f, 0.f, 0.f};
    const int k_pairs = K & ~63;
    auto chunk = [&](float (&acc)[4], int k0) {
      const uint4 wv = *reinterpret_cast<const uint4*>(w_row + 2 * k0);
      const uint4 lo = *reinterpret_cast<const uint4*>(a_lo + 2 * k0);
      const uint4 hi = two_halves ? *reinterpret_cast<const uint4*>(a_hi + 2 * k0) : zero;
      mma_bf16_16816(acc, lo.x, hi.x, lo.y, hi.y, wv.x, wv.y);
      mma_bf16_16816(acc, lo.z, hi.z, lo.w, hi.w, wv.z, wv.w);
    };
#pragma unroll 4
    for (int k0 = 0; k0 < k_pairs; k0 += 64) {
      chunk(c, k0);
      chunk(d, k0 + 32);
    }
    if (K - k_pairs >= 32) chunk(c, k_pairs);
    if (K & 31) {
      // the last, partial chunk: beyond K lies whatever the buffers held
      const int k0 = K & ~31;
      const bool in_k = k0 + 8 * j < K;
      uint4 wv = *reinterpret_cast<const uint4*>(w_row + 2 * k0);
      uint4 lo = *reinterpret_cast<const uint4*>(a_lo + 2 * k0);
      uint4 hi = two_halves ? *reinterpret_cast<const uint4*>(a_hi + 2 * k0) : zero;
      if (!in_k) wv = lo = hi = zero;
      mma_bf16_16816(d, lo.x, hi.x, lo.y, hi.y, wv.x, wv.y);
      mma_bf16_16816(d, lo.z, hi.z, lo.w, hi.w, wv.z, wv.w);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] += d[i];
    // every lane has read the buffer: the group after next may be copied into it (the reads were
    // ordinary ones, the copy goes through the async proxy)
    __syncwarp();
    if (lane == 0 && group + 2 * stride < n_groups) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      fetch(group + 2 * stride, stage);
    }
    // accumulator layout: c0, c1 = row g, columns 2j, 2j+1; c2, c3 = row g+8, the same columns
    const int n = group * 8 + 2 * j;
    const float bias0 = (bias != nullptr && n < N) ? bias[n] : 0.f;
    const float bias1 = (bias != nullptr && n + 1 < N) ? bias[n + 1] : 0.f;
    if (!sampling) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = g + (i >> 1) * 8, nn = n + (i & 1);
        if (m < M && nn < N) out[(size_t)m * ldo + nn] = c[i] + ((i & 1) ? bias1 : bias0);
      }
      continue;
    }
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      const float temp = temp2[hlf];
      float s0 = c[2 * hlf] + bias0, s1 = c[2 * hlf + 1] + bias1;
      if (temp > 0.f) {
        const float inv_t = 1.0f / temp;
        s0 = sample_key(s0, inv_t, seed2[hlf], counter2[hlf], (uint32_t)n);
        s1 = sample_key(s1, inv_t, seed2[hlf], counter2[hlf], (uint32_t)(n + 1));
      }
      ArgMax& best = hlf ? best_hi : best_lo;
      if (n < N) best = better(best, ArgMax{s0, n});
      if (n + 1 < N) best = better(best, ArgMax{s1, n + 1});
    }
  }
  if (!ok) {
    // copies that are still on their way end before the block does (bounded by time)
    const long long t0 = clock64();
    for (int d = 0; d < 2; ++d)
      while (!barrier_passed(bar0 + 8u * ((it + d) & 1), (uint32_t)((it + d) >> 1) & 1u) && clock64() - t0 < 400000000LL) {
      }
  }
  if (!sampling) return;
  // a warp's best per row over all its groups, offered once; then one ticket a block
  bool offered = false;
#pragma unroll
  for (int hlf = 0; hlf < 2; ++hlf) {
    ArgMax best = hlf ? best_hi : best_lo;
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      const ArgMax b{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, b);
    }
    const int m = hlf * 8 + g;
    if (j == 0 && m < M && best.i != 0x7fffffff) {
      const unsigned long long word =
          ((unsigned long long)ordered_bits(best.v) << 32) | (unsigned long long)(~(uint32_t)best.i);
      if (word > __ldcg(sample.best + m)) {
        atomicMax(sample.best + m, word);
        offered = true;
      }
    }
  }
  if (offered) __threadfence();
  __syncthreads();
  if (warp == 0) {
    int last = 0;
    if (lane == 0) last = atomicAdd(sample.ticket, 1) == (int)gridDim.x - 1;
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) sample_finish(sample, M, lane);
  }
}

static bool enabled = true;

// How many warps a block of this kernel gets for these sizes; 0 when the product is not one for it
// (few columns: the warps of one round of blocks would not all have their two groups).
static int plan_warps(int M, int N, int K, bool norm, int n_sms) {
  if (!enabled || M > 16 || K % 8 != 0 || (norm && K > 1024)) return 0;
  const int a_rows = M <= 8 ? 8 : 16;
  int warps = MAX_WARPS;
  while (warps > 0 && smem_bytes(a_rows, K, norm, warps) > (size_t)SMEM_LIMIT) --warps;
  if (warps < 2) return 0;
  if ((N + 7) / 8 < 4 * n_sms * warps) return 0;
  return warps;
}

template <bool NORM>
static cudaError_t launch(int warps, int n_sms, const __nv_bfloat16* a, long lda, const NormArgs& norm,
                          const __nv_bfloat16* w, const float* bias, float* out, long ldo, int M, int N, int K,
                          const SampleArgs& sample, int* status, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_rows_bulk_kernel<NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
    attr_set = true;
  }
  const size_t smem = smem_bytes(M <= 8 ? 8 : 16, K, NORM, warps);
  return launch_pdl(gemm_rows_bulk_kernel<NORM>, dim3(n_sms), dim3(32 * warps), smem, stream, a, lda, norm, w, bias, out,
                    ldo, M, N, K, sample, status);
}

}  // namespace bulk
}  // namespace rl
