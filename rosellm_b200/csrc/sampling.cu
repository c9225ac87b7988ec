// Next-token choice from a row of logits: greedy, temperature, top-k and top-p.
//
// What is sampled follows rosellm/roseinfer/engine.py:1104-1171: temperature <= 0 (or no
// sampling) takes the arg-max; otherwise logits are divided by the temperature, top-k keeps
// the k largest, top-p (applied to the softmax of what top-k kept) removes every token whose
// cumulative probability, largest first and counting itself, exceeds p, except the largest;
// one token is drawn from the softmax of the rest.
//
// How it is drawn differs: the reference calls torch.multinomial on a process-wide generator,
// so a request's tokens depend on what else is in the batch.  Here the draw is the arg-max of
// logit/T + Gumbel noise, the noise of vocabulary entry i being a function of (request seed,
// index of the generated token, i) through Philox-4x32-10: the same request gets the same
// tokens whatever shares its batch, and no sort or prefix sum is needed.  The thresholds of
// top-k and top-p are found by bisection on the bit pattern of the logits (32 counting passes
// each), which keeps exactly the set the sort-based formulation keeps when no two logits tie
// at the threshold.
#include <math_constants.h>

#include "common.cuh"

namespace rl {

__device__ __forceinline__ uint32_t ordered_bits(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint32_t philox_first(uint32_t c0, uint32_t c1, uint32_t k0, uint32_t k1) {
  uint32_t c2 = 0u, c3 = 0u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

// Gumbel noise of vocabulary entry `index` for the `counter`-th generated token of a request.
__device__ __forceinline__ float gumbel_noise(uint64_t seed, uint32_t counter, uint32_t index) {
  const uint32_t x = philox_first(index, counter, (uint32_t)seed, (uint32_t)(seed >> 32));
  const float u = ((float)(x >> 8) + 0.5f) * 5.9604644775390625e-08f;  // (0, 1), 2^-24 steps
  return -logf(-logf(u));
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ ArgMax block_argmax(ArgMax a, ArgMax* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b{__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
    a = better(a, b);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = a;
  __syncthreads();
  if (warp == 0) {
    ArgMax t = lane < nwarps ? scratch[lane] : ArgMax{-CUDART_INF_F, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax b{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
      t = better(t, b);
    }
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Blocks (row, chunk).  Rows that need no filter (greedy, or temperature alone) are handled by
// all `gridDim.y` blocks of the row, each over its part of the vocabulary; partial winners go
// to `part` ([rows][chunks][2]: score, index bits) and the block that ends last, known by a
// ticket from `tickets[row]` (zero before and after the call), picks among them.  Rows with
// top-k or top-p are handled whole by the row's first block.  kept[row] (optional) receives
// how many tokens survived the filters.
__global__ __launch_bounds__(256) void sample_kernel(
    const float* __restrict__ logits, long ld, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p,
    const long long* __restrict__ seeds, const int* __restrict__ counters, int* __restrict__ out_ids,
    int* __restrict__ kept, float* __restrict__ part, int* __restrict__ tickets) {
  __shared__ float fs[33];
  __shared__ ArgMax as[33];
  __shared__ int last_s;
  pdl_begin();
  const int row = blockIdx.x;
  const int n_chunks = gridDim.y, chunk_id = blockIdx.y;
  const float* x = logits + (size_t)row * ld;
  const float temp = temperature != nullptr ? temperature[row] : 0.f;
  const int k_row = (temp > 0.f && top_k != nullptr) ? top_k[row] : 0;
  const float p_row = (temp > 0.f && top_p != nullptr) ? top_p[row] : 1.f;
  const bool filtered = (k_row > 0 && k_row < vocab) || (p_row > 0.f && p_row < 1.f);
  if (!filtered) {
    const int span = (vocab + n_chunks - 1) / n_chunks;
    const int lo = chunk_id * span, hi = min(vocab, lo + span);
    ArgMax best{-CUDART_INF_F, 0x7fffffff};
    if (temp > 0.f) {
      const uint64_t seed = (uint64_t)seeds[row];
      const uint32_t counter = (uint32_t)counters[row];
      const float inv_t = 1.0f / temp;
      for (int i = lo + threadIdx.x; i < hi; i += blockDim.x)
        best = better(best, ArgMax{x[i] * inv_t + gumbel_noise(seed, counter, (uint32_t)i), i});
    } else {
      for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) best = better(best, ArgMax{x[i], i});
    }
    best = block_argmax(best, as);
    if (n_chunks == 1) {
      if (threadIdx.x == 0) {
        out_ids[row] = best.i;
        if (kept != nullptr) kept[row] = temp > 0.f ? vocab : 1;
      }
      return;
    }
    float* mine = part + ((size_t)row * n_chunks + chunk_id) * 2;
    if (threadIdx.x == 0) {
      mine[0] = best.v;
      mine[1] = __int_as_float(best.i);
      __threadfence();
      last_s = atomicAdd(&tickets[row], 1) == n_chunks - 1;
    }
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    ArgMax all{-CUDART_INF_F, 0x7fffffff};
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
      const float* theirs = part + ((size_t)row * n_chunks + c) * 2;
      all = better(all, ArgMax{__ldcg(theirs), __float_as_int(__ldcg(theirs + 1))});
    }
    all = block_argmax(all, as);
    if (threadIdx.x == 0) {
      out_ids[row] = all.i;
      if (kept != nullptr) kept[row] = temp > 0.f ? vocab : 1;
      tickets[row] = 0;
    }
    return;
  }
  if (chunk_id != 0) return;
  const int k = top_k != nullptr ? top_k[row] : 0;
  const float pp = top_p != nullptr ? top_p[row] : 1.f;
  const bool use_k = k > 0 && k < vocab;
  const bool use_p = pp > 0.f && pp < 1.f;
  uint32_t thr = 0u;  // keep entries whose ordered bits are >= thr
  if (use_k) {
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = thr | (1u << bit);
      float c = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += ordered_bits(x[i]) >= cand ? 1.f : 0.f;
      if (block_sum(c, fs) >= (float)k) thr = cand;
    }
  }
  if (use_p) {
    ArgMax best{-CUDART_INF_F, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, ArgMax{x[i], i});
    best = block_argmax(best, as);
    const float mx = best.v;
    const float inv_t = 1.0f / temp;
    float z = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x)
      if (ordered_bits(x[i]) >= thr) z += expf((x[i] - mx) * inv_t);
    z = block_sum(z, fs);
    const float limit = pp * z;
    // Largest threshold whose kept mass still exceeds the limit, built bit by bit from the
    // top: the mass kept at threshold c, among what top-k left, falls as c rises.
    uint32_t t = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = t | (1u << bit);
      const uint32_t cut = cand > thr ? cand : thr;
      float s = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x)
        if (ordered_bits(x[i]) >= cut) s += expf((x[i] - mx) * inv_t);
      if (block_sum(s, fs) > limit) t = cand;
    }
    const uint32_t top = ordered_bits(mx);
    thr = t >= top ? top : t + 1u;
  }
  const uint64_t seed = (uint64_t)seeds[row];
  const uint32_t counter = (uint32_t)counters[row];
  const float inv_t = 1.0f / temp;
  ArgMax best{-CUDART_INF_F, 0x7fffffff};
  float cnt = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = x[i];
    if (ordered_bits(v) >= thr) {
      cnt += 1.f;
      best = better(best, ArgMax{v * inv_t + gumbel_noise(seed, counter, (uint32_t)i), i});
    }
  }
  best = block_argmax(best, as);
  if (kept != nullptr) {
    cnt = block_sum(cnt, fs);
    if (threadIdx.x == 0) kept[row] = (int)cnt;
  }
  if (threadIdx.x == 0) out_ids[row] = best.i;
}

}  // namespace rl

// part: n_rows*n_chunks*2 floats of scratch and tickets: n_rows ints that are zero (they are
// zero again afterwards), both needed when n_chunks > 1.
RL_EXPORT int rl_sample(const float* logits, long ld, int n_rows, int vocab,
                        const float* temperature, const int* top_k, const float* top_p,
                        const long long* seeds, const int* counters, int* out_ids, int* kept,
                        int n_chunks, float* part, int* tickets, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (vocab <= 0) return -2;
  if (n_chunks < 1 || (n_chunks > 1 && (part == nullptr || tickets == nullptr))) return -3;
  rl::launch_pdl(rl::sample_kernel, dim3(n_rows, n_chunks), 256, 0, stream, logits, ld, vocab, temperature,
                 top_k, top_p, seeds, counters, out_ids, kept, part, tickets);
  RL_CHECK_LAUNCH();
  return 0;
}
