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
// top-k and top-p are found by a radix search on the bit pattern of the logits, most
// significant byte first: four passes each, a pass making a 256-bin histogram (of counts for
// top-k, of probability mass for top-p) of the entries that share the bytes chosen so far.
// Mass is summed in 40-bit fixed point, so that the sums do not depend on the order of the
// additions.  This keeps exactly the set the sort-based formulation keeps when no two logits
// tie at the threshold.
#include <math_constants.h>

#include <type_traits>

#include "common.cuh"
#include "sampling_key.cuh"

namespace rl {

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
// top-k or top-p are left to sample_filtered_kernel.  kept[row] (optional) receives how many
// tokens were candidates.
__global__ __launch_bounds__(256) void sample_kernel(
    const float* __restrict__ logits, long ld, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p,
    const long long* __restrict__ seeds, const int* __restrict__ counters, int* __restrict__ out_ids,
    int* __restrict__ kept, float* __restrict__ part, int* __restrict__ tickets) {
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
  if (filtered) return;  // sample_filtered_kernel has this row
  {
    const int span = (vocab + n_chunks - 1) / n_chunks;
    const int lo = chunk_id * span, hi = min(vocab, lo + span);
    ArgMax best{-CUDART_INF_F, 0x7fffffff};
    if (temp > 0.f) {
      const uint64_t seed = (uint64_t)seeds[row];
      const uint32_t counter = (uint32_t)counters[row];
      const float inv_t = 1.0f / temp;
      for (int i = lo + threadIdx.x; i < hi; i += blockDim.x)
        best = better(best, ArgMax{sample_key(x[i], inv_t, seed, counter, (uint32_t)i), i});
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
}

__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    unsigned long long t = lane < nwarps ? scratch[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Rows with top-k or top-p, one block of 1024 threads a row (rows without a filter return at
// once: sample_kernel has them).  kept[row] (optional) receives how many tokens survived.
constexpr int FILTER_THREADS = 1024;

__global__ __launch_bounds__(FILTER_THREADS) void sample_filtered_kernel(
    const float* __restrict__ logits, long ld, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const long long* __restrict__ seeds,
    const int* __restrict__ counters, int* __restrict__ out_ids, int* __restrict__ kept) {
  __shared__ unsigned int count_s[256];
  __shared__ unsigned long long mass_s[256];
  __shared__ float fs[33];
  __shared__ ArgMax as[33];
  __shared__ unsigned long long us[33];
  __shared__ uint32_t chosen_prefix;
  __shared__ int chosen_remaining;
  __shared__ unsigned long long chosen_above;
  pdl_begin();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31;
  const float* x = logits + (size_t)row * ld;
  const float temp = temperature != nullptr ? temperature[row] : 0.f;
  if (!(temp > 0.f)) return;
  const int k = top_k != nullptr ? top_k[row] : 0;
  const float pp = top_p != nullptr ? top_p[row] : 1.f;
  const bool use_k = k > 0 && k < vocab;
  const bool use_p = pp > 0.f && pp < 1.f;
  if (!use_k && !use_p) return;
  const float inv_t = 1.0f / temp;
  const int rounds = (vocab + FILTER_THREADS - 1) / FILTER_THREADS;  // the same for every thread
  uint32_t thr = 0u;  // keep entries whose ordered bits are >= thr
  if (use_k) {
    // the k-th largest key, byte by byte: among the entries that share the bytes chosen so
    // far, the bin in which the count from the top reaches what is still wanted
    uint32_t prefix = 0u, mask = 0u;
    int remaining = k;
    for (int level = 0; level < 4; ++level) {
      const int shift = 24 - 8 * level;
      if (tid < 256) count_s[tid] = 0u;
      __syncthreads();
      for (int r = 0; r < rounds; ++r) {
        const int i = r * FILTER_THREADS + tid;
        const uint32_t key = i < vocab ? ordered_bits(x[i]) : 0u;
        const bool on = i < vocab && (key & mask) == prefix;
        const uint32_t digit = (key >> shift) & 255u;
        // lanes of a warp that hit the same bin add once, together
        const unsigned peers = __match_any_sync(0xffffffffu, on ? digit : 0xffffffffu);
        if (on && lane == __ffs(peers) - 1) atomicAdd(&count_s[digit], (unsigned)__popc(peers));
      }
      __syncthreads();
      if (tid == 0) {
        int cum = 0, d = 255;
        for (; d > 0; --d) {
          if (cum + (int)count_s[d] >= remaining) break;
          cum += (int)count_s[d];
        }
        chosen_prefix = prefix | ((uint32_t)d << shift);
        chosen_remaining = remaining - cum;
      }
      __syncthreads();
      prefix = chosen_prefix;
      remaining = chosen_remaining;
      mask |= 255u << shift;
    }
    thr = prefix;
  }
  if (use_p) {
    ArgMax best{-CUDART_INF_F, 0x7fffffff};
    for (int i = tid; i < vocab; i += FILTER_THREADS) best = better(best, ArgMax{x[i], i});
    best = block_argmax(best, as);
    const float mx = best.v;
    // probability mass in units of 2^-40 of the largest entry's: integer sums are the same in
    // every order
    auto mass_of = [&](float v) { return __float2ull_rn(expf((v - mx) * inv_t) * 1099511627776.f); };
    unsigned long long z = 0ull;
    for (int i = tid; i < vocab; i += FILTER_THREADS)
      if (ordered_bits(x[i]) >= thr) z += mass_of(x[i]);
    z = block_sum_u64(z, us);
    const unsigned long long limit = (unsigned long long)((double)pp * (double)z);
    // the largest threshold t whose kept mass (entries >= t, among what top-k left) still
    // exceeds the limit, byte by byte: the mass kept falls as t rises
    uint32_t prefix = 0u, mask = 0u;
    unsigned long long above = 0ull;  // mass of the entries above every key with this prefix
    for (int level = 0; level < 4; ++level) {
      const int shift = 24 - 8 * level;
      if (tid < 256) mass_s[tid] = 0ull;
      __syncthreads();
      for (int r = 0; r < rounds; ++r) {
        const int i = r * FILTER_THREADS + tid;
        const float v = i < vocab ? x[i] : 0.f;
        const uint32_t key = ordered_bits(v);
        const bool on = i < vocab && key >= thr && (key & mask) == prefix;
        const uint32_t digit = (key >> shift) & 255u;
        // lanes of a warp that hit the same bin add once, together: their masses (below 2^41)
        // are summed in three pieces of at most 20 bits by the warp's integer reduction
        const unsigned peers = __match_any_sync(0xffffffffu, on ? digit : 0xffffffffu);
        const unsigned long long mv = on ? mass_of(v) : 0ull;
        const unsigned lo = __reduce_add_sync(peers, (unsigned)(mv & 0xfffffu));
        const unsigned mid = __reduce_add_sync(peers, (unsigned)((mv >> 20) & 0xfffffu));
        const unsigned hi = __reduce_add_sync(peers, (unsigned)(mv >> 40));
        if (on && lane == __ffs(peers) - 1)
          atomicAdd(&mass_s[digit], (unsigned long long)lo + ((unsigned long long)mid << 20) + ((unsigned long long)hi << 40));
      }
      __syncthreads();
      if (tid == 0) {
        unsigned long long cum = above;
        int d = 255;
        for (; d > 0; --d) {
          if (cum + mass_s[d] > limit) break;
          cum += mass_s[d];
        }
        chosen_prefix = prefix | ((uint32_t)d << shift);
        chosen_above = cum;
      }
      __syncthreads();
      prefix = chosen_prefix;
      above = chosen_above;
      mask |= 255u << shift;
    }
    const uint32_t top = ordered_bits(mx);
    thr = prefix >= top ? top : prefix + 1u;
  }
  const uint64_t seed = (uint64_t)seeds[row];
  const uint32_t counter = (uint32_t)counters[row];
  ArgMax best{-CUDART_INF_F, 0x7fffffff};
  float cnt = 0.f;
  for (int i = tid; i < vocab; i += FILTER_THREADS) {
    const float v = x[i];
    if (ordered_bits(v) >= thr) {
      cnt += 1.f;
      best = better(best, ArgMax{sample_key(v, inv_t, seed, counter, (uint32_t)i), i});
    }
  }
  best = block_argmax(best, as);
  if (kept != nullptr) {
    cnt = block_sum(cnt, fs);
    if (tid == 0) kept[row] = (int)cnt;
  }
  if (tid == 0) out_ids[row] = best.i;
}

// ---- the same, a row over a cluster of blocks -------------------------------------------------
//
// The blocks of a cluster (2, 4 or 8, as few as hold the row) each keep a contiguous part of the
// row in shared memory, so the row is read from memory once; a pass makes the block's histogram,
// and after a cluster barrier every block adds up the histograms of all through distributed
// shared memory and draws the same conclusion.  Histograms alternate between two buffers, so
// one barrier a pass is enough.  Every thread of the cluster reaches every barrier.
constexpr int FILTER_MAX_CLUSTER = 8;
constexpr int FILTER_PART = 26 * 1024;  // entries of a row one block keeps (104 KB)

__device__ __forceinline__ unsigned long long peer_u64(const unsigned long long* p, int rank) {
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v)
               : "r"(peer_addr((uint32_t)__cvta_generic_to_shared(p), (uint32_t)rank)) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t peer_u32(const void* p, int rank) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v)
               : "r"(peer_addr((uint32_t)__cvta_generic_to_shared(p), (uint32_t)rank)) : "memory");
  return v;
}

// Threads 0..255 hold the total of bin `tid`; S(d) is the sum of the bins from d up.  Finds the
// one bin d with base + S(d) > bound and base + S(d + 1) <= bound (S falls as d rises; the caller
// guarantees base + S(0) > bound) and returns it to every thread with S(d + 1) in *above_out.
// Called by all threads of the block.
__device__ __forceinline__ int choose_bin(unsigned long long total, unsigned long long base,
                                          unsigned long long bound, unsigned long long* warp_tot,
                                          unsigned long long* chosen, unsigned long long* above_out) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned long long v = tid < 256 ? total : 0ull;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_down_sync(0xffffffffu, v, o);
    if (lane + o < 32) v += t;
  }
  if (tid < 256 && lane == 0) warp_tot[warp] = v;
  __syncthreads();
  if (tid < 256) {
    unsigned long long s = v;
    for (int w = warp + 1; w < 8; ++w) s += warp_tot[w];
    const unsigned long long s_next = s - total;
    if (base + s > bound && base + s_next <= bound) {
      chosen[0] = (unsigned long long)tid;
      chosen[1] = s_next;
    }
  }
  __syncthreads();
  *above_out = chosen[1];
  return (int)chosen[0];
}

// Grid (cluster size, rows); `part` entries of the row per block, a multiple of the block size.
__global__ __launch_bounds__(FILTER_THREADS) void sample_filtered_cluster_kernel(
    const float* __restrict__ logits, long ld, int vocab, int part, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const long long* __restrict__ seeds,
    const int* __restrict__ counters, int* __restrict__ out_ids, int* __restrict__ kept) {
  extern __shared__ float row_s[];                // [part]: this block's entries of the row
  __shared__ unsigned long long hist_s[2][256];   // counts or mass, this block's
  __shared__ unsigned long long warp_tot[8], chosen[2], us[33];
  __shared__ ArgMax as[33];
  __shared__ float fs[33];
  __shared__ ArgMax my_max, my_best;              // read by the other blocks
  __shared__ unsigned long long my_mass;
  __shared__ float my_count;
  pdl_begin();
  const int row = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
  const int rank = (int)cluster_rank(), n_ranks = gridDim.x;
  const float* x = logits + (size_t)row * ld;
  const float temp = temperature != nullptr ? temperature[row] : 0.f;
  const int k = top_k != nullptr ? top_k[row] : 0;
  const float pp = top_p != nullptr ? top_p[row] : 1.f;
  const bool use_k = k > 0 && k < vocab;
  const bool use_p = pp > 0.f && pp < 1.f;
  if (!(temp > 0.f) || (!use_k && !use_p)) return;  // the whole cluster: sample_kernel has this row
  const float inv_t = 1.0f / temp;
  const int first = rank * part;                    // this block's entries: first .. first + mine
  const int mine = max(0, min(part, vocab - first));
  for (int j = tid; j < mine; j += FILTER_THREADS) row_s[j] = x[first + j];
  __syncthreads();

  int pass = 0;  // which histogram buffer
  // one radix pass: the cluster-wide total of bin `tid` (threads 0..255) of `add(value, key)`
  // over this cluster's entries for which `on(key)` holds
  auto histogram = [&](int shift, auto counts, auto on, auto add) -> unsigned long long {
    constexpr bool COUNTS = decltype(counts)::value;
    unsigned long long* h = hist_s[pass & 1];
    if (tid < 256) h[tid] = 0ull;
    __syncthreads();
    for (int j0 = 0; j0 < part; j0 += FILTER_THREADS) {  // the same trips for every thread
      const int j = j0 + tid;
      const float val = row_s[j < mine ? j : 0];
      const uint32_t key = ordered_bits(val);
      const bool o = j < mine && on(key);
      const uint32_t d = (key >> shift) & 255u;
      // lanes of a warp that hit the same bin add once, together: a count is the number of
      // such lanes; masses (below 2^37) are summed in two pieces of at most 19 bits by the
      // warp's integer reduction
      const unsigned peers = __match_any_sync(0xffffffffu, o ? d : 0xffffffffu);
      if constexpr (COUNTS) {
        if (o && lane == __ffs(peers) - 1) atomicAdd(&h[d], (unsigned long long)__popc(peers));
      } else {
        const unsigned long long a = o ? add(val, key) : 0ull;
        const unsigned lo = __reduce_add_sync(peers, (unsigned)(a & 0x7ffffu));
        const unsigned hi = __reduce_add_sync(peers, (unsigned)(a >> 19));
        if (o && lane == __ffs(peers) - 1) atomicAdd(&h[d], (unsigned long long)lo + ((unsigned long long)hi << 19));
      }
    }
    __syncwarp();
    cluster_sync();
    unsigned long long total = 0ull;
    if (tid < 256)
      for (int c = 0; c < n_ranks; ++c) total += peer_u64(&h[tid], c);
    ++pass;
    return total;
  };

  uint32_t thr = 0u;  // keep entries whose ordered bits are >= thr
  if (use_k) {
    // the k-th largest key, byte by byte: the bin in which the count from the top reaches what
    // is still wanted, among the entries that share the bytes chosen so far
    uint32_t prefix = 0u, mask = 0u;
    unsigned long long remaining = (unsigned long long)k;
    for (int level = 0; level < 4; ++level) {
      const int shift = 24 - 8 * level;
      const unsigned long long total = histogram(shift, std::true_type{}, [&](uint32_t key) { return (key & mask) == prefix; },
                                                 [&](float, uint32_t) { return 1ull; });
      unsigned long long above;
      const int d = choose_bin(total, 0ull, remaining - 1ull, warp_tot, chosen, &above);  // S(d) >= remaining
      prefix |= (uint32_t)d << shift;
      mask |= 255u << shift;
      remaining -= above;
    }
    thr = prefix;
  }
  if (use_p) {
    ArgMax best{-CUDART_INF_F, 0x7fffffff};
    for (int j = tid; j < mine; j += FILTER_THREADS) best = better(best, ArgMax{row_s[j], 0});
    best = block_argmax(best, as);
    if (tid == 0) my_max = best;
    __syncwarp();
    cluster_sync();
    float mx = -CUDART_INF_F;
    for (int c = 0; c < n_ranks; ++c) mx = fmaxf(mx, __uint_as_float(peer_u32(&my_max.v, c)));
    // probability mass in units of 2^-36 of the largest entry's: integer sums are the same in
    // every order
    const uint32_t thr_k = thr;
    auto mass = [&](float val) { return __float2ull_rn(expf((val - mx) * inv_t) * 68719476736.f); };
    unsigned long long z = 0ull;
    for (int j = tid; j < mine; j += FILTER_THREADS)
      if (ordered_bits(row_s[j]) >= thr_k) z += mass(row_s[j]);
    z = block_sum_u64(z, us);
    if (tid == 0) my_mass = z;
    __syncwarp();
    cluster_sync();
    z = 0ull;
    for (int c = 0; c < n_ranks; ++c) z += peer_u64(&my_mass, c);
    unsigned long long limit = (unsigned long long)((double)pp * (double)z);
    if (limit >= z) limit = z - 1ull;  // z >= 2^36: the largest entry's own mass
    // the largest threshold t whose kept mass (entries >= t, among what top-k left) still
    // exceeds the limit, byte by byte: the mass kept falls as t rises
    uint32_t prefix = 0u, mask = 0u;
    unsigned long long above = 0ull;  // mass of the entries above every key with this prefix
    for (int level = 0; level < 4; ++level) {
      const int shift = 24 - 8 * level;
      const unsigned long long total =
          histogram(shift, std::false_type{}, [&](uint32_t key) { return key >= thr_k && (key & mask) == prefix; },
                    [&](float val, uint32_t) { return mass(val); });
      unsigned long long inner;
      const int d = choose_bin(total, above, limit, warp_tot, chosen, &inner);
      prefix |= (uint32_t)d << shift;
      mask |= 255u << shift;
      above += inner;
    }
    const uint32_t top = ordered_bits(mx);
    thr = prefix >= top ? top : prefix + 1u;
  }
  const uint64_t seed = (uint64_t)seeds[row];
  const uint32_t counter = (uint32_t)counters[row];
  ArgMax best{-CUDART_INF_F, 0x7fffffff};
  float cnt = 0.f;
  for (int j = tid; j < mine; j += FILTER_THREADS) {
    const float val = row_s[j];
    if (ordered_bits(val) >= thr) {
      cnt += 1.f;
      best = better(best, ArgMax{sample_key(val, inv_t, seed, counter, (uint32_t)(first + j)), first + j});
    }
  }
  best = block_argmax(best, as);
  cnt = block_sum(cnt, fs);
  if (tid == 0) {
    my_best = best;
    my_count = cnt;
  }
  __syncwarp();
  cluster_sync();
  if (rank == 0 && tid == 0) {
    ArgMax all{-CUDART_INF_F, 0x7fffffff};
    float total = 0.f;
    for (int c = 0; c < n_ranks; ++c) {
      all = better(all, ArgMax{__uint_as_float(peer_u32(&my_best.v, c)), (int)peer_u32(&my_best.i, c)});
      total += __uint_as_float(peer_u32(&my_count, c));
    }
    out_ids[row] = all.i;
    if (kept != nullptr) kept[row] = (int)total;
  }
  __syncwarp();
  cluster_sync();  // no block leaves while the first may still read from it
}

// The cluster size for a vocabulary and a number of rows (0: the row is too long for eight
// blocks) and the entries per block: as many blocks a row as hold the row, and more while all
// clusters still run at once (a block fills an SM).
static int filtered_cluster_plan(int vocab, int n_rows, int* part) {
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    if (n_sms <= 0) n_sms = 148;
  }
  int cl = 2;
  auto per = [&](int c) { return ((vocab + c - 1) / c + FILTER_THREADS - 1) / FILTER_THREADS * FILTER_THREADS; };
  while (cl <= FILTER_MAX_CLUSTER && per(cl) > FILTER_PART) cl *= 2;
  if (cl > FILTER_MAX_CLUSTER) return 0;
  while (cl * 2 <= FILTER_MAX_CLUSTER && cl * 2 * n_rows <= n_sms && per(cl * 2) >= FILTER_THREADS) cl *= 2;
  *part = per(cl);
  return cl;
}

static cudaError_t launch_filtered_cluster(int cluster, int part, const float* logits, long ld, int n_rows, int vocab,
                                           const float* temperature, const int* top_k, const float* top_p,
                                           const long long* seeds, const int* counters, int* out_ids, int* kept,
                                           cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    note_launch(cudaFuncSetAttribute(sample_filtered_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     FILTER_PART * (int)sizeof(float)));
    attr_set = true;
  }
  prefer_common_carveout((const void*)sample_filtered_cluster_kernel);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cluster, n_rows);
  cfg.blockDim = dim3(FILTER_THREADS);
  cfg.dynamicSmemBytes = (size_t)part * sizeof(float);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return note_launch(cudaLaunchKernelEx(&cfg, sample_filtered_cluster_kernel, logits, ld, vocab, part, temperature,
                                        top_k, top_p, seeds, counters, out_ids, kept));
}

}  // namespace rl

// part: n_rows*n_chunks*2 floats of scratch and tickets: n_rows ints that are zero (they are
// zero again afterwards), both needed when n_chunks > 1.
// filtered != 0: some row may have top-k or top-p (the second kernel is launched for them).
RL_EXPORT int rl_sample(const float* logits, long ld, int n_rows, int vocab,
                        const float* temperature, const int* top_k, const float* top_p,
                        const long long* seeds, const int* counters, int* out_ids, int* kept,
                        int n_chunks, float* part, int* tickets, int filtered, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (vocab <= 0) return -2;
  if (n_chunks < 1 || (n_chunks > 1 && (part == nullptr || tickets == nullptr))) return -3;
  rl::launch_pdl(rl::sample_kernel, dim3(n_rows, n_chunks), 256, 0, stream, logits, ld, vocab, temperature,
                 top_k, top_p, seeds, counters, out_ids, kept, part, tickets);
  if (filtered && temperature != nullptr && (top_k != nullptr || top_p != nullptr)) {
    // a row over a cluster of blocks that keep it in shared memory; one block a row, re-reading
    // the row each pass, for small vocabularies and for those eight blocks cannot hold
    int part = 0;
    const int cluster = vocab >= 4096 ? rl::filtered_cluster_plan(vocab, n_rows, &part) : 0;
    cudaError_t e;
    if (cluster == 0)
      e = rl::launch_pdl(rl::sample_filtered_kernel, dim3(n_rows), rl::FILTER_THREADS, 0, stream, logits, ld, vocab,
                         temperature, top_k, top_p, seeds, counters, out_ids, kept);
    else
      e = rl::launch_filtered_cluster(cluster, part, logits, ld, n_rows, vocab, temperature, top_k, top_p, seeds,
                                      counters, out_ids, kept, stream);
    (void)e;  // noted by the launch itself
  }
  RL_CHECK_LAUNCH();
  return 0;
}
