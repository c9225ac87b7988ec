// Kernels of the attention over the paged cache, and the write of new keys and values into it.
//
// Every step first writes the step's keys and values into their pages, then attends over
// the cache: a query at absolute position p of a request sees the keys at positions j <= p
// (and j > p - window when the layer has a window) of the same request, scores are
// q.k * scale, softmax over the visible keys, output = sum of probabilities * values
// (rosellm/rosetrainer/model.py:169-185).  The softmax is computed online in float32 over
// tiles of keys, as rosellm/rosetrainer/paged_attention.py:80-109 does over pages:
//   m' = max(m, max s);  l = l e^{m-m'} + sum e^{s-m'};  o = o e^{m-m'} + sum e^{s-m'} v.
//
// Two kernels share these formulas.  `attn_tile_kernel` serves portions of prompts: a block
// takes 16 consecutive queries of one request and head and walks the keys in tiles held in
// shared memory.  `attn_decode_kernel` serves single decoded tokens: the keys of one request
// and head are split over several blocks (and the warps of each), whose partial (m, l, o)
// are merged by `attn_combine_kernel`; the reference's decode kernel has one program per
// (sequence, head) and no split (paged_attention.py:129-250).
//
// Cache layout of one layer: [pages][2: key, value][kv heads][page size][head dim].
#pragma once
#include <math_constants.h>

#include "common.cuh"
#include "gemm_vec.cuh"

namespace rl {

struct AttnParams {
  const void* q;      // query of token n, head h: q + n*q_stride + h*head_dim
  long q_stride;      // in elements
  const void* pool;   // this layer's pages
  const int* block_table;
  int bt_stride;      // entries per block-table row
  const int* q_start; // [requests+1] first token of each request in the step
  const int* kv_len;  // [requests] keys the request has after this step's write
  const int* slots;   // [requests] block-table row
  void* out;          // out + n*out_stride + h*head_dim
  long out_stride;
  int n_heads, n_kv_heads, head_dim, page_size, window;  // window 0: all keys
  float scale;
  int* status;
  // Nonzero: the keys and values at positions below kv_len - 1 of the decoded requests, and the
  // block table, were written by work that had completed before the kernel that precedes this
  // one on the stream started (they are of earlier steps, with a copy to the device in
  // between).  The decode kernel then fetches them before it waits for the kernels ahead.
  // Zero: it reads nothing before that wait.
  int old_keys_settled;
};

template <typename T>
__device__ __forceinline__ const T* kv_row(const AttnParams& p, int page, int which, int hkv,
                                           int pos) {
  return (const T*)p.pool +
         ((((size_t)page * 2 + which) * p.n_kv_heads + hkv) * p.page_size + (pos % p.page_size)) *
             p.head_dim;
}

constexpr int TILE_Q = 16;    // queries per block
constexpr int TILE_KV = 32;   // keys per tile: one per lane
constexpr int ROWS_PER_WARP = 4;

template <typename T, int NCHUNK>
__global__ __launch_bounds__(128) void attn_tile_kernel(AttnParams p, const int* __restrict__ tiles) {
  extern __shared__ __align__(16) float smem[];
  pdl_begin();
  const int dh = p.head_dim;
  float* q_s = smem;                       // [TILE_Q][dh], scaled
  float* v_s = q_s + TILE_Q * dh;          // [TILE_KV][dh]
  float* k_s = v_s + TILE_KV * dh;         // [TILE_KV][dh+1]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int req = tiles[2 * blockIdx.x], t0 = tiles[2 * blockIdx.x + 1];
  const int h = blockIdx.y;
  const int hkv = h / (p.n_heads / p.n_kv_heads);
  const int qs = p.q_start[req];
  const int q_len = p.q_start[req + 1] - qs;
  const int kv_len = p.kv_len[req];
  const int pos0 = kv_len - q_len;  // absolute position of the portion's first token
  const int rows = min(TILE_Q, q_len - t0);
  const int* bt = p.block_table + (size_t)p.slots[req] * p.bt_stride;
  const T* q = (const T*)p.q;

  for (int i = tid; i < TILE_Q * dh; i += blockDim.x) {
    const int r = i / dh, d = i - r * dh;
    q_s[i] = r < rows ? to_f32(q[(size_t)(qs + t0 + r) * p.q_stride + h * dh + d]) * p.scale : 0.f;
  }
  const int first_pos = pos0 + t0;
  const int kv_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int kv_hi = first_pos + rows;  // one past the last key any query of the tile sees

  float m[ROWS_PER_WARP], l[ROWS_PER_WARP], o[ROWS_PER_WARP][NCHUNK];
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r) {
    m[r] = -CUDART_INF_F;
    l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) o[r][c] = 0.f;
  }
  const int dh4 = dh >> 2;
  for (int kt = kv_lo / TILE_KV * TILE_KV; kt < kv_hi; kt += TILE_KV) {
    __syncthreads();  // the previous tile has been used (first pass: q_s is written)
    for (int i = tid; i < TILE_KV * dh4; i += blockDim.x) {
      const int j = i / dh4, d = (i - j * dh4) * 4;
      const int key = kt + j;
      float kk[4] = {0.f, 0.f, 0.f, 0.f}, vv[4] = {0.f, 0.f, 0.f, 0.f};
      if (key >= kv_lo && key < kv_hi) {
        const int page = bt[key / p.page_size];
        if (page < 0) {
          atomicOr(p.status, RL_STATUS_BAD_PAGE);
        } else {
          load4(kv_row<T>(p, page, 0, hkv, key) + d, kk);
          load4(kv_row<T>(p, page, 1, hkv, key) + d, vv);
        }
      }
      float* kd = k_s + j * (dh + 1) + d;
      kd[0] = kk[0]; kd[1] = kk[1]; kd[2] = kk[2]; kd[3] = kk[3];
      *reinterpret_cast<float4*>(v_s + j * dh + d) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    }
    __syncthreads();
    float s[ROWS_PER_WARP];
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r) s[r] = 0.f;
    const float* kr = k_s + lane * (dh + 1);
    const float* qr = q_s + warp * ROWS_PER_WARP * dh;
    for (int d = 0; d < dh; ++d) {
      const float kd = kr[d];
#pragma unroll
      for (int r = 0; r < ROWS_PER_WARP; ++r) s[r] = fmaf(qr[r * dh + d], kd, s[r]);
    }
    const int key = kt + lane;
    float pr[ROWS_PER_WARP];
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r) {
      const int row = warp * ROWS_PER_WARP + r;
      const int qpos = first_pos + row;
      const bool valid = row < rows && key >= kv_lo && key <= qpos &&
                         (p.window <= 0 || key > qpos - p.window);
      const float sv = valid ? s[r] : -CUDART_INF_F;
      const float m_new = fmaxf(m[r], warp_max(sv));
      const float alpha = m_new == -CUDART_INF_F ? 1.f : expf(m[r] - m_new);
      pr[r] = valid ? expf(sv - m_new) : 0.f;
      l[r] = l[r] * alpha + warp_sum(pr[r]);
#pragma unroll
      for (int c = 0; c < NCHUNK; ++c) o[r][c] *= alpha;
      m[r] = m_new;
    }
    const int cnt = min(TILE_KV, kv_hi - kt);
    for (int j = 0; j < cnt; ++j) {
      float pj[ROWS_PER_WARP];
#pragma unroll
      for (int r = 0; r < ROWS_PER_WARP; ++r) pj[r] = __shfl_sync(0xffffffffu, pr[r], j);
#pragma unroll
      for (int c = 0; c < NCHUNK; ++c) {
        const int d = lane + 32 * c;
        const float vv = d < dh ? v_s[j * dh + d] : 0.f;
#pragma unroll
        for (int r = 0; r < ROWS_PER_WARP; ++r) o[r][c] = fmaf(pj[r], vv, o[r][c]);
      }
    }
  }
  T* out = (T*)p.out;
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r) {
    const int row = warp * ROWS_PER_WARP + r;
    if (row >= rows) continue;
    const float inv = 1.0f / l[r];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int d = lane + 32 * c;
      if (d < dh) out[(size_t)(qs + t0 + row) * p.out_stride + h * dh + d] = from_f32<T>(o[r][c] * inv);
    }
  }
}

// Words of 4 bytes, loaded with the widest vector the count allows.
template <int W>
__device__ __forceinline__ void load_words(const uint32_t* __restrict__ p, uint32_t (&r)[W]) {
  if constexpr (W % 4 == 0) {
#pragma unroll
    for (int i = 0; i < W / 4; ++i) {
      const uint4 v = reinterpret_cast<const uint4*>(p)[i];
      r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
    }
  } else if constexpr (W % 2 == 0) {
#pragma unroll
    for (int i = 0; i < W / 2; ++i) {
      const uint2 v = reinterpret_cast<const uint2*>(p)[i];
      r[2 * i] = v.x; r[2 * i + 1] = v.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < W; ++i) r[i] = p[i];
  }
}

// Element e of a run of packed words, as float32.
template <typename T> __device__ __forceinline__ float word_elem(const uint32_t* w, int e);
template <> __device__ __forceinline__ float word_elem<float>(const uint32_t* w, int e) {
  return __uint_as_float(w[e]);
}
template <> __device__ __forceinline__ float word_elem<__nv_bfloat16>(const uint32_t* w, int e) {
  const uint32_t x = w[e >> 1];
  return __uint_as_float((e & 1) ? (x & 0xffff0000u) : (x << 16));
}

// Copies W 4-byte words from global to shared memory without passing through registers.
template <int W>
__device__ __forceinline__ void copy_words_async(uint32_t dst, const uint32_t* __restrict__ src) {
  if constexpr (W % 4 == 0) {
#pragma unroll
    for (int i = 0; i < W / 4; ++i)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16 * i), "l"(src + 4 * i) : "memory");
  } else if constexpr (W % 2 == 0) {
#pragma unroll
    for (int i = 0; i < W / 2; ++i)
      asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + 8 * i), "l"(src + 2 * i) : "memory");
  } else {
#pragma unroll
    for (int i = 0; i < W; ++i)
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4 * i), "l"(src + i) : "memory");
  }
}

// The decode attention: grid (decoded requests, heads, splits), four warps that take the tiles
// of the split's keys in turn.  part_o: [request][head][split][head_dim] float32; part_ml:
// [request][head][split][2] = (m, l).  With one split the result goes straight to out.
//
// Eight lanes share a key: lane i of the group holds elements [i*EPL, (i+1)*EPL) of the query
// and copies the same slice of the key and value rows, so a row is read in one contiguous run;
// a warp covers four keys at a time and SUB such groups of four form a tile.  A tile travels by
// cp.async into a ring of DECODE_STAGES tiles of the warp in shared memory (each lane reads
// back only what it copied itself, so no barrier is needed) while the tile before it is used.
// What is in flight is thus bounded by shared memory, not by registers: with 64 registers a
// thread and 4 KB a tile an SM holds six blocks, 24 warps (staging the tiles in registers
// allowed 16 and measured 0.55 of the memory bandwidth at batch 64, against 0.70 now and 0.92
// at batch 256).
//
// Two forms, both with a ring of two tiles a warp: four warps (many requests: the blocks fill
// the SMs and each warp streams) and sixteen warps (few requests: one block takes 256 keys a
// round, so that a request's keys need no split over blocks and no merge kernel).  A ring of
// one tile (STAGES == 1) measured slower at batch 4-8; the longest float32 rows use it.
template <int WORDS, int WARPS, int STAGES>
struct DecodeTile {
  static constexpr int SUB = WORDS <= 4 ? 4 : (WORDS <= 8 ? 2 : 1);  // at most 64 bytes a lane for the keys
  static constexpr int KEYS = 4 * SUB;
  static constexpr int HALF_WORDS = SUB * 32 * WORDS;  // the keys of a tile; the values follow
  static constexpr size_t SMEM = (size_t)WARPS * STAGES * 2 * HALF_WORDS * 4;
};

// DENSE: the same kernel as functions of their own that ask for more of an SM's memory as shared
// memory (launch_decode_form): 80 % (DENSE 1: five four-warp blocks of 33 KB an SM instead of
// three) or all of it (DENSE 2: six), each block somewhat slower the less L1 is left, for grids
// that would otherwise need a second, partly empty round.
template <typename T, int EPL, int WARPS, int STAGES, int DENSE = 0>
__global__ __launch_bounds__(32 * WARPS) void attn_decode_kernel(
    AttnParams p, const int* __restrict__ decode_reqs, int n_splits, float* __restrict__ part_o,
    float* __restrict__ part_ml) {
  constexpr int WORDS = EPL * (int)sizeof(T) / 4;      // 4-byte words per lane per row
  using Tile = DecodeTile<WORDS, WARPS, STAGES>;
  constexpr int SUB = Tile::SUB, TILE = Tile::KEYS, HALF_WORDS = Tile::HALF_WORDS;
  constexpr int AHEAD = STAGES > 1 ? STAGES - 1 : 1;  // tiles whose copies are issued before the first is used
  // bfloat16: scores in units of log 2 (the factor rides on the query's scale), so that the
  // exponentials are single ex2 instructions; float32 keeps the library's expf
  constexpr bool BASE2 = sizeof(T) == 2;
  auto ex = [](float x) { return BASE2 ? exp2f(x) : expf(x); };
  extern __shared__ __align__(16) uint32_t ring[];      // [warps][STAGES][2][SUB][32 lanes][WORDS]
  __shared__ float ml_s[WARPS][2];
  // The batch's description (written by the host before the step) and the keys and values of
  // earlier steps do not depend on the kernels ahead: they are fetched before the wait for
  // those.  What the kernel ahead does write is read after it: the query, and the key and
  // value at the request's last position.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!p.old_keys_settled) asm volatile("griddepcontrol.wait;" ::: "memory");  // the caller promises nothing
  const int dh = p.head_dim;  // == 8 * EPL
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grp = lane >> 3, li = lane & 7;
  const int di = blockIdx.x, h = blockIdx.y, sp = blockIdx.z;
  const int hkv = h / (p.n_heads / p.n_kv_heads);
  const int req = decode_reqs[di];
  const int n = p.q_start[req];
  const int slot = p.slots[req];
  if (slot < 0) {
    // padding of a fixed-size batch: no cache behind it; its output row is zero
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (sp == 0)
      for (int d = tid; d < dh; d += blockDim.x) ((T*)p.out)[(size_t)n * p.out_stride + h * dh + d] = from_f32<T>(0.f);
    return;
  }
  const int kv_len = p.kv_len[req];
  const int kv_lo = p.window > 0 ? max(0, kv_len - p.window) : 0;
  const int total = kv_len - kv_lo;
  const int chunk = ((total + n_splits - 1) / n_splits + 31) / 32 * 32;
  const int beg = kv_lo + sp * chunk;
  const int end = min(kv_len, beg + chunk);
  const int all_tiles = end > beg ? (end - beg + TILE - 1) / TILE : 0;
  // this warp's tiles: warp, warp + 4, ...; its i-th tile starts at key beg + (warp + 4 i) * TILE
  const int n_tiles = all_tiles > warp ? (all_tiles - warp + WARPS - 1) / WARPS : 0;
  const int* bt = p.block_table + (size_t)slot * p.bt_stride;
  const size_t head_stride = (size_t)p.page_size * dh;             // elements between kv heads
  const size_t page_stride = 2 * (size_t)p.n_kv_heads * head_stride;
  // page and place of a key: shifts when the page size is a power of two
  const int pshift = (p.page_size & (p.page_size - 1)) == 0 ? 31 - __clz(p.page_size) : -1;
  auto page_index = [&](int key) { return pshift >= 0 ? key >> pshift : key / p.page_size; };
  auto page_place = [&](int key) { return pshift >= 0 ? key & (p.page_size - 1) : key % p.page_size; };
  uint32_t* my_ring = ring + (size_t)warp * STAGES * 2 * HALF_WORDS + lane * WORDS;
  const uint32_t ring_base = (uint32_t)__cvta_generic_to_shared(my_ring);

  // A key past the end of the range is replaced by the range's last key (always present), so
  // that every copy is unconditional; its score is masked when the tile is used.  A missing
  // page is flagged and replaced by page 0.
  auto first_key = [&](int i) { return beg + (warp + WARPS * i) * TILE; };
  auto lookup = [&](int i, int (&pg)[SUB]) {
#pragma unroll
    for (int it = 0; it < SUB; ++it) pg[it] = bt[page_index(min(first_key(i) + it * 4 + grp, end - 1))];
  };
  auto issue = [&](int i, const int (&pg)[SUB]) {
    const uint32_t dst0 = ring_base + (uint32_t)((i % STAGES) * 2 * HALF_WORDS * 4);
#pragma unroll
    for (int it = 0; it < SUB; ++it) {
      const int key = first_key(i) + it * 4 + grp;
      const int kc = min(key, end - 1);
      int page = pg[it];
      if (page < 0) {
        if (key < end && li == 0) atomicOr(p.status, RL_STATUS_BAD_PAGE);
        page = 0;
      }
      const T* kr = (const T*)p.pool + (size_t)page * page_stride + hkv * head_stride +
                    (size_t)page_place(kc) * dh + li * EPL;
      const uint32_t dst = dst0 + (uint32_t)(it * 32 * WORDS * 4);
      copy_words_async<WORDS>(dst, reinterpret_cast<const uint32_t*>(kr));
      copy_words_async<WORDS>(dst + HALF_WORDS * 4, reinterpret_cast<const uint32_t*>(kr + p.n_kv_heads * head_stride));
    }
  };

  // the first tiles: their pages are looked up together, then their copies issued; a tile
  // that holds the request's last key waits for the kernel that writes it
  int first[AHEAD][SUB];
  if (n_tiles > 0) {
#pragma unroll
    for (int s = 0; s < AHEAD; ++s) lookup(min(s, n_tiles - 1), first[s]);
  }
  bool issued[AHEAD];
#pragma unroll
  for (int s = 0; s < AHEAD; ++s) {
    issued[s] = s < n_tiles && first_key(s) + TILE < kv_len;
    if (issued[s]) issue(s, first[s]);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  float qr[EPL];
  {
    const T* q = (const T*)p.q + (size_t)n * p.q_stride + h * dh + li * EPL;
    const float qs = BASE2 ? p.scale * 1.4426950408889634f : p.scale;
#pragma unroll
    for (int e = 0; e < EPL; ++e) qr[e] = to_f32(q[e]) * qs;
  }
  float m = -CUDART_INF_F, l = 0.f, o[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) o[e] = 0.f;

  if (n_tiles > 0) {
#pragma unroll
    for (int s = 0; s < AHEAD; ++s) {
      if (s < n_tiles && !issued[s]) issue(s, first[s]);
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    int pg[SUB];
    if (AHEAD < n_tiles) lookup(AHEAD, pg);
    for (int i = 0; i < n_tiles; ++i) {
      const int nxt = i + AHEAD;
      if constexpr (STAGES > 1) {
        if (nxt < n_tiles) issue(nxt, pg);  // into the place of tile i - 1, which has been used
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (nxt + 1 < n_tiles) lookup(nxt + 1, pg);
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 1) : "memory");  // tile i has arrived
      } else {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      const uint32_t* kt_s = my_ring + (size_t)(i % STAGES) * 2 * HALF_WORDS;
      const int kt = first_key(i);
      float s[SUB];
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int it = 0; it < SUB; ++it) {
        uint32_t kw[WORDS];
        load_words<WORDS>(kt_s + it * 32 * WORDS, kw);
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc = fmaf(qr[e], word_elem<T>(kw, e), acc);
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        s[it] = kt + it * 4 + grp < end ? acc : -CUDART_INF_F;
        mx = fmaxf(mx, s[it]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m, mx);  // finite: the tile's first key lies inside the range
      const float alpha = ex(m - m_new);
      float psum = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[e] *= alpha;
#pragma unroll
      for (int it = 0; it < SUB; ++it) {
        const float pj = ex(s[it] - m_new);  // 0 for a masked key
        psum += pj;
        uint32_t vw[WORDS];
        load_words<WORDS>(kt_s + HALF_WORDS + it * 32 * WORDS, vw);
#pragma unroll
        for (int e = 0; e < EPL; ++e) o[e] = fmaf(pj, word_elem<T>(vw, e), o[e]);
      }
      psum += __shfl_xor_sync(0xffffffffu, psum, 8);
      psum += __shfl_xor_sync(0xffffffffu, psum, 16);
      l = l * alpha + psum;
      m = m_new;
      if constexpr (STAGES == 1) {  // the one place is free again
        if (nxt < n_tiles) issue(nxt, pg);
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (nxt + 1 < n_tiles) lookup(nxt + 1, pg);
      }
    }
  }
  // the four key groups of the warp hold partial sums of the same output elements
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    o[e] += __shfl_xor_sync(0xffffffffu, o[e], 8);
    o[e] += __shfl_xor_sync(0xffffffffu, o[e], 16);
  }
  // merge the four warps: their outputs go to the start of the ring, which is free by now
  __syncthreads();
  float* o_s = reinterpret_cast<float*>(ring);  // [4][dh]: 4 dh floats <= the ring of one warp
  if (grp == 0) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) o_s[warp * dh + li * EPL + e] = o[e];
  }
  if (lane == 0) {
    ml_s[warp][0] = m;
    ml_s[warp][1] = l;
  }
  __syncthreads();
  float mm = -CUDART_INF_F;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, ml_s[w][0]);
  float f[WARPS], ll = 0.f;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) {
    f[w] = ml_s[w][0] == -CUDART_INF_F ? 0.f : ex(ml_s[w][0] - mm);
    ll += ml_s[w][1] * f[w];
  }
  const size_t base = ((size_t)di * p.n_heads + h) * n_splits + sp;
  for (int d = tid; d < dh; d += blockDim.x) {
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) acc = fmaf(o_s[w * dh + d], f[w], acc);
    if (n_splits == 1)
      ((T*)p.out)[(size_t)n * p.out_stride + h * dh + d] = from_f32<T>(acc / ll);
    else
      part_o[base * dh + d] = acc;
  }
  if (n_splits > 1 && tid == 0) {
    part_ml[2 * base] = BASE2 ? mm * 0.6931471805599453f : mm;  // the merge works in natural units
    part_ml[2 * base + 1] = ll;
  }
}

template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml, int n_splits,
                                    const int* __restrict__ decode_reqs,
                                    const int* __restrict__ q_start,
                                    const int* __restrict__ slots, T* __restrict__ out,
                                    long out_stride, int n_heads, int dh) {
  pdl_begin();
  const int di = blockIdx.x, h = blockIdx.y;
  const size_t base = ((size_t)di * n_heads + h) * n_splits;
  float mm = -CUDART_INF_F;
  for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, part_ml[2 * (base + s)]);
  float ll = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = part_ml[2 * (base + s)];
    if (ms != -CUDART_INF_F) ll += part_ml[2 * (base + s) + 1] * expf(ms - mm);
  }
  const int n = q_start[decode_reqs[di]];
  if (slots[decode_reqs[di]] < 0) return;  // padding row, zeroed by the decode kernel
  for (int d = threadIdx.x; d < dh; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = part_ml[2 * (base + s)];
      if (ms != -CUDART_INF_F) acc = fmaf(part_o[(base + s) * dh + d], expf(ms - mm), acc);
    }
    out[(size_t)n * out_stride + h * dh + d] = from_f32<T>(acc / ll);
  }
}

// One block per token: copies the token's new key and value rows of every kv head into the
// page its position falls in.
template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ k, const T* __restrict__ v, long stride,
                                T* __restrict__ pool, const int* __restrict__ block_table,
                                int bt_stride, const int* __restrict__ positions,
                                const int* __restrict__ req_of_token,
                                const int* __restrict__ slots, int n_tokens, int n_kv_heads,
                                int dh, int page_size, int max_pos, int* __restrict__ status) {
  constexpr int VEC = Vec16<T>::N;
  pdl_begin();
  const int n = blockIdx.x;
  if (n >= n_tokens) return;
  const int pos = positions[n];
  if (pos < 0 || pos >= max_pos) {
    if (threadIdx.x == 0) atomicOr(status, RL_STATUS_BAD_POSITION);
    return;
  }
  const int slot = slots[req_of_token[n]];
  if (slot < 0) return;  // padding of a fixed-size batch
  const int page = block_table[(size_t)slot * bt_stride + pos / page_size];
  if (page < 0) {
    if (threadIdx.x == 0) atomicOr(status, RL_STATUS_BAD_PAGE);
    return;
  }
  const int off = pos % page_size;
  const int per_head = dh / VEC;
  const int total = 2 * n_kv_heads * per_head;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int which = i / (n_kv_heads * per_head);
    const int rem = i - which * n_kv_heads * per_head;
    const int hk = rem / per_head, d = (rem - hk * per_head) * VEC;
    const T* src = (which == 0 ? k : v) + (size_t)n * stride + hk * dh + d;
    T* dst = pool + ((((size_t)page * 2 + which) * n_kv_heads + hk) * page_size + off) * dh + d;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
  }
}

template <typename T, int NCHUNK>
static inline void launch_tiles(const AttnParams& p, const int* tiles, int n_tiles, cudaStream_t stream) {
  const int dh = p.head_dim;
  const size_t smem = (size_t)(TILE_Q * dh + TILE_KV * dh + TILE_KV * (dh + 1)) * sizeof(float);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(attn_tile_kernel<T, NCHUNK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)smem);
  launch_pdl(attn_tile_kernel<T, NCHUNK>, dim3(n_tiles, p.n_heads), 128, smem, stream, p, tiles);
}

template <typename T, int EPL, int WARPS, int STAGES, int DENSE = 0>
static inline void launch_decode_form(const AttnParams& p, const int* decode_reqs, int n_decode, int n_splits,
                                      float* part_o, float* part_ml, cudaStream_t stream) {
  constexpr size_t smem = DecodeTile<EPL * (int)sizeof(T) / 4, WARPS, STAGES>::SMEM;
  static bool attr_set = false;
  if (!attr_set) {
    if (smem > 47 * 1024)  // the kernel has a little static shared memory too
      cudaFuncSetAttribute(attn_decode_kernel<T, EPL, WARPS, STAGES, DENSE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem);
    if (DENSE != 0)
      cudaFuncSetAttribute(attn_decode_kernel<T, EPL, WARPS, STAGES, DENSE>,
                           cudaFuncAttributePreferredSharedMemoryCarveout,
                           DENSE == 1 ? 80 : (int)cudaSharedmemCarveoutMaxShared);
    attr_set = true;
  }
  launch_pdl_split(DENSE == 0, attn_decode_kernel<T, EPL, WARPS, STAGES, DENSE>, dim3(n_decode, p.n_heads, n_splits),
                   dim3(32 * WARPS), smem, stream, p, decode_reqs, n_splits, part_o, part_ml);
}

// How many narrow (four-warp) blocks of these sizes the device holds at once with this share
// (percent) of an SM's memory as shared memory; half is the split every small kernel asks for.
template <typename T, int EPL>
static inline long narrow_blocks_at_once(int percent) {
  static int n_sms = 0, shared = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&shared, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
    if (n_sms <= 0) n_sms = 1;
  }
  const long block = (long)DecodeTile<EPL * (int)sizeof(T) / 4, 4, 2>::SMEM + 1024;
  long per_sm = ((long)shared * percent / 100) / block;
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 16) per_sm = 16;
  return (long)n_sms * per_sm;
}

// wide: sixteen warps a block instead of four.
template <typename T, int EPL>
static inline void launch_decode(const AttnParams& p, const int* decode_reqs, int n_decode, int n_splits,
                                 bool wide, float* part_o, float* part_ml, cudaStream_t stream) {
  const int dh = p.head_dim;
  if (wide) {
    // a ring of one tile where two would not fit an SM's shared memory (float32 rows of 256)
    constexpr int WIDE_STAGES = DecodeTile<EPL * (int)sizeof(T) / 4, 16, 2>::SMEM <= 200 * 1024 ? 2 : 1;
    launch_decode_form<T, EPL, 16, WIDE_STAGES>(p, decode_reqs, n_decode, n_splits, part_o, part_ml, stream);
  } else if ((long)n_decode * p.n_heads * n_splits > narrow_blocks_at_once<T, EPL>(80)) {
    launch_decode_form<T, EPL, 4, 2, 2>(p, decode_reqs, n_decode, n_splits, part_o, part_ml, stream);
  } else if ((long)n_decode * p.n_heads * n_splits > narrow_blocks_at_once<T, EPL>(50)) {
    launch_decode_form<T, EPL, 4, 2, 1>(p, decode_reqs, n_decode, n_splits, part_o, part_ml, stream);
  } else {
    launch_decode_form<T, EPL, 4, 2>(p, decode_reqs, n_decode, n_splits, part_o, part_ml, stream);
  }
  if (n_splits > 1)
    launch_pdl(attn_combine_kernel<T>, dim3(n_decode, p.n_heads), 64, 0, stream, (const float*)part_o,
               (const float*)part_ml, n_splits, decode_reqs, p.q_start, p.slots, (T*)p.out, p.out_stride,
               p.n_heads, dh);
}

template <typename T>
static inline int dispatch_attention(const AttnParams& p, const int* tiles, int n_tiles,
                                     const int* decode_reqs, int n_decode, int n_splits, bool decode_wide,
                                     float* part_o, float* part_ml, cudaStream_t stream) {
  if (p.head_dim % 16 != 0 || p.head_dim > 256) return -2;
  if (n_tiles > 0) {
    switch ((p.head_dim + 31) / 32) {
      case 1: launch_tiles<T, 1>(p, tiles, n_tiles, stream); break;
      case 2: launch_tiles<T, 2>(p, tiles, n_tiles, stream); break;
      case 3: launch_tiles<T, 3>(p, tiles, n_tiles, stream); break;
      case 4: launch_tiles<T, 4>(p, tiles, n_tiles, stream); break;
      case 5: launch_tiles<T, 5>(p, tiles, n_tiles, stream); break;
      case 6: launch_tiles<T, 6>(p, tiles, n_tiles, stream); break;
      case 7: launch_tiles<T, 7>(p, tiles, n_tiles, stream); break;
      case 8: launch_tiles<T, 8>(p, tiles, n_tiles, stream); break;
      default: return -2;
    }
  }
  if (n_decode > 0) {
#define RL_DECODE_CASE(E) \
  case E: launch_decode<T, E>(p, decode_reqs, n_decode, n_splits, decode_wide, part_o, part_ml, stream); break;
    switch (p.head_dim / 8) {
      RL_DECODE_CASE(2) RL_DECODE_CASE(4) RL_DECODE_CASE(6) RL_DECODE_CASE(8)
      RL_DECODE_CASE(10) RL_DECODE_CASE(12) RL_DECODE_CASE(14) RL_DECODE_CASE(16)
      RL_DECODE_CASE(18) RL_DECODE_CASE(20) RL_DECODE_CASE(22) RL_DECODE_CASE(24)
      RL_DECODE_CASE(26) RL_DECODE_CASE(28) RL_DECODE_CASE(30) RL_DECODE_CASE(32)
      default: return -2;
    }
#undef RL_DECODE_CASE
  }
  return 0;
}

}  // namespace rl
