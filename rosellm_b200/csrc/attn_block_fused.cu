// The attention half of a layer for a decode step of at most 16 requests in ONE kernel:
//   x += softmax(q k^T / sqrt(d)) v W_out^T + b_out,  q, k, v = LN(x) W_qkv^T + b_qkv
// (rosellm/rosetrainer/model.py:95-98, 169-185, 218-221, 372-413), the step's keys and values
// written to their cache pages on the way.  The unfused path runs three kernels for it (packed
// qkv product, attention over the pages, output product); a decode step of few requests is bound
// by the chain of dependent kernels, not by bytes, so the chain is what this kernel shortens.
//
// A cluster of C blocks owns one head.  Before the block waits for the kernels ahead of it
// (programmatic dependent launch) it starts what depends on no kernel of the step: copies of
// its slice of W_qkv (eight query, key and value columns of the head per block at head size 64)
// and of its slice of W_out (hidden/C output columns x the head's inputs) into shared memory,
// and the first tiles of its share of the cached keys and values (the cache below each request's
// newest position is of earlier steps).  After the wait:
//   1. every block normalises the rows (float32 statistics) and multiplies them by its W_qkv
//      slice on mma.sync m16n8k16; keys and values go to their pages, and all three stay in
//      shared memory for the cluster;
//   2. cluster barrier (the blocks have written their query columns into every peer's shared
//      memory); a block attends, for every request, over its eighth of the cached keys (online
//      softmax in float32, the loop of csrc/attention_kernels.cuh's decode kernel); the last block
//      of the cluster adds the newest key and value, which it takes from its peers, not the cache;
//   3. cluster barrier; every block merges the C partial results of every request (each block
//      has written its own into every peer's shared memory; the order is fixed), multiplies the
//      head's output by its slice
//      of W_out and adds the [rows, hidden/C] result into the float32 residual stream with
//      red.global.add (twelve heads add into each element, in whatever order they arrive).
// The rows that are normalised and the rows that are added to are the same memory: a block
// announces when it has read its rows and no block adds before all have (the seventeenth warp
// does the talking, as in csrc/mlp_fused.cu).  All blocks therefore run at once; the entry point
// refuses what the device does not hold in one wave.
#include <math_constants.h>

#include <mutex>
#include <unordered_map>

#include "gemm_epilogue.cuh"
#include "tc_common.cuh"

namespace rl {
namespace attf {

constexpr int WARPS = 16;
constexpr int CTHREADS = 32 * WARPS;
constexpr int THREADS = CTHREADS + 32;
constexpr int MAX_K4 = 8;       // hidden <= 1024 (a lane keeps a row's pieces while normalising)
constexpr int MAX_PAIRS = 16;   // (tile, part of K) pairs of the qkv product

__device__ unsigned int rows_taken_count = 0;
__device__ unsigned int rows_taken_generation = 0;

__device__ __forceinline__ unsigned int load_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool rows_taken_wait(unsigned int generation, int* status) {
  const long long t0 = clock64();
  while (load_acquire(&rows_taken_generation) == generation) {
    if (clock64() - t0 > 100000000LL) {
      atomicOr(status, RL_STATUS_WAIT_TIMEOUT);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr)
               : "memory");
}
__device__ __forceinline__ void ldmatrix2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void red_add2(float* addr, float a, float b) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void bar_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void compute_sync() { bar_sync(3, CTHREADS); }
__device__ __forceinline__ float ld_peer_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

__host__ __device__ inline int padded(int k) { return (k + 15) / 16 * 16 + 8; }

struct Args {
  float* x;  // [M, hidden] float32 residual stream: normalised, and added to
  long ldx;
  const float* gamma;
  const float* beta;  // may be nullptr
  float eps;
  const __nv_bfloat16* w_qkv;  // [3 * hidden, hidden]: queries, keys, values; head h owns rows h*dh.. of each
  const float* b_qkv;          // [3 * hidden] or nullptr
  const __nv_bfloat16* w_out;  // [heads][C][NO][dh + 8]: block (head, rank)'s slice of W_out as it lies in shared memory
  const float* b_out;          // [hidden] or nullptr
  __nv_bfloat16* pool;         // this layer's pages [pages][2][heads][page size][dh]
  const int* block_table;
  int bt_stride;
  const int* positions;        // [M] position of each request's new token
  const int* slots;            // [M] block-table row; -1: a padding row, nothing is read or written for it
  int M, hidden, n_heads, dh, page_size, max_pos, cluster;
  float scale;
  int* status;
};

// Shared memory of a block, in order (K = hidden, T = tiles of eight qkv columns a block owns
// (3 * dh / 8 / C), NO = output columns it owns (hidden / C rounded up to 8), M = rows):
//   bars 32 | a_s [16][lds] bf16 | wqkv_s [8 T][lds] bf16 | gb_s [2 K] f32 | wout_s [NO][dh + 8] bf16
//   | part_s [16 pairs][16][8] f32 | q_s [16][dh] f32 | kvn_s [2][16][dh] f32 | wpart_s [16 warps][dh + 2] f32
//   | call_s [C][M][dh + 4] f32 (o, m, l, 0, 0) | o_s [16][dh + 8] bf16 | bias_s [8 T + NO] f32 | dest_s [2][16] int | ring
struct Layout {
  int lds, T, NO, ldw;
  size_t a, wqkv, gb, wout, part, q, kvn, wpart, call, o, bias, dest, ring, total;
};
__host__ __device__ inline Layout layout(int hidden, int dh, int cluster, int rows, int ring_bytes) {
  Layout L;
  L.lds = padded(hidden);
  L.T = 3 * (dh / 8) / cluster;
  L.NO = ((hidden / 8 + cluster - 1) / cluster) * 8;
  L.ldw = dh + 8;
  size_t at = 32;
  L.a = at; at += (size_t)16 * L.lds * 2;
  L.wqkv = at; at += (size_t)8 * L.T * L.lds * 2;
  L.gb = at; at += (size_t)2 * hidden * 4;
  L.wout = at; at += (size_t)L.NO * L.ldw * 2;
  L.part = at; at += (size_t)MAX_PAIRS * 16 * 8 * 4;
  L.q = at; at += (size_t)16 * dh * 4;
  L.kvn = at; at += (size_t)2 * 16 * dh * 4;
  L.wpart = at; at += (size_t)WARPS * (dh + 2) * 4;
  L.call = at; at += (size_t)cluster * rows * (dh + 4) * 4;
  at = (at + 15) / 16 * 16;
  L.o = at; at += (size_t)16 * L.ldw * 2;
  L.bias = at; at += (size_t)(8 * L.T + L.NO) * 4;
  L.dest = at; at += 2 * 16 * 4;
  at = (at + 15) / 16 * 16;
  L.ring = at; at += ring_bytes;
  L.total = at;
  return L;
}

// Keys a warp's tile holds and the words of a tile half (keys; the values follow), for EPL
// elements a lane (head size 8 * EPL, bfloat16): at most 2 KB a tile.
template <int EPL>
struct Tile {
  static constexpr int WORDS = EPL / 2;                                  // 4-byte words a lane copies of a row
  static constexpr int SUB = WORDS <= 2 ? 4 : (WORDS <= 4 ? 2 : 1);      // groups of four keys
  static constexpr int KEYS = 4 * SUB;
  static constexpr int HALF_WORDS = SUB * 32 * WORDS;
  static constexpr int BYTES = 2 * HALF_WORDS * 4;
};

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
__device__ __forceinline__ float bf16_elem(const uint32_t* w, int e) {
  const uint32_t x = w[e >> 1];
  return __uint_as_float((e & 1) ? (x & 0xffff0000u) : (x << 16));
}
__device__ __forceinline__ void st_peer_f32x4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Where the key and value of a row's new token go: -1 a padding row, -2 refused (flagged).
constexpr int DEST_PADDING = -1, DEST_REFUSED = -2;

template <int EPL, int STAGES>
__global__ __launch_bounds__(THREADS) void attn_rows_fused_kernel(Args p) {
  using TL = Tile<EPL>;
  constexpr int WORDS = TL::WORDS, SUB = TL::SUB, TILE = TL::KEYS, HALF_WORDS = TL::HALF_WORDS;
  constexpr int DH = 8 * EPL;
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = p.hidden, C = p.cluster;
  const Layout L = layout(K, DH, C, p.M, WARPS * STAGES * TL::BYTES);
  const int lds = L.lds, T = L.T, ldw = L.ldw;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // [0] norm scale and shift, [1] weights
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 16);
  __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(smem + L.a);
  __nv_bfloat16* wqkv_s = reinterpret_cast<__nv_bfloat16*>(smem + L.wqkv);
  float* gb_s = reinterpret_cast<float*>(smem + L.gb);
  __nv_bfloat16* wout_s = reinterpret_cast<__nv_bfloat16*>(smem + L.wout);
  float* part_s = reinterpret_cast<float*>(smem + L.part);
  float* q_s = reinterpret_cast<float*>(smem + L.q);          // [16][DH]: the head's queries, scaled (written by all blocks of the cluster)
  float* kvn_s = reinterpret_cast<float*>(smem + L.kvn);      // [2][16][DH]: the newest keys and values (in the last block only)
  float* wpart_s = reinterpret_cast<float*>(smem + L.wpart);  // per warp: o[DH], m, l
  float* call_s = reinterpret_cast<float*>(smem + L.call);    // [C][M]: every block's o[DH], m, l of every request (each writes its own)
  __nv_bfloat16* o_s = reinterpret_cast<__nv_bfloat16*>(smem + L.o);
  float* bias_s = reinterpret_cast<float*>(smem + L.bias);    // of this block's qkv columns, then of its outputs
  int* dest_s = reinterpret_cast<int*>(smem + L.dest);        // [0][r] page, [1][r] place in it, of row r's new token
  uint32_t* ring = reinterpret_cast<uint32_t*>(smem + L.ring);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x / C;             // the head of this cluster
  const int rank = (int)cluster_rank();     // == blockIdx.x % C
  const int TQ = T / 3;                     // tiles of eight columns of each of q, k, v
  const uint32_t bar_g = tc::smem_u32(&bars[0]), bar_w = tc::smem_u32(&bars[1]);
  const int out0 = rank * L.NO;             // first output column of this block
  const int n_out = max(0, min(L.NO, K - out0));
  const int newest = C - 1;                 // the block that adds each request's newest key: its share of old keys is the shortest

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  RL_PHASE(0);
  if (tid == 0) {
    tc::mbar_init(bar_g, 1);
    tc::mbar_init(bar_w, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // ---- before the wait: the weights start travelling (a few copies: little to do for a block
  // that could only start when the kernel ahead had left its SM) ----
  if (tid == 0) {
    tc::mbar_expect_tx(bar_g, (uint32_t)(K * 4 * (p.beta != nullptr ? 2 : 1)));
    tc::mbar_expect_tx(bar_w, (uint32_t)(8 * T * K * 2 + L.NO * ldw * 2));
    bulk_copy(tc::smem_u32(gb_s), p.gamma, (uint32_t)K * 4, bar_g);
    if (p.beta != nullptr) bulk_copy(tc::smem_u32(gb_s + K), p.beta, (uint32_t)K * 4, bar_g);
    // this block's slice of W_out was laid out for it when the weights were bound: one copy
    bulk_copy(tc::smem_u32(wout_s), p.w_out + (size_t)blockIdx.x * L.NO * ldw, (uint32_t)(L.NO * ldw * 2), bar_w);
  }
  size_t qkv_row = 0;  // the row of W_qkv (and entry of its bias) behind row tid of this block's slice
  if (tid < 8 * T) {
    // tile t = tid / 8 is tile (t % TQ) of this block's q (t / TQ == 0), k or v columns
    const int t = tid >> 3, which = t / TQ, tt = t - which * TQ;
    qkv_row = (size_t)which * K + (size_t)h * DH + (size_t)(rank * TQ + tt) * 8 + (tid & 7);
    bulk_copy(tc::smem_u32(wqkv_s + (size_t)tid * lds), p.w_qkv + qkv_row * K, (uint32_t)K * 2, bar_w);
  }
  {
    const __nv_bfloat16 z = __float2bfloat16_rn(0.f);
    const int kt = lds - 8 - K;  // columns between K and the next multiple of 16: zero for the MMA
    if (kt > 0)
      for (int i = tid; i < (16 + 8 * T) * kt; i += THREADS) {
        const int r = i / kt, c = K + (i - r * kt);
        (r < 16 ? a_s + (size_t)r * lds : wqkv_s + (size_t)(r - 16) * lds)[c] = z;
      }
  }
  // What the step's description says of this warp's request (and, in the last computing warp, of
  // every row: where its new key and value go): asked for now, looked at after the wait.
  const int m_pad = p.M <= 1 ? 1 : (p.M <= 2 ? 2 : (p.M <= 4 ? 4 : (p.M <= 8 ? 8 : 16)));
  const int wpr = WARPS / m_pad;  // warps a request
  const int my_req = warp / wpr, my_sub = warp - my_req * wpr;
  int slot = -1, pos = 0, d_slot = -1, d_pos = 0;
  if (warp < WARPS && my_req < p.M) {
    slot = p.slots[my_req];
    pos = p.positions[my_req];
  }
  if (warp == WARPS - 1 && lane < p.M) {
    d_slot = p.slots[lane];
    d_pos = p.positions[lane];
  }
  RL_PHASE(1);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  RL_PHASE(2);

  if (warp == WARPS) {
    // ---- the talking warp: tells the other blocks that this one has read its rows ----
    // It takes part in the cluster's barriers like every warp, and must not hold them up: the
    // announcement is sent before the first, its answer (was this the last block?) looked at
    // after it, and the other blocks' announcements are waited for only after the second.
    unsigned int generation = 0, ticket = 0;
    if (lane == 0) generation = load_acquire(&rows_taken_generation);
    bar_sync(1, THREADS);
    if (lane == 0) {
      __threadfence();
      ticket = atomicAdd(&rows_taken_count, 1u);
    }
    cluster_sync();  // 1
    if (lane == 0 && ticket == gridDim.x - 1) {
      rows_taken_count = 0;  // everyone has arrived; nobody touches the counter before the next launch
      __threadfence();
      atomicAdd(&rows_taken_generation, 1u);
    }
    __syncwarp();
    cluster_sync();  // 2
    if (lane == 0 && !rows_taken_wait(generation, p.status)) *abort_flag = 1;
    __syncwarp();
    bar_arrive(2, THREADS);
    return;
  }

  // ---- 1. the rows, normalised (a warp a row); between its loads and their use, the loads that
  // the attention will need (slot and position of the warp's request, then its first pages) ----
  const int grp = lane >> 3, li = lane & 7;
  int beg = 0, end = 0, n_tiles = 0;
  const int* bt = p.block_table;
  uint32_t* my_ring = ring + (size_t)warp * STAGES * 2 * HALF_WORDS + lane * WORDS;
  const uint32_t ring_base = tc::smem_u32(my_ring);
  const size_t head_stride = (size_t)p.page_size * DH;
  const size_t page_stride = 2 * (size_t)p.n_heads * head_stride;
  const int pshift = (p.page_size & (p.page_size - 1)) == 0 ? 31 - __clz(p.page_size) : -1;
  auto page_index = [&](int key) { return pshift >= 0 ? key >> pshift : key / p.page_size; };
  auto page_place = [&](int key) { return pshift >= 0 ? key & (p.page_size - 1) : key % p.page_size; };
  auto first_key = [&](int i) { return beg + (my_sub + wpr * i) * TILE; };
  auto lookup = [&](int i, int (&pg)[SUB]) {  // the pages of tile i's keys (keys past the end repeat the last)
#pragma unroll
    for (int it = 0; it < SUB; ++it) pg[it] = bt[page_index(min(first_key(i) + it * 4 + grp, end - 1))];
  };
  auto copy = [&](int i, const int (&pg)[SUB]) {  // tile i of this warp into stage i % STAGES
    const uint32_t dst0 = ring_base + (uint32_t)((i % STAGES) * 2 * HALF_WORDS * 4);
#pragma unroll
    for (int it = 0; it < SUB; ++it) {
      const int key = first_key(i) + it * 4 + grp;
      int page = pg[it];
      if (page < 0) {
        if (key < end && li == 0) atomicOr(p.status, RL_STATUS_BAD_PAGE);
        page = 0;
      }
      const __nv_bfloat16* kr = p.pool + (size_t)page * page_stride + (size_t)h * head_stride +
                                (size_t)page_place(min(key, end - 1)) * DH + li * EPL;
      const uint32_t dst = dst0 + (uint32_t)(it * 32 * WORDS * 4);
      copy_words_async<WORDS>(dst, reinterpret_cast<const uint32_t*>(kr));
      copy_words_async<WORDS>(dst + HALF_WORDS * 4, reinterpret_cast<const uint32_t*>(kr + p.n_heads * head_stride));
    }
  };
  {
    const int n4 = K >> 2;
    const int row = warp;
    __nv_bfloat16* dst = a_s + (size_t)row * lds;
    float4 r[MAX_K4];
    if (row < p.M) {
      const float4* xr = reinterpret_cast<const float4*>(p.x + (size_t)row * p.ldx);
#pragma unroll
      for (int q = 0; q < MAX_K4; ++q) {
        const int d = lane + 32 * q;
        r[q] = xr[d < n4 ? d : 0];
      }
    }
    // behind the rows' loads: the biases of this block's columns, and the pages of the warp's
    // first tiles and of the rows' new tokens (slot and position were asked for before the wait)
    const float b_q = (tid < 8 * T && p.b_qkv != nullptr) ? p.b_qkv[qkv_row] : 0.f;
    const float b_o = (tid < n_out && h == 0 && p.b_out != nullptr) ? p.b_out[out0 + tid] : 0.f;
    if (slot >= 0 && pos >= 0 && pos < p.max_pos) {
      const int cached = pos;  // keys [0, pos) are in the cache; the newest one comes from this kernel
      const int chunk = ((cached + C - 1) / C + TILE - 1) / TILE * TILE;
      beg = rank * chunk;
      end = min(cached, beg + chunk);
      const int all = end > beg ? (end - beg + TILE - 1) / TILE : 0;
      n_tiles = all > my_sub ? (all - my_sub + wpr - 1) / wpr : 0;
      bt = p.block_table + (size_t)slot * p.bt_stride;
    } else {
      slot = -1;
    }
    int pg[STAGES][SUB];
#pragma unroll
    for (int s = 0; s < STAGES; ++s)
      if (s < n_tiles) lookup(s, pg[s]);
    int d_page = DEST_PADDING;
    if (d_slot >= 0) {
      if (d_pos < 0 || d_pos >= p.max_pos) {
        atomicOr(p.status, RL_STATUS_BAD_POSITION);
        d_page = DEST_REFUSED;
      } else {
        d_page = p.block_table[(size_t)d_slot * p.bt_stride + d_pos / p.page_size];
      }
    }
    float sum = 0.f;
    if (row < p.M) {
#pragma unroll
      for (int q = 0; q < MAX_K4; ++q) {
        if (lane + 32 * q >= n4) r[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        sum += (r[q].x + r[q].y) + (r[q].z + r[q].w);
      }
      sum = warp_sum(sum);  // every lane's loads have returned: the row is in registers
    }
    bar_arrive(1, THREADS);
    const bool ok = tc::mbar_wait(bar_g, 0, abort_flag, p.status);
    if (row >= p.M || !ok) {
      for (int d = lane; d < n4; d += 32) *reinterpret_cast<uint2*>(dst + 4 * d) = make_uint2(0u, 0u);
    } else {
      const float4* g4 = reinterpret_cast<const float4*>(gb_s);
      const float4* b4 = reinterpret_cast<const float4*>(gb_s + K);
      const float mean = sum / (float)K;
      float sq = 0.f;
#pragma unroll
      for (int q = 0; q < MAX_K4; ++q) {
        if (lane + 32 * q < n4) {
          const float a = r[q].x - mean, b = r[q].y - mean, c = r[q].z - mean, d = r[q].w - mean;
          sq += (a * a + b * b) + (c * c + d * d);
        }
      }
      const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)K + p.eps);
#pragma unroll
      for (int q = 0; q < MAX_K4; ++q) {
        const int d = lane + 32 * q;
        if (d < n4) {
          const float4 gm = g4[d];
          const float4 bt4 = p.beta != nullptr ? b4[d] : make_float4(0.f, 0.f, 0.f, 0.f);
          const float4 v = r[q];
          const __nv_bfloat162 lo = __floats2bfloat162_rn((v.x - mean) * rstd * gm.x + bt4.x, (v.y - mean) * rstd * gm.y + bt4.y);
          const __nv_bfloat162 hi = __floats2bfloat162_rn((v.z - mean) * rstd * gm.z + bt4.z, (v.w - mean) * rstd * gm.w + bt4.w);
          *reinterpret_cast<uint2*>(dst + 4 * d) =
              make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        }
      }
    }
    // the first tiles of old keys and values start travelling; they are used after the qkv product
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      if (s < n_tiles) copy(s, pg[s]);
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if (tid < 8 * T) bias_s[tid] = b_q;
    if (tid < L.NO) bias_s[8 * T + tid] = b_o;
    if (warp == WARPS - 1 && lane < 16) {
      if (d_slot >= 0 && d_page < 0 && d_page != DEST_REFUSED) {
        atomicOr(p.status, RL_STATUS_BAD_PAGE);
        d_page = DEST_REFUSED;
      }
      dest_s[lane] = d_page;
      dest_s[16 + lane] = d_pos % p.page_size;
    }
  }
  RL_PHASE(3);
  tc::mbar_wait(bar_w, 0, abort_flag, p.status);
  compute_sync();
  RL_PHASE(4);
  const bool dead = *abort_flag != 0;  // a wait gave up: go through the barriers, compute nothing

  // ---- the qkv product of this block's columns: [16, K] x wqkv_s^T ----
  const int g = lane >> 2, j = lane & 3;
  const int ksteps = (lds - 8) / 16;
  const int kparts = WARPS / T >= 1 ? WARPS / T : 1;  // T <= 16 tiles
  if (!dead && warp < T * kparts) {
    const int nt = warp % T, kp = warp / T;
    const int per = (ksteps + kparts - 1) / kparts;
    const int k_lo = kp * per, k_hi = min(ksteps, k_lo + per);
    float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};  // two chains of products
    const uint32_t a_addr = tc::smem_u32(a_s + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * lds + (lane >> 4) * 8);
    const uint32_t b_addr = tc::smem_u32(wqkv_s + (size_t)(nt * 8 + (lane & 7)) * lds + ((lane >> 3) & 1) * 8);
    int ks = k_lo;
#pragma unroll 2
    for (; ks + 1 < k_hi; ks += 2) {
      uint32_t af[4], bf[2], af2[4], bf2[2];
      ldmatrix4(af, a_addr + ks * 32);
      ldmatrix2(bf, b_addr + ks * 32);
      ldmatrix4(af2, a_addr + ks * 32 + 32);
      ldmatrix2(bf2, b_addr + ks * 32 + 32);
      mma_16816(c, af, bf[0], bf[1]);
      mma_16816(c2, af2, bf2[0], bf2[1]);
    }
    if (ks < k_hi) {
      uint32_t af[4], bf[2];
      ldmatrix4(af, a_addr + ks * 32);
      ldmatrix2(bf, b_addr + ks * 32);
      mma_16816(c, af, bf[0], bf[1]);
    }
    float* ps = part_s + (size_t)(kp * T + nt) * 16 * 8;
    *reinterpret_cast<float2*>(ps + g * 8 + 2 * j) = make_float2(c[0] + c2[0], c[1] + c2[1]);
    *reinterpret_cast<float2*>(ps + (g + 8) * 8 + 2 * j) = make_float2(c[2] + c2[2], c[3] + c2[3]);
  }
  compute_sync();
  RL_PHASE(5);
  {
    // One element of this block's q, k, v columns: bias, rounded to bfloat16 as the cache and the
    // unfused path keep them.  A query goes to every block of the cluster (scaled, in units of
    // log 2), keys and values to their page and to the block that adds the newest key.
    const float qs = p.scale * 1.4426950408889634f;
    const uint32_t q_base = tc::smem_u32(q_s), kvn_base = tc::smem_u32(kvn_s);
    for (int e = tid; !dead && e < p.M * T * 2; e += CTHREADS) {  // four columns an item
      const int e_row = e / (2 * T), rest = e - e_row * (2 * T);
      const int t = rest >> 1, c0 = (rest & 1) * 4;
      const int which = t / TQ, tt = t - which * TQ;
      float4 acc = *reinterpret_cast<const float4*>(bias_s + t * 8 + c0);
      for (int kp = 0; kp < kparts; ++kp) {
        const float4 v = *reinterpret_cast<const float4*>(part_s + ((size_t)(kp * T + t) * 16 + e_row) * 8 + c0);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
      const float f0 = __low2float(lo), f1 = __high2float(lo), f2 = __low2float(hi), f3 = __high2float(hi);
      const int d = (rank * TQ + tt) * 8 + c0;
      const uint32_t off = (uint32_t)((e_row * DH + d) * 4);
      if (which == 0) {
        for (int c = 0; c < C; ++c) st_peer_f32x4(peer_addr(q_base + off, c), f0 * qs, f1 * qs, f2 * qs, f3 * qs);
      } else {
        st_peer_f32x4(peer_addr(kvn_base + (uint32_t)((which - 1) * 16 * DH * 4) + off, newest), f0, f1, f2, f3);
        const int page = dest_s[e_row];
        if (page >= 0)
          *reinterpret_cast<uint2*>(p.pool + (size_t)page * page_stride + (size_t)(which - 1) * p.n_heads * head_stride +
                                    (size_t)h * head_stride + (size_t)dest_s[16 + e_row] * DH + d) =
              make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
      }
    }
  }
  RL_PHASE(6);
  cluster_sync();  // 1: the head's queries (and the newest keys and values) have arrived from every block
  RL_PHASE(7);

  // ---- 2. attention of this warp over its tiles of old keys ----
  float m = -CUDART_INF_F, l = 0.f, o[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) o[e] = 0.f;
  if (!dead && slot >= 0) {
    float qr[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) qr[e] = q_s[my_req * DH + li * EPL + e];
    int pg[SUB];
    if (STAGES < n_tiles) lookup(STAGES, pg);
    for (int i = 0; i < n_tiles; ++i) {
      asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 1) : "memory");  // tile i has arrived
      const uint32_t* kt_s = my_ring + (size_t)(i % STAGES) * 2 * HALF_WORDS;
      const int kt = first_key(i);
      float s[SUB];
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int it = 0; it < SUB; ++it) {
        uint32_t kw[WORDS];
#pragma unroll
        for (int w = 0; w < WORDS; ++w) kw[w] = kt_s[it * 32 * WORDS + w];
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc = fmaf(qr[e], bf16_elem(kw, e), acc);
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        s[it] = kt + it * 4 + grp < end ? acc : -CUDART_INF_F;
        mx = fmaxf(mx, s[it]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m, mx);  // finite: the tile's first key lies inside the range
      const float alpha = exp2f(m - m_new);
      float psum = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[e] *= alpha;
#pragma unroll
      for (int it = 0; it < SUB; ++it) {
        const float pj = exp2f(s[it] - m_new);
        psum += pj;
        uint32_t vw[WORDS];
#pragma unroll
        for (int w = 0; w < WORDS; ++w) vw[w] = kt_s[HALF_WORDS + it * 32 * WORDS + w];
#pragma unroll
        for (int e = 0; e < EPL; ++e) o[e] = fmaf(pj, bf16_elem(vw, e), o[e]);
      }
      psum += __shfl_xor_sync(0xffffffffu, psum, 8);
      psum += __shfl_xor_sync(0xffffffffu, psum, 16);
      l = l * alpha + psum;
      m = m_new;
      __syncwarp();
      const int nxt = i + STAGES;
      if (nxt < n_tiles) copy(nxt, pg);  // into the place of tile i, which has been used
      asm volatile("cp.async.commit_group;" ::: "memory");
      if (nxt + 1 < n_tiles) lookup(nxt + 1, pg);
    }
    if (rank == newest && my_sub == 0) {
      // the newest key and value of the request, which this kernel has just computed
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc = fmaf(qr[e], kvn_s[my_req * DH + li * EPL + e], acc);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      const float m_new = fmaxf(m, acc);
      const float alpha = exp2f(m - m_new), pj = exp2f(acc - m_new);
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        o[e] *= alpha;
        if (grp == 0) o[e] = fmaf(pj, kvn_s[16 * DH + my_req * DH + li * EPL + e], o[e]);  // once, not in every key group
      }
      l = l * alpha + pj;
      m = m_new;
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  RL_PHASE(8);
#pragma unroll
  for (int e = 0; e < EPL; ++e) {  // the four key groups of the warp hold partial sums of the same outputs
    o[e] += __shfl_xor_sync(0xffffffffu, o[e], 8);
    o[e] += __shfl_xor_sync(0xffffffffu, o[e], 16);
  }
  {
    float* wp = wpart_s + (size_t)warp * (DH + 2);
    if (grp == 0) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) wp[li * EPL + e] = o[e];
    }
    if (lane == 0) {
      wp[DH] = m;
      wp[DH + 1] = l;
    }
  }
  compute_sync();
  RL_PHASE(9);
  // this block's result of each request (the parts of its warps, in a fixed order) goes to every
  // block of the cluster
  if (!dead) {
    constexpr int RW = DH + 4, Q4 = RW / 4;  // a request's row: o[DH], m, l, 0, 0; in pieces of four
    const uint32_t call_base = tc::smem_u32(call_s) + (uint32_t)(rank * p.M * RW * 4);
    for (int i = tid; i < p.M * Q4; i += CTHREADS) {
      const int r = i / Q4, q4 = i - r * Q4;
      const float* wp0 = wpart_s + (size_t)(r * wpr) * (DH + 2);
      float mm = -CUDART_INF_F;
      for (int w = 0; w < wpr; ++w) mm = fmaxf(mm, wp0[w * (DH + 2) + DH]);
      float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
      for (int w = 0; w < wpr; ++w) {
        const float* wp = wp0 + w * (DH + 2);
        const float f = wp[DH] == -CUDART_INF_F ? 0.f : exp2f(wp[DH] - mm);
        if (q4 < DH / 4) {
          v0 = fmaf(wp[4 * q4], f, v0);
          v1 = fmaf(wp[4 * q4 + 1], f, v1);
          v2 = fmaf(wp[4 * q4 + 2], f, v2);
          v3 = fmaf(wp[4 * q4 + 3], f, v3);
        } else {
          v1 = fmaf(wp[DH + 1], f, v1);  // l
        }
      }
      if (q4 == DH / 4) v0 = mm;
      for (int c = 0; c < C; ++c) st_peer_f32x4(peer_addr(call_base + (uint32_t)(i * 16), c), v0, v1, v2, v3);
    }
  }
  RL_PHASE(10);
  cluster_sync();  // 2: every block's partial results have arrived
  RL_PHASE(11);

  // ---- 3. merge the cluster's parts (a warp a request, fixed order), output product, add into the residual stream ----
  {
    const int r = warp;  // sixteen warps, up to sixteen requests
    constexpr int EPW = (DH + 31) / 32;
    float val[EPW];
#pragma unroll
    for (int q = 0; q < EPW; ++q) val[q] = 0.f;
    if (!dead && r < p.M && dest_s[r] != DEST_PADDING) {
      const float* row = call_s + (size_t)r * (DH + 4);
      const size_t per_block = (size_t)p.M * (DH + 4);
      float mc = -CUDART_INF_F, lc = 0.f;
      if (lane < C) {
        mc = row[lane * per_block + DH];
        lc = row[lane * per_block + DH + 1];
      }
      const float mm = warp_max(mc);  // lane c holds block c's (m, l)
      const float f = mc == -CUDART_INF_F ? 0.f : exp2f(mc - mm);
      const float ll = warp_sum(lc * f);  // > 0: the newest key is always there
      for (int c = 0; c < C; ++c) {
        const float fc = __shfl_sync(0xffffffffu, f, c);
#pragma unroll
        for (int q = 0; q < EPW; ++q)
          if (lane + 32 * q < DH) val[q] = fmaf(row[c * per_block + lane + 32 * q], fc, val[q]);
      }
#pragma unroll
      for (int q = 0; q < EPW; ++q) val[q] = ll > 0.f ? val[q] / ll : 0.f;  // (no key at all: a refused row)
    }
#pragma unroll
    for (int q = 0; q < EPW; ++q)
      if (lane + 32 * q < DH) o_s[(size_t)r * ldw + lane + 32 * q] = __float2bfloat16_rn(val[q]);
  }
  compute_sync();
  RL_PHASE(12);
  {
    const int out_tiles = L.NO / 8;
    constexpr int K2 = DH / 16;
    constexpr int MAX_TILES = 2;  // hidden / C / 8 / 16 warps, rounded up
    float c[MAX_TILES][4];
    uint32_t af[K2][4];
    const uint32_t a_addr = tc::smem_u32(o_s + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * ldw + (lane >> 4) * 8);
    if (!dead) {
#pragma unroll
      for (int ks = 0; ks < K2; ++ks) ldmatrix4(af[ks], a_addr + ks * 32);
    }
#pragma unroll
    for (int t = 0; t < MAX_TILES; ++t) {
      const int nt = warp + t * WARPS;
      c[t][0] = c[t][1] = c[t][2] = c[t][3] = 0.f;
      if (!dead && nt < out_tiles) {
        const uint32_t b_addr = tc::smem_u32(wout_s + (size_t)(nt * 8 + (lane & 7)) * ldw + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int ks = 0; ks < K2; ++ks) {
          uint32_t bf[2];
          ldmatrix2(bf, b_addr + ks * 32);
          mma_16816(c[t], af[ks], bf[0], bf[1]);
        }
        const float b0 = bias_s[8 * T + nt * 8 + 2 * j], b1 = bias_s[8 * T + nt * 8 + 2 * j + 1];
        c[t][0] += b0; c[t][1] += b1; c[t][2] += b0; c[t][3] += b1;
      }
    }
    RL_PHASE(13);
    bar_sync(2, THREADS);  // every block of the grid has read its rows (the talking warp says so)
    RL_PHASE(14);
    if (!dead && *abort_flag == 0) {
#pragma unroll
      for (int t = 0; t < MAX_TILES; ++t) {
        const int nt = warp + t * WARPS;
        const int n = out0 + nt * 8 + 2 * j;
        if (nt < out_tiles && n < K) {  // K is a multiple of 8 and n even: the pair lies inside
          if (g < p.M) red_add2(p.x + (size_t)g * p.ldx + n, c[t][0], c[t][1]);
          if (g + 8 < p.M) red_add2(p.x + (size_t)(g + 8) * p.ldx + n, c[t][2], c[t][3]);
        }
      }
    }
  }
  RL_PHASE(15);
  // (no block touches a peer's shared memory after the second cluster barrier: each may leave)
}

constexpr size_t SMEM_LIMIT = 226 * 1024;

// Tiles a warp keeps in flight: three where shared memory has the room, else two.
template <int EPL>
static int stages_for(int hidden, int cluster, int rows) {
  return layout(hidden, 8 * EPL, cluster, rows, WARPS * 3 * Tile<EPL>::BYTES).total <= SMEM_LIMIT ? 3 : 2;
}

template <int EPL, int STAGES>
static void set_attributes() {
  static bool attr_set = false;
  if (!attr_set) {
    note_launch(cudaFuncSetAttribute(attn_rows_fused_kernel<EPL, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)SMEM_LIMIT));
    note_launch(cudaFuncSetAttribute(attn_rows_fused_kernel<EPL, STAGES>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     cudaSharedmemCarveoutMaxShared));
    attr_set = true;
  }
}

static void launch_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int n_heads, int cluster, size_t smem,
                          cudaStream_t stream) {
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3(n_heads * cluster);
  cfg->blockDim = dim3(THREADS);
  cfg->dynamicSmemBytes = smem;
  cfg->stream = stream;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 2;
}

// How many clusters of this size the device runs at once (0: the launch would not fit at all).
template <int EPL>
static int clusters_at_once(int hidden, int n_heads, int cluster) {
  // planned for sixteen rows (the most shared memory, two tiles a warp in flight): whatever
  // fits then fits with fewer rows
  const int stages = stages_for<EPL>(hidden, cluster, 16);
  const Layout L = layout(hidden, 8 * EPL, cluster, 16, WARPS * stages * Tile<EPL>::BYTES);
  if (L.total > SMEM_LIMIT) return 0;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  launch_config(&cfg, attr, n_heads, cluster, L.total, nullptr);
  int n = 0;
  cudaError_t e;
  if (stages == 3) {
    set_attributes<EPL, 3>();
    e = cudaOccupancyMaxActiveClusters(&n, attn_rows_fused_kernel<EPL, 3>, &cfg);
  } else {
    set_attributes<EPL, 2>();
    e = cudaOccupancyMaxActiveClusters(&n, attn_rows_fused_kernel<EPL, 2>, &cfg);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

// The cluster size for these sizes: the largest C <= 8 that divides the head's tiles of eight
// columns (every block then owns whole tiles of each of q, k and v), whose blocks have few enough
// tiles for sixteen warps, and of which the device runs one per head at once (the blocks wait
// for one another).  0: the kernel does not take these sizes.
static int plan_cluster(int hidden, int n_heads, int dh) {
  if (hidden != n_heads * dh || hidden % 8 != 0 || hidden > 32 * 4 * MAX_K4) return 0;
  if (dh != 16 && dh != 32 && dh != 64 && dh != 128) return 0;
  static std::mutex lock;
  static std::unordered_map<long long, int> known;
  const long long key = ((long long)hidden << 32) | ((long long)n_heads << 12) | dh;
  std::lock_guard<std::mutex> hold(lock);
  const auto it = known.find(key);
  if (it != known.end()) return it->second;
  int best = 0;
  for (int c = 8; c >= 1 && best == 0; --c) {
    if ((dh / 8) % c != 0) continue;
    if (3 * (dh / 8) / c > MAX_PAIRS) continue;                       // tiles of the qkv product a block
    if (((hidden / 8 + c - 1) / c + WARPS - 1) / WARPS > 2) continue;  // tiles of the output product a warp
    int at_once = 0;
    switch (dh) {
      case 16: at_once = clusters_at_once<2>(hidden, n_heads, c); break;
      case 32: at_once = clusters_at_once<4>(hidden, n_heads, c); break;
      case 64: at_once = clusters_at_once<8>(hidden, n_heads, c); break;
      case 128: at_once = clusters_at_once<16>(hidden, n_heads, c); break;
    }
    if (at_once >= n_heads) best = c;
  }
  known[key] = best;
  return best;
}

template <int EPL>
static int launch(const Args& p, cudaStream_t stream) {
  const int stages = stages_for<EPL>(p.hidden, p.cluster, p.M);
  const Layout L = layout(p.hidden, 8 * EPL, p.cluster, p.M, WARPS * stages * Tile<EPL>::BYTES);
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  launch_config(&cfg, attr, p.n_heads, p.cluster, L.total, stream);
  if (stages == 3) {
    set_attributes<EPL, 3>();
    note_launch(cudaLaunchKernelEx(&cfg, attn_rows_fused_kernel<EPL, 3>, p));
  } else {
    set_attributes<EPL, 2>();
    note_launch(cudaLaunchKernelEx(&cfg, attn_rows_fused_kernel<EPL, 2>, p));
  }
  return take_launch_error();
}

static bool fits(int M, int hidden, int n_heads, int dh) {
  return M >= 1 && M <= 16 && plan_cluster(hidden, n_heads, dh) > 0;
}

}  // namespace attf
}  // namespace rl

// The cluster size rl_attn_block_fused uses for these sizes (0: it does not take them); the
// output matrix has to be laid out for it (see rl_attn_block_fused).
RL_EXPORT int rl_attn_block_fused_cluster(int hidden, int n_heads, int dh) {
  return rl::attf::plan_cluster(hidden, n_heads, dh);
}

// Whether rl_attn_block_fused takes these sizes (every row a decoded request; as many key/value
// heads as heads; no window): at most 16 rows, hidden = heads * head size <= 1024, head size 16,
// 32, 64 or 128, and a grid of one cluster a head that the device holds at once.
RL_EXPORT int rl_attn_block_fused_fits(int M, int hidden, int n_heads, int dh) {
  return rl::attf::fits(M, hidden, n_heads, dh) ? 1 : 0;
}

// x [M <= 16, hidden] float32 += attention sublayer of LayerNorm(x), for M decoded requests (row r
// is the new token of request r at positions[r]; slots[r] < 0: a padding row).  The keys and
// values of the new tokens are written to their pages of `pool`; the keys below positions[r]
// must be of earlier steps.  w_out is not the matrix [hidden, hidden] but its slices as the blocks
// keep them: [heads][C][NO][dh + 8] bfloat16 with C = rl_attn_block_fused_cluster(...), NO = hidden / C
// rounded up to a multiple of 8; slice (h, c) holds W_out[c*NO : (c+1)*NO, h*dh : (h+1)*dh] (rows
// beyond hidden zero) with eight zero columns after it, so that a block fetches it with one copy.
RL_EXPORT int rl_attn_block_fused(float* x, long ldx, const float* gamma, const float* beta, float eps,
                                  const void* w_qkv, const float* b_qkv, const void* w_out, const float* b_out,
                                  void* pool, const int* block_table, int bt_stride, const int* positions,
                                  const int* slots, int M, int hidden, int n_heads, int dh, int page_size,
                                  int max_pos, float scale, int* status, cudaStream_t stream) {
  using namespace rl::attf;
  if (M <= 0) return 0;
  if (!fits(M, hidden, n_heads, dh) || status == nullptr || gamma == nullptr) return -2;
  if (ldx % 4 != 0 || ((uintptr_t)x % 16) != 0 || ((uintptr_t)w_qkv % 16) != 0 || ((uintptr_t)w_out % 16) != 0 ||
      ((uintptr_t)gamma % 16) != 0 || (beta != nullptr && ((uintptr_t)beta % 16) != 0) || ((uintptr_t)pool % 16) != 0)
    return -2;
  Args p{x, ldx, gamma, beta, eps, (const __nv_bfloat16*)w_qkv, b_qkv, (const __nv_bfloat16*)w_out, b_out,
         (__nv_bfloat16*)pool, block_table, bt_stride, positions, slots, M, hidden, n_heads, dh, page_size, max_pos,
         plan_cluster(hidden, n_heads, dh), scale, status};
  switch (dh) {
    case 16: return launch<2>(p, stream);
    case 32: return launch<4>(p, stream);
    case 64: return launch<8>(p, stream);
    case 128: return launch<16>(p, stream);
  }
  return -2;
}

RL_PHASE_READER(rl_attn_block_fused_phase_times)
