// Attention of prompt portions on tcgen05 (bfloat16, head size 64, no window): the same function
// as attn_mma_kernel (attention_mma.cuh; rosellm/rosetrainer/model.py:169-185 with the online
// softmax of rosellm/rosetrainer/paged_attention.py:80-109), with both products on the
// fifth-generation tensor cores and the scores in tensor memory.
//
// A block takes 128 consecutive queries of one request and head and walks the visible keys in
// tiles of 128, then (paired so that all blocks walk about as many tiles) 128 more queries of
// the same request and head.  Its warps have fixed roles:
//   warp 0     looks up the pages of each tile, a lane a page, and issues their TMA loads (a page
//              of one head is a contiguous [page size x 64] piece of the pool: one box a page)
//              for keys and values into a ring of three stages, and the load of the queries;
//   warp 1     allocates tensor memory (two score tiles of 128 columns, two P V tiles of 64); one
//              lane issues S = Q K^T (M=128, N=128, four steps of K=16) for the next tile as
//              soon as its keys have arrived, and P V (M=128, N=64, eight steps; V is read
//              as it lies in the cache, head dimension contiguous: the MN-major form of the B
//              operand) once the probabilities of the tile are in shared memory;
//   warps 2-17 softmax, four threads a query row (one for each quarter of a tile's keys and of
//              the output's columns; tensor memory lets a warp read only the lanes of its
//              quarter, so warps w, w + 4, w + 8 and w + 12 share rows): read the scores from
//              tensor memory, mask by
//              position, agree on the row's maximum through shared memory, update the running
//              maximum and sum in float32, write the probabilities as bfloat16 in the swizzled
//              K-major layout the second product reads, and, once the next tile's
//              probabilities are handed over, add each tile's P V (read back from tensor
//              memory) to the row's output, which they keep in registers and rescale there
//              when the maximum rose.
// Keys past the request's last visible key may hold anything (a partly filled page): their
// scores are masked by index, and their value rows are zeroed in shared memory before the
// second product, so that 0 * value stays 0.  Every wait on a barrier is bounded.
#pragma once
#include "attention_kernels.cuh"
#include "tc_common.cuh"

namespace rl {
namespace tc {

constexpr int ATT_Q = 128;       // queries per block
constexpr int ATT_KV = 128;      // keys per tile
constexpr int ATT_DH = 64;
constexpr int ATT_THREADS = 576;     // a TMA warp, an MMA warp, sixteen softmax warps
constexpr int ATT_SOFTMAX_THREADS = 512;
constexpr int ATT_Q_BYTES = ATT_Q * ATT_DH * 2;        // 16 KB
constexpr int ATT_KV_BYTES = ATT_KV * ATT_DH * 2;      // 16 KB: keys or values of a tile
constexpr int ATT_P_BYTES = ATT_Q * ATT_KV * 2;        // 32 KB: two K blocks of 64 keys
constexpr int ATT_STAGES = 3;                          // tiles of keys and values in shared memory
constexpr int ATT_SMEM = 2 * ATT_Q_BYTES + ATT_STAGES * 2 * ATT_KV_BYTES + ATT_P_BYTES + 128 + 3 * 4 * ATT_Q * 4 + 1024;

// Instruction descriptor of kind::f16, bfloat16 x bfloat16 -> float32, M = 128; b_mn: the B
// operand has its N dimension contiguous in shared memory (values as they lie in the cache).
__host__ __device__ constexpr uint32_t att_instr_desc(int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}

// Shared-memory descriptor of an MN-major tile with 128-byte swizzle: rows of 64 elements
// (one swizzle row) along N, groups of eight such rows (eight steps of K) 1024 bytes apart.
// With N = 64 there is one group across, so both strides name the step along K.
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(1024 >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Waits of this kernel give up after about 50 ms (a tile takes microseconds) and leave in the
// status word's upper half which wait it was.
__device__ __forceinline__ bool att_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                         int which) {
  const long long t0 = clock64();
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0x3fu) == 0x3fu) {
      if (*abort_flag) return false;
      if (clock64() - t0 > 100000000LL) {
        *abort_flag = 1;
        atomicOr(status, RL_STATUS_WAIT_TIMEOUT | (1 << (16 + which)));
        return false;
      }
    }
  }
}

__device__ __forceinline__ float att_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The 128 queries of a block's turn: where they start in the request's portion, how many there
// are, the position of the first, one past the last key any of them sees, and the key tiles.
struct AttQueries {
  int t0, rows, first_pos, kv_hi, n_tiles;
};

// tiles: [n][2] = (request, first query of a 64-query tile within the request's portion).  The
// entries whose first query is a multiple of 128 name 128 consecutive queries; of a request's k
// such pieces, the block of piece i < k - 1 - i takes pieces k - 1 - i and i, one after the
// other (under the causal mask the first sees the most keys and the last the fewest: together
// every block walks about the same number of key tiles, and all blocks run in one round), the
// block of the middle piece takes it alone, and the others' blocks leave at once.
// map_q: the step's queries [tokens][heads * 64]; map_kv: this layer's pool as rows of 64
// [pages * 2 * kv heads * page size][64], a box being one page of one head.
__global__ __launch_bounds__(ATT_THREADS, 1) void attn_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                 const __grid_constant__ CUtensorMap map_kv,
                                                                 AttnParams p, const int* __restrict__ tiles) {
  extern __shared__ uint8_t att_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)att_smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t q_addr = smem_u32(smem);                            // [2 turns][128 queries]
  const uint32_t kv_addr = q_addr + 2 * ATT_Q_BYTES;                 // [stage][keys 16 KB, values 16 KB]
  const uint32_t p_addr = kv_addr + ATT_STAGES * 2 * ATT_KV_BYTES;   // [2 K blocks][128 rows][128 bytes]
  const uint32_t bar_base = p_addr + ATT_P_BYTES;
  const uint32_t q_full0 = bar_base, kv_full0 = bar_base + 16, kv_empty0 = bar_base + 40, s_full0 = bar_base + 64,
                 p_ready = bar_base + 80, pv_full0 = bar_base + 88;
  uint8_t* after_p = smem + 2 * ATT_Q_BYTES + ATT_STAGES * 2 * ATT_KV_BYTES + ATT_P_BYTES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(after_p + 112);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = gridDim.x - 1 - blockIdx.x;
  const int req = tiles[2 * tile], entry_t0 = tiles[2 * tile + 1];
  if (entry_t0 % ATT_Q != 0) return;  // the second half of a piece
  const int h = blockIdx.y;
  const int hkv = h / (p.n_heads / p.n_kv_heads);
  const int qs = p.q_start[req];
  const int q_len = p.q_start[req + 1] - qs;
  const int kv_len = p.kv_len[req];
  const int slot = p.slots[req];
  const int piece = entry_t0 / ATT_Q, n_pieces = (q_len + ATT_Q - 1) / ATT_Q;
  if (piece > n_pieces - 1 - piece) return;  // taken by the block of its partner
  const int n_turns = piece < n_pieces - 1 - piece ? 2 : 1;
  auto queries_of = [&](int turn) {
    AttQueries q;
    q.t0 = (turn == 0 ? n_pieces - 1 - piece : piece) * ATT_Q;  // the longer walk first
    q.rows = min(ATT_Q, q_len - q.t0);
    q.first_pos = kv_len - q_len + q.t0;
    q.kv_hi = q.first_pos + q.rows;
    q.n_tiles = (q.kv_hi + ATT_KV - 1) / ATT_KV;
    return q;
  };
  RL_PHASE(0);

  if (threadIdx.x == 0) {
    mbar_init(q_full0, 1);
    mbar_init(q_full0 + 8, 1);
    for (int s = 0; s < ATT_STAGES; ++s) {
      mbar_init(kv_full0 + 8 * s, 1);
      mbar_init(kv_empty0 + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(s_full0 + 8 * s, 1);
      mbar_init(pv_full0 + 8 * s, 1);
    }
    mbar_init(p_ready, ATT_SOFTMAX_THREADS);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_pv = tmem_base + 256u;  // two tiles of 64 columns
  RL_PHASE(1);
  pdl_begin();
  RL_PHASE(2);

  // Key tiles are counted through both turns (g): stages, score and P V buffers and the phases
  // of their barriers go by that count.
  if (warp == 0) {
    // The whole warp brings the tiles: lane i looks up page i of a tile and issues its two
    // copies (keys, values), so that a tile of sixteen pages costs one table read and one round of
    // issues, not sixteen of each in a row; the table entry of the next tile is asked for before
    // this tile's copies go out.
    if (lane == 0) {
      for (int turn = 0; turn < n_turns; ++turn) {
        mbar_expect_tx(q_full0 + 8 * turn, ATT_Q_BYTES);
        tma_load_2d(q_addr + turn * ATT_Q_BYTES, &map_q, q_full0 + 8 * turn, h * ATT_DH, qs + queries_of(turn).t0);
      }
    }
    const int* bt = p.block_table + (size_t)slot * p.bt_stride;
    const int pages_per_tile = ATT_KV / p.page_size;
    const uint32_t page_bytes = (uint32_t)p.page_size * ATT_DH * 2;
    auto pages_of_tile = [&](int kv_hi, int t) { return min(pages_per_tile, (kv_hi - t * ATT_KV + p.page_size - 1) / p.page_size); };
    auto entry_of_tile = [&](int kv_hi, int t) { return lane < pages_of_tile(kv_hi, t) ? bt[t * pages_per_tile + lane] : 0; };
    int next_page = entry_of_tile(queries_of(0).kv_hi, 0);
    bool ok = true;
    int g = 0;
    for (int turn = 0; turn < n_turns && ok; ++turn) {
      const AttQueries q = queries_of(turn);
      for (int t = 0; t < q.n_tiles; ++t, ++g) {
        const int s = g % ATT_STAGES;
        const int n_pages = pages_of_tile(q.kv_hi, t);
        int page = next_page;
        if (t + 1 < q.n_tiles)
          next_page = entry_of_tile(q.kv_hi, t + 1);
        else if (turn + 1 < n_turns)
          next_page = entry_of_tile(queries_of(turn + 1).kv_hi, 0);
        ok = __all_sync(0xffffffffu, att_wait(kv_empty0 + 8 * s, ((g / ATT_STAGES) & 1u) ^ 1u, abort_flag, p.status, 0));
        if (!ok) break;
        if (lane == 0) mbar_expect_tx(kv_full0 + 8 * s, 2u * page_bytes * (uint32_t)n_pages);
        __syncwarp();
        if (lane < n_pages) {
          if (page < 0) {
            atomicOr(p.status, RL_STATUS_BAD_PAGE);
            page = 0;
          }
          const uint32_t k_dst = kv_addr + (uint32_t)s * 2u * ATT_KV_BYTES + (uint32_t)lane * page_bytes;
          const int row_k = ((page * 2) * p.n_kv_heads + hkv) * p.page_size;
          tma_load_2d(k_dst, &map_kv, kv_full0 + 8 * s, 0, row_k);
          tma_load_2d(k_dst + ATT_KV_BYTES, &map_kv, kv_full0 + 8 * s, 0, row_k + p.n_kv_heads * p.page_size);
        }
        if (g < 3) RL_PHASE(3 + g);
      }
    }
    if (lane == 0 && *abort_flag) {  // copies still in flight must land before the block leaves
      for (int turn = 0; turn < n_turns; ++turn) mbar_wait_quiet(q_full0 + 8 * turn, 0u);
      for (int k = max(0, g - ATT_STAGES); k < g; ++k) mbar_wait_quiet(kv_full0 + 8 * (k % ATT_STAGES), (k / ATT_STAGES) & 1u);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = att_instr_desc(ATT_KV, false);
      constexpr uint32_t idesc_o = att_instr_desc(ATT_DH, true);
      const int n_first = queries_of(0).n_tiles;
      const int n_all = n_first + (n_turns > 1 ? queries_of(1).n_tiles : 0);
      bool ok = true;
      // S = Q K^T of tile g (of the turn it falls in), once its keys (and that turn's queries) have arrived
      auto issue_s = [&](int g) {
        const int turn = g < n_first ? 0 : 1;
        if (g == 0 || g == n_first) ok = att_wait(q_full0 + 8 * turn, 0u, abort_flag, p.status, 1);
        if (ok) ok = att_wait(kv_full0 + 8 * (g % ATT_STAGES), (g / ATT_STAGES) & 1u, abort_flag, p.status, 2);
        if (!ok) return;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t k_addr = kv_addr + (uint32_t)(g % ATT_STAGES) * 2u * ATT_KV_BYTES;
        const uint32_t qa = q_addr + (uint32_t)turn * ATT_Q_BYTES;
#pragma unroll
        for (int k = 0; k < ATT_DH / 16; ++k)
          mma_f16(tmem_base + (uint32_t)(g & 1) * 128u, smem_desc(qa + k * 32), smem_desc(k_addr + k * 32), idesc_s,
                  k != 0 ? 1u : 0u);
        mma_commit(s_full0 + 8 * (g & 1));
      };
      if (n_all > 0) issue_s(0);
      RL_PHASE_OF(6, 32);
      for (int g = 0; g < n_all && ok; ++g) {
        // the scores of the next tile, while the softmax works on this one (its place was last
        // read for tile g - 1, whose probabilities have been waited for)
        if (g + 1 < n_all) {
          issue_s(g + 1);
          if (!ok) break;
        }
        ok = att_wait(p_ready, g & 1u, abort_flag, p.status, 3);
        if (!ok) break;
        if (g < 6) RL_PHASE_OF(10 + g, 32);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v_addr = kv_addr + (uint32_t)(g % ATT_STAGES) * 2u * ATT_KV_BYTES + ATT_KV_BYTES;
#pragma unroll
        for (int k = 0; k < ATT_KV / 16; ++k)  // 16 keys a step: two groups of eight value rows
          mma_f16(tmem_pv + (uint32_t)(g & 1) * 64u, smem_desc(p_addr + (uint32_t)(k >> 2) * (ATT_Q * 128) + (k & 3) * 32),
                  smem_desc_mn(v_addr + (uint32_t)k * 2048u), idesc_o, k != 0 ? 1u : 0u);
        mma_commit(kv_empty0 + 8 * (g % ATT_STAGES));
        mma_commit(pv_full0 + 8 * (g & 1));
      }
    }
  } else {
    // four threads a query row: warp w reads the tensor-memory lanes of its quarter (w % 4);
    // `part` says which 32 keys of a tile and which 16 columns of the output are this thread's
    const int quarter = warp & 3, part = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int st = threadIdx.x - 64;  // 0..511 among the softmax threads
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;  // scores in units of log 2
    float* mx_s = reinterpret_cast<float*>(after_p + 128);  // [2 tiles][4 parts][128], then the sums [4 parts][128]
    float* sum_s = mx_s + 2 * 4 * ATT_Q;
    // this thread's 32 probabilities of a tile: 64 bytes of the row in K block part / 2
    uint8_t* p_row = smem + 2 * ATT_Q_BYTES + ATT_STAGES * 2 * ATT_KV_BYTES + (size_t)(part >> 1) * (ATT_Q * 128) + (size_t)row * 128;
    const int sw = row & 7;  // swizzle of 16-byte chunks
    auto row_sync = [&]() { asm volatile("bar.sync 1, 512;" ::: "memory"); };
    float o[ATT_DH / 4];
    // adds tile g's P V (this thread's 16 columns) to the row's output, after its product has finished
    auto take_pv = [&](int g) -> bool {
      const bool arrived = __all_sync(0xffffffffu, att_wait(pv_full0 + 8 * (g & 1), (g >> 1) & 1u, abort_flag, p.status, 5));
      if (!arrived) return false;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t r[16];
      tmem_load16(tmem_pv + lane_base + (uint32_t)(g & 1) * 64u + (uint32_t)part * 16u, r);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int i = 0; i < 16; ++i) o[i] += __uint_as_float(r[i]);
      return true;
    };
    // Every softmax thread passes the row barrier once a tile and once at the end of a turn, also
    // after a wait gave up (ok false): the work is skipped then, the barrier never.
    bool ok = true;
    int g = 0;
    for (int turn = 0; turn < n_turns; ++turn) {
      const AttQueries q = queries_of(turn);
      const bool row_ok = row < q.rows;
      const int qpos = q.first_pos + row;
      float m = -CUDART_INF_F, l = 0.f;  // l: the sum over this thread's keys
#pragma unroll
      for (int d = 0; d < ATT_DH / 4; ++d) o[d] = 0.f;
      for (int t = 0; t < q.n_tiles; ++t, ++g) {
        const int kt = t * ATT_KV + part * 32;  // first key of this thread's quarter of the tile
        if (ok) ok = __all_sync(0xffffffffu, att_wait(s_full0 + 8 * (g & 1), (g >> 1) & 1u, abort_flag, p.status, 4));
        if (g < 4) RL_PHASE_OF(16 + 4 * g, 64);
        const uint32_t s_addr = tmem_base + lane_base + (uint32_t)(g & 1) * 128u + (uint32_t)part * 32u;
        // keys of this quarter the query sees: [0, n_vis); the whole warp sees all of them in
        // every tile but the last ones
        const int n_vis = row_ok ? max(0, min(32, qpos - kt + 1)) : 0;
        const bool all_vis = __all_sync(0xffffffffu, n_vis == 32);
        float mx = -CUDART_INF_F;
        uint32_t r[32];  // the scores stay in registers between the maximum and the exponentials
        if (ok) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          tmem_load32(s_addr, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (all_vis) {
            // four chains of eight instead of one of thirty-two: each fmax waits for the one before it
            float m4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(r[i]));
            mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < n_vis) mx = fmaxf(mx, __uint_as_float(r[i]));
          }
        }
        // the row's maximum over the four quarters
        float* mx_t = mx_s + (g & 1) * 4 * ATT_Q + row;
        mx_t[part * ATT_Q] = mx;
        row_sync();
        mx = fmaxf(fmaxf(mx_t[0], mx_t[ATT_Q]), fmaxf(mx_t[2 * ATT_Q], mx_t[3 * ATT_Q]));
        if (g < 4) RL_PHASE_OF(17 + 4 * g, 64);
        const float m_new = fmaxf(m, mx * sl2);
        const float alpha = m_new == -CUDART_INF_F ? 1.f : att_ex2(m - m_new);
        const float neg_m = m_new == -CUDART_INF_F ? 0.f : -m_new;
        if (!ok) continue;
        // probabilities of this thread's 32 keys, as bfloat16, into the operand of the second product
        float sum = 0.f;
        uint32_t packed[16];
        if (all_vis) {
          float s4[4] = {0.f, 0.f, 0.f, 0.f};  // four chains of additions, as for the maximum
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = att_ex2(fmaf(__uint_as_float(r[2 * i]), sl2, neg_m));
            const float p1 = att_ex2(fmaf(__uint_as_float(r[2 * i + 1]), sl2, neg_m));
            s4[i & 3] += p0 + p1;
            const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
            packed[i] = *reinterpret_cast<const uint32_t*>(&hh);
          }
          sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = 2 * i < n_vis ? att_ex2(fmaf(__uint_as_float(r[2 * i]), sl2, neg_m)) : 0.f;
            const float p1 = 2 * i + 1 < n_vis ? att_ex2(fmaf(__uint_as_float(r[2 * i + 1]), sl2, neg_m)) : 0.f;
            sum += p0 + p1;
            const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
            packed[i] = *reinterpret_cast<const uint32_t*>(&hh);
          }
        }
        // 32 keys = 64 bytes = four 16-byte chunks of the row: the first or the second half of it
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int chunk = (part & 1) * 4 + c;
          *reinterpret_cast<uint4*>(p_row + ((chunk ^ sw) << 4)) =
              make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
        }
        l = l * alpha + sum;
        m = m_new;
        // value rows of keys no query of the turn sees: zero, so that 0 * value stays 0
        if (t * ATT_KV + ATT_KV > q.kv_hi) {
          // the values of this tile have arrived: the scores could not be there otherwise, and
          // keys and values come under one barrier
          uint8_t* v_s = smem + 2 * ATT_Q_BYTES + (size_t)(g % ATT_STAGES) * 2 * ATT_KV_BYTES + ATT_KV_BYTES;
          const int first_bad = q.kv_hi - t * ATT_KV;
          for (int i = st + first_bad * 8; i < ATT_KV * 8; i += ATT_SOFTMAX_THREADS)
            *reinterpret_cast<uint4*>(v_s + (size_t)i * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(p_ready) : "memory");
        if (g < 4) RL_PHASE_OF(18 + 4 * g, 64);
        // Only now the P V of the tile before (whose product ran while this tile's exponentials
        // were taken: the second product waits for the probabilities, never the probabilities
        // for the second product): add it, then bring the output to the new maximum.
        if (t > 0) {
          ok = take_pv(g - 1);
          if (ok && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
            for (int d = 0; d < ATT_DH / 4; ++d) o[d] *= alpha;
          }
        }
        if (g < 4) RL_PHASE_OF(19 + 4 * g, 64);
      }
      if (ok && q.n_tiles > 0) ok = take_pv(g - 1);
      if (turn == 0) RL_PHASE_OF(7, 64);
      // the row's sum over the four quarters (every softmax thread comes here, also after a wait gave up)
      sum_s[part * ATT_Q + row] = l;
      row_sync();
      l = (sum_s[row] + sum_s[ATT_Q + row]) + (sum_s[2 * ATT_Q + row] + sum_s[3 * ATT_Q + row]);
      if (ok && row_ok) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        __nv_bfloat16* out = (__nv_bfloat16*)p.out + (size_t)(qs + q.t0 + row) * p.out_stride + h * ATT_DH + part * 16;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 hh = __floats2bfloat162_rn(o[8 * i + 2 * e] * inv, o[8 * i + 2 * e + 1] * inv);
            w[e] = *reinterpret_cast<const uint32_t*>(&hh);
          }
          *reinterpret_cast<uint4*>(out + i * 8) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  RL_PHASE(8);
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// Whether the tcgen05 kernel takes these sizes.
static inline bool attn_tc_fits(const AttnParams& p) {
  return p.head_dim == ATT_DH && p.window <= 0 && p.page_size >= 8 && p.page_size <= ATT_KV &&
         ATT_KV % p.page_size == 0 && (p.page_size & 7) == 0 && p.out_stride % 8 == 0 &&
         ((uintptr_t)p.out % 16) == 0;
}

// n_tokens: rows of the query matrix; n_pages: pages of this layer's pool.  Returns 0, or a
// negative code when a tensor map could not be made (the caller then takes the other kernel).
static inline int launch_attn_tc(const AttnParams& p, const int* tiles, int n_tiles, int n_tokens, long n_pages,
                                 cudaStream_t stream) {
  CUtensorMap mq, mkv;
  int rc = tensor_map(p.q, n_tokens, (long)p.n_heads * ATT_DH, p.q_stride, ATT_Q, &mq);
  if (rc != 0) return rc;
  rc = tensor_map(p.pool, n_pages * 2 * p.n_kv_heads * p.page_size, ATT_DH, ATT_DH, p.page_size, &mkv);
  if (rc != 0) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM);
    attr_set = true;
  }
  launch_pdl_split(false, attn_tc_kernel, dim3(n_tiles, p.n_heads), ATT_THREADS, ATT_SMEM, stream, mq, mkv, p, tiles);
  return 0;
}

}  // namespace tc
}  // namespace rl
