// Matrix products on the fifth-generation tensor cores of sm_100a (tcgen05), bfloat16 inputs,
// float32 accumulation in tensor memory, operands brought to shared memory by TMA:
//
//   out[M,N] = A[M,K] * W[N,K]^T  (+ bias[N]) (GELU) (or out += ..., the float32 residual stream)
//
// the same products and epilogues as gemm_simt.cu (rosellm/rosetrainer/model.py:95, 220,
// 334-337; fused_mlp.py:79-113), for the many-row case (prompt portions), where arithmetic and
// not memory is the bound.  The reference leaves these products to cuBLAS through torch.
//
// One block per SM walks the output tiles of 128 rows x BN columns; BN (a multiple of 32 up to
// 256) is chosen per product so that the tiles fill their rounds over the SMs (2048 x 3072 takes
// 192 columns: 256 tiles in two rounds; 2048 x 768 takes 96: 128 tiles in one).
// Its warps have fixed roles:
//   warp 0     one lane issues the TMA loads of the W tiles (BN x 64 bfloat16, 128-byte swizzle)
//              into a ring of shared-memory stages, running ahead over tiles; those of its first
//              stages it asks for before it waits for the kernels ahead (weights are written by
//              none of them);
//   warp 18    one lane issues the loads of the A tiles (128 x 64) into the same stages: one lane
//              for both took longer over a stage than the tensor pipe does;
//   warp 1     allocates tensor memory for two accumulators; one lane issues tcgen05.mma
//              (M=128, N=BN, K=16, four per stage) and commits to the stage's "empty" barrier
//              and, after a tile's last K block, to that accumulator's "full" barrier; ring
//              position and operand descriptors are stepped along, so that issuing a product
//              takes the lane less than the 129 clocks the pipe needs for the widest one;
//   warps 2-17 wait for an accumulator and read it with tcgen05.ld (four warps per quarter of the
//              128 lanes = rows, a lane holding 32 consecutive columns of its row), apply bias and
//              activation in registers, put the 32 x 32 piece into shared memory in the layout of
//              the output's tensor map and let TMA write it: a store, or for `out += ...` an
//              addition done in memory (cp.reduce.async.bulk: one float32 rounding an element, as
//              a read-add-write would give, without a read by the SM).  Keys and values of a
//              packed qkv product go from the registers straight to their cache pages.
//              Outputs whose rows do not start on 16-byte boundaries take an epilogue of plain
//              stores through a transposing buffer instead.
// The accumulator is double-buffered in tensor memory, so the epilogue of tile i runs under the
// MMAs of tile i+1.  Every wait on a barrier is bounded: after about two seconds the kernel sets
// a status bit, raises a block-wide abort flag and leaves, freeing its tensor memory on the way
// out.  No multicast and no clusters are used.  (A one-tile-per-block form with K split over
// blocks was tried for outputs of few tiles and measured about half as fast.)
#include "gemm_epilogue.cuh"
#include "sampling_key.cuh"
#include "tc_common.cuh"

namespace rl {
namespace tc {

constexpr int PEPI_WARPS = 16;                    // epilogue warps
constexpr int A_WARP = 2 + PEPI_WARPS;            // the warp that copies the tiles of A
constexpr int PTHREADS = 32 * (3 + PEPI_WARPS);   // + the warp that copies W, the MMA warp and the one for A
constexpr int MAX_STAGES = 8;
constexpr int MAX_CLUSTER = 8;  // parts of K: the portable cluster size
constexpr int A_BYTES = BM * BK * 2;
// How a tile leaves: through a transposing buffer with plain stores (any alignment), or through
// the output's tensor map (rows on 16-byte boundaries): stores, or for `out += ...` additions
// done in memory.  (Adding from the registers with red.global.add.v4, a lane a row, was tried:
// 16-byte additions at a row's stride cost more than the buffer they save.)
// Or not at all (a head): each row's next token is chosen from the accumulators (SampleArgs).
constexpr int EPI_PLAIN = 0, EPI_TMA = 1, EPI_SAMPLE = 2;
// The epilogue's buffers: a 32 x 32 piece a warp in the output's type for TMA, or 32 x 36
// floats a warp for the transposing epilogue.
template <typename TOut, int EPI>
__host__ __device__ constexpr int staging_bytes() {
  return EPI == EPI_SAMPLE ? 0 : EPI == EPI_TMA ? PEPI_WARPS * 32 * 32 * (int)sizeof(TOut) : PEPI_WARPS * 32 * 36 * 4;
}
// full[MAX_STAGES], empty[MAX_STAGES], acc_full[2], acc_empty[2], tensor-memory address, abort flag
constexpr int BAR_BYTES = (2 * MAX_STAGES + 4) * 8 + 16;
constexpr int SMEM_BUDGET = 227 * 1024;

__device__ __noinline__ float sample_key_call(float logit, float inv_t, uint64_t seed, uint32_t counter, uint32_t index) {
  return sample_key(logit, inv_t, seed, counter, index);
}

// What a launch is told beyond the tensor maps.
struct PArgs {
  const float* bias;
  void* out;
  long ldo;
  int M, N, K, act, residual;
  int bn;         // columns of a tile
  int stages;     // depth of the ring
  int tmem_cols;  // tensor-memory columns allocated: two accumulators of tmem_cols / 2
  int splits;     // parts of K a tile is cut into: the blocks of a cluster take one each
  int kb_per;     // K blocks of 64 a part
  KvScatter kv;
  int* status;
  SampleArgs sample;  // EPI_SAMPLE only
};

__host__ __device__ inline int stage_bytes(int bn) { return A_BYTES + bn * BK * 2; }

// Shared memory: stages | staging | barriers.  CLUSTER: the blocks of a cluster take the parts of
// K of one tile (one unit a block, no walk) and add them up through distributed shared memory.
template <typename TOut, int EPI, bool CLUSTER>
__global__ __launch_bounds__(PTHREADS, 1) void gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                      const __grid_constant__ CUtensorMap map_w,
                                                                      const __grid_constant__ CUtensorMap map_out,
                                                                      const PArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int BN = p.bn, PSTAGES = p.stages;
  const int STAGE = stage_bytes(BN);
  const uint32_t smem_base = smem_u32(smem);
  const int staging_offset = PSTAGES * STAGE;
  const int bar_offset = staging_offset + staging_bytes<TOut, EPI>();
  const uint32_t bar_base = smem_base + bar_offset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (2 * MAX_STAGES + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (2 * MAX_STAGES + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + bar_offset + (2 * MAX_STAGES + 4) * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int M = p.M, N = p.N;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  const int splits = p.splits;
  const int total_units = m_tiles * n_tiles * splits;  // a unit: a tile and a part of K
  const int num_kb = (p.K + BK - 1) / BK;
  const uint32_t acc_stride = (uint32_t)p.tmem_cols / 2;
  RL_PHASE(0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), PEPI_WARPS);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tma_prefetch_map(&map_a);
    tma_prefetch_map(&map_w);
    if (EPI == EPI_TMA) tma_prefetch_map(&map_out);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  RL_PHASE(1);

  if (warp == 0) {
    if (lane == 0) {
      // before the wait for the kernels ahead: the W tiles of the first stages of the first tile
      int ahead = 0;
      if ((int)blockIdx.x < total_units) {
        const int tile = (int)blockIdx.x / splits, kb0 = ((int)blockIdx.x - tile * splits) * p.kb_per;
        const int n0 = (tile / m_tiles) * BN;
        const int kbs = min(num_kb - kb0, p.kb_per);
        ahead = kbs < PSTAGES ? kbs : PSTAGES;
        for (int s = 0; s < ahead; ++s) {
          mbar_expect_tx(full_bar(s), (uint32_t)STAGE);
          tma_load_2d(smem_base + s * STAGE + A_BYTES, &map_w, full_bar(s), (kb0 + s) * BK, n0);
        }
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      RL_PHASE(2);
      // K blocks issued so far, over all tiles, and where the next one goes: ring position, its
      // phase and its address are stepped along, never divided out (the lane's own instructions
      // are what the copies wait for)
      uint32_t it = 0, s = 0, ph = 0, a_dst = smem_base;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const int tile = unit / splits, kb0 = (unit - tile * splits) * p.kb_per;
        const int kb1 = min(num_kb, kb0 + p.kb_per);
        const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          if (it >= (uint32_t)ahead) {
            ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status);
            if (!ok) break;
            mbar_expect_tx(full_bar(s), (uint32_t)STAGE);
            tma_load_2d(a_dst + A_BYTES, &map_w, full_bar(s), kb * BK, n0);
          }
          if (it == 0) RL_PHASE(3);
          if (it + 1 == (uint32_t)num_kb) RL_PHASE(4);
          if (++s == (uint32_t)PSTAGES) {
            s = 0;
            ph ^= 1u;
            a_dst = smem_base;
          } else {
            a_dst += STAGE;
          }
        }
      }
      if (*abort_flag) {
        for (uint32_t k = it > (uint32_t)PSTAGES ? it - PSTAGES : 0; k < it; ++k)
          mbar_wait_quiet(full_bar(k % PSTAGES), (k / PSTAGES) & 1u);
      }
    }
    if constexpr (CLUSTER) {  // the cluster's two barriers are reached by every thread on every path
      __syncwarp();
      cluster_sync();
      cluster_sync();
    }
  } else if (warp == A_WARP) {
    // The tiles of A, by a lane of their own: issuing a stage's two copies, with the wait and the
    // announcement before them, took one lane longer than the tensor pipe needs for the stage.
    // Both lanes wait for the same empty slot and their copies count on the same barrier, whose
    // expected bytes (the whole stage) the other lane announces; bytes that land before the
    // announcement are counted all the same.
    if (lane == 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");  // A is what the kernel ahead wrote
      uint32_t it = 0, s = 0, ph = 0, a_dst = smem_base;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const int tile = unit / splits, kb0 = (unit - tile * splits) * p.kb_per;
        const int kb1 = min(num_kb, kb0 + p.kb_per);
        const int m0 = (tile % m_tiles) * BM;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status);  // a slot's first use: passes at once
          if (!ok) break;
          tma_load_2d(a_dst, &map_a, full_bar(s), kb * BK, m0);
          if (++s == (uint32_t)PSTAGES) {
            s = 0;
            ph ^= 1u;
            a_dst = smem_base;
          } else {
            a_dst += STAGE;
          }
        }
      }
      if (*abort_flag) {
        for (uint32_t k = it > (uint32_t)PSTAGES ? it - PSTAGES : 0; k < it; ++k)
          mbar_wait_quiet(full_bar(k % PSTAGES), (k / PSTAGES) & 1u);
      }
    }
    if constexpr (CLUSTER) {
      __syncwarp();
      cluster_sync();
      cluster_sync();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // The tensor pipe takes a 128 x 256 x 16 product every 129 clocks, and a narrower one
      // sooner: the lane must not need longer than that to issue the next.  So ring position,
      // phase and the operands' descriptors are stepped along (a descriptor's address field
      // counts 16-byte units: the next K step of 32 bytes is +2, the next stage +STAGE/16), and
      // nothing is divided or built from scratch between two products.
      const uint32_t idesc = instr_desc(BN);
      const uint64_t desc_first = smem_desc(smem_base);
      constexpr uint32_t STEP16 = 32 >> 4;
      const uint32_t stage16 = (uint32_t)STAGE >> 4, b16 = (uint32_t)A_BYTES >> 4;
      uint32_t it = 0, local = 0, s = 0, ph = 0;
      uint64_t a_desc = desc_first;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++local) {
        const int buf = local & 1;
        const int kb0 = (unit % splits) * p.kb_per, kb1 = min(num_kb, kb0 + p.kb_per);
        ok = mbar_wait(acc_empty(buf), ((local >> 1) & 1u) ^ 1u, abort_flag, p.status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_addr = tmem_base + (uint32_t)buf * acc_stride;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          ok = mbar_wait(full_bar(s), ph, abort_flag, p.status);
          if (!ok) break;
          if (it < 16) RL_PHASE_OF(10 + it, 32);
          // (no tcgen05 fence here: the copies that completed this barrier and the products that
          // read what they brought both go through the async proxy; the fence after the wait for
          // the accumulator orders the products against the epilogue's reads of tensor memory)
          const uint64_t b_desc = a_desc + b16;
          mma_f16(d_addr, a_desc, b_desc, idesc, kb > kb0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < BK / 16; ++k) mma_f16(d_addr, a_desc + k * STEP16, b_desc + k * STEP16, idesc, 1u);
          mma_commit(empty_bar(s));
          if (++s == (uint32_t)PSTAGES) {
            s = 0;
            ph ^= 1u;
            a_desc = desc_first;
          } else {
            a_desc += stage16;
          }
        }
        if (ok) mma_commit(acc_full(buf));
        if (local == 0) RL_PHASE_OF(5, 32);
      }
    }
    if constexpr (CLUSTER) {
      __syncwarp();
      cluster_sync();
      cluster_sync();
    }
  } else {
    // sixteen warps: four per lane quarter of tensor memory, each taking every fourth 32-column
    // piece of the tile.  They read and write what kernels ahead wrote: each waits for those.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;
    const KvScatter& kv = p.kv;
    uint32_t local = 0;
    bool ok = true;
    if constexpr (EPI == EPI_SAMPLE) {
      // A lane holds the sums of its row: it keeps the best of the row's columns in this tile and
      // offers it once the tile is through.  Nothing is staged and nothing written but the offers.
      const SampleArgs& sm = p.sample;
      bool offered = false;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++local) {
        const int m0 = (unit % m_tiles) * BM, n0 = (unit / m_tiles) * BN;
        const int row = m0 + quarter * 32 + lane;
        const int buf = local & 1;
        const int rc = row < M ? row : 0;
        const float temp = sm.temperature != nullptr ? sm.temperature[rc] : 0.f;
        uint64_t seed = 0;
        uint32_t counter = 0;
        if (temp > 0.f) {
          seed = (uint64_t)sm.seeds[rc];
          counter = (uint32_t)sm.counters[rc];
        }
        const float inv_t = temp > 0.f ? 1.0f / temp : 1.0f;
        const bool any_sampled = __any_sync(0xffffffffu, temp > 0.f);
        float bias0 = 0.f, bias1 = 0.f;
        if (p.bias != nullptr) {
          const int col = n0 + part * 32 + lane;
          if (col < N) bias0 = p.bias[col];
          if (part + 4 < BN / 32 && col + 128 < N) bias1 = p.bias[col + 128];
        }
        ok = mbar_wait(acc_full(buf), (local >> 1) & 1u, abort_flag, p.status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * acc_stride;
        ArgMax best{-CUDART_INF_F, 0x7fffffff};
#pragma unroll 1
        for (int c = part; c < BN / 32; c += 4) {
          if (n0 + c * 32 >= N || m0 + quarter * 32 >= M) break;  // nothing of this piece exists
          uint32_t r[32];
          tmem_load32(acc_addr + (uint32_t)(c * 32), r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          const float bias_c = c == part ? bias0 : bias1;
          const int col0 = n0 + c * 32;
          if (!any_sampled) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float v = act_fn(__uint_as_float(r[i]) + __shfl_sync(0xffffffffu, bias_c, i), p.act);
              if (col0 + i < N) best = better(best, ArgMax{v, col0 + i});
            }
          } else {
            // the noise is a call, not thirty-two inlined copies: the loop of the rows that take
            // the arg-max (above) stays short, and so does what the instruction cache must hold
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float v = act_fn(__uint_as_float(r[i]) + __shfl_sync(0xffffffffu, bias_c, i), p.act);
              const float key = sample_key_call(v, inv_t, seed, counter, (uint32_t)(col0 + i));
              if (temp > 0.f) v = key;
              if (col0 + i < N) best = better(best, ArgMax{v, col0 + i});
            }
          }
        }
        // the buffer may be overwritten by the MMAs of the tile after next
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(buf)) : "memory");
        if (row < M && best.i != 0x7fffffff) {
          const unsigned long long word =
              ((unsigned long long)ordered_bits(best.v) << 32) | (unsigned long long)(~(uint32_t)best.i);
          if (word > __ldcg(sm.best + row)) {
            atomicMax(sm.best + row, word);
            offered = true;
          }
        }
      }
      // every offer of this block is in place before its ticket is taken; the block that takes
      // the last ticket writes the token ids
      if (offered) __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(PEPI_WARPS * 32) : "memory");
      if (warp == 2) {
        int last = 0;
        if (lane == 0) last = atomicAdd(sm.ticket, 1) == (int)gridDim.x - 1;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) sample_finish(sm, M, lane);
      }
    } else if constexpr (EPI != EPI_PLAIN) {
      constexpr int PIECE_BYTES = 32 * 32 * (int)sizeof(TOut);
      uint8_t* piece = smem + staging_offset + (warp - 2) * PIECE_BYTES;
      // the tile of the unit at hand, for finish_piece below
      int m0 = 0, n0 = 0, row0 = 0, row = 0;
      long long row_base = -1;
      bool tile_to_cache = false;
      auto begin_tile = [&](int tile) {
        m0 = (tile % m_tiles) * BM;
        n0 = (tile / m_tiles) * BN;
        row0 = m0 + quarter * 32;
        row = row0 + lane;
        // where the keys and values of this lane's row go (packed qkv product): the element
        // offset of (page, keys, head 0, place in the page, 0), or -1 for a row that is not
        // written; looked up while the tile still accumulates
        row_base = -1;
        tile_to_cache = kv.pool != nullptr && n0 + BN > kv.q_width;
        if (tile_to_cache && row < M) {
          const int slot = kv.slots[kv.req_of_token[row]];
          const int pos = kv.positions[row];
          if (slot >= 0) {  // slot -1: padding of a fixed-size batch
            if (pos < 0 || pos >= kv.max_pos) {
              atomicOr(kv.status, RL_STATUS_BAD_POSITION);
            } else {
              const int page = kv.block_table[(size_t)slot * kv.bt_stride + pos / kv.page_size];
              if (page < 0)
                atomicOr(kv.status, RL_STATUS_BAD_PAGE);
              else
                row_base = ((long long)page * 2 * kv.n_kv_heads * kv.page_size + pos % kv.page_size) * kv.head_dim;
            }
          }
        }
      };
      // Piece c of the tile (32 rows x 32 columns, v = the sums of this lane's row; bias_c = the
      // bias of column `lane` of the piece): bias, activation, and out it goes.
      auto finish_piece = [&](int c, float (&v)[32], float bias_c) {
        const int col0 = n0 + c * 32;
        if (p.act == RL_ACT_GELU_TANH) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = act_fn(v[i] + __shfl_sync(0xffffffffu, bias_c, i), RL_ACT_GELU_TANH);
        } else if (p.act == RL_ACT_GELU_ERF) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = act_fn(v[i] + __shfl_sync(0xffffffffu, bias_c, i), RL_ACT_GELU_ERF);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] += __shfl_sync(0xffffffffu, bias_c, i);
        }
        // keys and values: eight columns (16 bytes, inside one head) at a time to the row's page
        if (tile_to_cache && col0 + 32 > kv.q_width && row_base >= 0) {
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            const int col = col0 + 8 * g8;
            if (col >= kv.q_width && col < N) {
              const int cidx = col - kv.q_width;
              const int which = cidx / kv.kv_width;
              const int rem = cidx - which * kv.kv_width;
              const int head = rem / kv.head_dim;
              const long long off = ((long long)(which * kv.n_kv_heads + head) * kv.page_size) * kv.head_dim +
                                    (rem - head * kv.head_dim);
              const __nv_bfloat162 b0 = __floats2bfloat162_rn(v[8 * g8], v[8 * g8 + 1]);
              const __nv_bfloat162 b1 = __floats2bfloat162_rn(v[8 * g8 + 2], v[8 * g8 + 3]);
              const __nv_bfloat162 b2 = __floats2bfloat162_rn(v[8 * g8 + 4], v[8 * g8 + 5]);
              const __nv_bfloat162 b3 = __floats2bfloat162_rn(v[8 * g8 + 6], v[8 * g8 + 7]);
              *reinterpret_cast<uint4*>((__nv_bfloat16*)kv.pool + row_base + off) =
                  make_uint4(*reinterpret_cast<const uint32_t*>(&b0), *reinterpret_cast<const uint32_t*>(&b1),
                             *reinterpret_cast<const uint32_t*>(&b2), *reinterpret_cast<const uint32_t*>(&b3));
            }
          }
        }
        if (!tile_to_cache || col0 < kv.q_width) {
          // the rest goes to `out` (whose map ends at the query width in a packed qkv product)
          // the piece this warp handed to TMA before has been read out of the buffer
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
          if constexpr (sizeof(TOut) == 4) {
            // rows of 128 bytes, 16-byte pieces swizzled by the row (128-byte swizzle)
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<float4*>(piece + lane * 128 + ((q ^ (lane & 7)) << 4)) =
                  make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          } else {
            // rows of 64 bytes, 16-byte pieces swizzled by address bits 7-8 (64-byte swizzle)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const __nv_bfloat162 b0 = __floats2bfloat162_rn(v[8 * q], v[8 * q + 1]);
              const __nv_bfloat162 b1 = __floats2bfloat162_rn(v[8 * q + 2], v[8 * q + 3]);
              const __nv_bfloat162 b2 = __floats2bfloat162_rn(v[8 * q + 4], v[8 * q + 5]);
              const __nv_bfloat162 b3 = __floats2bfloat162_rn(v[8 * q + 6], v[8 * q + 7]);
              *reinterpret_cast<uint4*>(piece + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) =
                  make_uint4(*reinterpret_cast<const uint32_t*>(&b0), *reinterpret_cast<const uint32_t*>(&b1),
                             *reinterpret_cast<const uint32_t*>(&b2), *reinterpret_cast<const uint32_t*>(&b3));
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if (sizeof(TOut) == 4 && p.residual)
              tma_add_2d(&map_out, smem_u32(piece), col0, row0);
            else
              tma_store_2d(&map_out, smem_u32(piece), col0, row0);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      };
      if constexpr (CLUSTER) {
        // One unit: this block's part of K of the cluster's tile.  The 32 x 32 pieces of the tile
        // are dealt out to the blocks of the cluster (piece c to block c % splits); after the
        // first cluster barrier (every block's products are done: the rings are free) each block
        // sends each piece of its accumulator to the piece's owner, into the owner's ring, as
        // [sender][quarter][piece of the owner][8][32 lanes][4] float32; after the second the
        // owner adds the senders' pieces in their order and finishes the piece.
        const int rank = (int)cluster_rank();
        const int owned_max = (BN / 32 + splits - 1) / splits;
        begin_tile((int)blockIdx.x / splits);
        // the bias of the piece this warp will finish (piece part * splits + rank of the tile)
        const int own_c = part * splits + rank;
        float bias_own = 0.f;
        if (p.bias != nullptr && own_c < BN / 32 && n0 + own_c * 32 + lane < N) bias_own = p.bias[n0 + own_c * 32 + lane];
        ok = mbar_wait(acc_full(0), 0u, abort_flag, p.status);
        RL_PHASE_OF(6, 64);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        cluster_sync();
        RL_PHASE_OF(26, 64);
        if (ok) {
          const uint32_t acc_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
          for (int c = part; c < BN / 32; c += 4) {
            if (n0 + c * 32 >= N || row0 >= M) break;
            uint32_t r[32];
            tmem_load32(acc_addr + (uint32_t)(c * 32), r);
            const uint32_t slot = smem_base + (uint32_t)(((rank * 4 + quarter) * owned_max + c / splits) * 4096 + lane * 16);
            const uint32_t dst = peer_addr(slot, (uint32_t)(c % splits));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int q = 0; q < 8; ++q)
              asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + q * 512), "r"(r[4 * q]),
                           "r"(r[4 * q + 1]), "r"(r[4 * q + 2]), "r"(r[4 * q + 3])
                           : "memory");
          }
        }
        RL_PHASE_OF(27, 64);
        cluster_sync();
        RL_PHASE_OF(28, 64);
        if (ok && own_c < BN / 32 && n0 + own_c * 32 < N && row0 < M) {
          float v[32];
          const uint8_t* mine = smem + (quarter * owned_max + part) * 4096 + lane * 16;
          const int sender_stride = 4 * owned_max * 4096;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 t = *reinterpret_cast<const float4*>(mine + q * 512);
            v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
          }
          for (int sp = 1; sp < splits; ++sp) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 t = *reinterpret_cast<const float4*>(mine + sp * sender_stride + q * 512);
              v[4 * q] += t.x; v[4 * q + 1] += t.y; v[4 * q + 2] += t.z; v[4 * q + 3] += t.w;
            }
          }
          finish_piece(own_c, v, bias_own);
        }
        RL_PHASE_OF(7, 64);
      } else {
        for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++local) {
          begin_tile(unit);  // no parts of K here: a unit is a tile
          const int buf = local & 1;
          // the bias of this warp's (at most two) pieces, lane i that of column i: asked for
          // now, there when the accumulator is
          float bias0 = 0.f, bias1 = 0.f;
          if (p.bias != nullptr) {
            const int col = n0 + part * 32 + lane;
            if (col < N) bias0 = p.bias[col];
            if (part + 4 < BN / 32 && col + 128 < N) bias1 = p.bias[col + 128];
          }
          ok = mbar_wait(acc_full(buf), (local >> 1) & 1u, abort_flag, p.status);
          if (!ok) break;
          if (local == 0) RL_PHASE_OF(6, 64);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t acc_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * acc_stride;
#pragma unroll 1
          for (int c = part; c < BN / 32; c += 4) {
            if (n0 + c * 32 >= N || row0 >= M) break;  // nothing of this piece exists
            uint32_t r[32];
            tmem_load32(acc_addr + (uint32_t)(c * 32), r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            finish_piece(c, v, c == part ? bias0 : bias1);
          }
          // the buffer may be overwritten by the MMAs of the tile after next
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(buf)) : "memory");
          if (local == 0) RL_PHASE_OF(7, 64);
        }
      }
      // what was handed to TMA is written before the block ends
      if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    } else {
      TOut* out = (TOut*)p.out;
      const long ldo = p.ldo;
      constexpr int PITCH = 36;
      float* stage = reinterpret_cast<float*>(smem + staging_offset) + (warp - 2) * 32 * PITCH;
      const int sub_row = lane >> 3, col4 = (lane & 7) * 4;
      for (int tile = blockIdx.x; tile < total_units && ok; tile += gridDim.x, ++local) {  // no parts of K here
        const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
        const int buf = local & 1;
        long long row_base = -1;
        const bool tile_to_cache = kv.pool != nullptr && n0 + BN > kv.q_width;
        if (tile_to_cache) {
          const int m = m0 + quarter * 32 + lane;
          if (m < M) {
            const int slot = kv.slots[kv.req_of_token[m]];
            const int pos = kv.positions[m];
            if (slot >= 0) {
              if (pos < 0 || pos >= kv.max_pos) {
                atomicOr(kv.status, RL_STATUS_BAD_POSITION);
              } else {
                const int page = kv.block_table[(size_t)slot * kv.bt_stride + pos / kv.page_size];
                if (page < 0)
                  atomicOr(kv.status, RL_STATUS_BAD_PAGE);
                else
                  row_base = ((long long)page * 2 * kv.n_kv_heads * kv.page_size + pos % kv.page_size) * kv.head_dim;
              }
            }
          }
        }
        ok = mbar_wait(acc_full(buf), (local >> 1) & 1u, abort_flag, p.status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int c = part; c < BN / 32; c += 4) {
          uint32_t r[32];
          tmem_load32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * acc_stride + (uint32_t)(c * 32), r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(stage + lane * PITCH + 4 * q) =
                make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                            __uint_as_float(r[4 * q + 3]));
          __syncwarp();
          const int col = n0 + c * 32 + col4;
          // the four columns lie in one head: head sizes and the query width are multiples of 4
          const bool to_cache = tile_to_cache && col >= kv.q_width && col < N;
          long long col_off = 0;
          if (to_cache) {
            const int cidx = col - kv.q_width;
            const int which = cidx / kv.kv_width;
            const int rem = cidx - which * kv.kv_width;
            const int head = rem / kv.head_dim;
            col_off = ((long long)(which * kv.n_kv_heads + head) * kv.page_size) * kv.head_dim + (rem - head * kv.head_dim);
          }
          const int n_valid = min(4, N - col);
          const float* bias4 = p.bias != nullptr && col < N ? p.bias + col : nullptr;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = i * 4 + sub_row;
            const int row = m0 + quarter * 32 + rr;
            long long base = -1;
            if (tile_to_cache) base = __shfl_sync(0xffffffffu, row_base, rr);  // every lane, whatever its column
            if (col < N && row < M) {
              const float4 v = *reinterpret_cast<const float4*>(stage + rr * PITCH + col4);
              if (to_cache) {
                if (base >= 0)
                  finish4<__nv_bfloat16>((__nv_bfloat16*)kv.pool + base + col_off, v, bias4, p.act, 0, false, n_valid);
              } else {
                finish4<TOut>(out + (size_t)row * ldo + col, v, bias4, p.act, p.residual, false, n_valid);
              }
            }
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(buf)) : "memory");
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  RL_PHASE(8);
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                 : "memory");
  }
}

static int sm_count() {
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    if (n_sms <= 0) n_sms = 148;
  }
  return n_sms;
}

// How a product is cut: the width of a tile and the parts of K.  A block takes about the same
// time for a K block of 64 whatever the tile's width (measured: 0.37 us from 32 to 256 columns),
// so what counts is how many K blocks fall to the busiest SM; a tile costs its epilogue, and
// parts of K the trip of the accumulators through the cluster.  Parts are taken only where all
// the clusters run at once (the product of a narrow output and a long inner size: mlp.c_proj of
// a prompt portion, whose few tiles would leave most SMs idle).  Times in nanoseconds, from
// measurements of 2048-row products.  force_bn / force_splits != 0 fix one or both (for tests
// and measurements).
struct Cut {
  int bn, splits, kb_per;
};
static int ring_stages(int bn, int staging) {
  const int room = SMEM_BUDGET - 1024 - staging - BAR_BYTES;
  const int stages = room / stage_bytes(bn);
  return stages > MAX_STAGES ? MAX_STAGES : stages;
}
// How many clusters of `size` blocks of this kernel the device holds at once (a block fills an
// SM, and a cluster's SMs lie in one GPC: fewer than SMs / size).
static int clusters_at_once(int size) {
  static int known[MAX_CLUSTER + 1] = {0};
  if (size < 1 || size > MAX_CLUSTER) return 0;
  if (known[size] == 0) {
    cudaFuncSetAttribute(gemm_tc_persistent_kernel<float, EPI_TMA, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         SMEM_BUDGET);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(size * 64);
    cfg.blockDim = dim3(PTHREADS);
    cfg.dynamicSmemBytes = SMEM_BUDGET;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_persistent_kernel<float, EPI_TMA, true>, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = -1;
    }
    known[size] = n;
  }
  return known[size] > 0 ? known[size] : 0;
}

static Cut plan_cut(int M, int N, int K, bool may_split, int staging, int force_bn, int force_splits) {
  const long m_tiles = (M + BM - 1) / BM;
  const int num_kb = (K + BK - 1) / BK;
  const int n_sms = sm_count();
  Cut best{256, 1, num_kb};
  long best_cost = -1;
  static const int kSplits[] = {1, 2, 3, 4, 6, 8};
  for (int bn = 256; bn >= 64; bn -= 32) {
    if (force_bn != 0 && bn != force_bn) continue;
    const long tiles = (long)((N + bn - 1) / bn) * m_tiles;
    for (int want : kSplits) {
      if (force_splits != 0 && want != force_splits) continue;
      const int kb_per = (num_kb + want - 1) / want;
      const int splits = (num_kb + kb_per - 1) / kb_per;  // no part is empty
      if (splits != want) continue;
      if (splits > 1) {
        // the pieces sent round the cluster lie in the receiver's ring
        const int owned_max = (bn / 32 + splits - 1) / splits;
        if (!may_split || (long)splits * 4 * owned_max * 4096 > (long)ring_stages(bn, staging) * stage_bytes(bn)) continue;
        if (clusters_at_once(splits) < 1) continue;
        if (force_splits == 0 && (tiles > clusters_at_once(splits) || splits * 2 > num_kb)) continue;
      }
      const long rounds = (tiles * splits + n_sms - 1) / n_sms;
      long cost = rounds * (300L * kb_per + 600) + 1000 + 1500L * bn / 256;
      if (splits > 1) cost += 2500;
      if (best_cost < 0 || cost < best_cost) {
        best = Cut{bn, splits, kb_per};
        best_cost = cost;
      }
    }
  }
  if (best_cost < 0) best = Cut{force_bn != 0 ? force_bn : 256, 1, num_kb};  // what was forced cannot be had
  return best;
}

template <typename TOut, int EPI, bool CLUSTER>
static int launch_persistent(const void* A, long lda, const void* W, const float* bias, void* out, long ldo, int M,
                             int N, int K, int act, int residual, const KvScatter& kv, int* status, const Cut& cut,
                             cudaStream_t stream, const SampleArgs& sample = SampleArgs{}) {
  const int bn = cut.bn;
  CUtensorMap ma, mw, mo;
  int rc = tensor_map(A, M, K, lda, BM, &ma);
  if (rc != 0) return rc;
  rc = tensor_map(W, N, K, K, bn, &mw);
  if (rc != 0) return rc;
  if (EPI == EPI_TMA) {
    // in a packed qkv product only the queries go to `out`: its map ends where they end
    rc = tensor_map(out, M, kv.pool != nullptr ? kv.q_width : N, ldo, 32, &mo, 32, (int)sizeof(TOut));
    if (rc != 0) return rc;
  } else {
    mo = ma;
  }
  static bool attr_set = false;
  if (!attr_set) {
    note_launch(cudaFuncSetAttribute(gemm_tc_persistent_kernel<TOut, EPI, CLUSTER>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET));
    attr_set = true;
  }
  constexpr int STAGING_BYTES = staging_bytes<TOut, EPI>();
  const int stages = ring_stages(bn, STAGING_BYTES);
  if (stages < 2) return -2;
  const size_t smem = 1024 + (size_t)stages * stage_bytes(bn) + STAGING_BYTES + BAR_BYTES;
  PArgs p{bias, out, ldo, M, N, K, act, residual, bn, stages, bn > 128 ? 512 : (bn > 64 ? 256 : 128),
          cut.splits, cut.kb_per, kv, status, sample};
  const int units = ((M + BM - 1) / BM) * ((N + bn - 1) / bn) * cut.splits;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(CLUSTER ? units : (units < sm_count() ? units : sm_count()));
  cfg.blockDim = dim3(PTHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = CLUSTER ? cut.splits : 1;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = CLUSTER ? 2 : 1;
  note_launch(cudaLaunchKernelEx(&cfg, gemm_tc_persistent_kernel<TOut, EPI, CLUSTER>, ma, mw, mo, p));
  return take_launch_error();
}

}  // namespace tc
}  // namespace rl

RL_PHASE_READER(rl_gemm_tc_phase_times)

// bfloat16 A [M,K] (row stride lda) and W [N,K]; out bfloat16 or float32 [M,N] (row stride ldo).
// residual != 0: out (float32) += result.  kv_pool != nullptr: output columns from kv_q_width
// on are written into cache pages as keys and values, not to out (head size and query width
// multiples of 4).  K and lda multiples of 8, operands on 16-byte boundaries.  tile_width and
// splits: 0 = chosen here, else the columns of a tile (a multiple of 32 up to 256) and the parts
// of K (1, 2, 3, 4, 6 or 8; for tests and measurements).
// Returns 0, a CUDA error, or a negative code for refused arguments.
RL_EXPORT int rl_gemm_tc_cut(int out_dtype, const void* A, long lda, const void* W, const float* bias, void* out,
                             long ldo, int M, int N, int K, int act, int residual, void* kv_pool,
                             const int* kv_block_table, int kv_bt_stride, const int* kv_positions,
                             const int* kv_req_of_token, const int* kv_slots, int kv_q_width, int kv_width,
                             int kv_head_dim, int kv_page_size, int kv_heads, int kv_max_pos, int* status,
                             int tile_width, int splits, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0 || lda % 8 != 0 || ((uintptr_t)A % 16) != 0 || ((uintptr_t)W % 16) != 0) return -2;
  if (residual && out_dtype != RL_F32) return -3;
  if (out_dtype != RL_F32 && out_dtype != RL_BF16) return -4;
  if (kv_pool != nullptr && (kv_head_dim % 4 != 0 || kv_q_width % 4 != 0 || kv_width % 4 != 0 || act != 0 || residual))
    return -8;
  if (tile_width != 0 && (tile_width % 32 != 0 || tile_width < 32 || tile_width > 256)) return -2;
  if (splits < 0 || splits > 8 || status == nullptr) return -2;
  const rl::KvScatter kv{kv_pool, kv_block_table, kv_bt_stride, kv_positions, kv_req_of_token, kv_slots,
                         kv_q_width, kv_width, kv_head_dim, kv_page_size, kv_heads, kv_max_pos, status};
  // the output goes through a tensor map where its rows start on 16-byte boundaries (and keys
  // and values in pieces of eight columns where heads and the query width are multiples of 8)
  const long out_row_bytes = ldo * (out_dtype == RL_F32 ? 4 : 2);
  const bool tma_out = out_row_bytes % 16 == 0 && ((uintptr_t)out % 16) == 0 &&
                       (kv_pool == nullptr || (kv_head_dim % 8 == 0 && kv_q_width % 8 == 0 && kv_width % 8 == 0 &&
                                               ((uintptr_t)kv_pool % 16) == 0));
  using namespace rl::tc;
#define RL_TC(T, E)                                                                                                  \
  do {                                                                                                               \
    const Cut cut = plan_cut(M, N, K, E != EPI_PLAIN, staging_bytes<T, E>(), tile_width, splits);                     \
    if (E != EPI_PLAIN && cut.splits > 1)                                                                            \
      return launch_persistent<T, E == EPI_PLAIN ? EPI_TMA : E, true>(A, lda, W, bias, out, ldo, M, N, K, act, residual, kv, \
                                                                     status, cut, stream);                           \
    return launch_persistent<T, E, false>(A, lda, W, bias, out, ldo, M, N, K, act, residual, kv, status, cut, stream); \
  } while (0)
  if (out_dtype == RL_F32) {
    if (tma_out) RL_TC(float, EPI_TMA);
    RL_TC(float, EPI_PLAIN);
  }
  if (tma_out) RL_TC(__nv_bfloat16, EPI_TMA);
  RL_TC(__nv_bfloat16, EPI_PLAIN);
#undef RL_TC
}

RL_EXPORT int rl_gemm_tc(int out_dtype, const void* A, long lda, const void* W, const float* bias, void* out,
                         long ldo, int M, int N, int K, int act, int residual, void* kv_pool,
                         const int* kv_block_table, int kv_bt_stride, const int* kv_positions,
                         const int* kv_req_of_token, const int* kv_slots, int kv_q_width, int kv_width,
                         int kv_head_dim, int kv_page_size, int kv_heads, int kv_max_pos, int* status,
                         cudaStream_t stream) {
  return rl_gemm_tc_cut(out_dtype, A, lda, W, bias, out, ldo, M, N, K, act, residual, kv_pool, kv_block_table,
                        kv_bt_stride, kv_positions, kv_req_of_token, kv_slots, kv_q_width, kv_width, kv_head_dim,
                        kv_page_size, kv_heads, kv_max_pos, status, 0, 0, stream);
}

// The product on tcgen05 tiles with each row's next token chosen from the accumulators and no
// logits written (see SampleArgs): out_ids[m] is what rl_sample would choose from row m of
// A W^T (+ bias).  best [M] and ticket [1]: scratch, zero before the call and again after it.
RL_EXPORT int rl_gemm_tc_sample(const void* A, long lda, const void* W, const float* bias, int M, int N, int K,
                                const float* temperature, const long long* seeds, const int* counters, int* out_ids,
                                unsigned long long* best, int* ticket, int* host_ring, int ring_stride,
                                unsigned int* ring_step, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0 || lda % 8 != 0 || ((uintptr_t)A % 16) != 0 || ((uintptr_t)W % 16) != 0) return -2;
  if (out_ids == nullptr || best == nullptr || ticket == nullptr || status == nullptr) return -7;
  if (temperature != nullptr && (seeds == nullptr || counters == nullptr)) return -7;
  using namespace rl::tc;
  const rl::KvScatter kv{};
  if (host_ring != nullptr && (ring_step == nullptr || ring_stride < M)) return -7;
  const rl::SampleArgs sample{out_ids, temperature, seeds, counters, best, ticket, host_ring, ring_stride, ring_step};
  const Cut cut = plan_cut(M, N, K, false, 0, 0, 0);
  return launch_persistent<float, EPI_SAMPLE, false>(A, lda, W, bias, nullptr, 0, M, N, K, RL_ACT_NONE, 0, kv, status, cut,
                                                     stream, sample);
}

