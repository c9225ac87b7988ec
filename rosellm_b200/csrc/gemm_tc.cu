// Matrix products on the fifth-generation tensor cores of sm_100a (tcgen05), bfloat16 inputs,
// float32 accumulation in tensor memory, operands brought to shared memory by TMA:
//
//   out[M,N] = A[M,K] * W[N,K]^T  (+ bias[N]) (GELU) (or out += ..., the float32 residual stream)
//
// the same products and epilogues as gemm_simt.cu (rosellm/rosetrainer/model.py:95, 220,
// 334-337; fused_mlp.py:79-113), for the many-row case (prompt portions), where arithmetic and
// not memory is the bound.  The reference leaves these products to cuBLAS through torch.
//
// One block per SM walks the output tiles (128 x 256 or 128 x 128, whichever fills its rounds
// over the SMs better).
// Its warps have fixed roles:
//   warp 0     one lane issues the TMA loads of A and W tiles (128 x 64 and BN x 64 bfloat16,
//              128-byte swizzle) into a ring of shared-memory stages, running ahead over tiles;
//   warp 1     allocates 2 x BN columns of tensor memory; one lane issues tcgen05.mma
//              (M=128, N=BN, K=16, four per stage) and commits to the stage's "empty" barrier
//              and, after a tile's last K block, to that accumulator's "full" barrier;
//   warps 2-9  wait for an accumulator, read it with tcgen05.ld (two warps per quarter of the
//              128 lanes = rows), apply bias / activation / residual and store through shared
//              memory so that stores run along rows; then hand the accumulator back.
// The accumulator is double-buffered in tensor memory, so the epilogue of tile i runs under the
// MMAs of tile i+1.  Every wait on a barrier is bounded: after about two seconds the kernel sets
// a status bit, raises a block-wide abort flag and leaves, freeing its tensor memory on the way
// out.  No multicast and no clusters are used.  (A one-tile-per-block form with K split over
// blocks was tried for outputs of few tiles and measured about half as fast.)
#include "gemm_epilogue.cuh"
#include "tc_common.cuh"

namespace rl {
namespace tc {

constexpr int PEPI_WARPS = 8;                     // epilogue warps of the persistent kernel
constexpr int PTHREADS = 32 * (2 + PEPI_WARPS);   // + the TMA warp and the MMA warp

// One block per SM walks the output tiles (tile = blockIdx.x, + gridDim.x, ...).  The accumulator
// is double-buffered in tensor memory (2 x BN columns): while the epilogue warps drain tile i from
// one buffer, the MMA warp already accumulates tile i+1 in the other, and the TMA warp runs ahead
// of both through the same ring of stages.  Tiles are 128 x BN with BN up to 256, which halves
// the operand bytes per flop against 128 x 128.  The epilogue has a staging area of its own, since
// the pipeline's stages are never idle here.
template <int BN>
struct PSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int PSTAGES = BN == 256 ? 3 : 5;  // 3 x 48 KB or 5 x 32 KB, beside 36 KB of staging
  static constexpr int STAGING_OFFSET = PSTAGES * STAGE_BYTES;
  static constexpr int STAGING_BYTES = PEPI_WARPS * 32 * 36 * 4;
  static constexpr int BAR_OFFSET = STAGING_OFFSET + STAGING_BYTES;
  // full[PSTAGES], empty[PSTAGES], acc_full[2], acc_empty[2], tensor-memory address, abort flag
  static constexpr int TOTAL = BAR_OFFSET + (2 * PSTAGES + 4) * 8 + 16 + 1024;
};

template <int BN, typename TOut>
__global__ __launch_bounds__(PTHREADS) void gemm_tc_persistent_kernel(
    const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
    const float* __restrict__ bias, TOut* __restrict__ out, long ldo, int M, int N, int K, int act,
    int residual, KvScatter kv, int* __restrict__ status) {
  using S = PSmem<BN>;
  constexpr int PSTAGES = S::PSTAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + S::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (PSTAGES + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (2 * PSTAGES + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (2 * PSTAGES + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::BAR_OFFSET + (2 * PSTAGES + 4) * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  const int num_kb = (K + BK - 1) / BK;

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
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"((uint32_t)(2 * BN))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_begin();

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;  // K blocks issued so far, over all tiles
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % PSTAGES;
          const uint32_t ph = (it / PSTAGES) & 1u;
          ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, status);
          if (!ok) break;
          mbar_expect_tx(full_bar(s), S::STAGE_BYTES);
          const uint32_t a_dst = smem_base + s * S::STAGE_BYTES;
          tma_load_2d(a_dst, &map_a, full_bar(s), kb * BK, m0);
          tma_load_2d(a_dst + S::A_BYTES, &map_w, full_bar(s), kb * BK, n0);
        }
      }
      if (*abort_flag) {
        for (uint32_t k = it > (uint32_t)PSTAGES ? it - PSTAGES : 0; k < it; ++k)
          mbar_wait_quiet(full_bar(k % PSTAGES), (k / PSTAGES) & 1u);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BN);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        ok = mbar_wait(acc_empty(buf), ((local >> 1) & 1u) ^ 1u, abort_flag, status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_addr = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % PSTAGES;
          ok = mbar_wait(full_bar(s), (it / PSTAGES) & 1u, abort_flag, status);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_base + s * S::STAGE_BYTES;
          const uint32_t b_addr = a_addr + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            mma_f16(d_addr, smem_desc(a_addr + k * 32), smem_desc(b_addr + k * 32), idesc, (kb | k) != 0 ? 1u : 0u);
          mma_commit(empty_bar(s));
        }
        if (ok) mma_commit(acc_full(buf));
      }
    }
  } else {
    // eight warps: two per lane quarter of tensor memory, taking the even and the odd 32-column
    // chunks of the tile
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int PITCH = 36;
    float* stage = reinterpret_cast<float*>(smem + S::STAGING_OFFSET) + (warp - 2) * 32 * PITCH;
    const bool vec_ok = ((ldo * (long)sizeof(TOut)) % 16 == 0) && (((uintptr_t)out) % 16 == 0) &&
                        (bias == nullptr || ((uintptr_t)bias) % 16 == 0);
    const int sub_row = lane >> 3, col4 = (lane & 7) * 4;
    uint32_t local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
      const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
      const int buf = local & 1;
      // where the keys and values of this lane's row go (packed qkv product): the element offset
      // of (page, keys, head 0, place in the page, 0), or -1 for a row that is not written;
      // looked up while the tile still accumulates
      long long row_base = -1;
      const bool tile_to_cache = kv.pool != nullptr && n0 + BN > kv.q_width;
      if (tile_to_cache) {
        const int m = m0 + quarter * 32 + lane;
        if (m < M) {
          const int slot = kv.slots[kv.req_of_token[m]];
          const int pos = kv.positions[m];
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
      }
      ok = mbar_wait(acc_full(buf), (local >> 1) & 1u, abort_flag, status);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c = half; c < BN / 32; c += 2) {
        uint32_t r[32];
        tmem_load32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        __syncwarp();
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<float4*>(stage + lane * PITCH + 4 * q) =
              make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                          __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
        __syncwarp();
        const int col = n0 + c * 32 + col4;
        // the four columns lie in one head: head sizes and the query width are multiples of 16
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
        const float* bias4 = bias != nullptr && col < N ? bias + col : nullptr;
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
                finish4<__nv_bfloat16>((__nv_bfloat16*)kv.pool + base + col_off, v, bias4, act, 0, true, n_valid);
            } else {
              finish4<TOut>(out + (size_t)row * ldo + col, v, bias4, act, residual, vec_ok, n_valid);
            }
          }
        }
      }
      // the buffer may be overwritten by the MMAs of the tile after next
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(buf)) : "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)(2 * BN))
                 : "memory");
  }
}

template <int BN, typename TOut>
static int launch_persistent(const void* A, long lda, const void* W, const float* bias, void* out, long ldo,
                             int M, int N, int K, int act, int residual, const KvScatter& kv, int* status,
                             cudaStream_t stream) {
  CUtensorMap ma, mw;
  int rc = tensor_map(A, M, K, lda, BM, &ma);
  if (rc != 0) return rc;
  rc = tensor_map(W, N, K, K, BN, &mw);
  if (rc != 0) return rc;
  static bool attr_set = false;
  static int n_sms = 0;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         PSmem<BN>::TOTAL);
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    attr_set = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < n_sms ? tiles : n_sms;
  launch_pdl(gemm_tc_persistent_kernel<BN, TOut>, grid, PTHREADS, PSmem<BN>::TOTAL, stream, ma, mw, bias,
             (TOut*)out, ldo, M, N, K, act, residual, kv, status);
  return 0;
}

}  // namespace tc
}  // namespace rl

// bfloat16 A [M,K] (row stride lda) and W [N,K]; out bfloat16 or float32 [M,N] (row stride ldo).
// residual != 0: out (float32) += result.  kv_pool != nullptr: output columns from kv_q_width
// on are written into cache pages as keys and values, not to out (head size and query width
// multiples of 4).  K and lda multiples of 8, operands on 16-byte boundaries.  Returns 0, a
// CUDA error, or a negative code for refused arguments.
RL_EXPORT int rl_gemm_tc(int out_dtype, const void* A, long lda, const void* W, const float* bias, void* out,
                         long ldo, int M, int N, int K, int act, int residual, void* kv_pool,
                         const int* kv_block_table, int kv_bt_stride, const int* kv_positions,
                         const int* kv_req_of_token, const int* kv_slots, int kv_q_width, int kv_width,
                         int kv_head_dim, int kv_page_size, int kv_heads, int kv_max_pos, int* status,
                         cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0 || lda % 8 != 0 || ((uintptr_t)A % 16) != 0 || ((uintptr_t)W % 16) != 0) return -2;
  if (residual && out_dtype != RL_F32) return -3;
  if (out_dtype != RL_F32 && out_dtype != RL_BF16) return -4;
  if (kv_pool != nullptr && (kv_head_dim % 4 != 0 || kv_q_width % 4 != 0 || kv_width % 4 != 0 || act != 0 || residual))
    return -8;
  const rl::KvScatter kv{kv_pool, kv_block_table, kv_bt_stride, kv_positions, kv_req_of_token, kv_slots,
                         kv_q_width, kv_width, kv_head_dim, kv_page_size, kv_heads, kv_max_pos, status};
  // 128 x 256 tiles move fewer operand bytes per flop and cost about 1.7 times a 128 x 128 tile;
  // which of the two needs less time depends on how evenly its tiles fill the rounds over the SMs
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    if (n_sms <= 0) n_sms = 148;
  }
  const long m_tiles = (M + 127) / 128;
  const long tiles256 = (long)((N + 255) / 256) * m_tiles, tiles128 = (long)((N + 127) / 128) * m_tiles;
  const bool wide = 17 * ((tiles256 + n_sms - 1) / n_sms) <= 10 * ((tiles128 + n_sms - 1) / n_sms);
  int rc;
  if (wide)
    rc = out_dtype == RL_F32
             ? rl::tc::launch_persistent<256, float>(A, lda, W, bias, out, ldo, M, N, K, act, residual, kv, status, stream)
             : rl::tc::launch_persistent<256, __nv_bfloat16>(A, lda, W, bias, out, ldo, M, N, K, act, residual, kv, status, stream);
  else
    rc = out_dtype == RL_F32
             ? rl::tc::launch_persistent<128, float>(A, lda, W, bias, out, ldo, M, N, K, act, residual, kv, status, stream)
             : rl::tc::launch_persistent<128, __nv_bfloat16>(A, lda, W, bias, out, ldo, M, N, K, act, residual, kv, status, stream);
  if (rc != 0) return rc;
  RL_CHECK_LAUNCH();
  return 0;
}
