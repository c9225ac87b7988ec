// bfloat16 products of 17 to 128 rows (a batch of decoded tokens, a short prompt portion) on
// tcgen05, with K split over the blocks of a thread-block cluster:
//
//   out[M,N] = A[M,K] * W[N,K]^T  (+ bias[N]) (GELU) (or out += ..., the float32 residual stream)
//
// the products of rosellm/rosetrainer/model.py:95, 220, 334-337 for the batch sizes between
// the weight-streaming kernel (gemm_rows_mma.cu, where every warp re-reads the rows of A) and
// the tiled kernel for prompts (gemm_tc.cu, whose 128-row tiles leave most SMs idle here).
//
// Such a product is a stream of weights with little arithmetic, so the work is laid out for
// the stream: the roles of the operands are swapped.  A block takes 128 rows of W (output
// columns) as the 128-lane operand of tcgen05.mma and the M rows of A, rounded up to a multiple
// of 16, as the N operand; a cluster of blocks shares one such tile, each block taking a part
// of K small enough that all of its operands are fetched by TMA at once, with no ring.  The
// accumulator (lanes = output columns, columns = rows of A) goes from tensor memory to the
// block's shared memory as float32; after a cluster barrier every block sums, for the rows
// that fall to it, the partial results of all blocks through distributed shared memory in a
// fixed order, applies bias / activation / residual and stores along rows, or scatters key and
// value columns into cache pages.  Waits on mbarriers are bounded (status bit, abort flag);
// the two cluster barriers are reached by every thread on every path.
#include "gemm_epilogue.cuh"
#include "tc_common.cuh"

namespace rl {
namespace tc {

constexpr int RTHREADS = 256;
constexpr int RMAX_CLUSTER = 8;      // the portable limit
constexpr int RW_BYTES = BM * BK * 2;  // a 128 x 64 tile of W

// Shared memory of a block: kb_per stages of (W 128 x 64, A NT x 64) bfloat16, the float32
// partial result [NT][128], the element offsets of the rows' cache pages [128], then the
// barriers (one per stage, one for the accumulator), the tensor-memory address and the abort flag.
__host__ __device__ inline int rows_stage_bytes(int nt) { return RW_BYTES + nt * BK * 2; }
__host__ __device__ inline int rows_smem_bytes(int nt, int kb_per) {
  return kb_per * rows_stage_bytes(nt) + nt * BM * 4 + 128 * 8 + (kb_per + 1) * 8 + 16 + 1024;
}

// Grid (cluster size, tiles of 128 output columns); a cluster is one row of the grid.
// kb_per: K blocks of 64 per block; blocks whose part lies beyond K only help with the sums.
template <typename TOut>
__global__ __launch_bounds__(RTHREADS) void gemm_tc_rows_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
    const float* __restrict__ bias, TOut* __restrict__ out, long ldo, int M, int N, int K, int NT, int kb_per,
    int tmem_cols, int act, int residual, KvScatter kv, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  const int stage_bytes = rows_stage_bytes(NT);
  float* part = reinterpret_cast<float*>(smem + kb_per * stage_bytes);
  long long* row_base = reinterpret_cast<long long*>(part + NT * BM);
  const uint32_t bar_base = smem_u32(row_base + 128);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  const uint32_t acc_bar = bar_base + 8u * kb_per;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(row_base + 128) + (kb_per + 1) * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_rank(), n_ranks = gridDim.x;
  const int n0 = blockIdx.y * BM;
  const int num_kb = (K + BK - 1) / BK;
  const int kb_begin = rank * kb_per;
  const int nkb = max(0, min(num_kb, kb_begin + kb_per) - kb_begin);
  const int n_contrib = (num_kb + kb_per - 1) / kb_per;  // blocks that hold a partial result

  if (threadIdx.x == 0) {
    for (int s = 0; s < kb_per; ++s) mbar_init(full_bar(s), 1);
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_begin();

  if (threadIdx.x == 0 && nkb > 0) {
    // every operand of this block at once, then the MMAs as the K blocks arrive
    for (int s = 0; s < nkb; ++s) {
      mbar_expect_tx(full_bar(s), (uint32_t)stage_bytes);
      const uint32_t dst = smem_base + s * stage_bytes;
      tma_load_2d(dst, &map_w, full_bar(s), (kb_begin + s) * BK, n0);
      tma_load_2d(dst + RW_BYTES, &map_a, full_bar(s), (kb_begin + s) * BK, 0);
    }
    const uint32_t idesc = instr_desc(NT);
    bool ok = true;
    int waited = 0;
    for (int s = 0; s < nkb && ok; ++s) {
      ok = mbar_wait(full_bar(s), 0u, abort_flag, status);
      if (!ok) break;
      ++waited;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t w_addr = smem_base + s * stage_bytes;
      const uint32_t a_addr = w_addr + RW_BYTES;
#pragma unroll
      for (int k = 0; k < BK / 16; ++k)
        mma_f16(tmem_base, smem_desc(w_addr + k * 32), smem_desc(a_addr + k * 32), idesc, (s | k) != 0 ? 1u : 0u);
    }
    if (ok) {
      mma_commit(acc_bar);
    } else {
      for (int s = waited; s < nkb; ++s) mbar_wait_quiet(full_bar(s), 0u);  // copies still in flight
    }
  } else if (warp >= 4 && kv.pool != nullptr && n0 + BM > kv.q_width) {
    // where the keys and values of each row go: the element offset of (page, keys, head 0,
    // place in the page, 0), or -1 for a row that is not written
    const int m = threadIdx.x - 128;
    if (m < M) {
      long long base = -1;
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
            base = ((long long)page * 2 * kv.n_kv_heads * kv.page_size + pos % kv.page_size) * kv.head_dim;
        }
      }
      row_base[m] = base;
    }
  }
  __syncwarp();

  // accumulator -> this block's partial result: warp w reads lanes 32*(w%4).. (output columns),
  // the two warps of a quarter take the even and the odd chunks of 16 rows of A
  if (nkb > 0) {
    const bool ok = __all_sync(0xffffffffu, mbar_wait(acc_bar, 0u, abort_flag, status));  // one answer per warp
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const int quarter = warp & 3;
      for (int c = warp >> 2; c < NT / 16; c += 2) {
        uint32_t r[16];
        tmem_load16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 16), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 16; ++i) part[(c * 16 + i) * BM + quarter * 32 + lane] = __uint_as_float(r[i]);
      }
    }
    __syncwarp();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncwarp();
  cluster_sync();

  // rows rank, rank + n_ranks, ... of A fall to this block, one row to a warp at a time; a lane
  // owns four neighbouring output columns and sums their parts of K in a fixed order
  {
    const int col = 4 * lane;
    const int n = n0 + col;
    const uint32_t mine = smem_u32(part + col);
    uint32_t peer[RMAX_CLUSTER];
#pragma unroll
    for (int p = 0; p < RMAX_CLUSTER; ++p) peer[p] = peer_addr(mine, (uint32_t)min(p, n_contrib - 1));
    const int n_valid = min(4, N - n);
    const bool vec_ok = ((ldo * (long)sizeof(TOut)) % 16 == 0) && (((uintptr_t)out) % 16 == 0) &&
                        (bias == nullptr || ((uintptr_t)bias) % 16 == 0);
    const float* bias4 = bias != nullptr ? bias + n : nullptr;
    // the four columns lie in one head: head sizes and the query width are multiples of 16
    const bool to_cache = kv.pool != nullptr && n >= kv.q_width;
    long long col_off = 0;
    if (to_cache) {
      const int cidx = n - kv.q_width;
      const int which = cidx / kv.kv_width;
      const int rem = cidx - which * kv.kv_width;
      const int head = rem / kv.head_dim;
      col_off = ((long long)(which * kv.n_kv_heads + head) * kv.page_size) * kv.head_dim + (rem - head * kv.head_dim);
    }
    for (int t = rank + n_ranks * warp; t < M; t += n_ranks * (RTHREADS / 32)) {
      float4 r[RMAX_CLUSTER];
      const uint32_t off = (uint32_t)(t * BM * 4);
#pragma unroll
      for (int p = 0; p < RMAX_CLUSTER; ++p)
        asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(r[p].x), "=f"(r[p].y), "=f"(r[p].z), "=f"(r[p].w)
                     : "r"(peer[p] + off)
                     : "memory");
      if (n_valid <= 0) continue;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int p = 0; p < RMAX_CLUSTER; ++p)
        if (p < n_contrib) {
          acc.x += r[p].x; acc.y += r[p].y; acc.z += r[p].z; acc.w += r[p].w;
        }
      if (to_cache) {
        const long long base = row_base[t];
        if (base >= 0)
          finish4<__nv_bfloat16>((__nv_bfloat16*)kv.pool + base + col_off, acc, bias4, act, 0, true, n_valid);
      } else {
        finish4<TOut>(out + (size_t)t * ldo + n, acc, bias4, act, residual, vec_ok, n_valid);
      }
    }
  }
  __syncwarp();
  cluster_sync();  // no block leaves while another may still read its partial result
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)tmem_cols)
                 : "memory");
  }
}

// The split of K: as many blocks per tile as bring the grid near one block per SM, a power of
// two up to the portable cluster size, and few enough K blocks per block for shared memory.
// Returns false when the product does not fit this kernel.
static bool rows_plan(int M, int N, int K, int* nt, int* kb_per, int* cluster, int* tmem_cols) {
  if (M < 1 || M > 128) return false;
  *nt = (M + 15) / 16 * 16;
  *tmem_cols = *nt <= 32 ? 32 : (*nt <= 64 ? 64 : 128);
  const int num_kb = (K + BK - 1) / BK;
  const int tiles = (N + BM - 1) / BM;
  int ks = 1;
  while (ks < RMAX_CLUSTER && ks * 2 <= num_kb && tiles * ks * 2 <= 160) ks *= 2;
  while (ks < RMAX_CLUSTER && rows_smem_bytes(*nt, (num_kb + ks - 1) / ks) > 200 * 1024) ks *= 2;
  *kb_per = (num_kb + ks - 1) / ks;
  *cluster = ks;
  return rows_smem_bytes(*nt, *kb_per) <= 200 * 1024;
}

template <typename TOut>
static int launch_rows(const void* A, long lda, const void* W, const float* bias, void* out, long ldo, int M, int N,
                       int K, int act, int residual, const KvScatter& kv, int* status, cudaStream_t stream) {
  int nt, kb_per, cluster, tmem_cols;
  if (!rows_plan(M, N, K, &nt, &kb_per, &cluster, &tmem_cols)) return -7;
  CUtensorMap mw, ma;
  int rc = tensor_map(W, N, K, K, BM, &mw);
  if (rc != 0) return rc;
  rc = tensor_map(A, M, K, lda, nt, &ma);
  if (rc != 0) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    note_launch(cudaFuncSetAttribute(gemm_tc_rows_kernel<TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024));
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cluster, (N + BM - 1) / BM);
  cfg.blockDim = dim3(RTHREADS);
  cfg.dynamicSmemBytes = rows_smem_bytes(nt, kb_per);
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
  note_launch(cudaLaunchKernelEx(&cfg, gemm_tc_rows_kernel<TOut>, mw, ma, bias, (TOut*)out, ldo, M, N, K, nt, kb_per,
                                 tmem_cols, act, residual, kv, status));
  return take_launch_error();
}

}  // namespace tc
}  // namespace rl

// Whether rl_gemm_tc_rows takes a product of these sizes (1: yes).
RL_EXPORT int rl_gemm_tc_rows_fits(int M, int N, int K) {
  int nt, kb_per, cluster, tmem_cols;
  return rl::tc::rows_plan(M, N, K, &nt, &kb_per, &cluster, &tmem_cols) ? 1 : 0;
}

// bfloat16 A [M <= 128, K] (row stride lda) and W [N, K]; out bfloat16 or float32 [M, N].
// residual != 0: out (float32) += result.  kv_pool != nullptr: output columns from kv_q_width
// on are written into cache pages as keys and values, not to out.  Returns -7 when the sizes
// do not fit (K too long for one block's shared memory).
RL_EXPORT int rl_gemm_tc_rows(int out_dtype, const void* A, long lda, const void* W, const float* bias, void* out,
                              long ldo, int M, int N, int K, int act, int residual, void* kv_pool,
                              const int* kv_block_table, int kv_bt_stride, const int* kv_positions,
                              const int* kv_req_of_token, const int* kv_slots, int kv_q_width, int kv_width,
                              int kv_head_dim, int kv_page_size, int kv_heads, int kv_max_pos, int* status,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0 || lda % 8 != 0 || ((uintptr_t)A % 16) != 0 || ((uintptr_t)W % 16) != 0) return -2;
  if (residual && out_dtype != RL_F32) return -3;
  if (out_dtype != RL_F32 && out_dtype != RL_BF16) return -4;
  rl::KvScatter kv{kv_pool, kv_block_table, kv_bt_stride, kv_positions, kv_req_of_token, kv_slots,
                   kv_q_width, kv_width, kv_head_dim, kv_page_size, kv_heads, kv_max_pos, status};
  const int rc = out_dtype == RL_F32
                     ? rl::tc::launch_rows<float>(A, lda, W, bias, out, ldo, M, N, K, act, residual, kv, status, stream)
                     : rl::tc::launch_rows<__nv_bfloat16>(A, lda, W, bias, out, ldo, M, N, K, act, residual, kv,
                                                          status, stream);
  if (rc != 0) return rc;
  RL_CHECK_LAUNCH();
  return 0;
}
