// bfloat16 products of up to 64 rows (a decode step of many requests; large matrices at any batch):
//   out[M,N] = A[M,K] * W[N,K]^T (+ bias) (GELU) (or out += ..., the float32 residual stream),
// the same products and epilogues as the other matrix kernels (rosellm/rosetrainer/model.py:95,
// 220, 334-337).
//
// With this many rows the weight-streaming kernel (gemm_rows_mma.cu) re-reads the rows of A in
// every warp: at 64 rows of 768 that is 98 KB a block and tens of megabytes from L2 a product,
// which costs more than the weights themselves.  Here a block owns 8 to 32 output columns and a part
// of K and keeps BOTH operands in shared memory: its slice of W is a weight, so its copy is issued
// before the block waits for the kernels ahead (programmatic dependent launch) and travels under
// them; the rows of A follow after the wait, one copy a row; sixteen warps then take one
// (16 rows x 8 columns) tile each over the whole of the block's part of K on mma.sync m16n8k16
// from ldmatrix fragments (with fewer than 64 rows, several warps share a tile and split K).
// Products whose inner size is too long for shared memory (mlp.c_proj) are split over K between
// blocks, whose partial results are added into the float32 output with red.global.add: only
// `out += ...` products take that form, and the order of those additions is not fixed.
// (tcgen05 tiles are 128 rows: for 64 rows of a 768-wide output they leave most SMs idle.)
#include "gemm_epilogue.cuh"
#include "tc_common.cuh"

namespace rl {
namespace rsm {

constexpr int WARPS = 16;
constexpr int THREADS = 32 * WARPS;
constexpr size_t SMEM_LIMIT = 220 * 1024;  // shared memory a block may ask for

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
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

// Row stride in shared memory (elements): an odd number of 16-byte pieces, so that the eight rows
// an ldmatrix reads fall into distinct banks.
__host__ __device__ inline int padded(int k) { return (k + 15) / 16 * 16 + 8; }

struct Args {
  const __nv_bfloat16* a;  // [M, K], row stride lda
  long lda;
  const __nv_bfloat16* w;  // [N, K]
  const float* bias;       // [N] or nullptr
  void* out;               // [M, N] bfloat16 or float32, row stride ldo
  long ldo;
  int M, N, K, kc, act, residual, out_f32;
  KvScatter kv;
  int* status;
};

// Shared memory: bars 32 | a_s [16 * MT][ld] | w_s [8 * NT][ld] | part_s [WARPS][16][8] f32.
// MT: tiles of 16 rows; NT: tiles of eight output columns a block owns.
template <int MT, int NT>
__global__ __launch_bounds__(THREADS) void gemm_rows_smem_kernel(Args p) {
  constexpr int NB = 8 * NT;                 // output columns of the block
  constexpr int PAIRS = MT * NT;             // (16 rows, 8 columns) tiles of the block
  constexpr int KPARTS = WARPS / PAIRS >= 1 ? WARPS / PAIRS : 1;  // warps that share a tile split K
  extern __shared__ __align__(16) uint8_t smem[];
  const int kc = p.kc, ld = padded(kc);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // [0] W, [1] A
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 16);
  __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(smem + 32);
  __nv_bfloat16* w_s = a_s + (size_t)16 * MT * ld;
  float* part_s = reinterpret_cast<float*>(w_s + (size_t)NB * ld);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.x * NB;
  const int k0 = blockIdx.y * kc;
  const int k_here = min(kc, p.K - k0);  // a multiple of 8; the last part of K may be short
  const int cols_here = min(NB, p.N - n0);
  const uint32_t bar_w = tc::smem_u32(&bars[0]), bar_a = tc::smem_u32(&bars[1]);

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (tid == 0) {
    tc::mbar_init(bar_w, 1);
    tc::mbar_init(bar_a, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // ---- before the wait: the slice of W starts travelling ----
  if (tid == 0) tc::mbar_expect_tx(bar_w, (uint32_t)(cols_here * k_here * 2));
  if (tid < cols_here)
    bulk_copy(tc::smem_u32(w_s + (size_t)tid * ld), p.w + (size_t)(n0 + tid) * p.K + k0, (uint32_t)k_here * 2, bar_w);
  {
    // what no copy fills must be zero: columns from k_here to the next multiple of 16, rows of A
    // beyond M, rows of W beyond N
    const __nv_bfloat16 z = __float2bfloat16_rn(0.f);
    const int kz = (k_here + 15) / 16 * 16;
    if (kz > k_here)
      for (int i = tid; i < (16 * MT + NB) * (kz - k_here); i += THREADS) {
        const int r = i / (kz - k_here), c = k_here + i % (kz - k_here);
        (r < 16 * MT ? a_s + (size_t)r * ld : w_s + (size_t)(r - 16 * MT) * ld)[c] = z;
      }
    for (int i = tid; i < (16 * MT - p.M) * (kz / 8); i += THREADS) {
      const int r = p.M + i / (kz / 8), c = (i % (kz / 8)) * 8;
      *reinterpret_cast<uint4*>(a_s + (size_t)r * ld + c) = make_uint4(0u, 0u, 0u, 0u);
    }
    for (int i = tid; i < (NB - cols_here) * (kz / 8); i += THREADS) {
      const int r = cols_here + i / (kz / 8), c = (i % (kz / 8)) * 8;
      *reinterpret_cast<uint4*>(w_s + (size_t)r * ld + c) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  // where the keys and values of this lane's rows go (packed qkv product): asked for now (the
  // step's description and the block table are not written by the step's kernels)
  const int g = lane >> 2, j = lane & 3;
  const int pair = warp % PAIRS, kp = warp / PAIRS;  // this warp's tile, and its part of K
  const int mt = pair / NT, nt = pair % NT;
  const bool to_cache = p.kv.pool != nullptr && n0 + nt * 8 >= p.kv.q_width;
  int kv_page[2] = {-1, -1}, kv_place[2] = {0, 0};
  if (to_cache && kp == 0) {
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      const int m = mt * 16 + hlf * 8 + g;
      if (m < p.M) {
        const int slot = p.kv.slots[p.kv.req_of_token[m]];
        const int pos = p.kv.positions[m];
        if (slot >= 0) {  // slot -1: padding of a fixed-size batch
          if (pos < 0 || pos >= p.kv.max_pos) {
            atomicOr(p.kv.status, RL_STATUS_BAD_POSITION);
          } else {
            kv_page[hlf] = p.kv.block_table[(size_t)slot * p.kv.bt_stride + pos / p.kv.page_size];
            kv_place[hlf] = pos % p.kv.page_size;
            if (kv_page[hlf] < 0) atomicOr(p.kv.status, RL_STATUS_BAD_PAGE);
          }
        }
      }
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // ---- the rows of A (written by the kernel ahead): one copy a row ----
  if (tid == 0) tc::mbar_expect_tx(bar_a, (uint32_t)(p.M * k_here * 2));
  if (tid < p.M)
    bulk_copy(tc::smem_u32(a_s + (size_t)tid * ld), p.a + (size_t)tid * p.lda + k0, (uint32_t)k_here * 2, bar_a);
  bool ok = tc::mbar_wait(bar_w, 0, abort_flag, p.status);
  ok = tc::mbar_wait(bar_a, 0, abort_flag, p.status) && ok;
  __syncthreads();  // the zeros written above are in place too
  if (*abort_flag) {
    tc::mbar_wait_quiet(bar_w, 0);
    tc::mbar_wait_quiet(bar_a, 0);
    return;
  }

  // ---- this warp's tile over its part of K ----
  float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};  // two chains of products
  if (kp < KPARTS) {
    const int ksteps = (k_here + 15) / 16;
    const int per = (ksteps + KPARTS - 1) / KPARTS;
    const int k_lo = kp * per, k_hi = min(ksteps, k_lo + per);
    const uint32_t a_addr = tc::smem_u32(a_s + (size_t)(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + (lane >> 4) * 8);
    const uint32_t b_addr = tc::smem_u32(w_s + (size_t)(nt * 8 + (lane & 7)) * ld + ((lane >> 3) & 1) * 8);
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
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] += c2[i];
  }
  if constexpr (KPARTS > 1) {
    // the warps of a tile add their parts of K in a fixed order
    float* ps = part_s + (size_t)warp * 16 * 8;
    *reinterpret_cast<float2*>(ps + g * 8 + 2 * j) = make_float2(c[0], c[1]);
    *reinterpret_cast<float2*>(ps + (g + 8) * 8 + 2 * j) = make_float2(c[2], c[3]);
    __syncthreads();
    if (kp != 0) return;
#pragma unroll
    for (int q = 1; q < KPARTS; ++q) {
      const float* o = part_s + (size_t)(q * PAIRS + pair) * 16 * 8;
      c[0] += o[g * 8 + 2 * j]; c[1] += o[g * 8 + 2 * j + 1];
      c[2] += o[(g + 8) * 8 + 2 * j]; c[3] += o[(g + 8) * 8 + 2 * j + 1];
    }
  } else if (kp != 0) {
    return;
  }

  // ---- epilogue: c0, c1 = row g, columns 2j, 2j+1 of the tile; c2, c3 = row g + 8 ----
  const int n = n0 + nt * 8 + 2 * j;
  if (n >= p.N) return;
  const bool split = gridDim.y > 1;
  const bool with_bias = p.bias != nullptr && (!split || blockIdx.y == 0);
  const float b0 = with_bias ? p.bias[n] : 0.f, b1 = with_bias && n + 1 < p.N ? p.bias[n + 1] : 0.f;
  // pairs of columns are stored together where both exist and the pair is aligned (even widths
  // and strides: every product of a layer); an odd output width (a vocabulary) goes one by one
  const bool pair_ok = n + 1 < p.N && p.ldo % 2 == 0;
#pragma unroll
  for (int hlf = 0; hlf < 2; ++hlf) {
    const int m = mt * 16 + hlf * 8 + g;
    if (m >= p.M) continue;
    const float v0 = tc::act_fn(c[2 * hlf] + b0, p.act), v1 = tc::act_fn(c[2 * hlf + 1] + b1, p.act);
    if (to_cache) {
      if (kv_page[hlf] < 0) continue;
      const int cidx = n - p.kv.q_width;
      const int which = cidx / p.kv.kv_width;
      const int rem = cidx - which * p.kv.kv_width;
      const int head = rem / p.kv.head_dim, d = rem - head * p.kv.head_dim;
      __nv_bfloat16* dst = (__nv_bfloat16*)p.kv.pool +
                           ((((size_t)kv_page[hlf] * 2 + which) * p.kv.n_kv_heads + head) * p.kv.page_size + kv_place[hlf]) *
                               p.kv.head_dim + d;
      *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(v0, v1);  // d is even: 4-byte aligned
    } else if (p.out_f32) {
      float* dst = (float*)p.out + (size_t)m * p.ldo + n;
      if (split) {  // the parts of K meet in memory (out += ... only)
        if (pair_ok) {
          red_add2(dst, v0, v1);
        } else {
          atomicAdd(dst, v0);
          if (n + 1 < p.N) atomicAdd(dst + 1, v1);
        }
      } else if (pair_ok) {
        float2 r = make_float2(v0, v1);
        if (p.residual) {
          const float2 old = *reinterpret_cast<const float2*>(dst);
          r = make_float2(old.x + v0, old.y + v1);
        }
        *reinterpret_cast<float2*>(dst) = r;
      } else {
        dst[0] = p.residual ? dst[0] + v0 : v0;
        if (n + 1 < p.N) dst[1] = p.residual ? dst[1] + v1 : v1;
      }
    } else {
      __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (size_t)m * p.ldo + n;
      if (pair_ok) {
        *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(v0, v1);
      } else {
        dst[0] = __float2bfloat16_rn(v0);
        if (n + 1 < p.N) dst[1] = __float2bfloat16_rn(v1);
      }
    }
  }
}

static size_t smem_bytes(int mt, int nt, int kc) {
  const int ld = padded(kc);
  return 32 + (size_t)(16 * mt + 8 * nt) * ld * 2 + (size_t)WARPS * 16 * 8 * 4;
}

// How a product is cut: tiles of eight columns a block (nt), parts of K (parts) of kc elements.
struct Plan {
  int nt, parts, kc;
};

// The plan for a product of these sizes, nt == 0 where this kernel does not take it.  K is cut
// only for `out += ...` into float32 (the parts meet in memory), otherwise a block's part of K
// is all of it and must fit shared memory beside the rows.  Among the block widths that fit, the
// one is taken whose blocks go round the device in the least time (rounds x width; the wider on
// a tie, since it re-reads the rows less).
static Plan plan_for(int M, int N, int K, int residual, int out_f32, int act, bool to_cache) {
  Plan none{0, 0, 0};
  if (M < 1 || M > 64 || K % 8 != 0 || N < 1) return none;
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    if (n_sms <= 0) n_sms = 1;
  }
  const int mt = (M + 15) / 16;
  const bool may_split = residual && out_f32 && act == 0 && !to_cache;
  Plan best = none;
  long best_cost = 0;
  for (int nt = 4; nt >= 1; --nt) {
    if (mt * nt > WARPS) continue;
    if ((mt == 2 && nt == 3) || (mt == 3 && nt != 4) || (mt == 4 && (nt == 3 || nt == 1))) continue;  // forms that exist
    // the longest part of K that fits beside the rows
    int parts = 1;
    int kc = (K + 15) / 16 * 16;
    while (smem_bytes(mt, nt, kc) > SMEM_LIMIT) {
      ++parts;
      kc = ((K + parts - 1) / parts + 15) / 16 * 16;
    }
    if (parts > 1 && !may_split) continue;
    parts = (K + kc - 1) / kc;
    const long blocks = (long)((N + 8 * nt - 1) / (8 * nt)) * parts;
    const long per_sm = (long)((227 * 1024) / (smem_bytes(mt, nt, kc) + 1024));
    const long rounds = (blocks + n_sms * per_sm - 1) / (n_sms * per_sm);
    const long cost = rounds * nt * kc;
    if (best.nt == 0 || cost < best_cost) {
      best = Plan{nt, parts, kc};
      best_cost = cost;
    }
  }
  return best;
}

template <int MT, int NT>
static int launch(const Args& p, int parts, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    note_launch(cudaFuncSetAttribute(gemm_rows_smem_kernel<MT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)SMEM_LIMIT));
    note_launch(cudaFuncSetAttribute(gemm_rows_smem_kernel<MT, NT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     cudaSharedmemCarveoutMaxShared));
    attr_set = true;
  }
  launch_pdl_split(false, gemm_rows_smem_kernel<MT, NT>, dim3((p.N + 8 * NT - 1) / (8 * NT), parts), dim3(THREADS),
                   smem_bytes(MT, NT, p.kc), stream, p);
  return take_launch_error();
}

}  // namespace rsm
}  // namespace rl

// Whether rl_gemm_rows_smem takes a product of these sizes (see above).
RL_EXPORT int rl_gemm_rows_smem_fits(int M, int N, int K, int residual, int out_f32, int act, int to_cache) {
  return rl::rsm::plan_for(M, N, K, residual, out_f32, act, to_cache != 0).nt > 0 ? 1 : 0;
}

// bfloat16 A [M <= 64, K] (row stride lda, a multiple of 8) and W [N, K]; out bfloat16 or float32.
// residual != 0: out (float32) += result.  kv_pool != nullptr: columns from kv_q_width on go to
// cache pages as keys and values.  Returns -2 for sizes the kernel does not take.
RL_EXPORT int rl_gemm_rows_smem(int out_dtype, const void* A, long lda, const void* W, const float* bias, void* out,
                                long ldo, int M, int N, int K, int act, int residual, void* kv_pool,
                                const int* kv_block_table, int kv_bt_stride, const int* kv_positions,
                                const int* kv_req_of_token, const int* kv_slots, int kv_q_width, int kv_width,
                                int kv_head_dim, int kv_page_size, int kv_heads, int kv_max_pos, int* status,
                                cudaStream_t stream) {
  using namespace rl::rsm;
  if (M <= 0 || N <= 0) return 0;
  if (out_dtype != RL_F32 && out_dtype != RL_BF16) return -4;
  if (residual && out_dtype != RL_F32) return -3;
  if (lda % 8 != 0 || ((uintptr_t)A % 16) != 0 || ((uintptr_t)W % 16) != 0 || status == nullptr) return -2;
  if (((uintptr_t)out % (out_dtype == RL_F32 ? 8 : 4)) != 0) return -2;
  if (kv_pool != nullptr && (kv_head_dim % 8 != 0 || kv_q_width % 8 != 0 || kv_width % 8 != 0 || act != 0 || residual))
    return -8;
  const Plan plan = plan_for(M, N, K, residual, out_dtype == RL_F32, act, kv_pool != nullptr);
  if (plan.nt == 0) return -2;
  const int kc = plan.kc;  // parts of K begin on 16-byte boundaries (and on MMA steps)
  const rl::KvScatter kv{kv_pool, kv_block_table, kv_bt_stride, kv_positions, kv_req_of_token, kv_slots,
                         kv_q_width, kv_width, kv_head_dim, kv_page_size, kv_heads, kv_max_pos, status};
  Args p{(const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, bias, out, ldo, M, N, K, kc, act, residual,
         out_dtype == RL_F32 ? 1 : 0, kv, status};
  const int mt = (M + 15) / 16;
  switch (mt * 10 + plan.nt) {
    case 11: return launch<1, 1>(p, plan.parts, stream);
    case 12: return launch<1, 2>(p, plan.parts, stream);
    case 13: return launch<1, 3>(p, plan.parts, stream);
    case 14: return launch<1, 4>(p, plan.parts, stream);
    case 22: return launch<2, 2>(p, plan.parts, stream);
    case 24: return launch<2, 4>(p, plan.parts, stream);
    case 21: return launch<2, 1>(p, plan.parts, stream);
    case 34: return launch<3, 4>(p, plan.parts, stream);
    case 42: return launch<4, 2>(p, plan.parts, stream);
    case 44: return launch<4, 4>(p, plan.parts, stream);
  }
  return -2;
}
