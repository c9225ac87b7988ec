// Attention of prompt portions on the tensor cores (bfloat16): the same function as
// attn_tile_kernel (attention_kernels.cuh; rosellm/rosetrainer/model.py:169-185 with the online
// softmax of rosellm/rosetrainer/paged_attention.py:80-109), arranged for mma.sync m16n8k16.
//
// A block takes 64 consecutive queries of one request and head.  Its eight warps form two groups
// of four (16 queries per warp, the same queries in both groups); the groups take the visible
// tiles of 64 keys in turn, each gathering its tiles from their pages into shared memory of its
// own with cp.async, two in flight, and the results of the two groups are merged through shared
// memory at the end.  The time of a step's attention is that of the block with the most keys,
// so what matters is how fast one block walks them: two groups halve that walk.  Per tile a warp computes S = Q K^T (Q fragments stay in
// registers), masks by position, updates the running maximum and sum in float32, turns the
// probabilities into bfloat16 A-fragments in registers and accumulates O += P V in float32.
// Shared-memory rows are padded by 16 bytes, which spreads the eight rows of an ldmatrix over
// all banks for every head size that is a multiple of 16.  Head sizes up to 128; larger ones
// keep the CUDA-core kernel.  The reference calls FlashInfer / flash-attn here
// (rosellm/rosetrainer/attention_backends.py:456-577).
#pragma once
#include "attention_kernels.cuh"

namespace rl {

constexpr int MMA_TILE_Q = 64;
constexpr int MMA_TILE_KV = 64;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// 2^x by the hardware approximation (two units in the last place; -inf gives 0).
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// tiles: [n][2] = (request, first query of a 64-query tile within the request's portion).
// (Blocks of half a tile, tried for steps with few tiles, were slower: the time is that of the
// longest block's walk over its keys, not of idle SMs.)
#ifndef RL_MMA_GROUPS
#define RL_MMA_GROUPS 1
#endif
#ifndef RL_MMA_STAGES
#define RL_MMA_STAGES 2
#endif
constexpr int MMA_GROUPS = RL_MMA_GROUPS;
constexpr int MMA_STAGES = RL_MMA_STAGES;  // tiles of keys a group has in shared memory

__device__ __forceinline__ void group_sync(int group) {
  if (group == 0)  // barrier 0 is __syncthreads
    asm volatile("bar.sync 1, 128;" ::: "memory");
  else
    asm volatile("bar.sync 2, 128;" ::: "memory");
}

template <int DH>
__global__ __launch_bounds__(128 * MMA_GROUPS) void attn_mma_kernel(AttnParams p, const int* __restrict__ tiles) {
  constexpr int BLOCK_Q = MMA_TILE_Q;
  constexpr int ROW = DH + 8;            // padded row, in elements
  constexpr int CHUNKS = DH / 8;         // 16-byte pieces of a row
  constexpr int KSTEPS = DH / 16;        // mma steps along the head dimension
  constexpr int DTILES = DH / 8;         // 8-wide output tiles along the head dimension
  extern __shared__ __align__(16) uint8_t mma_smem[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(mma_smem);        // [64][ROW]
  const int group = threadIdx.x >> 7;                                     // which tiles of keys: t % 2 == group
  __nv_bfloat16* k_s = q_s + BLOCK_Q * ROW + group * 2 * MMA_STAGES * MMA_TILE_KV * ROW;  // [stages][64][ROW] of this group
  __nv_bfloat16* v_s = k_s + MMA_STAGES * MMA_TILE_KV * ROW;                              // [stages][64][ROW]
  pdl_begin();
  const int tid = threadIdx.x & 127, lane = tid & 31, warp = tid >> 5;    // within the group
  const int g = lane >> 2, j = lane & 3;
  // tiles are listed by rising position; the later a tile the more keys it sees, so the list is
  // walked from its end: the longest blocks start first and the short ones fill the tail
  const int tile = gridDim.x - 1 - blockIdx.x;
  const int req = tiles[2 * tile], t0 = tiles[2 * tile + 1];
  const int h = blockIdx.y;
  const int hkv = h / (p.n_heads / p.n_kv_heads);
  const int qs = p.q_start[req];
  const int q_len = p.q_start[req + 1] - qs;
  const int kv_len = p.kv_len[req];
  const int rows = min(BLOCK_Q, q_len - t0);
  const int first_pos = kv_len - q_len + t0;
  const int kv_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int kv_hi = first_pos + rows;
  const int* bt = p.block_table + (size_t)p.slots[req] * p.bt_stride;
  const __nv_bfloat16* pool = (const __nv_bfloat16*)p.pool;
  const size_t head_stride = (size_t)p.page_size * DH;
  const size_t page_stride = 2 * (size_t)p.n_kv_heads * head_stride;

  // queries of the tile -> shared memory (rows beyond the portion are zero)
  {
    const __nv_bfloat16* q = (const __nv_bfloat16*)p.q + (size_t)(qs + t0) * p.q_stride + h * DH;
    for (int i = threadIdx.x; i < BLOCK_Q * CHUNKS; i += blockDim.x) {
      const int r = i / CHUNKS, c = i - r * CHUNKS;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < rows) v = *reinterpret_cast<const uint4*>(q + (size_t)r * p.q_stride + c * 8);
      *reinterpret_cast<uint4*>(q_s + r * ROW + c * 8) = v;
    }
  }
  // page and place of a key: shifts when the page size is a power of two
  const int pshift = (p.page_size & (p.page_size - 1)) == 0 ? 31 - __clz(p.page_size) : -1;
  auto load_kv = [&](int kt, int buf) {
    __nv_bfloat16* kd = k_s + buf * MMA_TILE_KV * ROW;
    __nv_bfloat16* vd = v_s + buf * MMA_TILE_KV * ROW;
    for (int i = tid; i < MMA_TILE_KV * CHUNKS; i += 128) {
      const int r = i / CHUNKS, c = i - r * CHUNKS;
      const int key = kt + r;
      int page = -1;
      if (key >= kv_lo && key < kv_hi) {
        page = bt[pshift >= 0 ? key >> pshift : key / p.page_size];
        if (page < 0) atomicOr(p.status, RL_STATUS_BAD_PAGE);
      }
      if (page >= 0) {
        const __nv_bfloat16* src = pool + (size_t)page * page_stride + hkv * head_stride +
                                   (size_t)(pshift >= 0 ? key & (p.page_size - 1) : key % p.page_size) * DH + c * 8;
        cp_async16((uint32_t)__cvta_generic_to_shared(kd + r * ROW + c * 8), src);
        cp_async16((uint32_t)__cvta_generic_to_shared(vd + r * ROW + c * 8), src + p.n_kv_heads * head_stride);
      } else {
        // keys no query of the tile sees: zeros, so that 0 * value stays 0
        *reinterpret_cast<uint4*>(kd + r * ROW + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(vd + r * ROW + c * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const int kt_first = kv_lo / MMA_TILE_KV * MMA_TILE_KV;
  const int all_tiles = (kv_hi - kt_first + MMA_TILE_KV - 1) / MMA_TILE_KV;
  // this group's tiles: group, group + 2, ...; its t-th tile starts at key_of(t)
  const int n_tiles = all_tiles > group ? (all_tiles - group + MMA_GROUPS - 1) / MMA_GROUPS : 0;
  auto key_of = [&](int t) { return kt_first + (group + MMA_GROUPS * t) * MMA_TILE_KV; };
#pragma unroll
  for (int st = 0; st < MMA_STAGES - 1; ++st) {
    if (st < n_tiles) load_kv(key_of(st), st);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  __syncthreads();  // q_s is complete

  uint32_t qf[KSTEPS][4];
  {
    const int r = warp * 16 + (lane & 15);
    const int c = (lane >> 4) * 8;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
      ldmatrix_x4(qf[ks], (uint32_t)__cvta_generic_to_shared(q_s + r * ROW + ks * 16 + c));
  }
  float o[DTILES][4];
#pragma unroll
  for (int d = 0; d < DTILES; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
  const float sl2 = p.scale * 1.4426950408889634f;  // scores are kept in units of log2
  const int qpos0 = first_pos + warp * 16 + g, qpos1 = qpos0 + 8;
  const bool row0_ok = warp * 16 + g < rows, row1_ok = warp * 16 + g + 8 < rows;

  for (int t = 0; t < n_tiles; ++t) {
    const int kt = key_of(t);
    const int buf = t % MMA_STAGES;
    // the place of tile t - 1 (used, and left by every warp of the group at the last barrier)
    // takes tile t + STAGES - 1; a group is committed each time, so that the count below holds
    if (t + MMA_STAGES - 1 < n_tiles) load_kv(key_of(t + MMA_STAGES - 1), (t + MMA_STAGES - 1) % MMA_STAGES);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group %0;" ::"n"(MMA_STAGES - 1) : "memory");  // tile t has arrived
    group_sync(group);
    // a warp whose queries all lie before this tile has nothing to do in it
    const bool warp_active = kt <= first_pos + warp * 16 + 15 && warp * 16 < rows;
    if (warp_active) {
      const __nv_bfloat16* kb = k_s + buf * MMA_TILE_KV * ROW;
      const __nv_bfloat16* vb = v_s + buf * MMA_TILE_KV * ROW;
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {  // pairs of 8-key tiles
          uint32_t kf[4];
          const int r = np * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int c = ks * 16 + ((lane >> 3) & 1) * 8;
          ldmatrix_x4(kf, (uint32_t)__cvta_generic_to_shared(kb + r * ROW + c));
          mma_16816(s[2 * np], qf[ks], kf[0], kf[1]);
          mma_16816(s[2 * np + 1], qf[ks], kf[2], kf[3]);
        }
      }
      float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
      // a tile wholly before the warp's first query, inside the key range and (with a window)
      // inside the window of the warp's last query, is visible to every row: no masks needed
      const int warp_first = first_pos + warp * 16, warp_last = warp_first + 15;
      const bool all_visible = kt >= kv_lo && kt + MMA_TILE_KV - 1 <= warp_first && warp * 16 + 15 < rows &&
                               (p.window <= 0 || kt > warp_last - p.window);
      // Scores stay unscaled: with sl2 > 0 the maximum of the scaled scores is sl2 times the
      // maximum, and the scaling rides on the subtraction of the maximum (one FFMA, one ex2).
      if (!all_visible) {
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = kt + n * 8 + 2 * j + e;
            const bool in = key >= kv_lo && key < kv_hi;
            const bool v0 = in && row0_ok && key <= qpos0 && (p.window <= 0 || key > qpos0 - p.window);
            const bool v1 = in && row1_ok && key <= qpos1 && (p.window <= 0 || key > qpos1 - p.window);
            if (!v0) s[n][e] = -CUDART_INF_F;
            if (!v1) s[n][2 + e] = -CUDART_INF_F;
          }
        }
      }
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0 * sl2), mn1 = fmaxf(m1, mx1 * sl2);  // -inf * sl2 = -inf
      const float a0 = mn0 == -CUDART_INF_F ? 1.f : ex2(m0 - mn0);
      const float a1 = mn1 == -CUDART_INF_F ? 1.f : ex2(m1 - mn1);
      const float b0 = mn0 == -CUDART_INF_F ? 0.f : -mn0, b1 = mn1 == -CUDART_INF_F ? 0.f : -mn1;
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pf[4][4];  // probabilities as A fragments, 16 keys each
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const float p00 = ex2(fmaf(s[n][0], sl2, b0)), p01 = ex2(fmaf(s[n][1], sl2, b0));
        const float p10 = ex2(fmaf(s[n][2], sl2, b1)), p11 = ex2(fmaf(s[n][3], sl2, b1));
        sum0 += p00 + p01;
        sum1 += p10 + p11;
        pf[n >> 1][(n & 1) * 2] = pack_bf16(p00, p01);
        pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p10, p11);
      }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      l0 = l0 * a0 + sum0;
      l1 = l1 * a1 + sum1;
      m0 = mn0;
      m1 = mn1;
      // the output is rescaled only when some row's maximum rose (rare after the first tiles)
      if (__any_sync(0xffffffffu, a0 != 1.f || a1 != 1.f)) {
#pragma unroll
        for (int d = 0; d < DTILES; ++d) {
          o[d][0] *= a0; o[d][1] *= a0; o[d][2] *= a1; o[d][3] *= a1;
        }
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {      // 16 keys per step
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {  // pairs of 8-wide output tiles
          uint32_t vf[4];
          const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int c = dp * 16 + (lane >> 4) * 8;
          ldmatrix_x4_trans(vf, (uint32_t)__cvta_generic_to_shared(vb + r * ROW + c));
          mma_16816(o[2 * dp], pf[kk], vf[0], vf[1]);
          mma_16816(o[2 * dp + 1], pf[kk], vf[2], vf[3]);
        }
      }
    }
    group_sync(group);  // the buffer may be refilled by the next iteration's prefetch
  }
  // merge: the second group hands its running maximum, sum and output to the first through its
  // own (now idle) key buffers; thread for thread the two groups hold the same rows and columns
  if constexpr (MMA_GROUPS == 2) {
    float* x_s = reinterpret_cast<float*>(q_s + BLOCK_Q * ROW + 2 * MMA_STAGES * MMA_TILE_KV * ROW) + tid * (DTILES * 4 + 4);
    if (group == 1) {
      x_s[0] = m0; x_s[1] = m1; x_s[2] = l0; x_s[3] = l1;
#pragma unroll
      for (int d = 0; d < DTILES; ++d) {
        x_s[4 + 4 * d] = o[d][0]; x_s[5 + 4 * d] = o[d][1]; x_s[6 + 4 * d] = o[d][2]; x_s[7 + 4 * d] = o[d][3];
      }
    }
    __syncthreads();
    if (group == 1) return;
    const float pm0 = x_s[0], pm1 = x_s[1];
    const float mn0 = fmaxf(m0, pm0), mn1 = fmaxf(m1, pm1);
    const float fa0 = m0 == -CUDART_INF_F ? 0.f : exp2f(m0 - mn0), fb0 = pm0 == -CUDART_INF_F ? 0.f : exp2f(pm0 - mn0);
    const float fa1 = m1 == -CUDART_INF_F ? 0.f : exp2f(m1 - mn1), fb1 = pm1 == -CUDART_INF_F ? 0.f : exp2f(pm1 - mn1);
    l0 = l0 * fa0 + x_s[2] * fb0;
    l1 = l1 * fa1 + x_s[3] * fb1;
#pragma unroll
    for (int d = 0; d < DTILES; ++d) {
      o[d][0] = o[d][0] * fa0 + x_s[4 + 4 * d] * fb0;
      o[d][1] = o[d][1] * fa0 + x_s[5 + 4 * d] * fb0;
      o[d][2] = o[d][2] * fa1 + x_s[6 + 4 * d] * fb1;
      o[d][3] = o[d][3] * fa1 + x_s[7 + 4 * d] * fb1;
    }
  }
  __nv_bfloat16* out = (__nv_bfloat16*)p.out + (size_t)(qs + t0) * p.out_stride + h * DH;
  const float i0 = l0 > 0.f ? 1.0f / l0 : 0.f, i1 = l1 > 0.f ? 1.0f / l1 : 0.f;
#pragma unroll
  for (int d = 0; d < DTILES; ++d) {
    const int col = d * 8 + 2 * j;
    if (row0_ok)
      *reinterpret_cast<uint32_t*>(out + (size_t)(warp * 16 + g) * p.out_stride + col) =
          pack_bf16(o[d][0] * i0, o[d][1] * i0);
    if (row1_ok)
      *reinterpret_cast<uint32_t*>(out + (size_t)(warp * 16 + g + 8) * p.out_stride + col) =
          pack_bf16(o[d][2] * i1, o[d][3] * i1);
  }
}

template <int DH>
static inline void launch_mma_tiles(const AttnParams& p, const int* tiles, int n_tiles, cudaStream_t stream) {
  const size_t smem = (size_t)(MMA_TILE_Q + MMA_GROUPS * 2 * MMA_STAGES * MMA_TILE_KV) * (DH + 8) * sizeof(__nv_bfloat16);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(attn_mma_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_pdl_split(false, attn_mma_kernel<DH>, dim3(n_tiles, p.n_heads), 128 * MMA_GROUPS, smem, stream, p, tiles);
}

// Prompt portions in bfloat16 with head sizes the tensor-core kernel takes; false otherwise.
static inline bool dispatch_mma_tiles(const AttnParams& p, const int* tiles, int n_tiles, cudaStream_t stream) {
  switch (p.head_dim) {
    case 16: launch_mma_tiles<16>(p, tiles, n_tiles, stream); return true;
    case 32: launch_mma_tiles<32>(p, tiles, n_tiles, stream); return true;
    case 48: launch_mma_tiles<48>(p, tiles, n_tiles, stream); return true;
    case 64: launch_mma_tiles<64>(p, tiles, n_tiles, stream); return true;
    case 80: launch_mma_tiles<80>(p, tiles, n_tiles, stream); return true;
    case 96: launch_mma_tiles<96>(p, tiles, n_tiles, stream); return true;
    case 112: launch_mma_tiles<112>(p, tiles, n_tiles, stream); return true;
    case 128: launch_mma_tiles<128>(p, tiles, n_tiles, stream); return true;
    default: return false;
  }
}

}  // namespace rl
