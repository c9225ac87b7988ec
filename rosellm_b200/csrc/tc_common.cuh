// What the tcgen05 kernels share: barrier, TMA and MMA wrappers in inline PTX, shared-memory and
// instruction descriptors, and the host side that encodes tensor maps.
#pragma once
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

#define RL_ACT_NONE 0
#define RL_ACT_GELU_TANH 1
#define RL_ACT_GELU_ERF 2

namespace rl {
namespace tc {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bfloat16 = 128 bytes = one swizzle row

// The tanh form uses the hardware approximation (relative error about 2^-11): the result is
// stored in bfloat16, whose 8 bits of mantissa it does not touch, and a library tanhf in the
// epilogue of a product with short K costs more than the product.
__device__ __forceinline__ float act_fn(float u, int act) {
  if (act == RL_ACT_GELU_TANH) {
    const float c = 0.7978845608028654f;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(c * (u + 0.044715f * u * u * u)));
    return 0.5f * u * (1.0f + t);
  }
  if (act == RL_ACT_GELU_ERF) return 0.5f * u * (1.0f + erff(u * 0.7071067811865476f));
  return u;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Waits for the phase of `bar` with the given parity, for about two seconds at most.
// Returns false when it gave up or another thread of the block already had.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status) {
  if (mbar_try_wait(bar, parity)) return true;  // the usual case costs one instruction, no clock read
  const long long t0 = clock64();
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0xffu) == 0xffu) {
      if (*abort_flag) return false;
      if (clock64() - t0 > 4000000000LL) {
        *abort_flag = 1;
        atomicOr(status, RL_STATUS_WAIT_TIMEOUT);
        return false;
      }
    }
  }
}

// Waits for copies already issued while the block is giving up: bounded by time alone.
__device__ __forceinline__ void mbar_wait_quiet(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > 400000000LL) return;
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows 128 bytes apart, groups
// of eight rows 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;            // leading byte offset: unused with swizzled K-major tiles
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;            // descriptor version of sm_100
  d |= (uint64_t)2 << 61;            // 128-byte swizzle
  return d;
}

// Instruction descriptor of kind::f16: bfloat16 x bfloat16 -> float32, both operands K-major.
__host__ __device__ constexpr uint32_t instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Four consecutive outputs of one row: bias, activation, then store (or add into float32).
template <typename TOut>
__device__ __forceinline__ void finish4(TOut* dst, float4 v, const float* bias4, int act, int residual,
                                        bool vec_ok, int n_valid);

template <>
__device__ __forceinline__ void finish4<float>(float* dst, float4 v, const float* bias4, int act, int residual,
                                               bool vec_ok, int n_valid) {
  float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (bias4 != nullptr && i < n_valid) x[i] += bias4[i];
    x[i] = act_fn(x[i], act);
  }
  if (vec_ok && n_valid == 4) {
    float4 o = make_float4(x[0], x[1], x[2], x[3]);
    if (residual) {
      const float4 r = *reinterpret_cast<const float4*>(dst);
      o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
    }
    *reinterpret_cast<float4*>(dst) = o;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (i < n_valid) dst[i] = residual ? dst[i] + x[i] : x[i];
  }
}

template <>
__device__ __forceinline__ void finish4<__nv_bfloat16>(__nv_bfloat16* dst, float4 v, const float* bias4, int act,
                                                       int residual, bool vec_ok, int n_valid) {
  float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (bias4 != nullptr && i < n_valid) x[i] += bias4[i];
    x[i] = act_fn(x[i], act);
  }
  if (vec_ok && n_valid == 4) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]), hi = __floats2bfloat162_rn(x[2], x[3]);
    *reinterpret_cast<uint2*>(dst) =
        make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (i < n_valid) dst[i] = __float2bfloat16_rn(x[i]);
  }
}

// ---- host side: tensor maps -------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  long rows, cols, ld;
  int box_rows, box_cols, elem_bytes;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
           box_cols == o.box_cols && elem_bytes == o.elem_bytes;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h = h * 1000003u ^ std::hash<long>()(k.rows);
    h = h * 1000003u ^ std::hash<long>()(k.cols);
    h = h * 1000003u ^ std::hash<long>()(k.ld);
    h = h * 1000003u ^ (size_t)k.box_rows;
    return h * 1000003u ^ (size_t)(k.box_cols * 8 + k.elem_bytes);
  }
};

// A map of a row-major matrix [rows, cols] with row stride ld (elements), boxes of box_rows x
// box_cols, zero fill outside the matrix.  Operands: bfloat16, boxes of 64 columns = 128 bytes,
// 128-byte swizzle.  Outputs (elem_bytes 2: bfloat16, 4: float32): the swizzle is as wide as a
// box row (64 or 128 bytes).  Maps are remembered by what they describe.
inline int tensor_map(const void* ptr, long rows, long cols, long ld, int box_rows, CUtensorMap* out,
                      int box_cols = BK, int elem_bytes = 2) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex lock;
  const MapKey key{ptr, rows, cols, ld, box_rows, box_cols, elem_bytes};
  std::lock_guard<std::mutex> hold(lock);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -10;
  const int row_bytes = box_cols * elem_bytes;
  if (row_bytes != 128 && row_bytes != 64) return -11;
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)ld * (cuuint64_t)elem_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t estride[2] = {1, 1};
  CUtensorMap m;
  const CUresult rc = fn(&m, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                         const_cast<void*>(ptr), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return -11;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return 0;
}

// A tile in shared memory (rows of 64 or 128 bytes, swizzled as its map says) to global memory
// through the map: a plain store, or an addition into float32 (out += tile, one rounding an
// element, done where the data lives).  Coordinates in elements; x times the element size must
// be a multiple of 16 bytes; parts of the box outside the matrix are not written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_add_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

}  // namespace tc
}  // namespace rl
