// Shared helpers of the sm_100a kernels: element types, conversions, reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_set>

// Element type codes of the C interface.
#define RL_F32 0
#define RL_BF16 1

// Status bits a kernel ORs into the status word when its inputs are wrong.
// A kernel that sets one skips the access; it never traps.
#define RL_STATUS_BAD_TOKEN 1      // token id outside the table
#define RL_STATUS_BAD_POSITION 2   // position outside the table or the sequence limit
#define RL_STATUS_BAD_PAGE 4       // block table holds no page where one is read or written
#define RL_STATUS_WAIT_TIMEOUT 8   // a bounded wait on a barrier gave up

#define RL_EXPORT extern "C" __attribute__((visibility("default")))

// The entry points return the error of their own launches: every launch of the library notes a
// failure here (per host thread) and clears it from the CUDA runtime, so that it is neither left
// for a later, unrelated call to find nor mixed up with an error somebody else left behind.
namespace rl {
inline thread_local int launch_error_noted = 0;
inline cudaError_t note_launch(cudaError_t e) {
  if (e != cudaSuccess) {
    if (launch_error_noted == 0) launch_error_noted = (int)e;
    cudaGetLastError();  // a refused launch leaves its (non-sticky) error pending: take it back
  }
  return e;
}
inline int take_launch_error() {
  const int e = launch_error_noted;
  launch_error_noted = 0;
  return e;
}
}  // namespace rl

#define RL_CHECK_LAUNCH()                                   \
  do {                                                      \
    const int e__ = rl::take_launch_error();                \
    if (e__ != 0) return e__;                               \
  } while (0)

// Clock stamps of the phases of a kernel, compiled in with -DRL_PHASE_TIMING only (measurement
// builds): thread 0 (RL_PHASE_OF: a named thread) of one block notes clock64() at each mark, in an array of the source file
// that marks; RL_PHASE_READER(name) defines the exported function that reads them back (all
// zero in ordinary builds).
#ifdef RL_PHASE_TIMING
namespace rl {
static __device__ long long phase_clock[32];
}
#define RL_PHASE(i)                                                                      \
  do {                                                                                   \
    if (blockIdx.x == 5 % gridDim.x && threadIdx.x == 0) rl::phase_clock[i] = clock64(); \
  } while (0)
#define RL_PHASE_OF(i, thread)                                                                  \
  do {                                                                                          \
    if (blockIdx.x == 5 % gridDim.x && threadIdx.x == (thread)) rl::phase_clock[i] = clock64(); \
  } while (0)
#define RL_PHASE_READER(name)                                                          \
  RL_EXPORT int name(long long* out, int n) {                                          \
    if (n < 0 || n > 32) return -2;                                                    \
    return (int)cudaMemcpyFromSymbol(out, rl::phase_clock, sizeof(long long) * n);     \
  }
#else
#define RL_PHASE_OF(i, thread) \
  do {                         \
  } while (0)
#define RL_PHASE(i) \
  do {              \
  } while (0)
#define RL_PHASE_READER(name)                 \
  RL_EXPORT int name(long long* out, int n) { \
    if (n < 0 || n > 32) return -2;           \
    for (int i = 0; i < n; ++i) out[i] = 0;   \
    return 0;                                 \
  }
#endif

namespace rl {

// Programmatic dependent launch.  Every kernel of this library is launched with the
// "programmatic stream serialization" attribute and begins with pdl_begin(): it lets the
// next kernel of the stream start launching at once, then waits until the kernels before it
// have completed and their writes are visible.  Launch latency and prologues (barrier set-up,
// tensor-memory allocation, index arithmetic) thus overlap the tail of the previous kernel.
//
// What a kernel may read before its wait.  Kernel N starts once every block of kernel N-1 has
// passed its launch_dependents, which is at N-1's top: so N's part before the wait can run
// beside the body of N-1, and, N-1 itself having started that early, beside N-2 and earlier
// kernels.  Before its wait a kernel therefore reads only memory that no kernel of the same
// sequence of launches writes: weights and norm scales, the step's description (copied to the
// device before the step's first kernel; a copy is a full barrier between launches), and,
// where the caller has said so (AttnParams::old_keys_settled), keys and values of earlier
// steps.  Everything else is read after the wait.  Kernels that use pdl_begin() read nothing
// before it.
__device__ __forceinline__ void pdl_begin() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// The split of an SM's on-chip memory between L1 and shared memory is a property of the
// running kernel; where two kernels that follow one another want different splits, the SM
// has to run empty in between, which costs a decode step about two microseconds per change.
// So every kernel launched here with little shared memory asks for the same split (half);
// kernels that need more get what they need.
constexpr int RL_CARVEOUT_PERCENT = 50;
constexpr size_t RL_CARVEOUT_UP_TO = 96 * 1024;  // dynamic shared memory up to which the common split is asked for

inline void prefer_common_carveout(const void* kernel) {
  static std::mutex lock;
  static std::unordered_set<const void*> done;
  std::lock_guard<std::mutex> hold(lock);
  if (done.insert(kernel).second) {
    note_launch(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, RL_CARVEOUT_PERCENT));
  }
}

// common_split: ask for the common L1/shared-memory split (kernels that run for tens of
// microseconds and gain from more shared memory may keep the split the driver picks for them).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_split(bool common_split, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args... args) {
  if (common_split && smem <= RL_CARVEOUT_UP_TO) prefer_common_carveout((const void*)kernel);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return note_launch(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  return launch_pdl_split(true, kernel, grid, block, smem, stream, args...);
}

// Thread-block clusters: rank of this block, the barrier of all threads of the cluster, and
// the address of a shared-memory location in another block of the cluster.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_addr(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

}  // namespace rl
