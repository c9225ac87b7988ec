// rl_attention_decode_noalloc: the split decode attention with its scratch inside the library.
// What it is for, its limits and its rules are in attention_noalloc.h.
#include <mutex>

#include "attention_kernels.cuh"
#include "attention_noalloc.h"

// The scratch of every call on this device: partial outputs first, then (max, sum) pairs.
// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float rl_noalloc_scratch[RL_NOALLOC_SCRATCH_FLOATS];

namespace {

constexpr int kMaxDevices = 64;
float* g_scratch[kMaxDevices] = {};
std::mutex g_setup_lock;

// The device address of the scratch on the current device, looked up once per device.
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return RL_NOALLOC_SETUP_FAILED;
  std::lock_guard<std::mutex> hold(g_setup_lock);
  if (g_scratch[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, rl_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return RL_NOALLOC_SETUP_FAILED;
    g_scratch[dev] = (float*)p;
  }
  *out = g_scratch[dev];
  return 0;
}

}  // namespace

RL_EXPORT int rl_attention_decode_noalloc(int dtype, const void* q, long q_stride,
                                          const void* pool, const int* block_table, int bt_stride,
                                          const int* q_start, const int* kv_len, const int* slots,
                                          void* out, long out_stride, int n_heads, int n_kv_heads,
                                          int head_dim, int page_size, int window, float scale,
                                          const int* decode_reqs, int n_decode, int n_splits,
                                          int* status, cudaStream_t stream) {
  if (n_decode <= 0) return 0;
  if (head_dim % 16 != 0 || head_dim <= 0 || head_dim > 256) return RL_NOALLOC_BAD_HEAD_DIM;
  if (n_kv_heads <= 0 || n_heads <= 0 || n_heads % n_kv_heads != 0) return RL_NOALLOC_BAD_HEADS;
  if (n_splits < 1 || n_splits > RL_NOALLOC_MAX_SPLITS) return RL_NOALLOC_BAD_SPLITS;
  if (status == nullptr) return RL_NOALLOC_NO_STATUS;
  const long long rows = (long long)n_decode * n_heads * n_splits;
  // one split writes its result straight to out: no scratch is used, so none is asked for
  if (n_splits > 1 && rows * (head_dim + 2) > (long long)RL_NOALLOC_SCRATCH_FLOATS) return RL_NOALLOC_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  float* part_o = scratch;
  float* part_ml = scratch + (n_splits > 1 ? rows * head_dim : 0);
  // old_keys_settled = 0: a caller from outside the engine may have written the cache just
  // before this call; the kernel reads nothing before its wait for the kernels ahead
  rl::AttnParams p{q, q_stride, pool, block_table, bt_stride, q_start, kv_len, slots, out,
                   out_stride, n_heads, n_kv_heads, head_dim, page_size, window, scale, status, 0};
  int launched;
  if (dtype == RL_F32)
    launched = rl::dispatch_attention<float>(p, nullptr, 0, decode_reqs, n_decode, n_splits, false, part_o, part_ml, stream);
  else if (dtype == RL_BF16)
    launched = rl::dispatch_attention<__nv_bfloat16>(p, nullptr, 0, decode_reqs, n_decode, n_splits, false, part_o, part_ml, stream);
  else
    return RL_NOALLOC_SETUP_FAILED;
  if (launched != 0) return launched;
  RL_CHECK_LAUNCH();
  return 0;
}

RL_EXPORT const char* rl_attention_decode_noalloc_error(int code) {
  switch (code) {
    case 0: return "no error";
    case RL_NOALLOC_BAD_HEAD_DIM: return "head_dim must be a multiple of 16 between 16 and 256";
    case RL_NOALLOC_BAD_HEADS: return "n_heads must be a positive multiple of n_kv_heads";
    case RL_NOALLOC_BAD_SPLITS: return "n_splits must be between 1 and 65535 (it is a grid dimension)";
    case RL_NOALLOC_NO_STATUS:
      return "status must point to an int on the device: the kernels record a missing page there instead of "
             "reading through it";
    case RL_NOALLOC_TOO_LARGE:
      return "n_decode * n_heads * n_splits * (head_dim + 2) exceeds the library's scratch of "
             "1048576 floats; use fewer splits or rl_attention with scratch of your own";
    case RL_NOALLOC_SETUP_FAILED:
      return "the scratch array's device address could not be obtained, or the element type is unknown";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error code";
  }
}
