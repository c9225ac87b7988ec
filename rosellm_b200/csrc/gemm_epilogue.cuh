// Epilogues shared by the matrix kernels: activation, store or accumulation into the float32
// residual stream, and the scatter of key / value columns into cache pages.
#pragma once
#include "common.cuh"
#include "gemm_vec.cuh"

#define RL_ACT_NONE 0
#define RL_ACT_GELU_TANH 1
#define RL_ACT_GELU_ERF 2

namespace rl {

__device__ __forceinline__ float apply_act(float u, int act) {
  if (act == RL_ACT_GELU_TANH) {
    const float c = 0.7978845608028654f;  // sqrt(2/pi)
    return 0.5f * u * (1.0f + tanhf(c * (u + 0.044715f * u * u * u)));
  }
  if (act == RL_ACT_GELU_ERF) return 0.5f * u * (1.0f + erff(u * 0.7071067811865476f));
  return u;
}

template <typename TOut>
__device__ __forceinline__ void store_out(TOut* out, size_t idx, float v, int residual) {
  out[idx] = from_f32<TOut>(v);
}
template <>
__device__ __forceinline__ void store_out<float>(float* out, size_t idx, float v, int residual) {
  out[idx] = residual ? out[idx] + v : v;
}

// Output columns from q_width on are keys, then values, of kv heads: instead of the output
// buffer they go to the page of the row's position (pool == nullptr: off).  The reference
// appends keys and values in a kernel of its own (rosellm/roseinfer/kv_append_triton.py:28-165)
// or inside its decode attention (rosellm/rosetrainer/paged_attention.py:179-204).
struct KvScatter {
  void* pool;
  const int* block_table;
  int bt_stride;
  const int* positions;
  const int* req_of_token;
  const int* slots;
  int q_width, kv_width, head_dim, page_size, n_kv_heads, max_pos;
  int* status;
};

// The next token of every row chosen in the epilogue instead of the row's logits being written
// (out_ids == nullptr: off): what sample_kernel would choose from the same logits, the arg-max of
// logit (temperature <= 0) or of logit / temperature + the entry's Gumbel noise.  Whoever holds
// some columns of a row (a warp of the weight-streaming kernel its eight, a lane of the tcgen05
// epilogue those of its tile) offers the best of them to best[row] (ordered bits of the score
// above, the complement of the index below, so that the largest word is the largest score and
// among equals the lowest index) by an atomic maximum, which it skips when the word there is
// already larger; the warp or block that ends last, known by a ticket, turns the words into
// token ids and zeroes words and ticket for the next launch.  The reference's greedy path is an
// arg-max over logits it has written (rosellm/roseinfer/engine.py:1117-1118).
struct SampleArgs {
  int* out_ids;
  const float* temperature;  // per row; nullptr: every row takes the arg-max
  const long long* seeds;
  const int* counters;
  unsigned long long* best;  // [M], zero between launches
  int* ticket;               // zero between launches
  // Optionally the ids also go to the host without a copy of their own: host_ring is pinned host
  // memory that the device can write, RING slots of ring_stride ids; *ring_step (device memory)
  // counts the launches that have written, and names the slot of this one (the host counts along).
  int* host_ring;
  int ring_stride;
  unsigned int* ring_step;
};
constexpr unsigned int SAMPLE_RING = 4;

// What the warp does that took the last ticket (all 32 lanes): best words into token ids, words
// and ticket back to zero for the next launch.
__device__ __forceinline__ void sample_finish(const SampleArgs& s, int M, int lane) {
  __threadfence();
  const unsigned int slot = s.ring_step != nullptr ? (*s.ring_step % SAMPLE_RING) : 0u;
  for (int m = lane; m < M; m += 32) {
    const int id = (int)~(uint32_t)__ldcg(s.best + m);
    s.out_ids[m] = id;
    if (s.host_ring != nullptr) s.host_ring[(size_t)slot * s.ring_stride + m] = id;
    s.best[m] = 0ull;
  }
  __syncwarp();
  if (lane == 0) {
    *s.ticket = 0;
    if (s.ring_step != nullptr) *s.ring_step += 1u;
  }
}

template <typename T>
__device__ __forceinline__ bool scatter_kv(const KvScatter& kv, int m, int n, float v) {
  if (kv.pool == nullptr || n < kv.q_width) return false;
  const int c = n - kv.q_width;
  const int which = c / kv.kv_width;
  const int r = c - which * kv.kv_width;
  const int head = r / kv.head_dim, d = r - head * kv.head_dim;
  const int slot = kv.slots[kv.req_of_token[m]];
  if (slot < 0) return true;  // padding row of a fixed-size batch
  const int pos = kv.positions[m];
  if (pos < 0 || pos >= kv.max_pos) {
    atomicOr(kv.status, RL_STATUS_BAD_POSITION);
    return true;
  }
  const int page = kv.block_table[(size_t)slot * kv.bt_stride + pos / kv.page_size];
  if (page < 0) {
    atomicOr(kv.status, RL_STATUS_BAD_PAGE);
    return true;
  }
  T* dst = (T*)kv.pool +
           ((((size_t)page * 2 + which) * kv.n_kv_heads + head) * kv.page_size + pos % kv.page_size) * kv.head_dim + d;
  *dst = from_f32<T>(v);
  return true;
}

}  // namespace rl
