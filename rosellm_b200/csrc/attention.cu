// C entry points of the paged attention and of the cache write; the kernels are in
// attention_kernels.cuh.
#include "attention_mma.cuh"
#include "attention_tc.cuh"

// head_dim: a multiple of 16, at most 256.  tiles: [n_tiles][2] = (request, first query of the
// tile within the request's portion); tiles_wide: the same for 64-query tiles, which the
// tensor-core kernel takes (bfloat16, head_dim <= 128; other cases use `tiles`).
// decode_reqs: requests with a single query; decode_wide: their blocks have sixteen warps
// instead of four (few requests: a block then covers 256 keys a round).  With
// n_splits > 1, part_o holds n_decode*heads*n_splits*head_dim floats and part_ml
// n_decode*heads*n_splits*2.  n_tokens: rows of q; n_pages: pages of the pool (both bound the
// TMA tensor maps of the tcgen05 kernel).
//
// old_keys_settled: the decode kernel is launched with programmatic dependent launch and, when
// this is nonzero, fetches the batch description, the block table and the keys and values at
// positions below kv_len - 1 BEFORE it waits for the kernels ahead of it on the stream.  Pass
// nonzero only if all of those were written by work that had completed before the kernel
// preceding this call on the stream started (inside the engine they are of earlier steps, and
// every step begins with a copy to the device, which separates the steps' kernels).  A caller
// that writes several positions of the cache and attends over them back to back on one stream
// passes 0: the kernel then reads nothing before its wait.
RL_EXPORT int rl_attention(int dtype, const void* q, long q_stride, const void* pool,
                           const int* block_table, int bt_stride, const int* q_start,
                           const int* kv_len, const int* slots, void* out, long out_stride,
                           int n_heads, int n_kv_heads, int head_dim, int page_size, int window,
                           float scale, const int* tiles, int n_tiles, const int* tiles_wide,
                           int n_tiles_wide, const int* decode_reqs,
                           int n_decode, int n_splits, int decode_wide, float* part_o, float* part_ml,
                           int n_tokens, long n_pages, int prefill_path, int old_keys_settled, int* status,
                           cudaStream_t stream) {
  if (head_dim % 16 != 0 || head_dim <= 0 || head_dim > 256) return -2;
  if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return -3;
  if (n_splits < 1 || n_splits > 65535 || (n_splits > 1 && (part_o == nullptr || part_ml == nullptr))) return -4;
  if (status == nullptr) return -6;
  rl::AttnParams p{q, q_stride, pool, block_table, bt_stride, q_start, kv_len, slots, out,
                   out_stride, n_heads, n_kv_heads, head_dim, page_size, window, scale, status, old_keys_settled};
  int rc;
  if (dtype == RL_F32)
    rc = rl::dispatch_attention<float>(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, decode_wide != 0, part_o, part_ml, stream);
  else {
    // prompt portions: tcgen05 where its sizes fit (prefill_path 0: as fits, 1: mma.sync, 2: tcgen05
    // or refuse), else mma.sync, else (head sizes above 128) the CUDA-core tiles below
    if (n_tiles_wide > 0 && tiles_wide != nullptr) {
      bool done = false;
      if (prefill_path != 1 && rl::tc::attn_tc_fits(p) && n_tokens > 0 && n_pages > 0)
        done = rl::tc::launch_attn_tc(p, tiles_wide, n_tiles_wide, n_tokens, n_pages, stream) == 0;
      if (!done && prefill_path == 2) return -5;
      if (!done) done = rl::dispatch_mma_tiles(p, tiles_wide, n_tiles_wide, stream);
      if (done) n_tiles = 0;  // the prompt portions are done
    }
    rc = rl::dispatch_attention<__nv_bfloat16>(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, decode_wide != 0, part_o, part_ml, stream);
  }
  if (rc != 0) return rc;
  RL_CHECK_LAUNCH();
  return 0;
}

RL_EXPORT int rl_kv_write(int dtype, const void* k, const void* v, long stride, void* pool,
                          const int* block_table, int bt_stride, const int* positions,
                          const int* req_of_token, const int* slots, int n_tokens, int n_kv_heads,
                          int head_dim, int page_size, int max_pos, int* status,
                          cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (head_dim % 16 != 0 || stride % 8 != 0) return -2;
  if (dtype == RL_F32)
    rl::launch_pdl(rl::kv_write_kernel<float>, n_tokens, 128, 0, stream, (const float*)k, (const float*)v,
                   stride, (float*)pool, block_table, bt_stride, positions, req_of_token, slots, n_tokens,
                   n_kv_heads, head_dim, page_size, max_pos, status);
  else
    rl::launch_pdl(rl::kv_write_kernel<__nv_bfloat16>, n_tokens, 128, 0, stream, (const __nv_bfloat16*)k,
                   (const __nv_bfloat16*)v, stride, (__nv_bfloat16*)pool, block_table, bt_stride, positions,
                   req_of_token, slots, n_tokens, n_kv_heads, head_dim, page_size, max_pos, status);
  RL_CHECK_LAUNCH();
  return 0;
}

RL_PHASE_READER(rl_attention_phase_times)
