// Fused rotary embedding + KV append into pages: parameter block and launcher.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fa {

struct RopeAppendParams {
  const __half* q;            // [T, H_Q, D]
  const __half* k;            // [T, H_KV, D]
  const __half* v;            // [T, H_KV, D]
  const float* cos;           // [T, rot_dim] fp32 (angles repeat over the two halves)
  const float* sin;           // [T, rot_dim]
  __half* q_out;              // [T, H_Q, D] rotated queries
  __half* k_out;              // optional [T, H_KV, D] rotated keys (prefill attention reads them)
  __half* k_cache;            // optional [pages, H_KV, 16, D]
  __half* v_cache;
  const int32_t* block_table; // [batch, bt_stride]
  const int32_t* positions;   // decode: slot of the new token per sequence; packed: first slot per sequence (or null = 0)
  const int32_t* cu_seqlens;  // null: token i belongs to sequence i (T == batch); else packed [batch + 1]
  int32_t* status;            // sticky status word (page id outside the pool / no slot)
  int T, batch, H_Q, H_KV, D, rot_dim, bt_stride;
  long long num_pages;
  int bf16;                   // q / k / v, the outputs and the cache are bfloat16 instead of fp16
};

cudaError_t launch_rope_append(const RopeAppendParams& p, int sm_count, cudaStream_t stream);

// The decoder block's projection output to attention inputs in one launch: per-head RMSNorm of q and k
// (weights may be null), cast to fp16, full rotary embedding, k / v appended to the pages.
struct QkvRopeAppendParams {
  const void* qkv;            // [T, (H_Q + 2 H_KV) * D] bf16: q heads, then k heads, then v heads
  const void* q_weight;       // [D] bf16 or null
  const void* k_weight;       // [D] bf16 or null
  float eps;
  __half* v_out;              // optional [T, H_KV, D] fp16 copy of v (prefill attention reads it)
  RopeAppendParams r;         // cos, sin, q_out, k_out, caches, tables, sizes (q / k / v unused; rot_dim == D)
};
cudaError_t launch_qkv_rope_append(const QkvRopeAppendParams& p, cudaStream_t stream);

}  // namespace fa
