// Split-KV GQA decode: parameter block and launcher shared by the C-ABI entry points.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fa {

enum DecodeMode : int {
  kModePaged = 0,         // len = max(lens[b], 0); rows found through block_table
  kModeContigVarlen = 1,  // len = clamp(lens[b] + 1, 0, N); rows contiguous per (b, h_kv)
  kModeContigFixed = 2,   // len = fixed_len for every sequence; rows contiguous
};

enum DecodeKind : int {
  kKindF16 = 0,     // fp16 cache, fp16 arithmetic
  kKindInt8QK = 1,  // fp16 cache; Q and K quantised in the kernel, integer score dot products
  kKindInt8KV = 2,  // int8 cache with one fp16 scale per token, dequantised in the kernel
  kKindBF16 = 3,    // bfloat16 q and cache, bfloat16 MMAs (P rounded to bfloat16), bfloat16 output
};

struct DecodeParams {
  const __half* q;             // [B, H_Q, 1, D] (bfloat16 bits for kKindBF16, like the cache behind the tensor maps)
  __half* out;                 // [B, H_Q, 1, D]: fp16, or bfloat16 bits when out_bf16 is set
  int out_bf16;
  const int32_t* block_table;  // paged only
  const int32_t* lens;         // seq_lens / cache_lens, null in fixed mode
  const float* q_scale;        // int8 only: [B, H_Q]
  const float* k_scale;        // int8 only: [B, H_KV, N]
  int32_t* scores_out;         // int8 only, optional: [B, H_Q, N]
  const __half* k_scale_h;     // int8 cache only: [B, H_KV, N] fp16
  const __half* v_scale_h;     // int8 cache only: [B, H_KV, N] fp16
  int32_t* prefix;             // workspace: [B + 1] running page counts
  float* partials;             // workspace: [n_cta][2][slot_rows][D + 2]
  unsigned long long* counters;  // workspace: [kMaxDecodeCtas] arrivals (low word), one per split segment,
                                 // indexed by the first CTA that works on the segment; zero between launches
  int32_t* status;             // workspace: sticky status word
  int B, H_Q, H_KV, G;         // G = H_Q / H_KV
  int D_real;                  // head dimension of the tensors (<= the padded one the kernel is built for)
  int n_gblk;                  // ceil(G / 16): query-head blocks per KV head
  int HV;                      // H_KV * n_gblk
  int mode, fixed_len, N;      // N: tokens per (b, h_kv) row in contiguous modes
  // Sliding window + attention sink (contiguous fixed mode only): visible tokens are [0, sink) and
  // [win_start, fixed_len).  The pages of a sequence are the sink pages followed by the window pages:
  // unit page i maps to page i for i < sink_pages, else to win_first_page + (i - sink_pages).
  // Without a window: sink = 0, win_start = 0, sink_pages = INT_MAX (identity map).
  int sink, win_start, sink_pages, win_first_page, window_pages_total;
  int bt_stride;
  long long num_pages;
  int n_cta, stages, slot_rows;
  float scale;                 // 1 / sqrt(D)
  float scale_log2;            // scale * log2(e)
};

struct DecodeLaunchConfig {
  int warps;        // consumer warps per CTA
  int stages;       // TMA ring depth per warp
  int ctas_per_sm;  // persistent CTAs per SM
};

// Workspace layout helpers (host).
size_t decode_workspace_bytes(int B, int H_Q, int H_KV, int D, int max_ctas);
// Workspace layout: [status 256 B][arrival counters][prefix sums][partials].  The status word and the
// counters are at fixed offsets and are zeroed when the workspace is initialised; the counters are only
// ever written by the decode kernels (which leave them at "no arrivals"), so a launch never mistakes
// stale bytes of another region for arrivals, whatever shapes the workspace served before.
constexpr int kMaxDecodeCtas = 148 * 4 * 2;  // bound on the persistent grid, sizes the counters and partials
constexpr size_t kWsStatusOffset = 0;        // int32 status word (+ padding to 256 B)
constexpr size_t kWsCountersOffset = 256;    // u64 counters[kMaxDecodeCtas]
constexpr size_t kWsPrefixOffset = kWsCountersOffset + (((size_t)kMaxDecodeCtas * 8 + 255) & ~(size_t)255);  // int32 prefix[B + 1]
constexpr size_t kWsInitBytes = kWsPrefixOffset;   // what fa_decode_workspace_init zeroes

// Launch the decode on `stream` (one kernel; a prefix-sum pre-pass only when B is too large for
// the in-kernel scan).  kmap/vmap are 2-D tensor maps over
// K and V seen as [rows, D] fp16 with a 64-column x 16-row box and 128-byte swizzle; for the int8
// cache, [rows, D] bytes with a min(D, 128)-column x 16-row box (128-byte swizzle, none for D = 64).
cudaError_t launch_decode(const CUtensorMap& kmap, const CUtensorMap& vmap, const DecodeParams& p,
                          int D, int kind, int warps, size_t smem_bytes, cudaStream_t stream);

size_t decode_smem_bytes(int D, int warps, int stages, int slot_rows, int B, int kv_elem_bytes);

}  // namespace fa
