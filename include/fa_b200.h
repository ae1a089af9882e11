/*
 * fa_b200.h — C ABI of the B200 (sm_100a) attention library.
 *
 * This is the boundary a binding of the reference project's operator module
 * (`flash_attn_v100`, built from flash_attn.cpp) would call instead of that
 * project's own CUDA wrappers.  Plain pointers and sizes only: no torch types.
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer on the CURRENT CUDA device unless it is
 *    marked "host".  The caller makes the right device current.
 *  - All tensors are dense/contiguous in the layouts given per function.
 *  - Calls are asynchronous on `stream` (a cudaStream_t passed as void*; NULL is
 *    the legacy default stream).  Nothing here synchronises the device.
 *  - No OPERATOR allocates device memory.  Split-KV decode needs scratch
 *    ("workspace"); the caller owns it, sizes it with fa_decode_workspace_bytes()
 *    and may reuse it for calls that are ordered on one stream.  Calls that can
 *    overlap on the GPU need distinct workspaces.  The one exception is the set-up
 *    of the peer-memory collectives: fa_peer_alloc calls cudaMalloc three times and
 *    synchronises the device (memory that other processes map through CUDA IPC has
 *    to come from cudaMalloc); fa_peer_free releases it.
 *  - Return value: FA_OK or a negative fa_status; fa_last_error() gives the text
 *    for the calling thread.  Invalid arguments are rejected before any launch.
 *  - fp16 tensors are IEEE binary16; softmax scale is always 1/sqrt(D)
 *    (the reference wrappers compute it themselves, flash_attn_kernel.cu:265).
 *  - GQA head map everywhere: h_kv = h_q / (H_Q / H_KV) (flash_attn_kernel.cu:1662).
 *  - Supported head dims: any multiple of 8 up to 256 (multiples of 16 for
 *    the INT8 KV cache).  Kernels are built for 64, 128 and 256 columns; a
 *    dimension in between runs on the next larger build, the missing columns read
 *    as zeros.  (The reference takes any D <= 256.)
 */
#ifndef FA_B200_H_
#define FA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum fa_status {
  FA_OK = 0,
  FA_ERR_INVALID_ARGUMENT = -1,  /* shape / size / alignment / null pointer      */
  FA_ERR_UNSUPPORTED = -2,       /* valid in the reference, not built here (D)   */
  FA_ERR_WORKSPACE = -3,         /* workspace missing or too small               */
  FA_ERR_CUDA = -4,              /* a CUDA runtime/driver call or launch failed  */
  FA_ERR_DEVICE_STATUS = -5      /* a kernel recorded a bounded-wait timeout or a
                                    page id outside the pool (fa_decode_status)   */
} fa_status;

#define FA_PAGE_SIZE 16 /* tokens per KV page; flash_attn_kernel.cu:3389 PAGE_BLOCK_SIZE */

/* Library version (major*10000 + minor*100 + patch). */
int fa_version(void);

/* Text of the last error on the calling thread ("" if none). */
const char* fa_last_error(void);

/* Bytes of scratch the decode entry points need for a batch of B sequences with
 * H_Q query heads, H_KV KV heads and head dim D on the current device.
 * Returns 0 on invalid arguments. */
size_t fa_decode_workspace_bytes(int B, int H_Q, int H_KV, int D);

/* Zero the status word and the arrival counters at the head of a workspace.  REQUIRED once
 * after allocating it, before its first use (the counters must not start from arbitrary
 * bytes); afterwards the kernels keep them consistent (every launch leaves the counters at
 * zero), whatever shapes the workspace serves.  REQUIRED again after a launch that recorded a
 * device status (fa_decode_status != 0): such a launch may have left counters mid-count.
 * workspace == NULL (workspace_bytes ignored) re-initialises the built-in scratch of
 * fa_paged_decode_gqa_f16_static_scratch, i.e. clears its status word. */
int fa_decode_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* Read back (synchronously: it waits for `stream`) the sticky device-side status
 * word of a workspace: 0 = clean; bit 0 = a bounded wait on a copy barrier ran
 * out; bit 1 = a block_table entry used by a sequence was outside [0, num_pages).
 * Results of a launch that set a bit are undefined (but no fault is raised).
 * workspace == NULL reads the status word of the built-in scratch of
 * fa_paged_decode_gqa_f16_static_scratch. */
int fa_decode_status(const void* workspace, void* stream, int* host_status_out);

/* Tuning hook for the decode kernels: consumer warps per CTA, copy-ring depth per
 * warp and persistent CTAs per SM.  0 keeps the built-in choice for that field.
 * Process-wide; values that do not fit in shared memory are reduced.  The setting is a
 * plain global read by every decode call: change it only while no other thread is inside a
 * decode entry point (it is a measurement hook, not a per-call option). */
int fa_decode_set_tuning(int warps, int stages, int ctas_per_sm);

/*
 * Paged GQA decode.  Replaces flash_attn_forward_paged_decode_gqa_fp16
 * (flash_attn_kernel.cu:3516-3584; bound at flash_attn.cpp:238).
 *   q           [B, H_Q, 1, D] fp16
 *   k_cache,
 *   v_cache     [num_pages, H_KV, 16, D] fp16
 *   block_table [B, >= pages used] int32, row stride = block_table_stride
 *               elements (the reference passes this as `max_num_blocks`,
 *               flash_attn_kernel.cu:3438); unused entries are ignored
 *   seq_lens    [B] int32: tokens to attend, token t of sequence b lives at
 *               cache[block_table[b][t/16], h_kv, t%16, :]
 *   out         [B, H_Q, 1, D] fp16 (fully overwritten; seq_len <= 0 gives zeros,
 *               where the reference divides 0/0)
 *   max_seq_len upper bound on seq_lens used to size the grid only; pass
 *               block_table_stride*16 when unknown.
 */
int fa_paged_decode_gqa_f16(const void* q, const void* k_cache, const void* v_cache, void* out,
                            const int32_t* block_table, const int32_t* seq_lens,
                            int B, int H_Q, int H_KV, int D,
                            int64_t num_pages, int block_table_stride, int64_t max_seq_len,
                            void* workspace, size_t workspace_bytes, void* stream);

/*
 * fa_paged_decode_gqa_f16 with the output stored as bfloat16 (same shape, 2 bytes per element): for
 * callers whose activations are bfloat16, such as the decoder slice of this library, which would
 * otherwise convert the fp16 result in a kernel of its own.  q and the caches stay fp16; the result is the
 * same fp32 value rounded once to bfloat16.  No counterpart in the reference (its operators return fp16).
 */
int fa_paged_decode_gqa_f16_out_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                                     const int32_t* block_table, const int32_t* seq_lens,
                                     int B, int H_Q, int H_KV, int D,
                                     int64_t num_pages, int block_table_stride, int64_t max_seq_len,
                                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * Paged GQA decode without any caller-provided scratch.  This entry point has no
 * counterpart in the reference project.
 *
 * Who it is for: code that must not, or cannot, obtain device memory at the point
 * of the call - for example a binding that runs inside a serving process whose
 * memory pool already owns the whole GPU (a later cudaMalloc would fail), or a
 * latency-critical call site where the implicit device synchronisation of
 * cudaMalloc/cudaFree is not acceptable.  Such callers have nowhere to get the
 * split-KV workspace of fa_paged_decode_gqa_f16 from.
 *
 * Same arguments, layouts and results as fa_paged_decode_gqa_f16, minus the
 * workspace.  The scratch is an 8 MiB array built into the library image: every
 * GPU that loads the library keeps those 8 MiB until the process exits.
 *  - Limit: shapes whose fa_decode_workspace_bytes(B, H_Q, H_KV, D) exceeds 8 MiB
 *    are rejected with FA_ERR_WORKSPACE (nothing is launched).  The benchmark shape
 *    (B=64, 32/8 heads, D=128) needs 4.7 MiB.
 *  - The first call on each device (of this function, or of fa_decode_status /
 *    fa_decode_workspace_init with a NULL workspace) looks up the array's device
 *    address and clears the part that must start at zero: the status word and the
 *    arrival counters of split segments (the same bytes fa_decode_workspace_init
 *    clears in a caller-owned workspace).  It waits for that clear on `stream`, so
 *    make this first call outside of any stream capture.
 *  - Nothing in this call allocates or frees device memory.
 *  - Every argument is validated before the device is touched.
 *  - All calls on a device share the one array, and it keeps whatever the previous
 *    call left in it: the counters return to "no arrivals" at the end of every launch,
 *    prefix sums and partial results are rewritten by each call before it reads them.
 *    Two calls that can overlap on the GPU - different streams without an ordering
 *    between them - race on it; order them, or give all but one of them a workspace of
 *    their own through fa_paged_decode_gqa_f16.
 *  - Device-side conditions (a bounded wait that ran out, a block_table entry outside
 *    the pool) are recorded in the array's status word like in any workspace: read it
 *    with fa_decode_status(NULL, stream, &status) and clear it with
 *    fa_decode_workspace_init(NULL, 0, stream).
 */
int fa_paged_decode_gqa_f16_static_scratch(const void* q, const void* k_cache, const void* v_cache,
                                           void* out, const int32_t* block_table,
                                           const int32_t* seq_lens, int B, int H_Q, int H_KV, int D,
                                           int64_t num_pages, int block_table_stride,
                                           int64_t max_seq_len, void* stream);

/*
 * GQA decode over a contiguous cache with one length for the whole batch.
 * Replaces flash_attn_forward_decode_gqa_fp16 / _out / _stream
 * (flash_attn_kernel.cu:1800-1861, 3639-3675; flash_attn.cpp:232-233,241) and, with
 * H_KV == H_Q, flash_attn_forward_decode_fp16 (flash_attn_kernel.cu:1863-1913).
 *   q [B,H_Q,1,D], k/v [B,H_KV,N,D], out [B,H_Q,1,D], all fp16.
 *   The query sits at position cache_len (0 <= cache_len < N); key j is visible
 *   iff !causal || j <= cache_len (flash_attn_kernel.cu:1719).
 */
int fa_decode_gqa_f16(const void* q, const void* k, const void* v, void* out,
                      int B, int H_Q, int H_KV, int N, int D, int causal, int cache_len,
                      void* workspace, size_t workspace_bytes, void* stream);

/*
 * Sliding-window decode with attention sinks over a contiguous cache.  Replaces
 * flash_attn_forward_decode_sliding_window_gqa (flash_attn_kernel.cu:4484-4535;
 * kernel :4346-4482; flash_attn.cpp:197, :251).  Layouts as fa_decode_gqa_f16.
 *   Key j (0 <= j < N) is attended when j < sink_size, or when
 *   window_start <= j <= cache_len with
 *   window_start = max(0, min(cache_len + 1, N) - window_size) (:4386-4387, :4410-4412).
 *   Only the pages that hold attended keys are read.  No bound is placed on
 *   cache_len, window_size or sink_size, as in the reference.  When no key is
 *   attended the output is zeros (the reference divides 0 by 0 there).
 *   The reference's `causal` flag has no effect on its result (:4484-4535) and
 *   is not part of this signature.
 */
int fa_decode_sliding_window_gqa_f16(const void* q, const void* k, const void* v, void* out,
                                     int B, int H_Q, int H_KV, int N, int D, int cache_len,
                                     int window_size, int sink_size,
                                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * Decode over an INT8 KV cache with one fp16 scale per cached token.  Replaces
 * flash_attn_forward_decode_int8_kv_cache_gqa (flash_attn_kernel.cu:4164-4221;
 * kernel :4020-4162; flash_attn.cpp:183, :249).
 *   q [B,H_Q,1,D] fp16; k_int8 / v_int8 [B,H_KV,N,D] int8; k_scale / v_scale
 *   [B,H_KV,N] fp16; out [B,H_Q,1,D] fp16.
 *   Every cache element is dequantised as fp16(float(int8) * float(scale)) before
 *   use (:4083-4086), bit for bit; keys j <= cache_len (j < N) are attended
 *   (:4094-4098); fp32 softmax and accumulation.  cache_len is not bounded, as
 *   in the reference; cache_len < 0 gives zeros.  Scales of tokens that are not
 *   attended are never read.
 */
int fa_decode_int8_kv_cache_gqa(const void* q, const void* k_int8, const void* v_int8,
                                const void* k_scale, const void* v_scale, void* out,
                                int B, int H_Q, int H_KV, int N, int D, int cache_len,
                                void* workspace, size_t workspace_bytes, void* stream);

/*
 * Continuous-batching decode: contiguous cache padded to max_N, one length per
 * sequence.  Replaces flash_attn_forward_continuous_batching_fp16
 * (continuous_batching_kernel.cu:338-406; flash_attn.cpp:243).
 *   cache_lens [B] int32; sequence b attends keys [0, min(cache_lens[b]+1, max_N))
 *   (continuous_batching_kernel.cu:66-69).  `causal` is accepted for signature
 *   parity and has no effect, as in the reference (no key in range exceeds the
 *   query position).  cache_lens[b] < 0 gives zeros.
 */
int fa_decode_varlen_f16(const void* q, const void* k, const void* v, void* out,
                         const int32_t* cache_lens,
                         int B, int H_Q, int H_KV, int max_N, int D, int causal,
                         void* workspace, size_t workspace_bytes, void* stream);

/*
 * INT8-QK decode.  Replaces flash_attn_forward_decode_int8_gqa
 * (flash_attn_kernel.cu:2941-3003, kernel :2796-2939; flash_attn.cpp:239).
 *   q [B,H_Q,1,D], k/v [B,H_KV,N,D] fp16; q_scale [B,H_Q] fp32;
 *   k_scale [B,H_KV,N] fp32 (one scale per cached token: README.md:169-171 of the
 *   reference; its kernel reads a single scalar per (b,h_kv) from that tensor,
 *   flash_attn_kernel.cu:2825, which this library does not reproduce).
 *   q^ = clamp(roundf(q/q_s),-127,127), k^ likewise in IEEE fp32 (round half away
 *   from zero); dot = sum q^*k^ in int32 (exact); score = float(dot)*q_s*k_s/sqrt(D);
 *   keys j > cache_len masked; fp32 softmax; fp16 V, fp32 accumulation.
 *   scores_i32_out: optional [B,H_Q,N] int32 receiving the raw int32 dots of the
 *   visible keys (others left untouched); NULL to skip.
 */
int fa_decode_int8_gqa(const void* q, const void* k, const void* v, void* out,
                       const float* q_scale, const float* k_scale,
                       int B, int H_Q, int H_KV, int N, int D, int cache_len,
                       int32_t* scores_i32_out,
                       void* workspace, size_t workspace_bytes, void* stream);

/*
 * Dense causal/non-causal GQA prefill.  Replaces flash_attn_forward_fp16
 * (flash_attn_kernel.cu:1915-1962; H_KV == H_Q) and
 * flash_attn_forward_prefill_gqa_fp16 / _out (flash_attn_kernel.cu:2740-2794;
 * flash_attn.cpp:226,235-236).
 *   q [B,H_Q,N,D], k/v [B,H_KV,N,D], out [B,H_Q,N,D], all fp16.
 */
int fa_prefill_dense_f16(const void* q, const void* k, const void* v, void* out,
                         int B, int H_Q, int H_KV, int N, int D, int causal, void* stream);

/*
 * Packed variable-length GQA prefill.  Replaces
 * flash_attn_forward_varlen_prefill_fp16 / _stream (flash_attn_kernel.cu:3354-3387,
 * 3677-3712; flash_attn.cpp:240,242).  The reference requires H_KV == H_Q
 * (flash_attn_kernel.cu:217); this entry point also accepts H_Q % H_KV == 0.
 *   q [total,H_Q,D], k/v [total,H_KV,D], out [total,H_Q,D] fp16;
 *   cu_seqlens [batch+1] int32 (device), non-decreasing, cu_seqlens[0] == 0,
 *   cu_seqlens[batch] <= total; max_seqlen > 0 bounds the longest sequence (it
 *   sizes the grid; rows of longer sequences beyond it are not computed, as in the
 *   reference).  Rows not covered by any sequence are left untouched.
 */
int fa_prefill_varlen_f16(const void* q, const void* k, const void* v, void* out,
                          const int32_t* cu_seqlens, int batch, int64_t total,
                          int H_Q, int H_KV, int D, int max_seqlen, int causal, void* stream);
/* fa_prefill_varlen_f16 with the output stored as bfloat16 (see fa_paged_decode_gqa_f16_out_bf16). */
int fa_prefill_varlen_f16_out_bf16(const void* q, const void* k, const void* v, void* out,
                          const int32_t* cu_seqlens, int batch, int64_t total,
                          int H_Q, int H_KV, int D, int max_seqlen, int causal, void* stream);

/*
 * Fused rotary embedding + KV append into pages: the write side of the paged cache for one
 * layer and one step.  Replaces the reference's rotary embedding
 * (flash_attn_llm/models/rope.py:302-348, half rotation, optional partial rotary) followed by
 * its per-token cache copies (flash_attn_llm/kv_cache/manager.py:350-357,
 * tensor_parallel.py:285-327, models/attention.py:322-323).
 *   q [T,H_Q,D], k/v [T,H_KV,D] fp16 (T tokens); cos/sin [T,rot_dim] fp32 exactly as the
 *   reference computes them (cat(freqs,freqs).cos()); q_out [T,H_Q,D]; k_out optional [T,H_KV,D].
 *   Results are bit-identical to the reference's fp16 PyTorch expression
 *   (x*cos) + (rotate_half(x)*sin) with cos/sin cast to fp16.
 *   Token placement: without cu_seqlens, token i is the new token of sequence i at slot
 *   positions[i] (T == batch, a decode step); with cu_seqlens [batch+1] the tokens are packed
 *   prompts and token j of sequence s goes to slot positions[s] + j (positions may be NULL = 0).
 *   k (rotated) and v are stored at cache[block_table[s][slot/16], h_kv, slot%16, :];
 *   k_cache/v_cache may both be NULL (rotation only).  A token without a valid page sets bit 1
 *   of the status word read by fa_prefill_status and is not stored.
 */
int fa_rope_append_paged_f16(const void* q, const void* k, const void* v, const float* cos,
                             const float* sin, void* q_out, void* k_out, void* k_cache, void* v_cache,
                             const int32_t* block_table, const int32_t* positions,
                             const int32_t* cu_seqlens, int T, int batch, int H_Q, int H_KV, int D,
                             int rot_dim, int64_t num_pages, int block_table_stride, void* stream);

/*
 * Fused row-wise operators of the decoder block around the attention operators (bf16 activations).
 * They replace chains of PyTorch element-wise kernels in the reference's model code.
 *
 * fa_add_rmsnorm_bf16: x [rows, cols] bf16; if delta != NULL, x += delta (written back: the residual
 *   stream, flash_attn_llm/models/decoder_layer.py:69-85); out = RMSNorm(x) * weight with fp32
 *   statistics, the normalised value cast to bf16 before the multiplication by the weight
 *   (flash_attn_llm/models/norm.py:25-33).
 * fa_qk_norm_split_f16: qkv [T, (H_Q + 2*H_KV) * D] bf16 (q heads, k heads, v heads) -> q [T,H_Q,D],
 *   k [T,H_KV,D], v [T,H_KV,D] fp16 (the dtype of the attention operators), with the per-head RMSNorm
 *   of Qwen3-style attention on q and k (flash_attn_llm/models/attention.py:96-102, 230-233); NULL
 *   weights skip the norm.
 * fa_silu_mul_bf16: gate_up [T, 2*I] bf16 (gate, then up) -> out [T, I] = silu(gate) * up
 *   (flash_attn_llm/models/mlp.py:27).
 * fa_half_to_bf16: fp16 -> bf16 copy of n elements (attention output back to the bf16 stream).
 */
int fa_add_rmsnorm_bf16(void* x, const void* delta, const void* weight, void* out, int64_t rows,
                        int cols, float eps, void* stream);
int fa_qk_norm_split_f16(const void* qkv, const void* q_weight, const void* k_weight, void* q,
                         void* k, void* v, int64_t T, int H_Q, int H_KV, int D, float eps,
                         void* stream);
/* fa_qk_norm_split_f16 and fa_rope_append_paged_f16 (full rotary, rot_dim == D) in one launch, value
 * for value the same arithmetic: qkv [T, (H_Q + 2 H_KV) * D] bf16 -> per-head RMSNorm of q and k (weights may
 * be NULL) -> fp16 -> rotary embedding -> q_out [T,H_Q,D]; k and v go to the paged cache (when given) and,
 * optionally, to k_out / v_out [T,H_KV,D] (the packed prefill attention reads those).  cos / sin [T, D] fp32;
 * positions / cu_seqlens / block_table as in fa_rope_append_paged_f16. */
int fa_qkv_rope_append_f16(const void* qkv, const void* q_weight, const void* k_weight, const float* cos,
                           const float* sin, void* q_out, void* k_out, void* v_out, void* k_cache,
                           void* v_cache, const int32_t* block_table, const int32_t* positions,
                           const int32_t* cu_seqlens, int T, int batch, int H_Q, int H_KV, int D, float eps,
                           int64_t num_pages, int block_table_stride, void* stream);

/* ---------------------------------------------------------------------------
 * bfloat16 twins: the same operators for q / k / v, caches and outputs that hold
 * bfloat16 instead of fp16 (a model whose activations are bfloat16 keeps its
 * range; the reference's operators are fp16 only).  Same arguments, shapes and
 * error behaviour as the _f16 functions they are named after.  The score and
 * output MMAs take bfloat16 operands (P is rounded to bfloat16 before P V), all
 * accumulation, softmax and merging stay fp32.  fa_prefill_*_bf16 run on the
 * tcgen05 kernel (head dimension up to 128; FA_ERR_UNSUPPORTED above).
 * fa_rope_append_paged_bf16 / fa_qkv_rope_append_bf16 round cos / sin, each
 * product and the sum to bfloat16, as PyTorch does for
 * (x * cos) + (rotate_half(x) * sin) on bfloat16 tensors.
 * -------------------------------------------------------------------------- */
int fa_paged_decode_gqa_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                             const int32_t* block_table, const int32_t* seq_lens,
                             int B, int H_Q, int H_KV, int D,
                             int64_t num_pages, int block_table_stride, int64_t max_seq_len,
                             void* workspace, size_t workspace_bytes, void* stream);
int fa_decode_gqa_bf16(const void* q, const void* k, const void* v, void* out,
                       int B, int H_Q, int H_KV, int N, int D, int causal, int cache_len,
                       void* workspace, size_t workspace_bytes, void* stream);
int fa_prefill_dense_bf16(const void* q, const void* k, const void* v, void* out,
                          int B, int H_Q, int H_KV, int N, int D, int causal, void* stream);
int fa_prefill_varlen_bf16(const void* q, const void* k, const void* v, void* out,
                           const int32_t* cu_seqlens, int batch, int64_t total,
                           int H_Q, int H_KV, int D, int max_seqlen, int causal, void* stream);
int fa_rope_append_paged_bf16(const void* q, const void* k, const void* v, const float* cos,
                              const float* sin, void* q_out, void* k_out, void* k_cache, void* v_cache,
                              const int32_t* block_table, const int32_t* positions,
                              const int32_t* cu_seqlens, int T, int batch, int H_Q, int H_KV, int D,
                              int rot_dim, int64_t num_pages, int block_table_stride, void* stream);
int fa_qkv_rope_append_bf16(const void* qkv, const void* q_weight, const void* k_weight, const float* cos,
                            const float* sin, void* q_out, void* k_out, void* v_out, void* k_cache,
                            void* v_cache, const int32_t* block_table, const int32_t* positions,
                            const int32_t* cu_seqlens, int T, int batch, int H_Q, int H_KV, int D, float eps,
                            int64_t num_pages, int block_table_stride, void* stream);

int fa_silu_mul_bf16(const void* gate_up, void* out, int64_t T, int I, void* stream);
int fa_half_to_bf16(const void* in, void* out, int64_t n, void* stream);

/* Kernel choice for the prefill entry points: 0 = automatic (tcgen05 kernel for
 * D = 64/128, mma.sync kernel otherwise), 1 = always the mma.sync kernel, 2 = require
 * the tcgen05 kernel, 3 = tcgen05 kernel with every fourth pair of exp2 evaluated as a
 * polynomial on the FMA pipes.  Process-wide, a plain global like fa_decode_set_tuning: meant
 * for tests and measurements, not to be changed while another thread launches a prefill. */
int fa_prefill_set_impl(int impl);

/* Read back (synchronously on `stream`) the sticky status word of the prefill kernels
 * on the current device: 0 = clean, bit 0 = a bounded wait ran out (results of that
 * launch are undefined, no fault is raised).  `clear` != 0 resets it afterwards. */
int fa_prefill_status(void* stream, int* host_status_out, int clear);

/* --------------------------------------------------------------------------
 * Peer-memory collectives of the tensor-parallel decode step (one process per
 * GPU of one NVLink domain, at most 8 ranks).  They stand where the reference
 * calls dist.all_reduce / dist.all_gather (flash_attn_llm/parallel/
 * tensor_parallel.py:152-190; its single-process peer all-reduce export is
 * cross_gpu_allreduce_fp16, flash_attn.cpp:206, :252), as single kernels on
 * plain peer loads and stores that can be recorded into a CUDA graph.
 *
 * fa_peer_alloc: allocate this rank's data buffer (data_bytes, zeroed), flag
 *   array and local state, and return CUDA IPC handles (64 bytes each) of the
 *   first two for the other ranks.  fa_peer_open maps another rank's handle.
 *   All ranks must allocate the same data_bytes and make the same sequence of
 *   collective calls.
 * fa_peer_allreduce_sum_bf16: in-place sum of n_elems bf16 values at
 *   offset_bytes of every rank's data buffer (n_elems a multiple of 8 * world);
 *   each element is reduced in fp32, in rank order, by one rank and stored to
 *   all: the result is bit-identical on every rank.
 * fa_peer_allreduce_add_rmsnorm_bf16: the all-reduce of a row-parallel GEMM
 *   output together with the residual add and the RMS norm that follow it in a
 *   decoder block (decoder_layer.py:69-85, norm.py:7-34 of the reference's model
 *   code).  Three [rows, cols] bf16 regions of the data buffers, at the same
 *   offsets on every rank:  delta = bf16(sum over ranks of part);
 *   x = bf16(x + delta);  h = rmsnorm(x, eps) * weight.  x and h end up
 *   identical on every rank; part is left as it was.  rows a multiple of world,
 *   cols a multiple of 8 (<= 16384), weight [cols] bf16 in local memory.  The
 *   results are bit-identical to fa_peer_allreduce_sum_bf16 followed by
 *   fa_add_rmsnorm_bf16.
 * fa_peer_allgather: rank r's chunk_bytes at `src` (local memory) are stored
 *   at offset_bytes + r * chunk_bytes of every rank's data buffer.
 * data_ptrs / flag_ptrs: host arrays of `world` device pointers in rank order
 *   (own buffers at index `rank`).  Every wait for another rank is bounded;
 *   fa_peer_status reports a wait that ran out (FA_ERR_DEVICE_STATUS).
 * -------------------------------------------------------------------------- */
int fa_peer_alloc(size_t data_bytes, void** data, void** flags, void** state,
                  void* data_handle, void* flags_handle);
int fa_peer_open(const void* handle, void** ptr);
int fa_peer_close(void* ptr);
int fa_peer_free(void* data, void* flags, void* state);
int fa_peer_allreduce_sum_bf16(void* const* data_ptrs, void* const* flag_ptrs, void* state,
                               int rank, int world, int64_t offset_bytes, int64_t n_elems,
                               void* stream);
int fa_peer_allreduce_add_rmsnorm_bf16(void* const* data_ptrs, void* const* flag_ptrs, void* state,
                                       int rank, int world, int64_t part_offset_bytes,
                                       int64_t x_offset_bytes, int64_t h_offset_bytes, int64_t rows,
                                       int cols, const void* weight, float eps, void* stream);
int fa_peer_allgather(void* const* data_ptrs, void* const* flag_ptrs, void* state,
                      int rank, int world, const void* src, int64_t offset_bytes,
                      int64_t chunk_bytes, void* stream);
int fa_peer_status(const void* state, void* stream, int* host_status_out);
/* Way back from a wait that ran out.  The status word is sticky, and a rank that ran a collective
 * without its peers has advanced its epoch and stamped the peers' flags, so later collectives on the
 * same buffers would keep mismatching.  fa_peer_reset zeroes this rank's flag array and local state
 * (epoch, ticket, status) and waits for that on `stream`.  ALL ranks must call it, with no collective
 * in flight, between two host-side barriers (after the first nobody launches, after the second
 * everybody may again).  The alternative is to free the buffers and allocate new ones. */
int fa_peer_reset(void* flags, void* state, void* stream);
/* Bound of every wait for another rank, in polls of at least 100 ns (default 2^26;
 * applies to launches made after the call). */
int fa_peer_set_max_polls(unsigned int max_polls);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H_ */
