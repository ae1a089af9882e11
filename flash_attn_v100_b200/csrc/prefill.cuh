// Prefill parameter block shared by the prefill kernels and the C-ABI layer.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fa {

struct PrefillParams {
  const __half* q;
  const __half* k;
  const __half* v;
  __half* out;                // fp16, or bfloat16 bits when out_bf16 is set
  int out_bf16;
  int in_bf16;                // q, k, v are bfloat16 (tcgen05 kernel only: bfloat16 MMAs, P rounded to bfloat16)
  const int32_t* cu_seqlens;  // null => dense [B,H,N,D]; else packed [total,H,D]
  int batch;                  // sequences (dense: B)
  int H_Q, H_KV;
  int N;                      // dense sequence length (unused when packed)
  int max_seqlen;             // packed: grid bound; dense: N
  long long total;            // packed: rows in q/k/v
  long long q_batch_stride, q_head_stride, q_tok_stride;     // elements
  long long kv_batch_stride, kv_head_stride, kv_tok_stride;  // elements
  int causal;
  int D_real;                 // head dimension of the tensors; the kernels are built for 64 / 128 / 256 columns
                              // and take the columns [D_real, D) as zeros
  float scale_log2;           // log2(e) / sqrt(D_real)
};

cudaError_t launch_prefill_mma(const PrefillParams& p, int D, cudaStream_t stream);

// tcgen05 / TMEM kernel (D = 64 or 128).  `encode_fn` is cuTensorMapEncodeTiled.
bool prefill_tc5_supported(const PrefillParams& p, int D);
cudaError_t launch_prefill_tc5(const PrefillParams& p, int D, void* encode_fn, cudaStream_t stream);
void prefill_tc5_set_poly(bool on);
cudaError_t prefill_status(int* host_out, cudaStream_t stream);
cudaError_t prefill_status_ptr(int** out);  // device address of the status word (current device)
cudaError_t prefill_status_clear(cudaStream_t stream);

}  // namespace fa
