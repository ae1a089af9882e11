// Launchers of the decoder block's fused row-wise operators (bf16 activations).
#pragma once
#include <cuda_runtime.h>

namespace fa {

cudaError_t launch_add_rmsnorm(void* x, const void* delta, const void* w, void* out, long long rows, int cols,
                               float eps, cudaStream_t stream);
cudaError_t launch_qk_norm_split(const void* qkv, const void* qw, const void* kw, void* q, void* k, void* v,
                                 long long T, int HQ, int HKV, int D, float eps, cudaStream_t stream);
cudaError_t launch_silu_mul(const void* gu, void* out, long long T, int I, int sm_count, cudaStream_t stream);
cudaError_t launch_half_to_bf16(const void* in, void* out, long long n, int sm_count, cudaStream_t stream);

}  // namespace fa
