// Small fused element-wise / row-wise operators of the decoder block (bf16 activations), sm_100a.
//
// These replace chains of PyTorch element-wise kernels around the attention operators in the
// reference's model code: RMSNorm (flash_attn_llm/models/norm.py:7-34: fp32 statistics, cast back,
// times weight), the residual adds of the decoder layer (models/decoder_layer.py:69-85), the per-head
// QK RMSNorm of Qwen3-style attention (models/attention.py:96-102, 230-233) and SwiGLU
// (models/mlp.py:11-28).  All are HBM-bound: one pass over the data, 16-byte accesses.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "engine_ops.cuh"

namespace fa {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

union Bf8 {
  uint4 v;
  __nv_bfloat16 h[8];
};
union Hf8 {
  uint4 v;
  __half h[8];
};

// x [rows, cols] (+= delta if given, written back), out = rmsnorm(x) * w.  One CTA per row.
// cols is a multiple of 8 and at most 8 * 8 * blockDim (each thread keeps up to 8 chunks).
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(__nv_bfloat16* x, const __nv_bfloat16* delta,
                                                         const __nv_bfloat16* w, __nv_bfloat16* out, int cols,
                                                         float eps) {
  __shared__ float red[8];
  const long long row = blockIdx.x;
  __nv_bfloat16* xr = x + row * cols;
  const __nv_bfloat16* dr = delta ? delta + row * cols : nullptr;
  const int nchunk = cols / 8;
  Bf8 keep[8];
  float ss = 0.f;
  int n = 0;
  for (int c = threadIdx.x; c < nchunk; c += blockDim.x, ++n) {
    Bf8 a;
    a.v = *reinterpret_cast<const uint4*>(xr + c * 8);
    if (dr) {
      Bf8 d;
      d.v = *reinterpret_cast<const uint4*>(dr + c * 8);
#pragma unroll
      for (int i = 0; i < 8; ++i) a.h[i] = __float2bfloat16(__bfloat162float(a.h[i]) + __bfloat162float(d.h[i]));
      *reinterpret_cast<uint4*>(xr + c * 8) = a.v;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float f = __bfloat162float(a.h[i]);
      ss += f * f;
    }
    keep[n] = a;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)cols + eps);
  n = 0;
  for (int c = threadIdx.x; c < nchunk; c += blockDim.x, ++n) {
    Bf8 wv, o;
    wv.v = *reinterpret_cast<const uint4*>(w + c * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // normalise in fp32, cast to bf16, then multiply by the weight (norm.py:28-33)
      const __nv_bfloat16 nb = __float2bfloat16(__bfloat162float(keep[n].h[i]) * inv);
      o.h[i] = __float2bfloat16(__bfloat162float(wv.h[i]) * __bfloat162float(nb));
    }
    *reinterpret_cast<uint4*>(out + row * cols + c * 8) = o.v;
  }
}

// qkv [T, (HQ + 2*HKV) * D] bf16 -> q [T,HQ,D], k [T,HKV,D], v [T,HKV,D] fp16, with per-head RMSNorm
// (weights qw / kw [D], may be null = no norm) on q and k.  One warp per (token, head); D in {64,128,256}.
__global__ void __launch_bounds__(256) qk_norm_split_kernel(const __nv_bfloat16* qkv, const __nv_bfloat16* qw,
                                                           const __nv_bfloat16* kw, __half* q, __half* k, __half* v,
                                                           long long T, int HQ, int HKV, int D, float eps) {
  const int heads = HQ + 2 * HKV;
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= T * heads) return;
  const long long tok = wid / heads;
  const int hh = (int)(wid - tok * heads);
  const __nv_bfloat16* src = qkv + (tok * heads + hh) * D;
  const int per_lane = D / 32;   // 2, 4 or 8 elements
  float f[8];
  float ss = 0.f;
  for (int i = 0; i < per_lane; ++i) {
    f[i] = __bfloat162float(src[lane * per_lane + i]);
    ss += f[i] * f[i];
  }
  __half* dst;
  const __nv_bfloat16* w = nullptr;
  if (hh < HQ) { dst = q + (tok * HQ + hh) * D; w = qw; }
  else if (hh < HQ + HKV) { dst = k + (tok * HKV + (hh - HQ)) * D; w = kw; }
  else { dst = v + (tok * HKV + (hh - HQ - HKV)) * D; }
  if (w != nullptr) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)D + eps);
    for (int i = 0; i < per_lane; ++i) {
      const __nv_bfloat16 nb = __float2bfloat16(f[i] * inv);
      f[i] = __bfloat162float(__float2bfloat16(__bfloat162float(w[lane * per_lane + i]) * __bfloat162float(nb)));
    }
  }
  for (int i = 0; i < per_lane; ++i) dst[lane * per_lane + i] = __float2half_rn(f[i]);
}

// gu [T, 2*I] bf16 (gate then up) -> out [T, I] = silu(gate) * up
__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16* gu, __nv_bfloat16* out, long long T, int I) {
  const int chunks = I / 8;
  const long long total = T * chunks;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / chunks;
    const int c = (int)(idx - t * chunks);
    Bf8 g, u, o;
    g.v = *reinterpret_cast<const uint4*>(gu + t * 2 * I + c * 8);
    u.v = *reinterpret_cast<const uint4*>(gu + t * 2 * I + I + c * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float gf = __bfloat162float(g.h[i]);
      const __nv_bfloat16 s = __float2bfloat16(gf / (1.f + __expf(-gf)));   // silu in fp32, rounded to bf16
      o.h[i] = __float2bfloat16(__bfloat162float(s) * __bfloat162float(u.h[i]));
    }
    *reinterpret_cast<uint4*>(out + t * I + c * 8) = o.v;
  }
}

// fp16 [n] -> bf16 [n]
__global__ void __launch_bounds__(256) half_to_bf16_kernel(const __half* in, __nv_bfloat16* out, long long n8) {
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n8;
       idx += (long long)gridDim.x * blockDim.x) {
    Hf8 a;
    Bf8 o;
    a.v = *reinterpret_cast<const uint4*>(in + idx * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) o.h[i] = __float2bfloat16(__half2float(a.h[i]));
    *reinterpret_cast<uint4*>(out + idx * 8) = o.v;
  }
}

unsigned grid_for(long long threads, int sm_count) {
  long long blocks = (threads + 255) / 256;
  const long long cap = (long long)sm_count * 16;
  if (blocks > cap) blocks = cap;
  return (unsigned)(blocks < 1 ? 1 : blocks);
}

}  // namespace

cudaError_t launch_add_rmsnorm(void* x, const void* delta, const void* w, void* out, long long rows, int cols,
                               float eps, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  add_rmsnorm_kernel<<<(unsigned)rows, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(x),
                                                          static_cast<const __nv_bfloat16*>(delta),
                                                          static_cast<const __nv_bfloat16*>(w),
                                                          static_cast<__nv_bfloat16*>(out), cols, eps);
  return cudaGetLastError();
}

cudaError_t launch_qk_norm_split(const void* qkv, const void* qw, const void* kw, void* q, void* k, void* v,
                                 long long T, int HQ, int HKV, int D, float eps, cudaStream_t stream) {
  if (T == 0) return cudaSuccess;
  const long long warps = T * (HQ + 2 * HKV);
  const long long blocks = (warps * 32 + 255) / 256;
  qk_norm_split_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(qw),
      static_cast<const __nv_bfloat16*>(kw), static_cast<__half*>(q), static_cast<__half*>(k),
      static_cast<__half*>(v), T, HQ, HKV, D, eps);
  return cudaGetLastError();
}

cudaError_t launch_silu_mul(const void* gu, void* out, long long T, int I, int sm_count, cudaStream_t stream) {
  if (T == 0) return cudaSuccess;
  silu_mul_kernel<<<grid_for(T * (I / 8), sm_count), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(gu),
                                                                      static_cast<__nv_bfloat16*>(out), T, I);
  return cudaGetLastError();
}

cudaError_t launch_half_to_bf16(const void* in, void* out, long long n, int sm_count, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  half_to_bf16_kernel<<<grid_for(n / 8, sm_count), 256, 0, stream>>>(static_cast<const __half*>(in),
                                                                    static_cast<__nv_bfloat16*>(out), n / 8);
  return cudaGetLastError();
}

}  // namespace fa
