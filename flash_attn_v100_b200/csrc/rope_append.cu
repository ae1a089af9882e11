// Fused rotary embedding + KV append into pages (the write side of the paged cache), sm_100a.
//
// Replaces, for one layer and one step, the reference's per-token Python loops:
//   rotary embedding   flash_attn_llm/models/rope.py:302-348 (apply_rotary_emb, half rotation,
//                      optional partial rotary) called from models/attention.py:240-255, 300-315
//   cache append       flash_attn_llm/kv_cache/manager.py:350-357 (token-by-token copies),
//                      tensor_parallel.py:285-327 (per-batch page copies), models/attention.py:322-323
//                      (torch.cat growth of a dense cache)
// One launch rotates q and k of every token and stores k / v at
// cache[block_table[seq][pos / 16], h_kv, pos % 16, :] (the layout the paged decode kernel reads).
//
// Arithmetic follows the reference operation by operation so that the result is bit-identical to
// `(x * cos) + (rotate_half(x) * sin)` evaluated by PyTorch on fp16 tensors: cos / sin are rounded to
// fp16 first (`cos.to(q.dtype)`), every product is rounded to fp16, the sum is formed in fp32 from
// the two fp16 products and rounded to fp16 once more.
//
// HBM-bound element-wise work: one thread moves one 16-byte chunk pair (x1 from the first half of
// the rotary span and x2 from the second half) of one (token, head).
#include "common.cuh"
#include "rope_append.cuh"

#include <cuda_bf16.h>

namespace fa {
namespace {

// The element type of q / k / v and of the cache: fp16, or bfloat16 for the bfloat16 twins (the same
// operation-by-operation rounding, which is what PyTorch does on bfloat16 tensors as well).
__device__ __forceinline__ float el_f(__half x) { return __half2float(x); }
__device__ __forceinline__ float el_f(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T el_from(float x);
template <> __device__ __forceinline__ __half el_from<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 el_from<__nv_bfloat16>(float x) { return __float2bfloat16(x); }

template <typename T>
__device__ __forceinline__ T rope_lo(T x1, T x2, T c, T s) {
  // first half:  x1 * cos + (-x2) * sin
  const T a = el_from<T>(el_f(x1) * el_f(c));
  const T b = el_from<T>(-el_f(x2) * el_f(s));
  return el_from<T>(el_f(a) + el_f(b));
}
template <typename T>
__device__ __forceinline__ T rope_hi(T x1, T x2, T c, T s) {
  // second half: x2 * cos + x1 * sin
  const T a = el_from<T>(el_f(x2) * el_f(c));
  const T b = el_from<T>(el_f(x1) * el_f(s));
  return el_from<T>(el_f(a) + el_f(b));
}

template <typename T>
union Chunk {
  uint4 v;
  T h[8];
  __device__ Chunk() {}
};

template <typename T>
__global__ void __launch_bounds__(256) rope_append_kernel(const RopeAppendParams p) {
  const int D = p.D, R = p.rot_dim, half_r = R / 2;
  const int chunks_rot = half_r / 8;             // chunk pairs inside the rotary span
  const int chunks_pass = (D - R) / 8;           // pass-through chunks
  const int per_head = chunks_rot + chunks_pass;
  const int heads = p.H_Q + 2 * p.H_KV;          // q heads, then k heads, then v heads
  const long long total = (long long)p.T * heads * per_head;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % per_head);
    const long long r1 = idx / per_head;
    const int hh = (int)(r1 % heads);
    const int tok = (int)(r1 / heads);

    // which tensor / head
    int kind, h;   // 0 = q, 1 = k, 2 = v
    if (hh < p.H_Q) { kind = 0; h = hh; }
    else if (hh < p.H_Q + p.H_KV) { kind = 1; h = hh - p.H_Q; }
    else { kind = 2; h = hh - p.H_Q - p.H_KV; }

    // sequence and position of this token
    int seq, pos;
    if (p.cu_seqlens != nullptr) {
      int lo = 0, hi = p.batch;                  // largest seq with cu[seq] <= tok
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(p.cu_seqlens + mid) <= tok) lo = mid; else hi = mid;
      }
      seq = lo;
      pos = tok - __ldg(p.cu_seqlens + seq) + (p.positions ? __ldg(p.positions + seq) : 0);
    } else {
      seq = tok;
      pos = __ldg(p.positions + seq);
    }

    const T* src;
    if (kind == 0) src = reinterpret_cast<const T*>(p.q) + ((long long)tok * p.H_Q + h) * D;
    else if (kind == 1) src = reinterpret_cast<const T*>(p.k) + ((long long)tok * p.H_KV + h) * D;
    else src = reinterpret_cast<const T*>(p.v) + ((long long)tok * p.H_KV + h) * D;

    // destination(s)
    T* dst_lin = nullptr;     // q_out / k_out row
    T* dst_page = nullptr;    // cache row
    if (kind == 0) dst_lin = reinterpret_cast<T*>(p.q_out) + ((long long)tok * p.H_Q + h) * D;
    else {
      if (kind == 1 && p.k_out != nullptr) dst_lin = reinterpret_cast<T*>(p.k_out) + ((long long)tok * p.H_KV + h) * D;
      if (p.k_cache != nullptr) {
        const int blk = pos >> 4;
        int page = -1;
        if (pos >= 0 && blk < p.bt_stride) page = __ldg(p.block_table + (long long)seq * p.bt_stride + blk);
        if (page >= 0 && (long long)page < p.num_pages) {
          T* base = reinterpret_cast<T*>((kind == 1) ? p.k_cache : p.v_cache);
          dst_page = base + (((long long)page * p.H_KV + h) * 16 + (pos & 15)) * D;
        } else {
          atomicOr(p.status, kStatusBadPageId);   // no slot for this token: reported, nothing written
        }
      }
    }

    if (kind == 2) {
      // v is copied unchanged.  It has D/8 chunks but only per_head index slots: slot c < chunks_rot
      // moves chunks c and c + chunks_rot, slot c >= chunks_rot moves chunk c + chunks_rot.
      if (dst_page) {
        if (c < chunks_rot) *reinterpret_cast<uint4*>(dst_page + c * 8) = *reinterpret_cast<const uint4*>(src + c * 8);
        *reinterpret_cast<uint4*>(dst_page + (c + chunks_rot) * 8) =
            *reinterpret_cast<const uint4*>(src + (c + chunks_rot) * 8);
      }
      continue;
    }
    if (c >= chunks_rot) {
      // pass-through tail of q / k (partial rotary)
      const int off = R + (c - chunks_rot) * 8;
      const uint4 a = *reinterpret_cast<const uint4*>(src + off);
      if (dst_lin) *reinterpret_cast<uint4*>(dst_lin + off) = a;
      if (dst_page) *reinterpret_cast<uint4*>(dst_page + off) = a;
      continue;
    }

    // rotary chunk pair: elements [8c, 8c+8) of the first half and of the second half
    Chunk<T> x1, x2, o1, o2;
    x1.v = *reinterpret_cast<const uint4*>(src + c * 8);
    x2.v = *reinterpret_cast<const uint4*>(src + half_r + c * 8);
    const float* cs = p.cos + (long long)tok * R + c * 8;   // cos/sin repeat over the two halves
    const float* sn = p.sin + (long long)tok * R + c * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // the reference's tables hold cat(freqs, freqs): element i of the first half and element
      // half_r + i of the second half carry the same angle, but each is cast to fp16 on its own
      const T c1 = el_from<T>(__ldg(cs + i)), s1 = el_from<T>(__ldg(sn + i));
      const T c2 = el_from<T>(__ldg(cs + half_r + i)), s2 = el_from<T>(__ldg(sn + half_r + i));
      o1.h[i] = rope_lo(x1.h[i], x2.h[i], c1, s1);
      o2.h[i] = rope_hi(x1.h[i], x2.h[i], c2, s2);
    }
    if (dst_lin) {
      *reinterpret_cast<uint4*>(dst_lin + c * 8) = o1.v;
      *reinterpret_cast<uint4*>(dst_lin + half_r + c * 8) = o2.v;
    }
    if (dst_page) {
      *reinterpret_cast<uint4*>(dst_page + c * 8) = o1.v;
      *reinterpret_cast<uint4*>(dst_page + half_r + c * 8) = o2.v;
    }
  }
}

// qkv projection output -> attention inputs.  One warp per (token, head); lane L holds D/32 consecutive
// elements, its rotary partner (the element half a head away) lives in lane L ^ 16.  The arithmetic is that
// of the per-head norm kernel followed by the rotary kernel above, value for value, so the fused launch is
// bit-identical to the two it replaces.
template <int PER, typename T>
__global__ void __launch_bounds__(256) qkv_rope_append_kernel(const QkvRopeAppendParams p) {
  const RopeAppendParams& r = p.r;
  const int D = r.D, heads = r.H_Q + 2 * r.H_KV;
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)r.T * heads) return;
  const int tok = (int)(wid / heads);
  const int hh = (int)(wid - (long long)tok * heads);
  int kind, h;   // 0 = q, 1 = k, 2 = v
  if (hh < r.H_Q) { kind = 0; h = hh; }
  else if (hh < r.H_Q + r.H_KV) { kind = 1; h = hh - r.H_Q; }
  else { kind = 2; h = hh - r.H_Q - r.H_KV; }
  const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(p.qkv) + ((long long)tok * heads + hh) * D + lane * PER;
  float f[PER];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    f[i] = __bfloat162float(src[i]);
    ss += f[i] * f[i];
  }
  const __nv_bfloat16* w = kind == 0 ? static_cast<const __nv_bfloat16*>(p.q_weight)
                         : kind == 1 ? static_cast<const __nv_bfloat16*>(p.k_weight) : nullptr;
  if (w != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / (float)D + p.eps);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const __nv_bfloat16 nb = __float2bfloat16(f[i] * inv);
      f[i] = __bfloat162float(__float2bfloat16(__bfloat162float(w[lane * PER + i]) * __bfloat162float(nb)));
    }
  }
  T x[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) x[i] = el_from<T>(f[i]);

  // sequence and cache slot of this token
  int seq, pos;
  if (r.cu_seqlens != nullptr) {
    int lo = 0, hi = r.batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (__ldg(r.cu_seqlens + mid) <= tok) lo = mid; else hi = mid;
    }
    seq = lo;
    pos = tok - __ldg(r.cu_seqlens + seq) + (r.positions ? __ldg(r.positions + seq) : 0);
  } else {
    seq = tok;
    pos = __ldg(r.positions + seq);
  }
  T* dst_page = nullptr;
  if (kind != 0 && r.k_cache != nullptr) {
    const int blk = pos >> 4;
    int page = -1;
    if (pos >= 0 && blk < r.bt_stride) page = __ldg(r.block_table + (long long)seq * r.bt_stride + blk);
    if (page >= 0 && (long long)page < r.num_pages) {
      T* base = reinterpret_cast<T*>((kind == 1) ? r.k_cache : r.v_cache);
      dst_page = base + (((long long)page * r.H_KV + h) * 16 + (pos & 15)) * D + lane * PER;
    } else if (lane == 0) {
      atomicOr(r.status, kStatusBadPageId);   // no slot for this token: reported, nothing written
    }
  }
  T o[PER];
  if (kind == 2) {
#pragma unroll
    for (int i = 0; i < PER; ++i) o[i] = x[i];
  } else {
    // rotary: first half (lanes 0-15) x1 * cos - x2 * sin, second half x2 * cos + x1 * sin, with the partner
    // element from lane ^ 16 and cos / sin at the element's own index (the tables hold cat(freqs, freqs))
    const float* cs = r.cos + (long long)tok * D + lane * PER;
    const float* sn = r.sin + (long long)tok * D + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const unsigned short mine = *reinterpret_cast<const unsigned short*>(&x[i]);
      const unsigned short got = (unsigned short)__shfl_xor_sync(0xffffffffu, (unsigned int)mine, 16);
      const T other = *reinterpret_cast<const T*>(&got);
      const T c = el_from<T>(__ldg(cs + i)), s = el_from<T>(__ldg(sn + i));
      o[i] = lane < 16 ? rope_lo(x[i], other, c, s) : rope_hi(other, x[i], c, s);
    }
  }
  T* dst_lin = nullptr;
  if (kind == 0) dst_lin = reinterpret_cast<T*>(r.q_out) + ((long long)tok * r.H_Q + h) * D + lane * PER;
  else if (kind == 1 && r.k_out != nullptr) dst_lin = reinterpret_cast<T*>(r.k_out) + ((long long)tok * r.H_KV + h) * D + lane * PER;
  else if (kind == 2 && p.v_out != nullptr) dst_lin = reinterpret_cast<T*>(p.v_out) + ((long long)tok * r.H_KV + h) * D + lane * PER;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    if (dst_lin) dst_lin[i] = o[i];
    if (dst_page) dst_page[i] = o[i];
  }
}

}  // namespace

cudaError_t launch_qkv_rope_append(const QkvRopeAppendParams& p, cudaStream_t stream) {
  const long long warps = (long long)p.r.T * (p.r.H_Q + 2 * p.r.H_KV);
  if (warps == 0) return cudaSuccess;
  const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
  if (p.r.bf16) {
    switch (p.r.D) {
      case 64: qkv_rope_append_kernel<2, __nv_bfloat16><<<blocks, 256, 0, stream>>>(p); break;
      case 128: qkv_rope_append_kernel<4, __nv_bfloat16><<<blocks, 256, 0, stream>>>(p); break;
      case 256: qkv_rope_append_kernel<8, __nv_bfloat16><<<blocks, 256, 0, stream>>>(p); break;
      default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
  }
  switch (p.r.D) {
    case 64: qkv_rope_append_kernel<2, __half><<<blocks, 256, 0, stream>>>(p); break;
    case 128: qkv_rope_append_kernel<4, __half><<<blocks, 256, 0, stream>>>(p); break;
    case 256: qkv_rope_append_kernel<8, __half><<<blocks, 256, 0, stream>>>(p); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_rope_append(const RopeAppendParams& p, int sm_count, cudaStream_t stream) {
  const int per_head = (p.rot_dim / 2) / 8 + (p.D - p.rot_dim) / 8;
  const long long total = (long long)p.T * (p.H_Q + 2 * p.H_KV) * per_head;
  if (total == 0) return cudaSuccess;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sm_count * 8;   // grid-stride loop beyond this
  if (blocks > cap) blocks = cap;
  if (p.bf16) rope_append_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(p);
  else rope_append_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fa
