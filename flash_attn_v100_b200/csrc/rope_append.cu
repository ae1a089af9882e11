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

namespace fa {
namespace {

__device__ __forceinline__ __half rope_lo(__half x1, __half x2, __half c, __half s) {
  // first half:  x1 * cos + (-x2) * sin
  const __half a = __float2half_rn(__half2float(x1) * __half2float(c));
  const __half b = __float2half_rn(-__half2float(x2) * __half2float(s));
  return __float2half_rn(__half2float(a) + __half2float(b));
}
__device__ __forceinline__ __half rope_hi(__half x1, __half x2, __half c, __half s) {
  // second half: x2 * cos + x1 * sin
  const __half a = __float2half_rn(__half2float(x2) * __half2float(c));
  const __half b = __float2half_rn(__half2float(x1) * __half2float(s));
  return __float2half_rn(__half2float(a) + __half2float(b));
}

union Chunk {
  uint4 v;
  __half h[8];
};

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

    const __half* src;
    if (kind == 0) src = p.q + ((long long)tok * p.H_Q + h) * D;
    else if (kind == 1) src = p.k + ((long long)tok * p.H_KV + h) * D;
    else src = p.v + ((long long)tok * p.H_KV + h) * D;

    // destination(s)
    __half* dst_lin = nullptr;     // q_out / k_out row
    __half* dst_page = nullptr;    // cache row
    if (kind == 0) dst_lin = p.q_out + ((long long)tok * p.H_Q + h) * D;
    else {
      if (kind == 1 && p.k_out != nullptr) dst_lin = p.k_out + ((long long)tok * p.H_KV + h) * D;
      if (p.k_cache != nullptr) {
        const int blk = pos >> 4;
        int page = -1;
        if (pos >= 0 && blk < p.bt_stride) page = __ldg(p.block_table + (long long)seq * p.bt_stride + blk);
        if (page >= 0 && (long long)page < p.num_pages) {
          __half* base = (kind == 1) ? p.k_cache : p.v_cache;
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
    Chunk x1, x2, o1, o2;
    x1.v = *reinterpret_cast<const uint4*>(src + c * 8);
    x2.v = *reinterpret_cast<const uint4*>(src + half_r + c * 8);
    const float* cs = p.cos + (long long)tok * R + c * 8;   // cos/sin repeat over the two halves
    const float* sn = p.sin + (long long)tok * R + c * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // the reference's tables hold cat(freqs, freqs): element i of the first half and element
      // half_r + i of the second half carry the same angle, but each is cast to fp16 on its own
      const __half c1 = __float2half_rn(__ldg(cs + i)), s1 = __float2half_rn(__ldg(sn + i));
      const __half c2 = __float2half_rn(__ldg(cs + half_r + i)), s2 = __float2half_rn(__ldg(sn + half_r + i));
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

}  // namespace

cudaError_t launch_rope_append(const RopeAppendParams& p, int sm_count, cudaStream_t stream) {
  const int per_head = (p.rot_dim / 2) / 8 + (p.D - p.rot_dim) / 8;
  const long long total = (long long)p.T * (p.H_Q + 2 * p.H_KV) * per_head;
  if (total == 0) return cudaSuccess;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sm_count * 8;   // grid-stride loop beyond this
  if (blocks > cap) blocks = cap;
  rope_append_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fa
