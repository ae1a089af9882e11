// Tiled GQA prefill on mma.sync tensor cores (dense [B,H,N,D] and packed varlen).
//
// Replaces the reference's one-thread-per-query-row prefill kernels
// (flash_attn_kernel.cu:1138-1299, 2471-2605, 3005-3148).  This is the general
// path (any supported D, any length); the tcgen05 kernel in prefill_tc5.cu takes
// the D = 128 / D = 64 cases when it is enabled.
//
// One CTA = BM query rows of one (sequence, query head); each warp owns 16 rows.
// K/V tiles of 64 keys are double-buffered in shared memory with cp.async and an
// XOR swizzle on 16-byte chunks; S = Q K^T and O += P V use m16n8k16 with fp32
// accumulation; softmax is fp32, base 2, online.  Causal tiles above the diagonal
// are skipped; only the diagonal and the ragged last tile are masked per element.
#include "common.cuh"
#include "prefill.cuh"

namespace fa {
namespace {

constexpr int BN = 64;

template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  // byte offset of a 16-byte chunk in a [rows][D] fp16 tile
  return (uint32_t)(row * (D * 2) + (((chunk & ~7) | ((chunk & 7) ^ (row & 7))) << 4));
}

template <int D, int ROWS, int THREADS>
__device__ __forceinline__ void load_tile(uint32_t smem_base, const __half* gbase, long long tok_stride,
                                          int row0, int row_limit, int real_chunks, int tid) {
  // rows [row0, row0 + ROWS) of a sequence; rows >= row_limit and 16-byte chunks >= real_chunks (columns
  // past the tensors' head dimension) are zero-filled
  constexpr int CH = D / 8;
#pragma unroll
  for (int i = tid; i < ROWS * CH; i += THREADS) {
    const int r = i / CH, c = i - r * CH;
    const bool ok = (row0 + r) < row_limit && c < real_chunks;
    const __half* src = gbase + (long long)(ok ? (row0 + r) : 0) * tok_stride + (ok ? c : 0) * 8;
    cp_async_16(smem_base + swz<D>(r, c), src, ok);
  }
}

template <int D, int BM>
__global__ void __launch_bounds__(BM * 2) prefill_mma_kernel(const PrefillParams p) {
  constexpr int THREADS = BM * 2;
  constexpr int NT_S = BN / 8;   // score n-tiles per warp row block
  constexpr int NT_O = D / 8;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const uint32_t sQ = smem_u32(smem_raw);
  const uint32_t sK0 = sQ + BM * D * 2;
  const uint32_t sV0 = sK0 + 2 * BN * D * 2;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, cq = (lane & 3) * 2;
  const int m_block = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal tiles first
  const int h_q = blockIdx.y, seq = blockIdx.z;
  const int h_kv = h_q / (p.H_Q / p.H_KV);

  long long tok0;
  int len;
  if (p.cu_seqlens != nullptr) {
    const int a = __ldg(p.cu_seqlens + seq), e = __ldg(p.cu_seqlens + seq + 1);
    tok0 = a;
    len = e - a;
    if ((long long)e > p.total) len = (int)(p.total - a);
  } else {
    tok0 = 0;
    len = p.N;
  }
  if (len > p.max_seqlen) len = p.max_seqlen;
  const int q0 = m_block * BM;
  if (q0 >= len) return;

  const __half* qg = p.q + seq * p.q_batch_stride + (long long)h_q * p.q_head_stride + tok0 * p.q_tok_stride;
  const __half* kg = p.k + seq * p.kv_batch_stride + (long long)h_kv * p.kv_head_stride + tok0 * p.kv_tok_stride;
  const __half* vg = p.v + seq * p.kv_batch_stride + (long long)h_kv * p.kv_head_stride + tok0 * p.kv_tok_stride;
  __half* og = p.out + seq * p.q_batch_stride + (long long)h_q * p.q_head_stride + tok0 * p.q_tok_stride;

  const int kv_end = p.causal ? ((q0 + BM) < len ? (q0 + BM) : len) : len;
  const int n_tiles = (kv_end + BN - 1) / BN;

  const int real_chunks = p.D_real >> 3;
  load_tile<D, BM, THREADS>(sQ, qg, p.q_tok_stride, q0, len, real_chunks, tid);
  load_tile<D, BN, THREADS>(sK0, kg, p.kv_tok_stride, 0, len, real_chunks, tid);
  load_tile<D, BN, THREADS>(sV0, vg, p.kv_tok_stride, 0, len, real_chunks, tid);
  cp_async_commit();

  float acc[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int qrow0 = q0 + warp * 16 + g;  // this lane's rows: qrow0 and qrow0 + 8

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < n_tiles) {
      load_tile<D, BN, THREADS>(sK0 + (buf ^ 1) * BN * D * 2, kg, p.kv_tok_stride, (t + 1) * BN, len, real_chunks, tid);
      load_tile<D, BN, THREADS>(sV0 + (buf ^ 1) * BN * D * 2, vg, p.kv_tok_stride, (t + 1) * BN, len, real_chunks, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    const uint32_t sK = sK0 + buf * BN * D * 2, sV = sV0 + buf * BN * D * 2;
    const int k0 = t * BN;
    // warp-level skip: under causal masking a warp whose rows all precede the tile has no work
    const bool warp_active = !p.causal || (k0 <= q0 + warp * 16 + 15);
    if (warp_active) {
      float s[NT_S][4];
#pragma unroll
      for (int j = 0; j < NT_S; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t qa[4];
        {
          // A fragment: matrices (rows 0-7,k lo) (rows 8-15,k lo) (rows 0-7,k hi) (rows 8-15,k hi)
          const int mi = lane >> 3;
          const int r = warp * 16 + (lane & 7) + (mi & 1) * 8;
          ldmatrix_x4(qa, sQ + swz<D>(r, 2 * kk + (mi >> 1)));
        }
#pragma unroll
        for (int jp = 0; jp < NT_S / 2; ++jp) {
          const int mi = lane >> 3;
          const int r = jp * 16 + (lane & 7) + (mi >> 1) * 8;
          uint32_t kb[4];
          ldmatrix_x4(kb, sK + swz<D>(r, 2 * kk + (mi & 1)));
          mma_f16_16816(s[2 * jp], qa, kb[0], kb[1]);
          mma_f16_16816(s[2 * jp + 1], qa, kb[2], kb[3]);
        }
      }
      const bool need_mask = (k0 + BN > len) || (p.causal && (k0 + BN - 1 > q0 + warp * 16));
#pragma unroll
      for (int j = 0; j < NT_S; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x = s[j][e] * p.scale_log2;
          if (need_mask) {
            const int kj = k0 + j * 8 + cq + (e & 1);
            const int qi = qrow0 + (e >> 1) * 8;
            if (kj >= len || (p.causal && kj > qi)) x = -INFINITY;
          }
          s[j][e] = x;
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int j = 0; j < NT_S; ++j) {
        mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
        mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      // a row with nothing visible yet (only rows past the end of the sequence) keeps m = -inf
      const float ms0 = (mn0 == -INFINITY) ? 0.f : mn0, ms1 = (mn1 == -INFINITY) ? 0.f : mn1;
      const float a0 = fast_exp2(m0 - ms0), a1 = fast_exp2(m1 - ms1);
      m0 = mn0;
      m1 = mn1;
      float r0 = 0.f, r1 = 0.f;
      uint32_t pa[NT_S / 2][4];
#pragma unroll
      for (int j = 0; j < NT_S; ++j) {
        const float p0 = fast_exp2(s[j][0] - ms0), p1 = fast_exp2(s[j][1] - ms0);
        const float p2 = fast_exp2(s[j][2] - ms1), p3 = fast_exp2(s[j][3] - ms1);
        r0 += p0 + p1;
        r1 += p2 + p3;
        pa[j >> 1][(j & 1) * 2 + 0] = pack_half2(p0, p1);
        pa[j >> 1][(j & 1) * 2 + 1] = pack_half2(p2, p3);
      }
      l0 = l0 * a0 + r0;
      l1 = l1 * a1 + r1;
#pragma unroll
      for (int i = 0; i < NT_O; ++i) {
        acc[i][0] *= a0;
        acc[i][1] *= a0;
        acc[i][2] *= a1;
        acc[i][3] *= a1;
      }
#pragma unroll
      for (int ks = 0; ks < BN / 16; ++ks) {
#pragma unroll
        for (int c2 = 0; c2 < D / 16; ++c2) {
          const int mi = lane >> 3;
          const int r = ks * 16 + (lane & 7) + (mi & 1) * 8;
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, sV + swz<D>(r, 2 * c2 + (mi >> 1)));
          mma_f16_16816(acc[2 * c2], pa[ks], vb[0], vb[1]);
          mma_f16_16816(acc[2 * c2 + 1], pa[ks], vb[2], vb[3]);
        }
      }
    }
    __syncthreads();
  }

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  if (qrow0 < len) {
    __half* o = og + (long long)qrow0 * p.q_tok_stride;
#pragma unroll
    for (int i = 0; i < NT_O; ++i)
      if (i * 8 < p.D_real)
        *reinterpret_cast<uint32_t*>(o + i * 8 + cq) = pack_out16x2(acc[i][0] * inv0, acc[i][1] * inv0, p.out_bf16 != 0);
  }
  if (qrow0 + 8 < len) {
    __half* o = og + (long long)(qrow0 + 8) * p.q_tok_stride;
#pragma unroll
    for (int i = 0; i < NT_O; ++i)
      if (i * 8 < p.D_real)
        *reinterpret_cast<uint32_t*>(o + i * 8 + cq) = pack_out16x2(acc[i][2] * inv1, acc[i][3] * inv1, p.out_bf16 != 0);
  }
}

template <int D, int BM>
cudaError_t launch_mma_t(const PrefillParams& p, cudaStream_t stream) {
  auto kern = prefill_mma_kernel<D, BM>;
  const size_t smem = (size_t)BM * D * 2 + 4 * (size_t)BN * D * 2;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int max_len = p.cu_seqlens ? p.max_seqlen : p.N;
  dim3 grid((max_len + BM - 1) / BM, p.H_Q, p.batch);
  kern<<<grid, BM * 2, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_prefill_mma(const PrefillParams& p, int D, cudaStream_t stream) {
  switch (D) {
    case 64: return launch_mma_t<64, 128>(p, stream);
    case 128: return launch_mma_t<128, 128>(p, stream);
    case 256: return launch_mma_t<256, 64>(p, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace fa
