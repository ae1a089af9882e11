// Collectives of the tensor-parallel decode step over NVLink peer memory (one process per GPU).
//
// Every rank owns one data buffer and one flag array, allocated with cudaMalloc and opened by the
// other ranks through CUDA IPC handles; a kernel gets the `world` data pointers and flag pointers
// of all ranks.  Both collectives are single kernels on plain peer loads and stores (no multicast),
// synchronised by per-CTA flags with system-scope release / acquire, so they can be recorded into a
// CUDA graph together with the compute of the step: flags carry an epoch that every launch takes
// from, and advances in, device memory.
//
// all-reduce (sum, bf16, in place in the data buffers), two barriers and one pass:
//   barrier A   every rank's input is complete (its kernel has started)
//   reduce      rank r sums slice r of all `world` buffers in fp32, in rank order, and stores the
//               bf16 result into slice r of EVERY buffer: each element is reduced by exactly one
//               rank, so all ranks end up with bit-identical results
//   barrier B   all slices of my buffer have been written
// all-gather (bytes): barrier A, every rank stores its chunk into slot `rank` of every buffer,
// barrier B.
//
// Every flag wait is bounded; a wait that runs out sets a sticky status word, after which all
// waits of that rank return at once (results are then undefined, the kernels still terminate).
#include "peer_collectives.cuh"

#include <cuda_bf16.h>

namespace fa {

namespace {


__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Flag of (phase, cta, source rank) inside a rank's flag array.
__device__ __forceinline__ int flag_index(int phase, int cta, int src) {
  return (phase * kPeerMaxCtas + cta) * kPeerMaxWorld + src;
}

// Threads 0 .. world-1 of the CTA: tell rank `tid` that this CTA of `rank` reached `phase` in epoch e,
// then wait for the same from rank `tid`.  All threads: CTA barrier on both sides.
__device__ __forceinline__ void peer_barrier(const PeerPointers& pp, int rank, int world, int phase, uint32_t e,
                                             int32_t* status, unsigned int max_polls) {
  __syncthreads();
  const int tid = threadIdx.x;
  if (tid < world) {
    // The release store at system scope orders this CTA's earlier stores before the flag: the other threads'
    // stores were made visible to this thread by the CTA barrier above, and a release is cumulative over them.
    st_release_sys(pp.flags[tid] + flag_index(phase, blockIdx.x, rank), e);
    const uint32_t* mine = pp.flags[rank] + flag_index(phase, blockIdx.x, tid);
    bool ok = false;
    if (*reinterpret_cast<volatile int32_t*>(status) == 0) {
      for (unsigned int i = 0; i < max_polls; ++i) {
        if (ld_acquire_sys(mine) == e) { ok = true; break; }
        if (i >= 64u) __nanosleep(100);   // the peers are usually within a few microseconds: spin first
      }
    }
    if (!ok) atomicOr(status, kPeerStatusTimeout);
  }
  __syncthreads();
}

__device__ __forceinline__ uint32_t begin_epoch(const PeerState& s) {
  __shared__ uint32_t e_s;
  if (threadIdx.x == 0) e_s = *reinterpret_cast<volatile uint32_t*>(s.epoch) + 1u;
  __syncthreads();
  return e_s;
}
// The CTA that finishes last publishes the epoch for the next launch.
__device__ __forceinline__ void end_epoch(const PeerState& s, uint32_t e) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(s.ticket, 1u);
    if (t == gridDim.x - 1) {
      *s.ticket = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(s.epoch) = e;
    }
  }
}

__global__ void __launch_bounds__(512)
peer_allreduce_bf16_kernel(const PeerPointers pp, const PeerState st, int rank, int world, long long offset_bytes,
                           long long n_vec_per_slice) {
  const uint32_t e = begin_epoch(st);
  peer_barrier(pp, rank, world, 0, e, st.status, st.max_polls);
  // slice `rank`: n_vec_per_slice 16-byte vectors, strided over the CTAs
  const long long v0 = (long long)rank * n_vec_per_slice;
  // (the host picks the grid so that a thread has one or two vectors: every remote load of the slice is in
  // flight at once and the pass costs one NVLink round trip)
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec_per_slice;
       v += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    uint4 in[kPeerMaxWorld];
#pragma unroll
    for (int p = 0; p < kPeerMaxWorld; ++p)
      if (p < world) in[p] = __ldcg(reinterpret_cast<const uint4*>(pp.data[p] + offset_bytes + (v0 + v) * 16));   // L2 only
#pragma unroll
    for (int p = 0; p < kPeerMaxWorld; ++p) {
      if (p < world) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&in[p]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          acc[2 * i] += f.x;
          acc[2 * i + 1] += f.y;
        }
      }
    }
    uint4 out;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
#pragma unroll
    for (int p = 0; p < kPeerMaxWorld; ++p)
      if (p < world) *reinterpret_cast<uint4*>(pp.data[p] + offset_bytes + (v0 + v) * 16) = out;
  }
  peer_barrier(pp, rank, world, 1, e, st.status, st.max_polls);
  end_epoch(st, e);
}

// All-reduce of a row-parallel GEMM output fused with the residual add and the RMS norm that follow it in a
// decoder block:   delta = bf16(sum over ranks of part[rank]);  x = bf16(x + delta);  h = rmsnorm(x) * w.
// part, x and h are [rows, cols] bf16 regions of the peer buffers.  The slices of the all-reduce are whole
// rows (rows is a multiple of world): the rank that reduces a row holds all of it, so it also owns the
// row's sum of squares, and it stores the new x and h rows into every rank's buffer.  One CTA of 256
// threads per row (in turn), a thread keeps up to eight 16-byte chunks.  Thread layout, accumulation order
// and roundings repeat the separate all-reduce and add + norm kernels operation by operation (the sum is
// rounded to bf16 before it is added), so the results are bit-identical to theirs.
__global__ void __launch_bounds__(256)
peer_allreduce_add_rmsnorm_kernel(const PeerPointers pp, const PeerState st, int rank, int world,
                                  long long part_off, long long x_off, long long h_off, int rows_per_rank, int cols,
                                  const __nv_bfloat16* __restrict__ w, float eps) {
  __shared__ float red[8];
  const uint32_t e = begin_epoch(st);
  peer_barrier(pp, rank, world, 0, e, st.status, st.max_polls);
  const int nchunk = cols >> 3;
  for (int r = blockIdx.x; r < rows_per_rank; r += gridDim.x) {
    const long long row_bytes = ((long long)rank * rows_per_rank + r) * (long long)cols * 2;
    uint4 keep[8];
    float ss = 0.f;
    int n = 0;
    for (int c = threadIdx.x; c < nchunk; c += blockDim.x, ++n) {
      const long long off = row_bytes + (long long)c * 16;
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      uint4 in[kPeerMaxWorld];
#pragma unroll
      for (int p = 0; p < kPeerMaxWorld; ++p)
        if (p < world) in[p] = __ldcg(reinterpret_cast<const uint4*>(pp.data[p] + part_off + off));
      uint4 xv = __ldcg(reinterpret_cast<const uint4*>(pp.data[rank] + x_off + off));
#pragma unroll
      for (int p = 0; p < kPeerMaxWorld; ++p) {
        if (p < world) {
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&in[p]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h2[i]);
            acc[2 * i] += f.x;
            acc[2 * i + 1] += f.y;
          }
        }
      }
      __nv_bfloat16* xh = reinterpret_cast<__nv_bfloat16*>(&xv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = __bfloat162float(__float2bfloat16(acc[i]));      // the all-reduce's bf16 result
        xh[i] = __float2bfloat16(__bfloat162float(xh[i]) + d);           // residual add, rounded to bf16
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float f = __bfloat162float(xh[i]);
        ss += f * f;
      }
      keep[n] = xv;
#pragma unroll
      for (int p = 0; p < kPeerMaxWorld; ++p)
        if (p < world) *reinterpret_cast<uint4*>(pp.data[p] + x_off + off) = xv;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();                      // the previous row's readers of `red` are done
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
    const float inv = rsqrtf(tot / (float)cols + eps);
    n = 0;
    for (int c = threadIdx.x; c < nchunk; c += blockDim.x, ++n) {
      const long long off = row_bytes + (long long)c * 16;
      const uint4 wv = *reinterpret_cast<const uint4*>(w + (long long)c * 8);
      const __nv_bfloat16* wh = reinterpret_cast<const __nv_bfloat16*>(&wv);
      const __nv_bfloat16* xh = reinterpret_cast<const __nv_bfloat16*>(&keep[n]);
      uint4 ov;
      __nv_bfloat16* oh = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // normalise in fp32, cast to bf16, then multiply by the weight (as the separate norm kernel does)
        const __nv_bfloat16 nb = __float2bfloat16(__bfloat162float(xh[i]) * inv);
        oh[i] = __float2bfloat16(__bfloat162float(wh[i]) * __bfloat162float(nb));
      }
#pragma unroll
      for (int p = 0; p < kPeerMaxWorld; ++p)
        if (p < world) *reinterpret_cast<uint4*>(pp.data[p] + h_off + off) = ov;
    }
  }
  peer_barrier(pp, rank, world, 1, e, st.status, st.max_polls);
  end_epoch(st, e);
}

__global__ void __launch_bounds__(256)
peer_allgather_kernel(const PeerPointers pp, const PeerState st, int rank, int world, const uint8_t* src,
                      long long offset_bytes, long long chunk_bytes) {
  const uint32_t e = begin_epoch(st);
  peer_barrier(pp, rank, world, 0, e, st.status, st.max_polls);
  const long long n4 = chunk_bytes >> 2;   // chunk_bytes is a multiple of 4
  for (long long i = threadIdx.x; i < n4; i += blockDim.x) {
    const uint32_t w = reinterpret_cast<const uint32_t*>(src)[i];
    for (int p = 0; p < world; ++p)
      reinterpret_cast<uint32_t*>(pp.data[p] + offset_bytes + (long long)rank * chunk_bytes)[i] = w;
  }
  peer_barrier(pp, rank, world, 1, e, st.status, st.max_polls);
  end_epoch(st, e);
}

}  // namespace

cudaError_t launch_peer_allreduce_bf16(const PeerPointers& pp, const PeerState& st, int rank, int world,
                                       long long offset_bytes, long long n_elems, int ctas, cudaStream_t stream) {
  const long long n_vec_per_slice = n_elems / 8 / world;
  if (ctas < 1) ctas = 1;
  if (ctas > kPeerMaxCtas) ctas = kPeerMaxCtas;
  peer_allreduce_bf16_kernel<<<ctas, 512, 0, stream>>>(pp, st, rank, world, offset_bytes, n_vec_per_slice);
  return cudaGetLastError();
}

cudaError_t launch_peer_allreduce_add_rmsnorm(const PeerPointers& pp, const PeerState& st, int rank, int world,
                                              long long part_off, long long x_off, long long h_off, int rows, int cols,
                                              const void* w, float eps, cudaStream_t stream) {
  const int rows_per_rank = rows / world;
  int ctas = rows_per_rank < kPeerMaxCtas ? rows_per_rank : kPeerMaxCtas;
  if (ctas < 1) ctas = 1;
  peer_allreduce_add_rmsnorm_kernel<<<ctas, 256, 0, stream>>>(pp, st, rank, world, part_off, x_off, h_off,
                                                              rows_per_rank, cols,
                                                              static_cast<const __nv_bfloat16*>(w), eps);
  return cudaGetLastError();
}

cudaError_t launch_peer_allgather(const PeerPointers& pp, const PeerState& st, int rank, int world, const void* src,
                                  long long offset_bytes, long long chunk_bytes, cudaStream_t stream) {
  peer_allgather_kernel<<<1, 256, 0, stream>>>(pp, st, rank, world, static_cast<const uint8_t*>(src), offset_bytes,
                                               chunk_bytes);
  return cudaGetLastError();
}

}  // namespace fa
