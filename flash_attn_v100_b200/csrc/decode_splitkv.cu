// Split-KV GQA decode for sm_100a: paged, contiguous and INT8-QK variants of one kernel.
//
// Replaces the reference's one-CTA-per-query-head decode kernels
// (flash_attn_kernel.cu:1641-1797, 2796-2939, 3391-3514 and
// continuous_batching_kernel.cu:40-195).
//
// Work decomposition.  A "unit" is one 16-token page of one segment, a segment
// being (sequence b, KV head, block of <=16 query heads sharing that KV head).
// Units are numbered b-major, then segment, then page; the grid is persistent
// (a fixed number of CTAs per SM) and CTA c owns the contiguous unit range
// [c*per, (c+1)*per).  A CTA therefore reads an equal share of the KV bytes
// whatever the length spread, and a segment is split across CTAs only at range
// boundaries: at most two partial results per CTA.  The CTA that delivers the
// last partial of a split segment (an arrival counter per split segment, named
// by the first CTA that works on it, bumped with one atomic add per arrival and
// put back to zero by the last arriver, so that it never needs clearing after the
// workspace's one-time initialisation unless a launch recorded a device status)
// merges them by log-sum-exp.  The page prefix sums that define the unit numbering
// are recomputed by every CTA in shared memory: the whole decode is one launch.
//
// Data path.  Inside a CTA each warp streams its own pages (page i of a piece
// goes to warp i mod W) through a private ring of shared-memory stages filled
// by TMA (cp.async.bulk.tensor, 128-byte swizzle, completion on an mbarrier).
// K and V of a page for one KV head are 16 x D fp16 = one contiguous 4 KB block
// at D = 128.  All query heads of the group are processed together (they are
// the M rows of the MMA) so each K/V byte is read from HBM exactly once.
// S = Q K^T and O += P V run on mma.sync m16n8k16 (fp32 accumulate) with
// ldmatrix from the swizzled tiles; softmax is fp32, base-2, online.
#include "common.cuh"
#include "decode_splitkv.cuh"

#include <math.h>

namespace fa {

namespace {

__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  uint64_t ra = *reinterpret_cast<uint64_t*>(&a), rb = *reinterpret_cast<uint64_t*>(&b), rd;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  return *reinterpret_cast<float2*>(&rd);
}

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  uint64_t ra = *reinterpret_cast<uint64_t*>(&a), rb = *reinterpret_cast<uint64_t*>(&b),
           rc = *reinterpret_cast<uint64_t*>(&c), rd;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  return *reinterpret_cast<float2*>(&rd);
}
// max(a, |b|, |c|), NaN if any operand is NaN
__device__ __forceinline__ float fmax3_abs_nan(float a, float b, float c) {
  float d;
  asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(fabsf(b)), "f"(fabsf(c)));
  return d;
}

// clamp(roundf(x / s), -127, 127) exactly as IEEE fp32 evaluates it (the reference's quantiser)
__device__ __forceinline__ uint32_t quant_exact1(float x, float s) {
  const float t = fmaxf(-127.f, fminf(127.f, roundf(__fdiv_rn(x, s))));
  return static_cast<uint32_t>(static_cast<int>(t)) & 0xffu;
}

// Exact quantisation of K[tok][d] of an fp16 K page in shared memory (64-column slabs of 16 rows,
// 128-byte swizzle).  Out of line: it runs for a few values per page.
template <int SLAB_BYTES>
__device__ __noinline__ uint32_t quant_exact_elem(const uint8_t* kptr, int tok, int d, float s) {
  const int ch = d >> 3;
  const __half v = *reinterpret_cast<const __half*>(kptr + (ch >> 3) * SLAB_BYTES + tok * 128 +
                                                    (((ch & 7) ^ (tok & 7)) << 4) + (d & 7) * 2);
  return quant_exact1(__half2float(v), s);
}

// Fast quantisation of four values (two half2 registers) of one token, rcp = 1 / scale:
//   yn = -(x * rcp + 1.5 * 2^23)   one FMA: the low mantissa byte is rint(x * rcp) as int8
//   rn = yn + 1.5 * 2^23           = -rint(x * rcp), exact
//   u  = x * rcp + rn              = the distance to the nearest integer
// Returns the four bytes; umax / rmax collect max |u| and max |rint| (NaN-propagating), from which
// the caller decides whether any value needs the exact path (near a rounding tie, beyond the clamp
// range, NaN or Inf).
__device__ __forceinline__ uint32_t quant_fast4(uint32_t h01, uint32_t h23, float rcp, float& umax, float& rmax) {
  const float kMagic = 12582912.f;
  const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
  const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
  const float2 nr = make_float2(-rcp, -rcp), pr = make_float2(rcp, rcp);
  const float2 nm = make_float2(-kMagic, -kMagic), pm = make_float2(kMagic, kMagic);
  const float2 y01 = ffma2(f01, nr, nm), y23 = ffma2(f23, nr, nm);
  const float2 r01 = fadd2(y01, pm), r23 = fadd2(y23, pm);
  const float2 u01 = ffma2(f01, pr, r01), u23 = ffma2(f23, pr, r23);
  umax = fmax3_abs_nan(umax, u01.x, u01.y);
  umax = fmax3_abs_nan(umax, u23.x, u23.y);
  rmax = fmax3_abs_nan(rmax, r01.x, r01.y);
  rmax = fmax3_abs_nan(rmax, r23.x, r23.y);
  return __byte_perm(__byte_perm(__float_as_uint(y01.x), __float_as_uint(y01.y), 0x0040),
                     __byte_perm(__float_as_uint(y23.x), __float_as_uint(y23.y), 0x0040), 0x5410);
}
// |u| at or above this, or |rint| above 127.5: the fast result may differ from the IEEE quotient's
// rounding (|x * rcp - x / s| < 2.3e-5 for |x / s| < 128), so the value is redone exactly.
constexpr float kQuantTieGuard = 0.49997f;

constexpr int kMaxSmemPrefix = 4096;  // B + 1 <= this: prefix sums are staged in shared memory

__device__ __forceinline__ int seq_len_of(const DecodeParams& p, int b) {
  if (p.mode == kModeContigFixed) return p.fixed_len;
  int v = __ldg(p.lens + b);
  if (p.mode == kModePaged) {
    long long cap = (long long)p.bt_stride * 16;
    v = v < 0 ? 0 : v;
    return (long long)v > cap ? (int)cap : v;
  }
  // continuous batching: keys [0, min(cache_len + 1, max_N))
  long long n = (long long)v + 1;
  if (n > p.N) n = p.N;
  return n < 0 ? 0 : (int)n;
}

// MMA on the query-head block.  HM ("half M"): the block has at most 8 heads, so fragment rows 8-15 are
// all-zero padding: their A registers are passed as zero and their accumulators are not kept.
template <bool HM, bool BF = false>
__device__ __forceinline__ void mma_rows(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (HM && BF) {
    float d2, d3;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, "
        "{%0,%1,%9,%9};"
        : "+f"(c[0]), "+f"(c[1]), "=f"(d2), "=f"(d3)
        : "r"(a[0]), "r"(0u), "r"(a[2]), "r"(b0), "r"(b1), "f"(0.f));
  } else if constexpr (HM) {
    float d2, d3;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, "
        "{%0,%1,%9,%9};"
        : "+f"(c[0]), "+f"(c[1]), "=f"(d2), "=f"(d3)
        : "r"(a[0]), "r"(0u), "r"(a[2]), "r"(b0), "r"(b1), "f"(0.f));
  } else if constexpr (BF) {
    mma_bf16_16816(c, a, b0, b1);
  } else {
    mma_f16_16816(c, a, b0, b1);
  }
}
template <bool HM>
__device__ __forceinline__ void mma_s8_rows(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (HM) {
    int d2, d3;
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, "
        "{%0,%1,%5,%5};"
        : "+r"(c[0]), "+r"(c[1]), "=r"(d2), "=r"(d3)
        : "r"(a[0]), "r"(0u), "r"(a[2]), "r"(b0), "r"(b1));
  } else {
    mma_s8_16832(c, a, b0, b1);
  }
}

// ---- int8 KV cache helpers ---------------------------------------------------
// Byte offset of (token row, byte column) inside an int8 K or V page in shared memory: 128-byte-wide
// slabs of 16 rows with the 128-byte swizzle (16-byte chunk index XOR row), or plain 64-byte rows.
template <int D>
__device__ __forceinline__ int kv8_offset(int tok, int byte) {
  if constexpr (D == 64) {
    return tok * 64 + byte;
  } else {
    const int slab = byte >> 7, chunk = (byte >> 4) & 7;
    return slab * 2048 + tok * 128 + ((chunk ^ (tok & 7)) << 4) + (byte & 15);
  }
}

__device__ __forceinline__ uint32_t hsub_hmul(uint32_t x, uint32_t bias, uint32_t scale) {
  const __half2 d = __hsub2(*reinterpret_cast<const __half2*>(&x), *reinterpret_cast<const __half2*>(&bias));
  const __half2 r = __hmul2(d, *reinterpret_cast<const __half2*>(&scale));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// int8 -> fp16 without a conversion instruction: the byte b is placed in the mantissa of 1024.0 as
// b ^ 0x80 = b + 128, so 0x6400 | (b ^ 0x80) is the fp16 number 1152 + b, exactly.  For V, 1152 is
// subtracted (exact) and the fp16 product with the token's scale rounds the exact product once, as
// the reference's fp16(float(int8) * float(scale)) does (hsub_hmul).
// Four consecutive int8 -> two fp16 pairs holding 1152 + b each (exact); the caller removes the
// constant from the finished dot product.
__device__ __forceinline__ void dequant_k4_biased(uint32_t w, uint32_t& b0, uint32_t& b1) {
  const uint32_t u = w ^ 0x80808080u;
  b0 = __byte_perm(u, 0x64646464u, 0x4140);
  b1 = __byte_perm(u, 0x64646464u, 0x4342);
}

// NT bytes [NT*g, NT*g + NT) of V token row `tok` (NT = D / 8) into NT/4 words.
template <int D>
__device__ __forceinline__ void load_v_row(const uint8_t* vptr, int tok, int g, uint32_t (&w)[D / 32]) {
  constexpr int NT = D / 8;
  if constexpr (NT == 8) {
    const uint2 t = *reinterpret_cast<const uint2*>(vptr + kv8_offset<D>(tok, NT * g));
    w[0] = t.x; w[1] = t.y;
  } else {
#pragma unroll
    for (int i = 0; i < NT / 16; ++i) {
      const uint4 t = *reinterpret_cast<const uint4*>(vptr + kv8_offset<D>(tok, NT * g + 16 * i));
      w[4 * i] = t.x; w[4 * i + 1] = t.y; w[4 * i + 2] = t.z; w[4 * i + 3] = t.w;
    }
  }
}

// Byte J of the words of four token rows (2c, 2c+1 | 2c+8, 2c+9) -> the B fragment of one output
// tile, dequantised as in dequant_k4, then acc += P * V.
template <int J, bool HM>
__device__ __forceinline__ void dequant_v_pair(uint32_t wa, uint32_t wb, uint32_t wc, uint32_t wd, uint32_t sc_lo,
                                               uint32_t sc_hi, const uint32_t (&pa)[4], float (&acc)[4]) {
  constexpr uint32_t sel = ((4u + J) << 12) | ((4u + J) << 8) | (J << 4) | J;  // [a.bJ, a.bJ, b.bJ, b.bJ]
  uint32_t lo = __byte_perm(wa, wb, sel), hi = __byte_perm(wc, wd, sel);
  // low byte of each half: x ^ 0x80; high byte: 0x64   (f = a ? (t ^ b) : b, lut 0x6a)
  asm("lop3.b32 %0, %0, 0x00ff00ff, 0x64806480, 0x6a;" : "+r"(lo));
  asm("lop3.b32 %0, %0, 0x00ff00ff, 0x64806480, 0x6a;" : "+r"(hi));
  mma_rows<HM>(acc, pa, hsub_hmul(lo, 0x64806480u, sc_lo), hsub_hmul(hi, 0x64806480u, sc_hi));
}

__device__ __forceinline__ int pages_of(const DecodeParams& p, int b) {
  if (p.window_pages_total > 0) return p.window_pages_total;   // sink pages + window pages, same for all b
  return (seq_len_of(p, b) + 15) >> 4;
}

// ---------------------------------------------------------------------------
// plan: prefix[b] = number of pages of sequences 0..b-1  (one CTA)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) decode_plan_kernel(const DecodeParams p) {
  __shared__ int warp_tot[32];
  __shared__ int carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    carry_s = 0;
    p.prefix[0] = 0;
  }
  __syncthreads();
  for (int base = 0; base < p.B; base += 1024) {
    const int b = base + tid;
    int pages = 0;
    if (b < p.B) pages = pages_of(p, b);
    int incl = pages;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int t = warp_tot[lane];
      int ti = t;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int u = __shfl_up_sync(0xffffffffu, ti, o);
        if (lane >= o) ti += u;
      }
      warp_tot[lane] = ti - t;  // exclusive
    }
    __syncthreads();
    const int carry = carry_s;
    if (b < p.B) p.prefix[b + 1] = carry + warp_tot[warp] + incl;
    __syncthreads();
    if (tid == 1023) carry_s = carry + warp_tot[warp] + incl;
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------
#ifndef FA_F16_MINB
#define FA_F16_MINB 2
#endif
#ifndef FA_KV8_MINB
#define FA_KV8_MINB 3
#endif
#ifndef FA_I8QK_MINB
#define FA_I8QK_MINB 3
#endif
// Threads per CTA and CTAs per SM the kernel is compiled for.  The half-M variants keep half the
// accumulators, which leaves room for more resident CTAs (more pages in flight, more warps to hide
// the dequantisation latency); they run with at most 4 warps.
template <int D, int KIND, bool HM>
struct DecodeOccupancy {
  static constexpr int kThreads = HM ? 128 : 256;
  static constexpr int kMinBlocks =
      !HM ? 1 : (D == 64 ? 4 : (D == 256 ? 2 : ((KIND == kKindF16 || KIND == kKindBF16) ? FA_F16_MINB : (KIND == kKindInt8KV ? FA_KV8_MINB : FA_I8QK_MINB))));
};

template <int D, int KIND, bool HM>
__global__ void __launch_bounds__(DecodeOccupancy<D, KIND, HM>::kThreads, DecodeOccupancy<D, KIND, HM>::kMinBlocks)
decode_splitkv_kernel(const __grid_constant__ CUtensorMap kmap,
                      const __grid_constant__ CUtensorMap vmap, const DecodeParams p) {
  constexpr bool INT8 = KIND == kKindInt8QK;   // fp16 cache, K and Q quantised on the fly for the scores
  constexpr bool KV8 = KIND == kKindInt8KV;    // int8 cache with per-token fp16 scales
  constexpr bool BF = KIND == kKindBF16;       // bfloat16 q / cache: the fp16 path with bfloat16 MMAs and P
  constexpr int NR = HM ? 2 : 4;               // live accumulator registers per fragment (rows g | g, g + 8)
  constexpr int PAGE_BYTES = 16 * D * (KV8 ? 1 : 2);
  // One TMA box: 16 rows x 128 bytes (64 fp16 or 128 int8 columns), 128-byte swizzle;
  // D = 64 int8 rows are 64 bytes wide and are copied unswizzled.
  constexpr int SLAB_BYTES = (KV8 && D == 64) ? 16 * 64 : 16 * 128;
  constexpr int SLAB_COLS = KV8 ? (D == 64 ? 64 : 128) : 64;
  constexpr int NSLAB = D / SLAB_COLS;
  constexpr int NT = D / 8;  // 8-column output tiles
  constexpr int ROWLEN = D + 2;

  extern __shared__ uint8_t smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  uint8_t* smem = smem_dyn + ((1024u - (raw & 1023u)) & 1023u);

  const int W = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.stages;
  const int g = lane >> 2;         // fragment row (query head within the block)
  const int cq = (lane & 3) * 2;   // fragment column pair

  uint8_t* my_stages = smem + (size_t)(warp * S) * (2 * PAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)W * S * (2 * PAGE_BYTES));
  float* mbuf = reinterpret_cast<float*>(bars + W * S);
  int* s_prefix = reinterpret_cast<int*>(mbuf + (size_t)W * p.slot_rows * ROWLEN);
  const bool prefix_in_smem = (p.B + 1) <= kMaxSmemPrefix;
  const int* pre = prefix_in_smem ? s_prefix : p.prefix;

  __shared__ int s_scan[8];
  __shared__ int s_last_flag;
  if (prefix_in_smem) {
    // block-wide inclusive scan of pages per sequence: s_prefix[i + 1] = pages of sequences 0..i
    const int nthr = blockDim.x;
    const int chunk = (p.B + nthr - 1) / nthr;
    const int i0 = threadIdx.x * chunk, i1 = (i0 + chunk < p.B) ? (i0 + chunk) : p.B;
    int local = 0;
    for (int i = i0; i < i1; ++i) {
      local += pages_of(p, i);
      s_prefix[i + 1] = local;
    }
    int incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) s_scan[warp] = incl;
    __syncthreads();
    int offset = incl - local;
    for (int w = 0; w < warp; ++w) offset += s_scan[w];
    for (int i = i0; i < i1; ++i) s_prefix[i + 1] += offset;
    if (threadIdx.x == 0) s_prefix[0] = 0;
  }
  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(smem_u32(bars + warp * S + s), 1);
    mbar_fence_init();
    fence_proxy_async();
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&kmap);
    tma_prefetch_desc(&vmap);
  }
  __syncthreads();

  if (blockIdx.x == 0) {
    // sequences with nothing to attend: zeros by definition (no unit ever touches their output)
    for (int bb = 0; bb < p.B; ++bb) {
      if (pre[bb + 1] != pre[bb]) continue;
      __half* o = p.out + (size_t)bb * p.H_Q * p.D_real;
      for (int e = threadIdx.x; e < p.H_Q * p.D_real; e += blockDim.x) o[e] = __float2half_rn(0.f);
    }
  }
  const long long T = (long long)p.HV * pre[p.B];
  long long per = (T + p.n_cta - 1) / p.n_cta;
  if (per < 1) per = 1;
  long long u = (long long)blockIdx.x * per;
  const long long u1 = (u + per < T) ? (u + per) : T;
  if (u >= u1) return;

  const uint64_t policy = l2_policy_evict_first();
  const uint32_t bar0 = smem_u32(bars + warp * S);
  const uint32_t stage0 = smem_u32(my_stages);
  // ring position of the next page to issue / to consume, and the phase parity of the consumer side
  uint32_t st_issue = 0, st_cons = 0, par_cons = 0;

  // locate the sequence that holds unit u: largest b with HV * pre[b] <= u
  int b;
  {
    int lo = 0, hi = p.B;  // invariant: HV*pre[lo] <= u < HV*pre[hi]
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if ((long long)p.HV * pre[mid] <= u) lo = mid; else hi = mid;
    }
    b = lo;
  }

  // A piece: the pages [p0, p0 + cnt) of one (sequence, KV-head block) unit, the part of this CTA's range
  // [u, u1) that lies in that unit.
  struct Piece {
    int b, np, hv, p0, cnt;
  };
  auto locate = [&](long long uu, int bb) -> Piece {
    Piece q;
    while ((long long)p.HV * pre[bb + 1] <= uu) ++bb;  // also skips empty sequences
    q.b = bb;
    q.np = pre[bb + 1] - pre[bb];
    const long long rel = uu - (long long)p.HV * pre[bb];
    q.hv = (int)(rel / q.np);
    q.p0 = (int)(rel - (long long)q.hv * q.np);
    const long long left = u1 - uu;
    q.cnt = (q.np - q.p0) < left ? (q.np - q.p0) : (int)left;
    return q;
  };
  // One page copy (K and V rows of unit page `upage`) into the next ring stage of this warp; lane 0 issues.
  auto issue_page = [&](int upage, int pid, int h_kv_, long long contig_row0_) {
    if (lane == 0) {
      const int page = upage < p.sink_pages ? upage : p.win_first_page + (upage - p.sink_pages);
      long long row;
      if (p.mode == kModePaged) {
        if (pid < 0 || (long long)pid >= p.num_pages) {
          atomicOr(p.status, kStatusBadPageId);
          pid = 0;
        }
        row = ((long long)pid * p.H_KV + h_kv_) * 16;
      } else {
        row = contig_row0_ + (long long)page * 16;
      }
      const uint32_t st = st_issue;
      const uint32_t bar = bar0 + st * 8;
      const uint32_t dst = stage0 + st * (2 * PAGE_BYTES);
      mbar_expect_tx(bar, 2 * PAGE_BYTES);
#pragma unroll
      for (int sl = 0; sl < NSLAB; ++sl) {
        tma_load_2d(dst + sl * SLAB_BYTES, &kmap, sl * SLAB_COLS, (int)row, bar, policy);
        tma_load_2d(dst + PAGE_BYTES + sl * SLAB_BYTES, &vmap, sl * SLAB_COLS, (int)row, bar, policy);
      }
    }
    st_issue = (st_issue + 1 == (uint32_t)S) ? 0u : st_issue + 1;
  };
  // Pages of the NEXT piece that this warp has already put in flight while it finished the current one
  // (the ring never runs empty across a piece boundary: the copies of the next piece's first pages overlap
  // the merge of this one).
  int pre_issued = 0;

  int piece = 0;
  while (u < u1) {
    const Piece pc = locate(u, b);
    b = pc.b;
    const int np = pc.np, hv = pc.hv, p0 = pc.p0, cnt = pc.cnt;
    const bool complete = (p0 == 0) && (cnt == np);
    const int len = seq_len_of(p, b);
    const int h_kv = hv / p.n_gblk;
    const int gb0 = (hv - h_kv * p.n_gblk) * 16;
    const int Gb = (p.G - gb0) < 16 ? (p.G - gb0) : 16;
    const int head0 = h_kv * p.G + gb0;

    // ---- this warp's share of the piece: pages p0 + warp + n*W -------------------
    const int n_my = cnt > warp ? (cnt - warp + W - 1) / W : 0;

    // Q fragments (A operand).  Rows >= Gb are zero.
    constexpr int QREGS = INT8 ? (D / 32) : (D / 16);
    // KV8: the contraction index of k-step t, fragment slot pair (2c,2c+1 | 2c+8,2c+9) of lane c = lane & 3
    // stands for head dimensions d0 .. d0+3 with d0 = 128 * (t / KPS) + 4 * KPS * c + 4 * (t % KPS):
    // a lane then reads 16 consecutive int8 of a token row for four k-steps.  Q uses the same map.
    constexpr int KPS = (D >= 128) ? 8 : 4;
    uint32_t qa[QREGS][4];
    float q_s0 = 1.f, q_s1 = 1.f;
    float kbias0 = 0.f, kbias1 = 0.f;  // KV8 only
    {
      // D is the padded head dimension the kernel is built for, Dr the real one: columns [Dr, D) of K and V
      // read as zeros through the tensor maps, and the same columns of Q are taken as zero here.
      const int Dr = p.D_real;
      const bool v0 = g < Gb, v1 = !HM && (g + 8) < Gb;
      const __half* q0 = p.q + ((size_t)b * p.H_Q + head0 + g) * Dr;
      const __half* q1 = q0 + (size_t)8 * Dr;
      if constexpr (KV8) {
#pragma unroll
        for (int t = 0; t < D / 16; ++t) {
          const int d0 = 128 * (t / KPS) + 4 * KPS * (lane & 3) + 4 * (t % KPS);
          const uint2 a = (v0 && d0 < Dr) ? __ldg(reinterpret_cast<const uint2*>(q0 + d0)) : make_uint2(0u, 0u);
          const uint2 c = (v1 && d0 < Dr) ? __ldg(reinterpret_cast<const uint2*>(q1 + d0)) : make_uint2(0u, 0u);
          qa[t][0] = a.x; qa[t][1] = c.x; qa[t][2] = a.y; qa[t][3] = c.y;
          const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&a.x));
          const float2 a1 = __half22float2(*reinterpret_cast<const __half2*>(&a.y));
          const float2 c0 = __half22float2(*reinterpret_cast<const __half2*>(&c.x));
          const float2 c1 = __half22float2(*reinterpret_cast<const __half2*>(&c.y));
          kbias0 += (a0.x + a0.y) + (a1.x + a1.y);
          kbias1 += (c0.x + c0.y) + (c1.x + c1.y);
        }
        // K enters the score product as the fp16 number 1152 + k (see dequant_k4_biased), so every raw
        // score carries 1152 * sum_d q[d]; that constant of the query row is taken off again in fp32.
        kbias0 += __shfl_xor_sync(0xffffffffu, kbias0, 1);
        kbias0 += __shfl_xor_sync(0xffffffffu, kbias0, 2);
        kbias1 += __shfl_xor_sync(0xffffffffu, kbias1, 1);
        kbias1 += __shfl_xor_sync(0xffffffffu, kbias1, 2);
        kbias0 *= 1152.f;
        kbias1 *= 1152.f;
      } else if constexpr (!INT8) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const bool in_lo = kk * 16 + cq < Dr, in_hi = kk * 16 + 8 + cq < Dr;
          qa[kk][0] = (v0 && in_lo) ? __ldg(reinterpret_cast<const uint32_t*>(q0 + kk * 16 + cq)) : 0u;
          qa[kk][1] = (v1 && in_lo) ? __ldg(reinterpret_cast<const uint32_t*>(q1 + kk * 16 + cq)) : 0u;
          qa[kk][2] = (v0 && in_hi) ? __ldg(reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 8 + cq)) : 0u;
          qa[kk][3] = (v1 && in_hi) ? __ldg(reinterpret_cast<const uint32_t*>(q1 + kk * 16 + 8 + cq)) : 0u;
        }
      } else {
        if (v0) q_s0 = __ldg(p.q_scale + (size_t)b * p.H_Q + head0 + g);
        if (v1) q_s1 = __ldg(p.q_scale + (size_t)b * p.H_Q + head0 + g + 8);
        // Slot 4c+i of k-step kk of the int8 MMA stands for head dimension
        // 32*kk + {2c, 2c+1, 8+2c, 9+2c}[i], slot 16+4c+i for the same plus 16: these are the values a
        // lane holds after ldmatrix of the fp16 K tile, so K needs no shuffling before it is quantised.
        auto quant4 = [Dr](const __half* row, int d, float s) -> uint32_t {
          uint32_t out = 0;
          if (d < Dr) {
            const __half2 h01 = __ldg(reinterpret_cast<const __half2*>(row + d));
            out |= quant_exact1(__low2float(h01), s) | (quant_exact1(__high2float(h01), s) << 8);
          }
          if (d + 8 < Dr) {
            const __half2 h23 = __ldg(reinterpret_cast<const __half2*>(row + d + 8));
            out |= (quant_exact1(__low2float(h23), s) << 16) | (quant_exact1(__high2float(h23), s) << 24);
          }
          return out;
        };
#pragma unroll
        for (int kk = 0; kk < D / 32; ++kk) {
          qa[kk][0] = v0 ? quant4(q0, kk * 32 + cq, q_s0) : 0u;
          qa[kk][1] = v1 ? quant4(q1, kk * 32 + cq, q_s1) : 0u;
          qa[kk][2] = v0 ? quant4(q0, kk * 32 + 16 + cq, q_s0) : 0u;
          qa[kk][3] = v1 ? quant4(q1, kk * 32 + 16 + cq, q_s1) : 0u;
        }
      }
    }

    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    // Block-table entries of this warp's pages, 32 at a time, one batch ahead.
    const int32_t* bt_row = p.block_table + (size_t)b * p.bt_stride;
    int tbl_cur = 0, tbl_next = 0;
    auto load_tbl = [&](int batch) -> int {
      const int n = batch * 32 + lane;
      if (p.mode != kModePaged || n >= n_my) return 0;
      return __ldg(bt_row + p0 + warp + n * W);
    };
    tbl_cur = load_tbl(0);
    tbl_next = load_tbl(1);

    const long long contig_row0 = ((long long)b * p.H_KV + h_kv) * (long long)p.N;

    auto issue = [&](int n) {
      // every lane takes part in the shuffle; lane 0 issues the copies
      const int pid = __shfl_sync(0xffffffffu, tbl_cur, n & 31);
      issue_page(p0 + warp + n * W, pid, h_kv, contig_row0);
    };

    // The piece after this one (if this CTA has one): where it lies, this warp's share of it and the
    // block-table entries of its first pages, fetched now so that they are at hand when the ring has room.
    const bool has_next = u + cnt < u1;
    Piece nx = pc;
    int nx_n_my = 0, nx_tbl = 0, nx_h_kv = 0;
    long long nx_row0 = 0;
    if (has_next) {
      nx = locate(u + cnt, b);
      nx_n_my = nx.cnt > warp ? (nx.cnt - warp + W - 1) / W : 0;
      nx_h_kv = nx.hv / p.n_gblk;
      nx_row0 = ((long long)nx.b * p.H_KV + nx_h_kv) * (long long)p.N;
      if (p.mode == kModePaged && lane < nx_n_my && lane < S)
        nx_tbl = __ldg(p.block_table + (size_t)nx.b * p.bt_stride + nx.p0 + warp + lane * W);
    }

    int issued = pre_issued;   // pages of this piece that were put in flight during the previous one
    pre_issued = 0;
    for (; issued < S && issued < n_my; ++issued) issue(issued);

    // bit t of the result: token page*16 + t is attended (inside the length, and in the sink or the window)
    auto page_of = [&](int n) -> int {
      const int upage = p0 + warp + n * W;
      return upage < p.sink_pages ? upage : p.win_first_page + (upage - p.sink_pages);
    };
    auto vmask_of = [&](int page) -> uint32_t {
      auto low_bits = [](int n) -> uint32_t { return n <= 0 ? 0u : (n >= 16 ? 0xffffu : ((1u << n) - 1u)); };
      const int tok0 = page * 16;
      return low_bits(len - tok0) & (low_bits(p.sink - tok0) | (0xffffu & ~low_bits(p.win_start - tok0)));
    };

    // KV8: fp16 scales of the next page, fetched one page ahead: lanes 0-15 hold the K scale of token
    // `lane`, lanes 16-31 the V scale of token `lane - 16`; tokens that are not attended get scale 0,
    // so that whatever the cache holds there dequantises to zero.
    uint32_t sc_cur = 0, sc_next = 0;
    uint32_t vmask_next = n_my > 0 ? vmask_of(page_of(0)) : 0u;
    auto load_sc = [&](int n) -> uint32_t {
      if (n >= n_my) return 0u;
      const int page = page_of(n);
      const int t = lane & 15;
      if (!((vmask_next >> t) & 1u)) return 0u;
      const __half* base = (lane < 16) ? p.k_scale_h : p.v_scale_h;
      return __ldg(reinterpret_cast<const unsigned short*>(base) + ((size_t)b * p.H_KV + h_kv) * p.N + page * 16 + t);
    };
    if constexpr (KV8) sc_next = load_sc(0);

    // INT8: per-token K scales of the next page, fetched one page ahead.
    float ks_cur = 1.f, ks_next = 1.f;
    auto load_ks = [&](int n) -> float {
      if (n >= n_my) return 1.f;
      const int tok = (p0 + warp + n * W) * 16 + (lane & 15);
      if (tok >= p.N) return 1.f;
      return __ldg(p.k_scale + ((size_t)b * p.H_KV + h_kv) * p.N + tok);
    };
    if constexpr (INT8) ks_next = load_ks(0);

    // Per-page state, produced by begin_page() in page order: ring stage, visibility mask, page index and
    // the scales that go with the page.
    struct PageState {
      uint32_t st, vmask, sc;
      int page;
      float ks;
    };
    // Takes the next page of this warp: rotates the prefetched scales and masks, claims the ring stage and
    // waits for the page's data.  Called once per page, in order.
    auto begin_page = [&](int n) -> PageState {
      PageState ps;
      if constexpr (INT8) {
        ks_cur = ks_next;
        ks_next = load_ks(n + 1);
      }
      ps.vmask = vmask_next;
      vmask_next = (n + 1 < n_my) ? vmask_of(page_of(n + 1)) : 0u;
      if constexpr (KV8) {
        sc_cur = sc_next;
        sc_next = load_sc(n + 1);
      }
      ps.ks = ks_cur;
      ps.sc = sc_cur;
      ps.st = st_cons;
      const uint32_t parity = par_cons;
      if (++st_cons == (uint32_t)S) {
        st_cons = 0;
        par_cons ^= 1u;
      }
      if (!mbar_wait(bar0 + ps.st * 8, parity)) {
        if (lane == 0) atomicOr(p.status, kStatusWaitTimeout);
      }
      ps.page = page_of(n);
      return ps;
    };

    // Scores of one page (all tokens, not yet masked), base 2.
    auto compute_scores = [&](const PageState& ps, float (&s)[2][4]) {
      const uint32_t st = ps.st, vmask = ps.vmask;
      const int page = ps.page;
      const float ks_cur = ps.ks;
      const uint32_t sc_cur = ps.sc;
      const uint32_t kbase = stage0 + st * (2 * PAGE_BYTES);
      (void)vmask; (void)page; (void)ks_cur; (void)sc_cur; (void)kbase;
      // ---- S = Q K^T : [16 heads x 16 tokens] ------------------------------------
      if constexpr (KV8) {
#pragma unroll
        for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        const uint8_t* kptr = my_stages + (size_t)st * (2 * PAGE_BYTES);
#pragma unroll
        for (int q4 = 0; q4 < D / 64; ++q4) {  // 16 bytes = four k-steps per load; token g and token g + 8
          const int byte0 = 128 * ((q4 * 4) / KPS) + 4 * KPS * (lane & 3) + 4 * ((q4 * 4) % KPS);
          const uint4 wa = *reinterpret_cast<const uint4*>(kptr + kv8_offset<D>(g, byte0));
          const uint4 wb = *reinterpret_cast<const uint4*>(kptr + kv8_offset<D>(g + 8, byte0));
          const uint32_t w0[4] = {wa.x, wa.y, wa.z, wa.w};
          const uint32_t w1[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t b0, b1;
            dequant_k4_biased(w0[i], b0, b1);
            mma_rows<HM>(s[0], qa[q4 * 4 + i], b0, b1);
            dequant_k4_biased(w1[i], b0, b1);
            mma_rows<HM>(s[1], qa[q4 * 4 + i], b0, b1);
          }
        }
        // score = (raw - 1152 * sum q) * k_scale[token] / sqrt(D), in fp32, to base 2.  The per-element
        // product k * k_scale is not rounded to fp16 first: the score is the exact-dequantisation score
        // up to fp32 rounding.
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint32_t ka = __shfl_sync(0xffffffffu, sc_cur, 8 * j + cq);
          const uint32_t kb = __shfl_sync(0xffffffffu, sc_cur, 8 * j + cq + 1);
          const float ta = __half2float(__ushort_as_half((unsigned short)ka)) * p.scale_log2;
          const float tb = __half2float(__ushort_as_half((unsigned short)kb)) * p.scale_log2;
          s[j][0] = (s[j][0] - kbias0) * ta;
          s[j][1] = (s[j][1] - kbias0) * tb;
          if constexpr (!HM) {
            s[j][2] = (s[j][2] - kbias1) * ta;
            s[j][3] = (s[j][3] - kbias1) * tb;
          }
        }
      } else if constexpr (!INT8) {
#pragma unroll
        for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        const int mi = lane >> 3;
        const int r = (lane & 7) + (mi >> 1) * 8;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int chunk = 2 * kk + (mi & 1);
          const uint32_t addr = kbase + (chunk >> 3) * SLAB_BYTES + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
          uint32_t kb[4];
          ldmatrix_x4(kb, addr);
          mma_rows<HM, BF>(s[0], qa[kk], kb[0], kb[1]);
          mma_rows<HM, BF>(s[1], qa[kk], kb[2], kb[3]);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < NR; ++e) s[j][e] *= p.scale_log2;
      } else {
        int si[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) si[j][0] = si[j][1] = si[j][2] = si[j][3] = 0;
        // K scale of the token of this lane's B-fragment column in each n-tile (tokens g and g + 8)
        const float ksr0 = __shfl_sync(0xffffffffu, ks_cur, g);
        const float ksr1 = __shfl_sync(0xffffffffu, ks_cur, g + 8);
        const float rcp0 = __frcp_rn(ksr0), rcp1 = __frcp_rn(ksr1);
        float um[D / 16], rmax = 0.f;   // max |distance to the nearest integer| per 16-wide slice, max |rint|
        uint32_t bq[2][D / 32][2];
        const int mi = lane >> 3;
        const int lrow = (lane & 7) + (mi >> 1) * 8;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int chunk = 2 * kk + (mi & 1);
          const uint32_t addr = kbase + (chunk >> 3) * SLAB_BYTES + lrow * 128 + (((chunk & 7) ^ (lrow & 7)) << 4);
          uint32_t kb[4];
          ldmatrix_x4(kb, addr);
          um[kk] = 0.f;
          bq[0][kk >> 1][kk & 1] = quant_fast4(kb[0], kb[1], rcp0, um[kk], rmax);
          bq[1][kk >> 1][kk & 1] = quant_fast4(kb[2], kb[3], rcp1, um[kk], rmax);
        }
        float umax = um[0];
#pragma unroll
        for (int kk = 1; kk < D / 16; kk += 2) umax = fmax3_abs_nan(umax, um[kk], kk + 1 < D / 16 ? um[kk + 1] : 0.f);
        const bool redo = !(umax < kQuantTieGuard) || !(rmax <= 127.5f);   // NaN-safe
        if (__any_sync(0xffffffffu, redo)) {
          // Some value of some lane sits next to a rounding boundary (exact ties are common with
          // absmax / 127 scales) or beyond the clamp range.  The 16-wide slices concerned are redone with
          // the IEEE division by the whole warp: for one (lane L, slice) at a time, lanes 0-7 each
          // quantise one of L's eight values of that slice (two tokens x four values) and the bytes
          // are gathered back into L's fragment registers.
          uint32_t todo = 0;
          if (redo) {
            const bool all = !(rmax <= 127.5f);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) todo |= (all || !(um[kk] < kQuantTieGuard)) ? (1u << kk) : 0u;
          }
          const uint8_t* kptr = my_stages + (size_t)st * (2 * PAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t lanes = __ballot_sync(0xffffffffu, (todo >> kk) & 1u);
            while (lanes != 0) {
              const int L = __ffs(lanes) - 1;
              lanes &= lanes - 1;
              const float s0 = __shfl_sync(0xffffffffu, ksr0, L), s1 = __shfl_sync(0xffffffffu, ksr1, L);
              uint32_t w = 0;
              if (lane < 8) {
                const int j = lane >> 2, i = lane & 3;
                const int d = 16 * kk + (L & 3) * 2 + (i & 1) + 8 * (i >> 1);
                w = quant_exact_elem<SLAB_BYTES>(kptr, 8 * j + (L >> 2), d, j ? s1 : s0) << (8 * i);
              }
              w |= __shfl_xor_sync(0xffffffffu, w, 1);
              w |= __shfl_xor_sync(0xffffffffu, w, 2);
              const uint32_t w0 = __shfl_sync(0xffffffffu, w, 0), w1 = __shfl_sync(0xffffffffu, w, 4);
              if (lane == L) {
                bq[0][kk >> 1][kk & 1] = w0;
                bq[1][kk >> 1][kk & 1] = w1;
              }
            }
          }
        }
#pragma unroll
        for (int kk = 0; kk < D / 32; ++kk) {
          mma_s8_rows<HM>(si[0], qa[kk], bq[0][kk][0], bq[0][kk][1]);
          mma_s8_rows<HM>(si[1], qa[kk], bq[1][kk][0], bq[1][kk][1]);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float ks_a = __shfl_sync(0xffffffffu, ks_cur, 8 * j + cq);
          const float ks_b = __shfl_sync(0xffffffffu, ks_cur, 8 * j + cq + 1);
          // score = float(dot) * q_s * k_s * scale, then to base 2
          s[j][0] = ((static_cast<float>(si[j][0]) * q_s0) * ks_a) * p.scale * 1.4426950408889634f;
          s[j][1] = ((static_cast<float>(si[j][1]) * q_s0) * ks_b) * p.scale * 1.4426950408889634f;
          if constexpr (!HM) {
            s[j][2] = ((static_cast<float>(si[j][2]) * q_s1) * ks_a) * p.scale * 1.4426950408889634f;
            s[j][3] = ((static_cast<float>(si[j][3]) * q_s1) * ks_b) * p.scale * 1.4426950408889634f;
          }
          if (p.scores_out != nullptr) {
#pragma unroll
            for (int e = 0; e < NR; ++e) {
              const int row = g + (e >> 1) * 8;
              const int tin = 8 * j + cq + (e & 1);
              if (row < Gb && ((vmask >> tin) & 1u))
                p.scores_out[((size_t)b * p.H_Q + head0 + row) * p.N + page * 16 + tin] = si[j][e];
            }
          }
        }
      }

    };

    // (Computing the scores of page n+1 before the softmax of page n, with a third ring stage, was
    // measured for the INT8 kinds: no gain for INT8-QK, 4 % slower for INT8-KV.)
    for (int n = 0; n < n_my; ++n) {
      const PageState ps_cur = begin_page(n);
      float s[2][4];
      compute_scores(ps_cur, s);
      const uint32_t st = ps_cur.st, vmask = ps_cur.vmask;
      const uint32_t sc_cur = ps_cur.sc;
      const uint32_t vbase = stage0 + st * (2 * PAGE_BYTES) + PAGE_BYTES;
      (void)sc_cur; (void)vbase;

      if (vmask != 0xffffu) {
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < NR; ++e)
            if (!((vmask >> (8 * j + cq + (e & 1))) & 1u)) s[j][e] = -INFINITY;
      }

      // ---- online softmax (base 2) ----------------------------------------------
      float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      const float mn0 = fmaxf(m0, mx0);
      const float a0 = fast_exp2(m0 - mn0);
      m0 = mn0;
      float pr[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        pr[j][0] = fast_exp2(s[j][0] - mn0);
        pr[j][1] = fast_exp2(s[j][1] - mn0);
      }
      l0 = l0 * a0 + (pr[0][0] + pr[0][1] + pr[1][0] + pr[1][1]);
      float a1 = 1.f;
      uint32_t pa[4];
      pa[0] = BF ? pack_bf162(pr[0][0], pr[0][1]) : pack_half2(pr[0][0], pr[0][1]);
      pa[2] = BF ? pack_bf162(pr[1][0], pr[1][1]) : pack_half2(pr[1][0], pr[1][1]);
      pa[1] = pa[3] = 0u;
      if constexpr (!HM) {
        float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn1 = fmaxf(m1, mx1);
        a1 = fast_exp2(m1 - mn1);
        m1 = mn1;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          pr[j][2] = fast_exp2(s[j][2] - mn1);
          pr[j][3] = fast_exp2(s[j][3] - mn1);
        }
        l1 = l1 * a1 + (pr[0][2] + pr[0][3] + pr[1][2] + pr[1][3]);
        pa[1] = BF ? pack_bf162(pr[0][2], pr[0][3]) : pack_half2(pr[0][2], pr[0][3]);
        pa[3] = BF ? pack_bf162(pr[1][2], pr[1][3]) : pack_half2(pr[1][2], pr[1][3]);
      }
      if (__any_sync(0xffffffffu, (a0 != 1.f) || (a1 != 1.f))) {
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          acc[i][0] *= a0;
          acc[i][1] *= a0;
          if constexpr (!HM) {
            acc[i][2] *= a1;
            acc[i][3] *= a1;
          }
        }
      }

      if (!KV8 && vmask != 0xffffu) {
        // zero the V rows of tokens that are not attended so that 0 * garbage cannot make NaN
        uint8_t* vptr = my_stages + (size_t)st * (2 * PAGE_BYTES) + PAGE_BYTES;
        for (int i = lane; i < 16 * 8 * NSLAB; i += 32) {
          const int sl = i / 128, r = i - sl * 128;      // r: row * 8 + chunk
          if (!((vmask >> (r >> 3)) & 1u))
            *reinterpret_cast<uint4*>(vptr + sl * SLAB_BYTES + (r >> 3) * 128 + (r & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
      }

      // ---- O += P V --------------------------------------------------------------
      if constexpr (KV8) {
        // Lane (g, c) reads the NT bytes [NT*g, NT*g + NT) of token rows 2c, 2c+1, 2c+8, 2c+9: byte nt is
        // column g of output tile nt, so accumulator column n of tile nt is head dimension NT*n + nt.
        const uint8_t* vptr = my_stages + (size_t)st * (2 * PAGE_BYTES) + PAGE_BYTES;
        const int c2 = (lane & 3) * 2;
        const uint32_t s_a = __shfl_sync(0xffffffffu, sc_cur, 16 + c2);
        const uint32_t s_b = __shfl_sync(0xffffffffu, sc_cur, 16 + c2 + 1);
        const uint32_t s_c = __shfl_sync(0xffffffffu, sc_cur, 16 + c2 + 8);
        const uint32_t s_d = __shfl_sync(0xffffffffu, sc_cur, 16 + c2 + 9);
        const uint32_t sc_lo = s_a | (s_b << 16), sc_hi = s_c | (s_d << 16);
        constexpr int NW = NT / 4;  // 32-bit words per lane and token row
        uint32_t va[NW], vb[NW], vc[NW], vd[NW];
        load_v_row<D>(vptr, c2, g, va);
        load_v_row<D>(vptr, c2 + 1, g, vb);
        load_v_row<D>(vptr, c2 + 8, g, vc);
        load_v_row<D>(vptr, c2 + 9, g, vd);
#pragma unroll
        for (int wd = 0; wd < NW; ++wd) {
          dequant_v_pair<0, HM>(va[wd], vb[wd], vc[wd], vd[wd], sc_lo, sc_hi, pa, acc[wd * 4 + 0]);
          dequant_v_pair<1, HM>(va[wd], vb[wd], vc[wd], vd[wd], sc_lo, sc_hi, pa, acc[wd * 4 + 1]);
          dequant_v_pair<2, HM>(va[wd], vb[wd], vc[wd], vd[wd], sc_lo, sc_hi, pa, acc[wd * 4 + 2]);
          dequant_v_pair<3, HM>(va[wd], vb[wd], vc[wd], vd[wd], sc_lo, sc_hi, pa, acc[wd * 4 + 3]);
        }
      } else {
        const int mi = lane >> 3;
        const int r = (lane & 7) + (mi & 1) * 8;
#pragma unroll
        for (int c2 = 0; c2 < D / 16; ++c2) {
          const int chunk = 2 * c2 + (mi >> 1);
          const uint32_t addr = vbase + (chunk >> 3) * SLAB_BYTES + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, addr);
          mma_rows<HM, BF>(acc[2 * c2], pa, vb[0], vb[1]);
          mma_rows<HM, BF>(acc[2 * c2 + 1], pa, vb[2], vb[3]);
        }
      }

      if (!KV8 && vmask != 0xffffu) fence_proxy_async();  // generic writes to this stage precede its next TMA fill
      __syncwarp();
      if (issued < n_my) {
        if ((issued & 31) == 0) {
          tbl_cur = tbl_next;
          tbl_next = load_tbl((issued >> 5) + 1);
        }
        issue(issued);
        ++issued;
      } else if (pre_issued < nx_n_my && pre_issued < S) {
        // nothing left to fetch for this piece: the freed stage takes a page of the next piece
        const int pid = __shfl_sync(0xffffffffu, nx_tbl, pre_issued);
        issue_page(nx.p0 + warp + pre_issued * W, pid, nx_h_kv, nx_row0);
        ++pre_issued;
      }
    }

    // ---- merge the warps of this CTA ---------------------------------------------
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    if constexpr (!HM) {
      l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
      l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    }
    {
      float* mb = mbuf + (size_t)warp * p.slot_rows * ROWLEN;
      if (g < Gb) {
        float* rowp = mb + g * ROWLEN;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          if constexpr (KV8) {
            rowp[NT * cq + i] = acc[i][0];
            rowp[NT * (cq + 1) + i] = acc[i][1];
          } else {
            *reinterpret_cast<float2*>(rowp + i * 8 + cq) = make_float2(acc[i][0], acc[i][1]);
          }
        }
        if ((lane & 3) == 0) {
          rowp[D] = m0;
          rowp[D + 1] = l0;
        }
      }
      if (!HM && g + 8 < Gb) {
        float* rowp = mb + (g + 8) * ROWLEN;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          if constexpr (KV8) {
            rowp[NT * cq + i] = acc[i][2];
            rowp[NT * (cq + 1) + i] = acc[i][3];
          } else {
            *reinterpret_cast<float2*>(rowp + i * 8 + cq) = make_float2(acc[i][2], acc[i][3]);
          }
        }
        if ((lane & 3) == 0) {
          rowp[D] = m1;
          rowp[D + 1] = l1;
        }
      }
    }
    __syncthreads();
    {
      const int slot = (piece == 0) ? 0 : 1;
      float* part = p.partials + ((size_t)blockIdx.x * 2 + slot) * p.slot_rows * ROWLEN;
      for (int e = threadIdx.x; e < Gb * D; e += blockDim.x) {
        const int row = e / D, d = e - row * D;
        if (d >= p.D_real) continue;      // padding columns
        float M = -INFINITY;
        for (int w = 0; w < W; ++w) M = fmaxf(M, mbuf[((size_t)w * p.slot_rows + row) * ROWLEN + D]);
        float L = 0.f, O = 0.f;
        for (int w = 0; w < W; ++w) {
          const float* rp = mbuf + ((size_t)w * p.slot_rows + row) * ROWLEN;
          const float f = fast_exp2(rp[D] - M);
          L += rp[D + 1] * f;
          O += rp[d] * f;
        }
        if (complete) {
          p.out[((size_t)b * p.H_Q + head0 + row) * p.D_real + d] = to_out16(O / L, p.out_bf16 != 0);
        } else {
          part[row * ROWLEN + d] = O;
          if (d == 0) {
            part[row * ROWLEN + D] = M;
            part[row * ROWLEN + D + 1] = L;
          }
        }
      }
    }
    if (!complete) {
      // The segment is shared with neighbouring CTAs.  Publish the partial, count the arrival;
      // whoever arrives last merges all partials of the segment.
      const long long seg_start = (long long)p.HV * pre[b] + (long long)hv * np;
      const int first = (int)(seg_start / per), last = (int)((seg_start + np - 1) / per);
      const unsigned int n_parts = (unsigned int)(last - first + 1);
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        // At most one split segment starts in a CTA's range (segments that start and end inside it are
        // complete), so the first CTA of the segment names its counter.
        // One atomic add per arrival (a compare-and-swap loop on a tagged counter serialised the CTAs of a
        // segment: with a few long sequences spread over the whole grid that took longer than the
        // attention itself).  The counter is self-cleaning: the last arriver puts it back to zero, so a
        // workspace needs clearing only once - and again after a launch that recorded a device status,
        // whose counters may be left mid-count.
        unsigned int* cnt = reinterpret_cast<unsigned int*>(p.counters + first);
        const unsigned int arrivals = atomicAdd(cnt, 1u) + 1u;
        s_last_flag = (arrivals == n_parts) ? 1 : 0;
        if (arrivals == n_parts) *reinterpret_cast<volatile unsigned int*>(cnt) = 0u;
      }
      __syncthreads();
      if (s_last_flag) {
        __threadfence();
        __half* outp = p.out + ((size_t)b * p.H_Q + head0) * p.D_real;
        for (int e = threadIdx.x; e < Gb * D; e += blockDim.x) {
          const int row = e / D, d = e - row * D;
          if (d >= p.D_real) continue;
          // The partials sit in L2 (other CTAs wrote them): every read costs an L2 round trip, so the reads
          // of eight partials are issued together before any of them is used.  (A segment is split over
          // up to hundreds of CTAs when few sequences fill the grid; one dependent read per partial made the
          // merge the longest part of such launches.)
          constexpr int MB = 8;
          auto part_row = [&](int c) -> const float* {
            const int slot = ((long long)c * per >= seg_start) ? 0 : 1;
            return p.partials + ((size_t)c * 2 + slot) * p.slot_rows * ROWLEN + row * ROWLEN;
          };
          float M = -INFINITY;
          for (int c0 = first; c0 <= last; c0 += MB) {
            float mv[MB];
#pragma unroll
            for (int k = 0; k < MB; ++k) mv[k] = (c0 + k <= last) ? __ldcg(part_row(c0 + k) + D) : -INFINITY;
#pragma unroll
            for (int k = 0; k < MB; ++k) M = fmaxf(M, mv[k]);
          }
          float L = 0.f, O = 0.f;
          for (int c0 = first; c0 <= last; c0 += MB) {
            float mv[MB], lv[MB], ov[MB];
#pragma unroll
            for (int k = 0; k < MB; ++k) {
              const bool in = c0 + k <= last;
              const float* pr = part_row(in ? c0 + k : last);
              mv[k] = in ? __ldcg(pr + D) : -INFINITY;
              lv[k] = in ? __ldcg(pr + D + 1) : 0.f;
              ov[k] = in ? __ldcg(pr + d) : 0.f;
            }
#pragma unroll
            for (int k = 0; k < MB; ++k) {
              const float f = (mv[k] == -INFINITY) ? 0.f : fast_exp2(mv[k] - M);
              L += lv[k] * f;
              O += ov[k] * f;
            }
          }
          outp[(size_t)row * p.D_real + d] = to_out16(O / L, p.out_bf16 != 0);
        }
      }
    }
    __syncthreads();

    u += cnt;
    ++piece;
  }
}

template <int D, int KIND, bool HM>
cudaError_t launch_t(const CUtensorMap& kmap, const CUtensorMap& vmap, const DecodeParams& p,
                     int warps, size_t smem_bytes, cudaStream_t stream) {
  auto kern = decode_splitkv_kernel<D, KIND, HM>;
  if (warps * 32 > DecodeOccupancy<D, KIND, HM>::kThreads) return cudaErrorInvalidConfiguration;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
  if (e != cudaSuccess) return e;
  if (p.B + 1 > kMaxSmemPrefix) decode_plan_kernel<<<1, 1024, 0, stream>>>(p);  // else scanned in-kernel
  kern<<<p.n_cta, warps * 32, smem_bytes, stream>>>(kmap, vmap, p);
  return cudaGetLastError();
}

}  // namespace

size_t decode_smem_bytes(int D, int warps, int stages, int slot_rows, int B, int kv_elem_bytes) {
  size_t bytes = 1024;  // slack to align the first stage to 1024 B (128-byte swizzle atom)
  bytes += (size_t)warps * stages * (2 * 16 * D * kv_elem_bytes);
  bytes += (size_t)warps * stages * 8;
  bytes += (size_t)warps * slot_rows * (D + 2) * 4;
  if (B + 1 <= kMaxSmemPrefix) bytes += (size_t)(B + 1) * 4;
  return (bytes + 15) & ~(size_t)15;
}

size_t decode_workspace_bytes(int B, int H_Q, int H_KV, int D, int max_ctas) {
  const int G = H_Q / H_KV;
  const int slot_rows = G < 16 ? G : 16;
  const int HV = H_KV * ((G + 15) / 16);
  (void)HV;
  size_t bytes = kWsPrefixOffset;
  bytes += ((size_t)(B + 1) * 4 + 255) & ~(size_t)255;
  bytes += (size_t)max_ctas * 2 * slot_rows * (D + 2) * 4;
  return (bytes + 255) & ~(size_t)255;
}

cudaError_t launch_decode(const CUtensorMap& kmap, const CUtensorMap& vmap, const DecodeParams& p,
                          int D, int kind, int warps, size_t smem_bytes, cudaStream_t stream) {
#define FA_DECODE_KIND(DD, KK)                                                              \
  return p.G <= 8 ? launch_t<DD, KK, true>(kmap, vmap, p, warps, smem_bytes, stream)        \
                  : launch_t<DD, KK, false>(kmap, vmap, p, warps, smem_bytes, stream);
#define FA_DECODE_CASE(DD)                               \
  case DD:                                               \
    if (kind == kKindInt8QK) { FA_DECODE_KIND(DD, kKindInt8QK) } \
    if (kind == kKindInt8KV) { FA_DECODE_KIND(DD, kKindInt8KV) } \
    if (kind == kKindBF16) { FA_DECODE_KIND(DD, kKindBF16) } \
    FA_DECODE_KIND(DD, kKindF16)
  switch (D) {
    FA_DECODE_CASE(64)
    FA_DECODE_CASE(128)
    FA_DECODE_CASE(256)
    default:
      return cudaErrorInvalidValue;
  }
#undef FA_DECODE_CASE
#undef FA_DECODE_KIND
}

}  // namespace fa
