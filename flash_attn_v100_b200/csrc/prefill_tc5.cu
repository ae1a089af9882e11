// Causal / non-causal GQA prefill on 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// Replaces the reference's prefill kernels (flash_attn_kernel.cu:1138-1299, 2471-2605,
// 3005-3148) for D = 64 and D = 128, dense [B,H,N,D] and packed varlen [total,H,D].
//
// One CTA works on TWO 128-row query tiles that share one KV head and one KV range, so
// every K/V tile staged in shared memory feeds two score tiles:
//   - "head pair" mode (even group size): the same 128 rows of two adjacent query heads;
//   - "row pair" mode: two consecutive 128-row blocks of one query head.
// Warp roles (12 warps):
//   warp 0      TMA producer: Q once, then K_j / V_j tiles (128 keys) through a ring
//   warps 1, 3  MMA issuers (one lane each, warp 1 for tile 0 and warp 3 for tile 1):
//               S_t = Q_t K_j^T and O_t += P_t V_j with tcgen05.mma, accumulators in tensor
//               memory; completion signalled by tcgen05.commit; a token alternates the two
//   warp 2      tensor-memory allocation / release
//   warps 4-7   softmax of tile 0 (thread = one query row = one TMEM lane)
//   warps 8-11  softmax of tile 1
// The two softmax groups ping-pong: while one group turns S_0 into P_0, the tensor core
// runs the other tile's MMAs.  P is written back to tensor memory as fp16 over the first
// half of the S columns it came from and is the A operand of the PV MMA (no shared-memory
// round trip).  Softmax is fp32, base 2, online across KV tiles; O is rescaled in tensor
// memory only when a row maximum grows by more than 2^8 (stale maxima keep P <= 256, exact
// in fp16 range and compensated in the fp32 row sum).  Causal tiles above the diagonal are
// skipped; only the diagonal tile and the ragged last tile are masked per element.
//
// The kernel is persistent: one CTA per SM claims work items (tile pairs, heaviest first) from
// a global counter; barrier phases are running counters, so the copy and MMA lanes start the
// next item while the softmax groups still write the previous item's output.
//
// Tensor-memory map (512 columns x 128 lanes): S_0 [0,128) S_1 [128,256) O_0 [256,256+D)
// O_1 [256+D, 256+2D).  Every wait on an mbarrier is bounded; on a timeout the CTA sets an
// abort flag, records a status bit and runs to completion without further waiting.
#include "common.cuh"
#include "prefill.cuh"

#include <atomic>
#include <mutex>

namespace fa {

__device__ int g_prefill_status = 0;

#ifdef FA_TC5_PROF
// Instrumented build only (-DFA_TC5_PROF): cycles that one thread of each role spends in each kind of
// wait, summed over all CTAs.  Roles: 0 copy lane, 1/2 MMA lanes, 3/4 the thread of row 0 of each softmax group.
__device__ unsigned long long g_tc5_prof[5 * 16];
#define PROF_WAIT(role, cat, stmt)                                                     \
  do {                                                                                 \
    const long long prof_a_ = clock64();                                               \
    stmt;                                                                              \
    if (prof_on) prof_smem[(role) * 16 + (cat)] += (unsigned long long)(clock64() - prof_a_); \
  } while (0)
#define PROF_MARK(var) const long long var = clock64()
#define PROF_SPAN(role, cat, a, b) \
  do { if (prof_on) prof_smem[(role) * 16 + (cat)] += (unsigned long long)((b) - (a)); } while (0)
#define PROF_COUNT(role, cat) \
  do { if (prof_on) prof_smem[(role) * 16 + (cat)] += 1ull; } while (0)
// cross-role latencies: one role stamps the clock, another adds the time since that stamp
#define PROF_STAMP(idx) do { if (prof_on) prof_smem[5 * 16 + (idx)] = (unsigned long long)clock64(); } while (0)
#define PROF_SINCE(role, cat, idx) \
  do { if (prof_on) prof_smem[(role) * 16 + (cat)] += (unsigned long long)clock64() - prof_smem[5 * 16 + (idx)]; } while (0)
#else
#define PROF_STAMP(idx) do { } while (0)
#define PROF_SINCE(role, cat, idx) do { } while (0)
#define PROF_WAIT(role, cat, stmt) do { stmt; } while (0)
#define PROF_MARK(var) do { } while (0)
#define PROF_SPAN(role, cat, a, b) do { } while (0)
#define PROF_COUNT(role, cat) do { } while (0)
#endif

namespace {

constexpr uint32_t kTc5MaxPolls = 1u << 21;

struct Tc5Params {
  __half* out;
  const int32_t* cu_seqlens;
  int batch, H_Q, H_KV, N, max_seqlen;
  long long total;
  long long o_batch_stride, o_head_stride, o_tok_stride;
  int causal;
  int D_real;      // head dimension of the tensors (columns [D_real, D) read as zeros through the tensor maps)
  int pair_heads;  // 1: two heads x same rows; 0: one head x two row blocks
  int dense;
  int out_bf16;    // store O as bfloat16 instead of fp16
  int n_hg, n_rb;  // head groups and row blocks of the item grid (items = n_rb * batch * n_hg)
  unsigned long long* item_counter;  // next unclaimed item of this launch (zeroed in-stream before it)
  float scale_log2;
};

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test_wait(bar, parity)) return true;  // cheap probe: the phase is usually complete already
  for (uint32_t i = 0; i < kTc5MaxPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicOr(&g_prefill_status, kStatusWaitTimeout);
  return false;
}

// The same wait as a plain polling loop (mbarrier.test_wait never suspends the thread): tuning builds only.
template <bool SPIN>
__device__ __forceinline__ bool wait_sel(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if constexpr (!SPIN) {
    return wait_or_abort(bar, parity, abort_flag);
  } else {
    for (uint32_t i = 0; i < (kTc5MaxPolls << 2); ++i) {
      if (mbar_test_wait(bar, parity)) return true;
      if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicOr(&g_prefill_status, kStatusWaitTimeout);
    return false;
  }
}

// Bounded wait that does not look at the abort flag: used on the way out, to let asynchronous copies and
// MMAs that are still in flight finish before shared and tensor memory are given up.
__device__ __forceinline__ void drain_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kTc5MaxPolls; ++i)
    if (mbar_try_wait(bar, parity)) return;
  atomicOr(&g_prefill_status, kStatusWaitTimeout);
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// The MMA role runs with its whole warp converged and lets one elected lane issue (elect.sync): the
// addresses and descriptors are then uniform across the warp, which keeps the instruction stream of the
// issuing warp short (it shares its scheduler with four softmax warps).  Commits are issued the same way,
// so that they track the MMAs of the same thread.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  __syncwarp();
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar)
      : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// Packed fp32x2 arithmetic (one issue slot for two lanes of work).
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  uint64_t ra = *reinterpret_cast<uint64_t*>(&a), rb = *reinterpret_cast<uint64_t*>(&b),
           rc = *reinterpret_cast<uint64_t*>(&c), rd;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  return *reinterpret_cast<float2*>(&rd);
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  uint64_t ra = *reinterpret_cast<uint64_t*>(&a), rb = *reinterpret_cast<uint64_t*>(&b), rd;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  return *reinterpret_cast<float2*>(&rd);
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^x (x clamped to [-125, 126]) on the FMA/ALU pipes (keeps the MUFU free for the other half of the row):
// round-to-nearest split x = n + f with the 1.5*2^23 trick, degree-3 minimax polynomial for 2^f on
// [-0.5, 0.5] (relative error 7.7e-5, below fp16 resolution), exponent added through the integer bits.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  const float kMagic = 12582912.f;
  x.x = fminf(fmaxf(x.x, -125.f), 126.f);   // 2^126 still trips every overflow check downstream
  x.y = fminf(fmaxf(x.y, -125.f), 126.f);
  const float2 t = fadd2(x, make_float2(kMagic, kMagic));
  const float2 n = fadd2(t, make_float2(-kMagic, -kMagic));
  const float2 f = ffma2(n, make_float2(-1.f, -1.f), x);
  float2 r = ffma2(make_float2(0.05508868f, 0.05508868f), f, make_float2(0.24260405f, 0.24260405f));
  r = ffma2(r, f, make_float2(0.69327623f, 0.69327623f));
  r = ffma2(r, f, make_float2(0.99992895f, 0.99992895f));
  // bits(r) + (n << 23): one integer multiply-add each (the low bits of t hold n; overflow of the product is meant)
  r.x = __uint_as_float(__float_as_uint(t.x) * 0x800000u + __float_as_uint(r.x));
  r.y = __uint_as_float(__float_as_uint(t.y) * 0x800000u + __float_as_uint(r.y));
  return r;
}

// Which of the 16 value pairs of a 32-column chunk are exponentiated by the polynomial: NPOLY pairs of
// every eight, spread evenly so that polynomial and MUFU work interleave in the instruction stream.
template <int NPOLY>
__device__ __forceinline__ constexpr bool pair_uses_poly(int i) {
  return (((i & 7) * NPOLY) % 8) < NPOLY;
}

// One 32-column chunk of a score row: P = exp2(s * scale - m) as fp16 pairs, written to tensor memory at
// `taddr` (16 columns); the fp32 sum of the chunk is added to `rs`.
template <int NPOLY, int DBG = 0, bool BF = false>
__device__ __forceinline__ void exp_chunk_store(const float (&s)[32], float2 sc2, float2 nm2, float2& rs,
                                                uint32_t taddr) {
  uint32_t pk[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 x = ffma2(make_float2(s[2 * i], s[2 * i + 1]), sc2, nm2);
    float2 e;
    if (DBG & 1) {   // timing experiments only: no exponential
      e = x;
    } else if (pair_uses_poly<NPOLY>(i)) {
      e = exp2_poly2(x);
    } else {
      e.x = fast_exp2(x.x);
      e.y = fast_exp2(x.y);
    }
    rs = fadd2(rs, e);
    pk[i] = (DBG & 8) ? __float_as_uint(e.x) : (BF ? pack_bf162(e.x, e.y) : pack_half2(e.x, e.y));   // DBG 8: no conversion
  }
  tc_st16(taddr, pk);
}

__device__ __forceinline__ void zero_chunk_store(uint32_t taddr) {
  uint32_t pk[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) pk[i] = 0u;
  tc_st16(taddr, pk);
}

// Shared-memory matrix descriptor for 128-byte-swizzled tiles made of 128-byte rows.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // 128-byte swizzle
  return d;
}

// Work item = one pair of query tiles.  Items are numbered with the row block as the slowest
// index, running backwards, so the items with the most KV tiles (late causal blocks of the long
// sequences) come first.  CTAs claim items from a global counter (heaviest-first greedy
// scheduling): the copy lane claims, skips empty items, and publishes the item number to the
// other roles of its CTA through a small shared-memory queue.
struct Tc5Item {
  int head[2], row0[2], n_kv[2];
  int q_c1[2], q_c2[2], kv_c1, kv_c2;
  int seq, len, n_max;
  long long tok0;
};

__device__ __forceinline__ bool tc5_decode_item(const Tc5Params& p, long long item, Tc5Item& it) {
  constexpr int BM = 128, BN = 128;
  const int hg = (int)(item % p.n_hg);
  const long long r1 = item / p.n_hg;
  const int seq = (int)(r1 % p.batch);
  const int rb = p.n_rb - 1 - (int)(r1 / p.batch);
  if (p.pair_heads) {
    it.head[0] = 2 * hg; it.head[1] = it.head[0] + 1;
    it.row0[0] = it.row0[1] = rb * BM;
  } else {
    it.head[0] = it.head[1] = hg;
    it.row0[0] = rb * 2 * BM; it.row0[1] = it.row0[0] + BM;
  }
  const int h_kv = it.head[0] / (p.H_Q / p.H_KV);
  int len;
  if (p.cu_seqlens != nullptr) {
    const int a = __ldg(p.cu_seqlens + seq), e = __ldg(p.cu_seqlens + seq + 1);
    it.tok0 = a;
    len = e - a;
    if ((long long)e > p.total) len = (int)(p.total - a);
  } else {
    it.tok0 = 0;
    len = p.N;
  }
  if (len > p.max_seqlen) len = p.max_seqlen;
  it.len = len;
  it.seq = seq;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    if (it.row0[t] >= len) it.n_kv[t] = 0;
    else {
      const int kv_end = p.causal ? ((it.row0[t] + BM) < len ? (it.row0[t] + BM) : len) : len;
      it.n_kv[t] = (kv_end + BN - 1) / BN;
    }
    if (p.dense) { it.q_c1[t] = 0; it.q_c2[t] = (seq * p.H_Q + it.head[t]) * p.N + it.row0[t]; }
    else { it.q_c1[t] = it.head[t]; it.q_c2[t] = (int)it.tok0 + it.row0[t]; }
  }
  if (p.dense) { it.kv_c1 = 0; it.kv_c2 = (seq * p.H_KV + h_kv) * p.N; }
  else { it.kv_c1 = h_kv; it.kv_c2 = (int)it.tok0; }
  it.n_max = it.n_kv[0] > it.n_kv[1] ? it.n_kv[0] : it.n_kv[1];
  return it.n_kv[0] > 0;  // tile 0 holds the earlier rows: if it is empty the item is empty
}

// NPOLY: value pairs of every eight whose exp2 runs as a polynomial on the FMA pipes (0..4);
// SM: 0 every tile takes the full softmax path (row maximum and rescale decision first); 1 tiles that need no
// masking take the fast path described in the softmax role.
// DBG (tuning builds only, results are wrong): 1 no exp2, 2 no PV MMAs, 4 no QK MMAs, 8 no fp16 conversion,
// 16 the softmax hands over at once without computing anything, 32 no turn taking between the tiles (valid results).
// BF: q, k, v are bfloat16: the same kernel with bfloat16 MMA operands and P rounded to bfloat16.
template <int D, int NPOLY, int SM, int DBG = 0, bool BF = false>
__global__ void __launch_bounds__(640, 1)
prefill_tc5_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                   const __grid_constant__ CUtensorMap vmap, const Tc5Params p) {
  constexpr int BM = 128, BN = 128;
  constexpr int KV_STAGES = (D == 128) ? 2 : 4;
  constexpr int SLAB = 128 * 128;            // bytes of a [128 rows][64 cols] fp16 slab
  constexpr int NSLAB = D / 64;
  constexpr int TILE_BYTES = NSLAB * SLAB;   // one Q / K / V tile
  // instruction descriptor of kind::f16: fp32 accumulators (bit 4), operand formats (bits 7 and 10: 1 = bfloat16),
  // B taken MN-major for PV (bit 16), N / 8 at bit 17, M / 16 at bit 24
  constexpr uint32_t IDESC_FMT = BF ? ((1u << 7) | (1u << 10)) : 0u;
  constexpr uint32_t IDESC_QK = (1u << 4) | IDESC_FMT | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  constexpr uint32_t IDESC_PV =
      (1u << 4) | IDESC_FMT | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t O_COL0 = 256;
  // P (fp16, 64 columns = four quarters of 16) lies over columns [16, 80) of its S, and the quarters hold the
  // keys of the score chunks 0, 1, 3, 2 in that order.  With this placement every quarter is written over
  // score columns that its writer already holds in registers (see the softmax role), so the two threads of a
  // row never overwrite scores the other one still has to read from tensor memory.
  constexpr uint32_t P_COL = 16;
  constexpr int kItemQ = 4;                  // depth of the per-CTA item queue
  constexpr int kItemConsumers = 1 + 2 + 16; // the copy lane, two MMA lanes, one arrival per softmax warp

  extern __shared__ uint8_t smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  uint8_t* smem = smem_dyn + ((1024u - (raw & 1023u)) & 1023u);
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + 2 * TILE_BYTES;
  const uint32_t sV = sK + KV_STAGES * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 + 2 * KV_STAGES) * TILE_BYTES);
  // barrier indices
  constexpr int B_QFULL = 0, B_QEMPTY = 2, B_KFULL = B_QEMPTY + 2, B_KEMPTY = B_KFULL + KV_STAGES,
                B_VFULL = B_KEMPTY + KV_STAGES, B_VEMPTY = B_VFULL + KV_STAGES, B_SFULL = B_VEMPTY + KV_STAGES,
                B_PFULL = B_SFULL + 2, B_TOKEN = B_PFULL + 2,
                B_IFULL = B_TOKEN + 2, B_IEMPTY = B_IFULL + kItemQ, B_PAIR = B_IEMPTY + kItemQ,
                B_DRAIN = B_PAIR + 8, B_TURN = B_DRAIN + 2, B_COUNT = B_TURN + 2;
  volatile long long* item_slot = reinterpret_cast<volatile long long*>(bars + B_COUNT);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT + kItemQ);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // exchange area of the softmax role: per tile, three slots of [half][row] floats, and one redo tag per row quadrant
  float* xchg = reinterpret_cast<float*>(bars + 64);
  volatile uint32_t* redo_tag = reinterpret_cast<volatile uint32_t*>(xchg + 2 * 3 * 2 * 128);
  auto bar = [&](int i) -> uint32_t { return smem_u32(bars + i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long n_items = (long long)p.n_rb * p.batch * p.n_hg;
#ifdef FA_TC5_PROF
  unsigned long long* prof_smem = reinterpret_cast<unsigned long long*>(xchg + 2 * 3 * 2 * 128 + 8);
  if (threadIdx.x < 5 * 16) prof_smem[threadIdx.x] = 0ull;
  bool prof_on = false;    // true in the one thread per role that keeps the counters
  const long long prof_start = clock64();
#endif

  // ---- set-up (once per CTA) --------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(bar(B_KFULL + s), 1);
      mbar_init(bar(B_KEMPTY + s), 2);   // one arrival per issuing lane and use (see the MMA issuers)
      mbar_init(bar(B_VFULL + s), 1);
      mbar_init(bar(B_VEMPTY + s), 2);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar(B_QFULL + t), 1);
      mbar_init(bar(B_QEMPTY + t), 1);
      mbar_init(bar(B_SFULL + t), 1);
      mbar_init(bar(B_PFULL + t), 8);     // one arrival per softmax warp of the tile
      mbar_init(bar(B_TOKEN + t), 1);
      mbar_init(bar(B_DRAIN + t), 1);
      mbar_init(bar(B_TURN + t), 8);      // one arrival per softmax warp of the OTHER tile
    }
    for (int i = 0; i < 8; ++i) mbar_init(bar(B_PAIR + i), 64);   // the two warps that share 32 query rows
    for (int i = 0; i < kItemQ; ++i) {
      mbar_init(bar(B_IFULL + i), 1);
      mbar_init(bar(B_IEMPTY + i), kItemConsumers);
    }
    *abort_flag = 0;
    for (int i = 0; i < 8; ++i) redo_tag[i] = 0u;
    mbar_fence_init();
    fence_proxy_async();
    tma_prefetch_desc(&qmap);
    tma_prefetch_desc(&kmap);
    tma_prefetch_desc(&vmap);
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Running counters (identical in every role because every role walks the same item list):
  //   kv_it   KV tiles of all items so far        -> ring stage and phase of K/V barriers
  //   blk[t]  KV steps of tile t so far           -> phase of S / P / O barriers of tile t
  //   q_cnt / q_used[t]  items in which tile t was active -> phase of the Q barriers of tile t
  if (warp == 0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    // ============================ TMA producer ======================================
    if (lane == 0) {
#ifdef FA_TC5_PROF
      prof_on = true;
#endif
      uint32_t kv_it = 0;
      uint32_t q_used[2] = {0, 0};   // how often each Q buffer has been filled
      for (uint32_t ic = 0;; ++ic) {
        if (*abort_flag) break;
        // next item from the queue that warp 2 fills (-1: no more items)
        const int slot = ic % kItemQ;
        PROF_WAIT(0, 0, wait_or_abort(bar(B_IFULL + slot), (ic / kItemQ) & 1u, abort_flag));
        const long long item = item_slot[slot];
        mbar_arrive(bar(B_IEMPTY + slot));
        if (item < 0 || item >= n_items) break;
        Tc5Item it;
        tc5_decode_item(p, item, it);
        const int n_act = it.n_kv[1] > 0 ? 2 : 1;
        // Q buffers are free once the last QK of their previous item has completed
        for (int t = 0; t < n_act; ++t) {
          if (q_used[t] > 0) PROF_WAIT(0, 2, wait_or_abort(bar(B_QEMPTY + t), (q_used[t] - 1) & 1u, abort_flag));
          mbar_expect_tx(bar(B_QFULL + t), TILE_BYTES);
#pragma unroll
          for (int sl = 0; sl < NSLAB; ++sl)
            tma_load_3d(sQ + t * TILE_BYTES + sl * SLAB, &qmap, sl * 64, it.q_c1[t], it.q_c2[t],
                        bar(B_QFULL + t));
          ++q_used[t];
        }
        for (int j = 0; j < it.n_max; ++j, ++kv_it) {
          const int st = kv_it % KV_STAGES;
          const uint32_t ph = (kv_it / KV_STAGES) & 1u;
          if (kv_it >= KV_STAGES) PROF_WAIT(0, 3, wait_or_abort(bar(B_KEMPTY + st), ph ^ 1u, abort_flag));
          mbar_expect_tx(bar(B_KFULL + st), TILE_BYTES);
#pragma unroll
          for (int sl = 0; sl < NSLAB; ++sl)
            tma_load_3d(sK + st * TILE_BYTES + sl * SLAB, &kmap, sl * 64, it.kv_c1, it.kv_c2 + j * BN,
                        bar(B_KFULL + st));
          if (kv_it >= KV_STAGES) PROF_WAIT(0, 4, wait_or_abort(bar(B_VEMPTY + st), ph ^ 1u, abort_flag));
          mbar_expect_tx(bar(B_VFULL + st), TILE_BYTES);
#pragma unroll
          for (int sl = 0; sl < NSLAB; ++sl)
            tma_load_3d(sV + st * TILE_BYTES + sl * SLAB, &vmap, sl * 64, it.kv_c1, it.kv_c2 + j * BN,
                        bar(B_VFULL + st));
        }
      }
      // On the way out every copy issued above must have landed (on a regular exit they all have been
      // consumed; after an abort some may still be in flight): the last fill of every stage and Q buffer.
      for (int st = 0; st < KV_STAGES; ++st) {
        if (kv_it > (uint32_t)st) {
          const uint32_t last = kv_it - 1u - ((kv_it - 1u - (uint32_t)st) % KV_STAGES);   // last tile of this stage
          drain_wait(bar(B_KFULL + st), (last / KV_STAGES) & 1u);
          drain_wait(bar(B_VFULL + st), (last / KV_STAGES) & 1u);
        }
      }
      for (int t = 0; t < 2; ++t)
        if (q_used[t] > 0) drain_wait(bar(B_QFULL + t), (q_used[t] - 1u) & 1u);
    }
  } else if (warp == 1 || warp == 3) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    // ============================ MMA issuers =======================================
    // One issuing lane per query tile (warp 1: tile 0, warp 3: tile 1).  A token passed
    // between the two lanes keeps the issue order  QK(0,0) QK(1,0) | PV(0,j) QK(0,j+1) |
    // PV(1,j) QK(1,j+1) | ...  so the tiles stay half a period apart (one tile's softmax
    // overlaps the other tile's MMAs) while each lane's barrier waits, fences and commits
    // overlap the other lane's MMAs.  K/V stages are released when BOTH lanes have committed
    // (a lane whose tile does not use a stage arrives on it directly).
    const int t = warp == 1 ? 0 : 1;
    {
#ifdef FA_TC5_PROF
      prof_on = (lane == 0);
#endif
      constexpr uint32_t TILE16 = TILE_BYTES >> 4;
      const uint64_t qd = smem_desc(sQ + (uint32_t)t * TILE_BYTES, 16, 1024);
      const uint64_t kd0 = smem_desc(sK, 16, 1024);
      const uint64_t vd0 = smem_desc(sV, SLAB, 1024);
      const uint32_t dS = tmem_base + (uint32_t)t * 128u;
      const uint32_t dO = tmem_base + O_COL0 + (uint32_t)t * D;
      auto issue_qk = [&](int st) {
        __syncwarp();   // the lanes leave their barrier waits one by one; elect.sync needs them together
        const uint64_t b0 = kd0 + (uint64_t)((uint32_t)st * TILE16);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          constexpr uint32_t kSlab16 = SLAB >> 4;
          const uint32_t off = (uint32_t)(ks >> 2) * kSlab16 + (uint32_t)(ks & 3) * 2u;
          tc_mma_ss(dS, qd + off, b0 + off, IDESC_QK, ks > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int st, uint32_t acc) {
        __syncwarp();
        const uint64_t b0 = vd0 + (uint64_t)((uint32_t)st * TILE16);
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          // P quarter ks / 2 holds the keys of score chunk {0, 1, 3, 2}[ks / 2]: pick the matching rows of V
          const int kv = ks < 4 ? ks : (ks ^ 2);
          tc_mma_ts(dO, dS + P_COL + (uint32_t)ks * 8u, b0 + (uint32_t)kv * 128u, IDESC_PV, (acc | (ks > 0 ? 1u : 0u)));
        }
      };
      uint32_t kv_it = 0, q_cnt = 0, blk = 0, tok_waits = 0;
      for (uint32_t ic = 0;; ++ic) {
        if (*abort_flag) break;
        const int slot = ic % kItemQ;
        PROF_WAIT(1 + t, 0, wait_or_abort(bar(B_IFULL + slot), (ic / kItemQ) & 1u, abort_flag));
        const long long item = item_slot[slot];
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_IEMPTY + slot));
        if (item < 0 || item >= n_items) break;
        Tc5Item it;
        tc5_decode_item(p, item, it);
        const bool other_active = it.n_kv[1] > 0;   // tile 0 is always active in a non-empty item
        const int n_mine = it.n_kv[t];
        auto take_token = [&]() {
          if (!other_active) return;
          PROF_WAIT(1 + t, 6, wait_sel<(DBG & 64) != 0>(bar(B_TOKEN + t), tok_waits & 1u, abort_flag));
          ++tok_waits;
        };
        auto pass_token = [&]() {
          if (other_active && lane == 0) mbar_arrive(bar(B_TOKEN + (t ^ 1)));
        };
        if (n_mine > 0) {
          // block 0: S = Q K_0^T
          PROF_WAIT(1 + t, 1, wait_or_abort(bar(B_QFULL + t), q_cnt & 1u, abort_flag));
          ++q_cnt;
          {
            const int st = kv_it % KV_STAGES;
            PROF_WAIT(1 + t, 2, wait_or_abort(bar(B_KFULL + st), (kv_it / KV_STAGES) & 1u, abort_flag));
            tc_fence_after();
            if (t == 1) take_token();
            if (!(DBG & 4)) issue_qk(st);
            pass_token();
            tc_commit(bar(B_SFULL + t));
          }
          for (int j = 0; j < n_mine; ++j, ++blk) {
            const uint32_t g = kv_it + (uint32_t)j;
            const int st = g % KV_STAGES;
            const uint32_t ph = (g / KV_STAGES) & 1u;
            const bool more = j + 1 < n_mine;
            const int st1 = (g + 1) % KV_STAGES;
            const uint32_t ph1 = ((g + 1) / KV_STAGES) & 1u;
            PROF_COUNT(1 + t, 14);
            PROF_WAIT(1 + t, 3, wait_sel<(DBG & 64) != 0>(bar(B_VFULL + st), ph, abort_flag));
            if (more) PROF_WAIT(1 + t, 4, wait_sel<(DBG & 64) != 0>(bar(B_KFULL + st1), ph1, abort_flag));
            PROF_WAIT(1 + t, 5, wait_sel<(DBG & 64) != 0>(bar(B_PFULL + t), blk & 1u, abort_flag));
            PROF_SINCE(1 + t, 9, 2 + t);      // P arrival (row 0's warp) -> seen by the MMA lane
            // tile 1's block j+1 follows tile 0's block j+1; tile 0's block j+1 follows tile 1's
            // block j, which exists unless tile 1 has already run out of KV tiles
            if (t == 1 || j <= it.n_kv[1]) take_token();
            PROF_MARK(prof_t_i);
            tc_fence_after();
            if (!(DBG & 2)) issue_pv(st, j > 0 ? 1u : 0u);
            if (more && !(DBG & 4)) issue_qk(st1);
            pass_token();
            // ONE commit per batch (a tcgen05.commit costs the tensor pipe about as much as an MMA): the
            // batch barrier tells the softmax group that S(j+1) is complete and O holds PV(j); that group
            // passes the news on to the copy lane (K / V stages and the Q buffer that have become free)
            tc_commit(bar(B_SFULL + t));
            PROF_STAMP(t);
            PROF_MARK(prof_t_c);
            PROF_SPAN(1 + t, 11, prof_t_i, prof_t_c);   // issue of PV_hi + QK + commit
          }
          if (other_active) {
            // balance the token barriers before the next item: tile 0 hands tile 1 the token for a
            // block that tile 0 does not have (one more KV tile under causal masking in row-pair
            // mode) and then takes tile 1's final pass; each barrier sees one arrival per wait
            if (t == 0) {
              if (it.n_kv[1] > it.n_kv[0]) {
                take_token();
                pass_token();
              }
              take_token();
            }
          }
        }
        // Stages of this item that my tile does not use still need my arrival to be released.  The
        // arrival is made only after the stage's data has landed, i.e. after the barrier's previous
        // phase has completed, so that it can never be counted for the stage's previous use.
        for (int j = n_mine; j < it.n_max; ++j) {
          const uint32_t g = kv_it + (uint32_t)j;
          const int st = g % KV_STAGES;
          const uint32_t ph = (g / KV_STAGES) & 1u;
          PROF_WAIT(1 + t, 8, wait_or_abort(bar(B_KFULL + st), ph, abort_flag));
          if (lane == 0) mbar_arrive(bar(B_KEMPTY + st));
          PROF_WAIT(1 + t, 8, wait_sel<(DBG & 64) != 0>(bar(B_VFULL + st), ph, abort_flag));
          if (lane == 0) mbar_arrive(bar(B_VEMPTY + st));
        }
        kv_it += (uint32_t)it.n_max;
      }
      // every MMA of this lane must be complete before tensor memory is released
      tc_commit(bar(B_DRAIN + t));
      drain_wait(bar(B_DRAIN + t), 0u);
    }
  } else if (warp == 2) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    // ============================ item claimer ======================================
    // Claims work items from the global counter, skips the empty ones (row blocks past the end of a
    // sequence) and publishes the others through the item queue, up to kItemQ items ahead of the slowest
    // role: the latency of the global atomic stays off every other role's path.
    if (lane == 0) {
      for (uint32_t ic = 0;; ++ic) {
        if (*abort_flag) break;
        Tc5Item it;
        long long item;
        bool have = false;
        while (true) {
          item = (long long)atomicAdd(p.item_counter, 1ULL);
          if (item >= n_items) break;
          if (tc5_decode_item(p, item, it)) { have = true; break; }
        }
        const int slot = ic % kItemQ;
        if (ic >= kItemQ) wait_or_abort(bar(B_IEMPTY + slot), ((ic / kItemQ) & 1u) ^ 1u, abort_flag);
        item_slot[slot] = have ? item : -1;
        mbar_arrive(bar(B_IFULL + slot));
        if (!have) break;
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    // ============================ softmax groups ====================================
    // Sixteen warps: two per (query tile, row quadrant).  TWO threads share a query row: thread h of the pair
    // handles chunk h (32 columns) of the first part of the row and chunk 2 + h of the second part, half of the
    // O columns in every rescale and in the epilogue, and keeps the sum of its own columns.  Two warps per
    // scheduler and tile hide each other's tensor-memory round trips and MUFU latency; the row state that
    // must agree between the two threads (the reference exponent m) changes only on paths where they meet
    // at a 64-thread named barrier.
    // State per row: m (any finite number works as long as P = exp2(s * scale - m) stays inside the fp16
    // range), the partial row sums relative to m, and O in tensor memory, also relative to m.
    //   full path (first KV tile of an item, tiles that need masking, rows that left the window below): the
    //     two halves exchange their maxima through shared memory, m is raised when the row maximum grows by
    //     more than 2^8 with O rescaled in tensor memory, then the exponentials.
    //   fast path (SM 1, other tiles): no dependent chain in front of the exponentials.  The first-part chunk is
    //     exponentiated against the m carried over from the previous step while the raw maximum of the
    //     second-part chunk is formed in the same instruction stream; the step goes ahead if the first part's
    //     sum shows that nothing exceeded 2^15 and the second part's maximum stays below m + 15 (so P fits
    //     fp16) in BOTH warps of the pair (a tag in shared memory and the named barrier); otherwise nothing
    //     has been handed over yet and the step is redone on the full path.
    const int t = (warp - 4) >> 3;
    const int h = ((warp - 4) >> 2) & 1;       // which thread of the row pair
    const int wq = warp & 3;                   // TMEM lane quadrant of this warp
    const int row = wq * 32 + lane;            // row within the tile == TMEM lane
    const uint32_t lane_base = tmem_base + ((uint32_t)(wq * 32) << 16);
    const uint32_t tS = lane_base + (uint32_t)t * 128u;
    const uint32_t tP = tS + P_COL;
    const uint32_t tO = lane_base + O_COL0 + (uint32_t)t * D + (uint32_t)h * (D / 2);
    const int c_lo = h, c_hi = 2 + h;          // my 32-column chunks of the score row
    const int q_lo = h, q_hi = 3 - h;          // the quarters of P that their exponentials go to
    const uint32_t pair_bar = bar(B_PAIR + t * 4 + wq);
    uint32_t pair_ph = 0;    // completed phases of the pair barrier
    float* xch = xchg + t * (3 * 2 * 128);     // [slot][half][row]
    volatile uint32_t* my_tag = redo_tag + t * 4 + wq;
    // meeting point of the two warps of a row pair (orders their shared-memory exchange); a bounded wait like
    // every other wait of this kernel
    auto pair_sync = [&]() {
      mbar_arrive(pair_bar);
      wait_or_abort(pair_bar, pair_ph & 1u, abort_flag);
      ++pair_ph;
    };
    // hand-over of a finished P tile to the MMA lane: one arrival per warp
    auto hand_over = [&]() {
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_PFULL + t));
    };
#ifdef FA_TC5_PROF
    prof_on = (h == 0 && row == 0);
#endif
    // The exponentials of the two tiles take turns (tile 0, tile 1, tile 0, ...).  Both tiles share the four
    // MUFU pipes: when their softmax phases coincide each takes twice as long and the MMAs of both tiles end
    // up back to back as well, and nothing pulls such a lock-step apart again.  Taking turns makes the
    // half-period offset between the tiles (one tile's softmax under the other tile's MMAs) the stable
    // state.  Only when both tiles walk the same KV steps (head-pair mode).
    const bool take_turns = !(DBG & 32) && p.pair_heads != 0;
    auto turn_wait = [&](const uint32_t step) {
      if (!take_turns) return;
      if (t == 0) { if (step > 0) wait_or_abort(bar(B_TURN + 0), (step - 1u) & 1u, abort_flag); }
      else wait_or_abort(bar(B_TURN + 1), step & 1u, abort_flag);
    };
    auto turn_pass = [&]() {
      if (!take_turns) return;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_TURN + (t ^ 1)));
    };
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
    uint32_t sph = 0;        // completed phases of B_SFULL[t] that this thread has consumed
    uint32_t pph = 0;        // KV steps of this tile so far: tags of the redo vote, slots of the exchange
    uint32_t kv_it = 0;      // KV tiles of all items so far: ring stage of K / V
    // What a completed MMA batch implies is passed on to the copy lane by this role, as soon as the batch
    // barrier is seen (the copies that refill the stages have a latency of more than half a KV step, so an
    // early release matters): the barrier seen at the start of step j says that QK(j) and PV(j-1) are done,
    // so K stage j and V stage j-1 (and, after the last QK, the Q buffer) are free.  The three arrivals are
    // made by lane 0 of three different warps, one instruction each.  (A thread that takes part in every
    // step can never fall behind the barrier's phases; a separate forwarding thread could, by two phases,
    // and a parity wait cannot tell that apart from "not yet".)
    const int fwd = (h == 0 && lane == 0) ? wq : -1;   // 0: K stage, 1: V stage, 2: Q buffer
    auto forward_step = [&](const uint32_t kv0, const int j, const int n_mine) {
      if (fwd == 0) mbar_arrive(bar(B_KEMPTY + (int)((kv0 + (uint32_t)j) % KV_STAGES)));
      if (fwd == 1 && j > 0) mbar_arrive(bar(B_VEMPTY + (int)((kv0 + (uint32_t)j - 1u) % KV_STAGES)));
      if (fwd == 2 && j == n_mine - 1) mbar_arrive(bar(B_QEMPTY + t));
    };
    for (uint32_t ic = 0;; ++ic) {
      if (*abort_flag) break;
      const int slot = ic % kItemQ;
      PROF_WAIT(3 + t, 0, wait_or_abort(bar(B_IFULL + slot), (ic / kItemQ) & 1u, abort_flag));
      const long long item = item_slot[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_IEMPTY + slot));
      if (item < 0 || item >= n_items) break;
      Tc5Item it;
      tc5_decode_item(p, item, it);
      const int n_mine = it.n_kv[t];
      const uint32_t kv0 = kv_it;
      kv_it += (uint32_t)it.n_max;
      if (n_mine == 0) continue;
      const int len = it.len;
      const int grow = it.row0[t] + row;       // row within the sequence
      float m = 0.f, l = 0.f;
      for (int j = 0; j < n_mine; ++j, ++pph) {
        PROF_COUNT(3 + t, 14);
        PROF_WAIT(3 + t, 1, wait_sel<(DBG & 128) != 0>(bar(B_SFULL + t), sph & 1u, abort_flag));
        ++sph;
        if (j > 0) PROF_SINCE(3 + t, 8, t);   // commit issued by the MMA lane -> batch seen complete here
        PROF_MARK(prof_t_s);
        tc_fence_after();
        forward_step(kv0, j, n_mine);
        const int k0 = j * BN;
        const bool need_mask = (k0 + BN > len) || (p.causal && (k0 + BN - 1 > it.row0[t]));
        // ---- my half of the score row: chunk c_lo (kept in registers) and chunk c_hi (read for its maximum,
        // read again when its turn comes).  Where P is written: thread 0 of the pair writes quarter 0 over
        // columns 16-31 (its own chunk 0, in registers) and later quarter 3 over columns 64-79 (its own chunk 2,
        // after its second read); thread 1 writes quarter 1 over columns 32-47 and later quarter 2 over
        // columns 48-63 (both its own chunk 1, in registers).  Chunk 3 is never overwritten.
        float sv[32], sw[32];
        float2 rs_lo = make_float2(0.f, 0.f), rs_hi = make_float2(0.f, 0.f);
        if (DBG & 16) {
          tc_ld32(tS + c_lo * 32, sv);
          tc_ld32(tS + c_hi * 32, sw);
          tc_wait_ld();
          turn_wait(pph);
          turn_pass();
          PROF_STAMP(2 + t);
          hand_over();
          continue;
        }
        bool full_path = SM == 0 || need_mask || j == 0;
        bool lo_loaded = false;
        if (SM == 1 && !full_path) {
          PROF_MARK(pf0);
          tc_ld32(tS + c_hi * 32, sw);
          tc_wait_ld();
          PROF_MARK(pf1);
          float a0 = fmaxf(sw[0], sw[1]), a1 = fmaxf(sw[2], sw[3]);
#pragma unroll
          for (int i = 4; i < 32; i += 4) {
            a0 = fmax3(a0, sw[i], sw[i + 1]);
            a1 = fmax3(a1, sw[i + 2], sw[i + 3]);
          }
          tc_ld32(tS + c_lo * 32, sv);      // (one chunk in registers at a time: 104 registers per thread)
          tc_wait_ld();
          PROF_MARK(pf2);
          lo_loaded = true;
          turn_wait(pph);
          const float2 nm2 = make_float2(-m, -m);
          exp_chunk_store<NPOLY, DBG, BF>(sv, sc2, nm2, rs_lo, tP + q_lo * 16);
          const bool inside = (rs_lo.x + rs_lo.y <= 32768.f) && (fmaxf(a0, a1) * p.scale_log2 <= m + 15.f);   // false for NaN
          const uint32_t tag = pph + 1u;
          if (__any_sync(0xffffffffu, !inside) && lane == 0) *my_tag = tag;
          PROF_MARK(pf3);
          tc_ld32(tS + c_hi * 32, sw);        // chunk c_hi again: in flight across the pair barrier
          pair_sync();
          PROF_MARK(pf4);
          if (*my_tag == tag) {
            // nothing has been handed over yet: the step is redone below (chunk c_lo is still in registers)
            tc_wait_ld();
            full_path = true;
            rs_lo = make_float2(0.f, 0.f);
          } else {
            tc_wait_ld();
            PROF_MARK(pf6);
            exp_chunk_store<NPOLY, DBG, BF>(sw, sc2, nm2, rs_hi, tP + q_hi * 16);
            turn_pass();
            PROF_MARK(pf7);
            PROF_STAMP(2 + t);
            hand_over();
            PROF_MARK(pf8);
            PROF_SPAN(3 + t, 9, pf0, pf1);    // first tensor-memory read
            PROF_SPAN(3 + t, 10, pf1, pf2);   // maximum + second read
            PROF_SPAN(3 + t, 11, pf2, pf3);   // first exponentials + vote
            PROF_SPAN(3 + t, 12, pf3, pf4);   // pair barrier
            PROF_SPAN(3 + t, 2, pf4, pf6);    // third read
            PROF_SPAN(3 + t, 7, pf6, pf7);    // second exponentials
            PROF_SPAN(3 + t, 6, pf7, pf8);    // wait for the P stores, hand over
            l += (rs_lo.x + rs_lo.y) + (rs_hi.x + rs_hi.y);
          }
        }
        if (full_path) {
          // keys of this tile that the row may attend: [k0, k0 + lim); chunks past the warp's largest
          // lim are stored as zeros without any exponentials (upper part of a causal diagonal tile)
          int lim = BN;
          if (need_mask) {
            lim = len - k0;
            if (p.causal && grow - k0 + 1 < lim) lim = grow - k0 + 1;
            if (lim > BN) lim = BN;
          }
          const int lim_max = need_mask ? __reduce_max_sync(0xffffffffu, lim) : BN;
          const int lim_min = need_mask ? __reduce_min_sync(0xffffffffu, lim) : BN;
          auto mask_chunk = [&](float (&v)[32], const int c) {
            if (c * 32 + 32 > lim_min) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (c * 32 + i >= lim) v[i] = -INFINITY;
            }
          };
          auto max_chunk = [&](const float (&v)[32]) {
            float a0 = fmaxf(v[0], v[1]), a1 = fmaxf(v[2], v[3]);
#pragma unroll
            for (int i = 4; i < 32; i += 4) {
              a0 = fmax3(a0, v[i], v[i + 1]);
              a1 = fmax3(a1, v[i + 2], v[i + 3]);
            }
            return fmaxf(a0, a1);
          };
          tc_ld32(tS + c_hi * 32, sw);
          tc_wait_ld();
          mask_chunk(sw, c_hi);
          const float mx_hi = max_chunk(sw);
          if (!lo_loaded) {
            tc_ld32(tS + c_lo * 32, sv);
            tc_wait_ld();
          }
          mask_chunk(sv, c_lo);
          const float mxl = fmaxf(mx_hi, max_chunk(sv));
          // the other half of the row lives in the partner warp
          float* slot_f = xch + (int)(pph & 1u) * (2 * 128);
          slot_f[h * 128 + row] = mxl;
          pair_sync();
          const float mxs = fmaxf(mxl, slot_f[(h ^ 1) * 128 + row]) * p.scale_log2;
          const float m_new = (j == 0) ? mxs : fmaxf(m, mxs);
          const bool grow_big = (j == 0) || (m_new > m + 8.f);
          const float alpha = (j > 0 && grow_big) ? fast_exp2(m - m_new) : 1.f;
          if (j > 0 && __any_sync(0xffffffffu, grow_big)) {
            // O_t holds the result of PV(t, j-1): the batch barrier waited for above covers it.  My half.
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              float o[16];
              tc_ld16(tO + c * 16, o);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] *= alpha;
              tc_st16(tO + c * 16, reinterpret_cast<const uint32_t(&)[16]>(o));
            }
          }
          if (grow_big) m = m_new;
          l *= alpha;
          // ---- P = exp2(S * scale - m), fp16 ----
          const float neg_m = (m == -INFINITY) ? 0.f : -m;
          const float2 nm2 = make_float2(neg_m, neg_m);
          if (!lo_loaded) turn_wait(pph);     // (a redone step has taken its turn already)
          if (c_lo * 32 < lim_max) exp_chunk_store<NPOLY, DBG, BF>(sv, sc2, nm2, rs_lo, tP + q_lo * 16);
          else zero_chunk_store(tP + q_lo * 16);
          tc_ld32(tS + c_hi * 32, sw);        // chunk c_hi again (its columns are written by nobody but me)
          tc_wait_ld();
          mask_chunk(sw, c_hi);
          if (c_hi * 32 < lim_max) exp_chunk_store<NPOLY, DBG, BF>(sw, sc2, nm2, rs_hi, tP + q_hi * 16);
          else zero_chunk_store(tP + q_hi * 16);
          turn_pass();
          PROF_STAMP(2 + t);
          hand_over();                        // waits for the O rescale stores as well
          l += (rs_lo.x + rs_lo.y) + (rs_hi.x + rs_hi.y);
        }
        PROF_MARK(prof_t_e);
        PROF_SPAN(3 + t, 4, prof_t_s, prof_t_e);
      }
      // ---- epilogue: O / l -> fp16 -> global, my half of the columns.  The batch barrier of the last step
      // covers PV(n-1).  The next item's first PV of this tile cannot be issued before these threads have
      // produced its P, i.e. after these loads have completed.
      PROF_WAIT(3 + t, 3, wait_or_abort(bar(B_SFULL + t), sph & 1u, abort_flag));
      ++sph;
      PROF_MARK(prof_t_o);
      tc_fence_after();
      if (fwd == 1) mbar_arrive(bar(B_VEMPTY + (int)((kv0 + (uint32_t)n_mine - 1u) % KV_STAGES)));
      float* slot_l = xch + 2 * (2 * 128);     // a slot of its own: the steps' slots may be rewritten at once
      slot_l[h * 128 + row] = l;
      pair_sync();
      PROF_MARK(pe1);
      const float l_row = l + slot_l[(h ^ 1) * 128 + row];
      const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
      // My half of the row, scaled and packed: NU units of 16 bytes (8 columns each).
      constexpr int NU = D / 16;
      uint32_t u[NU][4];
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        float o[16];
        tc_ld16(tO + c * 16, o);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 8; ++i) u[2 * c + (i >> 2)][i & 3] = pack_out16x2(o[2 * i] * inv, o[2 * i + 1] * inv, p.out_bf16 != 0);
      }
      // A thread-per-row store would touch 32 different 128-byte lines per instruction (the rows of a warp lie
      // a whole row apart in memory), and the load/store unit handles one line per cycle.  Transpose the
      // units within groups of NU lanes instead (lane i of a group ends up with unit i of every row of the
      // group), so that NU consecutive lanes write NU * 16 contiguous bytes of one row.
      PROF_MARK(pe2);
      const int gi = lane & (NU - 1);
#pragma unroll
      for (int sft = NU / 2; sft >= 1; sft >>= 1) {
#pragma unroll
        for (int k = 0; k < NU; ++k) {
          if (k & sft) continue;
          const bool up = (gi & sft) != 0;
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const uint32_t send = up ? u[k][w] : u[k | sft][w];
            const uint32_t got = __shfl_xor_sync(0xffffffffu, send, sft);
            if (up) u[k][w] = got; else u[k | sft][w] = got;
          }
        }
      }
      // u[k] now holds unit gi of the row (lane - gi + k) of this warp's quadrant
      PROF_MARK(pe3);
      const int row_g = wq * 32 + (lane - gi);            // first row of my lane group within the tile
      const int col = h * (D / 2) + gi * 8;               // first column of the unit I store
      __half* obase;
      if (p.dense) obase = p.out + (long long)it.seq * p.o_batch_stride + (long long)it.head[t] * p.o_head_stride;
      else obase = p.out + it.tok0 * p.o_tok_stride + (long long)it.head[t] * p.o_head_stride;
#pragma unroll
      for (int k = 0; k < NU; ++k) {
        const int r = it.row0[t] + row_g + k;             // row within the sequence
        if (r < len && col < p.D_real)
          *reinterpret_cast<uint4*>(obase + (long long)r * p.o_tok_stride + col) = make_uint4(u[k][0], u[k][1], u[k][2], u[k][3]);
      }
      tc_fence_before();
      // the partner must have read my row sum before the next epilogue overwrites the slot: it did so right
      // behind the barrier above, and the next epilogue lies at least one KV step (with barriers that both
      // warps take part in) ahead
      PROF_MARK(prof_t_x);
      PROF_SPAN(3 + t, 5, prof_t_o, prof_t_x);
      if (t == 0) {   // epilogue pieces, kept in unused slots of the copy lane's row of counters
        PROF_SPAN(0, 5, prof_t_o, pe1);     // pair barrier
        PROF_SPAN(0, 6, pe1, pe2);          // tensor-memory reads, scaling, packing
        PROF_SPAN(0, 7, pe2, pe3);          // transpose
        PROF_SPAN(0, 8, pe3, prof_t_x);     // stores
      }
    }
  }

  // ---- tear-down ------------------------------------------------------------------
#ifdef FA_TC5_PROF
  if (prof_on) {
    const int role = warp == 0 ? 0 : warp == 1 ? 1 : warp == 3 ? 2 : 3 + ((warp - 4) >> 3);
    prof_smem[role * 16 + 15] += (unsigned long long)(clock64() - prof_start);
  }
#endif
  tc_fence_before();
  __syncthreads();
#ifdef FA_TC5_PROF
  if (threadIdx.x < 5 * 16) atomicAdd(&g_tc5_prof[threadIdx.x], prof_smem[threadIdx.x]);
#endif
  if (warp == 2) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 3-D map {D, heads, rows} with a {64, 1, 128} box and 128-byte swizzle.
bool make_map3(EncodeTiledFn enc, CUtensorMap* map, const void* base, int D, long long heads, long long rows,
               long long head_stride_elems, long long row_stride_elems) {
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)heads, (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)head_stride_elems * 2, (cuuint64_t)row_stride_elems * 2};
  cuuint32_t box[3] = {64, 1, 128};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Item counters of in-flight launches (one per launch, used round-robin, zeroed in-stream before
// the kernel).  More than kCounterPool prefill launches in flight at once on one device would share
// a counter; launches ordered on one stream never do.
constexpr int kCounterPool = 64;
__device__ unsigned long long g_tc5_item_counters[kCounterPool];
unsigned long long* g_counter_base[64] = {nullptr};
std::atomic<unsigned int> g_counter_next{0};
std::mutex g_counter_mu;

cudaError_t next_item_counter(unsigned long long** out, cudaStream_t stream) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  {
    std::lock_guard<std::mutex> lk(g_counter_mu);
    if (g_counter_base[dev] == nullptr) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_tc5_item_counters);
      if (e != cudaSuccess) return e;
      g_counter_base[dev] = static_cast<unsigned long long*>(ptr);
    }
  }
  unsigned long long* c = g_counter_base[dev] + (g_counter_next.fetch_add(1) % kCounterPool);
  e = cudaMemsetAsync(c, 0, sizeof(unsigned long long), stream);
  *out = c;
  return e;
}

bool g_tc5_poly = false;  // true: a quarter of the exponentials evaluated as a polynomial on the FMA pipes

using Tc5Kernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const Tc5Params);

#ifdef FA_TC5_SWEEP
// Tuning build only (-DFA_TC5_SWEEP): every variant below is compiled and one is picked at run time.
int g_tc5_variant = 0;
template <int D>
Tc5Kernel sweep_kernel(int v) {
  switch (v) {
    case 1: return prefill_tc5_kernel<D, 0, 1>;
    case 2: return prefill_tc5_kernel<D, 0, 1, 1>;         // no exp2
    case 4: return prefill_tc5_kernel<D, 0, 1, 16>;        // no softmax at all
    case 5: return prefill_tc5_kernel<D, 0, 1, 16 | 2>;    // no softmax, QK only
    case 6: return prefill_tc5_kernel<D, 0, 1, 16 | 4>;    // no softmax, PV only
    case 8: return prefill_tc5_kernel<D, 2, 1>;
    case 9: return prefill_tc5_kernel<D, 4, 1>;
    case 10: return prefill_tc5_kernel<D, 3, 1>;
    case 12: return prefill_tc5_kernel<D, 0, 1, 32>;       // no turn taking between the tiles
    case 13: return prefill_tc5_kernel<D, 2, 1, 32>;
    case 11: return prefill_tc5_kernel<D, 1, 1>;
    case 14: return prefill_tc5_kernel<D, 0, 1, 64>;       // the MMA lanes poll without suspending
    case 15: return prefill_tc5_kernel<D, 0, 1, 128>;      // the softmax threads poll the score barrier without suspending
    case 16: return prefill_tc5_kernel<D, 0, 1, 192>;
    default: return prefill_tc5_kernel<D, 0, 0>;
  }
}
#endif

template <int D>
Tc5Kernel pick_kernel() {
#ifdef FA_TC5_SWEEP
  return sweep_kernel<D>(g_tc5_variant);
#else
  return g_tc5_poly ? prefill_tc5_kernel<D, 2, 1> : prefill_tc5_kernel<D, 0, 1>;
#endif
}
template <int D>
Tc5Kernel pick_kernel_bf16() {
  return g_tc5_poly ? prefill_tc5_kernel<D, 2, 1, 0, true> : prefill_tc5_kernel<D, 0, 1, 0, true>;
}

template <int D>
cudaError_t launch_tc5_t(const PrefillParams& pp, void* encode_fn, cudaStream_t stream) {
  EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(encode_fn);
  const bool dense = pp.cu_seqlens == nullptr;
  CUtensorMap qmap, kmap, vmap;
  bool ok;
  if (dense) {
    const long long qrows = (long long)pp.batch * pp.H_Q * pp.N, krows = (long long)pp.batch * pp.H_KV * pp.N;
    const int Dr = pp.D_real;   // extent of the innermost dimension: the boxes' columns past it are zero-filled
    ok = make_map3(enc, &qmap, pp.q, Dr, 1, qrows, Dr, Dr) && make_map3(enc, &kmap, pp.k, Dr, 1, krows, Dr, Dr) &&
         make_map3(enc, &vmap, pp.v, Dr, 1, krows, Dr, Dr);
  } else {
    const int Dr = pp.D_real;
    ok = make_map3(enc, &qmap, pp.q, Dr, pp.H_Q, pp.total, Dr, (long long)pp.H_Q * Dr) &&
         make_map3(enc, &kmap, pp.k, Dr, pp.H_KV, pp.total, Dr, (long long)pp.H_KV * Dr) &&
         make_map3(enc, &vmap, pp.v, Dr, pp.H_KV, pp.total, Dr, (long long)pp.H_KV * Dr);
  }
  if (!ok) return cudaErrorInvalidValue;
  Tc5Params p;
  p.out = pp.out;
  p.cu_seqlens = pp.cu_seqlens;
  p.batch = pp.batch; p.H_Q = pp.H_Q; p.H_KV = pp.H_KV; p.N = pp.N; p.max_seqlen = pp.max_seqlen;
  p.total = pp.total;
  p.o_batch_stride = pp.q_batch_stride; p.o_head_stride = pp.q_head_stride; p.o_tok_stride = pp.q_tok_stride;
  p.causal = pp.causal;
  p.D_real = pp.D_real;
  p.pair_heads = ((pp.H_Q / pp.H_KV) % 2 == 0) ? 1 : 0;
  p.dense = dense ? 1 : 0;
  p.out_bf16 = (pp.out_bf16 || pp.in_bf16) ? 1 : 0;
  p.scale_log2 = pp.scale_log2;
  constexpr int KV_STAGES = (D == 128) ? 2 : 4;
  constexpr size_t TILE = (size_t)(D / 64) * 128 * 128;
  // tiles + barriers, item queue, flags + the softmax role's exchange area
  size_t smem = 1024 + (2 + 2 * KV_STAGES) * TILE + 64 * 8 + 2 * 3 * 2 * 128 * 4 + 8 * 4;
#ifdef FA_TC5_PROF
  smem += (5 * 16 + 8) * 8;
#endif
  Tc5Kernel kern = pp.in_bf16 ? pick_kernel_bf16<D>() : pick_kernel<D>();
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int max_len = dense ? pp.N : pp.max_seqlen;
  dim3 grid;
  if (p.pair_heads) { p.n_hg = pp.H_Q / 2; p.n_rb = (max_len + 127) / 128; }
  else { p.n_hg = pp.H_Q; p.n_rb = (max_len + 255) / 256; }
  const long long n_items = (long long)p.n_rb * pp.batch * p.n_hg;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  grid = dim3((unsigned)(n_items < sms ? n_items : sms));
  e = next_item_counter(&p.item_counter, stream);
  if (e != cudaSuccess) return e;
  kern<<<grid, 640, smem, stream>>>(qmap, kmap, vmap, p);
  return cudaGetLastError();
}

}  // namespace

bool prefill_tc5_supported(const PrefillParams& p, int D) {
  if (D != 64 && D != 128) return false;
  const long long qrows = p.cu_seqlens ? p.total : (long long)p.batch * p.H_Q * p.N;
  if (qrows >= (1ll << 31)) return false;
  return true;
}

cudaError_t launch_prefill_tc5(const PrefillParams& p, int D, void* encode_fn, cudaStream_t stream) {
  if (D == 128) return launch_tc5_t<128>(p, encode_fn, stream);
  if (D == 64) return launch_tc5_t<64>(p, encode_fn, stream);
  return cudaErrorInvalidValue;
}

#ifdef FA_TC5_PROF
// Instrumented build only: copy the wait counters to the host (and optionally clear them).
extern "C" int fa_debug_read_tc5_prof(unsigned long long* host, int clear) {
  cudaError_t e = cudaMemcpyFromSymbol(host, g_tc5_prof, sizeof(unsigned long long) * 5 * 16);
  if (e == cudaSuccess && clear) {
    static const unsigned long long zeros[5 * 16] = {0};
    e = cudaMemcpyToSymbol(g_tc5_prof, zeros, sizeof(zeros));
  }
  return (int)e;
}
#endif
#ifdef FA_TC5_SWEEP
extern "C" int fa_debug_tc5_set_variant(int v) {
  g_tc5_variant = v;
  return 0;
}
#endif

void prefill_tc5_set_poly(bool on) { g_tc5_poly = on; }

cudaError_t prefill_status_ptr(int** out) {
  void* ptr = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&ptr, g_prefill_status);
  *out = static_cast<int*>(ptr);
  return e;
}

cudaError_t prefill_status(int* host_out, cudaStream_t stream) {
  cudaError_t e = cudaMemcpyFromSymbolAsync(host_out, g_prefill_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return e;
  return cudaStreamSynchronize(stream);
}

cudaError_t prefill_status_clear(cudaStream_t stream) {
  int zero = 0;
  return cudaMemcpyToSymbolAsync(g_prefill_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
}

}  // namespace fa
