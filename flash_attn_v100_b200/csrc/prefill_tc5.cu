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
// runs the other tile's MMAs.  P is written back to tensor memory as fp16 over the second
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

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
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
__device__ __forceinline__ void tc_st32(uint32_t taddr, const float (&v)[32]) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
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
  r.x = __int_as_float(__float_as_int(r.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(r.y) + (__float_as_int(t.y) << 23));
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
template <int NPOLY, int DBG = 0>
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
    pk[i] = (DBG & 8) ? __float_as_uint(e.x) : pack_half2(e.x, e.y);   // DBG 8: no conversion
  }
  tc_st16(taddr, pk);
}

__device__ __forceinline__ void zero_chunk_store(uint32_t taddr) {
  uint32_t pk[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) pk[i] = 0u;
  tc_st16(taddr, pk);
}

// Maximum of a 128-value score row held in registers (two chains per chunk of three-input maxima).
__device__ __forceinline__ float row_max128(const float (&sv)[4][32]) {
  float mxc[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    float a0 = fmaxf(sv[c][0], sv[c][1]), a1 = fmaxf(sv[c][2], sv[c][3]);
#pragma unroll
    for (int i = 4; i < 32; i += 4) {
      a0 = fmax3(a0, sv[c][i], sv[c][i + 1]);
      a1 = fmax3(a1, sv[c][i + 2], sv[c][i + 3]);
    }
    mxc[c] = fmaxf(a0, a1);
  }
  return fmaxf(fmaxf(mxc[0], mxc[1]), fmaxf(mxc[2], mxc[3]));
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
// PSPLIT: 32-column chunks of P handed to the PV MMA with the first barrier (1..3);
// SM: 0 every tile takes the full softmax path (row maximum and rescale decision first); 1 tiles that need no
// masking take the fast path described in the softmax role.
// DBG (tuning builds only, results are wrong): 1 no exp2, 2 no PV MMAs, 4 no QK MMAs, 8 no fp16 conversion,
// 16 the softmax hands over at once without computing anything.
template <int D, int NPOLY, int PSPLIT, int SM, int DBG = 0>
__global__ void __launch_bounds__(384, 1)
prefill_tc5_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                   const __grid_constant__ CUtensorMap vmap, const Tc5Params p) {
  constexpr int BM = 128, BN = 128;
  constexpr int KV_STAGES = (D == 128) ? 2 : 4;
  constexpr int SLAB = 128 * 128;            // bytes of a [128 rows][64 cols] fp16 slab
  constexpr int NSLAB = D / 64;
  constexpr int TILE_BYTES = NSLAB * SLAB;   // one Q / K / V tile
  constexpr uint32_t IDESC_QK = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t O_COL0 = 256;
  constexpr uint32_t P_COL = 64;             // P (fp16, 64 columns) lies over the SECOND half of its S: writing the
                                             // first part of P leaves the first half of S intact in tensor memory
  constexpr int kPSplit = PSPLIT;            // P is handed to the PV MMA in two parts: 32*kPSplit keys, then the rest
  constexpr int kItemQ = 4;                  // depth of the per-CTA item queue
  constexpr int kItemConsumers = 2 + 256;    // two MMA lanes + every softmax thread

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
                B_PLO = B_SFULL + 2, B_PHI = B_PLO + 2, B_TOKEN = B_PHI + 2,
                B_IFULL = B_TOKEN + 2, B_IEMPTY = B_IFULL + kItemQ, B_COUNT = B_IEMPTY + kItemQ;
  volatile long long* item_slot = reinterpret_cast<volatile long long*>(bars + B_COUNT);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT + kItemQ);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) -> uint32_t { return smem_u32(bars + i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long n_items = (long long)p.n_rb * p.batch * p.n_hg;
#ifdef FA_TC5_PROF
  unsigned long long* prof_smem = reinterpret_cast<unsigned long long*>(bars + 64);
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
      mbar_init(bar(B_PLO + t), 128);
      mbar_init(bar(B_PHI + t), 128);
      mbar_init(bar(B_TOKEN + t), 1);
    }
    for (int i = 0; i < kItemQ; ++i) {
      mbar_init(bar(B_IFULL + i), 1);
      mbar_init(bar(B_IEMPTY + i), kItemConsumers);
    }
    *abort_flag = 0;
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
        // claim the next non-empty item and publish it (-1: no more items)
        Tc5Item it;
        long long item;
        bool have = false;
        PROF_WAIT(0, 0, while (true) {
          item = (long long)atomicAdd(p.item_counter, 1ULL);
          if (item >= n_items) break;
          if (tc5_decode_item(p, item, it)) { have = true; break; }
        });
        const int slot = ic % kItemQ;
        if (ic >= kItemQ) PROF_WAIT(0, 1, wait_or_abort(bar(B_IEMPTY + slot), ((ic / kItemQ) & 1u) ^ 1u, abort_flag));
        item_slot[slot] = have ? item : -1;
        mbar_arrive(bar(B_IFULL + slot));
        if (!have) break;
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
    if (lane == 0) {
#ifdef FA_TC5_PROF
      prof_on = true;
#endif
      constexpr uint32_t TILE16 = TILE_BYTES >> 4;
      const uint64_t qd = smem_desc(sQ + (uint32_t)t * TILE_BYTES, 16, 1024);
      const uint64_t kd0 = smem_desc(sK, 16, 1024);
      const uint64_t vd0 = smem_desc(sV, SLAB, 1024);
      const uint32_t dS = tmem_base + (uint32_t)t * 128u;
      const uint32_t dO = tmem_base + O_COL0 + (uint32_t)t * D;
      auto issue_qk = [&](int st) {
        const uint64_t b0 = kd0 + (uint64_t)((uint32_t)st * TILE16);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          constexpr uint32_t kSlab16 = SLAB >> 4;
          const uint32_t off = (uint32_t)(ks >> 2) * kSlab16 + (uint32_t)(ks & 3) * 2u;
          tc_mma_ss(dS, qd + off, b0 + off, IDESC_QK, ks > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int st, uint32_t acc, int half) {
        const uint64_t b0 = vd0 + (uint64_t)((uint32_t)st * TILE16);
        // first part: the keys whose P arrives with the first barrier (kPSplit chunks of 32 keys)
#pragma unroll
        for (int ks = half ? 2 * kPSplit : 0; ks < (half ? BN / 16 : 2 * kPSplit); ++ks) {
          tc_mma_ts(dO, dS + P_COL + (uint32_t)ks * 8u, b0 + (uint32_t)ks * 128u, IDESC_PV, (acc | (ks > 0 ? 1u : 0u)));
        }
      };
      uint32_t kv_it = 0, q_cnt = 0, blk = 0, tok_waits = 0;
      for (uint32_t ic = 0;; ++ic) {
        if (*abort_flag) break;
        const int slot = ic % kItemQ;
        PROF_WAIT(1 + t, 0, wait_or_abort(bar(B_IFULL + slot), (ic / kItemQ) & 1u, abort_flag));
        const long long item = item_slot[slot];
        mbar_arrive(bar(B_IEMPTY + slot));
        if (item < 0 || item >= n_items) break;
        Tc5Item it;
        tc5_decode_item(p, item, it);
        const bool other_active = it.n_kv[1] > 0;   // tile 0 is always active in a non-empty item
        const int n_mine = it.n_kv[t];
        auto take_token = [&]() {
          if (!other_active) return;
          PROF_WAIT(1 + t, 6, wait_or_abort(bar(B_TOKEN + t), tok_waits & 1u, abort_flag));
          ++tok_waits;
        };
        auto pass_token = [&]() {
          if (other_active) mbar_arrive(bar(B_TOKEN + (t ^ 1)));
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
            PROF_WAIT(1 + t, 3, wait_or_abort(bar(B_VFULL + st), ph, abort_flag));
            if (more) PROF_WAIT(1 + t, 4, wait_or_abort(bar(B_KFULL + st1), ph1, abort_flag));
            PROF_WAIT(1 + t, 5, wait_or_abort(bar(B_PLO + t), blk & 1u, abort_flag));
            PROF_SINCE(1 + t, 9, 2 + t);      // P_lo arrival (row 0) -> seen by the MMA lane
            // tile 1's block j+1 follows tile 0's block j+1; tile 0's block j+1 follows tile 1's
            // block j, which exists unless tile 1 has already run out of KV tiles
            if (t == 1 || j <= it.n_kv[1]) take_token();
            tc_fence_after();
            if (!(DBG & 2)) issue_pv(st, j > 0 ? 1u : 0u, 0);
            PROF_WAIT(1 + t, 7, wait_or_abort(bar(B_PHI + t), blk & 1u, abort_flag));
            PROF_SINCE(1 + t, 10, 4 + t);     // P_hi arrival (row 0) -> seen by the MMA lane
            PROF_MARK(prof_t_i);
            tc_fence_after();
            if (!(DBG & 2)) issue_pv(st, 1u, 1);
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
          mbar_arrive(bar(B_KEMPTY + st));
          PROF_WAIT(1 + t, 8, wait_or_abort(bar(B_VFULL + st), ph, abort_flag));
          mbar_arrive(bar(B_VEMPTY + st));
        }
        kv_it += (uint32_t)it.n_max;
      }
    }
  } else if (warp == 2) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // ============================ softmax groups ====================================
    // Thread = one query row.  State per row: a reference exponent m (any finite number works as long as
    // P = exp2(s * scale - m) stays inside the fp16 range), the row sum l relative to m, and O in tensor
    // memory, also relative to m.
    //   full path (first KV tile of an item, tiles that need masking, rows that left the window below):
    //     row maximum first, m raised when the maximum grows by more than 2^8 with O rescaled in tensor
    //     memory, then the exponentials.
    //   fast path (SM 1, other tiles): no dependent chain in front of the exponentials.  The first part of P
    //     is exponentiated against the m carried over from the previous step while the raw maximum of the
    //     second part is formed in the same instruction stream; the step goes ahead if the first part's sum
    //     shows that nothing exceeded 2^15 and the second part's maximum stays below m + 15 (so P fits fp16);
    //     otherwise nothing has been handed over yet and the step is redone on the full path.
    // The group also forwards what a completed MMA batch implies: the batch barrier B_SFULL of step j says
    // that PV(j-1) and QK(j) are done, so V stage j-1 and K stage j (and, after the last QK, the Q buffer) are
    // free; the thread of row 0 arrives on the copy lane's barriers for them.
    const int t = (warp - 4) >> 2;
    const int wq = warp & 3;                   // TMEM lane quadrant of this warp
    const int row = wq * 32 + lane;            // row within the tile == TMEM lane
    const uint32_t lane_base = tmem_base + ((uint32_t)(wq * 32) << 16);
    const uint32_t tS = lane_base + (uint32_t)t * 128u;
    const uint32_t tP = tS + P_COL;
    const uint32_t tO = lane_base + O_COL0 + (uint32_t)t * D;
#ifdef FA_TC5_PROF
    prof_on = (row == 0);
#endif
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
    uint32_t sph = 0;        // completed phases of B_SFULL[t] that this thread has consumed
    uint32_t pph = 0;        // KV steps of this tile so far: phase of B_PLO / B_PHI
    uint32_t kv_it = 0;      // KV tiles of all items so far: ring stage of K / V
    for (uint32_t ic = 0;; ++ic) {
      if (*abort_flag) break;
      const int slot = ic % kItemQ;
      PROF_WAIT(3 + t, 0, wait_or_abort(bar(B_IFULL + slot), (ic / kItemQ) & 1u, abort_flag));
      const long long item = item_slot[slot];
      mbar_arrive(bar(B_IEMPTY + slot));
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
        PROF_WAIT(3 + t, 1, wait_or_abort(bar(B_SFULL + t), sph & 1u, abort_flag));
        ++sph;
        if (j > 0) PROF_SINCE(3 + t, 8, t);   // commit issued by the MMA lane -> batch seen complete here
        PROF_MARK(prof_t_s);
        tc_fence_after();
        if (row == 0) {
          // QK(j) is complete: K stage j is free; so is PV(j-1): V stage j-1
          mbar_arrive(bar(B_KEMPTY + (int)((kv0 + (uint32_t)j) % KV_STAGES)));
          if (j > 0) mbar_arrive(bar(B_VEMPTY + (int)((kv0 + (uint32_t)j - 1u) % KV_STAGES)));
          if (j == n_mine - 1) mbar_arrive(bar(B_QEMPTY + t));   // that was the last QK of this item
        }
        const int k0 = j * BN;
        const bool need_mask = (k0 + BN > len) || (p.causal && (k0 + BN - 1 > it.row0[t]));
        // ---- the whole score row of this thread: 128 fp32 values, one round trip ----
        float sv[4][32];
        tc_ld32(tS, sv[0]);
        tc_ld32(tS + 32, sv[1]);
        tc_ld32(tS + 64, sv[2]);
        tc_ld32(tS + 96, sv[3]);
        tc_wait_ld();
        float2 rs2[4];
        if (DBG & 16) {
          tc_fence_before();
          PROF_STAMP(2 + t);
          mbar_arrive(bar(B_PLO + t));
          PROF_STAMP(4 + t);
          mbar_arrive(bar(B_PHI + t));
          continue;
        }
        bool full_path = SM == 0 || need_mask || j == 0;
        if (SM == 1 && !full_path) {
          float mx2 = -INFINITY;
#pragma unroll
          for (int c = kPSplit; c < 4; ++c) {
            float a0 = fmaxf(sv[c][0], sv[c][1]), a1 = fmaxf(sv[c][2], sv[c][3]);
#pragma unroll
            for (int i = 4; i < 32; i += 4) {
              a0 = fmax3(a0, sv[c][i], sv[c][i + 1]);
              a1 = fmax3(a1, sv[c][i + 2], sv[c][i + 3]);
            }
            mx2 = fmax3(mx2, a0, a1);
          }
          const float2 nm2 = make_float2(-m, -m);
#pragma unroll
          for (int c = 0; c < kPSplit; ++c) {
            rs2[c] = make_float2(0.f, 0.f);
            exp_chunk_store<NPOLY, DBG>(sv[c], sc2, nm2, rs2[c], tP + c * 16);
          }
          float part = 0.f;
#pragma unroll
          for (int c = 0; c < kPSplit; ++c) part += rs2[c].x + rs2[c].y;
          const bool inside = (part <= 32768.f) && (mx2 * p.scale_log2 <= m + 15.f);   // false for NaN
          if (__any_sync(0xffffffffu, !inside)) {
            // nothing has been handed over yet: the step is redone below.  The first half of S is still
            // intact in tensor memory (P lies over the second half, which the registers hold)
            full_path = true;
            tc_ld32(tS, sv[0]);
            tc_ld32(tS + 32, sv[1]);
            tc_wait_ld();
          } else {
            tc_wait_st();
            tc_fence_before();
            PROF_STAMP(2 + t);
            mbar_arrive(bar(B_PLO + t));
#pragma unroll
            for (int c = kPSplit; c < 4; ++c) {
              rs2[c] = make_float2(0.f, 0.f);
              exp_chunk_store<NPOLY, DBG>(sv[c], sc2, nm2, rs2[c], tP + c * 16);
            }
            tc_wait_st();
            tc_fence_before();
            PROF_STAMP(4 + t);
            mbar_arrive(bar(B_PHI + t));
#pragma unroll
            for (int c = kPSplit; c < 4; ++c) part += rs2[c].x + rs2[c].y;
            l += part;
          }
        }
        if (full_path) {
          PROF_COUNT(3 + t, 6);
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
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c * 32 + 32 > lim_min) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (c * 32 + i >= lim) sv[c][i] = -INFINITY;
            }
          }
          const float mxs = row_max128(sv) * p.scale_log2;
          const float m_new = (j == 0) ? mxs : fmaxf(m, mxs);
          const bool grow_big = (j == 0) || (m_new > m + 8.f);
          const float alpha = (j > 0 && grow_big) ? fast_exp2(m - m_new) : 1.f;
          if (j > 0 && __any_sync(0xffffffffu, grow_big)) {
            // O_t holds the result of PV(t, j-1): the batch barrier waited for above covers it
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              float o[32];
              tc_ld32(tO + c * 32, o);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] *= alpha;
              tc_st32(tO + c * 32, o);
            }
            tc_wait_st();
          }
          if (grow_big) m = m_new;
          l *= alpha;
          // ---- P = exp2(S * scale - m), fp16, written over the last 64 columns of S ----
          const float neg_m = (m == -INFINITY) ? 0.f : -m;
          const float2 nm2 = make_float2(neg_m, neg_m);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            rs2[c] = make_float2(0.f, 0.f);
            if (c * 32 < lim_max) exp_chunk_store<NPOLY, DBG>(sv[c], sc2, nm2, rs2[c], tP + c * 16);
            else zero_chunk_store(tP + c * 16);
            if (c == kPSplit - 1 || c == 3) {
              // the first kPSplit chunks / the rest of P are in tensor memory: let the PV MMA start on them
              tc_wait_st();
              tc_fence_before();
              PROF_STAMP((c == 3 ? 4 : 2) + t);
              mbar_arrive(bar((c == 3 ? B_PHI : B_PLO) + t));
            }
          }
          l += (rs2[0].x + rs2[0].y) + (rs2[1].x + rs2[1].y) + (rs2[2].x + rs2[2].y) + (rs2[3].x + rs2[3].y);
        }
        PROF_MARK(prof_t_e);
        PROF_SPAN(3 + t, 4, prof_t_s, prof_t_e);
      }
      // ---- epilogue: O / l -> fp16 -> global.  The batch barrier of the last step covers PV(n-1).  The
      // next item's first PV of this tile cannot be issued before these threads have produced its P, i.e.
      // after these loads have completed.
      PROF_WAIT(3 + t, 3, wait_or_abort(bar(B_SFULL + t), sph & 1u, abort_flag));
      ++sph;
      PROF_MARK(prof_t_o);
      tc_fence_after();
      if (row == 0) mbar_arrive(bar(B_VEMPTY + (int)((kv0 + (uint32_t)n_mine - 1u) % KV_STAGES)));
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __half* orow;
      if (p.dense) orow = p.out + (long long)it.seq * p.o_batch_stride + (long long)it.head[t] * p.o_head_stride +
                          (long long)grow * p.o_tok_stride;
      else orow = p.out + (it.tok0 + grow) * p.o_tok_stride + (long long)it.head[t] * p.o_head_stride;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        tc_ld32(tO + c * 32, o);
        tc_wait_ld();
        if (grow < len) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_half2(o[8 * i + 0] * inv, o[8 * i + 1] * inv);
            w.y = pack_half2(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
            w.z = pack_half2(o[8 * i + 4] * inv, o[8 * i + 5] * inv);
            w.w = pack_half2(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
            if (c * 32 + i * 8 < p.D_real) *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = w;
          }
        }
      }
      tc_fence_before();
      PROF_MARK(prof_t_x);
      PROF_SPAN(3 + t, 5, prof_t_o, prof_t_x);
    }
  }

  // ---- tear-down ------------------------------------------------------------------
#ifdef FA_TC5_PROF
  if (prof_on) {
    const int role = warp == 0 ? 0 : warp == 1 ? 1 : warp == 3 ? 2 : 3 + ((warp - 4) >> 2);
    prof_smem[role * 16 + 15] += (unsigned long long)(clock64() - prof_start);
  }
#endif
  tc_fence_before();
  __syncthreads();
#ifdef FA_TC5_PROF
  if (threadIdx.x < 5 * 16) atomicAdd(&g_tc5_prof[threadIdx.x], prof_smem[threadIdx.x]);
#endif
  if (warp == 2) {
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
    case 1: return prefill_tc5_kernel<D, 0, 2, 1>;
    case 2: return prefill_tc5_kernel<D, 0, 2, 1, 1>;         // no exp2
    case 3: return prefill_tc5_kernel<D, 0, 1, 1>;
    case 4: return prefill_tc5_kernel<D, 0, 2, 1, 16>;        // no softmax at all
    case 5: return prefill_tc5_kernel<D, 0, 2, 1, 16 | 2>;    // no softmax, QK only
    case 6: return prefill_tc5_kernel<D, 0, 2, 1, 16 | 4>;    // no softmax, PV only
    case 7: return prefill_tc5_kernel<D, 0, 3, 1>;
    case 8: return prefill_tc5_kernel<D, 2, 2, 1>;
    case 9: return prefill_tc5_kernel<D, 4, 2, 1>;
    default: return prefill_tc5_kernel<D, 0, 2, 0>;
  }
}
#endif

template <int D>
Tc5Kernel pick_kernel() {
#ifdef FA_TC5_SWEEP
  return sweep_kernel<D>(g_tc5_variant);
#else
  return g_tc5_poly ? prefill_tc5_kernel<D, 2, 2, 1> : prefill_tc5_kernel<D, 0, 2, 1>;
#endif
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
  p.scale_log2 = pp.scale_log2;
  constexpr int KV_STAGES = (D == 128) ? 2 : 4;
  constexpr size_t TILE = (size_t)(D / 64) * 128 * 128;
  size_t smem = 1024 + (2 + 2 * KV_STAGES) * TILE + 64 * 8 + 16;  // tiles + barriers, item queue, flags
#ifdef FA_TC5_PROF
  smem += (5 * 16 + 8) * 8;
#endif
  Tc5Kernel kern = pick_kernel<D>();
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
  kern<<<grid, 384, smem, stream>>>(qmap, kmap, vmap, p);
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
