// C-ABI entry points (see include/fa_b200.h): argument validation, tensor-map
// construction, launch configuration.  No device memory is allocated here.
#include "../../include/fa_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <climits>
#include <mutex>

#include "decode_splitkv.cuh"
#include "prefill.cuh"
#include "rope_append.cuh"
#include "engine_ops.cuh"
#include "peer_collectives.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define FA_REQUIRE(cond, ...) \
  do {                        \
    if (!(cond)) return fail(FA_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

#define FA_CUDA(call)                                                                      \
  do {                                                                                     \
    cudaError_t e__ = (call);                                                              \
    if (e__ != cudaSuccess) return fail(FA_ERR_CUDA, #call " failed: %s", cudaGetErrorString(e__)); \
  } while (0)

bool supported_d(int D) { return D == 64 || D == 128 || D == 256; }   // head dimensions the prefill kernels serve
// Decode kernels are built for 64, 128 and 256 columns; any head dimension up to 256 that keeps rows
// 16-byte aligned runs on the next larger build (the missing columns read as zeros through the tensor maps).
int padded_decode_d(int D) {
  if (D < 8 || D > 256 || D % 8 != 0) return 0;
  return D <= 64 ? 64 : (D <= 128 ? 128 : 256);
}

// ---- per-device facts -------------------------------------------------------
struct DeviceInfo {
  int sm_count = 0;
  int max_smem_optin = 0;
  bool ok = false;
};
DeviceInfo g_dev[64];
std::mutex g_dev_mu;

int device_info(DeviceInfo* out) {
  int dev = 0;
  FA_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(FA_ERR_CUDA, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_dev_mu);
  if (!g_dev[dev].ok) {
    int major = 0;
    FA_CUDA(cudaDeviceGetAttribute(&g_dev[dev].sm_count, cudaDevAttrMultiProcessorCount, dev));
    FA_CUDA(cudaDeviceGetAttribute(&g_dev[dev].max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    FA_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10)
      return fail(FA_ERR_UNSUPPORTED, "this library is built for sm_100a only; device %d has compute capability %d.x",
                  dev, major);
    g_dev[dev].ok = true;
  }
  *out = g_dev[dev];
  return FA_OK;
}

// ---- tensor maps ------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int get_encode(EncodeTiledFn* fn) {
  static std::once_flag once;
  static cudaError_t err = cudaSuccess;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
    if (err == cudaSuccess && qres == cudaDriverEntryPointSuccess) g_encode = reinterpret_cast<EncodeTiledFn>(sym);
  });
  if (g_encode == nullptr) return fail(FA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  *fn = g_encode;
  return FA_OK;
}

// 2-D map over a [rows, D] fp16 tensor: box = 64 columns x box_rows rows, 128-byte swizzle.
int make_rows_map(CUtensorMap* map, const void* base, long long rows, int D, int box_rows) {
  EncodeTiledFn enc;
  int rc = get_encode(&enc);
  if (rc != FA_OK) return rc;
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return FA_OK;
}

// 2-D map over a [rows, D] int8 tensor: box = min(D, 128) columns x 16 rows; 128-byte swizzle when the
// box is 128 bytes wide, none for 64-byte rows.
int make_rows_map_u8(CUtensorMap* map, const void* base, long long rows, int D) {
  EncodeTiledFn enc;
  int rc = get_encode(&enc);
  if (rc != FA_OK) return rc;
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)D};
  cuuint32_t box[2] = {(cuuint32_t)(D <= 64 ? 64 : 128), 16};   // columns past D read as zeros
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, D <= 64 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return FA_OK;
}

// ---- decode tuning ----------------------------------------------------------
fa::DecodeLaunchConfig g_cfg_override = {0, 0, 0};

fa::DecodeLaunchConfig pick_decode_config(int D, int G, int slot_rows, int B, int kv_elem_bytes, bool int8_qk,
                                          const DeviceInfo& di) {
  fa::DecodeLaunchConfig c;
  const bool half_m = G <= 8;  // kernels for at most 8 query heads per KV head: 128 threads, more CTAs per SM
  if (kv_elem_bytes == 1) c = {4, 2, (half_m && D <= 128) ? 3 : (D == 256 ? 1 : 2)};  // dequantisation-bound
  else if (int8_qk && half_m && D == 128) c = {4, 2, 3};   // quantisation-bound: a third CTA hides its latency
  else if (D == 256) c = {4, 2, 1};
  else if (D == 128) c = {4, 2, 2};
  else c = {4, 4, 2};
  if (g_cfg_override.warps > 0) c.warps = g_cfg_override.warps;
  if (g_cfg_override.stages > 0) c.stages = g_cfg_override.stages;
  if (g_cfg_override.ctas_per_sm > 0) c.ctas_per_sm = g_cfg_override.ctas_per_sm;
  if (c.warps > (half_m ? 4 : 8)) c.warps = half_m ? 4 : 8;
  if (c.stages > 8) c.stages = 8;
  if (c.stages < 2) c.stages = 2;
  // shrink until ctas_per_sm CTAs fit in shared memory
  const size_t sm_total = (size_t)di.max_smem_optin + 1024;  // per-SM capacity = opt-in max + 1 KB reserve
  while (true) {
    const size_t need = fa::decode_smem_bytes(D, c.warps, c.stages, slot_rows, B, kv_elem_bytes);
    if (need <= (size_t)di.max_smem_optin && (need + 1024) * c.ctas_per_sm <= sm_total) break;
    if (c.ctas_per_sm > 1) --c.ctas_per_sm;
    else if (c.stages > 2) --c.stages;
    else if (c.warps > 1) --c.warps;
    else break;
  }
  return c;
}

using fa::kMaxDecodeCtas;

struct DecodeCall {
  const void *q, *k, *v;
  void* out;
  const int32_t* block_table;
  const int32_t* lens;
  const float *q_scale, *k_scale;
  int32_t* scores_out;
  int B, H_Q, H_KV, D, mode, fixed_len, N, bt_stride;
  long long num_pages, rows_total, max_units;
  bool int8;
  bool out_bf16;                     // output stored as bfloat16 instead of fp16
  bool bf16;                         // q and the cache are bfloat16 (bfloat16 MMAs); implies out_bf16
  bool kv8;                          // int8 cache with fp16 per-token scales
  const void *k_scale_h, *v_scale_h;
  // sliding window + sink (contiguous fixed mode): see DecodeParams.  has_window = false: identity page map
  bool has_window;
  int sink, win_start, sink_pages, win_first_page, window_pages_total;
  void* ws;
  size_t ws_bytes;
  cudaStream_t stream;
};

int run_decode(const DecodeCall& c) {
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != FA_OK) return rc;
  const int G = c.H_Q / c.H_KV;
  const int slot_rows = G < 16 ? G : 16;
  const int Dp = padded_decode_d(c.D);      // head dimension of the kernel build that serves c.D
  if (Dp == 0 || (c.kv8 && c.D % 16 != 0))
    return fail(FA_ERR_UNSUPPORTED, "head dimension %d is not built for this operator", c.D);
  const size_t need_ws = fa::decode_workspace_bytes(c.B, c.H_Q, c.H_KV, Dp, kMaxDecodeCtas);
  if (c.ws == nullptr || c.ws_bytes < need_ws)
    return fail(FA_ERR_WORKSPACE, "decode workspace too small: need %zu bytes, got %zu", need_ws, c.ws_bytes);
  if ((reinterpret_cast<uintptr_t>(c.ws) & 255) != 0)
    return fail(FA_ERR_WORKSPACE, "decode workspace must be 256-byte aligned");
  if (c.rows_total >= (1ll << 31)) return fail(FA_ERR_UNSUPPORTED, "KV cache has too many rows for one tensor map");

  const int kv_elem_bytes = c.kv8 ? 1 : 2;
  fa::DecodeLaunchConfig cfg = pick_decode_config(Dp, G, slot_rows, c.B, kv_elem_bytes, c.int8, di);
  fa::DecodeParams p;
  memset(&p, 0, sizeof(p));
  p.q = static_cast<const __half*>(c.q);
  p.out = static_cast<__half*>(c.out);
  p.out_bf16 = (c.out_bf16 || c.bf16) ? 1 : 0;
  p.block_table = c.block_table;
  p.lens = c.lens;
  p.q_scale = c.q_scale;
  p.k_scale = c.k_scale;
  p.scores_out = c.scores_out;
  p.k_scale_h = static_cast<const __half*>(c.k_scale_h);
  p.v_scale_h = static_cast<const __half*>(c.v_scale_h);
  uint8_t* ws = static_cast<uint8_t*>(c.ws);
  p.status = reinterpret_cast<int32_t*>(ws + fa::kWsStatusOffset);
  p.prefix = reinterpret_cast<int32_t*>(ws + fa::kWsPrefixOffset);
  const size_t prefix_bytes = (((size_t)(c.B + 1) * 4 + 255) & ~(size_t)255);
  p.counters = reinterpret_cast<unsigned long long*>(ws + fa::kWsCountersOffset);
  p.partials = reinterpret_cast<float*>(ws + fa::kWsPrefixOffset + prefix_bytes);
  p.B = c.B; p.H_Q = c.H_Q; p.H_KV = c.H_KV; p.G = G;
  p.D_real = c.D;
  p.n_gblk = (G + 15) / 16;
  p.HV = c.H_KV * p.n_gblk;
  p.mode = c.mode; p.fixed_len = c.fixed_len; p.N = c.N;
  p.sink = 0; p.win_start = 0; p.sink_pages = INT_MAX; p.win_first_page = 0; p.window_pages_total = 0;
  if (c.has_window) {
    p.sink = c.sink; p.win_start = c.win_start; p.sink_pages = c.sink_pages;
    p.win_first_page = c.win_first_page; p.window_pages_total = c.window_pages_total;
  }
  p.bt_stride = c.bt_stride;
  p.num_pages = c.num_pages;
  p.stages = cfg.stages;
  p.slot_rows = slot_rows;
  p.scale = 1.0f / sqrtf((float)c.D);
  p.scale_log2 = p.scale * 1.4426950408889634f;
  long long n_cta = (long long)di.sm_count * cfg.ctas_per_sm;
  if (n_cta > kMaxDecodeCtas) n_cta = kMaxDecodeCtas;
  if (c.max_units > 0 && c.max_units < n_cta) n_cta = c.max_units;
  if (n_cta < 1) n_cta = 1;
  p.n_cta = (int)n_cta;

  CUtensorMap kmap, vmap;
  rc = c.kv8 ? make_rows_map_u8(&kmap, c.k, c.rows_total, c.D) : make_rows_map(&kmap, c.k, c.rows_total, c.D, 16);
  if (rc != FA_OK) return rc;
  rc = c.kv8 ? make_rows_map_u8(&vmap, c.v, c.rows_total, c.D) : make_rows_map(&vmap, c.v, c.rows_total, c.D, 16);
  if (rc != FA_OK) return rc;
  const size_t smem = fa::decode_smem_bytes(Dp, cfg.warps, cfg.stages, slot_rows, c.B, kv_elem_bytes);
  const int kind = c.kv8 ? fa::kKindInt8KV : (c.int8 ? fa::kKindInt8QK : (c.bf16 ? fa::kKindBF16 : fa::kKindF16));
  cudaError_t e = fa::launch_decode(kmap, vmap, p, Dp, kind, cfg.warps, smem, c.stream);
  if (e != cudaSuccess) return fail(FA_ERR_CUDA, "decode launch failed: %s", cudaGetErrorString(e));
  return FA_OK;
}

int check_decode_common(const void* q, const void* k, const void* v, const void* out, int B, int H_Q, int H_KV,
                        int D) {
  FA_REQUIRE(q && k && v && out, "null tensor pointer");
  FA_REQUIRE(B > 0 && H_Q > 0 && H_KV > 0 && D > 0, "B, H_Q, H_KV and D must be positive");
  FA_REQUIRE(H_Q >= H_KV, "H_Q must be >= H_KV");
  FA_REQUIRE(H_Q % H_KV == 0, "H_Q must be divisible by H_KV");
  FA_REQUIRE(D <= 256, "D must be <= 256");
  if (padded_decode_d(D) == 0)
    return fail(FA_ERR_UNSUPPORTED, "head dimension %d is not built (decode serves multiples of 8 up to 256)", D);
  FA_REQUIRE((reinterpret_cast<uintptr_t>(k) & 15) == 0 && (reinterpret_cast<uintptr_t>(v) & 15) == 0,
             "k and v must be 16-byte aligned");
  FA_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
             "q and out must be 16-byte aligned");
  return FA_OK;
}

// ---- built-in decode scratch (fa_paged_decode_gqa_f16_static_scratch) -------
constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_static_decode_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime, not a device
// address, so the device address is looked up once per device and cached.
void* g_static_scratch_ptr[64] = {nullptr};
std::mutex g_static_scratch_mu;

// Set-up, once per device, with that device current.  The status word and the arrival counters
// (the first kWsInitBytes of any decode workspace) must be zero before the first launch, exactly as
// fa_decode_workspace_init leaves a caller-owned workspace; everything behind them is written
// before it is read.  The clear is finished before the address is handed to any caller, so it can
// never wipe a status bit that a concurrent call has set.
int static_scratch_for_current_device(void** out, cudaStream_t stream) {
  int dev = 0;
  FA_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(FA_ERR_CUDA, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_static_scratch_mu);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    FA_CUDA(cudaGetSymbolAddress(&ptr, g_static_decode_scratch));
    if (ptr == nullptr) return fail(FA_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    FA_CUDA(cudaMemsetAsync(ptr, 0, fa::kWsInitBytes, stream));
    FA_CUDA(cudaStreamSynchronize(stream));
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return FA_OK;
}

int check_paged_args(const void* q, const void* k_cache, const void* v_cache, const void* out,
                     const int32_t* block_table, const int32_t* seq_lens, int B, int H_Q, int H_KV, int D,
                     int64_t num_pages, int block_table_stride) {
  int rc = check_decode_common(q, k_cache, v_cache, out, B, H_Q, H_KV, D);
  if (rc != FA_OK) return rc;
  FA_REQUIRE(block_table && seq_lens, "null block_table / seq_lens");
  FA_REQUIRE(num_pages > 0, "num_pages must be positive");
  FA_REQUIRE(block_table_stride > 0, "block_table_stride must be positive");
  return FA_OK;
}

}  // namespace

extern "C" {

int fa_version(void) { return 101; }

const char* fa_last_error(void) { return g_err; }

size_t fa_decode_workspace_bytes(int B, int H_Q, int H_KV, int D) {
  if (B <= 0 || H_Q <= 0 || H_KV <= 0 || H_Q % H_KV != 0 || padded_decode_d(D) == 0) return 0;
  return fa::decode_workspace_bytes(B, H_Q, H_KV, padded_decode_d(D), kMaxDecodeCtas);
}

int fa_decode_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  if (workspace == nullptr) {   // the built-in scratch of fa_paged_decode_gqa_f16_static_scratch
    int rc = static_scratch_for_current_device(&workspace, static_cast<cudaStream_t>(stream));
    if (rc != FA_OK) return rc;
    workspace_bytes = fa::kWsInitBytes;
  }
  FA_REQUIRE(workspace_bytes >= fa::kWsInitBytes, "workspace too small");
  FA_CUDA(cudaMemsetAsync(workspace, 0, fa::kWsInitBytes, static_cast<cudaStream_t>(stream)));
  return FA_OK;
}

int fa_decode_status(const void* workspace, void* stream, int* host_status_out) {
  FA_REQUIRE(host_status_out != nullptr, "null pointer");
  if (workspace == nullptr) {   // the built-in scratch of fa_paged_decode_gqa_f16_static_scratch
    void* builtin = nullptr;
    int rc = static_scratch_for_current_device(&builtin, static_cast<cudaStream_t>(stream));
    if (rc != FA_OK) return rc;
    workspace = builtin;
  }
  int32_t v = 0;
  FA_CUDA(cudaMemcpyAsync(&v, static_cast<const uint8_t*>(workspace) + fa::kWsStatusOffset, 4, cudaMemcpyDeviceToHost,
                          static_cast<cudaStream_t>(stream)));
  FA_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  *host_status_out = v;
  if (v != 0) return fail(FA_ERR_DEVICE_STATUS, "decode kernel recorded device status 0x%x", v);
  return FA_OK;
}

int fa_decode_set_tuning(int warps, int stages, int ctas_per_sm) {
  g_cfg_override = {warps, stages, ctas_per_sm};
  return FA_OK;
}

static int paged_decode_impl(const void* q, const void* k_cache, const void* v_cache, void* out,
                             const int32_t* block_table, const int32_t* seq_lens, int B, int H_Q, int H_KV, int D,
                             int64_t num_pages, int block_table_stride, int64_t max_seq_len, void* workspace,
                             size_t workspace_bytes, void* stream, bool out_bf16, bool bf16 = false) {
  int rc = check_paged_args(q, k_cache, v_cache, out, block_table, seq_lens, B, H_Q, H_KV, D, num_pages,
                            block_table_stride);
  if (rc != FA_OK) return rc;
  DecodeCall c{};
  c.q = q; c.k = k_cache; c.v = v_cache; c.out = out;
  c.block_table = block_table; c.lens = seq_lens;
  c.B = B; c.H_Q = H_Q; c.H_KV = H_KV; c.D = D;
  c.mode = fa::kModePaged; c.N = 0; c.bt_stride = block_table_stride;
  c.num_pages = num_pages;
  c.rows_total = (long long)num_pages * H_KV * 16;
  long long max_pages = block_table_stride;
  if (max_seq_len > 0 && (max_seq_len + 15) / 16 < max_pages) max_pages = (max_seq_len + 15) / 16;
  c.max_units = (long long)B * H_KV * ((H_Q / H_KV + 15) / 16) * max_pages;
  c.int8 = false;
  c.out_bf16 = out_bf16;
  c.bf16 = bf16;
  c.ws = workspace; c.ws_bytes = workspace_bytes; c.stream = static_cast<cudaStream_t>(stream);
  return run_decode(c);
}

int fa_paged_decode_gqa_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                             const int32_t* block_table, const int32_t* seq_lens, int B, int H_Q, int H_KV, int D,
                             int64_t num_pages, int block_table_stride, int64_t max_seq_len, void* workspace,
                             size_t workspace_bytes, void* stream) {
  return paged_decode_impl(q, k_cache, v_cache, out, block_table, seq_lens, B, H_Q, H_KV, D, num_pages,
                           block_table_stride, max_seq_len, workspace, workspace_bytes, stream, true, true);
}

int fa_paged_decode_gqa_f16(const void* q, const void* k_cache, const void* v_cache, void* out,
                            const int32_t* block_table, const int32_t* seq_lens, int B, int H_Q, int H_KV, int D,
                            int64_t num_pages, int block_table_stride, int64_t max_seq_len, void* workspace,
                            size_t workspace_bytes, void* stream) {
  return paged_decode_impl(q, k_cache, v_cache, out, block_table, seq_lens, B, H_Q, H_KV, D, num_pages,
                           block_table_stride, max_seq_len, workspace, workspace_bytes, stream, false);
}

int fa_paged_decode_gqa_f16_out_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                                     const int32_t* block_table, const int32_t* seq_lens, int B, int H_Q, int H_KV,
                                     int D, int64_t num_pages, int block_table_stride, int64_t max_seq_len,
                                     void* workspace, size_t workspace_bytes, void* stream) {
  return paged_decode_impl(q, k_cache, v_cache, out, block_table, seq_lens, B, H_Q, H_KV, D, num_pages,
                           block_table_stride, max_seq_len, workspace, workspace_bytes, stream, true);
}

static int decode_gqa_impl(const void* q, const void* k, const void* v, void* out, int B, int H_Q, int H_KV, int N,
                           int D, int causal, int cache_len, void* workspace, size_t workspace_bytes, void* stream,
                           bool bf16) {
  int rc = check_decode_common(q, k, v, out, B, H_Q, H_KV, D);
  if (rc != FA_OK) return rc;
  FA_REQUIRE(N > 0, "N must be positive");
  FA_REQUIRE(cache_len >= 0, "cache_len must be non-negative");
  FA_REQUIRE(cache_len < N, "cache_len must be less than sequence length");
  DecodeCall c{};
  c.q = q; c.k = k; c.v = v; c.out = out;
  c.B = B; c.H_Q = H_Q; c.H_KV = H_KV; c.D = D;
  c.mode = fa::kModeContigFixed; c.N = N;
  c.fixed_len = causal ? cache_len + 1 : N;
  c.bt_stride = 0; c.num_pages = 0;
  c.rows_total = (long long)B * H_KV * N;
  c.max_units = (long long)B * H_KV * ((H_Q / H_KV + 15) / 16) * ((c.fixed_len + 15) / 16);
  c.bf16 = bf16;
  c.ws = workspace; c.ws_bytes = workspace_bytes; c.stream = static_cast<cudaStream_t>(stream);
  return run_decode(c);
}

int fa_decode_gqa_f16(const void* q, const void* k, const void* v, void* out, int B, int H_Q, int H_KV, int N, int D,
                      int causal, int cache_len, void* workspace, size_t workspace_bytes, void* stream) {
  return decode_gqa_impl(q, k, v, out, B, H_Q, H_KV, N, D, causal, cache_len, workspace, workspace_bytes, stream, false);
}

int fa_decode_gqa_bf16(const void* q, const void* k, const void* v, void* out, int B, int H_Q, int H_KV, int N, int D,
                       int causal, int cache_len, void* workspace, size_t workspace_bytes, void* stream) {
  return decode_gqa_impl(q, k, v, out, B, H_Q, H_KV, N, D, causal, cache_len, workspace, workspace_bytes, stream, true);
}

int fa_decode_sliding_window_gqa_f16(const void* q, const void* k, const void* v, void* out, int B, int H_Q, int H_KV,
                                     int N, int D, int cache_len, int window_size, int sink_size, void* workspace,
                                     size_t workspace_bytes, void* stream) {
  int rc = check_decode_common(q, k, v, out, B, H_Q, H_KV, D);
  if (rc != FA_OK) return rc;
  FA_REQUIRE(N > 0, "N must be positive");
  // Attended keys: k < sink_size, or window_start <= k <= cache_len, always with k < N.
  long long end = (long long)cache_len + 1;
  if (end > N) end = N;
  long long wstart = end - (long long)window_size;   // window_size <= 0 leaves the window empty
  if (wstart < 0) wstart = 0;
  if (end < 0) end = 0;
  if (wstart > end) wstart = end;
  long long sink = sink_size < 0 ? 0 : sink_size;
  if (sink > N) sink = N;
  const long long vis_end = sink > end ? sink : end;
  const int ns = (int)((sink + 15) / 16);
  const int end_pages = (int)((end + 15) / 16);
  int first_w = (int)(wstart / 16);
  if (first_w < ns) first_w = ns;                     // pages shared with the sink are visited once
  int win_pages = wstart < end ? end_pages - first_w : 0;
  if (win_pages < 0) win_pages = 0;
  DecodeCall c{};
  c.q = q; c.k = k; c.v = v; c.out = out;
  c.B = B; c.H_Q = H_Q; c.H_KV = H_KV; c.D = D;
  c.mode = fa::kModeContigFixed; c.N = N;
  c.fixed_len = (int)vis_end;
  c.has_window = (ns + win_pages) > 0;
  c.sink = (int)sink; c.win_start = (int)wstart; c.sink_pages = ns; c.win_first_page = first_w;
  c.window_pages_total = ns + win_pages;
  c.bt_stride = 0; c.num_pages = 0;
  c.rows_total = (long long)B * H_KV * N;
  c.max_units = (long long)B * H_KV * ((H_Q / H_KV + 15) / 16) * (ns + win_pages);
  c.ws = workspace; c.ws_bytes = workspace_bytes; c.stream = static_cast<cudaStream_t>(stream);
  return run_decode(c);
}

int fa_decode_varlen_f16(const void* q, const void* k, const void* v, void* out, const int32_t* cache_lens, int B,
                         int H_Q, int H_KV, int max_N, int D, int causal, void* workspace, size_t workspace_bytes,
                         void* stream) {
  (void)causal;
  int rc = check_decode_common(q, k, v, out, B, H_Q, H_KV, D);
  if (rc != FA_OK) return rc;
  FA_REQUIRE(cache_lens != nullptr, "null cache_lens");
  FA_REQUIRE(max_N > 0, "max_N must be positive");
  DecodeCall c{};
  c.q = q; c.k = k; c.v = v; c.out = out; c.lens = cache_lens;
  c.B = B; c.H_Q = H_Q; c.H_KV = H_KV; c.D = D;
  c.mode = fa::kModeContigVarlen; c.N = max_N;
  c.rows_total = (long long)B * H_KV * max_N;
  c.max_units = (long long)B * H_KV * ((H_Q / H_KV + 15) / 16) * ((max_N + 15) / 16);
  c.ws = workspace; c.ws_bytes = workspace_bytes; c.stream = static_cast<cudaStream_t>(stream);
  return run_decode(c);
}

int fa_decode_int8_gqa(const void* q, const void* k, const void* v, void* out, const float* q_scale,
                       const float* k_scale, int B, int H_Q, int H_KV, int N, int D, int cache_len,
                       int32_t* scores_i32_out, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_decode_common(q, k, v, out, B, H_Q, H_KV, D);
  if (rc != FA_OK) return rc;
  FA_REQUIRE(q_scale && k_scale, "null q_scale / k_scale");
  FA_REQUIRE(N > 0, "N must be positive");
  FA_REQUIRE(cache_len >= 0, "cache_len must be non-negative");
  FA_REQUIRE(cache_len < N, "cache_len must be less than sequence length");
  DecodeCall c{};
  c.q = q; c.k = k; c.v = v; c.out = out;
  c.q_scale = q_scale; c.k_scale = k_scale; c.scores_out = scores_i32_out;
  c.B = B; c.H_Q = H_Q; c.H_KV = H_KV; c.D = D;
  c.mode = fa::kModeContigFixed; c.N = N; c.fixed_len = cache_len + 1;
  c.rows_total = (long long)B * H_KV * N;
  c.max_units = (long long)B * H_KV * ((H_Q / H_KV + 15) / 16) * ((c.fixed_len + 15) / 16);
  c.int8 = true;
  c.ws = workspace; c.ws_bytes = workspace_bytes; c.stream = static_cast<cudaStream_t>(stream);
  return run_decode(c);
}

int fa_decode_int8_kv_cache_gqa(const void* q, const void* k_int8, const void* v_int8, const void* k_scale,
                                const void* v_scale, void* out, int B, int H_Q, int H_KV, int N, int D, int cache_len,
                                void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_decode_common(q, k_int8, v_int8, out, B, H_Q, H_KV, D);
  if (rc != FA_OK) return rc;
  FA_REQUIRE(k_scale && v_scale, "null k_scale / v_scale");
  FA_REQUIRE(N > 0, "N must be positive");
  long long len = (long long)cache_len + 1;   // keys j <= cache_len, j < N
  if (len > N) len = N;
  if (len < 0) len = 0;
  DecodeCall c{};
  c.q = q; c.k = k_int8; c.v = v_int8; c.out = out;
  c.k_scale_h = k_scale; c.v_scale_h = v_scale;
  c.B = B; c.H_Q = H_Q; c.H_KV = H_KV; c.D = D;
  c.mode = fa::kModeContigFixed; c.N = N; c.fixed_len = (int)len;
  c.rows_total = (long long)B * H_KV * N;
  c.max_units = (long long)B * H_KV * ((H_Q / H_KV + 15) / 16) * ((c.fixed_len + 15) / 16);
  c.kv8 = true;
  c.ws = workspace; c.ws_bytes = workspace_bytes; c.stream = static_cast<cudaStream_t>(stream);
  return run_decode(c);
}

// ---------------------------------------------------------------------------
// Paged decode for callers that cannot allocate device memory.
//
// The split-KV scratch (status word, arrival counters, page prefix sums, per-CTA
// partial results) lives in a fixed array that is part of the loaded module image,
// so the call needs no cudaMalloc and no caller-provided workspace.  Every device
// that loads the library holds these bytes until the process exits.
// ---------------------------------------------------------------------------
int fa_paged_decode_gqa_f16_static_scratch(const void* q, const void* k_cache, const void* v_cache, void* out,
                                           const int32_t* block_table, const int32_t* seq_lens, int B, int H_Q,
                                           int H_KV, int D, int64_t num_pages, int block_table_stride,
                                           int64_t max_seq_len, void* stream) {
  // every argument check comes first, so that a bad call never touches the device
  int rc = check_paged_args(q, k_cache, v_cache, out, block_table, seq_lens, B, H_Q, H_KV, D, num_pages,
                            block_table_stride);
  if (rc != FA_OK) return rc;
  const size_t need = fa::decode_workspace_bytes(B, H_Q, H_KV, padded_decode_d(D), kMaxDecodeCtas);
  if (need > kStaticScratchBytes)
    return fail(FA_ERR_WORKSPACE,
                "this shape needs %zu bytes of decode scratch but the built-in scratch holds %zu: use "
                "fa_paged_decode_gqa_f16 with a caller-owned workspace",
                need, (size_t)kStaticScratchBytes);
  void* scratch = nullptr;
  rc = static_scratch_for_current_device(&scratch, static_cast<cudaStream_t>(stream));
  if (rc != FA_OK) return rc;
  return fa_paged_decode_gqa_f16(q, k_cache, v_cache, out, block_table, seq_lens, B, H_Q, H_KV, D, num_pages,
                                 block_table_stride, max_seq_len, scratch, kStaticScratchBytes, stream);
}

static int g_prefill_impl = 0;  // 0 auto, 1 mma.sync kernel, 2 tcgen05 kernel

int fa_prefill_set_impl(int impl) {
  FA_REQUIRE(impl >= 0 && impl <= 3, "impl must be 0 (auto), 1 (mma.sync), 2 (tcgen05) or 3 (tcgen05, half of exp2 as FMA polynomial)");
  fa::prefill_tc5_set_poly(impl == 3);
  g_prefill_impl = impl == 3 ? 0 : impl;  // 3: automatic choice, polynomial variant when the tcgen05 kernel runs
  return FA_OK;
}

int fa_prefill_status(void* stream, int* host_status_out, int clear) {
  FA_REQUIRE(host_status_out != nullptr, "null pointer");
  FA_CUDA(fa::prefill_status(host_status_out, static_cast<cudaStream_t>(stream)));
  if (clear) FA_CUDA(fa::prefill_status_clear(static_cast<cudaStream_t>(stream)));
  if (*host_status_out != 0)
    return fail(FA_ERR_DEVICE_STATUS, "prefill kernel recorded device status 0x%x", *host_status_out);
  return FA_OK;
}

static int run_prefill(fa::PrefillParams& p, int D, cudaStream_t stream) {
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != FA_OK) return rc;
  // kernels are built for 64, 128 and 256 columns; a head dimension in between runs on the next larger build
  const int Dp = padded_decode_d(D);
  if (Dp == 0)
    return fail(FA_ERR_UNSUPPORTED, "head dimension %d is not built (multiples of 8 up to 256 are)", D);
  p.D_real = D;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)D);
  D = Dp;
  cudaError_t e;
  const bool tc5_ok = fa::prefill_tc5_supported(p, D);
  if (g_prefill_impl == 2 && !tc5_ok)
    return fail(FA_ERR_UNSUPPORTED, "the tcgen05 prefill kernel supports D = 64 and 128 only");
  if (p.in_bf16 && !tc5_ok)
    return fail(FA_ERR_UNSUPPORTED, "bfloat16 prefill is served by the tcgen05 kernel: head dimension up to 128");
  if (tc5_ok && (g_prefill_impl != 1 || p.in_bf16)) {
    EncodeTiledFn enc;
    rc = get_encode(&enc);
    if (rc != FA_OK) return rc;
    e = fa::launch_prefill_tc5(p, D, reinterpret_cast<void*>(enc), stream);
  } else {
    e = fa::launch_prefill_mma(p, D, stream);
  }
  if (e != cudaSuccess) return fail(FA_ERR_CUDA, "prefill launch failed: %s", cudaGetErrorString(e));
  return FA_OK;
}

static int prefill_dense_impl(const void* q, const void* k, const void* v, void* out, int B, int H_Q, int H_KV, int N,
                              int D, int causal, void* stream, bool in_bf16) {
  int rc = check_decode_common(q, k, v, out, B, H_Q, H_KV, D);
  if (rc != FA_OK) return rc;
  FA_REQUIRE(N > 0, "N must be positive");
  FA_REQUIRE(B <= 65535 && H_Q <= 65535, "B and H_Q must be <= 65535");
  fa::PrefillParams p;
  memset(&p, 0, sizeof(p));
  p.q = static_cast<const __half*>(q); p.k = static_cast<const __half*>(k); p.v = static_cast<const __half*>(v);
  p.out = static_cast<__half*>(out);
  p.cu_seqlens = nullptr;
  p.batch = B; p.H_Q = H_Q; p.H_KV = H_KV; p.N = N; p.max_seqlen = N; p.total = (long long)B * N;
  p.q_batch_stride = (long long)H_Q * N * D; p.q_head_stride = (long long)N * D; p.q_tok_stride = D;
  p.kv_batch_stride = (long long)H_KV * N * D; p.kv_head_stride = (long long)N * D; p.kv_tok_stride = D;
  p.causal = causal ? 1 : 0;
  p.in_bf16 = in_bf16 ? 1 : 0;
  return run_prefill(p, D, static_cast<cudaStream_t>(stream));
}

int fa_prefill_dense_f16(const void* q, const void* k, const void* v, void* out, int B, int H_Q, int H_KV, int N,
                         int D, int causal, void* stream) {
  return prefill_dense_impl(q, k, v, out, B, H_Q, H_KV, N, D, causal, stream, false);
}

int fa_prefill_dense_bf16(const void* q, const void* k, const void* v, void* out, int B, int H_Q, int H_KV, int N,
                          int D, int causal, void* stream) {
  return prefill_dense_impl(q, k, v, out, B, H_Q, H_KV, N, D, causal, stream, true);
}

static int prefill_varlen_impl(const void* q, const void* k, const void* v, void* out, const int32_t* cu_seqlens,
                               int batch, int64_t total, int H_Q, int H_KV, int D, int max_seqlen, int causal,
                               void* stream, bool out_bf16, bool in_bf16 = false) {
  int rc = check_decode_common(q, k, v, out, batch, H_Q, H_KV, D);
  if (rc != FA_OK) return rc;
  FA_REQUIRE(cu_seqlens != nullptr, "null cu_seqlens");
  FA_REQUIRE(total > 0, "total must be positive");
  FA_REQUIRE(max_seqlen > 0, "max_seqlen must be positive");
  FA_REQUIRE(batch <= 65535 && H_Q <= 65535, "batch and H_Q must be <= 65535");
  fa::PrefillParams p;
  memset(&p, 0, sizeof(p));
  p.q = static_cast<const __half*>(q); p.k = static_cast<const __half*>(k); p.v = static_cast<const __half*>(v);
  p.out = static_cast<__half*>(out);
  p.cu_seqlens = cu_seqlens;
  p.batch = batch; p.H_Q = H_Q; p.H_KV = H_KV; p.N = 0; p.max_seqlen = max_seqlen; p.total = total;
  p.q_batch_stride = 0; p.q_head_stride = D; p.q_tok_stride = (long long)H_Q * D;
  p.kv_batch_stride = 0; p.kv_head_stride = D; p.kv_tok_stride = (long long)H_KV * D;
  p.causal = causal ? 1 : 0;
  p.out_bf16 = out_bf16 ? 1 : 0;
  p.in_bf16 = in_bf16 ? 1 : 0;
  return run_prefill(p, D, static_cast<cudaStream_t>(stream));
}

int fa_prefill_varlen_bf16(const void* q, const void* k, const void* v, void* out, const int32_t* cu_seqlens,
                           int batch, int64_t total, int H_Q, int H_KV, int D, int max_seqlen, int causal,
                           void* stream) {
  return prefill_varlen_impl(q, k, v, out, cu_seqlens, batch, total, H_Q, H_KV, D, max_seqlen, causal, stream, true,
                             true);
}

int fa_prefill_varlen_f16(const void* q, const void* k, const void* v, void* out, const int32_t* cu_seqlens,
                          int batch, int64_t total, int H_Q, int H_KV, int D, int max_seqlen, int causal,
                          void* stream) {
  return prefill_varlen_impl(q, k, v, out, cu_seqlens, batch, total, H_Q, H_KV, D, max_seqlen, causal, stream, false);
}

int fa_prefill_varlen_f16_out_bf16(const void* q, const void* k, const void* v, void* out, const int32_t* cu_seqlens,
                                   int batch, int64_t total, int H_Q, int H_KV, int D, int max_seqlen, int causal,
                                   void* stream) {
  return prefill_varlen_impl(q, k, v, out, cu_seqlens, batch, total, H_Q, H_KV, D, max_seqlen, causal, stream, true);
}

static int rope_append_impl(const void* q, const void* k, const void* v, const float* cos, const float* sin,
                            void* q_out, void* k_out, void* k_cache, void* v_cache, const int32_t* block_table,
                            const int32_t* positions, const int32_t* cu_seqlens, int T, int batch, int H_Q, int H_KV,
                            int D, int rot_dim, int64_t num_pages, int block_table_stride, void* stream, bool bf16) {
  FA_REQUIRE(q && k && v && cos && sin && q_out, "null tensor pointer");
  FA_REQUIRE(T >= 0 && batch > 0 && H_Q > 0 && H_KV > 0, "T must be >= 0; batch, H_Q, H_KV positive");
  FA_REQUIRE(D > 0 && D <= 256 && D % 8 == 0, "D must be a multiple of 8, at most 256");
  FA_REQUIRE(rot_dim > 0 && rot_dim <= D && rot_dim % 16 == 0 && (D - rot_dim) % 8 == 0,
             "rot_dim must be a multiple of 16, at most D, with D - rot_dim a multiple of 8");
  FA_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), "k_cache and v_cache must be given together");
  if (k_cache != nullptr) {
    FA_REQUIRE(block_table != nullptr && block_table_stride > 0 && num_pages > 0,
               "block_table, its stride and num_pages are required with a cache");
  }
  FA_REQUIRE(cu_seqlens != nullptr || (positions != nullptr && T == batch),
             "without cu_seqlens there is one token per sequence (T == batch) and positions is required");
  for (const void* ptr : {q, k, v, (const void*)q_out, (const void*)k_out, (const void*)k_cache, (const void*)v_cache})
    FA_REQUIRE((reinterpret_cast<uintptr_t>(ptr) & 15) == 0, "tensor pointers must be 16-byte aligned");
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != FA_OK) return rc;
  fa::RopeAppendParams p;
  memset(&p, 0, sizeof(p));
  p.q = static_cast<const __half*>(q); p.k = static_cast<const __half*>(k); p.v = static_cast<const __half*>(v);
  p.cos = cos; p.sin = sin;
  p.q_out = static_cast<__half*>(q_out); p.k_out = static_cast<__half*>(k_out);
  p.k_cache = static_cast<__half*>(k_cache); p.v_cache = static_cast<__half*>(v_cache);
  p.block_table = block_table; p.positions = positions; p.cu_seqlens = cu_seqlens;
  p.T = T; p.batch = batch; p.H_Q = H_Q; p.H_KV = H_KV; p.D = D; p.rot_dim = rot_dim;
  p.bt_stride = block_table_stride; p.num_pages = num_pages;
  p.bf16 = bf16 ? 1 : 0;
  FA_CUDA(fa::prefill_status_ptr(&p.status));
  cudaError_t e = fa::launch_rope_append(p, di.sm_count, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(FA_ERR_CUDA, "rope/append launch failed: %s", cudaGetErrorString(e));
  return FA_OK;
}

int fa_rope_append_paged_f16(const void* q, const void* k, const void* v, const float* cos, const float* sin,
                             void* q_out, void* k_out, void* k_cache, void* v_cache, const int32_t* block_table,
                             const int32_t* positions, const int32_t* cu_seqlens, int T, int batch, int H_Q, int H_KV,
                             int D, int rot_dim, int64_t num_pages, int block_table_stride, void* stream) {
  return rope_append_impl(q, k, v, cos, sin, q_out, k_out, k_cache, v_cache, block_table, positions, cu_seqlens, T,
                          batch, H_Q, H_KV, D, rot_dim, num_pages, block_table_stride, stream, false);
}

int fa_rope_append_paged_bf16(const void* q, const void* k, const void* v, const float* cos, const float* sin,
                              void* q_out, void* k_out, void* k_cache, void* v_cache, const int32_t* block_table,
                              const int32_t* positions, const int32_t* cu_seqlens, int T, int batch, int H_Q, int H_KV,
                              int D, int rot_dim, int64_t num_pages, int block_table_stride, void* stream) {
  return rope_append_impl(q, k, v, cos, sin, q_out, k_out, k_cache, v_cache, block_table, positions, cu_seqlens, T,
                          batch, H_Q, H_KV, D, rot_dim, num_pages, block_table_stride, stream, true);
}

static int qkv_rope_append_impl(const void* qkv, const void* q_weight, const void* k_weight, const float* cos,
                                const float* sin, void* q_out, void* k_out, void* v_out, void* k_cache, void* v_cache,
                                const int32_t* block_table, const int32_t* positions, const int32_t* cu_seqlens, int T,
                                int batch, int H_Q, int H_KV, int D, float eps, int64_t num_pages,
                                int block_table_stride, void* stream, bool bf16) {
  FA_REQUIRE(qkv && cos && sin && q_out, "null tensor pointer");
  FA_REQUIRE(T >= 0 && batch > 0 && H_Q > 0 && H_KV > 0, "T must be >= 0; batch, H_Q, H_KV positive");
  if (!supported_d(D)) return fail(FA_ERR_UNSUPPORTED, "head dimension %d is not built (supported: 64, 128, 256)", D);
  FA_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), "k_cache and v_cache must be given together");
  if (k_cache != nullptr) {
    FA_REQUIRE(block_table != nullptr && block_table_stride > 0 && num_pages > 0,
               "block_table, its stride and num_pages are required with a cache");
  }
  FA_REQUIRE(cu_seqlens != nullptr || (positions != nullptr && T == batch),
             "without cu_seqlens there is one token per sequence (T == batch) and positions is required");
  fa::QkvRopeAppendParams p;
  memset(&p, 0, sizeof(p));
  p.qkv = qkv; p.q_weight = q_weight; p.k_weight = k_weight; p.eps = eps;
  p.v_out = static_cast<__half*>(v_out);
  p.r.cos = cos; p.r.sin = sin;
  p.r.q_out = static_cast<__half*>(q_out); p.r.k_out = static_cast<__half*>(k_out);
  p.r.k_cache = static_cast<__half*>(k_cache); p.r.v_cache = static_cast<__half*>(v_cache);
  p.r.block_table = block_table; p.r.positions = positions; p.r.cu_seqlens = cu_seqlens;
  p.r.T = T; p.r.batch = batch; p.r.H_Q = H_Q; p.r.H_KV = H_KV; p.r.D = D; p.r.rot_dim = D;
  p.r.bt_stride = block_table_stride; p.r.num_pages = num_pages;
  p.r.bf16 = bf16 ? 1 : 0;
  FA_CUDA(fa::prefill_status_ptr(&p.r.status));
  cudaError_t e = fa::launch_qkv_rope_append(p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(FA_ERR_CUDA, "qkv norm/rope/append launch failed: %s", cudaGetErrorString(e));
  return FA_OK;
}

int fa_qkv_rope_append_f16(const void* qkv, const void* q_weight, const void* k_weight, const float* cos,
                           const float* sin, void* q_out, void* k_out, void* v_out, void* k_cache, void* v_cache,
                           const int32_t* block_table, const int32_t* positions, const int32_t* cu_seqlens, int T,
                           int batch, int H_Q, int H_KV, int D, float eps, int64_t num_pages, int block_table_stride,
                           void* stream) {
  return qkv_rope_append_impl(qkv, q_weight, k_weight, cos, sin, q_out, k_out, v_out, k_cache, v_cache, block_table,
                              positions, cu_seqlens, T, batch, H_Q, H_KV, D, eps, num_pages, block_table_stride,
                              stream, false);
}

int fa_qkv_rope_append_bf16(const void* qkv, const void* q_weight, const void* k_weight, const float* cos,
                            const float* sin, void* q_out, void* k_out, void* v_out, void* k_cache, void* v_cache,
                            const int32_t* block_table, const int32_t* positions, const int32_t* cu_seqlens, int T,
                            int batch, int H_Q, int H_KV, int D, float eps, int64_t num_pages, int block_table_stride,
                            void* stream) {
  return qkv_rope_append_impl(qkv, q_weight, k_weight, cos, sin, q_out, k_out, v_out, k_cache, v_cache, block_table,
                              positions, cu_seqlens, T, batch, H_Q, H_KV, D, eps, num_pages, block_table_stride,
                              stream, true);
}

int fa_add_rmsnorm_bf16(void* x, const void* delta, const void* weight, void* out, int64_t rows, int cols, float eps,
                        void* stream) {
  FA_REQUIRE(x && weight && out, "null tensor pointer");
  FA_REQUIRE(rows >= 0 && cols > 0 && cols % 8 == 0 && cols <= 8 * 8 * 256, "cols must be a multiple of 8, at most 16384");
  FA_CUDA(fa::launch_add_rmsnorm(x, delta, weight, out, rows, cols, eps, static_cast<cudaStream_t>(stream)));
  return FA_OK;
}

int fa_qk_norm_split_f16(const void* qkv, const void* q_weight, const void* k_weight, void* q, void* k, void* v,
                         int64_t T, int H_Q, int H_KV, int D, float eps, void* stream) {
  FA_REQUIRE(qkv && q && k && v, "null tensor pointer");
  FA_REQUIRE(T >= 0 && H_Q > 0 && H_KV > 0, "T must be >= 0, head counts positive");
  if (!supported_d(D)) return fail(FA_ERR_UNSUPPORTED, "head dimension %d is not built (supported: 64, 128, 256)", D);
  FA_CUDA(fa::launch_qk_norm_split(qkv, q_weight, k_weight, q, k, v, T, H_Q, H_KV, D, eps,
                                   static_cast<cudaStream_t>(stream)));
  return FA_OK;
}

int fa_silu_mul_bf16(const void* gate_up, void* out, int64_t T, int I, void* stream) {
  FA_REQUIRE(gate_up && out, "null tensor pointer");
  FA_REQUIRE(T >= 0 && I > 0 && I % 8 == 0, "I must be a positive multiple of 8");
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != FA_OK) return rc;
  FA_CUDA(fa::launch_silu_mul(gate_up, out, T, I, di.sm_count, static_cast<cudaStream_t>(stream)));
  return FA_OK;
}

int fa_half_to_bf16(const void* in, void* out, int64_t n, void* stream) {
  FA_REQUIRE(in && out, "null tensor pointer");
  FA_REQUIRE(n >= 0 && n % 8 == 0, "n must be a multiple of 8");
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != FA_OK) return rc;
  FA_CUDA(fa::launch_half_to_bf16(in, out, n, di.sm_count, static_cast<cudaStream_t>(stream)));
  return FA_OK;
}

// ---------------------------------------------------------------------------
// Peer-memory collectives (one process per GPU; buffers shared through CUDA IPC)
// ---------------------------------------------------------------------------
int fa_peer_alloc(size_t data_bytes, void** data, void** flags, void** state, void* data_handle, void* flags_handle) {
  FA_REQUIRE(data && flags && state && data_handle && flags_handle, "null pointer");
  FA_REQUIRE(data_bytes > 0 && data_bytes % 256 == 0, "data_bytes must be a positive multiple of 256");
  void *d = nullptr, *f = nullptr, *s = nullptr;
  FA_CUDA(cudaMalloc(&d, data_bytes));
  FA_CUDA(cudaMalloc(&f, fa::kPeerFlagBytes));
  FA_CUDA(cudaMalloc(&s, 256));
  FA_CUDA(cudaMemset(d, 0, data_bytes));
  FA_CUDA(cudaMemset(f, 0, fa::kPeerFlagBytes));
  FA_CUDA(cudaMemset(s, 0, 256));
  FA_CUDA(cudaDeviceSynchronize());
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are exchanged as 64 bytes");
  FA_CUDA(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(data_handle), d));
  FA_CUDA(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(flags_handle), f));
  *data = d; *flags = f; *state = s;
  return FA_OK;
}

int fa_peer_open(const void* handle, void** ptr) {
  FA_REQUIRE(handle && ptr, "null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  FA_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return FA_OK;
}

int fa_peer_close(void* ptr) {
  FA_REQUIRE(ptr, "null pointer");
  FA_CUDA(cudaIpcCloseMemHandle(ptr));
  return FA_OK;
}

int fa_peer_free(void* data, void* flags, void* state) {
  if (data) FA_CUDA(cudaFree(data));
  if (flags) FA_CUDA(cudaFree(flags));
  if (state) FA_CUDA(cudaFree(state));
  return FA_OK;
}

namespace {
// Bound of a flag wait in polls of >= 100 ns: tens of seconds by default, because ranks can be skewed
// by a whole CUDA-graph capture; tests shorten it.
unsigned int g_peer_max_polls = 1u << 26;

int fill_peer_args(void* const* data_ptrs, void* const* flag_ptrs, void* state, int rank, int world,
                   fa::PeerPointers* pp, fa::PeerState* st) {
  FA_REQUIRE(data_ptrs && flag_ptrs && state, "null pointer");
  FA_REQUIRE(world >= 1 && world <= fa::kPeerMaxWorld, "world must be between 1 and 8");
  FA_REQUIRE(rank >= 0 && rank < world, "rank out of range");
  memset(pp, 0, sizeof(*pp));
  for (int i = 0; i < world; ++i) {
    FA_REQUIRE(data_ptrs[i] && flag_ptrs[i], "null peer pointer");
    pp->data[i] = static_cast<uint8_t*>(data_ptrs[i]);
    pp->flags[i] = static_cast<uint32_t*>(flag_ptrs[i]);
  }
  uint8_t* s = static_cast<uint8_t*>(state);
  st->epoch = reinterpret_cast<uint32_t*>(s);
  st->ticket = reinterpret_cast<unsigned int*>(s + 64);
  st->status = reinterpret_cast<int32_t*>(s + 128);
  st->max_polls = g_peer_max_polls;
  return FA_OK;
}
}  // namespace

int fa_peer_allreduce_sum_bf16(void* const* data_ptrs, void* const* flag_ptrs, void* state, int rank, int world,
                               int64_t offset_bytes, int64_t n_elems, void* stream) {
  fa::PeerPointers pp;
  fa::PeerState st;
  int rc = fill_peer_args(data_ptrs, flag_ptrs, state, rank, world, &pp, &st);
  if (rc != FA_OK) return rc;
  FA_REQUIRE(offset_bytes >= 0 && offset_bytes % 16 == 0, "offset_bytes must be a non-negative multiple of 16");
  FA_REQUIRE(n_elems > 0 && n_elems % (8 * world) == 0, "n_elems must be a positive multiple of 8 * world");
  const long long vec_per_slice = n_elems / 8 / world;
  const int ctas = (int)((vec_per_slice + 511) / 512);
  FA_CUDA(fa::launch_peer_allreduce_bf16(pp, st, rank, world, offset_bytes, n_elems, ctas,
                                         static_cast<cudaStream_t>(stream)));
  return FA_OK;
}

int fa_peer_allreduce_add_rmsnorm_bf16(void* const* data_ptrs, void* const* flag_ptrs, void* state, int rank, int world,
                                       int64_t part_offset_bytes, int64_t x_offset_bytes, int64_t h_offset_bytes,
                                       int64_t rows, int cols, const void* weight, float eps, void* stream) {
  fa::PeerPointers pp;
  fa::PeerState st;
  int rc = fill_peer_args(data_ptrs, flag_ptrs, state, rank, world, &pp, &st);
  if (rc != FA_OK) return rc;
  FA_REQUIRE(weight, "null weight pointer");
  FA_REQUIRE(part_offset_bytes >= 0 && x_offset_bytes >= 0 && h_offset_bytes >= 0 && part_offset_bytes % 16 == 0 &&
                 x_offset_bytes % 16 == 0 && h_offset_bytes % 16 == 0,
             "region offsets must be non-negative multiples of 16");
  FA_REQUIRE(rows > 0 && rows % world == 0 && rows <= (1 << 24), "rows must be a positive multiple of world");
  FA_REQUIRE(cols > 0 && cols % 8 == 0 && cols <= 16384, "cols must be a multiple of 8, at most 16384");
  const int64_t bytes = rows * (int64_t)cols * 2;
  auto apart = [bytes](int64_t a, int64_t b) { return a + bytes <= b || b + bytes <= a; };
  FA_REQUIRE(apart(part_offset_bytes, x_offset_bytes) && apart(part_offset_bytes, h_offset_bytes) &&
                 apart(x_offset_bytes, h_offset_bytes),
             "the three regions must not overlap");
  FA_CUDA(fa::launch_peer_allreduce_add_rmsnorm(pp, st, rank, world, part_offset_bytes, x_offset_bytes,
                                                h_offset_bytes, (int)rows, cols, weight, eps,
                                                static_cast<cudaStream_t>(stream)));
  return FA_OK;
}

int fa_peer_allgather(void* const* data_ptrs, void* const* flag_ptrs, void* state, int rank, int world, const void* src,
                      int64_t offset_bytes, int64_t chunk_bytes, void* stream) {
  fa::PeerPointers pp;
  fa::PeerState st;
  int rc = fill_peer_args(data_ptrs, flag_ptrs, state, rank, world, &pp, &st);
  if (rc != FA_OK) return rc;
  FA_REQUIRE(src, "null source pointer");
  FA_REQUIRE(offset_bytes >= 0 && offset_bytes % 4 == 0, "offset_bytes must be a non-negative multiple of 4");
  FA_REQUIRE(chunk_bytes > 0 && chunk_bytes % 4 == 0, "chunk_bytes must be a positive multiple of 4");
  FA_CUDA(fa::launch_peer_allgather(pp, st, rank, world, src, offset_bytes, chunk_bytes,
                                    static_cast<cudaStream_t>(stream)));
  return FA_OK;
}

int fa_peer_reset(void* flags, void* state, void* stream) {
  FA_REQUIRE(flags && state, "null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  FA_CUDA(cudaMemsetAsync(flags, 0, fa::kPeerFlagBytes, s));
  FA_CUDA(cudaMemsetAsync(state, 0, 256, s));
  FA_CUDA(cudaStreamSynchronize(s));
  return FA_OK;
}

int fa_peer_set_max_polls(unsigned int max_polls) {
  FA_REQUIRE(max_polls > 0, "max_polls must be positive");
  g_peer_max_polls = max_polls;
  return FA_OK;
}

int fa_peer_status(const void* state, void* stream, int* host_status_out) {
  FA_REQUIRE(state && host_status_out, "null pointer");
  int32_t v = 0;
  FA_CUDA(cudaMemcpyAsync(&v, static_cast<const uint8_t*>(state) + 128, 4, cudaMemcpyDeviceToHost,
                          static_cast<cudaStream_t>(stream)));
  FA_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  *host_status_out = v;
  if (v != 0) return fail(FA_ERR_DEVICE_STATUS, "a peer collective gave up waiting for another rank (status 0x%x)", v);
  return FA_OK;
}

}  // extern "C"
