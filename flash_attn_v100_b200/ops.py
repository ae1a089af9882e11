"""Operator API of the reference's extension module, served by the sm_100a library.

Function names, positional signatures, tensor layouts, checks (-> RuntimeError)
and return conventions follow the reference's pybind module (flash_attn.cpp:224-255
and the wrappers in flash_attn_kernel.cu / continuous_batching_kernel.cu cited per
function).  PyTorch is used for device memory and streams only; all computation
happens in `libfa_b200.so` behind the C ABI of include/fa_b200.h.

Difference from the reference that a caller can observe: launches go to PyTorch's
current stream of the tensors' device (the reference's non-`_stream` wrappers use the
legacy default stream, e.g. flash_attn_kernel.cu:3567), so calls are ordered with
surrounding PyTorch work and can be captured in CUDA graphs.
"""
from __future__ import annotations

import contextlib
import ctypes
import threading
from typing import Dict, Tuple

import torch

from . import _lib

PAGE_BLOCK_SIZE = 16  # flash_attn_kernel.cu:3389
MAX_D_LARGE = 256     # flash_attn_kernel.cu:36
SUPPORTED_D = (64, 128, 256)

# Element type of q / k / v / caches that the wrappers below accept: float16, as in the reference, except inside
# the bfloat16 twins at the end of this file (same checks and launches, the library's *_bf16 entry points).
_elem_state = threading.local()


def _elem():
    return getattr(_elem_state, "dtype", torch.float16)


def _elem_name():
    return "bfloat16" if _elem() == torch.bfloat16 else "float16"


def _entry(lib, f16_name):
    """The C entry point for the current element type: fa_x_f16 or its twin fa_x_bf16."""
    return getattr(lib, f16_name[:-3] + "bf16") if _elem() == torch.bfloat16 else getattr(lib, f16_name)


@contextlib.contextmanager
def _bf16_elements():
    prev = _elem()
    _elem_state.dtype = torch.bfloat16
    try:
        yield
    finally:
        _elem_state.dtype = prev


_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}
_retired_workspaces: list = []


def _chk(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_input(t, name):
    # CHECK_INPUT (flash_attn_kernel.cu:15-17)
    _chk(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _chk(t.is_cuda, f"{name} must be a CUDA tensor")
    _chk(t.is_contiguous(), f"{name} must be a contiguous tensor")


def _check_dim(t, n, name):
    _chk(t.dim() == n, f"{name} must be a {n}D tensor")


def _same_device(a, b, an, bn):
    _chk(a.device == b.device, f"{an} and {bn} must be on the same device")


def _same_dtype(a, b, an, bn):
    _chk(a.dtype == b.dtype, f"{an} and {bn} must have the same dtype")


def _check_cache_len(cache_len, seq_len):
    # check_cache_len (flash_attn_kernel.cu:221-224)
    _chk(cache_len >= 0, "cache_len must be non-negative")
    _chk(cache_len < seq_len, "cache_len must be less than sequence length")


def _check_decode_gqa_shapes(q, k, v):
    # check_decode_gqa_input_shapes (flash_attn_kernel.cu:177-193)
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_dim(t, 4, n)
    _same_device(q, k, "q", "k"); _same_device(q, v, "q", "v")
    _same_dtype(q, k, "q", "k"); _same_dtype(q, v, "q", "v")
    _chk(q.size(0) == k.size(0) == v.size(0), "q, k, v batch size must match")
    _chk(k.size(1) == v.size(1), "k and v must have the same number of heads")
    _chk(k.size(2) == v.size(2), "k and v sequence length must match")
    _chk(q.size(3) == k.size(3) == v.size(3), "q, k, v head dimension must match")


def _check_prefill_gqa_shapes(q, k, v):
    # check_prefill_gqa_input_shapes (flash_attn_kernel.cu:160-175)
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_dim(t, 4, n)
    _same_device(q, k, "q", "k"); _same_device(q, v, "q", "v")
    _same_dtype(q, k, "q", "k"); _same_dtype(q, v, "q", "v")
    _chk(q.size(0) == k.size(0) == v.size(0), "q, k, v batch size must match")
    _chk(k.size(1) == v.size(1), "k and v must have the same number of heads")
    _chk(q.size(2) == k.size(2) == v.size(2), "q, k, v sequence length must match")
    _chk(q.size(3) == k.size(3) == v.size(3), "q, k, v head dimension must match")


def _check_gqa_heads(H_Q, H_KV):
    _chk(H_Q >= H_KV, "H_Q must be >= H_KV")
    _chk(H_Q % H_KV == 0, "H_Q must be divisible by H_KV")


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream_ptr(device, stream_int=None):
    if stream_int is None:
        stream_int = torch.cuda.current_stream(device).cuda_stream
    return int(stream_int)


def _workspace(device, stream_int, B, H_Q, H_KV, D):
    """Scratch for split-KV decode, owned by the library shim: one buffer per
    (device, stream), grown on demand.  Calls on one stream are ordered, so they
    may share it.

    A buffer that has been handed to a launch is never freed: a captured CUDA graph
    keeps its address in its kernel parameters, and a kernel on a stream that the
    caching allocator does not track (the `_stream` variants) may still be using it
    when a larger one replaces it.  Replaced buffers are therefore parked in
    `_retired_workspaces` for the life of the process (a few MiB each, and growth is
    rare: the size is dominated by the per-CTA partial results, which do not depend on
    the batch size)."""
    lib = _lib.load()
    _chk(8 <= D <= 256 and D % 8 == 0,
         f"head dimension {D} is not built (decode serves multiples of 8 up to 256)")
    need = int(lib.fa_decode_workspace_bytes(B, H_Q, H_KV, D))
    _chk(need > 0, f"unsupported decode configuration B={B} H_Q={H_Q} H_KV={H_KV} D={D}")
    dev_index = device.index if device.index is not None else torch.cuda.current_device()
    key = (dev_index, stream_int)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        if ws is not None:
            _retired_workspaces.append(ws)
        ws = torch.empty(max(2 * need, 8 << 20), dtype=torch.uint8, device=device)
        current = torch.cuda.current_stream(device)
        if int(current.cuda_stream) != int(stream_int):
            # the block may have been released by work still queued on torch's stream: the foreign
            # stream must not touch it before that work has finished
            ev = torch.cuda.Event()
            ev.record(current)
            torch.cuda.ExternalStream(stream_int, device=device).wait_event(ev)
        _lib.check(lib.fa_decode_workspace_init(_ptr(ws), ws.numel(), ctypes.c_void_p(stream_int)))
        _workspaces[key] = ws
    return ws


def check_async_errors(device=None) -> None:
    """Synchronise and raise RuntimeError if a decode kernel on `device` recorded a
    bounded-wait timeout or an out-of-pool page id since its workspace was created."""
    lib = _lib.load()
    for (dev, stream_int), ws in list(_workspaces.items()):
        if device is not None and torch.device(device).index not in (None, dev):
            continue
        with torch.cuda.device(dev):
            st = ctypes.c_int(0)
            _lib.check(lib.fa_decode_status(_ptr(ws), ctypes.c_void_p(stream_int), ctypes.byref(st)))


def set_prefill_impl(impl: int = 0) -> None:
    """0 = automatic, 1 = mma.sync kernel, 2 = tcgen05 kernel (tests and measurements)."""
    _lib.check(_lib.load().fa_prefill_set_impl(int(impl)))


def check_prefill_errors(device=None, clear: bool = True) -> None:
    """Synchronise and raise RuntimeError if a prefill kernel on `device` recorded a bounded-wait timeout."""
    lib = _lib.load()
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    with torch.cuda.device(dev):
        st = ctypes.c_int(0)
        s = torch.cuda.current_stream(dev).cuda_stream
        _lib.check(lib.fa_prefill_status(ctypes.c_void_p(s), ctypes.byref(st), 1 if clear else 0))


def set_decode_tuning(warps: int = 0, stages: int = 0, ctas_per_sm: int = 0) -> None:
    _lib.check(_lib.load().fa_decode_set_tuning(int(warps), int(stages), int(ctas_per_sm)))


# --------------------------------------------------------------------------
# decode
# --------------------------------------------------------------------------
def _decode_gqa(out, q, k, v, causal, cache_len, stream_int=None):
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_input(t, n)
    _check_decode_gqa_shapes(q, k, v)
    if out is not None:
        # check_decode_gqa_output_tensor (flash_attn_kernel.cu:226-239)
        _check_input(out, "out")
        _check_dim(out, 4, "out")
        _same_device(out, q, "out", "q"); _same_dtype(out, q, "out", "q")
        _chk(out.size(0) == q.size(0), "out batch size must match q")
        _chk(out.size(1) == q.size(1), "out head count must match q")
        _chk(out.size(2) == 1, "out sequence length must be 1 for decode mode")
        _chk(out.size(3) == q.size(3), "out head dimension must match q")
    _chk(q.dtype == _elem(), f"q, k, v must be {_elem_name()}")
    _chk(q.size(2) == 1, "q sequence length must be 1 for decode mode")
    B, H_Q, _, D = q.shape
    H_KV, N = k.size(1), k.size(2)
    _check_gqa_heads(H_Q, H_KV)
    _chk(D <= MAX_D_LARGE, "D must be less than or equal to MAX_D_LARGE(256)")
    cache_len = int(cache_len)
    _check_cache_len(cache_len, N)
    lib = _lib.load()
    with torch.cuda.device(q.device):
        if out is None:
            out = torch.empty((B, H_Q, 1, D), dtype=q.dtype, device=q.device)
        s = _stream_ptr(q.device, stream_int)
        ws = _workspace(q.device, s, B, H_Q, H_KV, D)
        _lib.check(_entry(lib, "fa_decode_gqa_f16")(_ptr(q), _ptr(k), _ptr(v), _ptr(out), B, H_Q, H_KV, N, D,
                                         1 if causal else 0, cache_len, _ptr(ws), ws.numel(), ctypes.c_void_p(s)))
    return out


def forward_decode_gqa_fp16(q, k, v, causal, cache_len):
    """flash_attn_forward_decode_gqa_fp16 (flash_attn_kernel.cu:1800-1833).
    q [B,H_Q,1,D], k/v [B,H_KV,N,D] fp16 -> new [B,H_Q,1,D]."""
    return _decode_gqa(None, q, k, v, causal, cache_len)


def forward_decode_gqa_fp16_out(out, q, k, v, causal, cache_len):
    """flash_attn_forward_decode_gqa_fp16_out (flash_attn_kernel.cu:1835-1861):
    writes into and returns the tensor passed as `out`."""
    return _decode_gqa(out, q, k, v, causal, cache_len)


def forward_decode_gqa_fp16_stream(q, k, v, causal, cache_len, stream_int):
    """flash_attn_forward_decode_gqa_fp16_stream (flash_attn_kernel.cu:3639-3675):
    `stream_int` is a raw cudaStream_t (torch.cuda.Stream().cuda_stream)."""
    return _decode_gqa(None, q, k, v, causal, cache_len, int(stream_int))


def forward_decode_fp16(q, k, v, causal, cache_len):
    """flash_attn_forward_decode_fp16 (flash_attn_kernel.cu:1863-1913): MHA decode,
    head counts must match (check_decode_mha_input_shapes, :143-158)."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_input(t, n)
        _check_dim(t, 4, n)
    _chk(q.size(1) == k.size(1) == v.size(1), "q, k, v head count must match")
    return _decode_gqa(None, q, k, v, causal, cache_len)


def forward_decode_sliding_window_gqa(q, k, v, causal, cache_len, window_size, sink_size):
    """flash_attn_forward_decode_sliding_window_gqa (flash_attn_kernel.cu:4484-4535).
    q [B,H_Q,1,D], k/v [B,H_KV,N,D] fp16 -> new [B,H_Q,1,D].  Key j is attended when
    j < sink_size or window_start <= j <= cache_len, window_start = max(0, min(cache_len+1, N) - window_size)
    (:4386-4387, :4410-4412).  `causal` has no effect, as in the reference; like the reference, no
    bound is checked on cache_len, window_size or sink_size."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_input(t, n)
    _chk(q.dtype == torch.float16, "q must be float16")
    _chk(k.dtype == torch.float16 and v.dtype == torch.float16, "k and v must be float16")
    _chk(q.dim() == 4 and k.dim() == 4 and v.dim() == 4, "q, k, v must be 4D tensors")
    _chk(q.size(2) == 1, "q sequence length must be 1 for decode mode")
    _same_device(q, k, "q", "k"); _same_device(q, v, "q", "v")
    _chk(k.shape == v.shape, "k and v must have the same shape")
    _chk(k.size(0) == q.size(0) and k.size(3) == q.size(3), "k must match q in batch size and head dimension")
    B, H_Q, _, D = q.shape
    H_KV, N = k.size(1), k.size(2)
    _check_gqa_heads(H_Q, H_KV)
    _chk(D <= MAX_D_LARGE, "D must be <= MAX_D_LARGE(256)")
    lib = _lib.load()
    with torch.cuda.device(q.device):
        out = torch.empty((B, H_Q, 1, D), dtype=q.dtype, device=q.device)
        s = _stream_ptr(q.device)
        ws = _workspace(q.device, s, B, H_Q, H_KV, D)
        _lib.check(lib.fa_decode_sliding_window_gqa_f16(
            _ptr(q), _ptr(k), _ptr(v), _ptr(out), B, H_Q, H_KV, N, D, int(cache_len), int(window_size),
            int(sink_size), _ptr(ws), ws.numel(), ctypes.c_void_p(s)))
    return out


def forward_decode_int8_kv_cache_gqa(q, k_int8, v_int8, k_scale, v_scale, cache_len):
    """flash_attn_forward_decode_int8_kv_cache_gqa (flash_attn_kernel.cu:4164-4221).
    q [B,H_Q,1,D] fp16; k_int8/v_int8 [B,H_KV,N,D] int8; k_scale/v_scale [B,H_KV,N] fp16 (one scale per
    cached token) -> new [B,H_Q,1,D] fp16.  Elements are dequantised as fp16(float(int8) * float(scale))
    (:4083-4086) and keys j <= cache_len are attended (:4094-4098)."""
    for t, n in ((q, "q"), (k_int8, "k_int8"), (v_int8, "v_int8"), (k_scale, "k_scale"), (v_scale, "v_scale")):
        _check_input(t, n)
    _chk(q.dtype == torch.float16, "q must be float16")
    _chk(k_int8.dtype == torch.int8, "k_int8 must be int8")
    _chk(v_int8.dtype == torch.int8, "v_int8 must be int8")
    _chk(k_scale.dtype == torch.float16, "k_scale must be float16")
    _chk(v_scale.dtype == torch.float16, "v_scale must be float16")
    _chk(q.dim() == 4 and k_int8.dim() == 4 and v_int8.dim() == 4, "q, k_int8, v_int8 must be 4D tensors")
    _chk(k_scale.dim() == 3 and v_scale.dim() == 3, "k_scale and v_scale must be 3D tensors")
    _chk(q.size(2) == 1, "q sequence length must be 1 for decode mode")
    for t, n in ((k_int8, "k_int8"), (v_int8, "v_int8"), (k_scale, "k_scale"), (v_scale, "v_scale")):
        _same_device(q, t, "q", n)
    B, H_Q, _, D = q.shape
    H_KV, N = k_int8.size(1), k_int8.size(2)
    _check_gqa_heads(H_Q, H_KV)
    _chk(D <= MAX_D_LARGE, "D must be <= MAX_D_LARGE(256)")
    _chk(k_int8.size(3) == D, "k_int8 last dim must match D")
    _chk(v_int8.size(3) == D, "v_int8 last dim must match D")
    _chk(k_int8.size(0) == B and v_int8.shape == k_int8.shape, "k_int8 and v_int8 must be [B, H_KV, N, D]")
    _chk(k_scale.size(2) == N, "k_scale size mismatch")
    _chk(v_scale.size(2) == N, "v_scale size mismatch")
    _chk(tuple(k_scale.shape) == (B, H_KV, N) and tuple(v_scale.shape) == (B, H_KV, N),
         "k_scale and v_scale must be [B, H_KV, N]")
    lib = _lib.load()
    with torch.cuda.device(q.device):
        out = torch.empty((B, H_Q, 1, D), dtype=q.dtype, device=q.device)
        s = _stream_ptr(q.device)
        ws = _workspace(q.device, s, B, H_Q, H_KV, D)
        _lib.check(lib.fa_decode_int8_kv_cache_gqa(
            _ptr(q), _ptr(k_int8), _ptr(v_int8), _ptr(k_scale), _ptr(v_scale), _ptr(out), B, H_Q, H_KV, N, D,
            int(cache_len), _ptr(ws), ws.numel(), ctypes.c_void_p(s)))
    return out


def forward_continuous_batching_fp16(q, k, v, cache_lens, causal):
    """flash_attn_forward_continuous_batching_fp16 (continuous_batching_kernel.cu:338-406).
    q [B,H_Q,1,D], k/v [B,H_KV,max_N,D] fp16, cache_lens [B] int32; sequence b attends
    keys [0, min(cache_lens[b]+1, max_N)).  `causal` has no effect (as in the reference)."""
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (cache_lens, "cache_lens")):
        _check_input(t, n)
    _chk(q.dtype == torch.float16, "q must be float16")
    _chk(k.dtype == torch.float16 and v.dtype == torch.float16, "k and v must be float16")
    _chk(q.dim() == 4 and k.dim() == 4 and v.dim() == 4, "q, k, v must be 4D tensors")
    _chk(q.size(2) == 1, "q sequence length must be 1 for decode mode")
    _chk(cache_lens.dim() == 1, "cache_lens must be 1D tensor")
    _chk(cache_lens.size(0) == q.size(0), "cache_lens size must match batch size")
    # the reference reads cache_lens through data_ptr<int>() (:394); other dtypes would be misread
    _chk(cache_lens.dtype == torch.int32, "cache_lens must be int32")
    _same_device(q, k, "q", "k"); _same_device(q, v, "q", "v"); _same_device(q, cache_lens, "q", "cache_lens")
    _chk(k.shape == v.shape, "k and v must have the same shape")
    _chk(k.size(0) == q.size(0) and k.size(3) == q.size(3), "k must match q in batch size and head dimension")
    B, H_Q, _, D = q.shape
    H_KV, max_N = k.size(1), k.size(2)
    _check_gqa_heads(H_Q, H_KV)
    _chk(D <= MAX_D_LARGE, "D must be <= MAX_D_CB_LARGE(256)")
    lib = _lib.load()
    with torch.cuda.device(q.device):
        out = torch.empty((B, H_Q, 1, D), dtype=q.dtype, device=q.device)
        s = _stream_ptr(q.device)
        ws = _workspace(q.device, s, B, H_Q, H_KV, D)
        _lib.check(lib.fa_decode_varlen_f16(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(cache_lens), B, H_Q, H_KV,
                                            max_N, D, 1 if causal else 0, _ptr(ws), ws.numel(), ctypes.c_void_p(s)))
    return out


def forward_paged_decode_gqa_fp16(q, k_cache, v_cache, block_table, seq_lens, max_num_blocks, out_dtype=None):
    """flash_attn_forward_paged_decode_gqa_fp16 (flash_attn_kernel.cu:3516-3584).
    q [B,H_Q,1,D]; k_cache/v_cache [pages,H_KV,16,D] fp16; block_table [B,*] int32 with
    row stride `max_num_blocks` (:3438); seq_lens [B] int32.  seq_len 0 gives zeros.
    `out_dtype=torch.bfloat16` (an addition) returns the result rounded to bfloat16 instead of fp16."""
    _chk(out_dtype in (None, torch.float16, torch.bfloat16), "out_dtype must be float16 or bfloat16")
    bf16_out = out_dtype == torch.bfloat16 and _elem() == torch.float16
    for t, n in ((q, "q"), (k_cache, "k_cache"), (v_cache, "v_cache"), (block_table, "block_table"),
                 (seq_lens, "seq_lens")):
        _check_input(t, n)
    _check_dim(q, 4, "q"); _check_dim(k_cache, 4, "k_cache"); _check_dim(v_cache, 4, "v_cache")
    _check_dim(block_table, 2, "block_table"); _check_dim(seq_lens, 1, "seq_lens")
    for t, n in ((k_cache, "k_cache"), (v_cache, "v_cache"), (block_table, "block_table"), (seq_lens, "seq_lens")):
        _same_device(q, t, "q", n)
    _chk(q.dtype == _elem(), f"q must be {_elem_name()}")
    _chk(k_cache.dtype == _elem(), f"k_cache must be {_elem_name()}")
    _chk(v_cache.dtype == _elem(), f"v_cache must be {_elem_name()}")
    _chk(block_table.dtype == torch.int32, "block_table must be int32")
    _chk(seq_lens.dtype == torch.int32, "seq_lens must be int32")
    _chk(q.size(2) == 1, "q sequence length must be 1 for decode mode")
    B, H_Q, _, D = q.shape
    H_KV = k_cache.size(1)
    _check_gqa_heads(H_Q, H_KV)
    _chk(D <= MAX_D_LARGE, "D must be <= MAX_D_LARGE(256)")
    _chk(k_cache.size(2) == PAGE_BLOCK_SIZE, "k_cache block size mismatch")
    _chk(v_cache.size(2) == PAGE_BLOCK_SIZE, "v_cache block size mismatch")
    _chk(block_table.size(0) == B, "block_table batch size must match q")
    _chk(seq_lens.size(0) == B, "seq_lens batch size must match q")
    _chk(k_cache.shape == v_cache.shape, "k_cache and v_cache must have the same shape")
    _chk(k_cache.size(3) == D, "k_cache head dimension must match q")
    max_num_blocks = int(max_num_blocks)
    _chk(max_num_blocks > 0, "max_num_blocks must be positive")
    _chk((B - 1) * max_num_blocks + min(max_num_blocks, block_table.size(1)) <= block_table.numel(),
         "max_num_blocks (row stride) is larger than block_table allows")
    lib = _lib.load()
    with torch.cuda.device(q.device):
        out = torch.empty((B, H_Q, 1, D), dtype=torch.bfloat16 if bf16_out else q.dtype, device=q.device)
        s = _stream_ptr(q.device)
        ws = _workspace(q.device, s, B, H_Q, H_KV, D)
        max_len = min(max_num_blocks, block_table.size(1)) * PAGE_BLOCK_SIZE
        entry = lib.fa_paged_decode_gqa_f16_out_bf16 if bf16_out else _entry(lib, "fa_paged_decode_gqa_f16")
        _lib.check(entry(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table),
                                               _ptr(seq_lens), B, H_Q, H_KV, D, k_cache.size(0), max_num_blocks,
                                               max_len, _ptr(ws), ws.numel(), ctypes.c_void_p(s)))
    return out


def forward_decode_int8_gqa(q, k, v, q_scale, k_scale, cache_len, return_scores=False):
    """flash_attn_forward_decode_int8_gqa (flash_attn_kernel.cu:2941-3003).
    q [B,H_Q,1,D], k/v [B,H_KV,N,D] fp16, q_scale [B,H_Q] fp32, k_scale [B,H_KV,N] fp32
    (per cached token).  With `return_scores=True` (an addition) also returns the raw
    int32 QK^T accumulators [B,H_Q,N] (entries past cache_len are zero)."""
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (q_scale, "q_scale"), (k_scale, "k_scale")):
        _check_input(t, n)
    _check_decode_gqa_shapes(q, k, v)
    _chk(q.dtype == torch.float16, "q, k, v must be float16")
    _chk(q_scale.dtype == torch.float32, "q_scale must be float32")
    _chk(k_scale.dtype == torch.float32, "k_scale must be float32")
    _chk(q.size(2) == 1, "q sequence length must be 1 for decode mode")
    B, H_Q, _, D = q.shape
    H_KV, N = k.size(1), k.size(2)
    _check_gqa_heads(H_Q, H_KV)
    _chk(D <= MAX_D_LARGE, "D must be <= MAX_D_LARGE(256)")
    _chk(q_scale.dim() == 2 and q_scale.size(0) == B and q_scale.size(1) == H_Q, "q_scale must be [B, H_Q]")
    _chk(k_scale.dim() == 3 and k_scale.size(0) == B and k_scale.size(1) == H_KV and k_scale.size(2) == N,
         "k_scale must be [B, H_KV, N]")
    _same_device(q, q_scale, "q", "q_scale"); _same_device(q, k_scale, "q", "k_scale")
    cache_len = int(cache_len)
    _check_cache_len(cache_len, N)
    lib = _lib.load()
    with torch.cuda.device(q.device):
        out = torch.empty((B, H_Q, 1, D), dtype=q.dtype, device=q.device)
        scores = torch.zeros((B, H_Q, N), dtype=torch.int32, device=q.device) if return_scores else None
        s = _stream_ptr(q.device)
        ws = _workspace(q.device, s, B, H_Q, H_KV, D)
        _lib.check(lib.fa_decode_int8_gqa(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(q_scale), _ptr(k_scale),
                                          B, H_Q, H_KV, N, D, cache_len,
                                          _ptr(scores) if scores is not None else None,
                                          _ptr(ws), ws.numel(), ctypes.c_void_p(s)))
    return (out, scores) if return_scores else out


# --------------------------------------------------------------------------
# prefill
# --------------------------------------------------------------------------
def _prefill_dense(out, q, k, v, causal):
    B, H_Q, N, D = q.shape
    H_KV = k.size(1)
    lib = _lib.load()
    with torch.cuda.device(q.device):
        if out is None:
            out = torch.empty((B, H_Q, N, D), dtype=q.dtype, device=q.device)
        s = _stream_ptr(q.device)
        _lib.check(_entry(lib, "fa_prefill_dense_f16")(_ptr(q), _ptr(k), _ptr(v), _ptr(out), B, H_Q, H_KV, N, D,
                                            1 if causal else 0, ctypes.c_void_p(s)))
    return out


def forward_fp16(q, k, v, causal):
    """flash_attn_forward_fp16 (flash_attn_kernel.cu:1915-1962): dense MHA,
    q/k/v [B,H,N,D] fp16 of identical shape (check_mha_input_shapes, :127-141)."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_input(t, n)
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_dim(t, 4, n)
    _same_device(q, k, "q", "k"); _same_device(q, v, "q", "v")
    _same_dtype(q, k, "q", "k"); _same_dtype(q, v, "q", "v")
    _chk(q.shape == k.shape, "q and k must have the same shape")
    _chk(q.shape == v.shape, "q and v must have the same shape")
    _chk(q.dtype == _elem(), f"q, k, v must be {_elem_name()}")
    _chk(q.size(3) <= MAX_D_LARGE, "D must be less than or equal to MAX_D_LARGE(256)")
    return _prefill_dense(None, q, k, v, causal)


def _prefill_gqa(out, q, k, v, causal):
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_input(t, n)
    _check_prefill_gqa_shapes(q, k, v)
    if out is not None:
        # check_prefill_gqa_output_tensor (flash_attn_kernel.cu:241-250)
        _check_input(out, "out")
        _check_dim(out, 4, "out")
        _same_device(out, q, "out", "q"); _same_dtype(out, q, "out", "q")
        _chk(out.shape == q.shape, "out shape must match q shape for prefill mode")
    _chk(q.dtype == _elem(), f"q, k, v must be {_elem_name()}")
    _check_gqa_heads(q.size(1), k.size(1))
    _chk(q.size(3) <= MAX_D_LARGE, "D must be <= MAX_D_LARGE(256)")
    return _prefill_dense(out, q, k, v, causal)


def forward_prefill_gqa_fp16(q, k, v, causal):
    """flash_attn_forward_prefill_gqa_fp16 (flash_attn_kernel.cu:2740-2769)."""
    return _prefill_gqa(None, q, k, v, causal)


def forward_prefill_gqa_fp16_out(out, q, k, v, causal):
    """flash_attn_forward_prefill_gqa_fp16_out (flash_attn_kernel.cu:2771-2794)."""
    return _prefill_gqa(out, q, k, v, causal)


def _varlen(q, k, v, cu_seqlens, max_seqlen, causal, stream_int=None, bf16_out=False):
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (cu_seqlens, "cu_seqlens")):
        _check_input(t, n)
    # check_varlen_prefill_input_shapes (flash_attn_kernel.cu:195-219); the head-count
    # equality of the reference (:217) is relaxed to GQA: H_Q % H_KV == 0.
    _check_dim(q, 3, "q"); _check_dim(k, 3, "k"); _check_dim(v, 3, "v"); _check_dim(cu_seqlens, 1, "cu_seqlens")
    _same_device(q, k, "q", "k"); _same_device(q, v, "q", "v"); _same_device(q, cu_seqlens, "q", "cu_seqlens")
    _same_dtype(q, k, "q", "k"); _same_dtype(q, v, "q", "v")
    _chk(k.size(0) == q.size(0) and v.size(0) == q.size(0), "k and v total length must match q")
    _chk(k.size(1) == v.size(1), "k and v must have the same number of heads")
    _chk(k.size(2) == q.size(2) and v.size(2) == q.size(2), "k and v head dimension must match q")
    _chk(q.dtype == _elem(), f"q, k, v must be {_elem_name()}")
    _chk(cu_seqlens.dtype == torch.int32, "cu_seqlens must be int32")
    bf16_out = bf16_out and _elem() == torch.float16
    total, H_Q, D = q.shape
    H_KV = k.size(1)
    _check_gqa_heads(H_Q, H_KV)
    batch = cu_seqlens.size(0) - 1
    _chk(D <= MAX_D_LARGE, "D must be <= MAX_D_LARGE(256)")
    max_seqlen = int(max_seqlen)
    _chk(max_seqlen > 0, "max_seqlen must be positive")
    _chk(batch > 0, "cu_seqlens must contain at least one sequence")
    lib = _lib.load()
    with torch.cuda.device(q.device):
        # rows outside every sequence stay zero, as in the reference (:3373)
        out = torch.zeros(q.shape, dtype=torch.bfloat16 if bf16_out else q.dtype, device=q.device)
        s = _stream_ptr(q.device, stream_int)
        if stream_int is not None and stream_int != torch.cuda.current_stream(q.device).cuda_stream:
            # zeros_like ran on the current stream; order the foreign stream after it
            ev = torch.cuda.Event()
            ev.record()
            torch.cuda.ExternalStream(stream_int, device=q.device).wait_event(ev)
        entry = lib.fa_prefill_varlen_f16_out_bf16 if bf16_out else _entry(lib, "fa_prefill_varlen_f16")
        _lib.check(entry(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(cu_seqlens), batch, total,
                         H_Q, H_KV, D, max_seqlen, 1 if causal else 0, ctypes.c_void_p(s)))
    return out


def forward_varlen_prefill_fp16(q, k, v, cu_seqlens, max_seqlen, causal, out_dtype=None):
    """flash_attn_forward_varlen_prefill_fp16 (flash_attn_kernel.cu:3354-3387).
    q [total,H_Q,D], k/v [total,H_KV,D] fp16 packed; cu_seqlens [batch+1] int32.
    `out_dtype=torch.bfloat16` (an addition) returns the result rounded to bfloat16 instead of fp16."""
    _chk(out_dtype in (None, torch.float16, torch.bfloat16), "out_dtype must be float16 or bfloat16")
    return _varlen(q, k, v, cu_seqlens, max_seqlen, causal, bf16_out=out_dtype == torch.bfloat16)


def forward_varlen_prefill_fp16_stream(q, k, v, cu_seqlens, max_seqlen, causal, stream_int):
    """flash_attn_forward_varlen_prefill_fp16_stream (flash_attn_kernel.cu:3677-3712)."""
    return _varlen(q, k, v, cu_seqlens, max_seqlen, causal, int(stream_int))


# --------------------------------------------------------------------------
# write side of the paged cache (an addition: the reference does this in Python)
# --------------------------------------------------------------------------
def rope_append_paged_fp16(q, k, v, cos, sin, k_cache, v_cache, block_table, positions, max_num_blocks,
                           cu_seqlens=None, return_k=False):
    """Rotary embedding of q and k plus the append of k / v into the paged cache, in one launch.

    Replaces the reference's `apply_rotary_emb` (flash_attn_llm/models/rope.py:302-348, half rotation,
    partial rotary when cos/sin are narrower than D) followed by its per-token cache copies
    (flash_attn_llm/kv_cache/manager.py:350-357, tensor_parallel.py:285-327).  Results are bit-identical
    to the reference's fp16 PyTorch expression.

    Decode step (cu_seqlens is None): q [B,H_Q,1,D], k/v [B,H_KV,1,D]; cos/sin [B,1,1,R] or [B,R] fp32 as
    `RotaryEmbedding.forward(1, position_ids)` returns them; positions [B] int32 = slot of the new token.
    Packed prompts: q [total,H_Q,D], k/v [total,H_KV,D], cos/sin [total,R], cu_seqlens [batch+1] int32;
    token j of sequence s is stored at slot positions[s] + j (positions None = 0).
    k_cache / v_cache [pages,H_KV,16,D] are updated in place (both None: rotation only);
    block_table [batch, *] int32 with row stride `max_num_blocks`.
    Returns q_rot (same shape as q), or (q_rot, k_rot) with return_k=True.
    """
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (cos, "cos"), (sin, "sin")):
        _check_input(t, n)
    _chk(q.dtype == _elem() and k.dtype == _elem() and v.dtype == _elem(), f"q, k, v must be {_elem_name()}")
    _chk(cos.dtype == torch.float32 and sin.dtype == torch.float32, "cos and sin must be float32")
    _chk(k.shape == v.shape, "k and v must have the same shape")
    packed = cu_seqlens is not None
    if packed:
        _check_dim(q, 3, "q"); _check_dim(k, 3, "k")
        T, H_Q, D = q.shape
        H_KV = k.size(1)
        _chk(k.size(0) == T and k.size(2) == D, "k must match q in tokens and head dimension")
        _check_input(cu_seqlens, "cu_seqlens")
        _chk(cu_seqlens.dtype == torch.int32 and cu_seqlens.dim() == 1, "cu_seqlens must be a 1D int32 tensor")
        batch = cu_seqlens.size(0) - 1
    else:
        _check_dim(q, 4, "q"); _check_dim(k, 4, "k")
        _chk(q.size(2) == 1 and k.size(2) == 1, "q and k sequence length must be 1 for a decode step")
        T, H_Q, _, D = q.shape
        H_KV = k.size(1)
        _chk(k.size(0) == T and k.size(3) == D, "k must match q in batch size and head dimension")
        batch = T
        _chk(positions is not None, "positions is required for a decode step")
    R = cos.shape[-1]
    _chk(cos.numel() == T * R and sin.shape == cos.shape, "cos and sin must hold one row of rot_dim values per token")
    _same_device(q, k, "q", "k"); _same_device(q, v, "q", "v")
    _same_device(q, cos, "q", "cos"); _same_device(q, sin, "q", "sin")
    has_cache = k_cache is not None
    _chk((k_cache is None) == (v_cache is None), "k_cache and v_cache must be given together")
    if has_cache:
        for t, n in ((k_cache, "k_cache"), (v_cache, "v_cache"), (block_table, "block_table")):
            _check_input(t, n)
            _same_device(q, t, "q", n)
        _chk(k_cache.dtype == _elem() and v_cache.dtype == _elem(), f"k_cache and v_cache must be {_elem_name()}")
        _chk(k_cache.dim() == 4 and k_cache.shape == v_cache.shape and k_cache.size(1) == H_KV and
             k_cache.size(2) == PAGE_BLOCK_SIZE and k_cache.size(3) == D, "cache must be [pages, H_KV, 16, D]")
        _chk(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.size(0) >= batch,
             "block_table must be int32 [batch, *]")
        # the kernel reads block_table[seq * stride + blk] for blk < stride: every such entry must exist
        max_num_blocks = int(max_num_blocks)
        _chk(max_num_blocks > 0, "max_num_blocks must be positive")
        _chk(batch * max_num_blocks <= block_table.numel(),
             "max_num_blocks (row stride) is larger than block_table allows")
    if positions is not None:
        _check_input(positions, "positions")
        _chk(positions.dtype == torch.int32 and positions.numel() == batch, "positions must be int32 [batch]")
    lib = _lib.load()
    with torch.cuda.device(q.device):
        q_out = torch.empty_like(q)
        k_out = torch.empty_like(k) if return_k else None
        s = _stream_ptr(q.device)
        _lib.check(_entry(lib, "fa_rope_append_paged_f16")(
            _ptr(q), _ptr(k), _ptr(v), _ptr(cos), _ptr(sin), _ptr(q_out), _ptr(k_out) if return_k else None,
            _ptr(k_cache) if has_cache else None, _ptr(v_cache) if has_cache else None,
            _ptr(block_table) if has_cache else None, _ptr(positions) if positions is not None else None,
            _ptr(cu_seqlens) if packed else None, T, batch, H_Q, H_KV, D, R,
            k_cache.size(0) if has_cache else 0, int(max_num_blocks) if has_cache else 0, ctypes.c_void_p(s)))
    return (q_out, k_out) if return_k else q_out


# --------------------------------------------------------------------------
# bfloat16 twins (additions: the reference's operators are fp16 only).  q / k / v, the caches and the result
# are bfloat16; everything else — shapes, checks, errors — is that of the fp16 function named in the body.
# --------------------------------------------------------------------------
def forward_decode_gqa_bf16(q, k, v, causal, cache_len):
    with _bf16_elements():
        return forward_decode_gqa_fp16(q, k, v, causal, cache_len)


def forward_paged_decode_gqa_bf16(q, k_cache, v_cache, block_table, seq_lens, max_num_blocks):
    with _bf16_elements():
        return forward_paged_decode_gqa_fp16(q, k_cache, v_cache, block_table, seq_lens, max_num_blocks)


def forward_prefill_gqa_bf16(q, k, v, causal):
    with _bf16_elements():
        return forward_prefill_gqa_fp16(q, k, v, causal)


def forward_varlen_prefill_bf16(q, k, v, cu_seqlens, max_seqlen, causal):
    with _bf16_elements():
        return forward_varlen_prefill_fp16(q, k, v, cu_seqlens, max_seqlen, causal)


def rope_append_paged_bf16(q, k, v, cos, sin, k_cache, v_cache, block_table, positions, max_num_blocks,
                           cu_seqlens=None, return_k=False):
    with _bf16_elements():
        return rope_append_paged_fp16(q, k, v, cos, sin, k_cache, v_cache, block_table, positions, max_num_blocks,
                                      cu_seqlens=cu_seqlens, return_k=return_k)


# --------------------------------------------------------------------------
# exports of the reference module that are outside the attention hot path
# --------------------------------------------------------------------------
_NOT_BUILT = [
    "forward", "forward_with_lse", "forward_fp16_with_lse", "backward", "async_h2d_transfer", "alloc_pinned_tensor",
    "pipeline_decode_step", "pipeline_decode_step_out", "speculative_verify",
    "token_eviction", "cross_gpu_allreduce_fp16", "scatter_heads", "gather_heads",
]


def _make_not_built(name):
    def fn(*args, **kwargs):
        raise NotImplementedError(
            f"flash_attn_v100.{name} is outside the attention hot path served by the sm_100a library")
    fn.__name__ = name
    return fn


for _n in _NOT_BUILT:
    globals()[_n] = _make_not_built(_n)


def forward_fp16_warp(q, k, v, causal):
    """flash_attn_forward_fp16_warp (flash_attn_kernel.cu:1440-1482): same math as forward_fp16."""
    return forward_fp16(q, k, v, causal)


def forward_fp16_wmma(q, k, v, causal):
    """flash_attn_forward_fp16_wmma (flash_attn_kernel.cu:2425-2468): same math as forward_fp16."""
    return forward_fp16(q, k, v, causal)


def forward_prefill_gqa_fp16_warp(q, k, v, causal):
    """flash_attn_forward_prefill_gqa_fp16_warp (flash_attn_kernel.cu:3586-3637)."""
    return forward_prefill_gqa_fp16(q, k, v, causal)


REFERENCE_EXPORTS = [
    "forward", "forward_fp16", "forward_with_lse", "forward_fp16_with_lse", "backward", "forward_fp16_warp",
    "forward_decode_fp16", "forward_decode_gqa_fp16", "forward_decode_gqa_fp16_out", "forward_fp16_wmma",
    "forward_prefill_gqa_fp16", "forward_prefill_gqa_fp16_out", "forward_prefill_gqa_fp16_warp",
    "forward_paged_decode_gqa_fp16", "forward_decode_int8_gqa", "forward_varlen_prefill_fp16",
    "forward_decode_gqa_fp16_stream", "forward_varlen_prefill_fp16_stream", "forward_continuous_batching_fp16",
    "async_h2d_transfer", "alloc_pinned_tensor", "pipeline_decode_step", "pipeline_decode_step_out",
    "speculative_verify", "forward_decode_int8_kv_cache_gqa", "token_eviction", "forward_decode_sliding_window_gqa",
    "cross_gpu_allreduce_fp16", "scatter_heads", "gather_heads",
]
