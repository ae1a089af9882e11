"""GPU: the paged decode entry point that carries its own scratch.

Some users of this library cannot hand it a workspace: their process has given all
device memory to a pool of its own, or they sit on a path where a cudaMalloc (and the
device-wide synchronisation it implies) is off limits.  For them
`fa_paged_decode_gqa_f16_static_scratch` keeps the split-KV scratch in an array inside
the library.  This test calls it through the C ABI twice in a row, on different inputs
(so anything the first call left in the shared array would show), and compares each
result with `fa_paged_decode_gqa_f16` given a caller-owned workspace and with the CPU
oracle.  Same kernels, same launch configuration: the outputs must agree to the
tolerance of the other decode tests (2e-3), and in practice bit for bit.  It also checks
the size limit, the order of argument validation, the shared array across calls of very
different shapes, and that the status word of the built-in scratch can be read and cleared.

The file sorts last so that a run that stops at the first failure has already run
every other test; it does not depend on them and passes in a fresh process too.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


def _make_case(seed, B, H_Q, H_KV, D, max_len, device, min_len=1):
    from flash_attn_v100_b200.synthetic import make_paged_tables
    t = make_paged_tables(B, min_len, max_len, seed)
    g = torch.Generator(device=device).manual_seed(seed)
    kc = torch.randn(t["n_pages"], H_KV, 16, D, generator=g, device=device, dtype=torch.float16)
    vc = torch.randn(t["n_pages"], H_KV, 16, D, generator=g, device=device, dtype=torch.float16)
    q = torch.randn(B, H_Q, 1, D, generator=g, device=device, dtype=torch.float16)
    return q, kc, vc, t["block_table"].to(device), t["seq_lens"].to(device), t["max_num_blocks"]


def _call_both(lib, stream, dev, q, kc, vc, bt, sl, mnb):
    """One call of each entry point on the same inputs: (workspace entry result, built-in scratch result)."""
    from flash_attn_v100_b200 import _lib
    B, H_Q, _, D = q.shape
    H_KV = kc.size(1)
    need = lib.fa_decode_workspace_bytes(B, H_Q, H_KV, D)
    ws = torch.zeros(need, dtype=torch.uint8, device=dev)
    out_ws = torch.full((B, H_Q, 1, D), 7.0, dtype=torch.float16, device=dev)
    out_st = torch.full((B, H_Q, 1, D), -7.0, dtype=torch.float16, device=dev)
    rc = lib.fa_paged_decode_gqa_f16(_vp(q), _vp(kc), _vp(vc), _vp(out_ws), _vp(bt), _vp(sl), B, H_Q, H_KV, D,
                                     kc.size(0), mnb, mnb * 16, _vp(ws), need, stream)
    assert rc == 0, _lib.last_error()
    rc = lib.fa_paged_decode_gqa_f16_static_scratch(_vp(q), _vp(kc), _vp(vc), _vp(out_st), _vp(bt), _vp(sl),
                                                    B, H_Q, H_KV, D, kc.size(0), mnb, mnb * 16, stream)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    st = ctypes.c_int(-1)
    assert lib.fa_decode_status(_vp(ws), stream, ctypes.byref(st)) == 0 and st.value == 0
    # the status word of the built-in scratch is read with a NULL workspace
    st = ctypes.c_int(-1)
    assert lib.fa_decode_status(None, stream, ctypes.byref(st)) == 0 and st.value == 0, _lib.last_error()
    return out_ws, out_st


def test_static_scratch_entry_point_matches_workspace_entry_point():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from flash_attn_v100_b200 import _lib
    from oracle import attention_oracle as orc
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    H_Q, H_KV, D = 32, 8, 128
    # two calls in a row; the second is larger, has other lengths and another batch size
    for seed, B, max_len in ((11, 5, 700), (12, 9, 3000)):
        q, kc, vc, bt, sl, mnb = _make_case(seed, B, H_Q, H_KV, D, max_len, dev)
        out_ws, out_st = _call_both(lib, stream, dev, q, kc, vc, bt, sl, mnb)
        assert not torch.isnan(out_st).any()
        err = (out_st.float() - out_ws.float()).abs().max().item()
        assert err <= TOL, err
        assert torch.equal(out_st, out_ws)
        # and against the CPU oracle, so that a fault shared by both entry points cannot hide
        ref = orc.paged_decode(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), sl.cpu(), final_cast=False)
        assert (out_st.float().cpu() - ref).abs().max().item() <= TOL


def test_static_scratch_small_split_batch_after_a_large_batch():
    """The array is shared by calls of every shape.  A large batch leaves its page prefix sums in it; a
    later small batch whose segments are all split across CTAs must not take such leftovers for arrival
    counters.  Many consecutive launches, each checked against the workspace entry point and the oracle."""
    from flash_attn_v100_b200 import _lib
    from oracle import attention_oracle as orc
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    q, kc, vc, bt, sl, mnb = _make_case(21, 4400, 8, 2, 64, 40, dev)     # B + 1 > 4096: prefix pre-pass
    out_ws, out_st = _call_both(lib, stream, dev, q, kc, vc, bt, sl, mnb)
    assert torch.equal(out_st, out_ws)
    q, kc, vc, bt, sl, mnb = _make_case(22, 2, 16, 16, 128, 33, dev, min_len=33)   # three pages per segment
    ref = orc.paged_decode(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), sl.cpu(), final_cast=False)
    for it in range(40):
        out_ws, out_st = _call_both(lib, stream, dev, q, kc, vc, bt, sl, mnb)
        assert torch.equal(out_st, out_ws), it
        assert (out_st.float().cpu() - ref).abs().max().item() <= TOL, it


def test_static_scratch_reports_a_bad_page_id_and_can_be_cleared():
    """A block_table entry outside the pool is recorded in the built-in scratch's status word (bit 1), read
    with a NULL workspace, and cleared by re-initialising the built-in scratch."""
    from flash_attn_v100_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    q, kc, vc, bt, sl, mnb = _make_case(31, 3, 32, 8, 128, 200, dev)
    bt = bt.clone()
    bt[1, 0] = kc.size(0) + 5
    out = torch.zeros_like(q)
    rc = lib.fa_paged_decode_gqa_f16_static_scratch(_vp(q), _vp(kc), _vp(vc), _vp(out), _vp(bt), _vp(sl), 3, 32, 8,
                                                    128, kc.size(0), mnb, mnb * 16, stream)
    assert rc == 0, _lib.last_error()
    st = ctypes.c_int(0)
    assert lib.fa_decode_status(None, stream, ctypes.byref(st)) == -5 and st.value == 2
    assert lib.fa_decode_workspace_init(None, 0, stream) == 0, _lib.last_error()
    assert lib.fa_decode_status(None, stream, ctypes.byref(st)) == 0 and st.value == 0


def test_static_scratch_validates_every_argument_before_touching_the_device():
    from flash_attn_v100_b200 import _lib
    lib = _lib.load()
    ok = ctypes.c_void_p(256)
    # null tensors, a null block table, a misaligned pointer, no pages, a zero stride
    for args in ((None, ok, ok, ok, ok, ok, 2, 32, 8, 128, 4, 1, 16),
                 (ok, ok, ok, ok, None, ok, 2, 32, 8, 128, 4, 1, 16),
                 (ctypes.c_void_p(260), ok, ok, ok, ok, ok, 2, 32, 8, 128, 4, 1, 16),
                 (ok, ok, ok, ok, ok, ok, 2, 32, 8, 128, 0, 1, 16),
                 (ok, ok, ok, ok, ok, ok, 2, 32, 8, 128, 4, 0, 16),
                 (ok, ok, ok, ok, ok, ok, 2, 32, 7, 128, 4, 1, 16)):
        assert lib.fa_paged_decode_gqa_f16_static_scratch(*args, None) == -1, args


def test_static_scratch_rejects_shapes_beyond_its_size():
    from flash_attn_v100_b200 import _lib
    lib = _lib.load()
    # 16 query heads per KV head at D=256 needs far more than 8 MiB of scratch
    assert lib.fa_decode_workspace_bytes(4, 32, 2, 256) > (8 << 20)
    dummy = ctypes.c_void_p(256)
    rc = lib.fa_paged_decode_gqa_f16_static_scratch(dummy, dummy, dummy, dummy, dummy, dummy, 4, 32, 2, 256,
                                                    1, 1, 16, None)
    assert rc == -3
    assert b"built-in scratch holds" in lib.fa_last_error()
