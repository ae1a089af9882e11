"""GPU: the paged decode entry point that carries its own scratch.

Some users of this library cannot hand it a workspace: their process has given all
device memory to a pool of its own, or they sit on a path where a cudaMalloc (and the
device-wide synchronisation it implies) is off limits.  For them
`fa_paged_decode_gqa_f16_static_scratch` keeps the split-KV scratch in an array inside
the library.  This test calls it through the C ABI twice in a row, on different inputs
(so anything the first call left in the shared array would show), and compares each
result with `fa_paged_decode_gqa_f16` given a caller-owned workspace.  Same kernels,
same launch configuration: the outputs must agree to the tolerance of the other decode
tests (2e-3), and in practice bit for bit.  It also checks the size limit.

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


def _make_case(seed, B, H_Q, H_KV, D, max_len, device):
    from flash_attn_v100_b200.synthetic import make_paged_tables
    t = make_paged_tables(B, 1, max_len, seed)
    g = torch.Generator(device=device).manual_seed(seed)
    kc = torch.randn(t["n_pages"], H_KV, 16, D, generator=g, device=device, dtype=torch.float16)
    vc = torch.randn(t["n_pages"], H_KV, 16, D, generator=g, device=device, dtype=torch.float16)
    q = torch.randn(B, H_Q, 1, D, generator=g, device=device, dtype=torch.float16)
    return q, kc, vc, t["block_table"].to(device), t["seq_lens"].to(device), t["max_num_blocks"]


def test_static_scratch_entry_point_matches_workspace_entry_point():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from flash_attn_v100_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    H_Q, H_KV, D = 32, 8, 128
    # two calls in a row; the second is larger, has other lengths and another batch size
    for seed, B, max_len in ((11, 5, 700), (12, 9, 3000)):
        q, kc, vc, bt, sl, mnb = _make_case(seed, B, H_Q, H_KV, D, max_len, dev)
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
        assert not torch.isnan(out_st).any()
        err = (out_st.float() - out_ws.float()).abs().max().item()
        assert err <= TOL, err
        assert torch.equal(out_st, out_ws)
        st = ctypes.c_int(-1)
        assert lib.fa_decode_status(_vp(ws), stream, ctypes.byref(st)) == 0 and st.value == 0


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
