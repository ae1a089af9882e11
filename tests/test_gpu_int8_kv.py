"""GPU parity of the INT8-KV-cache decode against the oracle and the fixture made from the reference's own
tests.  Tolerance: max-abs-err 2e-3 against the oracle's fp32 value (the reference's test accepts 0.1 against
the fp16 decode, test_kv_compress.py:56); 4e-3 against the fixture's fp16-cast output."""
import numpy as np
import pytest
import torch

import golden_cases as gc
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
TOL = 2e-3
TOL_FP16_FIXTURE = 4e-3


@pytest.fixture(scope="module")
def fa():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import flash_attn_v100
    return flash_attn_v100


def _err(a, b):
    return (a.detach().float().cpu() - torch.as_tensor(np.asarray(b)).float()).abs().max().item()


def _finish():
    import flash_attn_v100_b200
    torch.cuda.synchronize()
    flash_attn_v100_b200.check_async_errors()


def test_reference_test_cases(fa, golden_kv_compress):
    for i, q, k8, v8, ks, vs, k, v, cache_len in gc.int8_kv_cases(golden_kv_compress, orc.quantize_kv_int8):
        out = fa.forward_decode_int8_kv_cache_gqa(q.cuda(), k8.cuda(), v8.cuda(), ks.cuda(), vs.cuda(), cache_len)
        assert out.shape == q.shape and out.dtype == torch.float16
        assert _err(out, golden_kv_compress[f"i8kv{i}/out"]) < TOL_FP16_FIXTURE, i
        ref32 = orc.decode_int8_kv_cache_gqa(q, k8, v8, ks, vs, cache_len, final_cast=False)
        assert _err(out, ref32) < TOL, i
        # the reference's own acceptance test: within 0.1 of the fp16 decode on the unquantised cache
        fp16 = fa.forward_decode_gqa_fp16(q.cuda(), k.cuda(), v.cuda(), True, cache_len)
        assert (out.float() - fp16.float()).abs().max().item() < 0.1
    _finish()


@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("heads", [(8, 8), (8, 2), (32, 8), (40, 2)])
def test_shapes_and_lengths(fa, D, heads):
    H_Q, H_KV = heads
    torch.manual_seed(7 * D + H_Q)
    B, N = 3, 333
    q = torch.randn(B, H_Q, 1, D).half()
    k = (torch.randn(B, H_KV, N, D) * 1.7).half()
    v = (torch.randn(B, H_KV, N, D) * 0.6).half()
    k8, ks = orc.quantize_kv_int8(k)
    v8, vs = orc.quantize_kv_int8(v)
    dev = [t.cuda() for t in (q, k8, v8, ks, vs)]
    for cache_len in (332, 0, 15, 16, 100, 5000):
        out = fa.forward_decode_int8_kv_cache_gqa(*dev, cache_len)
        ref = orc.decode_int8_kv_cache_gqa(q, k8, v8, ks, vs, cache_len, final_cast=False)
        assert _err(out, ref) < TOL, (D, heads, cache_len)
    out = fa.forward_decode_int8_kv_cache_gqa(*dev, -1)
    assert out.abs().max().item() == 0
    _finish()


def test_dequantisation_is_the_reference_expression(fa):
    """The kernel's in-register dequantisation equals fp16(float(int8) * float(scale)): running the fp16 decode
    on a cache dequantised that way gives the same result up to the order of fp32 summation, for every int8
    value and for scales across the fp16 range (subnormal products included)."""
    torch.manual_seed(9)
    B, H_Q, H_KV, N, D = 1, 8, 2, 256, 128
    q = torch.randn(B, H_Q, 1, D).half()
    k8 = torch.randint(-128, 128, (B, H_KV, N, D), dtype=torch.int8)
    v8 = torch.randint(-128, 128, (B, H_KV, N, D), dtype=torch.int8)
    k8[0, 0, :, 0] = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8)   # every value once
    v8[0, 0, :, 1] = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8)
    ks = (torch.rand(B, H_KV, N) + 1.0) * torch.pow(2.0, torch.linspace(-20.0, -6.0, N))
    vs = (torch.rand(B, H_KV, N) + 1.0) * torch.pow(2.0, torch.linspace(-9.0, -20.0, N))
    ks, vs = ks.half(), vs.half()
    out = fa.forward_decode_int8_kv_cache_gqa(q.cuda(), k8.cuda(), v8.cuda(), ks.cuda(), vs.cuda(), N - 1)
    kd, vd = orc.dequantize_kv_int8(k8, ks), orc.dequantize_kv_int8(v8, vs)
    via_fp16 = fa.forward_decode_gqa_fp16(q.cuda(), kd.cuda(), vd.cuda(), True, N - 1)
    # two fp16 roundings of nearly equal fp32 values: at most one unit in the last place apart
    assert (out.float() - via_fp16.float()).abs().max().item() <= max(2e-4, 2.0 ** -10 * out.abs().max().item())
    ref = orc.decode_int8_kv_cache_gqa(q, k8, v8, ks, vs, N - 1, final_cast=False)
    assert _err(out, ref) < TOL
    _finish()


def test_tokens_past_cache_len_are_not_used(fa):
    torch.manual_seed(10)
    B, H_Q, H_KV, N, D = 2, 16, 4, 1000, 128
    q = torch.randn(B, H_Q, 1, D).half()
    k8, ks = orc.quantize_kv_int8(torch.randn(B, H_KV, N, D).half())
    v8, vs = orc.quantize_kv_int8(torch.randn(B, H_KV, N, D).half())
    cache_len = 700
    a = fa.forward_decode_int8_kv_cache_gqa(q.cuda(), k8.cuda(), v8.cuda(), ks.cuda(), vs.cuda(), cache_len)
    ks2, vs2, k82, v82 = ks.clone(), vs.clone(), k8.clone(), v8.clone()
    ks2[:, :, cache_len + 1:] = float("nan"); vs2[:, :, cache_len + 1:] = float("inf")
    k82[:, :, cache_len + 1:] = -128; v82[:, :, cache_len + 1:] = 127
    b = fa.forward_decode_int8_kv_cache_gqa(q.cuda(), k82.cuda(), v82.cuda(), ks2.cuda(), vs2.cuda(), cache_len)
    assert torch.equal(a, b)
    _finish()


def test_long_cache_split_across_ctas(fa):
    torch.manual_seed(12)
    B, H_Q, H_KV, N, D = 2, 32, 8, 16384, 128
    q = torch.randn(B, H_Q, 1, D, device="cuda").half()
    k = torch.randn(B, H_KV, N, D, device="cuda").half()
    v = torch.randn(B, H_KV, N, D, device="cuda").half()
    k8, ks = (t.cuda() for t in orc.quantize_kv_int8(k.cpu()))
    v8, vs = (t.cuda() for t in orc.quantize_kv_int8(v.cpu()))
    out = fa.forward_decode_int8_kv_cache_gqa(q, k8, v8, ks, vs, N - 1)
    kd = orc.dequantize_kv_int8(k8.cpu(), ks.cpu()).cuda()
    vd = orc.dequantize_kv_int8(v8.cpu(), vs.cpu()).cuda()
    via_fp16 = fa.forward_decode_gqa_fp16(q, kd, vd, True, N - 1)
    assert (out.float() - via_fp16.float()).abs().max().item() <= 2e-4
    _finish()


def test_input_checks(fa):
    q = torch.zeros(1, 8, 1, 64, device="cuda", dtype=torch.float16)
    k8 = torch.zeros(1, 2, 32, 64, device="cuda", dtype=torch.int8)
    s = torch.ones(1, 2, 32, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match="k_int8 must be int8"):
        fa.forward_decode_int8_kv_cache_gqa(q, k8.half(), k8, s, s, 31)
    with pytest.raises(RuntimeError, match="k_scale must be float16"):
        fa.forward_decode_int8_kv_cache_gqa(q, k8, k8, s.float(), s, 31)
    with pytest.raises(RuntimeError, match="v_scale size mismatch"):
        fa.forward_decode_int8_kv_cache_gqa(q, k8, k8, s, s[:, :, :16].contiguous(), 31)
    with pytest.raises(RuntimeError, match="last dim must match D"):
        fa.forward_decode_int8_kv_cache_gqa(q, k8[..., :32].contiguous(), k8, s, s, 31)
