"""GPU parity of the sliding-window + attention-sink decode against the oracle and the fixture made from the
reference's own tests.  Tolerance: max-abs-err 2e-3 against the oracle's fp32 value (the reference's test
accepts 1e-2, test_kv_compress.py:278); 4e-3 against the fixture's fp16-cast output."""
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
    for i, q, k, v, cache_len, window, sink in gc.sliding_window_cases(golden_kv_compress):
        out = fa.forward_decode_sliding_window_gqa(q.cuda(), k.cuda(), v.cuda(), True, cache_len, window, sink)
        assert out.shape == q.shape and out.dtype == torch.float16
        assert _err(out, golden_kv_compress[f"sw{i}/out"]) < TOL_FP16_FIXTURE, i
        assert _err(out, orc.sliding_window_decode(q, k, v, True, cache_len, window, sink, final_cast=False)) < TOL, i
    _finish()


@pytest.mark.parametrize("D", [64, 128, 256])
def test_window_and_sink_edges(fa, D):
    torch.manual_seed(100 + D)
    B, H_Q, H_KV, N = 2, 8, 2, 333
    q = torch.randn(B, H_Q, 1, D).half(); k = torch.randn(B, H_KV, N, D).half(); v = torch.randn(B, H_KV, N, D).half()
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    cases = [
        (332, 64, 4),     # the reference's shape of use
        (332, 1, 0),      # one key
        (200, 16, 16),    # page-aligned window and sink
        (200, 17, 15),    # neither aligned
        (100, 90, 30),    # sink and window overlap: shared pages visited once
        (40, 1000, 0),    # window wider than the cache: plain causal decode
        (10, 4, 50),      # sink reaches past cache_len (the sink is not bounded by it)
        (30, 0, 7),       # empty window, sink only
        (5, -3, 2),       # negative window is empty
        (999, 32, 3),     # cache_len past N: window ends at N
        (332, 32, 400),   # sink past N: everything
        (0, 8, 0),        # first token
    ]
    for cache_len, window, sink in cases:
        out = fa.forward_decode_sliding_window_gqa(qc, kc, vc, False, cache_len, window, sink)
        ref = orc.sliding_window_decode(q, k, v, False, cache_len, window, sink, final_cast=False)
        assert _err(out, ref) < TOL, (D, cache_len, window, sink)
    # nothing attended: zeros
    out = fa.forward_decode_sliding_window_gqa(qc, kc, vc, True, -1, 8, 0)
    assert out.abs().max().item() == 0
    _finish()


def test_equals_plain_decode_when_window_covers_cache(fa):
    torch.manual_seed(3)
    B, H_Q, H_KV, N, D = 3, 32, 8, 1000, 128
    q = torch.randn(B, H_Q, 1, D, device="cuda").half()
    k = torch.randn(B, H_KV, N, D, device="cuda").half()
    v = torch.randn(B, H_KV, N, D, device="cuda").half()
    a = fa.forward_decode_sliding_window_gqa(q, k, v, True, 700, 4096, 0)
    b = fa.forward_decode_gqa_fp16(q, k, v, True, 700)
    assert (a.float() - b.float()).abs().max().item() < 1e-3
    _finish()


def test_unread_pages_do_not_matter(fa):
    """Keys outside the sink and the window are never read: poisoning them with NaN leaves the output unchanged."""
    torch.manual_seed(4)
    B, H_Q, H_KV, N, D = 2, 16, 4, 4096, 128
    q = torch.randn(B, H_Q, 1, D, device="cuda").half()
    k = torch.randn(B, H_KV, N, D, device="cuda").half()
    v = torch.randn(B, H_KV, N, D, device="cuda").half()
    cache_len, window, sink = 4000, 512, 4
    a = fa.forward_decode_sliding_window_gqa(q, k, v, True, cache_len, window, sink)
    k2, v2 = k.clone(), v.clone()
    ws = cache_len + 1 - window
    k2[:, :, sink:ws] = float("nan"); v2[:, :, sink:ws] = float("nan")
    k2[:, :, cache_len + 1:] = float("nan"); v2[:, :, cache_len + 1:] = float("nan")
    b = fa.forward_decode_sliding_window_gqa(q, k2, v2, True, cache_len, window, sink)
    assert torch.equal(a, b)
    ref = orc.sliding_window_decode(q.cpu(), k.cpu(), v.cpu(), True, cache_len, window, sink, final_cast=False)
    assert _err(a, ref) < TOL
    _finish()


def test_input_checks(fa):
    q = torch.zeros(1, 8, 1, 64, device="cuda", dtype=torch.float16)
    k = torch.zeros(1, 3, 32, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match="divisible"):
        fa.forward_decode_sliding_window_gqa(q, k, k, True, 31, 8, 0)
    k = torch.zeros(1, 2, 32, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match="float16"):
        fa.forward_decode_sliding_window_gqa(q.float(), k, k, True, 31, 8, 0)
    with pytest.raises(RuntimeError, match="sequence length must be 1"):
        fa.forward_decode_sliding_window_gqa(torch.zeros(1, 8, 2, 64, device="cuda", dtype=torch.float16), k, k,
                                             True, 31, 8, 0)
