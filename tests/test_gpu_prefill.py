"""GPU parity of the prefill entry points (dense, GQA, packed varlen)."""
import numpy as np
import pytest
import torch

import golden_cases as gc
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
TOL = 2e-3
TOL_FP16_FIXTURE = 4e-3


@pytest.fixture(autouse=True, params=["auto", "mma", "tc5_poly"])
def prefill_impl(request):
    """Every prefill test runs with the automatic kernel choice (tcgen05 kernel for D = 64/128),
    with the mma.sync kernel forced, and with the tcgen05 kernel's polynomial-exp2 variant."""
    import flash_attn_v100_b200 as pkg
    pkg.set_prefill_impl({"auto": 0, "mma": 1, "tc5_poly": 3}[request.param])
    yield request.param
    torch.cuda.synchronize()
    pkg.set_prefill_impl(0)
    pkg.check_prefill_errors()


def _err(a, b):
    return (a.detach().float().cpu() - torch.as_tensor(np.asarray(b)).float()).abs().max().item()


def test_prefill_gqa_golden(golden):
    import flash_attn_v100 as fa
    for i in range(len(gc.PREFILL_CASES)):
        q, k, v = gc.prefill_case(golden, i)
        rows = golden[f"prefill{i}/rows"]
        out = fa.forward_prefill_gqa_fp16(q.cuda(), k.cuda(), v.cuda(), True)
        assert _err(out[:, :, rows], golden[f"prefill{i}/out"]) < TOL_FP16_FIXTURE, i
        assert _err(out, orc.prefill_gqa(q, k, v, True, final_cast=False)) < TOL, i
        assert torch.equal(fa.forward_prefill_gqa_fp16_warp(q.cuda(), k.cuda(), v.cuda(), True), out)
    for kind, i, q, k, v, N in gc.gqa_cases(golden):
        if kind != "prefill":
            continue
        rows = golden[f"gqa_prefill{i}/rows"]
        out = fa.forward_prefill_gqa_fp16(q.cuda(), k.cuda(), v.cuda(), True)
        assert _err(out[:, :, rows], golden[f"gqa_prefill{i}/out"]) < TOL_FP16_FIXTURE, i


def test_dense_mha_golden_and_out_variant(golden):
    import flash_attn_v100 as fa
    q, k, v = gc.dense_case(golden)
    rows = golden["dense/rows"]
    for causal in (False, True):
        out = fa.forward_fp16(q.cuda(), k.cuda(), v.cuda(), causal)
        assert _err(out[:, :, rows], golden[f"dense/causal{int(causal)}"]) < TOL_FP16_FIXTURE
        assert _err(out, orc.prefill_gqa(q, k, v, causal, final_cast=False)) < TOL
        # GQA entry point with H_Q == H_KV equals the MHA one (test_prefill_gqa.py:94-141)
        assert torch.equal(fa.forward_prefill_gqa_fp16(q.cuda(), k.cuda(), v.cuda(), causal), out)
    buf = torch.full(q.shape, -7.0, dtype=torch.float16, device="cuda")
    res = fa.forward_prefill_gqa_fp16_out(buf, q.cuda(), k.cuda(), v.cuda(), True)
    assert res.data_ptr() == buf.data_ptr()         # test.py:123-131
    assert torch.equal(res, fa.forward_prefill_gqa_fp16(q.cuda(), k.cuda(), v.cuda(), True))
    with pytest.raises(RuntimeError, match="out shape"):
        fa.forward_prefill_gqa_fp16_out(buf[:, :, :5].contiguous(), q.cuda(), k.cuda(), v.cuda(), True)


@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("N", [1, 15, 63, 64, 65, 127, 128, 129, 200, 257, 600])
def test_dense_ragged_lengths(D, N):
    import flash_attn_v100 as fa
    B, H_Q, H_KV = 2, 4, 2
    g = torch.Generator().manual_seed(N + D)
    q = torch.randn(B, H_Q, N, D, generator=g).half()
    k = torch.randn(B, H_KV, N, D, generator=g).half()
    v = torch.randn(B, H_KV, N, D, generator=g).half()
    for causal in (True, False):
        out = fa.forward_prefill_gqa_fp16(q.cuda(), k.cuda(), v.cuda(), causal)
        assert _err(out, orc.prefill_gqa(q, k, v, causal, final_cast=False)) < TOL, (N, D, causal)


@pytest.mark.parametrize("H_Q,H_KV,D", [(4, 4, 64), (8, 2, 128), (32, 8, 128), (4, 1, 256)])
def test_varlen_prefill(H_Q, H_KV, D):
    import flash_attn_v100 as fa
    lens = [64, 128, 256, 1, 17, 129, 300, 5]      # test_async.py:68-113 uses [64,128,256]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    total = int(cu[-1])
    g = torch.Generator().manual_seed(H_Q * D)
    q = torch.randn(total, H_Q, D, generator=g).half()
    k = torch.randn(total, H_KV, D, generator=g).half()
    v = torch.randn(total, H_KV, D, generator=g).half()
    for causal in (True, False):
        out = fa.forward_varlen_prefill_fp16(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), max(lens), causal)
        ref = orc.varlen_prefill(q, k, v, cu, causal, final_cast=False)
        assert _err(out, ref) < TOL, causal
    st = torch.cuda.Stream()
    qc, kc, vc, cuc = q.cuda(), k.cuda(), v.cuda(), cu.cuda()
    base = fa.forward_varlen_prefill_fp16(qc, kc, vc, cuc, max(lens), True)
    torch.cuda.synchronize()
    res = fa.forward_varlen_prefill_fp16_stream(qc, kc, vc, cuc, max(lens), True, st.cuda_stream)
    st.synchronize()
    assert torch.equal(res, base)                   # test_async.py:68-113
    # a sequence followed by unused rows: rows past cu_seqlens[-1] stay zero
    cu_short = cu[:-1].contiguous()
    out_s = fa.forward_varlen_prefill_fp16(qc, kc, vc, cu_short.cuda(), max(lens), True)
    assert (out_s[int(cu_short[-1]):] == 0).all()
    assert torch.equal(out_s[: int(cu_short[-1])], base[: int(cu_short[-1])])


def test_varlen_config3_shape_sample():
    """Benchmark config 3: 16 sequences, lengths U[128,4096], 32/8 heads, D=128, causal.
    A few sequences and query rows against the oracle; sequences are independent of
    their neighbours in the packing (permuting the packing permutes the output)."""
    import flash_attn_v100 as fa
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(128, 4097, (16,), generator=g).tolist()
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    total = int(cu[-1])
    gd = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(total, 32, 128, generator=gd, device="cuda", dtype=torch.float16)
    k = torch.randn(total, 8, 128, generator=gd, device="cuda", dtype=torch.float16)
    v = torch.randn(total, 8, 128, generator=gd, device="cuda", dtype=torch.float16)
    out = fa.forward_varlen_prefill_fp16(q, k, v, cu.cuda(), max(lens), True)
    order = sorted(range(16), key=lambda i: lens[i])
    for s in (order[0], order[7], order[-1]):
        a, n = int(cu[s]), lens[s]
        ref = orc.varlen_prefill(q[a:a + n].cpu(), k[a:a + n].cpu(), v[a:a + n].cpu(),
                                 torch.tensor([0, n], dtype=torch.int32), True, final_cast=False)
        assert _err(out[a:a + n], ref) < TOL, s
    # reverse the packing order
    segs = [(int(cu[s]), lens[s]) for s in reversed(range(16))]
    idx = torch.cat([torch.arange(a, a + n) for a, n in segs]).cuda()
    cu_r = torch.tensor([0] + list(np.cumsum([n for _, n in segs])), dtype=torch.int32)
    out_r = fa.forward_varlen_prefill_fp16(q[idx].contiguous(), k[idx].contiguous(), v[idx].contiguous(),
                                           cu_r.cuda(), max(lens), True)
    assert torch.equal(out_r, out[idx])


@pytest.mark.parametrize("D", [8, 40, 72, 96, 112, 160, 192, 248])
def test_head_dimensions_between_the_builds(D):
    """Head dimensions between the kernel builds (64, 128, 256) run on the next larger one; the reference
    takes any D <= 256.  Dense GQA (causal and not) and packed varlen."""
    import flash_attn_v100 as fa
    torch.manual_seed(D)
    B, H_Q, H_KV, N = 2, 4, 2, 150
    q = torch.randn(B, H_Q, N, D).half()
    k = torch.randn(B, H_KV, N, D).half()
    v = torch.randn(B, H_KV, N, D).half()
    for causal in (True, False):
        out = fa.forward_prefill_gqa_fp16(q.cuda(), k.cuda(), v.cuda(), causal)
        assert out.shape == q.shape
        assert _err(out, orc.prefill_gqa(q, k, v, causal, final_cast=False)) < TOL, (D, causal)
    lens = [37, 150, 1, 90]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    total = int(cu[-1])
    qp = torch.randn(total, H_Q, D).half()
    kp = torch.randn(total, H_KV, D).half()
    vp = torch.randn(total, H_KV, D).half()
    out = fa.forward_varlen_prefill_fp16(qp.cuda(), kp.cuda(), vp.cuda(), cu.cuda(), max(lens), True)
    ref = orc.varlen_prefill(qp, kp, vp, cu, True, final_cast=False)
    assert _err(out, ref) < TOL, D
