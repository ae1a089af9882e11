"""GPU parity of the decode entry points against the oracle and the golden
fixtures.  Tolerance: max-abs-err 2e-3 against the oracle's fp32 value (before
its closing fp16 cast); 4e-3 against fixtures that hold the reference oracle's
fp16-cast output (two independent fp16 roundings)."""
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


def _finish(fa):
    import flash_attn_v100_b200
    torch.cuda.synchronize()
    flash_attn_v100_b200.check_async_errors()


def test_continuous_batching_golden(fa, golden):
    for name, *_ in gc.CONT_BATCH_CASES:
        q, k, v, lens = gc.cont_batch_case(golden, name)
        for causal in (False, True):
            out = fa.forward_continuous_batching_fp16(q.cuda(), k.cuda(), v.cuda(), lens.cuda(), causal)
            assert out.shape == q.shape and out.dtype == torch.float16
            assert _err(out, golden[f"{name}/causal{int(causal)}"]) < TOL_FP16_FIXTURE, name
            ref32 = orc.continuous_batching_decode(q, k, v, lens, causal, final_cast=False)
            assert _err(out, ref32) < TOL, name
    _finish(fa)


def test_decode_gqa_golden(fa, golden):
    for kind, i, q, k, v, N in gc.gqa_cases(golden):
        if kind != "decode":
            continue
        out = fa.forward_decode_gqa_fp16(q.cuda(), k.cuda(), v.cuda(), True, N - 1)
        assert _err(out, golden[f"gqa_decode{i}/out"]) < TOL_FP16_FIXTURE, i
        assert _err(out, orc.decode_gqa(q, k, v, True, N - 1, final_cast=False)) < TOL, i
    _finish(fa)


def test_paged_decode_golden(fa, golden):
    q, k, v, seq_lens = gc.paged_case(golden)
    kc, vc, bt, mnb = orc.build_paged_cache(k, v, seq_lens, gc.PAGED_ORDER)
    out = fa.forward_paged_decode_gqa_fp16(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), seq_lens.cuda(), mnb)
    assert _err(out, golden["paged/out"]) < TOL_FP16_FIXTURE
    # cache reuse: updating one block changes the result and still matches (test_decode.py:296-322)
    k2, v2 = k.clone(), v.clone()
    k2[1, :, 16:23] += 0.5
    v2[1, :, 16:23] -= 0.25
    kc2, vc2, _, _ = orc.build_paged_cache(k2, v2, seq_lens, gc.PAGED_ORDER)
    out2 = fa.forward_paged_decode_gqa_fp16(q.cuda(), kc2.cuda(), vc2.cuda(), bt.cuda(), seq_lens.cuda(), mnb)
    assert _err(out2, golden["paged/out_updated"]) < TOL_FP16_FIXTURE
    assert (out2.float() - out.float()).abs().max().item() > 1e-4
    _finish(fa)


@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("H_Q,H_KV", [(8, 8), (8, 2), (32, 8), (8, 1), (32, 1), (40, 2)])
def test_paged_every_length_up_to_three_pages(fa, D, H_Q, H_KV):
    """All lengths 0..49 (page boundary, partial pages, empty sequence) in one batch,
    stale (NaN) data in the unused slots of the pool."""
    lens = torch.arange(0, 50, dtype=torch.int32)
    B = lens.numel()
    g = torch.Generator().manual_seed(100 + D + H_Q)
    k = torch.randn(B, H_KV, 49, D, generator=g).half()
    v = torch.randn(B, H_KV, 49, D, generator=g).half()
    q = torch.randn(B, H_Q, 1, D, generator=g).half()
    n_pages = int(((lens + 15) // 16).sum())
    order = torch.randperm(n_pages + 3, generator=g).tolist()
    kc, vc, bt, mnb = orc.build_paged_cache(k, v, lens, order, num_physical_blocks=n_pages + 3)
    # poison what a sequence must never read: slots past its length and unused pages
    used = torch.zeros(n_pages + 3, 16, dtype=torch.bool)
    for b in range(B):
        for t in range(int(lens[b])):
            used[bt[b, t // 16], t % 16] = True
    poison = ~used[:, None, :, None].expand(-1, H_KV, -1, D)
    kc[poison] = float("nan")
    vc[poison] = float("nan")
    out = fa.forward_paged_decode_gqa_fp16(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), lens.cuda(), mnb)
    ref = orc.paged_decode(q, torch.nan_to_num(kc), torch.nan_to_num(vc), bt, lens, final_cast=False)
    assert not torch.isnan(out).any()
    assert (out[0] == 0).all()                      # empty sequence: zeros by definition
    assert _err(out, ref) < TOL
    _finish(fa)


@pytest.mark.parametrize("D,N", [(64, 65), (128, 257), (256, 129), (128, 1), (128, 16), (128, 4099)])
def test_contiguous_decode_masks(fa, D, N):
    B, H_Q, H_KV = 3, 16, 4
    g = torch.Generator().manual_seed(N)
    q = torch.randn(B, H_Q, 1, D, generator=g).half()
    k = torch.randn(B, H_KV, N, D, generator=g).half()
    v = torch.randn(B, H_KV, N, D, generator=g).half()
    for causal, cache_len in ((True, N - 1), (True, N // 2), (False, N // 2), (True, 0)):
        out = fa.forward_decode_gqa_fp16(q.cuda(), k.cuda(), v.cuda(), causal, cache_len)
        ref = orc.decode_gqa(q, k, v, causal, cache_len, final_cast=False)
        assert _err(out, ref) < TOL, (causal, cache_len)
    # MHA entry point and the _out / _stream variants
    qm = torch.randn(B, H_KV, 1, D, generator=g).half()
    out = fa.forward_decode_fp16(qm.cuda(), k.cuda(), v.cuda(), True, N - 1)
    assert _err(out, orc.decode_gqa(qm, k, v, True, N - 1, final_cast=False)) < TOL
    buf = torch.full((B, H_Q, 1, D), 123.0, dtype=torch.float16, device="cuda")
    res = fa.forward_decode_gqa_fp16_out(buf, q.cuda(), k.cuda(), v.cuda(), True, N - 1)
    assert res.data_ptr() == buf.data_ptr()        # test.py:116-121
    base = fa.forward_decode_gqa_fp16(q.cuda(), k.cuda(), v.cuda(), True, N - 1)
    assert torch.equal(res, base)
    st = torch.cuda.Stream()
    qc, kc_, vc_ = q.cuda(), k.cuda(), v.cuda()
    torch.cuda.synchronize()
    res_s = fa.forward_decode_gqa_fp16_stream(qc, kc_, vc_, True, N - 1, st.cuda_stream)
    st.synchronize()
    assert torch.equal(res_s, base)                # test_async.py:37-66
    _finish(fa)


def test_continuous_batching_edge_lengths(fa):
    B, H_Q, H_KV, D, max_N = 6, 32, 8, 128, 70
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, H_Q, 1, D, generator=g).half()
    k = torch.randn(B, H_KV, max_N, D, generator=g).half()
    v = torch.randn(B, H_KV, max_N, D, generator=g).half()
    lens = torch.tensor([0, 15, 16, 69, 200, -1], dtype=torch.int32)   # 200 clips to max_N; -1 => zeros
    out = fa.forward_continuous_batching_fp16(q.cuda(), k.cuda(), v.cuda(), lens.cuda(), True)
    ref = orc.continuous_batching_decode(q, k, v, lens, True, final_cast=False)
    assert _err(out, ref) < TOL
    assert (out[5] == 0).all()
    _finish(fa)


def test_error_paths_raise_runtime_error(fa):
    q = torch.randn(2, 8, 1, 64, device="cuda", dtype=torch.float16)
    k = torch.randn(2, 8, 32, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match="same dtype"):            # test.py:70-78
        fa.forward_fp16(k, k.float(), k, True)
    with pytest.raises(RuntimeError, match="non-negative"):          # test.py:80-89
        fa.forward_decode_gqa_fp16(q, k, k, True, -1)
    with pytest.raises(RuntimeError, match="less than sequence length"):
        fa.forward_decode_gqa_fp16(q, k, k, True, 32)
    with pytest.raises(RuntimeError, match="out sequence length"):   # test.py:133-139
        fa.forward_decode_gqa_fp16_out(torch.empty(2, 8, 2, 64, device="cuda", dtype=torch.float16), q, k, k, True, 31)
    with pytest.raises(RuntimeError, match="contiguous"):
        fa.forward_decode_gqa_fp16(q, k.transpose(1, 2), k, True, 31)
    with pytest.raises(RuntimeError, match="divisible"):
        fa.forward_decode_gqa_fp16(q, k[:, :3].contiguous(), k[:, :3].contiguous(), True, 31)
    with pytest.raises(RuntimeError, match="block size mismatch"):
        fa.forward_paged_decode_gqa_fp16(q, k, k, torch.zeros(2, 1, dtype=torch.int32, device="cuda"),
                                         torch.ones(2, dtype=torch.int32, device="cuda"), 1)
    q100 = torch.randn(2, 8, 1, 100, device="cuda", dtype=torch.float16)
    k100 = torch.randn(2, 8, 32, 100, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match="not built"):
        fa.forward_decode_gqa_fp16(q100, k100, k100, True, 31)


def test_bad_page_id_is_reported_not_faulted(fa):
    import flash_attn_v100_b200
    q = torch.randn(1, 8, 1, 64, device="cuda", dtype=torch.float16)
    kc = torch.randn(4, 8, 16, 64, device="cuda", dtype=torch.float16)
    bt = torch.tensor([[99]], dtype=torch.int32, device="cuda")     # outside the 4-page pool
    lens = torch.tensor([5], dtype=torch.int32, device="cuda")
    fa.forward_paged_decode_gqa_fp16(q, kc, kc, bt, lens, 1)
    with pytest.raises(RuntimeError, match="device status"):
        flash_attn_v100_b200.check_async_errors()
    # the status word is sticky per workspace: clear it for the tests that follow
    from flash_attn_v100_b200 import ops, _lib
    for ws in ops._workspaces.values():
        ws[:256].zero_()
    torch.cuda.synchronize()
    flash_attn_v100_b200.check_async_errors()


def test_paged_config2_shape_properties(fa):
    """Benchmark config 2 at full size: B=64, 32/8 heads, D=128, lens U[512,8192].
    (a) a sample of sequences against the oracle; (b) relabelling the physical
    pages (another permutation + the matching block table) leaves the output
    bit-identical; (c) the output is linear in V."""
    w = orc.make_paged_workload(64, 32, 8, 128, 512, 8192, seed=0, fill=False)
    n_pages, bt, lens = w["n_pages"], w["block_table"], w["seq_lens"]
    g = torch.Generator(device="cuda").manual_seed(0)
    kc = torch.randn(n_pages, 8, 16, 128, generator=g, device="cuda", dtype=torch.float16)
    vc = torch.randn(n_pages, 8, 16, 128, generator=g, device="cuda", dtype=torch.float16)
    q = w["q"].cuda()
    out = fa.forward_paged_decode_gqa_fp16(q, kc, vc, bt.cuda(), lens.cuda(), w["max_num_blocks"])
    torch.cuda.synchronize()
    sample = [0, 17, 63, int(lens.argmax()), int(lens.argmin())]
    for b in sample:
        idx = bt[b, : (int(lens[b]) + 15) // 16].long()
        kb, vb = kc[idx.cuda()].cpu(), vc[idx.cuda()].cpu()
        bt_b = torch.arange(idx.numel(), dtype=torch.int32)[None]
        ref = orc.paged_decode(w["q"][b:b + 1], kb, vb, bt_b, lens[b:b + 1], final_cast=False)
        assert _err(out[b:b + 1], ref) < TOL, b
    # (b) relabel pages
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(1))
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(n_pages)
    kc2, vc2 = kc[perm.cuda()], vc[perm.cuda()]          # new page j holds old page perm[j]
    bt2 = bt.clone()
    m = bt2 >= 0
    bt2[m] = inv[bt2[m].long()].int()
    out2 = fa.forward_paged_decode_gqa_fp16(q, kc2, vc2, bt2.cuda(), lens.cuda(), w["max_num_blocks"])
    assert torch.equal(out, out2)
    del kc2, vc2
    # (c) linearity in V: out(V) with V = 0.5 * V1 equals 0.5 * out(V1) up to fp16 rounding
    out_half = fa.forward_paged_decode_gqa_fp16(q, kc, vc * 0.5, bt.cuda(), lens.cuda(), w["max_num_blocks"])
    assert (out_half.float() * 2 - out.float()).abs().max().item() < 1e-3
    _finish(fa)


def test_paged_large_batch_uses_the_prefix_pre_pass(fa):
    """B + 1 > 4096: the page prefix sums come from the one-CTA pre-pass instead of the in-kernel scan."""
    torch.manual_seed(21)
    B, H_Q, H_KV, D = 4500, 8, 2, 64
    lens = torch.randint(0, 40, (B,), dtype=torch.int32)
    max_len = 48
    k = torch.randn(B, H_KV, max_len, D).half()
    v = torch.randn(B, H_KV, max_len, D).half()
    q = torch.randn(B, H_Q, 1, D).half()
    order = torch.randperm(B * 3, generator=torch.Generator().manual_seed(5)).tolist()
    kc, vc, bt, mnb = orc.build_paged_cache(k, v, lens, order)
    out = fa.forward_paged_decode_gqa_fp16(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), lens.cuda(), mnb)
    sel = torch.arange(0, B, 37)
    ref = orc.paged_decode(q[sel], kc, vc, bt[sel], lens[sel], final_cast=False)
    assert _err(out[sel.cuda()], ref) < TOL
    assert out[(lens == 0).cuda()].abs().max().item() == 0
    _finish(fa)


@pytest.mark.parametrize("heads", [(12, 1), (24, 2), (20, 1), (48, 3)])
def test_group_sizes_beyond_eight_heads(fa, heads):
    """More than 8 query heads per KV head: full 16-row fragments, and more than 16: several head blocks."""
    H_Q, H_KV = heads
    torch.manual_seed(H_Q)
    B, N, D = 2, 203, 128
    q = torch.randn(B, H_Q, 1, D).half()
    k = torch.randn(B, H_KV, N, D).half()
    v = torch.randn(B, H_KV, N, D).half()
    for cache_len in (202, 17):
        out = fa.forward_decode_gqa_fp16(q.cuda(), k.cuda(), v.cuda(), True, cache_len)
        assert _err(out, orc.decode_gqa(q, k, v, True, cache_len, final_cast=False)) < TOL, (heads, cache_len)
    _finish(fa)


def test_split_segments_after_a_large_batch_on_the_same_workspace(fa):
    """The scratch of a stream is shared by calls of any shape.  A large batch leaves its page prefix sums
    (all small integers) in it; the arrival counters of later calls must not be read from such leftovers.
    Small batches whose segments are all split across CTAs, over many consecutive launches."""
    torch.manual_seed(33)
    Bl, H_Q, H_KV, D = 4500, 8, 2, 64
    lens = torch.randint(1, 40, (Bl,), dtype=torch.int32)
    k = torch.randn(Bl, H_KV, 48, D).half()
    v = torch.randn(Bl, H_KV, 48, D).half()
    q = torch.randn(Bl, H_Q, 1, D).half()
    order = torch.randperm(Bl * 3, generator=torch.Generator().manual_seed(6)).tolist()
    kc, vc, bt, mnb = orc.build_paged_cache(k, v, lens, order)
    fa.forward_paged_decode_gqa_fp16(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), lens.cuda(), mnb)
    # 2 sequences x 16 KV heads x 2 pages: one page per CTA, every segment is merged from two partials
    B, H, N, Ds = 2, 16, 33, 128
    qs = torch.randn(B, H, 1, Ds).half()
    ks_ = torch.randn(B, H, N, Ds).half()
    vs_ = torch.randn(B, H, N, Ds).half()
    ref = orc.decode_gqa(qs, ks_, vs_, True, 20, final_cast=False)
    qc, kc2, vc2 = qs.cuda(), ks_.cuda(), vs_.cuda()
    for it in range(60):
        out = fa.forward_decode_gqa_fp16(qc, kc2, vc2, True, 20)
        assert _err(out, ref) < TOL, it
    _finish(fa)


@pytest.mark.parametrize("D", [8, 32, 48, 72, 80, 96, 112, 160, 192, 248])
def test_head_dimensions_between_the_builds(fa, D):
    """Any head dimension up to 256 that is a multiple of 8 (the reference takes any D <= 256): the next
    larger kernel build serves it, the missing columns read as zeros."""
    torch.manual_seed(D)
    B, H_Q, H_KV, N = 3, 8, 2, 77
    q = torch.randn(B, H_Q, 1, D).half()
    k = torch.randn(B, H_KV, N, D).half()
    v = torch.randn(B, H_KV, N, D).half()
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    out = fa.forward_decode_gqa_fp16(qc, kc, vc, True, 60)
    assert out.shape == q.shape
    assert _err(out, orc.decode_gqa(q, k, v, True, 60, final_cast=False)) < TOL
    lens = torch.tensor([0, 33, 76], dtype=torch.int32)
    out = fa.forward_continuous_batching_fp16(qc, kc, vc, lens.cuda(), True)
    assert _err(out, orc.continuous_batching_decode(q, k, v, lens, True, final_cast=False)) < TOL
    seq_lens = torch.tensor([5, 0, 77], dtype=torch.int32)
    kp, vp, bt, mnb = orc.build_paged_cache(k, v, seq_lens, [4, 1, 7, 0, 9, 3, 8, 2, 5, 6, 10, 11, 12, 13, 14])
    out = fa.forward_paged_decode_gqa_fp16(qc, kp.cuda(), vp.cuda(), bt.cuda(), seq_lens.cuda(), mnb)
    assert _err(out, orc.paged_decode(q, kp, vp, bt, seq_lens, final_cast=False)) < TOL
    out = fa.forward_decode_sliding_window_gqa(qc, kc, vc, True, 70, 24, 3)
    assert _err(out, orc.sliding_window_decode(q, k, v, True, 70, 24, 3, final_cast=False)) < TOL
    if D % 16 == 0:
        k8, ks = orc.quantize_kv_int8(k)
        v8, vs = orc.quantize_kv_int8(v)
        out = fa.forward_decode_int8_kv_cache_gqa(qc, k8.cuda(), v8.cuda(), ks.cuda(), vs.cuda(), 70)
        assert _err(out, orc.decode_int8_kv_cache_gqa(q, k8, v8, ks, vs, 70, final_cast=False)) < TOL
    qs = (q.abs().amax(-1).float().squeeze(-1) / 127).contiguous()
    ksc = (k.abs().amax(-1).float() / 127).contiguous()
    out, scores = fa.forward_decode_int8_gqa(qc, kc, vc, qs.cuda(), ksc.cuda(), 70, return_scores=True)
    ref_out, ref_dots = orc.decode_int8_gqa(q, k, v, qs, ksc, 70, final_cast=False)
    assert torch.equal(scores.cpu()[:, :, :71], ref_dots[:, :, :71])
    assert _err(out, ref_out) < TOL
    _finish(fa)


def test_bf16_output_variants_round_the_same_fp32_result(fa):
    """`out_dtype=torch.bfloat16` (paged decode, varlen prefill): the same fp32 result rounded once to
    bfloat16 - within one bfloat16 rounding (2^-9 relative) of the oracle's fp32 value plus the usual 2e-3."""
    w = orc.make_paged_workload(B=5, H_Q=32, H_KV=8, D=128, min_len=1, max_len=500, seed=3)
    args = (w["q"].cuda(), w["k_cache"].cuda(), w["v_cache"].cuda(), w["block_table"].cuda(), w["seq_lens"].cuda(),
            w["max_num_blocks"])
    out16 = fa.forward_paged_decode_gqa_fp16(*args)
    outb = fa.forward_paged_decode_gqa_fp16(*args, out_dtype=torch.bfloat16)
    assert outb.dtype == torch.bfloat16 and outb.shape == out16.shape
    ref = orc.paged_decode(w["q"], w["k_cache"], w["v_cache"], w["block_table"], w["seq_lens"], final_cast=False)
    tol = TOL + ref.abs() * 2.0 ** -8
    assert ((outb.float().cpu() - ref).abs() <= tol).all()
    assert (outb.float() - out16.float()).abs().max().item() < 2.0 ** -7      # two roundings of values below 2
    lens = [70, 1, 200, 33]
    cu = torch.tensor([0, 70, 71, 271, 304], dtype=torch.int32)
    g = torch.Generator().manual_seed(8)
    q = torch.randn(304, 8, 128, generator=g).half()
    k = torch.randn(304, 2, 128, generator=g).half()
    v = torch.randn(304, 2, 128, generator=g).half()
    for impl in (0, 1):                     # tcgen05 kernel and mma.sync kernel
        flash_attn_v100_b200_set_impl(impl)
        outb = fa.forward_varlen_prefill_fp16(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), max(lens), True,
                                              out_dtype=torch.bfloat16)
        ref = orc.varlen_prefill(q, k, v, cu, True, final_cast=False)
        assert outb.dtype == torch.bfloat16
        assert ((outb.float().cpu() - ref).abs() <= TOL + ref.abs() * 2.0 ** -8).all(), impl
    flash_attn_v100_b200_set_impl(0)
    _finish(fa)


def flash_attn_v100_b200_set_impl(impl):
    import flash_attn_v100_b200
    flash_attn_v100_b200.set_prefill_impl(impl)
