"""GPU: the bfloat16 twins of the decode / prefill / rope operators against the same oracles as the fp16
operators, evaluated in fp32 on the bfloat16 inputs.  Tolerance: the result is rounded to bfloat16 (8-bit
mantissa: 2^-9 = 2e-3 relative from that rounding alone) and P enters the P V product as bfloat16, so the bound
is 1e-2 relative to 1 + |reference| (the fp16 operators are held to 2e-3)."""
import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from test_kv_cache_cpu import ROPE_CASES, rope_golden  # noqa: F401

pytestmark = pytest.mark.gpu
TOL = 1e-2


def rel_err(out, ref):
    return ((out.float().cpu() - ref).abs() / (1.0 + ref.abs())).max().item()


@pytest.mark.parametrize("B,H_Q,H_KV,D,lens", [
    (3, 8, 2, 128, [1, 100, 777]), (2, 32, 8, 128, [2048, 513]), (4, 4, 4, 64, [16, 17, 0, 300]),
    (2, 40, 2, 128, [300, 31]), (1, 8, 1, 256, [500]), (2, 6, 2, 96, [129, 64])])
def test_paged_decode_bf16_matches_oracle(B, H_Q, H_KV, D, lens):
    import flash_attn_v100 as fa
    g = torch.Generator().manual_seed(B * 1000 + D)
    max_len = max(max(lens), 1)
    q = torch.randn(B, H_Q, 1, D, generator=g).bfloat16()
    k = torch.randn(B, H_KV, max_len, D, generator=g).bfloat16()
    v = torch.randn(B, H_KV, max_len, D, generator=g).bfloat16()
    seq_lens = torch.tensor(lens, dtype=torch.int32)
    n_blocks = sum((n + 15) // 16 for n in lens) + 3
    order = torch.randperm(n_blocks, generator=g).tolist()
    kc, vc, bt, mnb = orc.build_paged_cache(k, v, seq_lens, order, n_blocks)
    kc = kc + 0  # pages that no sequence uses hold whatever they hold
    out = fa.forward_paged_decode_gqa_bf16(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), seq_lens.cuda(), mnb)
    assert out.dtype == torch.bfloat16 and out.shape == q.shape
    ref = orc.paged_decode(q, kc, vc, bt, seq_lens, final_cast=False)
    assert rel_err(out, ref) < TOL
    # the fp16 entry point refuses bfloat16 tensors, as the reference's does
    with pytest.raises(RuntimeError):
        fa.forward_paged_decode_gqa_fp16(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), seq_lens.cuda(), mnb)
    with pytest.raises(RuntimeError):
        fa.forward_paged_decode_gqa_bf16(q.half().cuda(), kc.cuda(), vc.cuda(), bt.cuda(), seq_lens.cuda(), mnb)
    import flash_attn_v100_b200 as pkg
    pkg.check_async_errors()


@pytest.mark.parametrize("B,H_Q,H_KV,N,D,cache_len", [(2, 8, 2, 300, 128, 299), (1, 32, 8, 1000, 128, 511),
                                                      (3, 4, 1, 64, 64, 0)])
def test_contiguous_decode_bf16_matches_oracle(B, H_Q, H_KV, N, D, cache_len):
    import flash_attn_v100 as fa
    g = torch.Generator().manual_seed(N + D)
    q = torch.randn(B, H_Q, 1, D, generator=g).bfloat16()
    k = torch.randn(B, H_KV, N, D, generator=g).bfloat16()
    v = torch.randn(B, H_KV, N, D, generator=g).bfloat16()
    out = fa.forward_decode_gqa_bf16(q.cuda(), k.cuda(), v.cuda(), True, cache_len)
    ke, ve = orc.expand_kv_heads(k, v, H_Q)
    ref = orc.sdpa_decode(q, ke, ve, torch.tensor([cache_len + 1] * B), final_cast=False)
    assert out.dtype == torch.bfloat16 and rel_err(out, ref) < TOL


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("H_Q,H_KV,D,lens", [(8, 2, 128, [300, 129, 1000, 1]), (4, 4, 64, [128, 257, 77]),
                                             (6, 2, 96, [200, 40])])
def test_varlen_prefill_bf16_matches_oracle(causal, H_Q, H_KV, D, lens):
    import flash_attn_v100 as fa
    import flash_attn_v100_b200 as pkg
    g = torch.Generator().manual_seed(sum(lens) + D)
    T = sum(lens)
    q = torch.randn(T, H_Q, D, generator=g).bfloat16()
    k = torch.randn(T, H_KV, D, generator=g).bfloat16()
    v = torch.randn(T, H_KV, D, generator=g).bfloat16()
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    out = fa.forward_varlen_prefill_bf16(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), max(lens), causal)
    ref = orc.varlen_prefill(q, k, v, cu, causal=causal, final_cast=False)
    assert out.dtype == torch.bfloat16 and rel_err(out, ref) < TOL
    pkg.check_prefill_errors()


def test_dense_prefill_bf16_matches_oracle_and_large_head_dim_is_refused():
    import flash_attn_v100 as fa
    g = torch.Generator().manual_seed(3)
    q = torch.randn(2, 8, 260, 128, generator=g).bfloat16()
    k = torch.randn(2, 2, 260, 128, generator=g).bfloat16()
    v = torch.randn(2, 2, 260, 128, generator=g).bfloat16()
    out = fa.forward_prefill_gqa_bf16(q.cuda(), k.cuda(), v.cuda(), True)
    ref = orc.prefill_gqa(q, k, v, causal=True, final_cast=False)
    assert out.dtype == torch.bfloat16 and rel_err(out, ref) < TOL
    q2 = torch.randn(1, 2, 64, 256).bfloat16().cuda()
    with pytest.raises(RuntimeError):          # bfloat16 prefill runs on the tcgen05 kernel: head dimension <= 128
        fa.forward_prefill_gqa_bf16(q2, q2, q2, True)


def test_rope_append_bf16_bit_exact_against_reference_fixture(rope_golden):  # noqa: F811
    import flash_attn_v100_b200 as pkg
    from flash_attn_v100_b200 import ops
    for name, B, H_Q, H_KV, D, theta, prf, positions in ROPE_CASES:
        torch.manual_seed(77)
        q = torch.randn(B, H_Q, 1, D).bfloat16()
        k = torch.randn(B, H_KV, 1, D).bfloat16()
        cos = torch.from_numpy(rope_golden[f"{name}/cos"]).cuda()
        sin = torch.from_numpy(rope_golden[f"{name}/sin"]).cuda()
        q_rot, k_rot = ops.rope_append_paged_bf16(q.cuda(), k.cuda(), torch.zeros_like(k).cuda(), cos, sin, None, None,
                                                  None, torch.tensor(positions, dtype=torch.int32).cuda(), 0,
                                                  return_k=True)
        assert np.array_equal(q_rot.cpu().view(torch.int16).numpy(), rope_golden[f"{name}/q_bf16"]), name
        assert np.array_equal(k_rot.cpu().view(torch.int16).numpy(), rope_golden[f"{name}/k_bf16"]), name
    pkg.check_prefill_errors()


def test_rope_append_bf16_writes_pages_like_the_oracle():
    from flash_attn_v100_b200 import ops
    H_Q, H_KV, D = 8, 2, 128
    lens, start = [5, 33, 16], [0, 7, 16]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    T = int(cu[-1])
    g = torch.Generator().manual_seed(9)
    q = torch.randn(T, H_Q, D, generator=g).bfloat16()
    k = torch.randn(T, H_KV, D, generator=g).bfloat16()
    v = torch.randn(T, H_KV, D, generator=g).bfloat16()
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(start, lens)])
    cos, sin = orc.rope_cos_sin(pos, D, 1e6)
    bt = torch.tensor([[3, -1, -1], [0, 5, 7], [1, 2, -1]], dtype=torch.int32)
    kc = torch.randn(8, H_KV, 16, D, generator=g).bfloat16()
    vc = torch.randn(8, H_KV, 16, D, generator=g).bfloat16()
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q_ref, k_ref = orc.apply_rotary_emb(q, k, cos[:, None, :], sin[:, None, :])
    for b in range(3):
        a = int(cu[b])
        orc.append_to_pages(kc_ref, vc_ref, bt, b, start[b], k_ref[a:a + lens[b]], v[a:a + lens[b]])
    kc_d, vc_d = kc.cuda(), vc.cuda()
    q_rot, k_rot = ops.rope_append_paged_bf16(q.cuda(), k.cuda(), v.cuda(), cos.cuda(), sin.cuda(), kc_d, vc_d, bt.cuda(),
                                              torch.tensor(start, dtype=torch.int32).cuda(), 3, cu_seqlens=cu.cuda(),
                                              return_k=True)
    assert torch.equal(q_rot.cpu(), q_ref) and torch.equal(k_rot.cpu(), k_ref)
    assert torch.equal(kc_d.cpu(), kc_ref) and torch.equal(vc_d.cpu(), vc_ref)
