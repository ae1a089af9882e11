"""GPU: fused rotary embedding + KV append into pages.  Bit-exact against the reference module's
outputs (fixtures) and against the oracle; then a serving-shaped loop (prompt append, several decode
steps through the block manager) against dense attention."""
import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from test_kv_cache_cpu import ROPE_CASES, rope_case, rope_golden  # noqa: F401

pytestmark = pytest.mark.gpu


def test_rotation_bit_exact_against_reference_fixture(rope_golden):  # noqa: F811
    import flash_attn_v100_b200 as pkg
    for name, *_ in ROPE_CASES:
        q, k, rot, theta, pos = rope_case(rope_golden, name)
        cos = torch.from_numpy(rope_golden[f"{name}/cos"]).cuda()
        sin = torch.from_numpy(rope_golden[f"{name}/sin"]).cuda()
        v = torch.zeros_like(k)
        q_rot, k_rot = pkg.rope_append_paged_fp16(q.cuda(), k.cuda(), v.cuda(), cos, sin, None, None, None,
                                                   pos.int().cuda(), 0, return_k=True)
        assert torch.equal(q_rot.cpu(), torch.from_numpy(rope_golden[f"{name}/q"])), name
        assert torch.equal(k_rot.cpu(), torch.from_numpy(rope_golden[f"{name}/k"])), name
    pkg.check_prefill_errors()


@pytest.mark.parametrize("D,rot", [(128, 128), (64, 64), (128, 64), (256, 256)])
def test_packed_prompt_append_matches_oracle(D, rot):
    import flash_attn_v100_b200 as pkg
    H_Q, H_KV = 8, 2
    lens, start = [5, 33, 16, 1], [0, 7, 16, 31]          # prompts appended after `start` cached tokens
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    T = int(cu[-1])
    g = torch.Generator().manual_seed(D + rot)
    q = torch.randn(T, H_Q, D, generator=g).half()
    k = torch.randn(T, H_KV, D, generator=g).half()
    v = torch.randn(T, H_KV, D, generator=g).half()
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(start, lens)])
    cos, sin = orc.rope_cos_sin(pos, rot, 1e6)
    n_blocks = 16
    bt = torch.full((4, 4), -1, dtype=torch.int32)
    perm = torch.randperm(n_blocks, generator=g).int()
    cur = 0
    for b in range(4):
        nb = (start[b] + lens[b] + 15) // 16
        bt[b, :nb] = perm[cur:cur + nb]; cur += nb
    kc = torch.randn(n_blocks, H_KV, 16, D, generator=g).half()
    vc = torch.randn(n_blocks, H_KV, 16, D, generator=g).half()
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q_ref, k_ref = orc.apply_rotary_emb(q, k, cos[:, None, :], sin[:, None, :])
    for b in range(4):
        a = int(cu[b])
        orc.append_to_pages(kc_ref, vc_ref, bt, b, start[b], k_ref[a:a + lens[b]], v[a:a + lens[b]])
    kc_d, vc_d = kc.cuda(), vc.cuda()
    q_rot, k_rot = pkg.rope_append_paged_fp16(q.cuda(), k.cuda(), v.cuda(), cos.cuda(), sin.cuda(), kc_d, vc_d,
                                               bt.cuda(), torch.tensor(start, dtype=torch.int32).cuda(), 4,
                                               cu_seqlens=cu.cuda(), return_k=True)
    assert torch.equal(q_rot.cpu(), q_ref) and torch.equal(k_rot.cpu(), k_ref)
    assert torch.equal(kc_d.cpu(), kc_ref) and torch.equal(vc_d.cpu(), vc_ref)      # untouched slots unchanged
    pkg.check_prefill_errors()


def test_token_without_a_page_is_reported():
    import flash_attn_v100_b200 as pkg
    q = torch.randn(1, 4, 1, 64).half().cuda(); k = torch.randn(1, 2, 1, 64).half().cuda()
    cos, sin = orc.rope_cos_sin(torch.tensor([40]), 64)
    kc = torch.zeros(2, 2, 16, 64, dtype=torch.float16, device="cuda")
    bt = torch.tensor([[0, -1]], dtype=torch.int32, device="cuda")      # slot 40 needs a third block
    pkg.rope_append_paged_fp16(q, k, k, cos.cuda(), sin.cuda(), kc, kc.clone(), bt,
                               torch.tensor([40], dtype=torch.int32).cuda(), 2)
    with pytest.raises(RuntimeError, match="device status"):
        pkg.check_prefill_errors()
    pkg.check_prefill_errors()      # cleared by the previous read


def test_serving_loop_prompt_then_decode_steps():
    """Two requests: packed prompt prefill through the block manager, then 20 decode steps
    (rope+append, paged decode).  Every step is compared with dense fp32 attention over the rotated
    keys kept on the host."""
    import flash_attn_v100 as fa
    import flash_attn_v100_b200 as pkg
    H_Q, H_KV, D, theta = 8, 2, 128, 1e6
    kv = pkg.PagedKVCache(num_blocks=32, num_layers=1, num_kv_heads=H_KV, head_dim=D, max_batch=2, max_blocks_per_seq=8)
    g = torch.Generator().manual_seed(9)
    prompts = {"r0": 37, "r1": 16}
    ids = list(prompts)
    for r, n in prompts.items():
        kv.allocate(r, n)
    lens = [prompts[r] for r in ids]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    T = int(cu[-1])
    q = torch.randn(T, H_Q, D, generator=g).half(); k = torch.randn(T, H_KV, D, generator=g).half()
    v = torch.randn(T, H_KV, D, generator=g).half()
    pos = torch.cat([torch.arange(n) for n in lens])
    cos, sin = orc.rope_cos_sin(pos, D, theta)
    q_rot, k_rot = kv.append_prefill(0, ids, q.cuda(), k.cuda(), v.cuda(), cos.cuda(), sin.cuda(), cu.cuda())
    out = fa.forward_varlen_prefill_fp16(q_rot, k_rot, v.cuda(), cu.cuda(), max(lens), True)
    for r, n in prompts.items():
        kv.commit(r, n)
    q_ref, k_ref = orc.apply_rotary_emb(q, k, cos[:, None, :], sin[:, None, :])
    ref = orc.varlen_prefill(q_ref, k_ref, v, cu, True, final_cast=False)
    assert (out.float().cpu() - ref).abs().max().item() < 2e-3
    hist_k = [k_ref[int(cu[i]):int(cu[i + 1])] for i in range(2)]
    hist_v = [v[int(cu[i]):int(cu[i + 1])] for i in range(2)]
    for step in range(20):
        for r in ids:
            kv.reserve(r, kv.get_cache_len(r) + 1)
        qn = torch.randn(2, H_Q, 1, D, generator=g).half(); kn = torch.randn(2, H_KV, 1, D, generator=g).half()
        vn = torch.randn(2, H_KV, 1, D, generator=g).half()
        posn = torch.tensor([kv.get_cache_len(r) for r in ids])
        cosn, sinn = orc.rope_cos_sin(posn, D, theta)
        q_rot = kv.append_decode(0, ids, qn.cuda(), kn.cuda(), vn.cuda(), cosn.cuda(), sinn.cuda())
        for r in ids:
            kv.commit(r, 1)
        table, seq_lens = kv.batch_view(ids)
        out = fa.forward_paged_decode_gqa_fp16(q_rot, kv.k_pools[0], kv.v_pools[0], table, seq_lens, kv.max_blocks_per_seq)
        qr, kr = orc.apply_rotary_emb(qn, kn, cosn.view(2, 1, 1, D), sinn.view(2, 1, 1, D))
        assert torch.equal(q_rot.cpu(), qr)
        for i in range(2):
            hist_k[i] = torch.cat([hist_k[i], kr[i].transpose(0, 1)])
            hist_v[i] = torch.cat([hist_v[i], vn[i].transpose(0, 1)])
            n = hist_k[i].size(0)
            refd = orc.decode_gqa(qr[i:i + 1], hist_k[i].transpose(0, 1)[None], hist_v[i].transpose(0, 1)[None],
                                  True, n - 1, final_cast=False)
            assert (out[i:i + 1].float().cpu() - refd).abs().max().item() < 2e-3, (step, i)
    torch.cuda.synchronize()
    pkg.check_async_errors(); pkg.check_prefill_errors()
    kv.release("r0"); kv.release("r1")
    assert kv.get_num_free_blocks() == 32
