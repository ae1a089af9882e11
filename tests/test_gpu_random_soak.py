"""GPU: randomly drawn shapes (seeded) of the paged decode and the varlen prefill, fp16 and bfloat16, against
the oracle.  The fixed cases of the other test files are chosen by hand around known boundaries; these cover
combinations nobody thought of (batch sizes, group sizes, head dimensions, lengths from empty to several
thousand tokens, so that CTAs hold one piece, several pieces, or parts of split segments)."""
import random

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


def rel_err(out, ref):
    return ((out.float().cpu() - ref).abs() / (1.0 + ref.abs())).max().item()


def test_paged_decode_random_shapes_match_oracle():
    import flash_attn_v100 as fa
    import flash_attn_v100_b200 as pkg
    rng = random.Random(1)
    for it in range(120):
        B = rng.choice([1, 2, 3, 5, 8, 17])
        H_KV = rng.choice([1, 2, 4, 8])
        G = rng.choice([1, 2, 4, 8, 12, 16])
        D = rng.choice([64, 128])
        max_len = rng.choice([40, 300, 1500, 5000])
        min_len = rng.choice([0, 1, max_len // 2])
        w = orc.make_paged_workload(B=B, H_Q=H_KV * G, H_KV=H_KV, D=D, min_len=min_len, max_len=max_len, seed=1000 + it)
        bf = rng.random() < 0.3
        q, kc, vc = w["q"], w["k_cache"], w["v_cache"]
        if bf:
            q, kc, vc = q.bfloat16(), kc.bfloat16(), vc.bfloat16()
        f = fa.forward_paged_decode_gqa_bf16 if bf else fa.forward_paged_decode_gqa_fp16
        out = f(q.cuda(), kc.cuda(), vc.cuda(), w["block_table"].cuda(), w["seq_lens"].cuda(), w["max_num_blocks"])
        ref = orc.paged_decode(q, kc, vc, w["block_table"], w["seq_lens"], final_cast=False)
        err = rel_err(out, ref)
        assert err < (1e-2 if bf else 2e-3), (it, B, H_KV, G, D, w["seq_lens"].tolist()[:8], bf, err)
    pkg.check_async_errors()


def test_varlen_prefill_random_shapes_match_oracle():
    import flash_attn_v100 as fa
    import flash_attn_v100_b200 as pkg
    rng = random.Random(2)
    for it in range(60):
        nseq = rng.choice([1, 2, 3, 5])
        H_KV = rng.choice([1, 2, 4])
        G = rng.choice([1, 2, 3, 4, 8])
        D = rng.choice([64, 128, 96])
        lens = [rng.choice([1, 17, 127, 128, 129, 255, 256, 257, 400, 700]) for _ in range(nseq)]
        causal = rng.random() < 0.7
        bf = rng.random() < 0.4
        g = torch.Generator().manual_seed(500 + it)
        T = sum(lens)
        dt = torch.bfloat16 if bf else torch.float16
        q = torch.randn(T, H_KV * G, D, generator=g).to(dt)
        k = torch.randn(T, H_KV, D, generator=g).to(dt)
        v = torch.randn(T, H_KV, D, generator=g).to(dt)
        cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
        f = fa.forward_varlen_prefill_bf16 if bf else fa.forward_varlen_prefill_fp16
        out = f(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), max(lens), causal)
        ref = orc.varlen_prefill(q, k, v, cu, causal=causal, final_cast=False)
        err = rel_err(out, ref)
        assert err < (1e-2 if bf else 2e-3), (it, lens, H_KV, G, D, causal, bf, err)
    pkg.check_prefill_errors()


def test_other_decode_operators_random_shapes_match_oracle():
    """INT8-QK (int32 dots bit-exact), INT8-KV cache, sliding window + sink, continuous batching and the
    contiguous decode on seeded random shapes."""
    import flash_attn_v100 as fa
    import flash_attn_v100_b200 as pkg
    rng = random.Random(3)
    for it in range(60):
        B = rng.choice([1, 2, 3, 6])
        H_KV = rng.choice([1, 2, 8])
        G = rng.choice([1, 2, 4, 8])
        H_Q = H_KV * G
        D = rng.choice([64, 128])
        N = rng.choice([17, 64, 130, 700, 2100])
        cache_len = rng.choice([0, N // 3, N - 1])
        g = torch.Generator().manual_seed(7000 + it)
        q = torch.randn(B, H_Q, 1, D, generator=g).half()
        k = torch.randn(B, H_KV, N, D, generator=g).half()
        v = torch.randn(B, H_KV, N, D, generator=g).half()
        kind = it % 5
        what = (it, kind, B, H_Q, H_KV, N, D, cache_len)
        if kind == 0:      # INT8-QK
            qs = (q.abs().amax(-1).float().squeeze(-1) / 127).contiguous()
            ks = (k.abs().amax(-1).float() / 127).contiguous()
            out, scores = fa.forward_decode_int8_gqa(q.cuda(), k.cuda(), v.cuda(), qs.cuda(), ks.cuda(), cache_len,
                                                     return_scores=True)
            ref, dots = orc.decode_int8_gqa(q, k, v, qs, ks, cache_len, final_cast=False)
            assert torch.equal(scores.cpu()[:, :, :cache_len + 1], dots[:, :, :cache_len + 1]), what
            assert rel_err(out, ref) < 2e-3, what
        elif kind == 1:    # INT8 KV cache
            k8, ksc = orc.quantize_kv_int8(k)
            v8, vsc = orc.quantize_kv_int8(v)
            out = fa.forward_decode_int8_kv_cache_gqa(q.cuda(), k8.cuda(), v8.cuda(), ksc.cuda(), vsc.cuda(), cache_len)
            ref = orc.decode_int8_kv_cache_gqa(q, k8, v8, ksc, vsc, cache_len, final_cast=False)
            assert rel_err(out, ref) < 2e-3, what
        elif kind == 2:    # sliding window + sink
            window, sink = rng.choice([1, 16, 100, 5000]), rng.choice([0, 3, 16, 40])
            out = fa.forward_decode_sliding_window_gqa(q.cuda(), k.cuda(), v.cuda(), True, cache_len, window, sink)
            ref = orc.sliding_window_decode(q, k, v, True, cache_len, window, sink, final_cast=False)
            assert rel_err(out, ref) < 2e-3, what + (window, sink)
        elif kind == 3:    # continuous batching: one cache length per sequence
            lens = torch.tensor([rng.randrange(0, N) for _ in range(B)], dtype=torch.int32)
            out = fa.forward_continuous_batching_fp16(q.cuda(), k.cuda(), v.cuda(), lens.cuda(), True)
            ke, ve = orc.expand_kv_heads(k, v, H_Q)
            ref = orc.sdpa_decode(q, ke, ve, lens + 1, final_cast=False)
            assert rel_err(out, ref) < 2e-3, what + (lens.tolist(),)
        else:              # contiguous decode
            out = fa.forward_decode_gqa_fp16(q.cuda(), k.cuda(), v.cuda(), True, cache_len)
            ke, ve = orc.expand_kv_heads(k, v, H_Q)
            ref = orc.sdpa_decode(q, ke, ve, torch.tensor([cache_len + 1] * B), final_cast=False)
            assert rel_err(out, ref) < 2e-3, what
    pkg.check_async_errors()
