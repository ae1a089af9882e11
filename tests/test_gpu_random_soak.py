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
