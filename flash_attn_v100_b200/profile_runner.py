"""Run a handful of launches of one kernel on a small case, for `ncu`.

    python -m flash_attn_v100_b200.profile_runner --case paged_decode --batch 16 --iters 3

The case keeps a few hundred MB on the device (more than L2, so DRAM counters mean
something) and launches the kernel `iters` times after one warm-up call.
(The reference has the same kind of one-shot runner for its profiler: tp_profile_runner.py.)
"""
from __future__ import annotations

import argparse

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="paged_decode",
                    choices=["paged_decode", "int8_decode", "varlen_prefill", "contig_decode", "int8_kv_decode",
                             "sliding_window_decode"])
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    import flash_attn_v100 as fa
    import flash_attn_v100_b200
    from flash_attn_v100_b200.synthetic import make_paged_tables
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(args.seed)
    H_Q, H_KV, D = 32, 8, 128
    if args.case == "paged_decode":
        t = make_paged_tables(args.batch, 512, 8192, args.seed)
        kc = torch.randn(t["n_pages"], H_KV, 16, D, generator=g, device=dev, dtype=torch.float16)
        vc = torch.randn(t["n_pages"], H_KV, 16, D, generator=g, device=dev, dtype=torch.float16)
        q = torch.randn(args.batch, H_Q, 1, D, generator=g, device=dev, dtype=torch.float16)
        bt, sl = t["block_table"].to(dev), t["seq_lens"].to(dev)
        run = lambda: fa.forward_paged_decode_gqa_fp16(q, kc, vc, bt, sl, t["max_num_blocks"])
        tokens = int(t["seq_lens"].sum())
        print(f"case paged_decode: B={args.batch} tokens={tokens} kv_bytes={tokens * 4096}")
    elif args.case in ("int8_decode", "contig_decode"):
        N = 4096
        q = torch.randn(args.batch, H_Q, 1, D, generator=g, device=dev, dtype=torch.float16)
        k = torch.randn(args.batch, H_KV, N, D, generator=g, device=dev, dtype=torch.float16)
        v = torch.randn(args.batch, H_KV, N, D, generator=g, device=dev, dtype=torch.float16)
        if args.case == "int8_decode":
            qs = (q.abs().amax(-1).float().squeeze(-1) / 127).contiguous()
            ks = (k.abs().amax(-1).float() / 127).contiguous()
            run = lambda: fa.forward_decode_int8_gqa(q, k, v, qs, ks, N - 1)
        else:
            run = lambda: fa.forward_decode_gqa_fp16(q, k, v, True, N - 1)
        print(f"case {args.case}: B={args.batch} N={N} kv_bytes={args.batch * H_KV * N * D * 4}")
    elif args.case == "int8_kv_decode":
        N = 8192
        q = torch.randn(args.batch, H_Q, 1, D, generator=g, device=dev, dtype=torch.float16)
        k8 = torch.randint(-127, 128, (args.batch, H_KV, N, D), generator=g, device=dev, dtype=torch.int8)
        v8 = torch.randint(-127, 128, (args.batch, H_KV, N, D), generator=g, device=dev, dtype=torch.int8)
        ks = (torch.rand(args.batch, H_KV, N, generator=g, device=dev) * 0.01 + 0.02).half()
        vs = (torch.rand(args.batch, H_KV, N, generator=g, device=dev) * 0.01 + 0.02).half()
        run = lambda: fa.forward_decode_int8_kv_cache_gqa(q, k8, v8, ks, vs, N - 1)
        print(f"case int8_kv_decode: B={args.batch} N={N} kv_bytes={args.batch * H_KV * N * (D * 2 + 4)}")
    elif args.case == "sliding_window_decode":
        N, window, sink = 8192, 4096, 4
        q = torch.randn(args.batch, H_Q, 1, D, generator=g, device=dev, dtype=torch.float16)
        k = torch.randn(args.batch, H_KV, N, D, generator=g, device=dev, dtype=torch.float16)
        v = torch.randn(args.batch, H_KV, N, D, generator=g, device=dev, dtype=torch.float16)
        run = lambda: fa.forward_decode_sliding_window_gqa(q, k, v, True, N - 1, window, sink)
        print(f"case sliding_window_decode: B={args.batch} N={N} window={window} sink={sink} "
              f"kv_bytes={args.batch * H_KV * (window + 16) * D * 4}")
    else:
        gl = torch.Generator().manual_seed(args.seed)
        lens = torch.randint(128, 4097, (args.batch,), generator=gl).tolist()
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        total = cu[-1]
        q = torch.randn(total, H_Q, D, generator=g, device=dev, dtype=torch.float16)
        k = torch.randn(total, H_KV, D, generator=g, device=dev, dtype=torch.float16)
        v = torch.randn(total, H_KV, D, generator=g, device=dev, dtype=torch.float16)
        cut = torch.tensor(cu, dtype=torch.int32, device=dev)
        run = lambda: fa.forward_varlen_prefill_fp16(q, k, v, cut, max(lens), True)
        flops = sum(4 * H_Q * D * n * (n + 1) // 2 for n in lens)
        print(f"case varlen_prefill: seqs={args.batch} total={total} flops={flops}")
    run()
    torch.cuda.synchronize()
    for _ in range(args.iters):
        run()
    torch.cuda.synchronize()
    flash_attn_v100_b200.check_async_errors()
    print("done")


if __name__ == "__main__":
    main()
