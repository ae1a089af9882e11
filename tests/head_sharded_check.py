"""Run under torchrun with >= 2 ranks: ONE batch split over the ranks by KV-head group
(the reference's multi-GPU partition, tensor_parallel.py:435-457, :553-571, :593).  Every rank runs the
operators on its own heads only; the per-rank outputs, put side by side, must equal the CPU oracle on the
full batch (the check of test_multi_gpu.py:672-727: tensor parallel == single GPU).  No collective takes part
in the attention itself; the gather below only brings the slices together for the comparison."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import flash_attn_v100 as fa  # noqa: E402
import flash_attn_v100_b200  # noqa: E402
from flash_attn_v100_b200.sharding import shard_decode_inputs, shard_heads, head_shard  # noqa: E402
from oracle import attention_oracle as orc  # noqa: E402

TOL = 2e-3


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    H_Q, H_KV, D = 32, 8, 128

    # ---- paged decode: the same seeded batch on every rank (host), each rank keeps its heads ----
    w = orc.make_paged_workload(B=7, H_Q=H_Q, H_KV=H_KV, D=D, min_len=1, max_len=700, seed=41)
    q_r, k_r, v_r, shard = shard_decode_inputs(w["q"], w["k_cache"], w["v_cache"], rank, world)
    out_r = fa.forward_paged_decode_gqa_fp16(q_r.to(dev), k_r.to(dev), v_r.to(dev), w["block_table"].to(dev),
                                             w["seq_lens"].to(dev), w["max_num_blocks"])
    parts = [torch.empty_like(out_r) for _ in range(world)]
    dist.all_gather(parts, out_r.contiguous())
    full = torch.cat(parts, dim=1).float().cpu()
    ref = orc.paged_decode(w["q"], w["k_cache"], w["v_cache"], w["block_table"], w["seq_lens"], final_cast=False)
    err = (full - ref).abs().max().item()
    ok &= err < TOL
    if rank == 0:
        print(f"paged decode, {world} head shards: max-abs-err vs oracle {err:.2e}", flush=True)

    # ---- varlen causal prefill: packed q [T, H_Q, D], k / v [T, H_KV, D] split along the head axis ----
    lens = [130, 1, 77, 300]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    g = torch.Generator().manual_seed(42)
    T = sum(lens)
    q = torch.randn(T, H_Q, D, generator=g).half()
    k = torch.randn(T, H_KV, D, generator=g).half()
    v = torch.randn(T, H_KV, D, generator=g).half()
    s = head_shard(H_Q, H_KV, rank, world)
    out_p = fa.forward_varlen_prefill_fp16(shard_heads(q, *s.q_heads).to(dev), shard_heads(k, *s.kv_heads).to(dev),
                                           shard_heads(v, *s.kv_heads).to(dev), cu.to(dev), max(lens), True)
    parts = [torch.empty_like(out_p) for _ in range(world)]
    dist.all_gather(parts, out_p.contiguous())
    full = torch.cat(parts, dim=1).float().cpu()
    ref = orc.varlen_prefill(q, k, v, cu, True, final_cast=False)
    err = (full - ref).abs().max().item()
    ok &= err < TOL
    if rank == 0:
        print(f"varlen prefill, {world} head shards: max-abs-err vs oracle {err:.2e}", flush=True)

    torch.cuda.synchronize()
    flash_attn_v100_b200.check_async_errors()
    flash_attn_v100_b200.check_prefill_errors()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("HEAD_SHARDED_OK" if int(flag.item()) == 1 else "HEAD_SHARDED_MISMATCH", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
