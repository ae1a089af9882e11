"""CPU, world_size 2 over gloo: the head-shard rule partitions a decode batch so that the
per-rank results (computed here by the oracle, since there is no GPU) concatenate to the
full result, with no exchange other than the final gather."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_attn_v100_b200.sharding import gather_head_outputs, head_shard, shard_decode_inputs


def test_head_shard_rule_matches_reference_partition():
    s = head_shard(32, 8, 3, 8)
    assert s.q_heads == (12, 16) and s.kv_heads == (3, 4)       # TP=8: 4 Q heads + 1 KV head per rank
    s = head_shard(32, 8, 1, 2)
    assert s.q_heads == (16, 32) and s.kv_heads == (4, 8)
    # every query head's KV head lives on the same rank
    for world in (1, 2, 4, 8):
        for r in range(world):
            s = head_shard(32, 8, r, world)
            for hq in range(*s.q_heads):
                assert s.kv_heads[0] <= hq // 4 < s.kv_heads[1]
    with pytest.raises(ValueError):
        head_shard(32, 8, 0, 3)
    with pytest.raises(ValueError):
        head_shard(32, 8, 2, 2)


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import attention_oracle as orc
        torch.manual_seed(0)                                       # same full tensors on every rank
        B, H_Q, H_KV, N, D = 3, 8, 4, 37, 64
        q = torch.randn(B, H_Q, 1, D).half()
        k = torch.randn(B, H_KV, N, D).half()
        v = torch.randn(B, H_KV, N, D).half()
        lens = torch.tensor([5, 36, 17], dtype=torch.int32)
        ql, kl, vl, s = shard_decode_inputs(q, k, v, rank, world)
        local = orc.continuous_batching_decode(ql, kl, vl, lens, True, final_cast=False)
        full = gather_head_outputs(local, world)
        ref = orc.continuous_batching_decode(q, k, v, lens, True, final_cast=False)
        ok = torch.equal(full, ref) and torch.equal(local, ref[:, s.q_heads[0]:s.q_heads[1]])
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_rank_head_sharded_decode_equals_full():
    world = 2
    port = 29600 + (os.getpid() % 300)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert ret.get(0) is True and ret.get(1) is True
