"""CPU: block-manager bookkeeping and the rotary oracle against the reference's own outputs."""
import numpy as np
import pytest
import torch

from flash_attn_v100_b200.kv_cache import PagedKVCache
from oracle import attention_oracle as orc
import golden_cases as gc

ROPE_CASES = [  # tests/golden/make_golden_rope.py
    ("qwen3_like", 3, 32, 8, 128, 1e6, 1.0, [0, 17, 4095]),
    ("llama_d64", 2, 8, 2, 64, 1e4, 1.0, [1, 1000]),
    ("partial", 2, 4, 4, 128, 1e4, 0.5, [7, 300]),
]


@pytest.fixture(scope="module")
def rope_golden():
    import os
    return np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_rope_outputs.npz"))


def rope_case(rope_golden, name):
    for n, B, H_Q, H_KV, D, theta, prf, positions in ROPE_CASES:
        if n == name:
            torch.manual_seed(77)
            q = torch.randn(B, H_Q, 1, D).half()
            k = torch.randn(B, H_KV, 1, D).half()
            assert gc.digest(q, k) == str(rope_golden[f"{name}/digest"])
            return q, k, int(D * prf), theta, torch.tensor(positions)
    raise KeyError(name)


def test_rope_oracle_is_bit_identical_to_reference_module(rope_golden):
    for name, *_ in ROPE_CASES:
        q, k, rot, theta, pos = rope_case(rope_golden, name)
        cos, sin = orc.rope_cos_sin(pos, rot, theta)
        assert np.array_equal(cos.numpy(), rope_golden[f"{name}/cos"].reshape(cos.shape))
        assert np.array_equal(sin.numpy(), rope_golden[f"{name}/sin"].reshape(sin.shape))
        qe, ke = orc.apply_rotary_emb(q, k, cos.view(-1, 1, 1, rot), sin.view(-1, 1, 1, rot))
        assert torch.equal(qe, torch.from_numpy(rope_golden[f"{name}/q"]))
        assert torch.equal(ke, torch.from_numpy(rope_golden[f"{name}/k"]))


def test_block_manager_alloc_reserve_release():
    kv = PagedKVCache(num_blocks=6, num_layers=2, num_kv_heads=2, head_dim=64, max_batch=3, max_blocks_per_seq=4,
                      device="cpu")
    assert kv.get_num_free_blocks() == 6 and kv.can_allocate(96) and not kv.can_allocate(97)
    r0 = kv.allocate("a", 17)                     # 2 blocks
    assert kv.get_block_table("a") == [0, 1] and kv.get_num_free_blocks() == 4
    assert kv.block_table[r0].tolist() == [0, 1, -1, -1]
    kv.commit("a", 17)
    kv.reserve("a", 32)                            # still 2 blocks
    assert kv.get_block_table("a") == [0, 1]
    kv.reserve("a", 33)                            # third block, only the new entry is written
    assert kv.get_block_table("a") == [0, 1, 2] and kv.block_table[r0].tolist() == [0, 1, 2, -1]
    r1 = kv.allocate("b", 40)                      # 3 blocks -> pool empty
    assert kv.get_num_free_blocks() == 0 and r1 != r0
    with pytest.raises(MemoryError):
        kv.allocate("c", 1)
    assert "c" not in kv._tables and len(kv._free_rows) == 1        # failed allocation leaves no trace
    with pytest.raises(MemoryError):
        kv.reserve("a", 100)                       # beyond max_blocks_per_seq
    with pytest.raises(ValueError):
        kv.commit("b", 49)
    kv.release("a")
    assert kv.get_num_free_blocks() == 3 and kv.block_table[r0].tolist() == [-1] * 4
    # LIFO: the block freed last is handed out first
    r2 = kv.allocate("c", 16)
    assert kv.get_block_table("c") == [0]
    table, lens = kv.batch_view(["b", "c"])
    assert lens.tolist() == [0, 0] and table.shape == (2, 4)
    kv.commit("b", 40)
    assert kv.batch_view(["b"], extra_tokens=1)[1].tolist() == [41]
    with pytest.raises(ValueError):
        kv.allocate("b", 1)
