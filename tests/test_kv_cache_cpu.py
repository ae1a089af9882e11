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


def test_rope_oracle_on_bfloat16_is_bit_identical_to_reference_module(rope_golden):
    """The pin of the *_bf16 twins: the reference module evaluated on bfloat16 tensors."""
    for name, B, H_Q, H_KV, D, theta, prf, positions in ROPE_CASES:
        torch.manual_seed(77)
        q = torch.randn(B, H_Q, 1, D).bfloat16()
        k = torch.randn(B, H_KV, 1, D).bfloat16()
        assert gc.digest(q.view(torch.int16), k.view(torch.int16)) == str(rope_golden[f"{name}/digest_bf16"])
        rot = int(D * prf)
        cos, sin = orc.rope_cos_sin(torch.tensor(positions), rot, theta)
        qe, ke = orc.apply_rotary_emb(q, k, cos.view(-1, 1, 1, rot), sin.view(-1, 1, 1, rot))
        assert qe.dtype == torch.bfloat16
        assert np.array_equal(qe.view(torch.int16).numpy(), rope_golden[f"{name}/q_bf16"])
        assert np.array_equal(ke.view(torch.int16).numpy(), rope_golden[f"{name}/k_bf16"])


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


def _mk(num_blocks=12, **kw):
    return PagedKVCache(num_blocks=num_blocks, num_layers=1, num_kv_heads=1, head_dim=64, max_batch=4,
                        max_blocks_per_seq=8, device="cpu", **kw)


def _check_accounting(kv):
    """Every block is either free exactly once or held; reference counts match the holders."""
    free = kv._free
    assert len(free) == len(set(free))
    held = [0] * kv.num_blocks
    for table in kv._tables.values():
        for b in table:
            if b >= 0:
                held[b] += 1
    for blocks in kv._prefix_cache.values():
        for b in blocks:
            held[b] += 1
    assert held == kv._refs
    assert sorted(free) == [b for b in range(kv.num_blocks) if held[b] == 0]
    for rid, row in kv._row.items():
        t = kv._tables[rid]
        assert kv.block_table[row, : len(t)].tolist() == t
        assert (kv.block_table[row, len(t):] == -1).all()


def test_prefix_cache_key_and_longest_match():
    # the key is the SHA-256 of the comma-joined ids (flash_attn_llm/kv_cache/manager.py:496-506)
    import hashlib
    assert PagedKVCache.get_prefix_cache_key([1, 2, 3]) == hashlib.sha256(b"1,2,3").hexdigest()
    kv = _mk()
    prompt = list(range(100, 140))                       # 40 tokens: two full blocks
    kv.allocate("a", len(prompt))
    assert kv.cache_prefix(prompt, "a") == 0             # nothing written yet
    kv.commit("a", len(prompt))
    assert kv.lookup_prefix(prompt) is None
    assert kv.cache_prefix(prompt, "a") == 32            # only full blocks (manager.py:551-556)
    assert kv.cache_prefix(prompt[:15], "a") == 0
    assert kv.lookup_prefix(prompt) == kv.get_block_table("a")[:2]
    assert kv.lookup_prefix(prompt[:32] + [7] * 20) == kv.get_block_table("a")[:2]    # longest aligned prefix
    assert kv.lookup_prefix(prompt[:31]) is None and kv.lookup_prefix([5] * 64) is None
    assert kv.cache_prefix(prompt, "a") == 32            # publishing twice attaches once
    assert kv._prefix_ref_count[kv.get_prefix_cache_key(prompt[:32])] == 1
    off = _mk(enable_prefix_cache=False)
    off.allocate("a", 40); off.commit("a", 40)
    assert off.cache_prefix(prompt, "a") == 0 and off.lookup_prefix(prompt) is None
    _check_accounting(kv)


def test_prefix_adoption_shares_blocks_and_frees_each_block_once():
    kv = _mk()
    prompt = list(range(48)) + [9, 9, 9]                 # three full blocks + 3 tokens
    kv.allocate("a", len(prompt)); kv.commit("a", len(prompt))
    assert kv.cache_prefix(prompt, "a") == 48
    a_blocks = kv.get_block_table("a")
    free0 = kv.get_num_free_blocks()
    rb = kv.allocate("b", len(prompt), token_ids=prompt)
    assert kv.get_cache_len("b") == 48                    # only 3 tokens left to prefill
    assert kv.get_block_table("b")[:3] == a_blocks[:3] and kv.get_block_table("b")[3] != a_blocks[3]
    assert kv.get_num_free_blocks() == free0 - 1
    assert kv.block_table[rb, :4].tolist() == kv.get_block_table("b")
    # a prompt that is cached in full keeps its last block to compute (one token at least)
    kv.allocate("c", 48, token_ids=prompt[:48])
    assert kv.get_cache_len("c") == 32 and kv.get_block_table("c")[:2] == a_blocks[:2]
    _check_accounting(kv)
    # the publisher goes first: the shared blocks stay with their other holders
    # (the reference would free all three here and put two of them on the free list twice, manager.py:452-463)
    kv.release("a")
    _check_accounting(kv)
    assert kv.lookup_prefix(prompt) == a_blocks[:3] and all(kv._refs[b] >= 2 for b in a_blocks[:2])
    kv.release("c")
    _check_accounting(kv)
    kv.release("b")                                       # last attached request: the entry goes, everything is free
    _check_accounting(kv)
    assert kv.lookup_prefix(prompt) is None and kv.get_num_free_blocks() == 12 and not kv._prefix_cache


def test_sliding_window_eviction_keeps_positions():
    kv = _mk(sliding_window=32)
    r = kv.allocate("a", 40)
    kv.commit("a", 40)                                    # 40 - 32 = 8 tokens outside: no full block yet
    assert kv.window_start("a") == 0 and kv.get_num_free_blocks() == 9
    kv.reserve("a", 80); kv.commit("a", 40)               # 48 outside -> 3 blocks (manager.py:588-596)
    assert kv.window_start("a") == 48 and kv.get_num_free_blocks() == 7 + 3
    t = kv.get_block_table("a")
    assert t[:3] == [-1, -1, -1] and all(b >= 0 for b in t[3:]) and len(t) == 5   # entry i stays logical block i
    assert kv.block_table[r, :5].tolist() == t
    kv.reserve("a", 81); kv.commit("a", 1)                # 49 outside: still 3
    assert kv.window_start("a") == 48
    _check_accounting(kv)
    kv.release("a")
    _check_accounting(kv)
    assert kv.get_num_free_blocks() == 12
    # a shared prefix block that leaves one request's window lives on for the other holder
    kv = _mk(sliding_window=16)
    prompt = list(range(32))
    kv.allocate("a", 32); kv.commit("a", 32)              # evicts a's first block at once ...
    assert kv.cache_prefix(prompt, "a") == 0              # ... so there is nothing whole to publish
    kv2 = _mk()
    kv2.allocate("a", 32); kv2.commit("a", 32); kv2.cache_prefix(prompt, "a")
    kv2.sliding_window = 16
    kv2.allocate("b", 33, token_ids=prompt + [1]); kv2.commit("b", 1)
    assert kv2.get_block_table("b")[0] == -1 and kv2.get_block_table("a")[0] >= 0
    _check_accounting(kv2)
    kv2.release("a"); kv2.release("b")
    _check_accounting(kv2)
    assert kv2.get_num_free_blocks() == 12


def test_block_manager_random_walk_keeps_accounting():
    rng = np.random.default_rng(5)
    kv = _mk(num_blocks=24, sliding_window=48)
    prompts = [list(rng.integers(0, 50, 16 * k)) for k in (1, 2, 3)]
    live = {}
    for step in range(400):
        op = rng.integers(0, 4)
        if op == 0 and len(live) < 4:
            rid = f"r{step}"
            base = prompts[rng.integers(0, 3)]
            toks = base + list(rng.integers(0, 50, rng.integers(1, 20)))
            try:
                kv.allocate(rid, len(toks), token_ids=toks)
            except MemoryError:
                _check_accounting(kv)
                continue
            kv.commit(rid, len(toks) - kv.get_cache_len(rid))
            kv.cache_prefix(toks, rid)
            live[rid] = len(toks)
        elif op == 1 and live:
            rid = list(live)[rng.integers(0, len(live))]
            n = int(rng.integers(1, 20))
            try:
                kv.reserve(rid, live[rid] + n)
            except MemoryError:
                continue
            kv.commit(rid, n)
            live[rid] += n
        elif op == 2 and live:
            rid = list(live)[rng.integers(0, len(live))]
            kv.release(rid)
            del live[rid]
        _check_accounting(kv)
    for rid in list(live):
        kv.release(rid)
    _check_accounting(kv)
    assert kv.get_num_free_blocks() == 24 and not kv._prefix_cache
