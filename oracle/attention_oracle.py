"""CPU oracle for the attention operator path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch on host fp32 tensors, the eager attention
routines that the reference project's own tests use as ground truth.  It is
the checker for the CUDA kernels: only the test-suite, the smoke check and the
CPU-baseline leg of the benchmark may import it.  The product path never does.

Parity status: pinned.  `tests/golden/*.npz` were produced by running the
reference's own oracle functions (imported from the reference source tree,
see `tests/golden/make_golden.py`) and `tests/test_oracle_golden.py` checks
every function below against them.  Exception: the INT8-QK decode has no test
or oracle in the reference ("parity unpinned" by the reference); the
restatement follows the reference kernel's arithmetic with per-token K scales.

Each function cites the reference file:line it follows.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np
import torch
import torch.nn.functional as F

PAGE_BLOCK_SIZE = 16  # flash_attn_kernel.cu:3389, test_decode.py:6


# --------------------------------------------------------------------------
# decode over a contiguous, per-sequence-length cache
# --------------------------------------------------------------------------
def continuous_batching_decode(q, k, v, cache_lens, causal=True, final_cast=True):
    """test_continuous_batching.py:323-346 (`reference_continuous_batching_decode`).

    q [B,H_Q,1,D], k/v [B,H_KV,max_N,D]; sequence b attends keys
    [0, min(cache_lens[b]+1, max_N)).  `final_cast=False` returns the fp32
    value before the reference's closing `.half()` so that a 2e-3 gate is not
    blurred by a second fp16 rounding.
    """
    B, H_Q, _, D = q.shape
    H_KV, max_N = k.size(1), k.size(2)
    group = H_Q // H_KV
    scale = 1.0 / (D ** 0.5)
    out = torch.zeros((B, H_Q, 1, D), dtype=torch.float32)
    for b in range(B):
        cur_len = int(cache_lens[b])
        current_N = min(cur_len + 1, max_N)
        if current_N <= 0:
            continue  # the reference would divide 0/0; this build defines zeros
        for h_q in range(H_Q):
            h_kv = h_q // group
            q_vec = q[b, h_q, 0].float()
            k_mat = k[b, h_kv, :current_N].float()
            v_mat = v[b, h_kv, :current_N].float()
            scores = (k_mat @ q_vec) * scale
            if causal:
                mask = torch.arange(current_N) > cur_len
                scores = scores.masked_fill(mask, float("-inf"))
            probs = torch.softmax(scores, dim=0)
            out[b, h_q, 0] = probs @ v_mat
    return out.half() if final_cast else out


def decode_gqa(q, k, v, causal, cache_len, final_cast=True):
    """Semantics of `forward_decode_gqa_fp16` (flash_attn_kernel.cu:1800-1833,
    mask at :1719): the query sits at position `cache_len`; key j is visible
    iff `not causal or j <= cache_len`.  Checked by the reference against SDPA
    in test_gqa.py:120-169 with N = cache_len + 1.
    """
    B, H_Q, _, D = q.shape
    N = k.size(2)
    n_vis = min(cache_len + 1, N) if causal else N
    lens = torch.full((B,), n_vis - 1, dtype=torch.int32)
    return continuous_batching_decode(q, k[:, :, :n_vis], v[:, :, :n_vis], lens, False, final_cast)


def sliding_window_mask(N, cache_len, window_size, sink_size):
    """Keys attended by `forward_decode_sliding_window_gqa` (flash_attn_kernel.cu:4386-4387,
    :4410-4412): j < sink_size, or window_start <= j <= cache_len, with
    window_start = max(0, min(cache_len + 1, N) - window_size).  The sink is NOT
    bounded by cache_len.  The reference's test builds the same mask from
    `mask[:sink] = True; mask[window_start:effective_end] = True` (test_kv_compress.py:265-270)."""
    effective_end = min(cache_len + 1, N)
    window_start = max(0, effective_end - window_size)
    j = torch.arange(N)
    return (j < sink_size) | ((j >= window_start) & (j <= cache_len))


def sliding_window_decode(q, k, v, causal, cache_len, window_size, sink_size, final_cast=True):
    """Semantics of `forward_decode_sliding_window_gqa` (flash_attn_kernel.cu:4346-4535):
    fp32 softmax(q.k / sqrt(D)) over the attended keys only, times v; `causal` is ignored
    by the reference.  A row with no attended key is returned as zeros here (the
    reference computes 0/0 there, :4476-4480)."""
    B, H_Q, _, D = q.shape
    H_KV, N = k.size(1), k.size(2)
    G = H_Q // H_KV
    mask = sliding_window_mask(N, int(cache_len), int(window_size), int(sink_size))
    out = torch.zeros(B, H_Q, 1, D, dtype=torch.float32)
    if bool(mask.any()):
        kf = k.float().repeat_interleave(G, dim=1)[:, :, mask]
        vf = v.float().repeat_interleave(G, dim=1)[:, :, mask]
        s = torch.einsum("bhqd,bhnd->bhqn", q.float(), kf) * (1.0 / math.sqrt(D))
        out = torch.einsum("bhqn,bhnd->bhqd", torch.softmax(s, dim=-1), vf)
    return out.half() if final_cast else out


def quantize_kv_int8(kv):
    """Per-token symmetric int8 quantisation of a KV tensor [B,H,N,D], the helper the
    reference tests feed `forward_decode_int8_kv_cache_gqa` with (test_kv_compress.py:7-19):
    scale = max(|x|, over D) / 127 clamped at 1e-8, stored as fp16; q = clamp(round(x / scale))."""
    x = kv.float()
    scale = (x.abs().amax(dim=-1, keepdim=True) / 127.0).clamp(min=1e-8)
    q8 = (x / scale).round().clamp(-128, 127).to(torch.int8)
    return q8.contiguous(), scale.squeeze(-1).half().contiguous()


def dequantize_kv_int8(kv_int8, scale_f16):
    """Dequantisation inside the reference kernel (flash_attn_kernel.cu:4083-4086):
    fp16(float(int8) * float(scale_fp16)) per element."""
    return (kv_int8.float() * scale_f16.float().unsqueeze(-1)).half()


def decode_int8_kv_cache_gqa(q, k_int8, v_int8, k_scale, v_scale, cache_len, final_cast=True):
    """Semantics of `forward_decode_int8_kv_cache_gqa` (flash_attn_kernel.cu:4020-4221): K and V
    are dequantised to fp16 (see `dequantize_kv_int8`), then keys j <= cache_len (j < N) are
    attended exactly as in the fp16 GQA decode (:4094-4098)."""
    return decode_gqa(q, dequantize_kv_int8(k_int8, k_scale), dequantize_kv_int8(v_int8, v_scale), True,
                      int(cache_len), final_cast)


# --------------------------------------------------------------------------
# SDPA-based oracles
# --------------------------------------------------------------------------
def expand_kv_heads(k, v, num_q_heads):
    """test_gqa.py:12-14."""
    rep = num_q_heads // k.size(1)
    return k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)


def sdpa_decode(q, k_expanded, v_expanded, seq_lens, final_cast=True):
    """test_decode.py:9-19 (`sdpa_decode_reference`): fp32 SDPA with a -inf
    mask past `seq_lens[b]`; k/v already expanded to H_Q heads."""
    q_ref, k_ref, v_ref = q.float(), k_expanded.float(), v_expanded.float()
    B, H, max_len = q.size(0), q.size(1), k_expanded.size(2)
    attn_mask = torch.zeros(B, H, 1, max_len, dtype=torch.float32)
    for b, seq_len in enumerate(seq_lens.tolist()):
        if seq_len < max_len:
            attn_mask[b, :, :, seq_len:] = float("-inf")
    out = F.scaled_dot_product_attention(q_ref, k_ref, v_ref, attn_mask=attn_mask,
                                         dropout_p=0.0, is_causal=False)
    return out.to(q.dtype) if final_cast else out


def sdpa_gqa(q, k, v, causal=True, seq_lens=None, final_cast=True):
    """test_gqa.py:17-39 (`sdpa_reference_gqa`)."""
    k_e, v_e = expand_kv_heads(k, v, q.size(1))
    q_ref, k_ref, v_ref = q.float(), k_e.float(), v_e.float()
    attn_mask = None
    if seq_lens is not None:
        max_len = k_ref.size(-2)
        attn_mask = torch.zeros(q_ref.size(0), q_ref.size(1), q_ref.size(2), max_len,
                                dtype=torch.float32)
        for b, seq_len in enumerate(seq_lens.tolist()):
            if seq_len < max_len:
                attn_mask[b, :, :, seq_len:] = float("-inf")
    out = F.scaled_dot_product_attention(q_ref, k_ref, v_ref, attn_mask=attn_mask,
                                         dropout_p=0.0,
                                         is_causal=causal and q.size(2) > 1)
    return out.to(q.dtype) if final_cast else out


def prefill_gqa(q, k, v, causal=True, final_cast=True):
    """test_prefill_gqa.py:7-31 (`reference_gqa_attention`), evaluated in fp32
    (the reference runs it in the input dtype on the GPU; fp32 is the stricter
    statement of the same formula and is what a 2e-3 gate needs)."""
    d = q.size(-1)
    H_Q, H_KV = q.size(1), k.size(1)
    group = H_Q // H_KV
    B, _, N, D = q.shape
    out = torch.zeros(q.shape, dtype=torch.float32)
    for h_q in range(H_Q):
        h_kv = h_q // group
        q_h, k_h, v_h = q[:, h_q].float(), k[:, h_kv].float(), v[:, h_kv].float()
        scores = torch.matmul(q_h, k_h.transpose(-1, -2)) / (d ** 0.5)
        if causal:
            mask = torch.triu(torch.ones(N, N), diagonal=1)
            scores = scores.masked_fill(mask.bool(), float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        out[:, h_q] = torch.matmul(probs, v_h)
    return out.to(q.dtype) if final_cast else out


def varlen_prefill(q, k, v, cu_seqlens, causal=True, final_cast=True):
    """Packed varlen prefill: q [total,H_Q,D], k/v [total,H_KV,D], int32
    `cu_seqlens` [batch+1].  The reference has no independent varlen oracle
    (test_async.py:68-113 only compares two launches of its own kernel); the
    kernel's meaning (flash_attn_kernel.cu:3005-3148: causal attention inside
    each [cu[i], cu[i+1]) span) is the dense oracle applied per sequence."""
    out = torch.zeros(q.shape, dtype=torch.float32)
    cu = [int(x) for x in cu_seqlens.tolist()]
    for s in range(len(cu) - 1):
        a, b = cu[s], cu[s + 1]
        if b <= a:
            continue
        qs = q[a:b].transpose(0, 1).unsqueeze(0)
        ks = k[a:b].transpose(0, 1).unsqueeze(0)
        vs = v[a:b].transpose(0, 1).unsqueeze(0)
        o = sdpa_gqa(qs, ks, vs, causal=causal, final_cast=False)
        out[a:b] = o[0].transpose(0, 1)
    return out.to(q.dtype) if final_cast else out


# --------------------------------------------------------------------------
# paged cache helpers and paged decode
# --------------------------------------------------------------------------
def build_paged_cache(k, v, seq_lens, physical_block_order, num_physical_blocks=None):
    """test_decode.py:22-44 (`build_non_contiguous_paged_cache`): scatter
    contiguous k/v [B,H_KV,max_len,D] into pools [pages,H_KV,16,D] following
    `physical_block_order`; unused table entries are -1."""
    B, H_KV, _, D = k.shape
    lens = [int(x) for x in seq_lens.tolist()]
    max_num_blocks = max(max((n + PAGE_BLOCK_SIZE - 1) // PAGE_BLOCK_SIZE for n in lens), 1)
    if num_physical_blocks is None:
        num_physical_blocks = max(physical_block_order[: B * max_num_blocks]) + 1
    k_cache = torch.zeros(num_physical_blocks, H_KV, PAGE_BLOCK_SIZE, D, dtype=k.dtype)
    v_cache = torch.zeros_like(k_cache)
    block_table = torch.full((B, max_num_blocks), -1, dtype=torch.int32)
    cursor = 0
    for b in range(B):
        used = (lens[b] + PAGE_BLOCK_SIZE - 1) // PAGE_BLOCK_SIZE
        for blk in range(used):
            phys = int(physical_block_order[cursor]); cursor += 1
            block_table[b, blk] = phys
            start = blk * PAGE_BLOCK_SIZE
            end = min(start + PAGE_BLOCK_SIZE, lens[b])
            k_cache[phys, :, : end - start].copy_(k[b, :, start:end])
            v_cache[phys, :, : end - start].copy_(v[b, :, start:end])
    return k_cache, v_cache, block_table, max_num_blocks


def gather_paged_sequence(cache, block_table_row, seq_len):
    """Inverse of `build_paged_cache` for one sequence: [H_KV, seq_len, D].
    Token t lives at cache[block_table[t // 16], h, t % 16]
    (flash_attn_kernel.cu:3438-3446)."""
    used = (seq_len + PAGE_BLOCK_SIZE - 1) // PAGE_BLOCK_SIZE
    ids = block_table_row[:used].long()
    pages = cache[ids]                       # [used, H_KV, 16, D]
    seq = pages.permute(1, 0, 2, 3).reshape(cache.size(1), used * PAGE_BLOCK_SIZE, cache.size(3))
    return seq[:, :seq_len]


def paged_decode(q, k_cache, v_cache, block_table, seq_lens, final_cast=True):
    """Oracle of `forward_paged_decode_gqa_fp16` (flash_attn_kernel.cu:3516-3584):
    per sequence, rebuild contiguous K/V from the pages and run the reference's
    SDPA decode oracle (test_decode.py:284-290).  One sequence at a time keeps
    host memory bounded at large sizes.  seq_len == 0 gives zeros (the reference
    kernel divides 0/0 there)."""
    B, H_Q, _, D = q.shape
    out = torch.zeros(B, H_Q, 1, D, dtype=torch.float32)
    for b in range(B):
        n = int(seq_lens[b])
        if n <= 0:
            continue
        kb = gather_paged_sequence(k_cache, block_table[b], n).unsqueeze(0)
        vb = gather_paged_sequence(v_cache, block_table[b], n).unsqueeze(0)
        ke, ve = expand_kv_heads(kb, vb, H_Q)
        out[b] = sdpa_decode(q[b:b + 1], ke, ve, torch.tensor([n]), final_cast=False)[0]
    return out.to(q.dtype) if final_cast else out


# --------------------------------------------------------------------------
# INT8-QK decode (no oracle exists in the reference: parity unpinned there)
# --------------------------------------------------------------------------
def round_half_away(x: torch.Tensor) -> torch.Tensor:
    """C `roundf` (flash_attn_kernel.cu:2837, :2856); torch.round is half-even."""
    # |x| + 0.5 in double: exact, so that 0.49999997f does not round up to 1 on the way
    return (torch.sign(x).double() * torch.floor(x.abs().double() + 0.5)).to(x.dtype)


def quantize_int8(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """clamp(roundf(x / s), -127, 127) in IEEE fp32 (flash_attn_kernel.cu:2837)."""
    t = x.float() / scale.float()
    return torch.clamp(round_half_away(t), -127.0, 127.0)


def int8_scores(q, k, q_scale, k_scale):
    """int32 QK^T accumulators [B,H_Q,N] (flash_attn_kernel.cu:2871-2885) with
    per-token K scales k_scale[b,h_kv,n] (README.md:169-171).  The products are
    integers below 2^24 so an fp32 matmul is exact."""
    B, H_Q, _, D = q.shape
    H_KV = k.size(1)
    g = H_Q // H_KV
    qq = quantize_int8(q[:, :, 0], q_scale.unsqueeze(-1))          # [B,H_Q,D]
    kq = quantize_int8(k, k_scale.unsqueeze(-1))                   # [B,H_KV,N,D]
    qq = qq.view(B, H_KV, g, D)
    dots = torch.matmul(qq.double(), kq.double().transpose(-1, -2))  # [B,H_KV,g,N]
    return dots.reshape(B, H_Q, -1).to(torch.int32)


def decode_int8_gqa(q, k, v, q_scale, k_scale, cache_len, final_cast=True):
    """`forward_decode_int8_gqa` (flash_attn_kernel.cu:2796-2939): score =
    float(int_dot) * q_s * k_s * (1/sqrt(D)) (:2888), keys j > cache_len masked
    (:2866), fp32 softmax, fp16 V with fp32 accumulation.  Returns (out, int_dot)."""
    B, H_Q, _, D = q.shape
    H_KV, N = k.size(1), k.size(2)
    g = H_Q // H_KV
    dots = int8_scores(q, k, q_scale, k_scale)                     # [B,H_Q,N] int32
    scale = np.float32(1.0 / math.sqrt(D))
    ks = k_scale.float().repeat_interleave(g, dim=1)               # [B,H_Q,N]
    s = dots.float() * q_scale.float().unsqueeze(-1) * ks * float(scale)
    n_vis = min(cache_len + 1, N)
    s = s[:, :, :n_vis]
    p = torch.softmax(s, dim=-1)
    ve = v.float().repeat_interleave(g, dim=1)[:, :, :n_vis]       # [B,H_Q,n,D]
    out = torch.einsum("bhn,bhnd->bhd", p, ve).unsqueeze(2)
    return (out.half() if final_cast else out), dots


# --------------------------------------------------------------------------
# seeded synthetic workloads (shapes/distributions of the benchmark configs)
# --------------------------------------------------------------------------
def make_paged_workload(B, H_Q, H_KV, D, min_len, max_len, seed=0, dtype=torch.float16,
                        fill=True):
    """Seeded paged-decode workload: seq_lens uniform in [min_len, max_len],
    pool of sum(ceil(len/16)) pages, block_table a random permutation of it."""
    from flash_attn_v100_b200.synthetic import make_paged_tables
    t = make_paged_tables(B, min_len, max_len, seed)
    g, seq_lens, block_table = t["generator"], t["seq_lens"], t["block_table"]
    n_pages, max_blocks = t["n_pages"], t["max_num_blocks"]
    q = torch.randn(B, H_Q, 1, D, generator=g).to(dtype)
    if fill:
        k_cache = torch.randn(max(n_pages, 1), H_KV, PAGE_BLOCK_SIZE, D, generator=g).to(dtype)
        v_cache = torch.randn(max(n_pages, 1), H_KV, PAGE_BLOCK_SIZE, D, generator=g).to(dtype)
    else:
        k_cache = v_cache = None
    return dict(q=q, k_cache=k_cache, v_cache=v_cache, block_table=block_table,
                seq_lens=seq_lens, max_num_blocks=max_blocks, n_pages=n_pages)


# --------------------------------------------------------------------------
# rotary embedding + append into pages (the write side of the paged cache)
# --------------------------------------------------------------------------
def rope_cos_sin(positions, rot_dim, theta=10000.0):
    """fp32 cos/sin tables [T, rot_dim] for integer positions [T], as
    flash_attn_llm/models/rope.py:17-37 and :228-266 compute them:
    inv_freq = 1 / theta^(2i/rot_dim), emb = cat(freqs, freqs)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    freqs = torch.outer(positions.float().flatten(), inv_freq)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x):
    """rope.py:269-283."""
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_emb(q, k, cos, sin):
    """rope.py:302-348 (half-rotation layout; partial rotary when cos is narrower than D).
    q [..., H_Q, D] / k [..., H_KV, D] in fp16, cos/sin broadcastable [..., 1, rot_dim] fp32.
    Evaluated with PyTorch fp16 tensor ops exactly as the reference does."""
    rot = cos.shape[-1]
    cos = cos.to(q.dtype)
    sin = sin.to(q.dtype)

    def emb(x):
        xr, xp = x[..., :rot], x[..., rot:]
        out = (xr * cos) + (rotate_half(xr) * sin)
        return torch.cat([out, xp], dim=-1) if xp.shape[-1] else out

    return emb(q), emb(k)


def append_to_pages(k_cache, v_cache, block_table, seq, first_slot, k_rows, v_rows):
    """Store tokens (k_rows/v_rows [n, H_KV, D]) of sequence `seq` at slots first_slot..;
    token at slot s lives at cache[block_table[seq][s // 16], :, s % 16]
    (flash_attn_llm/kv_cache/manager.py:350-357, kernel layout flash_attn_kernel.cu:3446)."""
    for i in range(k_rows.shape[0]):
        s = first_slot + i
        page = int(block_table[seq, s // PAGE_BLOCK_SIZE])
        k_cache[page, :, s % PAGE_BLOCK_SIZE] = k_rows[i]
        v_cache[page, :, s % PAGE_BLOCK_SIZE] = v_rows[i]
