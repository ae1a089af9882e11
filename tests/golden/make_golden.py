"""Generate the golden fixtures in this folder from the reference's OWN oracles.

Run once where the reference source tree is available:

    python tests/golden/make_golden.py /path/to/reference

The reference's test files import its CUDA extension at module top, so an
empty stand-in module named `flash_attn_v100` is placed in `sys.modules`
first; only the pure-PyTorch oracle functions of those files are called
(on CPU tensors).  Inputs are drawn from torch's CPU generator with the seeds
the reference tests use; each fixture stores a SHA-256 of the input bytes
(so a drifting RNG is detected rather than silently compared) and the
reference oracle's output.  The fixtures pin `oracle/attention_oracle.py`.
"""
import hashlib
import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def digest(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().numpy().tobytes())
    return h.hexdigest()


def sample_rows(n):
    """Query rows kept in a fixture for prefill outputs (keeps the file small):
    the first and last rows, tile-boundary neighbours and a fixed stride."""
    keep = sorted(set([0, 1, n - 1, n - 2, n // 2] + [r for r in (15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129) if r < n]
                      + list(range(5, n, 37))))
    return np.asarray(keep, dtype=np.int64)


def gen_qkv(seed, q_shape, kv_shape):
    """CPU-generator restatement of `torch.manual_seed(seed); randn(q); randn(k); randn(v)`."""
    torch.manual_seed(seed)
    q = torch.randn(*q_shape, dtype=torch.float32).half()
    k = torch.randn(*kv_shape, dtype=torch.float32).half()
    v = torch.randn(*kv_shape, dtype=torch.float32).half()
    return q, k, v


CONT_BATCH_CASES = [  # test_continuous_batching.py:358-361 + benchmark config 1
    ("cb_d64", 3, 8, 2, 64, 17, [0, 3, 15]),
    ("cb_d256", 2, 32, 8, 256, 33, [0, 31]),
    ("cb_config1", 4, 32, 8, 128, 101, [10, 50, 100, 20]),
]
GQA_DECODE_CASES = [(1, 8, 4, 65, 64), (2, 16, 4, 127, 64), (1, 32, 8, 257, 128), (1, 32, 8, 129, 256)]
GQA_PREFILL_CASES = [(1, 8, 4, 64, 64), (2, 16, 4, 96, 64), (1, 32, 8, 128, 128), (1, 32, 8, 64, 256)]
PREFILL_CASES = [  # test_prefill_gqa.py:39-50 (B,H_Q,H_KV,D,N)
    (1, 8, 8, 64, 128), (1, 8, 4, 64, 128), (1, 8, 2, 64, 128), (1, 8, 1, 64, 128),
    (1, 32, 8, 64, 128), (2, 8, 4, 64, 128), (1, 8, 4, 64, 256), (1, 8, 4, 128, 128),
    (1, 32, 8, 128, 256), (1, 32, 8, 256, 128),
]


def main(ref_root):
    sys.modules.setdefault("flash_attn_v100", types.ModuleType("flash_attn_v100"))
    sys.path.insert(0, ref_root)
    t_cb = importlib.import_module("test_continuous_batching")
    t_dec = importlib.import_module("test_decode")
    t_gqa = importlib.import_module("test_gqa")
    t_pre = importlib.import_module("test_prefill_gqa")
    t_main = importlib.import_module("test")
    torch.set_num_threads(max(os.cpu_count() or 1, 1))
    out = {}

    for name, B, H_Q, H_KV, D, max_N, lens in CONT_BATCH_CASES:
        q, k, v = gen_qkv(0, (B, H_Q, 1, D), (B, H_KV, max_N, D))
        cl = torch.tensor(lens, dtype=torch.int32)
        out[f"{name}/digest"] = digest(q, k, v)
        for causal in (False, True):
            ref = t_cb.reference_continuous_batching_decode(q, k, v, cl, causal)
            out[f"{name}/causal{int(causal)}"] = ref.numpy()

    # test_decode.py:275-323 — paged decode, non-contiguous physical order
    torch.manual_seed(2025)
    B, H_Q, H_KV, D = 3, 8, 4, 64
    seq_lens = torch.tensor([16, 23, 33], dtype=torch.int32)
    max_len = int(seq_lens.max())
    q = torch.randn(B, H_Q, 1, D).half()
    k = torch.randn(B, H_KV, max_len, D).half()
    v = torch.randn(B, H_KV, max_len, D).half()
    order = [5, 2, 7, 1, 9, 3]
    ke, ve = k.repeat_interleave(H_Q // H_KV, 1), v.repeat_interleave(H_Q // H_KV, 1)
    out["paged/digest"] = digest(q, k, v)
    out["paged/out"] = t_dec.sdpa_decode_reference(q, ke, ve, seq_lens).numpy()
    kc, vc, bt, mnb = t_dec.build_non_contiguous_paged_cache(k, v, seq_lens, order)
    out["paged/block_table"] = bt.numpy()
    out["paged/cache_digest"] = digest(kc, vc)
    out["paged/max_num_blocks"] = np.int64(mnb)
    k2, v2 = k.clone(), v.clone()
    k2[1, :, 16:23] += 0.5
    v2[1, :, 16:23] -= 0.25
    out["paged/out_updated"] = t_dec.sdpa_decode_reference(
        q, k2.repeat_interleave(H_Q // H_KV, 1), v2.repeat_interleave(H_Q // H_KV, 1), seq_lens).numpy()

    # test_gqa.py:126-167 — one generator stream, seed 1234, decode then prefill cases
    torch.manual_seed(1234)
    for i, (B, H_Q, H_KV, N, D) in enumerate(GQA_DECODE_CASES):
        q = torch.randn(B, H_Q, 1, D).half()
        k = torch.randn(B, H_KV, N, D).half()
        v = torch.randn(B, H_KV, N, D).half()
        sl = torch.full((B,), N, dtype=torch.int32)
        out[f"gqa_decode{i}/digest"] = digest(q, k, v)
        out[f"gqa_decode{i}/out"] = t_gqa.sdpa_reference_gqa(q, k, v, causal=False, seq_lens=sl).numpy()
    for i, (B, H_Q, H_KV, N, D) in enumerate(GQA_PREFILL_CASES):
        q = torch.randn(B, H_Q, N, D).half()
        k = torch.randn(B, H_KV, N, D).half()
        v = torch.randn(B, H_KV, N, D).half()
        out[f"gqa_prefill{i}/digest"] = digest(q, k, v)
        rows = sample_rows(N)
        out[f"gqa_prefill{i}/rows"] = rows
        out[f"gqa_prefill{i}/out"] = t_gqa.sdpa_reference_gqa(q, k, v, causal=True).numpy()[:, :, rows]

    # test_prefill_gqa.py:39-91 — seed 42 per case.  The reference evaluates its
    # oracle in the input dtype on the GPU; half matmul on CPU is slow/unsupported
    # in places, so the oracle is fed fp32 copies of the same fp16 values.
    for i, (B, H_Q, H_KV, D, N) in enumerate(PREFILL_CASES):
        q, k, v = gen_qkv(42, (B, H_Q, N, D), (B, H_KV, N, D))
        out[f"prefill{i}/digest"] = digest(q, k, v)
        rows = sample_rows(N)
        out[f"prefill{i}/rows"] = rows
        out[f"prefill{i}/out"] = t_pre.reference_gqa_attention(q.float(), k.float(), v.float(), True).half().numpy()[:, :, rows]

    # test.py:19-57 — dense MHA forward_fp16 B2 H8 N256 D64 seed 0 (inputs drawn in fp32)
    torch.manual_seed(0)
    q = torch.randn(2, 8, 256, 64); k = torch.randn(2, 8, 256, 64); v = torch.randn(2, 8, 256, 64)
    qh, kh, vh = q.half(), k.half(), v.half()
    out["dense/digest"] = digest(qh, kh, vh)
    rows = sample_rows(256)
    out["dense/rows"] = rows
    out["dense/causal1"] = t_main.reference(qh.float(), kh.float(), vh.float(), True).half().numpy()[:, :, rows]
    out["dense/causal0"] = t_main.reference(qh.float(), kh.float(), vh.float(), False).half().numpy()[:, :, rows]

    np.savez_compressed(os.path.join(HERE, "reference_oracle_outputs.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
