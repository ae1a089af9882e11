"""Golden vectors for the rotary embedding from the reference's own module.

    python tests/golden/make_golden_rope.py /path/to/reference

Loads flash_attn_llm/models/rope.py of the reference by file path (no package import needed),
runs RotaryEmbedding + apply_rotary_emb on seeded fp16 (and bfloat16) CPU tensors and stores inputs' SHA-256 and
the outputs in tests/golden/reference_rope_outputs.npz.
"""
import hashlib
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = [  # (name, B, H_Q, H_KV, D, theta, partial_rotary_factor, positions)
    ("qwen3_like", 3, 32, 8, 128, 1e6, 1.0, [0, 17, 4095]),
    ("llama_d64", 2, 8, 2, 64, 1e4, 1.0, [1, 1000]),
    ("partial", 2, 4, 4, 128, 1e4, 0.5, [7, 300]),
]


def digest(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().numpy().tobytes())
    return h.hexdigest()


def main(ref_root):
    spec = importlib.util.spec_from_file_location("ref_rope", os.path.join(ref_root, "flash_attn_llm/models/rope.py"))
    rope = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rope)
    out = {}
    for name, B, H_Q, H_KV, D, theta, prf, positions in CASES:
        torch.manual_seed(77)
        q = torch.randn(B, H_Q, 1, D).half()
        k = torch.randn(B, H_KV, 1, D).half()
        emb = rope.RotaryEmbedding(D, 8192, theta, None, prf)
        cos, sin = emb(1, torch.tensor(positions).view(B, 1))
        qe, ke = rope.apply_rotary_emb(q, k, cos, sin)
        out[f"{name}/digest"] = digest(q, k)
        out[f"{name}/cos"] = cos.numpy()
        out[f"{name}/sin"] = sin.numpy()
        out[f"{name}/q"] = qe.numpy()
        out[f"{name}/k"] = ke.numpy()
        # the same case on bfloat16 tensors (stored as their 16-bit patterns): the pin of the *_bf16 twins
        torch.manual_seed(77)
        qb = torch.randn(B, H_Q, 1, D).bfloat16()
        kb = torch.randn(B, H_KV, 1, D).bfloat16()
        qeb, keb = rope.apply_rotary_emb(qb, kb, cos, sin)
        out[f"{name}/digest_bf16"] = digest(qb.view(torch.int16), kb.view(torch.int16))
        out[f"{name}/q_bf16"] = qeb.view(torch.int16).numpy()
        out[f"{name}/k_bf16"] = keb.view(torch.int16).numpy()
    np.savez_compressed(os.path.join(HERE, "reference_rope_outputs.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
