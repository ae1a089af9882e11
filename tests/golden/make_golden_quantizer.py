"""Golden vectors for the INT8 quantiser from the reference's own module.

    python tests/golden/make_golden_quantizer.py /path/to/reference

Loads flash_attn_llm/quantization/quantizer.py of the reference by file path and runs its
`quantize_kv_cache_int8` (quantizer.py:231-252: scale = absmax over the head dimension / 127,
values = round(x / scale) clamped) on seeded fp16 tensors shaped like the K operand of the INT8 decode
benchmark.  Stored in tests/golden/reference_quantizer_outputs.npz: a digest of the inputs, the
reference's scales and int8 values, and a mask of the elements where x / scale is an exact rounding
tie (n + 0.5): there, and only there, the reference's two quantisers differ from each other - its
Python helper rounds half to even (torch.round), its INT8 decode kernel rounds half away from zero
(roundf, flash_attn_kernel.cu:2837 and :2855) - and the kernel is what the operator follows.
"""
import hashlib
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = [("bench_like", 2, 8, 96, 128, 1.0), ("small_values", 1, 2, 40, 64, 0.01), ("large_values", 1, 4, 33, 128, 40.0)]


def main(ref_root):
    path = os.path.join(ref_root, "flash_attn_llm/quantization/quantizer.py")
    spec = importlib.util.spec_from_file_location("ref_quantizer", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    quantize = None
    for name in dir(mod):          # the helper is a static method of the module's quantizer class
        obj = getattr(mod, name)
        if isinstance(obj, type) and hasattr(obj, "quantize_kv_cache_int8"):
            quantize = obj.quantize_kv_cache_int8
    assert quantize is not None, "quantize_kv_cache_int8 not found in the reference module"
    out = {}
    for name, B, H, N, D, amp in CASES:
        g = torch.Generator().manual_seed(len(name) * 1000 + N)
        x = (torch.randn(B, H, N, D, generator=g) * amp).half()
        q8, scale = quantize(x.float())              # fp32 arithmetic, as the decode kernel's (float(k) / k_s)
        ratio = x.float() / (x.float().abs().amax(-1, keepdim=True) / 127.0).clamp(min=1e-8)
        ties = (ratio - torch.floor(ratio)) == 0.5
        out[f"{name}/digest"] = hashlib.sha256(x.numpy().tobytes()).hexdigest()
        out[f"{name}/shape"] = np.array([B, H, N, D])
        out[f"{name}/amp"] = np.array([amp], dtype=np.float64)
        out[f"{name}/q8"] = q8.numpy()
        out[f"{name}/scale"] = scale.numpy()
        out[f"{name}/ties"] = ties.numpy()
    np.savez_compressed(os.path.join(HERE, "reference_quantizer_outputs.npz"), **out)
    print("wrote", len(out), "arrays; ties:", {k: int(v.sum()) for k, v in out.items() if k.endswith("/ties")})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
