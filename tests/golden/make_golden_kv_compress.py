"""Pin the sliding-window and INT8-KV-cache oracles with the reference's OWN tests, and write the fixture.

Run once where the reference source tree is available:

    python tests/golden/make_golden_kv_compress.py /path/to/reference

The reference's `test_kv_compress.py` holds its expected values inline in the test
bodies (a masked softmax for the sliding window, a comparison against the fp16
decode for the INT8 cache), so there is no oracle function to import.  Instead
the reference's test functions themselves are run on CPU tensors, with a
stand-in `flash_attn_v100` module whose three operators are the functions of
`oracle/attention_oracle.py`; `torch.randn` is wrapped to drop `device='cuda'`.
If the reference's assertions pass, the oracle satisfies the reference's own
acceptance test.  The operator calls the tests made (inputs and oracle
outputs) are then stored, with a SHA-256 of the inputs.
"""
import hashlib
import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))

from oracle import attention_oracle as ao  # noqa: E402


def digest(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().numpy().tobytes())
    return h.hexdigest()


def main(ref_root):
    calls = []

    stub = types.ModuleType("flash_attn_v100")

    def forward_decode_gqa_fp16(q, k, v, causal, cache_len):
        return ao.decode_gqa(q, k, v, causal, cache_len)

    def forward_decode_sliding_window_gqa(q, k, v, causal, cache_len, window_size, sink_size):
        out = ao.sliding_window_decode(q, k, v, causal, cache_len, window_size, sink_size)
        calls.append(("sw", dict(q=q, k=k, v=v, out=out,
                                 args=np.asarray([cache_len, window_size, sink_size], dtype=np.int64))))
        return out

    def forward_decode_int8_kv_cache_gqa(q, k_int8, v_int8, k_scale, v_scale, cache_len):
        out = ao.decode_int8_kv_cache_gqa(q, k_int8, v_int8, k_scale, v_scale, cache_len)
        calls.append(("i8kv", dict(q=q, k_int8=k_int8, v_int8=v_int8, k_scale=k_scale, v_scale=v_scale, out=out,
                                   args=np.asarray([cache_len], dtype=np.int64))))
        return out

    stub.forward_decode_gqa_fp16 = forward_decode_gqa_fp16
    stub.forward_decode_sliding_window_gqa = forward_decode_sliding_window_gqa
    stub.forward_decode_int8_kv_cache_gqa = forward_decode_int8_kv_cache_gqa
    sys.modules["flash_attn_v100"] = stub
    sys.path.insert(0, ref_root)

    real_randn = torch.randn

    def cpu_randn(*a, **kw):
        kw.pop("device", None)
        dt = kw.pop("dtype", torch.float32)
        return real_randn(*a, dtype=torch.float32, **kw).to(dt)

    torch.randn = cpu_randn
    try:
        tk = importlib.import_module("test_kv_compress")
        # the helper of the reference's tests and the oracle's restatement must agree bit for bit
        torch.manual_seed(7)
        x = torch.randn(2, 3, 40, 64, dtype=torch.float16)
        a8, a_s = tk.quantize_kv_to_int8(x)
        b8, b_s = ao.quantize_kv_int8(x)
        assert torch.equal(a8, b8) and torch.equal(a_s, b_s)
        assert tk.test_int8_kv_cache_correctness()
        assert tk.test_sliding_window_correctness()
        assert tk.test_sliding_window_no_sink()
    finally:
        torch.randn = real_randn

    out = {}
    n = {"sw": 0, "i8kv": 0}
    for kind, d in calls:
        name = f"{kind}{n[kind]}"
        n[kind] += 1
        ins = [t for key, t in d.items() if key not in ("out", "args")]
        out[f"{name}/digest"] = np.asarray(digest(*ins))
        out[f"{name}/args"] = d["args"]
        out[f"{name}/shape"] = np.asarray(list(d["q"].shape[:2]) + [d[("k" if kind == "sw" else "k_int8")].size(1),
                                                                   d[("k" if kind == "sw" else "k_int8")].size(2),
                                                                   d["q"].size(3)], dtype=np.int64)
        out[f"{name}/out"] = d["out"].numpy()
    path = os.path.join(HERE, "reference_kv_compress_outputs.npz")
    np.savez_compressed(path, **out)
    print("reference tests passed with the oracle as the operator;", n, "calls ->", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
