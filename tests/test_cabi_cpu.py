"""CPU: the C-ABI library loads and exports every symbol the header declares;
argument validation that needs no device; the Python mirror's checks."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "fa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from flash_attn_v100_b200 import _lib
    from flash_attn_v100_b200.build import build
    build()
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)
    assert lib.fa_version() >= 100


def test_workspace_size_query_and_invalid_arguments():
    from flash_attn_v100_b200 import _lib
    lib = _lib.load()
    assert lib.fa_decode_workspace_bytes(64, 32, 8, 128) > 0
    assert lib.fa_decode_workspace_bytes(64, 32, 8, 96) == lib.fa_decode_workspace_bytes(64, 32, 8, 128)  # padded
    assert lib.fa_decode_workspace_bytes(64, 32, 8, 100) == 0     # rows would not be 16-byte aligned
    assert lib.fa_decode_workspace_bytes(64, 32, 8, 48) == lib.fa_decode_workspace_bytes(64, 32, 8, 64)   # padded
    assert lib.fa_decode_workspace_bytes(64, 32, 8, 4) == 0       # not a multiple of 8
    assert lib.fa_decode_workspace_bytes(64, 32, 5, 128) == 0     # H_Q % H_KV != 0
    # validation happens before any CUDA call, so it can be exercised without a device
    rc = lib.fa_decode_gqa_f16(None, None, None, None, 1, 8, 8, 16, 64, 1, 0, None, 0, None)
    assert rc == -1 and b"null" in lib.fa_last_error()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.c_void_p((ctypes.addressof(buf) + 255) & ~255)
    rc = lib.fa_decode_gqa_f16(p, p, p, p, 1, 8, 8, 16, 64, 1, -1, None, 0, None)
    assert rc == -1 and b"cache_len must be non-negative" in lib.fa_last_error()
    rc = lib.fa_decode_gqa_f16(p, p, p, p, 1, 8, 8, 16, 64, 1, 16, None, 0, None)
    assert rc == -1 and b"less than sequence length" in lib.fa_last_error()
    rc = lib.fa_decode_gqa_f16(p, p, p, p, 1, 8, 3, 16, 64, 1, 0, None, 0, None)
    assert rc == -1 and b"divisible" in lib.fa_last_error()
    rc = lib.fa_decode_gqa_f16(p, p, p, p, 1, 8, 8, 16, 84, 1, 0, None, 0, None)
    assert rc == -2 and b"not built" in lib.fa_last_error()
    rc = lib.fa_prefill_varlen_f16(p, p, p, p, None, 1, 16, 8, 8, 64, 16, 1, None)
    assert rc == -1 and b"cu_seqlens" in lib.fa_last_error()


def test_drop_in_module_exports_reference_names():
    import flash_attn_v100
    import flash_attn_v100_b200 as pkg
    assert len(pkg.REFERENCE_EXPORTS) == 30          # flash_attn.cpp:225-254
    for name in pkg.REFERENCE_EXPORTS:
        assert callable(getattr(flash_attn_v100, name)), name
    with pytest.raises(NotImplementedError):
        flash_attn_v100.backward()


def test_python_checks_raise_runtime_error_like_torch_check():
    import flash_attn_v100 as fa
    q = torch.zeros(1, 8, 1, 64, dtype=torch.float16)
    k = torch.zeros(1, 8, 16, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        fa.forward_decode_gqa_fp16(q, k, k, True, 15)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        fa.forward_fp16(k, k, k, True)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        fa.forward_paged_decode_gqa_fp16(q, k, k, q, q, 1)


def test_decode_workspace_layout_is_shape_independent_at_its_head():
    """The status word and the arrival counters sit at fixed offsets (zeroed by fa_decode_workspace_init);
    only what follows them depends on the shape."""
    from flash_attn_v100_b200 import _lib
    lib = _lib.load()
    head = 256 + 1184 * 8                                   # status + one counter per possible CTA
    assert head % 256 == 0
    for B, H_Q, H_KV, D in [(1, 8, 8, 64), (64, 32, 8, 128), (4500, 8, 2, 64), (3, 40, 2, 256)]:
        G = H_Q // H_KV
        rows = min(G, 16)
        want = head + ((B + 1) * 4 + 255) // 256 * 256 + 1184 * 2 * rows * (D + 2) * 4
        want = (want + 255) // 256 * 256
        assert lib.fa_decode_workspace_bytes(B, H_Q, H_KV, D) == want
    assert lib.fa_decode_workspace_bytes(2, 8, 3, 128) == 0      # H_Q not divisible by H_KV
    assert lib.fa_decode_workspace_bytes(2, 8, 2, 100) == 0      # head dimension not built
