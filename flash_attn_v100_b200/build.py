"""Build recipe for the sm_100a shared library (`libfa_b200.so`, kept in-tree).

    python -m flash_attn_v100_b200.build            # rebuild what is out of date
    python -m flash_attn_v100_b200.build --force
    python -m flash_attn_v100_b200.build -v         # also print ptxas resource usage

Every `.cu` file is compiled to an object of its own (in parallel, cached under
`_build/` by source time stamps and flags) and the objects are linked into one
library.  nvcc cross-compiles without a GPU.  The library links only the CUDA
runtime (static); it has no libtorch dependency.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_PATH = os.path.join(PKG_DIR, "libfa_b200.so")
OBJ_DIR = os.path.join(PKG_DIR, "_build")

COMPILE_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]
LINK_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC"]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if not f.endswith(".cu")]
    deps += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return deps


def needs_build(lib_path: str = LIB_PATH) -> bool:
    if not os.path.exists(lib_path):
        return True
    t = os.path.getmtime(lib_path)
    return any(os.path.getmtime(d) > t for d in sources() + _headers())


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libfa_b200.so")
    return nvcc


def _run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    return res.stderr


def build(force: bool = False, verbose: bool = False, extra_flags=None, lib_path: str = LIB_PATH) -> str:
    """Compile the sources that changed and link `lib_path`.  `extra_flags` (or the environment
    variable FA_B200_NVCC_FLAGS) adds compiler flags, e.g. `-DFA_TC5_PROF` for the instrumented
    prefill kernel; objects built with different flags are cached side by side."""
    extra = list(extra_flags) if extra_flags is not None else os.environ.get("FA_B200_NVCC_FLAGS", "").split()
    if not force and not extra and lib_path == LIB_PATH and not needs_build():
        return LIB_PATH
    nvcc = find_nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    flags = COMPILE_FLAGS + extra + (["-Xptxas", "-v"] if verbose else [])
    tag = hashlib.sha1(" ".join(COMPILE_FLAGS + extra).encode()).hexdigest()[:10]
    hdr_time = max(os.path.getmtime(h) for h in _headers())
    jobs, objs = [], []
    for src in sources():
        obj = os.path.join(OBJ_DIR, f"{os.path.splitext(os.path.basename(src))[0]}.{tag}.o")
        objs.append(obj)
        stale = force or verbose or not os.path.exists(obj) or \
            os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time)
        if stale:
            jobs.append([nvcc, *flags, "-I", INCLUDE, "-c", src, "-o", obj])
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        logs = list(pool.map(_run, jobs))
    if verbose:
        sys.stderr.write("".join(logs))
    _run([nvcc, *LINK_FLAGS, "-o", lib_path, *objs])
    return lib_path


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
