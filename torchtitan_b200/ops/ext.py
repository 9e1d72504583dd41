"""Loader for the in-tree sm_100a extension.

The shared object is built by :func:`build` (nvcc, ``-gencode
arch=compute_100a,code=sm_100a``) into ``torchtitan_b200/ops/_build`` and is
loaded with ``torch.ops.load_library``; its operators live under
``torch.ops.tb200``.  CUDA tensors require it: :func:`require` raises instead of
falling back to library kernels.
"""

from __future__ import annotations

import glob
import os
import subprocess
import sys
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
BUILD_DIR = os.path.join(_HERE, "_build")
LIB_NAME = "tb200_ops"
LIB_PATH = os.path.join(BUILD_DIR, f"lib{LIB_NAME}.so")

_lock = threading.Lock()
_loaded = False
_load_error: str | None = None

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "--expt-extended-lambda",
    "-DTORCH_EXTENSION_NAME=tb200_ops",
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    return any(os.path.getmtime(s) > t for s in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every source under ``csrc/`` into one shared object (in-tree)."""
    from torch.utils import cpp_extension as ce

    if not force and not _stale():
        return LIB_PATH
    os.makedirs(BUILD_DIR, exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    inc = []
    for p in ce.include_paths("cuda"):
        inc += ["-isystem", p]
    import sysconfig

    inc += ["-isystem", sysconfig.get_paths()["include"]]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(BUILD_DIR, os.path.basename(src) + ".o")
        objs.append(obj)
        deps = [src] + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
        if not force and os.path.exists(obj) and all(os.path.getmtime(d) <= os.path.getmtime(obj) for d in deps):
            continue
        cmd = [nvcc, "-c", src, "-o", obj, f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-I", CSRC] + NVCC_FLAGS + inc
        if src.endswith(".cpp"):
            cmd += ["-x", "cu"]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = []
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(f"--- nvcc {os.path.basename(src)} ---\n{out}\n")
        if p.returncode != 0:
            failed.append(src)
    if failed:
        raise RuntimeError(f"nvcc failed for: {failed}")
    libdirs = ce.library_paths("cuda")
    link = [nvcc, "-shared", "-o", LIB_PATH] + objs
    for d in libdirs:
        link += ["-L", d]
    link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcuda", "-lcudart"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("linking the extension failed")
    return LIB_PATH


def load() -> bool:
    """Load the built library if present; returns availability."""
    global _loaded, _load_error
    with _lock:
        if _loaded:
            return True
        if not os.path.exists(LIB_PATH):
            _load_error = f"{LIB_PATH} has not been built (run `python -m torchtitan_b200.ops.ext`)"
            return False
        try:
            torch.ops.load_library(LIB_PATH)
            _loaded = True
        except OSError as e:  # pragma: no cover - depends on the box
            _load_error = str(e)
        return _loaded


def available() -> bool:
    return load()


def require():
    """Return ``torch.ops.tb200`` or raise: CUDA tensors never fall back silently."""
    if not load():
        raise RuntimeError(
            "torchtitan_b200 CUDA operators were requested for a CUDA tensor but the sm_100a "
            f"extension is not loadable: {_load_error}"
        )
    return torch.ops.tb200


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
