"""The built extension registers every operator with a schema that matches its C++ signature.

``torch.ops.load_library`` checks each ``m.def`` schema against the bound function when the library is
loaded, so loading it is enough; no GPU is needed.  On a machine without the NVIDIA driver the CUDA
toolkit's stub ``libcuda`` stands in for ``libcuda.so.1`` (nothing is launched)."""

import os
import subprocess
import sys

import pytest

from torchtitan_b200.ops import ext

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_extension_loads_and_schemas_match(tmp_path):
    if not os.path.exists(ext.LIB_PATH):
        pytest.skip("extension not built")
    env = dict(os.environ)
    stub = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "lib64", "stubs", "libcuda.so")
    if os.path.exists(stub):
        os.symlink(stub, tmp_path / "libcuda.so.1")
        env["LD_LIBRARY_PATH"] = env.get("LD_LIBRARY_PATH", "") + os.pathsep + str(tmp_path)   # a real driver, if any, wins
    code = (
        "import torch\n"
        f"torch.ops.load_library({ext.LIB_PATH!r})\n"
        "ops = torch.ops.tb200\n"
        "for name in ('gemm_bf16', 'flash_fwd', 'flash_bwd', 'symm_barrier', 'gemm_allgather_bf16', 'adamw_allgather_',\n"
        "             'reduce_scatter_pull', 'all_gather_pull', 'rmsnorm_fwd'):\n"
        "    assert hasattr(ops, name), name\n"
        "print('ok')\n")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]
