"""The reference's own op shim (core/torch/torch_bindings.cpp, unmodified, read where it lies) must compile against this
repository's include/ directory: same namespace, structs, signatures and exception types as core/include/bf16n/*.h.
Compile-only (the translation unit is parsed and type-checked by g++); skipped where the reference checkout is absent."""
import os
import subprocess
import sysconfig

import pytest

from oracle import cpu_oracle as o

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(o.reference_checkout() is None, reason="reference checkout not present")
def test_reference_torch_bindings_compile_against_our_headers():
    import torch.utils.cpp_extension as ext
    src = os.path.join(o.reference_checkout(), "core", "torch", "torch_bindings.cpp")
    cuda_home = os.environ.get("CUDA_HOME") or "/usr/local/cuda"
    inc = [os.path.join(ROOT, "include"), *ext.include_paths(), os.path.join(cuda_home, "include"), sysconfig.get_paths()["include"]]
    cmd = ["g++", "-std=c++17", "-fsyntax-only", "-DTORCH_EXTENSION_NAME=_C", *[f"-I{p}" for p in inc], src]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-4000:]
