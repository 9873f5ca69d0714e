"""The C++ surface (attention_hpc::BackendFactory / FlashAttention / PagedAttention).

CPU: the library exports the classes and the surface test binary links against it.
GPU: tests/cpp/test_surface (the reference's own test and example callers restated with seeded inputs,
checked against the C oracle) runs to completion.
"""
import os
import shutil
import subprocess

import pytest

from attention_b200 import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("nm") is None, reason="nm not installed")
def test_library_exports_the_cpp_classes(native_lib):
    out = subprocess.run(["nm", "-DC", "--defined-only", build.LIB_PATH], capture_output=True, text=True, check=True).stdout
    for symbol in ["attention_hpc::BackendFactory::createFlashAttention(attention_hpc::BackendType)",
                   "attention_hpc::BackendFactory::createPagedAttention(attention_hpc::BackendType)",
                   "attention_hpc::BackendFactory::registerBackend(",
                   "attention_hpc::FlashAttention::forward(",
                   "attention_hpc::FlashAttention::configure(",
                   "attention_hpc::PagedAttention::forward_batch(",
                   "attention_hpc::PagedAttention::append_kv_cache(",
                   "attention_hpc::PagedAttention::create_sequence("]:
        assert symbol in out, f"{symbol} is not exported"


def test_surface_binary_is_built_and_linked(native_lib):
    exe = build.cpp_test_binary()
    assert os.path.exists(exe), "tests/cpp/test_surface was not built (python -m attention_b200.build)"
    if shutil.which("ldd"):
        out = subprocess.run(["ldd", exe], capture_output=True, text=True).stdout
        assert "libahpc_b200.so" in out and "not found" not in out.split("libahpc_b200.so")[1].splitlines()[0]


def test_cpu_backend_is_not_offered_without_a_gpu(native_lib):
    """Without a device the factory must offer nothing: run the binary and expect its first check to fail."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    r = subprocess.run([build.cpp_test_binary()], capture_output=True, text=True)
    assert r.returncode != 0 and "isBackendAvailable(BackendType::CUDA)" in r.stdout


@pytest.mark.gpu
def test_reference_callers_restated_in_cpp():
    r = subprocess.run([build.cpp_test_binary()], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "checks passed" in r.stdout
