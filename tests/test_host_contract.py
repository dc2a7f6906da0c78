"""CPU tests of the boundary: the shared library exports what the header declares, the
ctypes table covers it, argument errors are reported before any CUDA work, and the
``cuda_ops`` mirror keeps the reference's public surface."""

import ctypes
import inspect
import re
from pathlib import Path

import pytest
import torch

from rnn_with_grm_b200 import cabi, cuda_ops
from rnn_with_grm_b200.build import build_all

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build_all()
    return cabi.load()


def declared_functions():
    text = (ROOT / "include" / "grmx.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(grmx_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = declared_functions()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/grmx.h but not exported"
        assert name in cabi.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(cabi.SIGNATURES) == names


def test_version_and_error_text(lib):
    assert lib.grmx_version() >= 100
    assert lib.grmx_chunk_scan_fwd(None, None, None, None, None, None, 1, 4, 0, 8, 0.97, 0, 0, 0, None) == 1
    assert b"K must be positive" in lib.grmx_last_error()
    assert lib.grmx_query_device(0, None) == 1


def test_argument_errors_need_no_gpu(lib):
    # every call below must be rejected (or be a no-op) before touching the device
    assert lib.grmx_apply_query_fwd(None, None, None, -1, 1, 1, 1, 0, None) == 1
    assert lib.grmx_apply_query_fwd(None, None, None, 0, 1, 1, 1, 0, None) == 0          # empty: no-op
    assert lib.grmx_apply_query_fwd(None, None, None, 2, 1, 1, 4, 0, None) == 1          # NULL tensors
    assert lib.grmx_batched_gather(None, None, None, 2, 3, 2, 16, 3, None) == 1          # elem size
    assert lib.grmx_batched_gather(None, None, None, 0, 3, 2, 16, 4, None) == 0
    assert lib.grmx_topk_route(None, None, None, 1, 1, 4, 8, 33, 1.0, 1.0, None, None, None, None) == 1
    assert b"top_k" in lib.grmx_last_error()
    assert lib.grmx_topk_route(None, None, None, 1, 1, 5000, 8, 4, 1.0, 1.0, None, None, None, None) == 1
    assert lib.grmx_topk_select(None, None, 0, 1, 4, 2, 1.0, None, None, None) == 0
    assert lib.grmx_retrieve_fuse(None, None, None, None, None, None, None, 1e-5, None, 1, 1, 1, 1, 4, 4, 7, None) == 1
    assert lib.grmx_retrieve_fuse(None, None, None, None, None, None, None, 1e-5, None, 1, 1, 1, 40, 4, 4, 0, None) == 1
    assert lib.grmx_linear_scan(None, None, None, None, 1, 1, None, None, 0, 4, 8, 8,
                                0.9, 0.1, 1.0, 1.0, 0, 0, 0, 0, 0, None) == 0           # B == 0
    assert lib.grmx_chunk_scan_bwd(*([None] * 10), 1, 4, 8, 8, 0.97, 0, 0, 0, None) == 1


def test_static_workspace_admission_is_decided_on_the_host(lib):
    # The allocation-free scan refuses a call whose cut needs more than the built-in array holds.  On a
    # B200 (148 multiprocessors) no shape gets there, so the decision is tested as the host computation
    # it is: the workspace a shape needs on a device of a given size, and the admission test on it.
    cap = lib.grmx_static_scratch_capacity()
    assert cap == 4 << 20
    state = 64 * 64 * 4
    on_b200 = lib.grmx_chunk_scan_scratch_bytes_on(64, 2048, 64, 64, 148)
    assert 0 < on_b200 <= cap and on_b200 % state == 0
    assert lib.grmx_static_scratch_admits(on_b200) == 0
    assert lib.grmx_static_scratch_admits(cap) == 0
    # a (fictitious) device of 4096 multiprocessors would cut 64 rows x 128 chunks far finer
    on_giant = lib.grmx_chunk_scan_scratch_bytes_on(64, 16384, 64, 64, 4096)
    assert on_giant > cap
    assert lib.grmx_static_scratch_admits(on_giant) == 2
    text = lib.grmx_last_error()
    assert b"built-in one holds 4194304" in text and str(on_giant).encode() in text
    assert lib.grmx_static_scratch_admits(cap + 1) == 2
    assert lib.grmx_static_scratch_admits(-1) == 1
    # wide heads are never cut over the workspace; a shape outside the tensor-core scan needs none
    assert lib.grmx_chunk_scan_scratch_bytes_on(8, 4096, 128, 128, 148) == 0
    assert lib.grmx_chunk_scan_scratch_bytes_on(0, 4096, 64, 64, 148) == 0


def test_cuda_ops_public_surface_matches_the_reference():
    assert cuda_ops.__all__ == [
        "cuda_apply_query", "cuda_batched_memory_gather", "cuda_chunk_update", "get_grm_cuda_runtime_status",
        "is_grm_cpp_extension_available", "is_grm_cuda_available", "load_grm_cuda_extension",
    ]
    sig = inspect.signature(cuda_ops.cuda_chunk_update)
    assert list(sig.parameters) == ["keys", "values", "queries", "memory", "memory_decay", "enabled", "debug_fallback"]
    for name in ("enabled", "debug_fallback"):
        assert sig.parameters[name].kind is inspect.Parameter.KEYWORD_ONLY
    assert list(inspect.signature(cuda_ops.cuda_apply_query).parameters) == ["memories", "queries", "enabled", "debug_fallback"]
    assert list(inspect.signature(cuda_ops.cuda_batched_memory_gather).parameters) == [
        "memories_per_batch", "topk_indices", "enabled", "debug_fallback"]


def test_runtime_status_schema(lib, monkeypatch):
    # the checks of the reference's status test (examples/test_grm.py:116-151)
    status = cuda_ops.get_grm_cuda_runtime_status()
    assert set(status) == {
        "load_attempted", "extension_loaded", "compiled_with_cuda_sources", "compiled_with_cuda_kernels",
        "torch_cuda_available", "cuda_backend_available", "load_error", "module_name", "registered_ops",
        "dispatch_kernels", "kernel_policy"}
    assert status["extension_loaded"] and status["compiled_with_cuda_sources"] and status["compiled_with_cuda_kernels"]
    assert status["load_error"] == "" and status["module_name"].endswith("grm_cuda_ext")
    assert set(status["kernel_policy"]) == {"global", "chunk_update", "apply_query", "batched_memory_gather"}
    assert set(status["kernel_policy"].values()) <= {"auto", "native", "fallback"}
    assert set(status["registered_ops"]) == set(status["dispatch_kernels"]) == {
        "chunk_update_forward", "chunk_update_backward", "apply_query_forward", "apply_query_backward",
        "batched_memory_gather"}
    assert all(entry["cuda"] for entry in status["dispatch_kernels"].values())
    assert status["cuda_backend_available"] == torch.cuda.is_available()
    monkeypatch.setenv("GRM_CUDA_KERNEL_POLICY", "native")
    monkeypatch.setenv("GRM_CUDA_APPLY_QUERY_POLICY", "FALLBACK ")
    monkeypatch.setenv("GRM_CUDA_BATCHED_GATHER_POLICY", "bogus")
    policy = cuda_ops.get_grm_cuda_runtime_status()["kernel_policy"]
    assert policy == {"global": "native", "chunk_update": "native", "apply_query": "fallback",
                      "batched_memory_gather": "native"}


def test_ops_refuse_cpu_tensors_and_fallback_requests(lib, monkeypatch):
    k = torch.zeros(1, 2, 4)
    with pytest.raises(RuntimeError, match="CUDA device"):
        cuda_ops.cuda_chunk_update(k, k, k, torch.zeros(1, 4, 4), 0.97)
    with pytest.raises(RuntimeError, match="fallback"):
        cuda_ops.cuda_batched_memory_gather(torch.zeros(1, 2, 3, 4), torch.zeros(1, 2, dtype=torch.long),
                                            debug_fallback=True)
    monkeypatch.setenv("GRM_CUDA_CHUNK_UPDATE_POLICY", "fallback")
    with pytest.raises(RuntimeError, match="fallback"):
        cuda_ops.cuda_chunk_update(k, k, k, torch.zeros(1, 4, 4), 0.97)
    with pytest.raises(NotImplementedError):          # no CPU kernel is registered with the dispatcher
        torch.ops.grm_cuda.batched_memory_gather(torch.zeros(1, 2, 3, 4), torch.zeros(1, 2, dtype=torch.long))


def test_install_as_grm_cuda_ops_serves_the_reference_import_path(lib):
    import sys

    cuda_ops.install_as_grm_cuda_ops()
    try:
        assert sys.modules["grm.core.cuda_ops"] is cuda_ops
    finally:
        sys.modules.pop("grm.core.cuda_ops", None)
