"""The reference's own models on the GPU with this engine installed under them.

``install_as_grm_cuda_ops()`` puts the engine's op layer where the reference's models import
``grm.core.cuda_ops`` from (grm/core/paper_grm.py:15-20; the stacked model goes through the same layer,
grm/core/multilayer_grm.py:71-98).  The reference package itself is imported untouched from the copy the
oracle recipe stages under ``oracle/_ref/python``; the comparison arm is the same model run on the CPU
through the reference's own PyTorch fallback in a separate interpreter (``tests/reference_models.py``),
where the engine is not installed.  Forward results at the fp32 tolerance, gradients (which pass
through ``ChunkUpdateCudaFn.backward`` and ``ApplyQueryCudaFn.backward``) at the gradient tolerance.
"""

import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from oracle import grm_oracle as go

pytestmark = pytest.mark.gpu

HERE = Path(__file__).resolve().parent
FP32_TOL = 1e-5
FP32_GRAD_TOL = 5e-5
DEV = "cuda:0"


@pytest.fixture(scope="module")
def reference_on_cpu(tmp_path_factory):
    staged = oracle.reference_python()
    if staged is None:
        pytest.skip("the reference package is not staged under oracle/_ref/python (python oracle/build_oracle.py)")
    out = tmp_path_factory.mktemp("refcpu") / "reference_cpu.npz"
    subprocess.run([sys.executable, str(HERE / "reference_models.py"), "--python-path", str(staged), "--out", str(out)],
                   check=True, timeout=600)
    with np.load(out) as data:
        return {k: data[k] for k in data.files}


@pytest.fixture(scope="module")
def grm_on_engine():
    staged = oracle.reference_python()
    if staged is None:
        pytest.skip("the reference package is not staged under oracle/_ref/python (python oracle/build_oracle.py)")
    from rnn_with_grm_b200 import cuda_ops as engine

    assert not any(name == "grm" or name.startswith("grm.") for name in sys.modules), "grm was imported before the engine was installed"
    engine.install_as_grm_cuda_ops()
    sys.path.insert(0, str(staged))
    try:
        import grm
        import grm.core.multilayer_grm
        import grm.core.paper_grm
        yield grm, engine
    finally:
        sys.path.remove(str(staged))
        for name in [n for n in sys.modules if n == "grm" or n.startswith("grm.")]:
            sys.modules.pop(name, None)


def test_reference_modules_bind_the_engine_ops(grm_on_engine):
    grm, engine = grm_on_engine
    from grm.core import paper_grm

    assert paper_grm.cuda_chunk_update is engine.cuda_chunk_update
    assert paper_grm.cuda_apply_query is engine.cuda_apply_query
    assert paper_grm.cuda_batched_memory_gather is engine.cuda_batched_memory_gather
    assert grm.cuda_chunk_update is engine.cuda_chunk_update and grm.get_grm_cuda_runtime_status is engine.get_grm_cuda_runtime_status
    # the reference's runtime-status test (examples/test_grm.py:116-151) on the status the models see
    status = grm.get_grm_cuda_runtime_status()
    required = {"load_attempted", "extension_loaded", "compiled_with_cuda_sources", "compiled_with_cuda_kernels",
                "torch_cuda_available", "cuda_backend_available", "load_error", "module_name", "registered_ops",
                "dispatch_kernels", "kernel_policy"}
    assert required <= set(status)
    assert set(status["kernel_policy"]) == {"global", "chunk_update", "apply_query", "batched_memory_gather"}
    assert all(v in {"auto", "native", "fallback"} for v in status["kernel_policy"].values())
    assert status["extension_loaded"] and status["compiled_with_cuda_kernels"] and status["cuda_backend_available"]
    assert all(entry["cuda"] for entry in status["dispatch_kernels"].values())


@pytest.mark.parametrize("name", ["single", "stack"])
def test_reference_model_forward_and_backward_through_the_engine(grm_on_engine, reference_on_cpu, name):
    _, engine = grm_on_engine
    sys.path.insert(0, str(HERE))
    import reference_models

    from rnn_with_grm_b200 import cabi

    model, x = reference_models.build(name)
    launches_before = cabi.load().grmx_launch_count()
    got = reference_models.run(model.to(DEV), x.to(DEV))
    engine.check_device_errors()
    assert cabi.load().grmx_launch_count() - launches_before >= 8       # the engine's kernels ran, forward and backward
    want = {k[len(name) + 2:]: v for k, v in reference_on_cpu.items() if k.startswith(name + "::")}
    assert set(got) == set(want) and any(k.startswith("grad::") and "memory_cell" in k for k in got)
    for key in ("outputs", "h_final", "memory_final", "loss"):
        assert go.rel_err(got[key], want[key]) < FP32_TOL, key
    for key in sorted(k for k in got if k.startswith("grad::")):
        assert np.isfinite(got[key]).all()
        assert go.rel_err(got[key], want[key]) < FP32_GRAD_TOL, key
