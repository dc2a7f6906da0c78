"""The reference-facing layer on a GPU: ``cuda_ops`` entry points, ``torch.ops.grm_cuda.*``,
autograd, and the runtime status (mirrors examples/test_grm.py tests 7-10 of the reference,
with the oracle standing in for its ``debug_fallback=True`` arm)."""

import numpy as np
import pytest
import torch

from oracle import grm_oracle as go
from rnn_with_grm_b200 import cuda_ops

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
FP32_TOL = 1e-5
FP32_GRAD_TOL = 5e-5


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t.to(dtype) if dtype is not None else t


def close(actual, expected, tol):
    err = go.rel_err(actual.detach().float().cpu().numpy(), expected)
    assert err < tol, f"rel err {err:.3e} >= {tol:.1e}"


def test_runtime_status_on_gpu():
    status = cuda_ops.get_grm_cuda_runtime_status()
    assert status["extension_loaded"] and status["compiled_with_cuda_sources"]
    assert status["compiled_with_cuda_kernels"] and status["cuda_backend_available"]
    assert all(status["registered_ops"].values())
    assert all(entry["cuda"] for entry in status["dispatch_kernels"].values())
    assert cuda_ops.is_grm_cuda_available() and cuda_ops.is_grm_cpp_extension_available()


@pytest.mark.parametrize("name", ["small", "ragged", "long"])
def test_cuda_chunk_update_forward_and_autograd(golden, name):
    g = golden(f"chunk_update_{name}")
    leaves = [dev(g[k]).requires_grad_(True) for k in ("keys", "values", "queries", "memory")]
    hidden, m_out = cuda_ops.cuda_chunk_update(*leaves, memory_decay=float(g["decay"]))
    close(hidden, g["hidden"], FP32_TOL)
    close(m_out, g["memory_out"], FP32_TOL)
    (hidden.square().mean() + m_out.square().mean()).backward()      # loss of examples/test_grm.py:88
    for leaf, key in zip(leaves, ("grad_keys", "grad_values", "grad_queries", "grad_memory")):
        close(leaf.grad, g[key], FP32_GRAD_TOL)


def test_cuda_chunk_update_mixed_precision_autograd():
    rng = np.random.default_rng(3)
    k = torch.nn.functional.normalize(dev(rng.standard_normal((2, 64, 64)).astype(np.float32)), dim=-1)
    q = torch.nn.functional.normalize(dev(rng.standard_normal((2, 64, 64)).astype(np.float32)), dim=-1)
    v = dev(rng.standard_normal((2, 64, 64)).astype(np.float32))
    m = dev(rng.standard_normal((2, 64, 64)).astype(np.float32))
    leaves = [t.to(torch.bfloat16).requires_grad_(True) for t in (k, v, q)] + [m.clone().requires_grad_(True)]
    hidden, m_out = cuda_ops.cuda_chunk_update(*leaves, memory_decay=0.97)
    assert hidden.dtype == torch.bfloat16 and m_out.dtype == torch.float32
    (hidden.float().square().mean() + m_out.square().mean()).backward()
    f = [t.detach().float().cpu().numpy() for t in leaves]
    want_h, want_m = go.chunk_update_sequential(*f, 0.97)
    close(hidden, want_h, 2e-2)
    close(m_out, want_m, 2e-2)
    want = go.chunk_update_backward(2 * want_h / want_h.size, 2 * want_m / want_m.size, *f, 0.97)
    for leaf, w in zip(leaves, want):
        assert leaf.grad.dtype == leaf.dtype
        close(leaf.grad, w, 3e-2)


def test_cuda_chunk_update_accepts_non_contiguous_and_empty():
    rng = np.random.default_rng(4)
    k = dev(rng.standard_normal((2, 8, 16)).astype(np.float32))
    v = dev(rng.standard_normal((2, 12, 8)).astype(np.float32)).transpose(1, 2)      # [2,8,12] strided
    q = dev(rng.standard_normal((2, 8, 16)).astype(np.float32))
    m = dev(rng.standard_normal((2, 12, 16)).astype(np.float32))
    hidden, m_out = cuda_ops.cuda_chunk_update(k, v, q, m, 0.97)
    want_h, want_m = go.chunk_update_sequential(*(t.cpu().numpy() for t in (k, v, q, m)), 0.97)
    close(hidden, want_h, FP32_TOL)
    hidden0, m0 = cuda_ops.cuda_chunk_update(k[:, :0], v[:, :0], q[:, :0], m, 0.97)
    assert hidden0.shape == (2, 0, 12) and torch.equal(m0, m)


def test_cuda_apply_query_and_autograd(golden):
    g = golden("apply_query")
    for tag in ("r5", "r4"):
        mem = dev(g[f"{tag}_memories"]).requires_grad_(True)
        qry = dev(g[f"{tag}_queries"]).requires_grad_(True)
        hidden = cuda_ops.cuda_apply_query(mem, qry)
        close(hidden, g[f"{tag}_hidden"], FP32_TOL)
        hidden.square().mean().backward()
        close(mem.grad, g[f"{tag}_grad_memories"], FP32_TOL)
        close(qry.grad, g[f"{tag}_grad_queries"], FP32_TOL)
    with pytest.raises(ValueError):
        cuda_ops.cuda_apply_query(torch.zeros(2, 3, 4, device=DEV), torch.zeros(2, 4, device=DEV))


def test_cuda_batched_memory_gather(golden):
    g = golden("gather")
    mem = dev(g["memories"])
    out3 = cuda_ops.cuda_batched_memory_gather(mem, dev(g["idx3"]))
    out2 = cuda_ops.cuda_batched_memory_gather(mem, dev(g["idx2"]).to(torch.int32))   # any integer dtype
    assert np.array_equal(out3.cpu().numpy(), g["out3"]) and np.array_equal(out2.cpu().numpy(), g["out2"])
    with pytest.raises(ValueError):
        cuda_ops.cuda_batched_memory_gather(mem[0], dev(g["idx2"]))
    with pytest.raises(RuntimeError, match="batch dim mismatch"):
        torch.ops.grm_cuda.batched_memory_gather(mem, dev(g["idx2"])[:1])


def test_shape_errors_carry_the_reference_messages():
    z = lambda *s: torch.zeros(*s, device=DEV)
    with pytest.raises(RuntimeError, match=r"keys must have shape \[B, T, K\]"):
        torch.ops.grm_cuda.chunk_update_forward(z(2, 4), z(2, 4, 3), z(2, 4, 5), z(2, 3, 5), 0.97)
    with pytest.raises(RuntimeError, match="memory key dim must match keys key dim"):
        torch.ops.grm_cuda.chunk_update_forward(z(2, 4, 5), z(2, 4, 3), z(2, 4, 5), z(2, 3, 6), 0.97)
    with pytest.raises(RuntimeError, match="queries must have shape"):
        torch.ops.grm_cuda.apply_query_forward(z(2, 3, 4, 5), z(2, 3, 5))


def test_cpu_tensors_and_fallback_requests_fail_loudly():
    k = torch.zeros(1, 2, 4)
    with pytest.raises(RuntimeError, match="CUDA device"):
        cuda_ops.cuda_chunk_update(k, k, k, torch.zeros(1, 4, 4), 0.97)
    kd = k.to(DEV)
    with pytest.raises(RuntimeError, match="fallback"):
        cuda_ops.cuda_chunk_update(kd, kd, kd, torch.zeros(1, 4, 4, device=DEV), 0.97, debug_fallback=True)
    with pytest.raises(RuntimeError, match="fallback"):
        cuda_ops.cuda_apply_query(torch.zeros(1, 1, 4, 4, device=DEV), torch.zeros(1, 4, device=DEV), enabled=False)
    with pytest.raises(NotImplementedError):
        torch.ops.grm_cuda.apply_query_forward(torch.zeros(1, 1, 4, 4), torch.zeros(1, 4))
