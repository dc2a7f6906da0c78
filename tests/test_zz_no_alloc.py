"""The allocation-free entry point, checked against the entry point that takes a workspace.

Who needs it: a host that cannot call cudaMalloc where it runs the scan -- an inference server
whose memory pool already owns the whole device, a callback with a latency bound that an
allocation could break, a plugin that is handed nothing but its input and output buffers.
``grmx_chunk_scan_fwd_static`` keeps its workspace in a fixed array inside the library, so the
call allocates nothing; this test calls it twice in a row through the C ABI and compares each
result with ``grmx_chunk_scan_fwd_ws`` on the same inputs.

The file name makes pytest collect it last, so that a run stopping at the first failure has
already been through every other test.
"""

import numpy as np
import pytest
import torch

from rnn_with_grm_b200 import cabi

import grmx_calls as gx

pytestmark = pytest.mark.gpu

LOWP_TOL = 2e-2   # tolerance of the bf16 tests; the two entry points run the same kernels


def _inputs(seed, B, T):
    g = torch.Generator(device="cuda:0").manual_seed(seed)
    k = torch.nn.functional.normalize(torch.randn(B, T, 64, device="cuda:0", generator=g), dim=-1)
    q = torch.nn.functional.normalize(torch.randn(B, T, 64, device="cuda:0", generator=g), dim=-1)
    v = torch.randn(B, T, 64, device="cuda:0", generator=g)
    m = torch.randn(B, 64, 64, device="cuda:0", generator=g)
    return k.bfloat16(), v.bfloat16(), q.bfloat16(), m


def _static_call(k, v, q, m, decay):
    lib = cabi.load()
    B, T, K = k.shape
    hidden = torch.empty_like(v)
    m_out = torch.empty_like(m)
    cabi.check(lib.grmx_chunk_scan_fwd_static(cabi.ptr(k), cabi.ptr(v), cabi.ptr(q), cabi.ptr(m), cabi.ptr(hidden),
                                              cabi.ptr(m_out), B, T, K, v.shape[2], decay, cabi.current_stream()))
    return hidden, m_out


def _rel(a, b):
    a, b = a.float(), b.float()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def test_static_workspace_scan_matches_workspace_entry_twice_in_a_row():
    lib = cabi.load()
    assert lib.grmx_static_scratch_capacity() == 4 << 20
    for call, (seed, B, T) in enumerate([(11, 8, 2048), (12, 5, 1000)]):
        k, v, q, m = _inputs(seed, B, T)
        nbytes = gx.chunk_scan_scratch_bytes(B, T, 64, 64, torch.bfloat16, torch.float32)
        assert 0 < nbytes <= lib.grmx_static_scratch_capacity()          # the cut path is exercised
        scratch = torch.empty(nbytes, device="cuda:0", dtype=torch.uint8)
        want_h, want_m = gx.chunk_scan_fwd_ws(k, v, q, m, 0.97, scratch)
        got_h, got_m = _static_call(k, v, q, m, 0.97)
        torch.cuda.synchronize()
        assert _rel(got_h, want_h) < LOWP_TOL and _rel(got_m, want_m) < LOWP_TOL, f"call {call}"
        assert torch.equal(got_h, want_h) and torch.equal(got_m, want_m)   # same kernels, same order of sums
    assert cabi.device_error_word() == 0


def test_static_workspace_scan_refuses_what_it_cannot_hold():
    lib = cabi.load()
    k, v, q, m = _inputs(13, 2, 256)
    # d_k = 32 is outside what the tensor-core scan covers: refused, nothing runs
    rc = lib.grmx_chunk_scan_fwd_static(cabi.ptr(k), cabi.ptr(v), cabi.ptr(q), cabi.ptr(m), cabi.ptr(v), cabi.ptr(m),
                                        2, 256, 32, 64, 0.97, cabi.current_stream())
    assert rc == 2 and b"multiples of 64" in lib.grmx_last_error()
    # a call that needs no cut still works (it simply does not touch the workspace)
    got_h, got_m = _static_call(k, v, q, m, 0.97)
    want_h, want_m = gx.chunk_scan_fwd(k, v, q, m, 0.97, cabi.PATH_TCGEN05)
    assert torch.equal(got_h, want_h) and torch.equal(got_m, want_m)
