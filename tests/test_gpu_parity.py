"""GPU parity: the CUDA path, called through the C ABI, against the oracle.

Tolerances (relative to the largest reference magnitude, ``oracle.rel_err``):
float32 mode 1e-5; bf16/fp16 inputs with float32 state 2e-2; gathered
matrices, routing scores and top-k indices bit for bit.
"""

import numpy as np
import pytest
import torch

import oracle
from oracle import grm_oracle as go
from rnn_with_grm_b200 import cabi

import grmx_calls as gx

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
FP32_GRAD_TOL = 5e-5   # the golden gradients are float32 results of the reference (see test_oracle.py)
LOWP_TOL = 2e-2
DEV = "cuda:0"


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t.to(dtype) if dtype is not None else t


def host(t):
    return t.detach().float().cpu().numpy()


def close(actual, expected, tol):
    err = go.rel_err(host(actual) if isinstance(actual, torch.Tensor) else actual, expected)
    assert err < tol, f"rel err {err:.3e} >= {tol:.1e}"


def make_chunk(seed, B, T, K, H, zero_state=False):
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((B, T, K)).astype(np.float32)
    q = rng.standard_normal((B, T, K)).astype(np.float32)
    k /= np.maximum(np.linalg.norm(k, axis=-1, keepdims=True), 1e-6)
    q /= np.maximum(np.linalg.norm(q, axis=-1, keepdims=True), 1e-6)
    v = rng.standard_normal((B, T, H)).astype(np.float32)
    m = np.zeros((B, H, K), np.float32) if zero_state else rng.standard_normal((B, H, K)).astype(np.float32)
    return k, v, q, m


# --------------------------------------------------------------------------- chunk scan, fp32

@pytest.mark.parametrize("name", ["small", "ragged", "cfg1", "long"])
def test_chunk_scan_matches_reference_fixture(golden, name):
    g = golden(f"chunk_update_{name}")
    decay = float(g["decay"])
    hidden, m_out = gx.chunk_scan_fwd(dev(g["keys"]), dev(g["values"]), dev(g["queries"]), dev(g["memory"]),
                                      decay, cabi.PATH_FFMA)
    close(hidden, g["hidden"], FP32_TOL)
    close(m_out, g["memory_out"], FP32_TOL)
    grads = gx.chunk_scan_bwd(dev(g["grad_hidden"]), dev(g["grad_memory_out"]), dev(g["keys"]), dev(g["values"]),
                              dev(g["queries"]), dev(g["memory"]), decay, cabi.PATH_FFMA)
    for got, key in zip(grads, ("grad_keys", "grad_values", "grad_queries", "grad_memory")):
        close(got, g[key], FP32_GRAD_TOL)


@pytest.mark.parametrize("K", [1, 2, 7, 8, 16, 33, 64, 128, 200])
@pytest.mark.parametrize("H,T", [(1, 1), (5, 17), (32, 16), (33, 100), (128, 64)])
def test_chunk_scan_shape_sweep(K, H, T):
    k, v, q, m = make_chunk(K * 1000 + H * 10 + T, 2, T, K, H)
    want_h, want_m = go.chunk_update_sequential(k, v, q, m, 0.97)
    hidden, m_out = gx.chunk_scan_fwd(dev(k), dev(v), dev(q), dev(m), 0.97, cabi.PATH_FFMA)
    close(hidden, want_h, FP32_TOL)
    close(m_out, want_m, FP32_TOL)


def test_chunk_scan_backward_seeded():
    k, v, q, m = make_chunk(77, 3, 45, 24, 40)
    rng = np.random.default_rng(78)
    gh = rng.standard_normal((3, 45, 40)).astype(np.float32)
    gm = rng.standard_normal((3, 40, 24)).astype(np.float32)
    want = go.chunk_update_backward(gh, gm, k, v, q, m, 0.9)
    got = gx.chunk_scan_bwd(dev(gh), dev(gm), dev(k), dev(v), dev(q), dev(m), 0.9, cabi.PATH_FFMA)
    for a, b in zip(got, want):
        close(a, b, FP32_TOL)


def test_chunk_scan_degenerate_calls():
    k, v, q, m = make_chunk(5, 2, 4, 8, 16)
    # zero tokens: state passes through (grm/csrc/grm_cuda.cpp:59-65)
    hidden, m_out = gx.chunk_scan_fwd(dev(k[:, :0]), dev(v[:, :0]), dev(q[:, :0]), dev(m), 0.97)
    assert hidden.shape == (2, 0, 16) and torch.equal(m_out, dev(m))
    gk, gv, gq, gmem = gx.chunk_scan_bwd(dev(v[:, :0]), dev(m), dev(k[:, :0]), dev(v[:, :0]), dev(q[:, :0]),
                                         dev(m), 0.97)
    assert torch.equal(gmem, dev(m))
    # zero batch rows
    hidden, m_out = gx.chunk_scan_fwd(dev(k[:0]), dev(v[:0]), dev(q[:0]), dev(m[:0]), 0.97)
    assert hidden.numel() == 0 and m_out.numel() == 0


def test_chunk_scan_is_independent_of_call_splitting():
    k, v, q, m = make_chunk(9, 4, 256, 64, 64)
    tk, tv, tq, tm = dev(k), dev(v), dev(q), dev(m)
    whole_h, whole_m = gx.chunk_scan_fwd(tk, tv, tq, tm, 0.97, cabi.PATH_FFMA)
    state, pieces = tm, []
    for s in range(0, 256, 64):
        h, state = gx.chunk_scan_fwd(tk[:, s:s + 64].contiguous(), tv[:, s:s + 64].contiguous(),
                                     tq[:, s:s + 64].contiguous(), state, 0.97, cabi.PATH_FFMA)
        pieces.append(h)
    # the fp32 kernel is token-serial, so splitting the call changes nothing, bit for bit
    assert torch.equal(torch.cat(pieces, dim=1), whole_h) and torch.equal(state, whole_m)
    again_h, again_m = gx.chunk_scan_fwd(tk, tv, tq, tm, 0.97, cabi.PATH_FFMA)
    assert torch.equal(again_h, whole_h) and torch.equal(again_m, whole_m)


@pytest.mark.parametrize("io,state,tol", [(torch.bfloat16, torch.float32, LOWP_TOL),
                                         (torch.bfloat16, torch.bfloat16, 5e-2),
                                         (torch.float16, torch.float32, LOWP_TOL),
                                         (torch.float16, torch.float16, LOWP_TOL)])
def test_chunk_scan_low_precision_inputs(io, state, tol):
    k, v, q, m = make_chunk(21, 3, 96, 64, 64)
    tk, tv, tq = dev(k, io), dev(v, io), dev(q, io)
    tm = dev(m, state)
    # oracle on exactly the rounded inputs, in float64
    want_h, want_m = go.chunk_update_sequential(host(tk), host(tv), host(tq), host(tm), 0.97)
    hidden, m_out = gx.chunk_scan_fwd(tk, tv, tq, tm, 0.97, cabi.PATH_FFMA)
    assert hidden.dtype == io and m_out.dtype == state
    close(hidden, want_h, tol)
    close(m_out, want_m, tol)


@pytest.mark.parametrize("reverse", [False, True])
@pytest.mark.parametrize("no_decay_first", [False, True])
def test_linear_scan_general_form(reverse, no_decay_first):
    k, v, q, m = make_chunk(31, 2, 37, 12, 20)
    want_h, want_m = go.linear_scan(k, v, q, m, 0.93, 0.31, hidden_scale=1.7, memory_out_scale=0.6,
                                    reverse=reverse, first_step_no_decay=no_decay_first)
    hidden, m_out = gx.linear_scan(dev(k), dev(v), dev(q), dev(m), 0.93, 0.31, 1.7, 0.6, reverse, no_decay_first,
                                   cabi.PATH_FFMA)
    close(hidden, want_h, FP32_TOL)
    close(m_out, want_m, FP32_TOL)
    # the same state handed over transposed
    m_t = np.ascontiguousarray(m.transpose(0, 2, 1))
    hidden_t, m_out_t = gx.linear_scan(dev(k), dev(v), dev(q), dev(m_t), 0.93, 0.31, 1.7, 0.6, reverse,
                                       no_decay_first, cabi.PATH_FFMA, transposed_state=True)
    assert torch.equal(hidden_t, hidden) and torch.equal(m_out_t, m_out)


def test_chunk_scan_rejects_bad_arguments():
    lib = cabi.load()
    k, v, q, m = (dev(a) for a in make_chunk(1, 1, 4, 8, 8))
    out_h, out_m = torch.empty_like(v), torch.empty_like(m)
    args = [cabi.ptr(k), cabi.ptr(v), cabi.ptr(q), cabi.ptr(m), cabi.ptr(out_h), cabi.ptr(out_m)]
    assert lib.grmx_chunk_scan_fwd(*args, 1, 4, 0, 8, 0.97, 0, 0, 0, None) == 1          # K == 0
    assert lib.grmx_chunk_scan_fwd(*args, 1, 4, 8, 8, 0.97, 7, 0, 0, None) == 1          # bad dtype
    assert lib.grmx_chunk_scan_fwd(*args, 1, 4, 8, 8, 0.97, 0, 1, 0, None) == 1          # state dtype != io, != f32
    assert lib.grmx_chunk_scan_fwd(*args, 1, 4, 300, 8, 0.97, 0, 0, 1, None) == 2        # K > 256 unsupported
    assert b"key dim" in lib.grmx_last_error()
    with pytest.raises(cabi.GrmxError):
        gx.chunk_scan_fwd(k, v, q, m, 0.97, path=9)


# --------------------------------------------------------------------------- apply query

def test_apply_query_matches_reference_fixture(golden):
    g = golden("apply_query")
    for tag in ("r5", "r4"):
        mem, qry = dev(g[f"{tag}_memories"]), dev(g[f"{tag}_queries"])
        close(gx.apply_query_fwd(mem, qry), g[f"{tag}_hidden"], FP32_TOL)
        gm, gq = gx.apply_query_bwd(dev(g[f"{tag}_grad_hidden"]), mem, qry)
        close(gm, g[f"{tag}_grad_memories"], FP32_TOL)
        close(gq, g[f"{tag}_grad_queries"], FP32_TOL)


@pytest.mark.parametrize("shape", [(3, 2, 64, 64), (2, 5, 4, 128, 64), (4, 1, 7, 6), (2, 3, 300, 20), (1, 2, 9, 513)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_TOL), (torch.bfloat16, LOWP_TOL), (torch.float16, LOWP_TOL)])
def test_apply_query_shapes_and_dtypes(shape, dtype, tol):
    rng = np.random.default_rng(sum(shape))
    mem = dev(rng.standard_normal(shape).astype(np.float32), dtype)
    qry = dev(rng.standard_normal(shape[:-3] + shape[-1:]).astype(np.float32), dtype)
    want = go.apply_query(host(mem), host(qry))
    close(gx.apply_query_fwd(mem, qry), want, tol)
    gh = dev(rng.standard_normal(shape[:-1]).astype(np.float32), dtype)
    want_gm, want_gq = go.apply_query_backward(host(gh), host(mem), host(qry))
    gm, gq = gx.apply_query_bwd(gh, mem, qry)
    close(gm, want_gm, tol)
    close(gq, want_gq, tol)


# --------------------------------------------------------------------------- gather

def test_gather_matches_reference_fixture_bit_for_bit(golden):
    g = golden("gather")
    mem = dev(g["memories"])
    assert np.array_equal(host(gx.batched_gather(mem, dev(g["idx3"]))), g["out3"])
    assert np.array_equal(host(gx.batched_gather(mem, dev(g["idx2"]))), g["out2"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hk", [(64, 64), (5, 3), (128, 64), (7, 2)])
def test_gather_random_bit_exact(dtype, hk):
    rng = np.random.default_rng(hk[0])
    B, S, Q, R = 3, 11, 5, 4
    mem = dev(rng.standard_normal((B, S) + hk).astype(np.float32), dtype)
    idx = dev(rng.integers(0, S, size=(B, Q, R)))
    out = gx.batched_gather(mem, idx)
    want, bad = oracle.c_batched_gather(mem.cpu().view(torch.int16 if dtype != torch.float32 else torch.int32).numpy(),
                                        idx.cpu().numpy())
    assert bad == 0
    got = out.cpu().view(torch.int16 if dtype != torch.float32 else torch.int32).numpy()
    assert np.array_equal(got, want)


def test_gather_empty_slots_and_bad_indices():
    lib = cabi.load()
    cabi.check(lib.grmx_device_error_reset(cabi.current_stream()))
    mem = dev(np.arange(2 * 3 * 4 * 4, dtype=np.float32).reshape(2, 3, 4, 4))
    out = gx.batched_gather(mem, dev(np.array([[2, -1], [0, 1]])))
    assert torch.equal(out[0, 0], mem[0, 2]) and not out[0, 1].any()
    assert cabi.device_error_word() == 0                      # -1 is the empty-slot marker
    out = gx.batched_gather(mem, dev(np.array([[3, 0], [0, -2]])))
    assert not out[0, 0].any() and not out[1, 1].any() and torch.equal(out[0, 1], mem[0, 0])
    assert cabi.device_error_word() & 1
    cabi.check(lib.grmx_device_error_reset(cabi.current_stream()))
    assert cabi.device_error_word() == 0
    # empty archive / empty index list
    assert gx.batched_gather(mem[:, :0], dev(np.zeros((2, 0), dtype=np.int64))).shape == (2, 0, 4, 4)


@pytest.mark.parametrize("H,K", [(64, 64), (5, 3), (512, 64)])
def test_archive_push_writes_the_slot_and_its_bf16_copy(H, K):
    rng = np.random.default_rng(29 + H)
    B, S = 3, 4
    archive = dev(rng.standard_normal((B, S, H, K)).astype(np.float32))
    shadow = archive.to(torch.bfloat16)
    before, before_shadow = archive.clone(), shadow.clone()
    memory = dev(rng.standard_normal((B, H, K)).astype(np.float32))
    gx.archive_push(memory, archive, shadow, 2)
    gx.archive_push(memory, archive, None, 0)                  # without the bf16 ring
    before[:, 2] = memory
    before[:, 0] = memory
    before_shadow[:, 2] = memory.to(torch.bfloat16)
    assert torch.equal(archive, before) and torch.equal(shadow, before_shadow)
    lib = cabi.load()
    rc = lib.grmx_archive_push(cabi.ptr(memory), cabi.ptr(archive), None, B, S, S, H * K, cabi.current_stream())
    assert rc == 1 and b"slot" in lib.grmx_last_error()        # GRMX_ERR_ARG, nothing launched


@pytest.mark.parametrize("N,K", [(1, 8), (7, 64), (1000, 64), (33, 128), (5, 512), (64, 24)])
def test_normalize_rows_matches_normalize_in_float64(N, K):
    rng = np.random.default_rng(71 + K)
    x = rng.standard_normal((N, K)).astype(np.float32)
    x[0] = 0.0                                                 # a zero row stays zero (the eps clamp)
    if N > 2:
        x[2] *= 1e-9                                           # norm below eps: divided by eps, not by the norm
    def want(v):
        v = v.astype(np.float64)
        return v / np.maximum(np.linalg.norm(v, axis=-1, keepdims=True), 1e-6)
    close(gx.normalize_rows(dev(x)), want(x), FP32_TOL)
    xb = dev(x, torch.bfloat16)
    close(gx.normalize_rows(xb), want(host(xb)), LOWP_TOL)
    close(gx.normalize_rows(dev(x), out_dtype=torch.bfloat16), want(x), LOWP_TOL)
    inplace = dev(x)
    lib = cabi.load()
    cabi.check(lib.grmx_normalize_rows(cabi.ptr(inplace), cabi.ptr(inplace), N, K, 1e-6, cabi.F32, cabi.F32,
                                       cabi.current_stream()))
    assert torch.equal(inplace, gx.normalize_rows(dev(x)))
    rc = lib.grmx_normalize_rows(cabi.ptr(inplace), cabi.ptr(inplace), 1, 6, 1e-6, cabi.F32, cabi.F32, cabi.current_stream())
    assert rc == 2 and b"16-byte" in lib.grmx_last_error()      # GRMX_ERR_UNSUPPORTED: the caller keeps F.normalize


@pytest.mark.parametrize("rows,D,with_bias", [(128, 64, True), (1000, 512, True), (4096 + 77, 192, False), (5, 128, True)])
def test_project_normalize_matches_linear_then_normalize(rows, D, with_bias):
    """Key and query projections with the normalisation in the epilogue against x W^T + b followed by
    F.normalize in float64 (the bf16 values of x and W, fp32 bias)."""
    rng = np.random.default_rng(71 + rows)
    x = dev(rng.standard_normal((rows, D)).astype(np.float32), torch.bfloat16)
    w = dev((rng.standard_normal((128, D)) / np.sqrt(D)).astype(np.float32), torch.bfloat16)
    bias = dev(rng.standard_normal(128).astype(np.float32) * 0.1) if with_bias else None
    a, b = gx.project_normalize(x, w, bias)
    y = host(x).astype(np.float64) @ host(w).astype(np.float64).T + (host(bias).astype(np.float64) if with_bias else 0.0)
    for got, want in ((a, y[:, :64]), (b, y[:, 64:])):
        want = want / np.maximum(np.linalg.norm(want, axis=-1, keepdims=True), 1e-6)
        close(got, want, LOWP_TOL)
        assert float((got.float().norm(dim=-1) - 1).abs().max()) < 1e-2
    # a zero row stays zero (norm below eps), as F.normalize leaves it
    x[3] = 0
    a0, _ = gx.project_normalize(x, w, None)
    assert float(a0[3].float().abs().max()) == 0.0
    lib = cabi.load()
    rc = lib.grmx_project_normalize(cabi.ptr(x), cabi.ptr(w), None, cabi.ptr(a), cabi.ptr(b), rows, D, 32, 1e-6, cabi.current_stream())
    assert rc == 2 and b"width 64" in lib.grmx_last_error()
    assert cabi.device_error_word() == 0


# --------------------------------------------------------------------------- routing

def test_topk_route_bit_exact_against_c_oracle():
    rng = np.random.default_rng(41)
    B, Q, S, D, top_k = 6, 9, 32, 64, 4
    qv = rng.standard_normal((B, Q, D)).astype(np.float32)
    kv = rng.standard_normal((B, S, D)).astype(np.float32)
    visible = np.array([0, 1, 3, 4, 5, 9, 17, 32, 40], dtype=np.int32)
    want_scores = oracle.c_route_scores(qv, kv, 0.125)
    want_idx, want_gates = oracle.c_topk_select(want_scores, top_k, 0.7, visible)
    idx, gates, scores = gx.topk_route(dev(qv), dev(kv), top_k, 0.125, 0.7, dev(visible))
    assert np.array_equal(host(scores), want_scores)          # same fused multiply-add order
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    close(gates, want_gates, FP32_TOL)
    idx2, gates2, _ = gx.topk_route(dev(qv), dev(kv), top_k, 0.125, 0.7, dev(visible), want_scores=False)
    assert torch.equal(idx2, idx) and torch.equal(gates2, gates)


@pytest.mark.parametrize("B,Q,S,D,top_k", [(2, 64, 1, 64, 4), (3, 70, 5, 36, 4), (2, 512, 15, 512, 4), (1, 97, 16, 128, 16),
                                           (2, 130, 9, 4, 2), (1, 64, 16, 1024, 3), (1, 64, 16, 1028, 3), (2, 64, 3, 8, 20), (2, 8200, 15, 64, 4),
                                           (2, 8200, 15, 512, 4), (4, 4100, 16, 128, 8), (1, 16400, 7, 192, 3), (8, 2100, 1, 64, 2),
                                           (2, 8200, 13, 96, 4), (128, 32, 32, 64, 4), (3, 16, 17, 8, 4), (2, 41, 31, 128, 8),
                                           (5, 33, 32, 1024, 32), (2, 300, 20, 36, 20)])
def test_topk_route_with_few_keys_and_many_queries_bit_exact(B, Q, S, D, top_k):
    """Shapes with at most 32 keys take the kernels that stage the keys in shared memory (a lane per key: a
    half-warp per query up to 16 keys, the warp from 17 to 32; from 16384 queries on, with the features in
    whole tiles of 64, a block of 4 queries x 4 keys per lane); their scores, indices and gates must be those
    of the C oracle bit for bit, ragged last CTA included."""
    rng = np.random.default_rng(47 + Q + S)
    qv = rng.standard_normal((B, Q, D)).astype(np.float32)
    kv = rng.standard_normal((B, S, D)).astype(np.float32)
    kv[:, S // 2] = kv[:, 0]                                   # equal scores: the lower index wins
    visible = rng.integers(0, S + 2, size=Q).astype(np.int32)
    scale = 1.0 / np.sqrt(D)
    want_scores = oracle.c_route_scores(qv, kv, scale)
    for vis in (None, visible):
        want_idx, want_gates = oracle.c_topk_select(want_scores, top_k, 0.9, vis)
        idx, gates, scores = gx.topk_route(dev(qv), dev(kv), top_k, scale, 0.9, None if vis is None else dev(vis))
        assert np.array_equal(host(scores), want_scores)
        assert np.array_equal(idx.cpu().numpy(), want_idx)
        close(gates, want_gates, FP32_TOL)
    assert cabi.device_error_word() == 0


@pytest.mark.parametrize("B,Q,S,D,top_k", [(2, 512, 15, 512, 4), (3, 70, 5, 40, 4), (1, 97, 16, 1024, 16), (2, 8200, 15, 64, 4),
                                           (2, 8200, 15, 512, 4), (3, 5500, 16, 128, 8)])
def test_topk_route_reads_bf16_queries_as_if_widened(B, Q, S, D, top_k):
    rng = np.random.default_rng(53 + Q)
    q16 = dev(rng.standard_normal((B, Q, D)).astype(np.float32), torch.bfloat16)
    kv = dev(rng.standard_normal((B, S, D)).astype(np.float32))
    visible = dev(rng.integers(0, S + 2, size=Q).astype(np.int32))
    want = gx.topk_route(q16.float(), kv, top_k, 0.1, 0.9, visible)
    got = gx.topk_route(q16, kv, top_k, 0.1, 0.9, visible)
    for a, b in zip(got, want):
        assert torch.equal(a, b)                               # indices, gates and scores bit for bit
    # shapes outside the per-token case are refused, nothing runs
    lib = cabi.load()
    idx = torch.empty(B, 8, top_k, device=DEV, dtype=torch.int64)
    gates = torch.empty(B, 8, top_k, device=DEV)
    rc = lib.grmx_topk_route_bf16q(cabi.ptr(q16), cabi.ptr(kv), None, B, 8, S, D, top_k, 0.1, 0.9, cabi.ptr(idx),
                                   cabi.ptr(gates), None, cabi.current_stream())
    assert rc == 2 and b"widen" in lib.grmx_last_error()


def test_topk_matches_reference_retriever_fixtures(golden):
    for name in ("topk", "identity"):
        g = golden(f"retriever_{name}")
        pq = torch.nn.functional.linear(dev(g["query"]), dev(g["w_query"]))
        pk = torch.nn.functional.linear(dev(g["keys"]), dev(g["w_key"]))
        top_k = int(g["top_k"])
        idx, gates, scores = gx.topk_route(pq[:, None, :].contiguous(), pk.contiguous(), top_k,
                                           1.0 / np.sqrt(g["w_query"].shape[0]))
        R = g["indices"].shape[1]
        assert np.array_equal(idx.cpu().numpy()[:, 0, :R], g["indices"])
        close(gates[:, 0, :R], g["gates"], FP32_TOL)
        close(scores[:, 0], g["scores"], FP32_TOL)


def test_topk_select_ties_nan_and_masks():
    scores = np.zeros((1, 3, 8), dtype=np.float32)
    scores[0, 1, [2, 5]] = 1.0
    scores[0, 2] = [np.nan, -np.inf, 3.0, 3.0, -0.0, 0.0, -np.inf, 2.0]
    idx, gates = gx.topk_select(dev(scores), 4)
    assert idx.cpu().tolist() == [[[0, 1, 2, 3], [2, 5, 0, 1], [0, 2, 3, 7]]]
    assert torch.isnan(gates[0, 2]).all() and torch.allclose(gates[0, 0], torch.full((4,), 0.25, device=DEV))
    rng = np.random.default_rng(43)
    big = rng.standard_normal((4, 7, 300)).astype(np.float32)
    big[:, :, ::7] = -np.inf
    big[1, 2, :] = 0.5                                          # all equal
    want_idx, want_gates = oracle.c_topk_select(big, 8, 2.0)
    idx, gates = gx.topk_select(dev(big), 8, 2.0)
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    close(gates, want_gates, FP32_TOL)
    # more routes requested than keys: identity order, padded
    idx, gates = gx.topk_select(dev(big[:, :, :3]), 8)
    assert idx[0, 0].cpu().tolist() == [0, 1, 2, -1, -1, -1, -1, -1] and float(gates[0, 0, 3:].abs().sum()) == 0.0


# --------------------------------------------------------------------------- fused retrieval

@pytest.mark.parametrize("H,K", [(64, 64), (16, 8), (20, 6), (128, 64), (512, 64)])
def test_retrieve_fuse_modes(H, K):
    rng = np.random.default_rng(H + K)
    B, S, Q, R = 3, 9, 5, 4
    archive = rng.standard_normal((B, S, H, K)).astype(np.float32)
    idx = rng.integers(0, S, size=(B, Q, R))
    idx[1, 2] = -1
    idx[0, 1, 2:] = -1
    gates = rng.random((B, Q, R)).astype(np.float32)
    queries = rng.standard_normal((B, Q, K)).astype(np.float32)
    online = rng.standard_normal((B, Q, H)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, H).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, H).astype(np.float32)
    t = dict(archive=dev(archive), indices=dev(idx), gates=dev(gates), queries=dev(queries))
    for mode, name in ((cabi.FUSE_RETRIEVED, "retrieved"), (cabi.FUSE_CONTRIB, "contrib")):
        got = gx.retrieve_fuse(**t, mode=mode)
        close(got, go.retrieve_fuse(archive, idx, gates, queries, mode=name), FP32_TOL)
    got = gx.retrieve_fuse(**t, online=dev(online), ln_weight=dev(w), ln_bias=dev(b), mode=cabi.FUSE_RESIDUAL_LN)
    close(got, go.retrieve_fuse(archive, idx, gates, queries, online, w, b), FP32_TOL)
    assert torch.equal(got[1, 2], dev(online)[1, 2])          # no archived segment: online passes through
    got = gx.retrieve_fuse(**t, online=dev(online), mode=cabi.FUSE_RESIDUAL_LN)
    close(got, go.retrieve_fuse(archive, idx, gates, queries, online), FP32_TOL)


@pytest.mark.parametrize("B,S,Q,R,H,K", [(3, 9, 5, 4, 64, 64), (2, 32, 32, 8, 128, 128), (70, 32, 32, 4, 64, 64),
                                         (2, 5, 7, 3, 20, 32), (1, 40, 3, 2, 100, 96), (2, 6, 1, 6, 33, 160),
                                         (2, 3, 40, 2, 256, 32), (3, 17, 9, 5, 1, 64), (3, 9, 20, 5, 100, 128),
                                         (2, 4, 13, 4, 33, 128), (65, 32, 32, 8, 128, 128), (2, 300, 4, 8, 32, 32),
                                         (1, 64, 64, 1, 64, 64)])
def test_retrieve_fuse_slot_major_form(B, S, Q, R, H, K):
    """One CTA per batch row that reads every chosen matrix once: same results as the query-major kernel
    to fp32 rounding (the sum over a query's routes runs in slot order), empty routes, repeated slots and
    queries without any route included."""
    rng = np.random.default_rng(B + S + Q + R + H + K)
    archive = rng.standard_normal((B, S, H, K)).astype(np.float32)
    idx = rng.integers(0, S, size=(B, Q, R))
    idx[0, 0, :] = -1                                   # nothing to retrieve
    idx[B - 1, Q - 1, R - 1] = -1                       # one empty route
    if R >= 2:
        idx[0, Q - 1, 1] = idx[0, Q - 1, 0]             # the same slot twice
    gates = rng.random((B, Q, R)).astype(np.float32)
    queries = rng.standard_normal((B, Q, K)).astype(np.float32)
    online = rng.standard_normal((B, Q, H)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, H).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, H).astype(np.float32)
    t = dict(archive=dev(archive), indices=dev(idx), gates=dev(gates), queries=dev(queries))
    got = gx.retrieve_fuse_rows(**t, mode=cabi.FUSE_CONTRIB)
    close(got, go.retrieve_fuse(archive, idx, gates, queries, mode="contrib"), FP32_TOL)
    got = gx.retrieve_fuse_rows(**t, online=dev(online), ln_weight=dev(w), ln_bias=dev(b))
    close(got, go.retrieve_fuse(archive, idx, gates, queries, online, w, b), FP32_TOL)
    assert torch.equal(got[0, 0], dev(online)[0, 0])    # no archived segment: online passes through
    got = gx.retrieve_fuse_rows(**t, online=dev(online))
    close(got, go.retrieve_fuse(archive, idx, gates, queries, online), FP32_TOL)
    assert cabi.device_error_word() == 0


def test_retrieve_fuse_slot_major_form_limits():
    lib = cabi.load()
    a = torch.zeros(1, 2, 8, 48, device=DEV)            # K = 48 is not a multiple of 32
    i = torch.zeros(1, 1, 1, device=DEV, dtype=torch.int64)
    g = torch.ones(1, 1, 1, device=DEV)
    q = torch.zeros(1, 1, 48, device=DEV)
    o = torch.zeros(1, 1, 8, device=DEV)
    rc = lib.grmx_retrieve_fuse_rows(cabi.ptr(a), cabi.ptr(i), cabi.ptr(g), cabi.ptr(q), None, None, None, 1e-5,
                                     cabi.ptr(o), 1, 2, 1, 1, 8, 48, cabi.FUSE_CONTRIB, cabi.current_stream())
    assert rc == 2 and b"multiple of 32" in lib.grmx_last_error()
    # an index beyond the archive sets the error word and is skipped, as in the query-major kernel
    a = torch.ones(1, 2, 8, 32, device=DEV)
    i = torch.tensor([[[5]]], device=DEV, dtype=torch.int64)
    q = torch.ones(1, 1, 32, device=DEV)
    out = gx.retrieve_fuse_rows(a, i, g, q, mode=cabi.FUSE_CONTRIB)
    assert float(out.abs().sum()) == 0.0 and cabi.device_error_word() == 1
    cabi.check(lib.grmx_device_error_reset(cabi.current_stream()))


def test_retrieve_fuse_equals_gather_then_apply(golden):
    rng = np.random.default_rng(51)
    B, S, Q, R, H, K = 2, 6, 4, 3, 64, 64
    archive = dev(rng.standard_normal((B, S, H, K)).astype(np.float32))
    idx = dev(rng.integers(0, S, size=(B, Q, R)))
    queries = dev(rng.standard_normal((B, Q, K)).astype(np.float32))
    gathered = gx.batched_gather(archive, idx)
    two_step = gx.apply_query_fwd(gathered, queries)
    fused = gx.retrieve_fuse(archive, idx, None, queries, mode=cabi.FUSE_RETRIEVED)
    assert torch.equal(fused, two_step)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_TOL), (torch.bfloat16, LOWP_TOL)])
@pytest.mark.parametrize("H", [64, 512, 1000])
def test_select_fuse_equals_the_fused_chain_on_dense_candidates(dtype, tol, H):
    """Applying the query to every candidate first (what the caller does with one GEMM) and then
    selecting must give what gather -> apply-query -> weighted sum -> LayerNorm gives."""
    rng = np.random.default_rng(61 + H)
    B, S, Q, R, K = 2, 5, 7, 3, 16
    archive = rng.standard_normal((B, S, H, K)).astype(np.float32)
    queries = rng.standard_normal((B, Q, K)).astype(np.float32)
    idx = rng.integers(0, S, size=(B, Q, R))
    idx[0, 1, 2] = -1                       # an empty route
    idx[1, 3, :] = -1                       # a token with nothing to retrieve
    gates = rng.random((B, Q, R)).astype(np.float32)
    online = rng.standard_normal((B, Q, H)).astype(np.float32)
    ln_w = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    ln_b = (0.1 * rng.standard_normal(H)).astype(np.float32)
    states = np.einsum("bshk,bqk->bqsh", archive.astype(np.float64), queries.astype(np.float64))
    t_states, t_online = dev(states.astype(np.float32), dtype), dev(online, dtype)
    # oracle on the values the kernel actually sees
    seen_states, seen_online = host(t_states).astype(np.float64), host(t_online).astype(np.float64)
    live = idx >= 0
    picked = np.take_along_axis(seen_states, np.clip(idx, 0, None)[..., None], axis=2)
    contrib = (picked * np.where(live, gates, 0.0)[..., None]).sum(axis=2)
    got = gx.select_fuse(t_states, dev(idx), dev(gates), mode=cabi.FUSE_CONTRIB)
    close(got, contrib, tol)
    x = seen_online + contrib
    want = (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5) * ln_w + ln_b
    want[1, 3] = seen_online[1, 3]          # no live route: the online state passes through
    got = gx.select_fuse(t_states, dev(idx), dev(gates), t_online, dev(ln_w), dev(ln_b), 1e-5, cabi.FUSE_RESIDUAL_LN)
    close(got, want, tol)
    if dtype == torch.float32:              # and the same as the gather-based kernel on the archive itself
        fused = gx.retrieve_fuse(dev(archive), dev(idx), dev(gates), dev(queries), dev(online), dev(ln_w), dev(ln_b))
        close(got, host(fused), FP32_TOL)
    assert cabi.device_error_word() == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_TOL), (torch.bfloat16, LOWP_TOL)])
@pytest.mark.parametrize("rows,H", [(5, 64), (4099, 512), (33, 1000), (7, 1024), (3, 8)])
def test_add_layer_norm_is_the_residual_rule_with_one_candidate(dtype, tol, rows, H):
    """LayerNorm(a + b) in one pass: against float64 on the values the kernel sees, and bit for bit the same as
    the fusion kernel's residual rule with b as the only candidate and a unit gate."""
    rng = np.random.default_rng(rows + H)
    a, b = (dev(rng.standard_normal((rows, H)).astype(np.float32), dtype) for _ in range(2))
    w = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(H)).astype(np.float32)
    got = gx.add_layer_norm(a, b, dev(w), dev(bias))
    x = host(a).astype(np.float64) + host(b).astype(np.float64)
    want = (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5) * w + bias
    close(got, want, tol)
    unit_idx = torch.zeros(1, rows, 1, device=DEV, dtype=torch.int64)
    unit_gate = torch.ones(1, rows, 1, device=DEV)
    same = gx.select_fuse(b.view(1, rows, 1, H), unit_idx, unit_gate, a.view(1, rows, H), dev(w), dev(bias), 1e-5,
                          cabi.FUSE_RESIDUAL_LN)
    assert torch.equal(got, same.view(rows, H))
    plain = gx.add_layer_norm(a, b)                          # no affine part
    close(plain, (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5), tol)
    lib = cabi.load()
    odd = torch.zeros(2, 6, device=DEV, dtype=dtype)        # rows that are not whole 16-byte pieces
    rc = lib.grmx_add_layer_norm(cabi.ptr(odd), cabi.ptr(odd), None, None, 1e-5, cabi.ptr(odd), 2, 6,
                                 cabi.F32 if dtype == torch.float32 else cabi.BF16, cabi.current_stream())
    assert rc == 2 and b"16-byte" in lib.grmx_last_error()


# --------------------------------------------------------------------------- chunk scan, tcgen05 path

@pytest.mark.parametrize("B,S,Q,R,H,seg,mode", [(1, 3, 128, 2, 64, None, cabi.FUSE_RESIDUAL_LN),
                                                (2, 5, 300, 2, 128, 64, cabi.FUSE_RESIDUAL_LN),
                                                (2, 7, 257, 3, 192, 32, cabi.FUSE_CONTRIB),
                                                (3, 15, 512, 4, 512, 32, cabi.FUSE_RESIDUAL_LN),
                                                (1, 32, 384, 8, 256, None, cabi.FUSE_RESIDUAL_LN)])
def test_tensor_core_retrieval_matches_the_fused_chain(B, S, Q, R, H, seg, mode):
    """Per-token retrieval straight from the bf16 ring (one accumulated product per chosen slot and tile of
    128 tokens) against gather -> apply-query -> gate-weighted sum -> residual LayerNorm in float64 on the
    same bf16 values; causal visible counts leave early tokens with fewer routes or none (those keep their
    online state untouched)."""
    rng = np.random.default_rng(61 + Q)
    arch = dev(rng.standard_normal((B, S, H, 64)).astype(np.float32), torch.bfloat16)
    qv = rng.standard_normal((B, Q, 64)).astype(np.float32)
    qv /= np.linalg.norm(qv, axis=-1, keepdims=True)
    q = dev(qv, torch.bfloat16)
    online = dev(rng.standard_normal((B, Q, H)).astype(np.float32), torch.bfloat16)
    ln_w = dev(rng.uniform(0.5, 1.5, H).astype(np.float32))
    ln_b = dev(rng.uniform(-0.5, 0.5, H).astype(np.float32))
    visible = None if seg is None else np.minimum(np.arange(Q) // seg, S).astype(np.int32)
    idx, gates = oracle.c_topk_select(rng.standard_normal((B, Q, S)).astype(np.float32), R, 1.0, visible)
    got = gx.retrieve_fuse_tc(arch, dev(idx), dev(gates), q, online, ln_w, ln_b, 1e-5, mode)
    assert got.dtype == torch.bfloat16 and cabi.device_error_word() == 0
    if mode == cabi.FUSE_RESIDUAL_LN:
        want = go.retrieve_fuse(host(arch), idx, gates, host(q), host(online), host(ln_w), host(ln_b), 1e-5)
        if visible is not None:                                     # tokens that see no segment: passed through bit for bit
            none = torch.from_numpy(visible == 0).to(DEV)
            assert torch.equal(got[:, none], online[:, none])
    else:
        want = go.retrieve_fuse(host(arch), idx, gates, host(q), mode="contrib")
    close(got, want, LOWP_TOL)
    # the selection kernel on dense candidate states is the other route to the same result
    states = torch.einsum("bshk,bqk->bqsh", arch.float(), q.float()).to(torch.bfloat16).contiguous()
    other = gx.select_fuse(states, dev(idx), dev(gates), online, ln_w, ln_b, 1e-5, mode)
    close(got, host(other), LOWP_TOL)


def test_tensor_core_retrieval_argument_contract():
    lib = cabi.load()
    arch = torch.zeros(1, 2, 64, 64, device=DEV, dtype=torch.bfloat16)
    q = torch.zeros(1, 128, 64, device=DEV, dtype=torch.bfloat16)
    online = torch.ones(1, 128, 64, device=DEV, dtype=torch.bfloat16)
    idx = torch.zeros(1, 128, 1, device=DEV, dtype=torch.int64)
    gates = torch.ones(1, 128, 1, device=DEV)
    out = torch.empty_like(online)
    def call(S, R, H, K):
        return lib.grmx_retrieve_fuse_tc(cabi.ptr(arch), cabi.ptr(idx), cabi.ptr(gates), cabi.ptr(q), cabi.ptr(online), None, None,
                                         1e-5, cabi.ptr(out), 1, S, 128, R, H, K, cabi.FUSE_RESIDUAL_LN, cabi.current_stream())
    assert call(2, 1, 64, 32) == 2 and b"grmx_retrieve_fuse" in lib.grmx_last_error()      # key dim other than 64
    assert call(2, 1, 96, 64) == 2 and call(40, 1, 64, 64) == 2 and call(2, 9, 64, 64) == 2
    # an index outside the ring is an empty route: the token keeps its online state and the error word says so
    idx[0, 5, 0] = 7
    assert call(2, 1, 64, 64) == 0
    torch.cuda.synchronize()
    assert cabi.device_error_word() & 1
    cabi.check(lib.grmx_device_error_reset(cabi.current_stream()))
    assert torch.equal(out[0, 5], online[0, 5]) and cabi.device_error_word() == 0


@pytest.mark.parametrize("B,T,L,K,H", [(2, 1024, 256, 64, 64), (8, 2048, 512, 64, 128), (64, 2048, 128, 64, 64),
                                       (1, 4096, 512, 128, 64)])
def test_scan_over_whole_segments_leaves_every_segment_state_in_the_archive(B, T, L, K, H):
    """One launch over all segments (rows cut along T inside the kernel where rows are few) against one
    call per segment with the state carried: hidden states, final state and every archived state."""
    k, v, q, m = make_chunk(B + T + L, B, T, K, H)
    tk, tv, tq = dev(k, torch.bfloat16), dev(v, torch.bfloat16), dev(q, torch.bfloat16)
    n, first, capacity = T // L, 2, T // L + 3
    archive = torch.full((B, capacity, H, K), 7.0, device=DEV)
    hidden, m_out = gx.chunk_scan_fwd_segments(tk, tv, tq, dev(m), 0.97, archive, first, L)
    carried = dev(m)
    for j in range(n):
        sl = slice(j * L, (j + 1) * L)
        want_h, carried = gx.chunk_scan_fwd(tk[:, sl].contiguous(), tv[:, sl].contiguous(), tq[:, sl].contiguous(),
                                            carried, 0.97, cabi.PATH_TCGEN05)
        close(hidden[:, sl], host(want_h), LOWP_TOL)
        close(archive[:, first + j], host(carried), LOWP_TOL)
    close(m_out, host(carried), LOWP_TOL)
    assert torch.equal(archive[:, first + n - 1], m_out)          # the last segment's state is the final state
    untouched = torch.cat([archive[:, :first], archive[:, first + n:]], dim=1)
    assert bool((untouched == 7.0).all())                          # other slots are not written
    # against the sequential oracle as well, on the values the kernel sees
    want = go.chunk_update_sequential(host(tk), host(tv), host(tq), m, 0.97)
    close(hidden, want[0], LOWP_TOL)
    close(m_out, want[1], LOWP_TOL)
    assert cabi.device_error_word() == 0
    lib = cabi.load()
    rc = lib.grmx_chunk_scan_fwd_segments(cabi.ptr(tk), cabi.ptr(tv), cabi.ptr(tq), cabi.ptr(dev(m)), cabi.ptr(hidden),
                                          cabi.ptr(m_out), cabi.ptr(archive), capacity, first, 192, B, T, K, H, 0.97,
                                          cabi.BF16, cabi.F32, cabi.current_stream())
    assert rc == 2 and b"128" in lib.grmx_last_error()


def _tc_case(seed, B, T, decay, zero_state):
    k, v, q, m = make_chunk(seed, B, T, 64, 64, zero_state=zero_state)
    tk, tv, tq = dev(k, torch.bfloat16), dev(v, torch.bfloat16), dev(q, torch.bfloat16)
    tm = dev(m)
    want = go.chunk_update_sequential(host(tk), host(tv), host(tq), m, decay)
    return (tk, tv, tq, tm), want


@pytest.mark.parametrize("B,T,decay,zero_state", [(1, 128, 0.97, True), (2, 256, 0.97, False), (3, 1024, 0.9, False),
                                                  (5, 384, 0.999, False), (2, 512, 0.5, False), (2, 256, 0.0, False),
                                                  (2, 256, 1.0, False)])
def test_tcgen05_scan_matches_oracle(B, T, decay, zero_state):
    args, (want_h, want_m) = _tc_case(B * 7 + T, B, T, decay, zero_state)
    hidden, m_out = gx.chunk_scan_fwd(*args, decay, cabi.PATH_TCGEN05)
    assert hidden.dtype == torch.bfloat16 and m_out.dtype == torch.float32
    close(hidden, want_h, LOWP_TOL)
    close(m_out, want_m, LOWP_TOL)
    assert cabi.device_error_word() == 0
    # the two kernel families agree with each other far inside the tolerance
    ffma_h, ffma_m = gx.chunk_scan_fwd(*args, decay, cabi.PATH_FFMA)
    close(hidden, host(ffma_h), LOWP_TOL)
    close(m_out, host(ffma_m), LOWP_TOL)


def test_tcgen05_scan_full_size_kernel_alone_config():
    # B=8 x H=8 rows, T=2048, d_k=d_v=64, zero start state: the benchmark's workload
    args, (want_h, want_m) = _tc_case(2, 64, 2048, 0.97, True)
    hidden, m_out = gx.chunk_scan_fwd(*args, 0.97, cabi.PATH_AUTO)
    close(hidden, want_h, LOWP_TOL)
    close(m_out, want_m, LOWP_TOL)
    again_h, again_m = gx.chunk_scan_fwd(*args, 0.97, cabi.PATH_AUTO)
    assert torch.equal(again_h, hidden) and torch.equal(again_m, m_out)          # run-to-run deterministic
    # one call over T equals 16 calls of 128 tokens carrying the state
    state, pieces = args[3], []
    for s in range(0, 2048, 128):
        h, state = gx.chunk_scan_fwd(*(t[:, s:s + 128].contiguous() for t in args[:3]), state, 0.97, cabi.PATH_TCGEN05)
        pieces.append(h)
    assert torch.equal(torch.cat(pieces, dim=1), hidden) and torch.equal(state, m_out)


def test_tcgen05_scan_is_linear_in_values_and_state():
    # size-independent property: the scan is linear in (values, start state)
    (tk, tv, tq, tm), _ = _tc_case(9, 4, 512, 0.97, False)
    h1, m1 = gx.chunk_scan_fwd(tk, tv, tq, tm, 0.97, cabi.PATH_TCGEN05)
    h2, m2 = gx.chunk_scan_fwd(tk, (tv.float() * 2).to(torch.bfloat16), tq, tm * 2, 0.97, cabi.PATH_TCGEN05)
    close(h2, 2 * host(h1), LOWP_TOL)
    close(m2, 2 * host(m1), 1e-6)


def test_tcgen05_path_refuses_what_it_does_not_cover():
    k, v, q, m = make_chunk(1, 1, 100, 32, 64)
    with pytest.raises(cabi.GrmxError, match="multiples of 64"):
        gx.chunk_scan_fwd(dev(k, torch.bfloat16), dev(v, torch.bfloat16), dev(q, torch.bfloat16), dev(m), 0.97,
                          cabi.PATH_TCGEN05)
    with pytest.raises(cabi.GrmxError, match="bf16"):
        gx.chunk_scan_fwd(dev(k), dev(v), dev(q), dev(m), 0.97, cabi.PATH_TCGEN05)
    # auto falls back to the fp32 kernel for the same request
    hidden, _ = gx.chunk_scan_fwd(dev(k), dev(v), dev(q), dev(m), 0.97, cabi.PATH_AUTO)
    close(hidden, go.chunk_update_sequential(k, v, q, m, 0.97)[0], FP32_TOL)


@pytest.mark.parametrize("T", [1, 5, 127, 129, 200, 300, 1000])
def test_tcgen05_scan_ragged_lengths(T):
    args, (want_h, want_m) = _tc_case(T, 3, T, 0.95, False)
    hidden, m_out = gx.chunk_scan_fwd(*args, 0.95, cabi.PATH_TCGEN05)
    close(hidden, want_h, LOWP_TOL)
    close(m_out, want_m, LOWP_TOL)
    assert cabi.device_error_word() == 0


@pytest.mark.parametrize("T", [128, 333])
@pytest.mark.parametrize("reverse", [False, True])
@pytest.mark.parametrize("no_decay_first", [False, True])
def test_tcgen05_linear_scan_general_form(T, reverse, no_decay_first):
    k, v, q, m = make_chunk(T + 3, 2, T, 64, 64)
    tk, tv, tq, tm = dev(k, torch.bfloat16), dev(v, torch.bfloat16), dev(q, torch.bfloat16), dev(m)
    want_h, want_m = go.linear_scan(host(tk), host(tv), host(tq), m, 0.93, 0.31, hidden_scale=1.7,
                                    memory_out_scale=0.6, reverse=reverse, first_step_no_decay=no_decay_first)
    hidden, m_out = gx.linear_scan(tk, tv, tq, tm, 0.93, 0.31, 1.7, 0.6, reverse, no_decay_first, cabi.PATH_TCGEN05)
    close(hidden, want_h, LOWP_TOL)
    close(m_out, want_m, LOWP_TOL)
    m_t = dev(np.ascontiguousarray(m.transpose(0, 2, 1)))
    hidden_t, m_out_t = gx.linear_scan(tk, tv, tq, m_t, 0.93, 0.31, 1.7, 0.6, reverse, no_decay_first,
                                       cabi.PATH_TCGEN05, transposed_state=True)
    assert torch.equal(hidden_t, hidden) and torch.equal(m_out_t, m_out)


def test_tcgen05_backward_through_three_scans():
    k, v, q, m = make_chunk(61, 3, 200, 64, 64)
    rng = np.random.default_rng(62)
    gh = rng.standard_normal((3, 200, 64)).astype(np.float32)
    gm = rng.standard_normal((3, 64, 64)).astype(np.float32)
    tk, tv, tq, tgh = (dev(a, torch.bfloat16) for a in (k, v, q, gh))
    want = go.chunk_update_backward(host(tgh), gm, host(tk), host(tv), host(tq), m, 0.97)
    got = gx.chunk_scan_bwd(tgh, dev(gm), tk, tv, tq, dev(m), 0.97, cabi.PATH_TCGEN05)
    for a, b in zip(got, want):
        close(a, b, LOWP_TOL)


@pytest.mark.parametrize("B,T,K,H", [(2, 300, 64, 128), (2, 512, 128, 128), (1, 640, 64, 512), (3, 256, 128, 64),
                                     (150, 256, 128, 128), (2, 1024, 192, 64), (2, 300, 128, 256), (1, 130, 128, 128),
                                     (2, 1000, 128, 192), (3, 1, 128, 128), (2, 2048, 128, 128)])
def test_tcgen05_scan_wide_heads_run_as_blocks(B, T, K, H):
    """Heads wider than 64 are scanned as 64 x 64 blocks of the state; the outputs of the key/query
    blocks are summed in the bf16 output (one more rounding per block), the state is exact per block.
    Forward scans with d_k = 128 take the one-pass kernels instead: one CTA per row and 128 value features
    when d_v is a multiple of 128, per 64 value features otherwise."""
    k, v, q, m = make_chunk(K + H + T, B, T, K, H)
    tk, tv, tq = dev(k, torch.bfloat16), dev(v, torch.bfloat16), dev(q, torch.bfloat16)
    want_h, want_m = go.chunk_update_sequential(host(tk), host(tv), host(tq), m, 0.97)
    hidden, m_out = gx.chunk_scan_fwd(tk, tv, tq, dev(m), 0.97, cabi.PATH_TCGEN05)
    close(hidden, want_h, LOWP_TOL)
    close(m_out, want_m, LOWP_TOL)
    assert cabi.device_error_word() == 0
    # the general form as well: reverse order, no decay on the first step, transposed start state
    want = go.linear_scan(host(tk), host(tv), host(tq), m, 0.93, update_coeff=0.31, hidden_scale=1.7,
                          memory_out_scale=0.6, reverse=True, first_step_no_decay=True)
    got_h, got_m = gx.linear_scan(tk, tv, tq, dev(m), 0.93, 0.31, 1.7, 0.6, True, True, cabi.PATH_TCGEN05)
    close(got_h, want[0], LOWP_TOL)
    close(got_m, want[1], LOWP_TOL)


@pytest.mark.parametrize("B,T", [(1, 2048), (8, 2048), (64, 2048), (3, 1000), (16, 517), (2, 32768)])
def test_tcgen05_scan_cut_along_time_matches_uncut(B, T):
    args, (want_h, want_m) = _tc_case(B + T, B, T, 0.97, False)
    nbytes = gx.chunk_scan_scratch_bytes(B, T, 64, 64, torch.bfloat16, torch.float32)
    assert nbytes > 0
    scratch = torch.empty(nbytes, device=DEV, dtype=torch.uint8)
    hidden, m_out = gx.chunk_scan_fwd_ws(*args, 0.97, scratch)
    close(hidden, want_h, LOWP_TOL)
    close(m_out, want_m, LOWP_TOL)
    plain_h, plain_m = gx.chunk_scan_fwd(*args, 0.97, cabi.PATH_TCGEN05)
    close(hidden, host(plain_h), 1e-2)       # same math, pieces start from a re-derived state
    close(m_out, host(plain_m), 1e-4)
    assert cabi.device_error_word() == 0
    # a workspace that is too small, or none, silently takes the uncut kernel
    small_h, _ = gx.chunk_scan_fwd_ws(*args, 0.97, scratch[:16])
    none_h, _ = gx.chunk_scan_fwd_ws(*args, 0.97, None)
    assert torch.equal(small_h, plain_h) and torch.equal(none_h, plain_h)


def test_scratch_size_query():
    # 64 rows on 148 SMs: two pieces, the first piece's state as the sum of two terms
    assert gx.chunk_scan_scratch_bytes(64, 2048, 64, 64, torch.bfloat16, torch.float32) == 64 * 2 * 64 * 64 * 4
    assert gx.chunk_scan_scratch_bytes(512, 2048, 64, 64, torch.bfloat16, torch.float32) == 0    # enough rows
    assert gx.chunk_scan_scratch_bytes(64, 256, 64, 64, torch.bfloat16, torch.float32) == 0      # too short
    assert gx.chunk_scan_scratch_bytes(64, 2048, 64, 64, torch.float32, torch.float32) == 0      # fp32 path
    assert gx.chunk_scan_scratch_bytes(64, 2048, 128, 128, torch.bfloat16, torch.float32) == 0


def test_bounded_wait_gives_up_and_reports_without_losing_the_context():
    """A wait that nothing will ever satisfy runs out of polls, the kernel returns, bit 1 of the
    device error word is set, and the next launch on the same context works."""
    lib = cabi.load()
    assert cabi.device_error_word() == 0
    cabi.check(lib.grmx_selftest_bounded_wait(1 << 12, cabi.current_stream()))
    torch.cuda.synchronize()
    assert cabi.device_error_word() == 2
    cabi.check(lib.grmx_device_error_reset(cabi.current_stream()))
    assert cabi.device_error_word() == 0
    args, (want_h, _) = _tc_case(3, 2, 256, 0.97, False)
    hidden, _ = gx.chunk_scan_fwd(*args, 0.97, cabi.PATH_TCGEN05)
    close(hidden, want_h, LOWP_TOL)
    assert cabi.device_error_word() == 0

