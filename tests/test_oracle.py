"""The oracle against the reference: golden fixtures and the compiled reference C++.

These are CPU tests.  They pin the checker that the GPU parity tests rely on.
"""

import numpy as np
import pytest
import torch

import oracle
from oracle import grm_oracle as go

FP32_TOL = 1e-5  # the reference's own CPU parity tolerance (examples/test_grm.py:67-68)
# The fixtures are the reference's float32 results; its autograd gradients over 300 tokens at
# decay 0.999 carry about 1e-5 of float32 rounding themselves (measured against float64).
FP32_GRAD_TOL = 5e-5

CHUNK_CASES = ["small", "ragged", "cfg1", "long"]


@pytest.mark.parametrize("name", CHUNK_CASES)
def test_chunk_update_forward_matches_reference_python(golden, name):
    g = golden(f"chunk_update_{name}")
    decay = float(g["decay"])
    for fn in (go.chunk_update_sequential, go.chunk_update_vectorized):
        hidden, m_out = fn(g["keys"], g["values"], g["queries"], g["memory"], decay)
        assert go.rel_err(hidden, g["hidden"]) < FP32_TOL
        assert go.rel_err(m_out, g["memory_out"]) < FP32_TOL
    hidden, m_out = oracle.c_chunk_update(g["keys"], g["values"], g["queries"], g["memory"], decay)
    assert go.rel_err(hidden, g["hidden"]) < FP32_TOL
    assert go.rel_err(m_out, g["memory_out"]) < FP32_TOL


@pytest.mark.parametrize("name", CHUNK_CASES)
def test_chunk_update_backward_matches_reference_autograd(golden, name):
    g = golden(f"chunk_update_{name}")
    grads = go.chunk_update_backward(g["grad_hidden"], g["grad_memory_out"], g["keys"], g["values"],
                                     g["queries"], g["memory"], float(g["decay"]))
    for got, key in zip(grads, ("grad_keys", "grad_values", "grad_queries", "grad_memory")):
        assert go.rel_err(got, g[key]) < FP32_GRAD_TOL, key


def test_linear_scan_generalises_the_chunk_update(golden):
    g = golden("chunk_update_ragged")
    decay = float(g["decay"])
    K = g["keys"].shape[2]
    hidden, m_out = go.linear_scan(g["keys"], g["values"], g["queries"], g["memory"], decay,
                                   (1.0 - decay) / np.sqrt(K))
    assert go.rel_err(hidden, g["hidden"]) < FP32_TOL
    assert go.rel_err(m_out, g["memory_out"]) < FP32_TOL


def test_chunking_does_not_change_the_result(golden):
    g = golden("chunk_update_long")
    decay = float(g["decay"])
    m = g["memory"]
    pieces = []
    for start in range(0, g["keys"].shape[1], 64):
        sl = slice(start, start + 64)
        h, m = go.chunk_update_vectorized(g["keys"][:, sl], g["values"][:, sl], g["queries"][:, sl], m, decay)
        pieces.append(h)
    assert go.rel_err(np.concatenate(pieces, axis=1), g["hidden"]) < FP32_TOL
    assert go.rel_err(m, g["memory_out"]) < FP32_TOL


def test_chunk_update_empty_chunk():
    m = np.ones((2, 3, 4), dtype=np.float32)
    hidden, m_out = go.chunk_update_vectorized(np.zeros((2, 0, 4)), np.zeros((2, 0, 3)), np.zeros((2, 0, 4)), m, 0.97)
    assert hidden.shape == (2, 0, 3)
    assert np.array_equal(m_out, m)


def test_apply_query_matches_reference(golden):
    g = golden("apply_query")
    for tag in ("r5", "r4"):
        hid = go.apply_query(g[f"{tag}_memories"], g[f"{tag}_queries"])
        assert go.rel_err(hid, g[f"{tag}_hidden"]) < FP32_TOL
        assert go.rel_err(oracle.c_apply_query(g[f"{tag}_memories"], g[f"{tag}_queries"]), g[f"{tag}_hidden"]) < FP32_TOL
        gm, gq = go.apply_query_backward(g[f"{tag}_grad_hidden"], g[f"{tag}_memories"], g[f"{tag}_queries"])
        assert go.rel_err(gm, g[f"{tag}_grad_memories"]) < FP32_TOL
        assert go.rel_err(gq, g[f"{tag}_grad_queries"]) < FP32_TOL
    with pytest.raises(ValueError):
        go.apply_query(np.zeros((2, 3, 4)), np.zeros((2, 4)))


def test_gather_matches_reference_bit_for_bit(golden):
    g = golden("gather")
    for idx_key, out_key in (("idx3", "out3"), ("idx2", "out2")):
        assert np.array_equal(go.batched_gather(g["memories"], g[idx_key]), g[out_key])
        out, bad = oracle.c_batched_gather(g["memories"], g[idx_key])
        assert bad == 0 and np.array_equal(out, g[out_key])
    out, bad = oracle.c_batched_gather(g["memories"], np.array([[-1, 7], [0, 1]]))
    assert bad == 1 and not out[0].any()
    with pytest.raises(ValueError):
        go.batched_gather(g["memories"][0], g["idx2"])


def _retriever_scores(g):
    """Projected, scaled scores of the fixture in the engine's summation order."""
    pq = (g["query"].astype(np.float64) @ g["w_query"].astype(np.float64).T).astype(np.float32)
    pk = (g["keys"].astype(np.float64) @ g["w_key"].astype(np.float64).T).astype(np.float32)
    scale = 1.0 / np.sqrt(g["w_query"].shape[0])
    return oracle.c_route_scores(pq[:, None, :], pk, scale)[:, 0, :]


@pytest.mark.parametrize("name", ["topk", "identity", "causal", "masked"])
def test_routing_matches_reference_retriever(golden, name):
    g = golden(f"retriever_{name}")
    scores = _retriever_scores(g)
    ref_scores = g["scores"]
    finite = np.isfinite(ref_scores)
    # the reference masks with -inf after scoring (grm/core/gating_unit.py:73-79)
    if g["attention_mask"].size:
        scores = np.where(g["attention_mask"], scores, -np.inf).astype(np.float32)
    offset, S = int(g["segment_offset"]), scores.shape[1]
    if 0 < offset < S:
        scores[:, offset:] = -np.inf
    assert np.array_equal(np.isfinite(scores), finite)
    assert go.rel_err(scores[finite], ref_scores[finite]) < FP32_TOL
    top_k = int(g["top_k"])
    for select in (lambda s: go.topk_route(s, top_k), lambda s: oracle.c_topk_select(s, top_k)):
        idx, gates = select(scores[:, None, :])
        R = g["indices"].shape[1]
        assert np.array_equal(idx[:, 0, :R], g["indices"])
        assert (idx[:, 0, R:] == -1).all() and (gates[:, 0, R:] == 0).all()
        assert go.rel_err(gates[:, 0, :R], g["gates"]) < FP32_TOL


def test_topk_tie_rules():
    scores = np.zeros((1, 3, 8), dtype=np.float32)
    scores[0, 1, [2, 5]] = 1.0
    scores[0, 2] = [np.nan, -np.inf, 3.0, 3.0, -0.0, 0.0, -np.inf, 2.0]
    for select in (go.topk_route, oracle.c_topk_select):
        idx, gates = select(scores, 4)
        assert idx[0, 0].tolist() == [0, 1, 2, 3]           # all equal -> lowest indices
        assert idx[0, 1].tolist() == [2, 5, 0, 1]
        assert idx[0, 2].tolist() == [0, 2, 3, 7]           # NaN first, then 3.0 (lower index first)
        assert np.allclose(gates[0, 0], 0.25)
        assert np.isnan(gates[0, 2]).all()
    # identity order when every visible key is selected, padding beyond
    idx, gates = oracle.c_topk_select(scores, 4, visible=np.array([0, 3, 8], dtype=np.int32))
    assert idx[0, 0].tolist() == [-1, -1, -1, -1] and (gates[0, 0] == 0).all()
    assert idx[0, 1].tolist() == [0, 1, 2, -1]
    idx2, gates2 = go.topk_route(scores, 4, visible=np.array([0, 3, 8]))
    assert np.array_equal(idx, idx2) and np.allclose(gates, gates2, equal_nan=True)


def test_c_scores_agree_with_double_precision():
    rng = np.random.default_rng(5)
    q = rng.standard_normal((3, 4, 64)).astype(np.float32)
    k = rng.standard_normal((3, 9, 64)).astype(np.float32)
    assert go.rel_err(oracle.c_route_scores(q, k, 0.125), go.route_scores(q, k, 0.125)) < FP32_TOL


@pytest.mark.parametrize("size", ["", "cfg3_"])
@pytest.mark.parametrize("mode", ["residual", "concat", "gate", "linear"])
def test_fusion_matches_reference(golden, mode, size):
    g = golden(f"fusion_{size}{mode}")
    params = {k[len("param::"):]: v for k, v in g.items() if k.startswith("param::")}
    fused = go.retrieved_state_fusion(g["online"], g["retrieved"], g["gates"], mode, params, float(g["eps"]))
    assert go.rel_err(fused, g["fused"]) < FP32_TOL


def test_model_restatement_matches_reference_model_cfg1(golden):
    """Config 1: the reference's single-layer model forward, fp32 -- outputs, every token's fused state,
    the final memory and every segment's routing decisions."""
    g = golden("model_cfg1")
    params = {k[len("param::"):]: v for k, v in g.items() if k.startswith("param::")}
    out, hidden, memory, routes = go.segment_model_forward(params, g["x"], segment_length=128, retrieval_top_k=2,
                                                           memory_capacity_segments=8)
    assert go.rel_err(out, g["outputs"]) < FP32_TOL
    assert go.rel_err(hidden, g["hidden_states"]) < FP32_TOL
    assert go.rel_err(memory, g["memory_final"]) < FP32_TOL
    assert len(routes) == 3
    for i, (idx, gates) in enumerate(routes, start=1):
        assert np.array_equal(idx, g[f"route{i}_indices"])
        assert go.rel_err(gates, g[f"route{i}_gates"]) < FP32_TOL


@pytest.mark.parametrize("mode", ["concat", "gate", "linear"])
def test_model_restatement_matches_reference_model_with_other_fusion_rules(golden, mode):
    g = golden(f"model_fusion_{mode}")
    params = {k[len("param::"):]: v for k, v in g.items() if k.startswith("param::")}
    out, hidden, memory, routes = go.segment_model_forward(params, g["x"], segment_length=64, retrieval_top_k=2,
                                                           memory_capacity_segments=8, mode=mode)
    assert int(g["num_segments"]) == 4 and len(routes) == 3
    assert go.rel_err(hidden, g["hidden_states"]) < FP32_TOL
    assert go.rel_err(out, g["outputs"]) < FP32_TOL
    assert go.rel_err(memory, g["memory_final"]) < FP32_TOL


def test_retrieve_fuse_chain_equals_its_parts(golden):
    g = golden("fusion_residual")
    rng = np.random.default_rng(7)
    B, S, Q, R, H, K = 2, 5, 3, 2, 16, 8
    archive = rng.standard_normal((B, S, H, K)).astype(np.float32)
    idx = rng.integers(0, S, size=(B, Q, R))
    idx[1, 2] = -1
    idx[0, 1, 1] = -1
    gates = rng.random((B, Q, R)).astype(np.float32)
    queries = rng.standard_normal((B, Q, K)).astype(np.float32)
    online = rng.standard_normal((B, Q, H)).astype(np.float32)
    w, b = g["param::layer_norm.weight"], g["param::layer_norm.bias"]
    fused = go.retrieve_fuse(archive, idx, gates, queries, online, w, b)
    # parts: gather -> apply_query -> fusion module, on the live slots
    for bi in range(B):
        for qi in range(Q):
            live = idx[bi, qi] >= 0
            if not live.any():
                assert np.array_equal(fused[bi, qi], online[bi, qi].astype(np.float64))
                continue
            sel = go.batched_gather(archive[bi:bi + 1], idx[bi:bi + 1, qi, live])
            ret = go.apply_query(sel, queries[bi:bi + 1, qi])
            want = go.retrieved_state_fusion(online[bi:bi + 1, qi], ret, gates[bi:bi + 1, qi, live], "residual",
                                             {"layer_norm.weight": w, "layer_norm.bias": b})
            assert go.rel_err(fused[bi, qi], want[0]) < 1e-12
    assert go.rel_err(oracle.c_retrieve_fuse(archive, idx, gates, queries, online, w, b), fused) < FP32_TOL


# ---- against the reference's own compiled CPU code (oracle/_ref), when built ----

@pytest.fixture(scope="module")
def ref_ops():
    ops = oracle.reference_ops()
    if ops is None:
        pytest.skip("oracle/_ref was not built (no reference checkout at build time)")
    return ops


def test_oracle_vs_compiled_reference_chunk_update(ref_ops):
    rng = np.random.default_rng(3)
    B, T, K, H = 2, 50, 16, 24
    k, q = (rng.standard_normal((B, T, K)).astype(np.float32) for _ in range(2))
    v = rng.standard_normal((B, T, H)).astype(np.float32)
    m = rng.standard_normal((B, H, K)).astype(np.float32)
    t = [torch.from_numpy(a) for a in (k, v, q, m)]
    hidden, m_out, aux = ref_ops.chunk_update_forward(*t, 0.97)
    assert aux.numel() == 0
    h_o, m_o = go.chunk_update_sequential(k, v, q, m, 0.97)
    assert go.rel_err(hidden.numpy(), h_o) < FP32_TOL and go.rel_err(m_out.numpy(), m_o) < FP32_TOL
    gh = rng.standard_normal((B, T, H)).astype(np.float32)
    gm = rng.standard_normal((B, H, K)).astype(np.float32)
    grads = ref_ops.chunk_update_backward(torch.from_numpy(gh), torch.from_numpy(gm), *t, aux, 0.97)
    for got, want in zip(go.chunk_update_backward(gh, gm, k, v, q, m, 0.97), grads):
        assert go.rel_err(got, want.numpy()) < FP32_TOL
    # degenerate call: zero tokens (grm/csrc/grm_cuda.cpp:59-65)
    hidden0, m0, _ = ref_ops.chunk_update_forward(t[0][:, :0], t[1][:, :0], t[2][:, :0], t[3], 0.97)
    assert hidden0.shape == (B, 0, H) and torch.equal(m0, t[3])


def test_oracle_vs_compiled_reference_gather_and_apply(ref_ops, golden):
    g = golden("gather")
    out = ref_ops.batched_memory_gather(torch.from_numpy(g["memories"]), torch.from_numpy(g["idx3"]))
    assert np.array_equal(out.numpy(), go.batched_gather(g["memories"], g["idx3"]))
    a = golden("apply_query")
    hid = ref_ops.apply_query_forward(torch.from_numpy(a["r5_memories"]), torch.from_numpy(a["r5_queries"]))
    assert go.rel_err(go.apply_query(a["r5_memories"], a["r5_queries"]), hid.numpy()) < FP32_TOL
