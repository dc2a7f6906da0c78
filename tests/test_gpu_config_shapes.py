"""The retrieval configuration (config 3) and rows of the scale-out configuration (config 5) at their
own shapes, composed the way the configurations compose them, against the oracle; the weight-bearing
fusion rules through the segment runner against outputs of the reference model; the rank-2 retriever
with its masks against the reference retriever fixtures.

Inputs follow the synthetic definitions of the configurations: q, k ~ N(0,1) L2-normalised along the
feature axis, v ~ N(0,1), one CPU generator per tensor seeded 0, 1, 2, ... in the order q, k, v, extra.
"""

import math

import numpy as np
import pytest
import torch

import oracle
from oracle import grm_oracle as go
from rnn_with_grm_b200 import cabi
from rnn_with_grm_b200.retriever import topk_memory_retrieve
from rnn_with_grm_b200.segment_memory import SegmentMemoryRunner

import grmx_calls as gx

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
FP32_TOL = 1e-5
LOWP_TOL = 2e-2


def _randn(seed, *shape):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def _unit(t):
    return torch.nn.functional.normalize(t, dim=-1, eps=1e-6)


def _fusion_runner(mode, params_npz, hidden, key_dim):
    """A SegmentMemoryRunner that carries the fusion parameters of a fixture (the projections of the
    memory cell and the router are placeholders: only the fusion rule is exercised)."""
    params = {"memory_cell.key_proj.weight": torch.zeros(key_dim, 2), "memory_cell.value_proj.weight": torch.zeros(hidden, 2),
              "gating_unit.query_projection.weight": torch.zeros(2, 2)}
    for name, value in params_npz.items():
        if name.startswith("param::"):
            params["aggregator." + name[len("param::"):]] = torch.from_numpy(value)
    params = {k: v.to(DEV) for k, v in params.items()}
    return SegmentMemoryRunner(params, segment_length=256, retrieval_top_k=4, memory_capacity_segments=32,
                               retrieval_fusion_mode=mode)


# --------------------------------------------------------------------------- config 3

def test_config3_routing_gather_and_fusion_composed(golden):
    """B'=128 rows (16 x 8), T=8192, segment 256 -> 32 segment queries and 32 archived 64 x 64 fp32
    matrices per row; causal top-4 (segment j sees s < j, identity order while j <= 4, nothing for
    j = 0); gather; apply-query; all four fusion rules of RetrievedStateFusion(64)."""
    rows, T, L, K, V, top_k = 128, 8192, 256, 64, 64, 4
    S = T // L
    seg_q = _unit(_randn(0, rows, T, K)).view(rows, S, L, K).mean(dim=2).contiguous()
    seg_k = _unit(_randn(1, rows, T, K)).view(rows, S, L, K).mean(dim=2).contiguous()
    archive = _randn(2, rows, S, V, K)
    online = _randn(3, rows, S, V)
    visible = np.arange(S, dtype=np.int32)

    # routing: scores and indices bit for bit, gates to tolerance
    want_scores = oracle.c_route_scores(seg_q.numpy(), seg_k.numpy(), 1.0)
    want_idx, want_gates = oracle.c_topk_select(want_scores, top_k, 1.0, visible)
    assert (want_idx[:, 0] == -1).all() and (want_idx[:, 3, :3] == np.arange(3)).all() and (want_idx[:, 3, 3] == -1).all()
    assert (want_idx[:, 4] == np.arange(4)).all()                       # j == top_k: identity order, no sort
    d_q, d_k, d_arch, d_online = (t.to(DEV) for t in (seg_q, seg_k, archive, online))
    idx, gates, scores = gx.topk_route(d_q, d_k, top_k, 1.0, 1.0, torch.from_numpy(visible).to(DEV))
    assert np.array_equal(scores.cpu().numpy(), want_scores)
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    assert go.rel_err(gates.cpu().numpy(), want_gates) < FP32_TOL

    # gather of the selected matrices: bit for bit (empty slots are zero rows)
    gathered = gx.batched_gather(d_arch, idx)
    want_gathered, bad = oracle.c_batched_gather(archive.numpy(), want_idx)
    assert bad == 0 and gathered.shape == (rows, S, top_k, V, K)
    assert torch.equal(gathered.cpu(), torch.from_numpy(want_gathered))

    # apply-query on the gathered matrices (the unfused chain) and the fused kernel agree with the oracle
    applied = gx.apply_query_fwd(gathered, d_q)
    want_retrieved = go.retrieve_fuse(archive.numpy(), want_idx, want_gates, seg_q.numpy(), mode="retrieved")
    assert go.rel_err(applied.cpu().numpy(), want_retrieved) < FP32_TOL
    retrieved = gx.retrieve_fuse(d_arch, idx, gates, d_q, mode=cabi.FUSE_RETRIEVED)
    assert go.rel_err(retrieved.cpu().numpy(), want_retrieved) < FP32_TOL

    live = (want_idx >= 0)
    gates_live = np.where(live, want_gates, 0.0)
    flat = lambda a: a.reshape(rows * S, *a.shape[2:])
    for mode in ("residual", "concat", "gate", "linear"):
        f = golden(f"fusion_cfg3_{mode}")
        params = {k[len("param::"):]: v for k, v in f.items() if k.startswith("param::")}
        want = go.retrieved_state_fusion(flat(online.numpy()), flat(want_retrieved), flat(gates_live), mode, params,
                                         float(f["eps"])).reshape(rows, S, V)
        want[:, 0] = online.numpy()[:, 0]                               # no archived segment: no fusion at all
        if mode == "residual":
            got = gx.retrieve_fuse(d_arch, idx, gates, d_q, d_online, torch.from_numpy(params["layer_norm.weight"]).to(DEV),
                                   torch.from_numpy(params["layer_norm.bias"]).to(DEV), float(f["eps"]))
        else:
            contrib = gx.retrieve_fuse(d_arch, idx, gates, d_q, mode=cabi.FUSE_CONTRIB)
            runner = _fusion_runner(mode, f, V, K)
            got = runner._fuse_rule(d_online, contrib)
            got[:, 0] = d_online[:, 0]
        assert go.rel_err(got.cpu().numpy(), want) < FP32_TOL, mode
    assert cabi.device_error_word() == 0


# --------------------------------------------------------------------------- config 5

def test_config5_rows_scan_snapshots_routing_and_retrieval():
    """A handful of (b, h) rows of the scale-out configuration at its own shape: T=32768, d_k=d_v=128,
    segment 1024 (32 segments, 8 chunks per archived state), top-k 8, bf16 tokens with fp32 state.
    One scan launch leaves all 32 segment-end states in the archive; every one of them is checked
    against the sequential oracle, then the causal top-8 routing over the 31 earlier summaries (bit
    for bit) and the fused retrieval from the archive the scan wrote."""
    rows, T, L, d, top_k, decay = 5, 32768, 1024, 128, 8, 0.97
    S = T // L
    q = _unit(_randn(0, rows, T, d)).to(torch.bfloat16)
    k = _unit(_randn(1, rows, T, d)).to(torch.bfloat16)
    v = _randn(2, rows, T, d).to(torch.bfloat16)
    online = _randn(3, rows, S, d)
    m0 = torch.zeros(rows, d, d)

    archive = torch.full((rows, S, d, d), float("nan"), device=DEV)
    hidden, m_out = gx.chunk_scan_fwd_segments(k.to(DEV), v.to(DEV), q.to(DEV), m0.to(DEV), decay, archive, 0, L)
    torch.cuda.synchronize()
    assert cabi.device_error_word() == 0

    kf, vf, qf = (t.float().numpy() for t in (k, v, q))
    memory = m0.numpy().astype(np.float64)
    want_archive = np.empty((rows, S, d, d), dtype=np.float64)
    worst_h = 0.0
    got_hidden = hidden.float().cpu().numpy()
    for j in range(S):
        tok = slice(j * L, (j + 1) * L)
        want_h, memory = go.chunk_update_sequential(kf[:, tok], vf[:, tok], qf[:, tok], memory, decay)
        want_archive[:, j] = memory
        worst_h = max(worst_h, go.rel_err(got_hidden[:, tok], want_h))
    assert worst_h < LOWP_TOL
    got_archive = archive.cpu().numpy()
    assert np.isfinite(got_archive).all()
    for j in range(S):                                                  # every snapshot
        assert go.rel_err(got_archive[:, j], want_archive[:, j]) < LOWP_TOL, f"segment {j}"
    assert go.rel_err(m_out.cpu().numpy(), memory) < LOWP_TOL
    assert torch.equal(m_out, archive[:, S - 1])

    # routing: one query per segment (mean of q), keys = mean of k, causal, top-8
    seg_q = q.float().view(rows, S, L, d).mean(dim=2).contiguous()
    seg_k = k.float().view(rows, S, L, d).mean(dim=2).contiguous()
    visible = np.arange(S, dtype=np.int32)
    want_scores = oracle.c_route_scores(seg_q.numpy(), seg_k.numpy(), 1.0)
    want_idx, want_gates = oracle.c_topk_select(want_scores, top_k, 1.0, visible)
    idx, gates, scores = gx.topk_route(seg_q.to(DEV), seg_k.to(DEV), top_k, 1.0, 1.0, torch.from_numpy(visible).to(DEV))
    assert np.array_equal(scores.cpu().numpy(), want_scores) and np.array_equal(idx.cpu().numpy(), want_idx)
    assert go.rel_err(gates.cpu().numpy(), want_gates) < FP32_TOL

    # fused retrieval: the kernel on the archive the scan wrote, the oracle on its own archive
    fused = gx.retrieve_fuse(archive, idx, gates, seg_q.to(DEV), online.to(DEV))
    want = go.retrieve_fuse(want_archive, want_idx, want_gates, seg_q.numpy(), online.numpy())
    assert go.rel_err(fused.cpu().numpy(), want) < LOWP_TOL
    # and exactly (fp32 tolerance) when both read the same archive
    want_same = go.retrieve_fuse(got_archive, want_idx, want_gates, seg_q.numpy(), online.numpy())
    assert go.rel_err(fused.cpu().numpy(), want_same) < FP32_TOL


def test_config5_scan_per_segment_calls_equal_the_single_launch():
    """The reference drives one chunk-update call per 1024-token segment (grm/core/paper_grm.py:702-728);
    the state carried from call to call must give what the single launch over all segments gives."""
    rows, T, L, d, decay = 3, 8192, 1024, 128, 0.97
    g = torch.Generator(device=DEV).manual_seed(5)
    q = _unit(torch.randn(rows, T, d, device=DEV, generator=g)).to(torch.bfloat16)
    k = _unit(torch.randn(rows, T, d, device=DEV, generator=g)).to(torch.bfloat16)
    v = torch.randn(rows, T, d, device=DEV, generator=g).to(torch.bfloat16)
    archive = torch.zeros(rows, T // L, d, d, device=DEV)
    hidden, m_out = gx.chunk_scan_fwd_segments(k, v, q, torch.zeros(rows, d, d, device=DEV), decay, archive, 0, L)
    memory = torch.zeros(rows, d, d, device=DEV)
    for j in range(T // L):
        tok = slice(j * L, (j + 1) * L)
        h, memory = gx.chunk_scan_fwd(k[:, tok].contiguous(), v[:, tok].contiguous(), q[:, tok].contiguous(), memory, decay)
        assert go.rel_err(h.float().cpu().numpy(), hidden[:, tok].float().cpu().numpy()) < LOWP_TOL
        assert go.rel_err(memory.cpu().numpy(), archive[:, j].cpu().numpy()) < 1e-3
    assert cabi.device_error_word() == 0


# --------------------------------------------------------------------------- fusion rules through the runner

@pytest.mark.parametrize("mode", ["concat", "gate", "linear"])
def test_runner_with_weight_bearing_fusion_rules_matches_reference_model(golden, mode):
    """SegmentMemoryRunner against the reference's SegmentRecurrentMemoryModel(retrieval_fusion_mode=mode):
    outputs of every token, last hidden state and final memory at the fp32 tolerance."""
    g = golden(f"model_fusion_{mode}")
    params = {k[len("param::"):]: torch.from_numpy(v).to(DEV) for k, v in g.items() if k.startswith("param::")}
    x = torch.from_numpy(g["x"]).to(DEV)
    for dense in (True, False):                                         # both retrieval forms feed the rule
        runner = SegmentMemoryRunner(params, segment_length=64, retrieval_top_k=2, memory_capacity_segments=8,
                                     memory_decay=0.97, retrieval_fusion_mode=mode, memory_storage_dtype=torch.float32)
        runner.dense_retrieval = dense
        out, h_final, memory, aux = runner.forward(x, reset_memory=True)
        assert aux["num_segments"] == int(g["num_segments"]) == 4
        assert go.rel_err(out.cpu().numpy(), g["outputs"]) < FP32_TOL
        assert go.rel_err(h_final.cpu().numpy(), g["h_final"]) < FP32_TOL
        assert go.rel_err(memory.cpu().numpy(), g["memory_final"]) < FP32_TOL


# --------------------------------------------------------------------------- rank-2 retriever with masks

@pytest.mark.parametrize("name", ["topk", "identity", "causal", "masked"])
def test_rank2_retriever_with_masks_matches_reference_fixtures(golden, name):
    g = golden(f"retriever_{name}")
    mask = torch.from_numpy(g["attention_mask"]).to(DEV) if g["attention_mask"].size else None
    gates, indices, scores = topk_memory_retrieve(
        torch.from_numpy(g["query"]).to(DEV), torch.from_numpy(g["keys"]).to(DEV), torch.from_numpy(g["w_query"]).to(DEV),
        torch.from_numpy(g["w_key"]).to(DEV), int(g["top_k"]), segment_offset=int(g["segment_offset"]), attention_mask=mask)
    assert indices.shape == g["indices"].shape and indices.dtype == torch.int64
    assert np.array_equal(indices.cpu().numpy(), g["indices"])
    assert go.rel_err(gates.cpu().numpy(), g["gates"]) < FP32_TOL
    finite = np.isfinite(g["scores"])
    got_scores = scores.cpu().numpy()
    assert np.array_equal(np.isfinite(got_scores), finite)
    assert go.rel_err(got_scores[finite], g["scores"][finite]) < FP32_TOL
    # rank-3 queries (one per token) route each token like a rank-2 call of its own
    q3 = torch.from_numpy(g["query"]).to(DEV)[:, None, :].expand(-1, 3, -1).contiguous()
    gates3, indices3, _ = topk_memory_retrieve(
        q3, torch.from_numpy(g["keys"]).to(DEV), torch.from_numpy(g["w_query"]).to(DEV), torch.from_numpy(g["w_key"]).to(DEV),
        int(g["top_k"]), segment_offset=int(g["segment_offset"]), attention_mask=mask)
    assert torch.equal(indices3[:, 1], indices) and torch.equal(gates3[:, 2], gates)
