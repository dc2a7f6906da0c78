"""CPU restatement of GRM's segment-memory path -- TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA kernels are compared against.  Nothing in
the product package imports it; only ``tests/``, ``__graft_entry__.smoke()``
and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may.

Parity status: PINNED.  Every function below is checked in
``tests/test_oracle.py`` against fixtures under ``tests/golden/`` that were
produced by importing the reference's own Python implementation
(``tests/golden/make_golden.py``) and against the compiled reference C++
(``oracle/_ref``) when that library has been built.  The reference ships no
golden vectors of its own for this path (its tests are relational, with the
one literal fixture being the index tensors of examples/test_grm.py:203-210,
which the gather fixture reuses).

Top-k: the reference delegates selection to ``torch.topk`` (PyTorch, not
vendored, version unpinned by the reference: README.md:41); its order on equal
scores is unspecified.  ``topk_route`` here states the stricter rule this
engine implements -- equal scores resolve to the lower index -- which agrees
with ``torch.topk`` whenever the selected scores are distinct.

All citations are paths inside the Sggggt/RNN_with_GRM project.
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import numpy as np


# --------------------------------------------------------------------------- #
# chunked linear-memory update + query
# --------------------------------------------------------------------------- #

def chunk_update_sequential(keys, values, queries, memory, decay: float, dtype=np.float64):
    """Token-by-token definition (grm/csrc/grm_cuda.cpp:67-83).

    ``M <- M*decay + (v k^T * 1/sqrt(K)) * (1-decay)``; ``h_t = M q_t`` after
    the update (inclusive).  Returns ``(hidden[B,T,H], memory_out[B,H,K])``.
    """
    k = np.asarray(keys, dtype=dtype)
    v = np.asarray(values, dtype=dtype)
    q = np.asarray(queries, dtype=dtype)
    m = np.array(memory, dtype=dtype, copy=True)
    B, T, K = k.shape
    H = v.shape[2]
    inv_scale = dtype(1.0 / math.sqrt(float(K)))
    beta = dtype(1.0 - decay)
    lam = dtype(decay)
    hidden = np.zeros((B, T, H), dtype=dtype)
    for t in range(T):
        update = (v[:, t, :, None] * k[:, t, None, :]) * inv_scale
        m = m * lam + update * beta
        hidden[:, t] = np.einsum("bhk,bk->bh", m, q[:, t])
    return hidden, m


def chunk_update_vectorized(keys, values, queries, memory, decay: float, dtype=np.float64):
    """Closed form over one chunk (grm/core/cuda_ops.py:218-254).

    ``h_i = decay^(i+1) M0 q_i + (1-decay) sum_{j<=i} decay^(i-j) (q_i.k_j / sqrt(K)) v_j``
    ``M_T = decay^T M0 + sum_j (1-decay) decay^(T-1-j) / sqrt(K) v_j k_j^T``
    """
    k = np.asarray(keys, dtype=dtype)
    v = np.asarray(values, dtype=dtype)
    q = np.asarray(queries, dtype=dtype)
    m = np.asarray(memory, dtype=dtype)
    B, T, K = k.shape
    H = v.shape[2]
    if T == 0:
        return np.zeros((B, 0, H), dtype=dtype), m.copy()
    lam = dtype(decay)
    beta = dtype(1.0) - lam
    pos = np.arange(T, dtype=dtype)
    start = np.einsum("bhk,btk->bth", m, q) * np.power(lam, pos + 1)[None, :, None]
    scores = np.einsum("bik,bjk->bij", q, k) / dtype(math.sqrt(float(K)))
    rel = pos[:, None] - pos[None, :]
    weights = np.where(rel >= 0, np.power(lam, np.clip(rel, 0, None)), 0).astype(dtype)
    local = beta * np.einsum("bij,bjh->bih", scores * weights[None], v)
    hidden = start + local
    end = beta * np.power(lam, (T - 1) - pos) / dtype(math.sqrt(float(K)))
    delta = np.einsum("bth,btk->bhk", v * end[None, :, None], k)
    memory_out = np.power(lam, dtype(T)) * m + delta
    return hidden, memory_out


def chunk_update_backward(grad_hidden, grad_memory_out, keys, values, queries, memory, decay: float,
                          dtype=np.float64):
    """Gradients of the sequential definition by reverse accumulation.

    The reference obtains them by autograd replay of the same loop
    (grm/csrc/grm_cuda.cpp:92-126); this is that computation written out.
    Returns ``(grad_keys, grad_values, grad_queries, grad_memory)``.
    """
    k = np.asarray(keys, dtype=dtype)
    v = np.asarray(values, dtype=dtype)
    q = np.asarray(queries, dtype=dtype)
    gh = np.asarray(grad_hidden, dtype=dtype)
    m0 = np.asarray(memory, dtype=dtype)
    B, T, K = k.shape
    coeff = dtype((1.0 - decay) / math.sqrt(float(K)))
    lam = dtype(decay)
    states = np.zeros((T,) + m0.shape, dtype=dtype)
    m = m0.copy()
    for t in range(T):
        m = m * lam + coeff * v[:, t, :, None] * k[:, t, None, :]
        states[t] = m
    gk = np.zeros_like(k)
    gv = np.zeros_like(v)
    gq = np.zeros_like(q)
    a = np.array(grad_memory_out, dtype=dtype, copy=True)  # dL/dM_t accumulated from the future
    for t in range(T - 1, -1, -1):
        a = a + gh[:, t, :, None] * q[:, t, None, :]
        gq[:, t] = np.einsum("bhk,bh->bk", states[t], gh[:, t])
        gv[:, t] = coeff * np.einsum("bhk,bk->bh", a, k[:, t])
        gk[:, t] = coeff * np.einsum("bhk,bh->bk", a, v[:, t])
        a = a * lam
    return gk, gv, gq, a


def linear_scan(keys, values, queries, memory, decay, update_coeff, hidden_scale=1.0, memory_out_scale=1.0,
                reverse=False, first_step_no_decay=False, dtype=np.float64):
    """The generalised recurrence behind ``grmx_linear_scan`` (no reference counterpart)."""
    k = np.asarray(keys, dtype=dtype)
    v = np.asarray(values, dtype=dtype)
    q = np.asarray(queries, dtype=dtype)
    m = np.array(memory, dtype=dtype, copy=True)
    B, T, _ = k.shape
    hidden = np.zeros((B, T, v.shape[2]), dtype=dtype)
    order = range(T - 1, -1, -1) if reverse else range(T)
    for step, t in enumerate(order):
        a = dtype(1.0) if (first_step_no_decay and step == 0) else dtype(decay)
        m = a * m + dtype(update_coeff) * v[:, t, :, None] * k[:, t, None, :]
        hidden[:, t] = dtype(hidden_scale) * np.einsum("bhk,bk->bh", m, q[:, t])
    return hidden, m * dtype(memory_out_scale)


# --------------------------------------------------------------------------- #
# apply-query and gather
# --------------------------------------------------------------------------- #

def apply_query(memories, queries, dtype=np.float64):
    """``brhk,bk->brh`` / ``bqrhk,bqk->bqrh`` (grm/core/cuda_ops.py:257-262)."""
    m = np.asarray(memories, dtype=dtype)
    q = np.asarray(queries, dtype=dtype)
    if m.ndim == 5:
        return np.einsum("bqrhk,bqk->bqrh", m, q)
    if m.ndim == 4:
        return np.einsum("brhk,bk->brh", m, q)
    raise ValueError(f"Unsupported memory rank for apply-query: {m.ndim}")


def apply_query_backward(grad_hidden, memories, queries, dtype=np.float64):
    """``dM = dh (x) q``, ``dq = sum_{r,h} dh M`` (grm/csrc/apply_query.cu:77-169)."""
    m = np.asarray(memories, dtype=dtype)
    q = np.asarray(queries, dtype=dtype)
    g = np.asarray(grad_hidden, dtype=dtype)
    if m.ndim == 5:
        return np.einsum("bqrh,bqk->bqrhk", g, q), np.einsum("bqrh,bqrhk->bqk", g, m)
    return np.einsum("brh,bk->brhk", g, q), np.einsum("brh,brhk->bk", g, m)


def batched_gather(memories_per_batch, topk_indices):
    """``out[b,(q),r] = mem[b, idx[b,(q),r]]`` (grm/core/cuda_ops.py:265-284).  Bit copy."""
    mem = np.asarray(memories_per_batch)
    idx = np.asarray(topk_indices).astype(np.int64)
    if mem.ndim != 4:
        raise ValueError(f"Expected memories_per_batch rank 4, got {mem.ndim}")
    if idx.ndim not in (2, 3):
        raise ValueError(f"Expected topk_indices rank 2 or 3, got {idx.ndim}")
    out = np.empty((mem.shape[0],) + idx.shape[1:] + mem.shape[2:], dtype=mem.dtype)
    for b in range(mem.shape[0]):
        out[b] = mem[b][idx[b].reshape(-1)].reshape(out[b].shape)
    return out


# --------------------------------------------------------------------------- #
# routing: scores, top-k, gates
# --------------------------------------------------------------------------- #

def route_scores(queries, keys, scale: float):
    """fp32 dot products in double, rounded once -- NOT the bit-exact form.

    The engine's contract is a sequential fp32 fused multiply-add over the
    feature index; numpy has no fma, so the bit-exact restatement lives in the
    C oracle (``oracle/grm_oracle.c: grm_route_scores``).  This version is for
    tolerance checks of the scores tensor only.
    """
    q = np.asarray(queries, dtype=np.float64)
    k = np.asarray(keys, dtype=np.float64)
    return (np.einsum("bqd,bsd->bqs", q, k) * float(scale)).astype(np.float32)


def _order_key(x: np.float32) -> Tuple[int, float]:
    # NaN ranks above everything (torch.topk convention), then by value
    if np.isnan(x):
        return (1, 0.0)
    return (0, float(x))


def topk_route(scores, top_k: int, temperature: float = 1.0, visible=None):
    """Selection + gates on given scores ``[B,Q,S]`` (fp32).

    Rules (grm/core/gating_unit.py:81-90, grm/core/paper_grm.py:576-588):
    ``R = min(top_k, n_visible)``; when ``R == n_visible`` the routes are
    ``0..R-1`` in index order (no sort); else the R best in descending score
    order, equal scores to the lower index; gates = softmax(selected /
    temperature).  Slots beyond R hold index -1 and gate 0.
    """
    sc = np.asarray(scores, dtype=np.float32)
    B, Q, S = sc.shape
    idx = np.full((B, Q, top_k), -1, dtype=np.int64)
    gates = np.zeros((B, Q, top_k), dtype=np.float32)
    for qi in range(Q):
        n_vis = S if visible is None else int(min(max(int(visible[qi]), 0), S))
        R = min(top_k, n_vis)
        for b in range(B):
            row = sc[b, qi, :n_vis]
            if R == n_vis:
                sel = list(range(R))
            else:
                order = sorted(range(n_vis), key=lambda s: (tuple(-c for c in _order_key(row[s])), s))
                sel = order[:R]
            if R == 0:
                continue
            x = (row[sel] / np.float32(temperature)).astype(np.float32)
            with np.errstate(invalid="ignore", over="ignore"):
                e = np.exp((x - np.max(x)).astype(np.float32)).astype(np.float32)
                g = (e / np.sum(e, dtype=np.float32)).astype(np.float32)
            if np.isnan(x).any():
                g = np.full_like(g, np.nan)
            idx[b, qi, :R] = sel
            gates[b, qi, :R] = g
    return idx, gates


# --------------------------------------------------------------------------- #
# fusion
# --------------------------------------------------------------------------- #

def layer_norm(x, weight=None, bias=None, eps: float = 1e-5):
    x = np.asarray(x, dtype=np.float64)
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    y = (x - mean) / np.sqrt(var + eps)
    if weight is not None:
        y = y * np.asarray(weight, dtype=np.float64)
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)
    return y


def retrieved_state_fusion(online, retrieved, gates, mode: str = "residual",
                           params: Optional[Dict[str, np.ndarray]] = None, eps: float = 1e-5,
                           use_layer_norm: bool = True):
    """``RetrievedStateFusion.forward`` (grm/core/aggregator.py:66-145), dropout off.

    ``online[N,H]``, ``retrieved[N,R,H]``, ``gates[N,R]``; ``params`` holds the
    module's tensors by their state_dict names (``layer_norm.weight``,
    ``output_projection.weight`` ...).  Linear layers follow ``y = x W^T + b``.
    """
    p = {k: np.asarray(v, dtype=np.float64) for k, v in (params or {}).items()}
    h = np.asarray(online, dtype=np.float64)
    r = np.asarray(retrieved, dtype=np.float64)
    if r.shape[1] == 0:
        contrib = np.zeros_like(h)
    else:
        g = np.asarray(gates, dtype=np.float64)
        contrib = (r * g[..., None]).sum(axis=1)

    def linear(name, x):
        y = x @ p[f"{name}.weight"].T
        if f"{name}.bias" in p:
            y = y + p[f"{name}.bias"]
        return y

    if mode == "residual":
        fused = h + contrib
        if "output_projection.weight" in p:
            fused = linear("output_projection", fused)
    elif mode == "concat":
        fused = linear("output_projection", np.concatenate([h, contrib], axis=-1))
    elif mode == "gate":
        gate = 1.0 / (1.0 + np.exp(-linear("gate_projection", np.concatenate([h, contrib], axis=-1))))
        fused = gate * h + (1.0 - gate) * contrib
    elif mode == "linear":
        fused = linear("online_projection", h) + linear("memory_projection", contrib)
    else:
        raise ValueError(f"Unknown retrieval_fusion_mode: {mode}")
    if use_layer_norm:
        fused = layer_norm(fused, p.get("layer_norm.weight"), p.get("layer_norm.bias"), eps)
    return fused


def retrieve_fuse(archive, indices, gates, queries, online=None, ln_weight=None, ln_bias=None,
                  eps: float = 1e-5, mode: str = "residual_ln"):
    """The chain gather -> apply-query -> gate-weighted sum -> residual LayerNorm
    (grm/core/paper_grm.py:229-234,301-307,604-611; grm/core/aggregator.py:104-105,116-119,144)
    on ``archive[B,S,H,K]``, ``indices[B,Q,R]`` (-1 = empty slot), ``queries[B,Q,K]``.
    A query with no live slot returns ``online`` untouched (paper_grm.py:620-621).
    """
    arch = np.asarray(archive, dtype=np.float64)
    idx = np.asarray(indices).astype(np.int64)
    q = np.asarray(queries, dtype=np.float64)
    B, Q, R = idx.shape
    H = arch.shape[2]
    retrieved = np.zeros((B, Q, R, H), dtype=np.float64)
    for b in range(B):
        for qi in range(Q):
            for r in range(R):
                if idx[b, qi, r] >= 0:
                    retrieved[b, qi, r] = arch[b, idx[b, qi, r]] @ q[b, qi]
    if mode == "retrieved":
        return retrieved
    g = np.asarray(gates, dtype=np.float64)
    live = idx >= 0
    contrib = (retrieved * np.where(live, g, 0.0)[..., None]).sum(axis=2)
    if mode == "contrib":
        return contrib
    h = np.asarray(online, dtype=np.float64)
    fused = layer_norm(h + contrib, ln_weight, ln_bias, eps)
    none_live = ~live.any(axis=2)
    fused[none_live] = h[none_live]
    return fused


# --------------------------------------------------------------------------- #
# the single-layer model: segment loop over the pieces above
# --------------------------------------------------------------------------- #

def segment_model_forward(params: Dict[str, np.ndarray], x, *, segment_length: int, retrieval_top_k: int,
                          memory_capacity_segments: int, memory_decay: float = 0.97, mode: str = "residual",
                          eps: float = 1e-5):
    """``SegmentRecurrentMemoryModel.forward`` (grm/core/paper_grm.py:647-747) in float64, dropout off,
    ``memory_initialization_mode='checkpoint'``, zero start state, empty archive.

    Per segment: project and L2-normalise (``:491-493``, ``F.normalize`` eps 1e-6), scan (``:495``), route every
    token over the summaries of the archived segments (``:566-589``: bias-free projections, scale
    ``1/sqrt(route_dim)``, top-k or identity order, softmax over the selected scores), apply the token's
    query to the selected memories (``:301-307``), fuse (``:604-611``), project (``:709``), then archive the
    segment-end memory with the mean of the segment's inputs (``:522-523,721-725``), oldest evicted first.
    Returns ``(outputs [B,T,out], hidden_states [B,T,H], memory_final [B,H,K], routes)`` with
    ``routes[i] = (indices, gates)`` of the i-th segment that saw a non-empty archive.
    """
    p = {k: np.asarray(v, dtype=np.float64) for k, v in params.items()}
    x = np.asarray(x, dtype=np.float64)
    B, T, _ = x.shape

    def linear(name, t):
        y = t @ p[f"{name}.weight"].T
        return y + p[f"{name}.bias"] if f"{name}.bias" in p else y

    def unit(t):
        return t / np.maximum(np.linalg.norm(t, axis=-1, keepdims=True), 1e-6)

    H, K = p["memory_cell.value_proj.weight"].shape[0], p["memory_cell.key_proj.weight"].shape[0]
    route_dim = p["gating_unit.query_projection.weight"].shape[0]
    fusion_params = {k[len("aggregator."):]: v for k, v in p.items() if k.startswith("aggregator.")}
    memory = np.zeros((B, H, K))
    archive, summaries = [], []
    hidden_all, routes = [], []
    for s0 in range(0, T, segment_length):
        seg = x[:, s0:s0 + segment_length]
        k, v, q = unit(linear("memory_cell.key_proj", seg)), linear("memory_cell.value_proj", seg), \
            unit(linear("memory_cell.query_proj", seg))
        h_online, memory = chunk_update_sequential(k, v, q, memory, memory_decay)
        if archive:
            keys = np.stack(summaries, axis=1)
            scores = (seg @ p["gating_unit.query_projection.weight"].T) @ \
                np.swapaxes(keys @ p["gating_unit.key_projection.weight"].T, 1, 2) / math.sqrt(route_dim)
            idx, gates = topk_route(scores.astype(np.float32), retrieval_top_k)
            R = min(retrieval_top_k, len(archive))
            idx, gates = idx[..., :R], gates[..., :R]
            # gates from the float64 scores, so that this restatement stays a float64 one
            sel = np.take_along_axis(scores, idx, axis=-1)
            e = np.exp(sel - sel.max(axis=-1, keepdims=True))
            gates64 = e / e.sum(axis=-1, keepdims=True)
            stack = np.stack(archive, axis=1)                                   # [B, S, H, K]
            retrieved = np.einsum("bcrhk,bck->bcrh", stack[np.arange(B)[:, None, None], idx], q)
            C = seg.shape[1]
            fused = retrieved_state_fusion(h_online.reshape(B * C, H), retrieved.reshape(B * C, R, H),
                                           gates64.reshape(B * C, R), mode, fusion_params, eps).reshape(B, C, H)
            routes.append((idx, gates))
        else:
            fused = h_online                                                      # paper_grm.py:620-621
        hidden_all.append(fused)
        archive.append(memory.copy())
        summaries.append(seg.mean(axis=1))
        if len(archive) > memory_capacity_segments:
            archive.pop(0)
            summaries.pop(0)
    hidden = np.concatenate(hidden_all, axis=1) if hidden_all else np.zeros((B, 0, H))
    return linear("output_proj", hidden), hidden, memory, routes


def rel_err(actual, expected) -> float:
    """``max|a-b| / max|b|`` -- the parity metric the tolerances are stated in."""
    a = np.asarray(actual, dtype=np.float64)
    b = np.asarray(expected, dtype=np.float64)
    if b.size == 0:
        return 0.0
    denom = float(np.max(np.abs(b)))
    return float(np.max(np.abs(a - b))) / (denom if denom > 0 else 1.0)
