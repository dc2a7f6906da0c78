"""Checkers for the CUDA path -- TEST INFRASTRUCTURE ONLY (see grm_oracle.py).

``c_oracle()`` returns the ctypes handle of the plain-C restatement,
``reference_ops()`` the ``torch.ops.grm_ref`` namespace served by the
reference's own compiled CPU code, or ``None`` when that library was not built,
``reference_python()`` the folder that holds the staged reference package ``grm``
(to be put on ``sys.path``), or ``None`` when it was not staged.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p
from pathlib import Path

from . import grm_oracle  # noqa: F401

_HERE = Path(__file__).resolve().parent
_C_LIB = None
_REF_LOADED = False


def c_oracle() -> ctypes.CDLL:
    global _C_LIB
    if _C_LIB is None:
        path = _HERE / "_build" / "libgrm_oracle.so"
        if not path.exists():
            from .build_oracle import build_c_oracle

            build_c_oracle()
        lib = ctypes.CDLL(str(path))
        lib.grm_chunk_update_seq_f32.restype = None
        lib.grm_chunk_update_seq_f32.argtypes = [c_void_p] * 6 + [c_int64] * 4 + [c_float]
        lib.grm_apply_query_f32.restype = None
        lib.grm_apply_query_f32.argtypes = [c_void_p] * 3 + [c_int64] * 4
        lib.grm_batched_gather.restype = c_int64
        lib.grm_batched_gather.argtypes = [c_void_p] * 3 + [c_int64] * 4
        lib.grm_route_scores.restype = None
        lib.grm_route_scores.argtypes = [c_void_p] * 3 + [c_int64] * 4 + [c_float]
        lib.grm_topk_select.restype = None
        lib.grm_topk_select.argtypes = [c_void_p, c_void_p] + [c_int64] * 3 + [c_int, c_float, c_void_p, c_void_p]
        lib.grm_retrieve_fuse_f32.restype = None
        lib.grm_retrieve_fuse_f32.argtypes = [c_void_p] * 7 + [c_float, c_void_p] + [c_int64] * 6
        _C_LIB = lib
    return _C_LIB


def reference_ops():
    """``torch.ops.grm_ref`` (the reference's compiled CPU ops) or ``None``."""
    global _REF_LOADED
    import torch

    path = _HERE / "_ref" / "grm_ref_ops.so"
    if not path.exists():
        return None
    if not _REF_LOADED:
        torch.ops.load_library(str(path))
        _REF_LOADED = True
    return torch.ops.grm_ref


def reference_python():
    """Folder holding the staged reference package (``oracle/_ref/python``) or ``None``."""
    path = _HERE / "_ref" / "python"
    return path if (path / "grm" / "__init__.py").exists() else None


# ---- numpy-facing wrappers of the C functions ----

def _np():
    import numpy as np

    return np


def c_chunk_update(keys, values, queries, memory, decay: float):
    np = _np()
    k = np.ascontiguousarray(keys, dtype=np.float32)
    v = np.ascontiguousarray(values, dtype=np.float32)
    q = np.ascontiguousarray(queries, dtype=np.float32)
    m = np.ascontiguousarray(memory, dtype=np.float32)
    B, T, K = k.shape
    H = v.shape[2]
    hidden = np.empty((B, T, H), dtype=np.float32)
    m_out = np.empty_like(m)
    c_oracle().grm_chunk_update_seq_f32(k.ctypes.data, v.ctypes.data, q.ctypes.data, m.ctypes.data,
                                        hidden.ctypes.data, m_out.ctypes.data, B, T, K, H, float(decay))
    return hidden, m_out


def c_apply_query(memories, queries):
    np = _np()
    m = np.ascontiguousarray(memories, dtype=np.float32)
    q = np.ascontiguousarray(queries, dtype=np.float32)
    K = m.shape[-1]
    H = m.shape[-2]
    R = m.shape[-3]
    N = m.size // max(R * H * K, 1)
    out = np.empty(m.shape[:-1], dtype=np.float32)
    c_oracle().grm_apply_query_f32(m.ctypes.data, q.ctypes.data, out.ctypes.data, N, R, H, K)
    return out


def c_batched_gather(memories, indices):
    np = _np()
    mem = np.ascontiguousarray(memories)
    idx = np.ascontiguousarray(indices, dtype=np.int64)
    B, S = mem.shape[:2]
    J = idx.size // max(B, 1)
    row_bytes = mem[0, 0].nbytes if S > 0 else int(np.prod(mem.shape[2:])) * mem.itemsize
    out = np.empty(idx.shape + mem.shape[2:], dtype=mem.dtype)
    bad = c_oracle().grm_batched_gather(mem.ctypes.data, idx.ctypes.data, out.ctypes.data, B, S, J, row_bytes)
    return out, int(bad)


def c_route_scores(queries, keys, scale: float):
    np = _np()
    q = np.ascontiguousarray(queries, dtype=np.float32)
    k = np.ascontiguousarray(keys, dtype=np.float32)
    B, Q, D = q.shape
    S = k.shape[1]
    scores = np.empty((B, Q, S), dtype=np.float32)
    c_oracle().grm_route_scores(q.ctypes.data, k.ctypes.data, scores.ctypes.data, B, Q, S, D, float(scale))
    return scores


def c_topk_select(scores, top_k: int, temperature: float = 1.0, visible=None):
    np = _np()
    if top_k > 64:
        raise ValueError("top_k above 64 is outside the oracle's range")
    sc = np.ascontiguousarray(scores, dtype=np.float32)
    B, Q, S = sc.shape
    idx = np.empty((B, Q, top_k), dtype=np.int64)
    gates = np.empty((B, Q, top_k), dtype=np.float32)
    vis = None if visible is None else np.ascontiguousarray(visible, dtype=np.int32)
    c_oracle().grm_topk_select(sc.ctypes.data, None if vis is None else vis.ctypes.data, B, Q, S, int(top_k),
                               float(temperature), idx.ctypes.data, gates.ctypes.data)
    return idx, gates


def c_retrieve_fuse(archive, indices, gates, queries, online, ln_weight=None, ln_bias=None, eps: float = 1e-5):
    np = _np()
    a = np.ascontiguousarray(archive, dtype=np.float32)
    idx = np.ascontiguousarray(indices, dtype=np.int64)
    g = np.ascontiguousarray(gates, dtype=np.float32)
    q = np.ascontiguousarray(queries, dtype=np.float32)
    h = np.ascontiguousarray(online, dtype=np.float32)
    w = None if ln_weight is None else np.ascontiguousarray(ln_weight, dtype=np.float32)
    b = None if ln_bias is None else np.ascontiguousarray(ln_bias, dtype=np.float32)
    B, S, H, K = a.shape
    _, Q, R = idx.shape
    out = np.empty((B, Q, H), dtype=np.float32)
    c_oracle().grm_retrieve_fuse_f32(a.ctypes.data, idx.ctypes.data, g.ctypes.data, q.ctypes.data, h.ctypes.data,
                                     None if w is None else w.ctypes.data, None if b is None else b.ctypes.data,
                                     float(eps), out.ctypes.data, B, S, Q, R, H, K)
    return out
