"""Thin callers of the C ABI for the GPU tests: torch tensors in, torch tensors out.

Each helper allocates the outputs, passes raw device pointers and the current
stream through ``rnn_with_grm_b200.cabi`` (ctypes) and returns the outputs.  No
torch op computes anything here.
"""

from __future__ import annotations

import math

import torch

from rnn_with_grm_b200 import cabi


def chunk_scan_fwd(keys, values, queries, memory, decay, path=cabi.PATH_AUTO):
    lib = cabi.load()
    B, T, K = keys.shape
    H = values.shape[2]
    hidden = torch.empty(B, T, H, device=keys.device, dtype=values.dtype)
    memory_out = torch.empty_like(memory)
    cabi.check(lib.grmx_chunk_scan_fwd(
        cabi.ptr(keys), cabi.ptr(values), cabi.ptr(queries), cabi.ptr(memory), cabi.ptr(hidden),
        cabi.ptr(memory_out), B, T, K, H, float(decay), cabi.dtype_code(keys.dtype),
        cabi.dtype_code(memory.dtype), path, cabi.current_stream()))
    return hidden, memory_out


def chunk_scan_scratch_bytes(B, T, K, H, io_dtype, state_dtype):
    return int(cabi.load().grmx_chunk_scan_scratch_bytes(B, T, K, H, cabi.dtype_code(io_dtype),
                                                         cabi.dtype_code(state_dtype)))


def chunk_scan_fwd_ws(keys, values, queries, memory, decay, scratch, path=cabi.PATH_AUTO):
    """Forward scan with a caller-provided workspace (a uint8 CUDA tensor, or None)."""
    lib = cabi.load()
    B, T, K = keys.shape
    H = values.shape[2]
    hidden = torch.empty(B, T, H, device=keys.device, dtype=values.dtype)
    memory_out = torch.empty_like(memory)
    cabi.check(lib.grmx_chunk_scan_fwd_ws(
        cabi.ptr(keys), cabi.ptr(values), cabi.ptr(queries), cabi.ptr(memory), cabi.ptr(hidden),
        cabi.ptr(memory_out), B, T, K, H, float(decay), cabi.dtype_code(keys.dtype),
        cabi.dtype_code(memory.dtype), path, cabi.ptr(scratch), 0 if scratch is None else scratch.numel(),
        cabi.current_stream()))
    return hidden, memory_out


def chunk_scan_bwd(grad_hidden, grad_memory_out, keys, values, queries, memory, decay, path=cabi.PATH_AUTO):
    lib = cabi.load()
    B, T, K = keys.shape
    H = values.shape[2]
    gk, gv, gq, gm = (torch.empty_like(t) for t in (keys, values, queries, memory))
    cabi.check(lib.grmx_chunk_scan_bwd(
        cabi.ptr(grad_hidden), cabi.ptr(grad_memory_out), cabi.ptr(keys), cabi.ptr(values), cabi.ptr(queries),
        cabi.ptr(memory), cabi.ptr(gk), cabi.ptr(gv), cabi.ptr(gq), cabi.ptr(gm), B, T, K, H, float(decay),
        cabi.dtype_code(keys.dtype), cabi.dtype_code(memory.dtype), path, cabi.current_stream()))
    return gk, gv, gq, gm


def linear_scan(keys, values, queries, memory, decay, update_coeff, hidden_scale=1.0, memory_out_scale=1.0,
                reverse=False, first_step_no_decay=False, path=cabi.PATH_AUTO, transposed_state=False):
    lib = cabi.load()
    B, T, K = keys.shape
    H = values.shape[2]
    hidden = torch.empty(B, T, H, device=keys.device, dtype=values.dtype)
    memory_out = torch.empty(B, H, K, device=keys.device, dtype=memory.dtype)
    rs, cs = (1, H) if transposed_state else (K, 1)
    cabi.check(lib.grmx_linear_scan(
        cabi.ptr(keys), cabi.ptr(values), cabi.ptr(queries), cabi.ptr(memory), rs, cs, cabi.ptr(hidden),
        cabi.ptr(memory_out), B, T, K, H, float(decay), float(update_coeff), float(hidden_scale),
        float(memory_out_scale), int(reverse), int(first_step_no_decay), cabi.dtype_code(keys.dtype),
        cabi.dtype_code(memory.dtype), path, cabi.current_stream()))
    return hidden, memory_out


def apply_query_fwd(memories, queries):
    lib = cabi.load()
    R, H, K = memories.shape[-3:]
    N = memories.numel() // max(R * H * K, 1)
    hidden = torch.empty(memories.shape[:-1], device=memories.device, dtype=memories.dtype)
    cabi.check(lib.grmx_apply_query_fwd(cabi.ptr(memories), cabi.ptr(queries), cabi.ptr(hidden), N, R, H, K,
                                        cabi.dtype_code(memories.dtype), cabi.current_stream()))
    return hidden


def apply_query_bwd(grad_hidden, memories, queries):
    lib = cabi.load()
    R, H, K = memories.shape[-3:]
    N = memories.numel() // max(R * H * K, 1)
    gm, gq = torch.empty_like(memories), torch.empty_like(queries)
    cabi.check(lib.grmx_apply_query_bwd(cabi.ptr(grad_hidden), cabi.ptr(memories), cabi.ptr(queries), cabi.ptr(gm),
                                        cabi.ptr(gq), N, R, H, K, cabi.dtype_code(memories.dtype),
                                        cabi.current_stream()))
    return gm, gq


def batched_gather(memories, indices):
    lib = cabi.load()
    B, S = memories.shape[:2]
    row_elems = math.prod(memories.shape[2:])
    J = indices.numel() // max(B, 1)
    out = torch.empty(tuple(indices.shape) + tuple(memories.shape[2:]), device=memories.device, dtype=memories.dtype)
    cabi.check(lib.grmx_batched_gather(cabi.ptr(memories), cabi.ptr(indices), cabi.ptr(out), B, S, J, row_elems,
                                       memories.element_size(), cabi.current_stream()))
    return out


def topk_route(queries, keys, top_k, scale=1.0, temperature=1.0, visible=None, want_scores=True):
    lib = cabi.load()
    B, Q, D = queries.shape
    S = keys.shape[1]
    idx = torch.empty(B, Q, top_k, device=queries.device, dtype=torch.int64)
    gates = torch.empty(B, Q, top_k, device=queries.device, dtype=torch.float32)
    scores = torch.empty(B, Q, S, device=queries.device, dtype=torch.float32) if want_scores else None
    entry = lib.grmx_topk_route_bf16q if queries.dtype == torch.bfloat16 else lib.grmx_topk_route
    cabi.check(entry(cabi.ptr(queries), cabi.ptr(keys), cabi.ptr(visible), B, Q, S, D, top_k,
                                   float(scale), float(temperature), cabi.ptr(idx), cabi.ptr(gates),
                                   cabi.ptr(scores), cabi.current_stream()))
    return idx, gates, scores


def topk_select(scores, top_k, temperature=1.0, visible=None):
    lib = cabi.load()
    B, Q, S = scores.shape
    idx = torch.empty(B, Q, top_k, device=scores.device, dtype=torch.int64)
    gates = torch.empty(B, Q, top_k, device=scores.device, dtype=torch.float32)
    cabi.check(lib.grmx_topk_select(cabi.ptr(scores), cabi.ptr(visible), B, Q, S, top_k, float(temperature),
                                    cabi.ptr(idx), cabi.ptr(gates), cabi.current_stream()))
    return idx, gates


def retrieve_fuse(archive, indices, gates, queries, online=None, ln_weight=None, ln_bias=None, eps=1e-5,
                  mode=cabi.FUSE_RESIDUAL_LN):
    lib = cabi.load()
    B, S, H, K = archive.shape
    _, Q, R = indices.shape
    shape = (B, Q, R, H) if mode == cabi.FUSE_RETRIEVED else (B, Q, H)
    out = torch.empty(shape, device=archive.device, dtype=torch.float32)
    cabi.check(lib.grmx_retrieve_fuse(cabi.ptr(archive), cabi.ptr(indices), cabi.ptr(gates), cabi.ptr(queries),
                                      cabi.ptr(online), cabi.ptr(ln_weight), cabi.ptr(ln_bias), float(eps),
                                      cabi.ptr(out), B, S, Q, R, H, K, mode, cabi.current_stream()))
    return out


def retrieve_fuse_rows(archive, indices, gates, queries, online=None, ln_weight=None, ln_bias=None, eps=1e-5,
                       mode=cabi.FUSE_RESIDUAL_LN):
    """The slot-major form, asked for by name (grmx_retrieve_fuse picks it by shape)."""
    lib = cabi.load()
    B, S, H, K = archive.shape
    _, Q, R = indices.shape
    out = torch.empty(B, Q, H, device=archive.device, dtype=torch.float32)
    cabi.check(lib.grmx_retrieve_fuse_rows(cabi.ptr(archive), cabi.ptr(indices), cabi.ptr(gates), cabi.ptr(queries),
                                           cabi.ptr(online), cabi.ptr(ln_weight), cabi.ptr(ln_bias), float(eps),
                                           cabi.ptr(out), B, S, Q, R, H, K, mode, cabi.current_stream()))
    return out


def retrieve_fuse_tc(archive, indices, gates, queries, online=None, ln_weight=None, ln_bias=None, eps=1e-5,
                     mode=cabi.FUSE_RESIDUAL_LN):
    """Tensor-core retrieval: bf16 archive, queries, online state and output."""
    lib = cabi.load()
    B, S, H, K = archive.shape
    _, Q, R = indices.shape
    out = torch.empty(B, Q, H, device=archive.device, dtype=torch.bfloat16)
    cabi.check(lib.grmx_retrieve_fuse_tc(cabi.ptr(archive), cabi.ptr(indices), cabi.ptr(gates), cabi.ptr(queries),
                                         cabi.ptr(online), cabi.ptr(ln_weight), cabi.ptr(ln_bias), float(eps),
                                         cabi.ptr(out), B, S, Q, R, H, K, mode, cabi.current_stream()))
    return out


def add_layer_norm(a, b, ln_weight=None, ln_bias=None, eps=1e-5):
    lib = cabi.load()
    H = a.shape[-1]
    out = torch.empty_like(a)
    dtype = cabi.F32 if a.dtype == torch.float32 else cabi.BF16
    cabi.check(lib.grmx_add_layer_norm(cabi.ptr(a), cabi.ptr(b), cabi.ptr(ln_weight), cabi.ptr(ln_bias), float(eps),
                                       cabi.ptr(out), a.numel() // H, H, dtype, cabi.current_stream()))
    return out


def select_fuse(states, indices, gates, online=None, ln_weight=None, ln_bias=None, eps=1e-5,
                mode=cabi.FUSE_RESIDUAL_LN):
    lib = cabi.load()
    B, Q, S, H = states.shape
    R = indices.shape[2]
    out = torch.empty(B, Q, H, device=states.device, dtype=states.dtype)
    cabi.check(lib.grmx_select_fuse(cabi.ptr(states), cabi.ptr(indices), cabi.ptr(gates), cabi.ptr(online),
                                    cabi.ptr(ln_weight), cabi.ptr(ln_bias), float(eps), cabi.ptr(out), B, Q, S, R, H,
                                    cabi.dtype_code(states.dtype), mode, cabi.current_stream()))
    return out



def archive_push(memory, archive, shadow, slot):
    lib = cabi.load()
    B, S, H, K = archive.shape
    cabi.check(lib.grmx_archive_push(cabi.ptr(memory), cabi.ptr(archive), cabi.ptr(shadow), B, S, slot, H * K,
                                     cabi.current_stream()))


def normalize_rows(x, eps=1e-6, out_dtype=None):
    lib = cabi.load()
    out = torch.empty_like(x, dtype=out_dtype or x.dtype)
    K = x.shape[-1]
    cabi.check(lib.grmx_normalize_rows(cabi.ptr(x), cabi.ptr(out), x.numel() // K, K, float(eps),
                                       cabi.dtype_code(x.dtype), cabi.dtype_code(out.dtype), cabi.current_stream()))
    return out


def project_normalize(x, weights, bias=None, eps=1e-6):
    lib = cabi.load()
    D = x.shape[-1]
    K = weights.shape[0] // 2
    rows = x.numel() // D
    a = torch.empty(*x.shape[:-1], K, device=x.device, dtype=torch.bfloat16)
    b = torch.empty_like(a)
    cabi.check(lib.grmx_project_normalize(cabi.ptr(x), cabi.ptr(weights), cabi.ptr(bias), cabi.ptr(a), cabi.ptr(b), rows, D, K,
                                          float(eps), cabi.current_stream()))
    return a, b


def chunk_scan_fwd_segments(k, v, q, m, decay, archive, first_slot, segment_tokens):
    lib = cabi.load()
    B, T, K = k.shape
    H = v.shape[2]
    hidden = torch.empty_like(v)
    m_out = torch.empty_like(m)
    cabi.check(lib.grmx_chunk_scan_fwd_segments(cabi.ptr(k), cabi.ptr(v), cabi.ptr(q), cabi.ptr(m), cabi.ptr(hidden),
                                                cabi.ptr(m_out), cabi.ptr(archive), archive.shape[1], first_slot,
                                                segment_tokens, B, T, K, H, float(decay), cabi.dtype_code(k.dtype),
                                                cabi.dtype_code(m.dtype), cabi.current_stream()))
    return hidden, m_out
