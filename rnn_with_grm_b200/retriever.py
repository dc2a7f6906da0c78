"""``TopKMemoryRetriever.forward`` of the reference (grm/core/gating_unit.py:54-91) on this engine's kernels.

The reference module owns two bias-free projections and routes one query per batch row (rank 2) over
``S`` segment keys: scores ``(W_q x)(W_k s)^T / sqrt(hidden_dim)``, an optional attention mask and the
causal mask ``s >= segment_offset`` applied as ``-inf`` after scoring, ``torch.topk`` over all ``S``
scores (identity order when ``top_k >= S``), softmax over the selected scores.  Here the projections
stay ``torch.nn.functional.linear`` (cuBLAS), the scores come from ``torch.ops.grmx.topk_route`` (the
sequential fp32 multiply-add of the engine's routing contract), masks are applied to that score
tensor exactly as the reference does, and the selection and gates come from
``torch.ops.grmx.topk_select``: equal scores -- which includes every masked ``-inf`` -- go to the lower
index, where ``torch.topk`` leaves the order unspecified.

Returns what the reference returns: ``(routing_weights [B, R], top_indices [B, R], scores [B, S])`` with
``R = min(top_k, S)``; rank-3 queries ``[B, C, D]`` (one query per token) give ``[B, C, R]`` and ``[B, C, S]``.
CUDA tensors only.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor

from . import cuda_ops


def topk_memory_retrieve(query: Tensor, keys: Tensor, query_weight: Tensor, key_weight: Tensor, retrieval_top_k: int,
                         *, temperature: float = 1.0, segment_offset: int = 0,
                         attention_mask: Optional[Tensor] = None,
                         use_causal_mask: bool = True) -> Tuple[Tensor, Tensor, Tensor]:
    if not cuda_ops.load_grm_cuda_extension():
        raise RuntimeError("topk_memory_retrieve: the grm_cuda extension is not loaded: "
                           + str(cuda_ops.get_grm_cuda_runtime_status()["load_error"]))
    if query.device.type != "cuda":
        raise RuntimeError("topk_memory_retrieve: tensors must be on a CUDA device; this engine has no CPU path")
    per_token = query.dim() == 3
    if query.dim() not in (2, 3):
        raise ValueError(f"query must have shape [B, D] or [B, C, D], got rank {query.dim()}")
    batch = query.shape[0]
    if keys.dim() == 2:                                    # gating_unit.py:64-65: shared keys
        keys = keys.unsqueeze(0).expand(batch, -1, -1)
    num_keys = keys.shape[1]
    hidden_dim = query_weight.shape[0]
    projected_query = F.linear(query.float(), query_weight.float())
    projected_keys = F.linear(keys.float(), key_weight.float()).contiguous()
    q3 = projected_query if per_token else projected_query.unsqueeze(1)
    routes = min(int(retrieval_top_k), num_keys)
    if num_keys == 0:
        shape = q3.shape[:2]
        empty = (torch.zeros(*shape, 0, device=query.device), torch.zeros(*shape, 0, device=query.device, dtype=torch.int64),
                 torch.zeros(*shape, 0, device=query.device))
        return empty if per_token else tuple(t[:, 0] for t in empty)
    masked = attention_mask is not None or (use_causal_mask and 0 < segment_offset < num_keys)
    gates, indices, scores = torch.ops.grmx.topk_route(q3.contiguous(), projected_keys, None, routes,
                                                       1.0 / math.sqrt(hidden_dim), float(temperature), True)
    if masked:
        if attention_mask is not None:                      # gating_unit.py:73-74
            mask = attention_mask.bool()
            scores = scores.masked_fill(~(mask if per_token and mask.dim() == 3 else mask.unsqueeze(1)), float("-inf"))
        if use_causal_mask and 0 < segment_offset < num_keys:     # gating_unit.py:77-79
            scores[..., segment_offset:] = float("-inf")
        gates, indices = torch.ops.grmx.topk_select(scores, None, routes, float(temperature))
    if per_token:
        return gates, indices, scores
    return gates[:, 0], indices[:, 0], scores[:, 0]
