"""Drop-in for the reference's runtime-op layer ``grm/core/cuda_ops.py``.

Same seven public names, same signatures and keyword arguments, same
``get_grm_cuda_runtime_status`` fields and the same two ``autograd.Function``
shapes (reference: grm/core/cuda_ops.py:62-89 loader, :185-215 status,
:287-344 autograd, :347-402 ops, :405-413 ``__all__``).  What differs is what
sits underneath: ``torch.ops.grm_cuda.*`` is served by hand-written sm_100a
kernels behind the C ABI of ``include/grmx.h``, and there is no other path.

* Tensors must live on a CUDA device; a CPU tensor raises ``RuntimeError``.
* ``enabled=False``, ``debug_fallback=True`` and the ``fallback`` kernel policy
  are accepted for signature compatibility but raise ``RuntimeError``: this
  engine ships no PyTorch fallback math (the reference's
  ``_vectorized_chunk_update`` and friends, :218-284, have no counterpart
  here).
* ``memory`` may be float32 while keys/values/queries are bf16/fp16 (fp32
  carried state); the reference requires one dtype for all four tensors
  (grm/csrc/chunk_update.cu:498-502).
"""

from __future__ import annotations

import importlib
import os
import sys
from typing import Any, Dict, Optional, Tuple

import torch
from torch import Tensor

_IMPORT_CANDIDATES = ("rnn_with_grm_b200.grm_cuda_ext", "grm_cuda_ext", "grm.grm_cuda_ext")
_REGISTERED_OPS = (
    "chunk_update_forward",
    "chunk_update_backward",
    "apply_query_forward",
    "apply_query_backward",
    "batched_memory_gather",
)

_EXTENSION_MODULE: Optional[Any] = None
_EXTENSION_LOAD_ATTEMPTED = False
_EXTENSION_LOAD_ERROR = ""
_KERNEL_POLICY_ENV = "GRM_CUDA_KERNEL_POLICY"
_KERNEL_POLICY_OP_ENVS = {
    "chunk_update": "GRM_CUDA_CHUNK_UPDATE_POLICY",
    "apply_query": "GRM_CUDA_APPLY_QUERY_POLICY",
    "batched_memory_gather": "GRM_CUDA_BATCHED_GATHER_POLICY",
}
_VALID_KERNEL_POLICIES = {"auto", "native", "fallback"}
_SCAN_PATHS = {"auto": 0, "ffma": 1, "tcgen05": 2}


def _has_registered_ops() -> bool:
    namespace = getattr(torch.ops, "grm_cuda", None)
    if namespace is None:
        return False
    return all(hasattr(namespace, op_name) for op_name in _REGISTERED_OPS)


def _has_dispatch_kernel(op_name: str, dispatch_key: str) -> bool:
    checker = getattr(torch._C, "_dispatch_has_kernel_for_dispatch_key", None)
    if checker is None:
        return False
    try:
        return bool(checker(f"grm_cuda::{op_name}", dispatch_key))
    except Exception:
        return False


def _get_dispatch_kernel_status() -> Dict[str, Dict[str, bool]]:
    return {
        op_name: {
            "cuda": _has_dispatch_kernel(op_name, "CUDA"),
            "composite_explicit_autograd": _has_dispatch_kernel(op_name, "CompositeExplicitAutograd"),
        }
        for op_name in _REGISTERED_OPS
    }


def load_grm_cuda_extension(force: bool = False) -> bool:
    """Import the compiled extension once per process (reference :62-89)."""
    global _EXTENSION_MODULE, _EXTENSION_LOAD_ATTEMPTED, _EXTENSION_LOAD_ERROR

    if _EXTENSION_MODULE is not None and not force:
        return True
    if _EXTENSION_LOAD_ATTEMPTED and not force:
        return False

    _EXTENSION_LOAD_ATTEMPTED = True
    _EXTENSION_MODULE = None
    _EXTENSION_LOAD_ERROR = ""

    errors = []
    for module_name in _IMPORT_CANDIDATES:
        try:
            module = importlib.import_module(module_name)
        except Exception as exc:
            errors.append(f"{module_name}: {type(exc).__name__}: {exc}")
            continue
        if not _has_registered_ops():
            errors.append(f"{module_name}: torch.ops.grm_cuda registration missing")
            continue
        _EXTENSION_MODULE = module
        scan_path = os.environ.get("GRMX_SCAN_PATH", "").strip().lower()
        if scan_path in _SCAN_PATHS and hasattr(module, "set_scan_path"):
            module.set_scan_path(_SCAN_PATHS[scan_path])
        return True

    _EXTENSION_LOAD_ERROR = "; ".join(errors)
    return False


def is_grm_cpp_extension_available() -> bool:
    return load_grm_cuda_extension()


def _get_kernel_policy(op_name: str) -> str:
    env_names = (_KERNEL_POLICY_OP_ENVS.get(op_name, ""), _KERNEL_POLICY_ENV)
    for env_name in env_names:
        if not env_name:
            continue
        value = os.environ.get(env_name, "").strip().lower()
        if value in _VALID_KERNEL_POLICIES:
            return value
    return "auto"


def is_grm_cuda_available() -> bool:
    if not load_grm_cuda_extension():
        return False
    dispatch_status = _get_dispatch_kernel_status()
    return all(status["cuda"] for status in dispatch_status.values()) and torch.cuda.is_available()


def get_grm_cuda_runtime_status() -> Dict[str, Any]:
    """Field-for-field the dict of the reference (grm/core/cuda_ops.py:198-215)."""
    extension_loaded = load_grm_cuda_extension()
    namespace = getattr(torch.ops, "grm_cuda", None)
    registered_ops = {op_name: bool(namespace and hasattr(namespace, op_name)) for op_name in _REGISTERED_OPS}
    compiled_with_cuda_sources = bool(
        getattr(_EXTENSION_MODULE, "__grm_cuda_with_kernels__", False) if _EXTENSION_MODULE is not None else False
    )
    dispatch_kernels = _get_dispatch_kernel_status() if extension_loaded else {
        op_name: {"cuda": False, "composite_explicit_autograd": False} for op_name in _REGISTERED_OPS
    }
    compiled_with_cuda_kernels = compiled_with_cuda_sources and all(
        dispatch_status["cuda"] for dispatch_status in dispatch_kernels.values()
    )
    return {
        "load_attempted": _EXTENSION_LOAD_ATTEMPTED,
        "extension_loaded": extension_loaded,
        "compiled_with_cuda_sources": compiled_with_cuda_sources,
        "compiled_with_cuda_kernels": compiled_with_cuda_kernels,
        "torch_cuda_available": torch.cuda.is_available(),
        "cuda_backend_available": compiled_with_cuda_kernels and torch.cuda.is_available(),
        "load_error": _EXTENSION_LOAD_ERROR,
        "module_name": getattr(_EXTENSION_MODULE, "__name__", "") if _EXTENSION_MODULE is not None else "",
        "registered_ops": registered_ops,
        "dispatch_kernels": dispatch_kernels,
        "kernel_policy": {
            "global": _get_kernel_policy(""),
            "chunk_update": _get_kernel_policy("chunk_update"),
            "apply_query": _get_kernel_policy("apply_query"),
            "batched_memory_gather": _get_kernel_policy("batched_memory_gather"),
        },
    }


def set_scan_path(path: str) -> None:
    """Pin the chunk-scan kernel family: ``auto``, ``ffma`` (exact fp32) or ``tcgen05``."""
    if path not in _SCAN_PATHS:
        raise ValueError(f"scan path must be one of {sorted(_SCAN_PATHS)}, got {path!r}")
    _require_extension("set_scan_path")
    _EXTENSION_MODULE.set_scan_path(_SCAN_PATHS[path])


def _require_extension(op_name: str) -> None:
    if not load_grm_cuda_extension():
        raise RuntimeError(
            f"{op_name}: the grm_cuda extension is not loaded ({_EXTENSION_LOAD_ERROR or 'not built'}). "
            "Build it with `python -m rnn_with_grm_b200.build`; this engine has no fallback path."
        )


def _require_native(op_name: str, policy_key: str, device: torch.device, *, enabled: bool, debug_fallback: bool) -> None:
    if not enabled or debug_fallback or _get_kernel_policy(policy_key) == "fallback":
        raise RuntimeError(
            f"{op_name}: a fallback path was requested (enabled={enabled}, debug_fallback={debug_fallback}, "
            f"policy={_get_kernel_policy(policy_key)!r}) but this engine ships only the sm_100a kernels."
        )
    _require_extension(op_name)
    if device.type != "cuda":
        raise RuntimeError(f"{op_name}: tensors must be on a CUDA device, got {device}; this engine has no CPU path.")


class ChunkUpdateCudaFn(torch.autograd.Function):
    """Same contract as the reference class (grm/core/cuda_ops.py:287-321)."""

    @staticmethod
    def forward(ctx, keys: Tensor, values: Tensor, queries: Tensor, memory: Tensor, memory_decay: float):
        hidden, memory_out, aux = torch.ops.grm_cuda.chunk_update_forward(
            keys, values, queries, memory, float(memory_decay)
        )
        ctx.memory_decay = float(memory_decay)
        ctx.save_for_backward(keys, values, queries, memory, aux)
        return hidden, memory_out

    @staticmethod
    def backward(ctx, grad_hidden: Tensor, grad_memory_out: Tensor):
        keys, values, queries, memory, aux = ctx.saved_tensors
        if grad_hidden.dtype != keys.dtype:
            grad_hidden = grad_hidden.to(keys.dtype)
        # the carried state may be fp32 while the tokens are bf16
        if grad_memory_out.dtype != memory.dtype:
            grad_memory_out = grad_memory_out.to(memory.dtype)
        grad_k, grad_v, grad_q, grad_memory = torch.ops.grm_cuda.chunk_update_backward(
            grad_hidden.contiguous(),
            grad_memory_out.contiguous(),
            keys,
            values,
            queries,
            memory,
            aux,
            float(ctx.memory_decay),
        )
        return grad_k, grad_v, grad_q, grad_memory, None


class ApplyQueryCudaFn(torch.autograd.Function):
    """Same contract as the reference class (grm/core/cuda_ops.py:324-344)."""

    @staticmethod
    def forward(ctx, memories: Tensor, queries: Tensor):
        hidden = torch.ops.grm_cuda.apply_query_forward(memories, queries)
        ctx.save_for_backward(memories, queries)
        return hidden

    @staticmethod
    def backward(ctx, grad_hidden: Tensor):
        memories, queries = ctx.saved_tensors
        if grad_hidden.dtype != memories.dtype:
            grad_hidden = grad_hidden.to(memories.dtype)
        grad_memories, grad_queries = torch.ops.grm_cuda.apply_query_backward(
            grad_hidden.contiguous(), memories, queries
        )
        return grad_memories, grad_queries


def cuda_chunk_update(
    keys: Tensor,
    values: Tensor,
    queries: Tensor,
    memory: Tensor,
    memory_decay: float,
    *,
    enabled: bool = True,
    debug_fallback: bool = False,
) -> Tuple[Tensor, Tensor]:
    """``hidden[B,T,H], memory_out[B,H,K]`` of the decayed linear-memory scan (reference :347-367)."""
    _require_native("cuda_chunk_update", "chunk_update", memory.device, enabled=enabled, debug_fallback=debug_fallback)
    return ChunkUpdateCudaFn.apply(keys, values, queries, memory, float(memory_decay))


def cuda_apply_query(
    memories: Tensor,
    queries: Tensor,
    *,
    enabled: bool = True,
    debug_fallback: bool = False,
) -> Tensor:
    """``brhk,bk->brh`` / ``bqrhk,bqk->bqrh`` (reference :370-385)."""
    _require_native("cuda_apply_query", "apply_query", memories.device, enabled=enabled, debug_fallback=debug_fallback)
    if memories.ndim not in (4, 5):
        raise ValueError(f"Unsupported memory rank for apply-query: {memories.ndim}")
    return ApplyQueryCudaFn.apply(memories, queries)


def cuda_batched_memory_gather(
    memories_per_batch: Tensor,
    topk_indices: Tensor,
    *,
    enabled: bool = True,
    debug_fallback: bool = False,
) -> Tensor:
    """``out[b,(q),r] = memories_per_batch[b, topk_indices[b,(q),r]]`` (reference :388-402)."""
    _require_native(
        "cuda_batched_memory_gather",
        "batched_memory_gather",
        memories_per_batch.device,
        enabled=enabled,
        debug_fallback=debug_fallback,
    )
    if memories_per_batch.ndim != 4:
        raise ValueError(f"Expected memories_per_batch rank 4, got {memories_per_batch.ndim}")
    if topk_indices.ndim not in {2, 3}:
        raise ValueError(f"Expected topk_indices rank 2 or 3, got {topk_indices.ndim}")
    return torch.ops.grm_cuda.batched_memory_gather(memories_per_batch, topk_indices)


def install_as_grm_cuda_ops() -> None:
    """Serve ``grm.core.cuda_ops`` from this module.

    Call before ``import grm``: the reference's models then resolve their
    ``from .cuda_ops import ...`` (grm/core/paper_grm.py:15-20) to this engine.
    """
    sys.modules["grm.core.cuda_ops"] = sys.modules[__name__]


__all__ = [
    "cuda_apply_query",
    "cuda_batched_memory_gather",
    "cuda_chunk_update",
    "get_grm_cuda_runtime_status",
    "is_grm_cpp_extension_available",
    "is_grm_cuda_available",
    "load_grm_cuda_extension",
]
