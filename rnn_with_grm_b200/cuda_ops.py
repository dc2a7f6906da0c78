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

_OP_NAMES = (
    "chunk_update_forward",
    "chunk_update_backward",
    "apply_query_forward",
    "apply_query_backward",
    "batched_memory_gather",
)
_SCAN_PATHS = {"auto": 0, "ffma": 1, "tcgen05": 2}
_POLICY_VALUES = ("auto", "native", "fallback")
# policy slot -> environment variables consulted, most specific first (reference :26-32)
_POLICY_ENV = {
    "global": ("GRM_CUDA_KERNEL_POLICY",),
    "chunk_update": ("GRM_CUDA_CHUNK_UPDATE_POLICY", "GRM_CUDA_KERNEL_POLICY"),
    "apply_query": ("GRM_CUDA_APPLY_QUERY_POLICY", "GRM_CUDA_KERNEL_POLICY"),
    "batched_memory_gather": ("GRM_CUDA_BATCHED_GATHER_POLICY", "GRM_CUDA_KERNEL_POLICY"),
}
_ERROR_BITS = {
    1: "an index outside the archive reached a gather or retrieval kernel (the row was zero-filled)",
    2: "a bounded wait inside a tensor-core kernel gave up (outputs of that call are incomplete)",
}


class _Extension:
    """The one import attempt of the compiled module, remembered for the process."""

    candidates = ("rnn_with_grm_b200.grm_cuda_ext", "grm_cuda_ext", "grm.grm_cuda_ext")
    module: Optional[Any] = None
    tried = False
    error = ""

    @classmethod
    def ops_registered(cls) -> Dict[str, bool]:
        namespace = getattr(torch.ops, "grm_cuda", None)
        return {name: namespace is not None and hasattr(namespace, name) for name in _OP_NAMES}

    @classmethod
    def load(cls, force: bool) -> bool:
        if not force and (cls.module is not None or cls.tried):
            return cls.module is not None
        cls.tried, cls.module, problems = True, None, []
        for name in cls.candidates:
            try:
                module = importlib.import_module(name)
            except Exception as exc:  # ImportError, OSError from the loader, ...
                problems.append(f"{name}: {type(exc).__name__}: {exc}")
                continue
            if all(cls.ops_registered().values()):
                cls.module = module
                break
            problems.append(f"{name}: torch.ops.grm_cuda registration missing")
        cls.error = "" if cls.module is not None else "; ".join(problems)
        if cls.module is not None:
            wanted = os.environ.get("GRMX_SCAN_PATH", "").strip().lower()
            if wanted in _SCAN_PATHS and hasattr(cls.module, "set_scan_path"):
                cls.module.set_scan_path(_SCAN_PATHS[wanted])
        return cls.module is not None


def _dispatch_table() -> Dict[str, Dict[str, bool]]:
    """Which dispatch keys hold a kernel for each op (reference :42-59)."""
    probe = getattr(torch._C, "_dispatch_has_kernel_for_dispatch_key", None)

    def has(op: str, key: str) -> bool:
        try:
            return probe is not None and bool(probe(f"grm_cuda::{op}", key))
        except Exception:
            return False

    return {op: {"cuda": has(op, "CUDA"), "composite_explicit_autograd": has(op, "CompositeExplicitAutograd")}
            for op in _OP_NAMES}


def _policy(slot: str) -> str:
    for variable in _POLICY_ENV[slot]:
        value = os.environ.get(variable, "").strip().lower()
        if value in _POLICY_VALUES:
            return value
    return "auto"


def load_grm_cuda_extension(force: bool = False) -> bool:
    """Import the compiled extension once per process (reference :62-89)."""
    return _Extension.load(force)


def is_grm_cpp_extension_available() -> bool:
    return _Extension.load(False)


def is_grm_cuda_available() -> bool:
    if not (_Extension.load(False) and torch.cuda.is_available()):
        return False
    return all(entry["cuda"] for entry in _dispatch_table().values())


def get_grm_cuda_runtime_status() -> Dict[str, Any]:
    """Field-for-field the dict of the reference (grm/core/cuda_ops.py:198-215)."""
    loaded = _Extension.load(False)
    module = _Extension.module
    dispatch = _dispatch_table()
    if not loaded:
        dispatch = {op: dict.fromkeys(entry, False) for op, entry in dispatch.items()}
    with_sources = bool(getattr(module, "__grm_cuda_with_kernels__", False))
    with_kernels = with_sources and all(entry["cuda"] for entry in dispatch.values())
    gpu = torch.cuda.is_available()
    return {
        "load_attempted": _Extension.tried,
        "extension_loaded": loaded,
        "compiled_with_cuda_sources": with_sources,
        "compiled_with_cuda_kernels": with_kernels,
        "torch_cuda_available": gpu,
        "cuda_backend_available": with_kernels and gpu,
        "load_error": _Extension.error,
        "module_name": getattr(module, "__name__", "") if module is not None else "",
        "registered_ops": _Extension.ops_registered(),
        "dispatch_kernels": dispatch,
        "kernel_policy": {slot: _policy(slot) for slot in _POLICY_ENV},
    }


def check_device_errors(reset: bool = True) -> None:
    """Raise ``RuntimeError`` if a kernel of this engine reported a failure it could not raise itself.

    Kernels never trap: a bounded wait that gives up, or a routing index outside the archive, sets a
    bit in a per-device error word and the launch still returns success, so the outputs of that call
    may be incomplete.  This reads the word of the current device (which waits for the current stream)
    and raises if it is non-zero.  Call it wherever a synchronisation is acceptable -- after a forward
    pass, before a checkpoint -- or set ``GRMX_CHECK_ERRORS=1`` to have every op of this module and the
    segment runners check after each call (a debugging mode: it serialises host and device).
    """
    _require_extension("check_device_errors")
    word = int(_Extension.module.device_error_word())
    if word == 0:
        return
    if reset:
        _Extension.module.device_error_reset()
    reasons = [text for bit, text in _ERROR_BITS.items() if word & bit] or [f"unknown bits {word:#x}"]
    raise RuntimeError(f"grm_cuda: device error word {word:#x}: " + "; ".join(reasons))


def _checking_each_call() -> bool:
    return os.environ.get("GRMX_CHECK_ERRORS", "").strip().lower() in ("1", "true", "on", "yes")


def set_scan_path(path: str) -> None:
    """Pin the chunk-scan kernel family: ``auto``, ``ffma`` (exact fp32) or ``tcgen05``."""
    if path not in _SCAN_PATHS:
        raise ValueError(f"scan path must be one of {sorted(_SCAN_PATHS)}, got {path!r}")
    _require_extension("set_scan_path")
    _Extension.module.set_scan_path(_SCAN_PATHS[path])


def _require_extension(op_name: str) -> None:
    if not _Extension.load(False):
        raise RuntimeError(
            f"{op_name}: the grm_cuda extension is not loaded ({_Extension.error or 'not built'}). "
            "Build it with `python -m rnn_with_grm_b200.build`; this engine has no fallback path."
        )


def _require_native(op_name: str, policy_key: str, device: torch.device, *, enabled: bool, debug_fallback: bool) -> None:
    if not enabled or debug_fallback or _policy(policy_key) == "fallback":
        raise RuntimeError(
            f"{op_name}: a fallback path was requested (enabled={enabled}, debug_fallback={debug_fallback}, "
            f"policy={_policy(policy_key)!r}) but this engine ships only the sm_100a kernels."
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
    out = ChunkUpdateCudaFn.apply(keys, values, queries, memory, float(memory_decay))
    if _checking_each_call():
        check_device_errors()
    return out


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
    out = ApplyQueryCudaFn.apply(memories, queries)
    if _checking_each_call():
        check_device_errors()
    return out


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
    out = torch.ops.grm_cuda.batched_memory_gather(memories_per_batch, topk_indices)
    if _checking_each_call():
        check_device_errors()
    return out


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
