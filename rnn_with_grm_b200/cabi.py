"""ctypes binding of ``libgrmx.so`` -- the C ABI declared in ``include/grmx.h``.

This is the binding a non-PyTorch host would write: plain pointers, sizes and a
stream handle.  The helpers at the bottom accept torch CUDA tensors only to
fetch ``data_ptr()`` and the current stream; no torch type crosses the ABI.
Nothing here computes: if the library is missing, loading raises.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_void_p
from pathlib import Path
from typing import Optional

LIB_PATH = Path(__file__).resolve().parent / "libgrmx.so"

F32, BF16, F16 = 0, 1, 2
PATH_AUTO, PATH_FFMA, PATH_TCGEN05 = 0, 1, 2
FUSE_RETRIEVED, FUSE_CONTRIB, FUSE_RESIDUAL_LN = 0, 1, 2


class DeviceInfo(ctypes.Structure):
    _fields_ = [
        ("device", c_int32),
        ("cc_major", c_int32),
        ("cc_minor", c_int32),
        ("sm_count", c_int32),
        ("max_smem_per_block", c_int32),
        ("has_tcgen05", c_int32),
        ("total_mem", c_int64),
    ]


# name -> (restype, argtypes); one entry per declaration in include/grmx.h
SIGNATURES = {
    "grmx_version": (c_int, []),
    "grmx_last_error": (c_char_p, []),
    "grmx_query_device": (c_int, [c_int, POINTER(DeviceInfo)]),
    "grmx_launch_count": (c_int64, []),
    "grmx_chunk_scan_fwd": (
        c_int,
        [c_void_p] * 6 + [c_int64] * 4 + [c_float, c_int, c_int, c_int, c_void_p],
    ),
    "grmx_chunk_scan_scratch_bytes": (c_int64, [c_int64] * 4 + [c_int, c_int]),
    "grmx_chunk_scan_fwd_ws": (
        c_int,
        [c_void_p] * 6 + [c_int64] * 4 + [c_float, c_int, c_int, c_int, c_void_p, c_int64, c_void_p],
    ),
    "grmx_static_scratch_capacity": (c_int64, []),
    "grmx_chunk_scan_scratch_bytes_on": (c_int64, [c_int64] * 4 + [c_int]),
    "grmx_static_scratch_admits": (c_int, [c_int64]),
    "grmx_chunk_scan_fwd_static": (c_int, [c_void_p] * 6 + [c_int64] * 4 + [c_float, c_void_p]),
    "grmx_chunk_scan_bwd": (
        c_int,
        [c_void_p] * 10 + [c_int64] * 4 + [c_float, c_int, c_int, c_int, c_void_p],
    ),
    "grmx_linear_scan": (
        c_int,
        [c_void_p] * 4 + [c_int64, c_int64, c_void_p, c_void_p] + [c_int64] * 4 + [c_float] * 4
        + [c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "grmx_apply_query_fwd": (c_int, [c_void_p] * 3 + [c_int64] * 4 + [c_int, c_void_p]),
    "grmx_apply_query_bwd": (c_int, [c_void_p] * 5 + [c_int64] * 4 + [c_int, c_void_p]),
    "grmx_batched_gather": (c_int, [c_void_p] * 3 + [c_int64] * 4 + [c_int, c_void_p]),
    "grmx_topk_route": (
        c_int,
        [c_void_p] * 3 + [c_int64] * 4 + [c_int, c_float, c_float] + [c_void_p] * 3 + [c_void_p],
    ),
    "grmx_topk_route_bf16q": (
        c_int,
        [c_void_p] * 3 + [c_int64] * 4 + [c_int, c_float, c_float] + [c_void_p] * 3 + [c_void_p],
    ),
    "grmx_topk_select": (
        c_int,
        [c_void_p, c_void_p] + [c_int64] * 3 + [c_int, c_float] + [c_void_p] * 2 + [c_void_p],
    ),
    "grmx_retrieve_fuse": (
        c_int,
        [c_void_p] * 7 + [c_float, c_void_p] + [c_int64] * 6 + [c_int, c_void_p],
    ),
    "grmx_retrieve_fuse_rows": (
        c_int,
        [c_void_p] * 7 + [c_float, c_void_p] + [c_int64] * 6 + [c_int, c_void_p],
    ),
    "grmx_retrieve_fuse_tc": (
        c_int,
        [c_void_p] * 7 + [c_float, c_void_p] + [c_int64] * 6 + [c_int, c_void_p],
    ),
    "grmx_add_layer_norm": (
        c_int,
        [c_void_p] * 4 + [c_float, c_void_p, c_int64, c_int64, c_int, c_void_p],
    ),
    "grmx_select_fuse": (
        c_int,
        [c_void_p] * 6 + [c_float, c_void_p] + [c_int64] * 5 + [c_int, c_int, c_void_p],
    ),
    "grmx_chunk_scan_fwd_segments": (
        c_int,
        [c_void_p] * 7 + [c_int64] * 7 + [c_float, c_int, c_int, c_void_p],
    ),
    "grmx_normalize_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_float, c_int, c_int, c_void_p]),
    "grmx_project_normalize": (c_int, [c_void_p] * 5 + [c_int64] * 3 + [c_float, c_void_p]),
    "grmx_archive_push": (c_int, [c_void_p] * 3 + [c_int64] * 4 + [c_void_p]),
    "grmx_device_error_word": (c_int, [POINTER(c_uint32), c_void_p]),
    "grmx_device_error_reset": (c_int, [c_void_p]),
    "grmx_selftest_bounded_wait": (c_int, [c_uint32, c_void_p]),
}

_LIB: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Load ``libgrmx.so`` from the package directory and type every entry point."""
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m rnn_with_grm_b200.build`")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _LIB = lib
    return _LIB


class GrmxError(RuntimeError):
    pass


def check(rc: int) -> None:
    if rc != 0:
        raise GrmxError(f"grmx error {rc}: {load().grmx_last_error().decode()}")


def dtype_code(torch_dtype) -> int:
    import torch

    codes = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
    if torch_dtype not in codes:
        raise TypeError(f"unsupported dtype {torch_dtype}")
    return codes[torch_dtype]


def ptr(tensor) -> Optional[int]:
    """Device address of a contiguous CUDA tensor (None stays NULL)."""
    if tensor is None:
        return None
    if not tensor.is_cuda or not tensor.is_contiguous():
        raise ValueError("the C ABI takes contiguous CUDA tensors")
    return tensor.data_ptr()


def current_stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def device_error_word() -> int:
    out = c_uint32(0)
    check(load().grmx_device_error_word(ctypes.byref(out), current_stream()))
    return int(out.value)
