"""In-tree build of the engine's native code for sm_100a.

Two artefacts land next to this file:

* ``libgrmx.so``      -- the CUDA kernels behind the C ABI of ``include/grmx.h``
                         (nvcc, ``-gencode arch=compute_100a,code=sm_100a``).
* ``grm_cuda_ext*.so`` -- the PyTorch shim that registers ``torch.ops.grm_cuda.*``
                         and links against ``libgrmx.so``.

Both builds are incremental on file modification times.  nvcc cross-compiles
without a GPU, so this runs on a CPU-only host.

    python -m rnn_with_grm_b200.build [--force] [--verbose]
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from pathlib import Path
from typing import Iterable, List

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
INCLUDE = ROOT / "include"
LIB_PATH = PKG_DIR / "libgrmx.so"
EXT_PATH = PKG_DIR / "grm_cuda_ext.so"

CUDA_SOURCES = [
    "cabi.cu",
    "chunk_scan.cu",
    "chunk_scan_ffma.cu",
    "tc_host.cu",
    "chunk_scan_tc_pipe.cu",
    "chunk_scan_tc_split.cu",
    "chunk_scan_tc_wide.cu",
    "chunk_scan_tc_square.cu",
    "apply_query.cu",
    "gather.cu",
    "topk_route.cu",
    "retrieve_fuse.cu",
    "retrieve_fuse_tc.cu",
    "select_fuse.cu",
    "archive_push.cu",
    "normalize_rows.cu",
    "project_normalize.cu",
]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _cuda_home() -> Path:
    for candidate in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if candidate and (Path(candidate) / "bin" / "nvcc").exists():
            return Path(candidate)
    raise RuntimeError("nvcc not found: set CUDA_HOME")


def _stale(target: Path, deps: Iterable[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: List[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed ({proc.returncode}): {' '.join(map(str, cmd))}\n{proc.stdout}")
    if verbose and proc.stdout:
        print(proc.stdout)


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu file into an object and link ``libgrmx.so``."""
    nvcc = _cuda_home() / "bin" / "nvcc"
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    obj_dir = PKG_DIR / "build"
    obj_dir.mkdir(exist_ok=True)
    objects = []
    for name in CUDA_SOURCES:
        src = CSRC / name
        obj = obj_dir / (src.stem + ".o")
        objects.append(obj)
        if force or _stale(obj, [src, *headers]):
            _run([str(nvcc), *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", "-c", str(src), "-o", str(obj)], verbose)
    if force or _stale(LIB_PATH, objects):
        _run([str(nvcc), "-shared", "-o", str(LIB_PATH), *map(str, objects)], verbose)
    return LIB_PATH


def build_torch_extension(force: bool = False, verbose: bool = False) -> Path:
    """Compile the torch shim against the installed PyTorch and link it to libgrmx."""
    import torch
    from torch.utils import cpp_extension

    src = CSRC / "torch_shim.cpp"
    if not (force or _stale(EXT_PATH, [src, INCLUDE / "grmx.h", LIB_PATH])):
        return EXT_PATH
    cxx = os.environ.get("CXX", "g++")
    includes = cpp_extension.include_paths() + [
        sysconfig.get_paths()["include"],
        str(_cuda_home() / "include"),
        str(INCLUDE),
    ]
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    cmd = [
        cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wno-attributes",
        "-DTORCH_EXTENSION_NAME=grm_cuda_ext", "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        *[f"-I{p}" for p in includes],
        str(src), "-o", str(EXT_PATH),
        f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
        f"-L{PKG_DIR}", "-lgrmx",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}",
    ]
    _run(cmd, verbose)
    return EXT_PATH


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_torch_extension(force=force, verbose=verbose)


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--force", action="store_true", help="rebuild even when up to date")
    parser.add_argument("--verbose", action="store_true", help="print the compiler commands")
    args = parser.parse_args(argv)
    build_all(force=args.force, verbose=args.verbose)
    print(f"built {LIB_PATH.name} and {EXT_PATH.name} in {PKG_DIR}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
