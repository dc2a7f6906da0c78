"""Builds the checkers under ``oracle/`` -- TEST INFRASTRUCTURE ONLY.

* ``oracle/_build/libgrm_oracle.so`` -- gcc build of ``oracle/grm_oracle.c``.
* ``oracle/_ref/grm_ref_ops.so``     -- the reference's own CPU implementation
  (``grm/csrc/grm_cuda.cpp``, compiled from the reference checkout where it
  lies) plus ``oracle/ref_binding.cpp``.
* ``oracle/_ref/python/grm/``        -- the reference's Python package staged as it is
  (its ``*.py`` files only), so that the machine that runs the GPU tests and the
  benchmark -- which has no reference checkout -- can import the reference's models
  and time the reference's default CPU path.

Both ``_ref`` outputs exist only when a reference checkout is present at build time;
the folder is ignored by git (nothing of the reference enters the history) and travels
with the working tree.  The checkout is found through ``--reference``, the
``GRM_REFERENCE_ROOT`` environment variable, or a ``reference`` folder beside this
repository.

    python oracle/build_oracle.py [--reference /path/to/RNN_with_GRM] [--force]
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
C_SRC = HERE / "grm_oracle.c"
C_LIB = HERE / "_build" / "libgrm_oracle.so"
REF_LIB = HERE / "_ref" / "grm_ref_ops.so"
REF_PYTHON = HERE / "_ref" / "python"


def default_reference() -> Path:
    """Where the reference checkout is looked for when none is named."""
    env = os.environ.get("GRM_REFERENCE_ROOT", "").strip()
    return Path(env) if env else HERE.parent.parent / "reference"


def _stale(target: Path, deps) -> bool:
    return not target.exists() or any(Path(d).stat().st_mtime > target.stat().st_mtime for d in deps)


def build_c_oracle(force: bool = False) -> Path:
    if force or _stale(C_LIB, [C_SRC]):
        C_LIB.parent.mkdir(exist_ok=True)
        cmd = ["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-mfma",
               str(C_SRC), "-o", str(C_LIB), "-lm"]
        subprocess.run(cmd, check=True)
    return C_LIB


def stage_reference_python(reference: Path = None, force: bool = False):
    """Copies the reference's ``grm`` package (``*.py`` only) to ``oracle/_ref/python/grm``.

    Returns the folder to put on ``sys.path``, or None when there is neither a checkout nor an
    earlier staging."""
    reference = default_reference() if reference is None else reference
    package = reference / "grm"
    target = REF_PYTHON / "grm"
    if not (package / "__init__.py").exists():
        return REF_PYTHON if (target / "__init__.py").exists() else None
    sources = sorted(package.rglob("*.py"))
    marker = target / "__init__.py"
    if force or _stale(marker, sources) or len(list(target.rglob("*.py"))) != len(sources):
        if target.exists():
            shutil.rmtree(target)
        for src in sources:
            dst = target / src.relative_to(package)
            dst.parent.mkdir(parents=True, exist_ok=True)
            shutil.copyfile(src, dst)
        os.utime(marker)
    return REF_PYTHON


def build_reference_cpu(reference: Path = None, force: bool = False):
    """Returns the library path, or None when no reference checkout is available."""
    reference = default_reference() if reference is None else reference
    src = reference / "grm" / "csrc" / "grm_cuda.cpp"
    if not src.exists():
        return REF_LIB if REF_LIB.exists() else None
    binding = HERE / "ref_binding.cpp"
    if not (force or _stale(REF_LIB, [src, binding])):
        return REF_LIB
    import torch
    from torch.utils import cpp_extension

    REF_LIB.parent.mkdir(exist_ok=True)
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    includes = cpp_extension.include_paths() + [sysconfig.get_paths()["include"], str(src.parent)]
    cmd = [
        os.environ.get("CXX", "g++"), "-O3", "-std=c++17", "-fPIC", "-shared", "-Wno-attributes",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        *[f"-I{p}" for p in includes],
        str(src), str(binding), "-o", str(REF_LIB),
        f"-L{torch_lib}", "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python",
        f"-Wl,-rpath,{torch_lib}",
    ]
    subprocess.run(cmd, check=True)
    return REF_LIB


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--reference", type=Path, default=None,
                        help="reference checkout (default: $GRM_REFERENCE_ROOT, else ../reference)")
    parser.add_argument("--force", action="store_true")
    args = parser.parse_args(argv)
    print("c oracle:", build_c_oracle(force=args.force))
    print("reference cpu library:", build_reference_cpu(args.reference, force=args.force))
    print("reference python package:", stage_reference_python(args.reference, force=args.force))
    return 0


if __name__ == "__main__":
    sys.exit(main())
