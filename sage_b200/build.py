"""Builds libsage_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m sage_b200.build [--force] [--verbose]

No fast-math: the dense dequantisation must round exactly like the reference
(its `_C` target is also built without fast-math, CMakeLists.txt:36-41,52-53 there).
"""

from __future__ import annotations

import argparse
import os
import pathlib
import shutil
import subprocess
import sys

PACKAGE = pathlib.Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libsage_b200.so"
TRACE_LIBRARY = PACKAGE / "libsage_b200_trace.so"
INCLUDE = PACKAGE.parent / "include"

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-shared",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
]


def sources() -> list[pathlib.Path]:
    return sorted(CSRC.glob("*.cu"))


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and pathlib.Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; libsage_b200.so cannot be built")


def is_stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    inputs = list(CSRC.glob("*")) + list(INCLUDE.glob("*.h")) + [pathlib.Path(__file__)]
    return any(path.stat().st_mtime > built for path in inputs)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> pathlib.Path:
    """Compile every .cu under csrc/ into one shared library; returns its path.  `trace` adds
    -DSAGEB200_TRACE: the decode kernel's phase clocks (sageb200_debug_trace) and the
    SAGEB200_PATHS switch, both compiled out of the default build."""
    if not force and not trace and not is_stale():
        return LIBRARY
    flags = NVCC_FLAGS + (["-DSAGEB200_TRACE"] if trace else [])
    # the profiling build goes beside the product library (select it with SAGEB200_LIBRARY)
    target = TRACE_LIBRARY if trace else LIBRARY
    command = [_nvcc(), *flags, f"-I{INCLUDE}", "-o", str(target), *map(str, sources())]
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose or result.returncode:
        sys.stderr.write(" ".join(command) + "\n" + result.stdout + result.stderr)
    if result.returncode:
        raise RuntimeError("nvcc failed building libsage_b200.so")
    if not trace:
        (PACKAGE / "build_log.txt").write_text(result.stdout + result.stderr)
    return target


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    parser.add_argument("--trace", action="store_true", help="profiling build (-DSAGEB200_TRACE)")
    args = parser.parse_args()
    print(build(force=args.force, verbose=args.verbose, trace=args.trace))
