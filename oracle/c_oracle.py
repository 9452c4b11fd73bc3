"""ctypes access to the checker libraries.  TEST INFRASTRUCTURE ONLY.

  libsage_oracle.so      this repo's plain-C restatement (oracle/sage_oracle.c)
  _ref/libsage_ref.so    the reference project's own SAGE CUDA kernels, compiled
                         from the reference checkout by `make -C oracle ref`
                         (present only where that checkout existed at build time)

Nothing under sage_b200/ imports this module.
"""

from __future__ import annotations

import ctypes
import pathlib
import subprocess

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent
ORACLE_LIB = HERE / "libsage_oracle.so"
REF_LIB = HERE / "_ref" / "libsage_ref.so"

_u16p = ctypes.POINTER(ctypes.c_uint16)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)


def build(reference: str | None = None) -> None:
    """Compile the C oracle; with `reference` given and present, also the comparator."""
    subprocess.run(["make", "-C", str(HERE)], check=True, capture_output=True)
    if reference and pathlib.Path(reference, "csrc/sage/sage_gemv_cuda.cu").exists():
        subprocess.run(
            ["make", "-C", str(HERE), "ref", f"REFERENCE={reference}"],
            check=True,
            capture_output=True,
        )


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not ORACLE_LIB.exists():
            build()
        handle = ctypes.CDLL(str(ORACLE_LIB))
        handle.sage_oracle_decode_fp16.restype = ctypes.c_int
        handle.sage_oracle_decode_fp16.argtypes = [
            _u32p, _u32p, _u16p, _u16p, _i32p, ctypes.c_int, ctypes.c_int, ctypes.c_int, _u16p,
        ]
        handle.sage_oracle_linear.restype = ctypes.c_int
        handle.sage_oracle_linear.argtypes = [
            _u16p, _u32p, _u32p, _u16p, _u16p, _i32p, _f32p,
            ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        ]
        handle.sage_oracle_max_threads.restype = ctypes.c_int
        _lib = handle
    return _lib


def _np(value, dtype) -> np.ndarray:
    if hasattr(value, "detach"):
        value = value.detach().cpu().numpy()
    return np.ascontiguousarray(value).view(dtype)


def _buffers(packed):
    codes = _np(packed["packed_codes"], np.uint32)
    radii = _np(packed["radius_codes"], np.uint32)
    grid = _np(packed["radius_grid"], np.uint16)
    book = _np(packed["codebook"], np.uint16)
    perm = _np(packed["permutation"], np.int32)
    k = codes.shape[1] * 128
    entries = book.shape[1]
    perm_ptr = perm.ctypes.data_as(_i32p) if perm.size else None
    keep = (codes, radii, grid, book, perm)
    args = (
        codes.ctypes.data_as(_u32p),
        radii.ctypes.data_as(_u32p),
        grid.ctypes.data_as(_u16p),
        book.ctypes.data_as(_u16p),
        perm_ptr,
    )
    return keep, args, k, entries


def decode_fp16(packed, n: int, *, apply_permutation: bool = True) -> np.ndarray:
    """FP16 dequantised weight [n, K] from the C oracle."""
    keep, args, k, entries = _buffers(packed)
    if not apply_permutation:
        args = args[:4] + (None,)
    out = np.empty((n, k), dtype=np.uint16)
    status = lib().sage_oracle_decode_fp16(*args, n, k, entries, out.ctypes.data_as(_u16p))
    if status:
        raise RuntimeError(f"sage_oracle_decode_fp16 failed with status {status}")
    return out.view(np.float16)


def linear_fp32(x, packed, n: int, *, threads: int = 0) -> np.ndarray:
    """FP32 `x.float() @ W16.float().T` from the C oracle; x is FP16 [..., K]."""
    keep, args, k, entries = _buffers(packed)
    xb = _np(x, np.uint16)
    rows = xb.size // k
    y = np.empty((rows, n), dtype=np.float32)
    status = lib().sage_oracle_linear(
        xb.ctypes.data_as(_u16p), *args, y.ctypes.data_as(_f32p), rows, n, k, entries, threads
    )
    if status:
        raise RuntimeError(f"sage_oracle_linear failed with status {status}")
    return y.reshape(*xb.shape[:-1], n)


def max_threads() -> int:
    return int(lib().sage_oracle_max_threads())


def reference_kernels():
    """The reference project's compiled CUDA launchers, or None when not built."""
    if not REF_LIB.exists():
        return None
    handle = ctypes.CDLL(str(REF_LIB))
    vp, ci = ctypes.c_void_p, ctypes.c_int
    handle.sage_ref_fuses_permutation.restype = ci
    handle.sage_ref_fuses_permutation.argtypes = [ci, ci]
    handle.sage_ref_gemm_splits.restype = ci
    handle.sage_ref_gemm_splits.argtypes = [ci, ci, ci, ci]
    handle.sage_ref_gemv.restype = ci
    handle.sage_ref_gemv.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]
    handle.sage_ref_gemm.restype = ci
    handle.sage_ref_gemm.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]
    return handle
