"""Torch operator for the SAGE packed linear, backed by libsage_b200.so.

Mirrors the reference's dispatcher registration (weight_vq/inference/ops.py:42-61):
`sage(x, packed_codes, radius_codes, radius_grid, codebook, permutation, out_features)`
is a `torch.library.custom_op` with `mutates_args=()`, CUDA only, plus a fake kernel that
returns `x.new_empty((*x.shape[:-1], out_features))`.  The op is registered as
`wvq::sage`, the reference's name, unless that name is already taken in this process
(the reference package was imported first), in which case it is `sage_b200::sage`.

Argument checks and their messages follow the reference's native entry point
(csrc/bindings.cpp:13-48).
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib

_COUNTER_REGION_BYTES = 64 * 1024  # the front of the scratch the kernels expect (and leave) zero
_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}
_RETIRED: list[torch.Tensor] = []  # outgrown buffers a captured graph may still point at


def _workspace(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    """Zero-filled scratch, one per (device, stream); the kernels restore the zeros."""
    key = (device.index, stream)
    buffer = _WORKSPACES.get(key)
    if buffer is None or buffer.numel() < nbytes:
        if buffer is not None:
            _RETIRED.append(buffer)
        buffer = torch.zeros(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = buffer
    return buffer


def _check_layout(x, codes, radii, grid, book, permutation, out_features):
    if not (x.is_cuda and x.dtype == torch.float16 and x.is_contiguous() and x.dim() >= 1):
        raise RuntimeError("SAGE requires contiguous CUDA FP16 input")
    for tensor in (codes, radii, grid, book, permutation):
        if tensor.device != x.device or not tensor.is_contiguous():
            raise RuntimeError("SAGE buffers must be contiguous and on the input device")
    k = x.shape[-1]
    tiles = (out_features + 15) // 16
    if not (k > 0 and k % 128 == 0 and out_features > 0):
        raise RuntimeError("SAGE requires positive N and K divisible by 128")
    if not (book.dim() == 3 and book.shape[0] == 4 and book.shape[2] == 2 and book.shape[1] in (64, 128, 256)):
        raise RuntimeError("SAGE codebook must have shape [4, 64/128/256, 2]")
    groups = k // 128
    if not (
        codes.dtype == torch.int32
        and tuple(codes.shape) == (tiles, groups, 16, 8)
        and radii.dtype == torch.int32
        and tuple(radii.shape) == (tiles, groups, 16)
        and grid.dtype == torch.float16
        and tuple(grid.shape) == (tiles, groups, 16, 2)
        and book.dtype == torch.float16
        and permutation.dtype == torch.int32
        and permutation.dim() == 1
        and permutation.numel() in (0, k)
    ):
        raise RuntimeError("Invalid SAGE packed layout")
    if (grid.data_ptr() & 3) or (book.data_ptr() & 3):
        raise RuntimeError("SAGE grid and codebook require 4-byte aligned storage")
    return k


def sage_forward(
    x: torch.Tensor,
    packed_codes: torch.Tensor,
    radius_codes: torch.Tensor,
    radius_grid: torch.Tensor,
    codebook: torch.Tensor,
    permutation: torch.Tensor,
    out_features: int,
) -> torch.Tensor:
    """The native entry point's Python twin (reference csrc/bindings.cpp:8-79)."""
    return _forward(x, packed_codes, radius_codes, radius_grid, codebook, permutation, out_features, None)


def sage_forward_scratch(
    x: torch.Tensor,
    packed_codes: torch.Tensor,
    radius_codes: torch.Tensor,
    radius_grid: torch.Tensor,
    codebook: torch.Tensor,
    permutation: torch.Tensor,
    out_features: int,
    scratch: torch.Tensor,
) -> torch.Tensor:
    """`sage_forward` with scratch memory the caller owns: a zero-filled uint8 tensor on x's device of
    at least `sageb200_workspace_bytes(rows, out_features, K)` bytes, 256-byte aligned, used by one
    stream at a time (the kernels leave its arrival counters at zero).  A caller that runs many
    linears on a stream of its own - a decode step being captured in a CUDA graph - thereby avoids
    the temporary and its fill kernel that `sage_forward` takes on any stream but the default one."""
    return _forward(x, packed_codes, radius_codes, radius_grid, codebook, permutation, out_features, scratch)


def _forward(x, packed_codes, radius_codes, radius_grid, codebook, permutation, out_features, scratch):
    k = _check_layout(x, packed_codes, radius_codes, radius_grid, codebook, permutation, out_features)
    output = torch.empty((*x.shape[:-1], out_features), dtype=x.dtype, device=x.device)
    rows = x.numel() // k
    if rows == 0:
        return output
    if rows > 65535:
        raise RuntimeError("SAGE launch dimensions exceed supported range")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        nbytes = lib.sageb200_workspace_bytes(rows, out_features, k)
        workspace = None
        if nbytes and scratch is not None:
            if scratch.device != x.device or scratch.dtype != torch.uint8 or scratch.numel() < nbytes:
                raise RuntimeError(f"SAGE scratch must be a uint8 tensor of at least {nbytes} bytes on the input device")
            workspace = scratch
        elif nbytes and stream == 0:
            workspace = _workspace(x.device, stream, nbytes)  # the default stream's cached scratch
        elif nbytes:
            # Any other stream may be one that is being captured, or the private stream of a
            # compiled graph whose memory pool accepts no allocation that outlives the call: take
            # the scratch as a temporary of this call, as the reference's entry point does
            # (csrc/bindings.cpp:63-66), and zero the arrival counters at its front.
            workspace = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
            workspace[: min(nbytes, _COUNTER_REGION_BYTES)].zero_()
        _lib.check(
            lib.sageb200_linear(
                x.data_ptr(),
                packed_codes.data_ptr(),
                radius_codes.data_ptr(),
                radius_grid.data_ptr(),
                codebook.data_ptr(),
                permutation.data_ptr() if permutation.numel() else None,
                output.data_ptr(),
                workspace.data_ptr() if workspace is not None else None,
                workspace.numel() if workspace is not None else 0,
                rows,
                out_features,
                k,
                codebook.shape[1],
                stream,
            )
        )
    return output


def _fake(x, packed_codes, radius_codes, radius_grid, codebook, permutation, out_features):
    return x.new_empty((*x.shape[:-1], out_features))


def _register(namespace: str):
    op = torch.library.custom_op(f"{namespace}::sage", mutates_args=(), device_types="cuda")(
        sage_forward
    )
    op.register_fake(_fake)
    return op


try:
    sage = _register("wvq")
except RuntimeError:  # the reference package already owns wvq::sage in this process
    sage = _register("sage_b200")


def sage_dequantize(
    packed_codes: torch.Tensor,
    radius_codes: torch.Tensor,
    radius_grid: torch.Tensor,
    codebook: torch.Tensor,
    permutation: torch.Tensor,
    out_features: int,
    *,
    original_order: bool = True,
) -> torch.Tensor:
    """Dense FP16 weight [out_features, K], bit-exact with the reference's dequantisation."""
    k = packed_codes.shape[1] * 128
    dummy = torch.empty((0, k), dtype=torch.float16, device=packed_codes.device)
    _check_layout(dummy, packed_codes, radius_codes, radius_grid, codebook, permutation, out_features)
    weight = torch.empty((out_features, k), dtype=torch.float16, device=packed_codes.device)
    lib = _lib.load()
    with torch.cuda.device(weight.device):
        stream = torch.cuda.current_stream(weight.device).cuda_stream
        use_perm = original_order and permutation.numel() > 0
        _lib.check(
            lib.sageb200_dequant(
                packed_codes.data_ptr(),
                radius_codes.data_ptr(),
                radius_grid.data_ptr(),
                codebook.data_ptr(),
                permutation.data_ptr() if use_perm else None,
                weight.data_ptr(),
                out_features,
                k,
                codebook.shape[1],
                stream,
            )
        )
    return weight


def sage_grouped(problems: list[tuple], out_features: list[int], activation: tuple | None = None,
                 outputs: list[torch.Tensor] | None = None) -> list[torch.Tensor]:
    """Several packed linears (rows <= 16 each) in one launch.

    `outputs` (optional): contiguous FP16 tensors to write into, one per problem, instead of fresh
    ones - e.g. row ranges of one tensor when the problems are row blocks of the same linear.

    `problems[i]` = (x, packed_codes, radius_codes, radius_grid, codebook, permutation).
    `activation` = (kind, eps, a, b, weight, residual_out) fuses the producer of the shared
    input into the launch (kind 1: residual add + RMSNorm, kind 2: SwiGLU; see
    `sageb200_activation` in include/sage_b200.h); `x` then only supplies shape and dtype.
    """
    if len(problems) > _lib.MAX_GROUPED:
        raise RuntimeError("too many problems for one grouped launch")
    lib = _lib.load()
    array = (_lib.Problem * len(problems))()
    given, outputs = outputs, []
    device = problems[0][0].device
    for i, ((x, codes, radii, grid, book, perm), n) in enumerate(zip(problems, out_features)):
        k = _check_layout(x, codes, radii, grid, book, perm, n)
        rows = x.numel() // k
        if given is None:
            y = torch.empty((*x.shape[:-1], n), dtype=x.dtype, device=x.device)
        else:
            y = given[i]
            if not (y.is_contiguous() and y.dtype == x.dtype and y.device == x.device and y.numel() == rows * n):
                raise RuntimeError("SAGE grouped outputs must be contiguous FP16 tensors of rows x out_features")
        outputs.append(y)
        array[i] = _lib.Problem(
            x.data_ptr(), codes.data_ptr(), radii.data_ptr(), grid.data_ptr(), book.data_ptr(),
            perm.data_ptr() if perm.numel() else None, y.data_ptr(), rows, n, k, book.shape[1],
        )
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        if activation is None:
            total = lib.sageb200_grouped_workspace_bytes(array, len(problems))
            workspace = _workspace(device, stream, total) if total else None
            _lib.check(
                lib.sageb200_linear_grouped(
                    array,
                    len(problems),
                    workspace.data_ptr() if workspace is not None else None,
                    workspace.numel() if workspace is not None else 0,
                    stream,
                )
            )
        else:
            kind, eps, a, b, weight, residual_out = activation
            pointer = lambda t: t.data_ptr() if t is not None else None  # noqa: E731
            act = _lib.Activation(kind, eps, pointer(a), pointer(b), pointer(weight), pointer(residual_out))
            total = lib.sageb200_fused_workspace_bytes(array, len(problems))
            workspace = _workspace(device, stream, total) if total else None
            _lib.check(
                lib.sageb200_linear_grouped_fused(
                    array,
                    len(problems),
                    ctypes.byref(act),
                    workspace.data_ptr() if workspace is not None else None,
                    workspace.numel() if workspace is not None else 0,
                    stream,
                )
            )
    return outputs
