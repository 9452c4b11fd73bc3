"""SPHQuant 64/4 packed linear: operator and module with the reference's names.

Mirrors the reference's `wvq::sphquant` op and fake (weight_vq/inference/ops.py:21-39), its
native entry point's checks and messages (csrc/sphquant/sph_gemv_cuda.cu:403-446) and
`SPHQuantLinear` (weight_vq/inference/linear.py:252-271: buffers `packed_codes`,
`radius_extra`, `radius_scales`, `radius_mins`, `codebook`, `bias`; out_features and
in_features derived from the code tensor).  The op is registered as `wvq::sphquant` unless the
reference package already owns that name in this process, then as `sage_b200::sphquant`.
"""

from __future__ import annotations

import torch
from torch import nn

from . import _lib


def sph_gemv_forward(
    x: torch.Tensor,
    packed_codes: torch.Tensor,
    radius_extra: torch.Tensor,
    radius_scales: torch.Tensor,
    radius_mins: torch.Tensor,
    codebook: torch.Tensor,
    group_size: int = 128,
) -> torch.Tensor:
    """Python twin of the reference's `sph_gemv_forward_cuda`."""
    tensors = (x, packed_codes, radius_extra, radius_scales, radius_mins, codebook)
    if not all(t.is_cuda for t in tensors):
        raise RuntimeError("sph_gemv expects CUDA tensors")
    if not all(t.dtype == torch.float16 for t in (x, radius_scales, radius_mins, codebook)):
        raise RuntimeError("sph_gemv currently supports FP16 tensors only")
    if packed_codes.dtype != torch.int16 or radius_extra.dtype != torch.int32:
        raise RuntimeError("invalid SPH packed tensor dtypes")
    if not all(t.is_contiguous() for t in tensors):
        raise RuntimeError("sph_gemv expects contiguous tensors")
    if group_size != 128:
        raise RuntimeError("sph_gemv currently requires group_size=128")
    k = x.shape[-1]
    n = packed_codes.shape[0]
    groups = k // 128
    if k % 128 or groups > 128 or k == 0:
        raise RuntimeError("invalid SPH input dimension")
    if packed_codes.dim() != 2 or packed_codes.shape[1] != k // 8:
        raise RuntimeError("invalid SPH packed code shape")
    if not all(tuple(t.shape) == (n, groups) for t in (radius_extra, radius_scales, radius_mins)):
        raise RuntimeError("invalid SPH radius metadata shape")
    if tuple(codebook.shape) != (64, 8):
        raise RuntimeError("SPH codebook must have shape [64, 8]")
    output = torch.empty((*x.shape[:-1], n), dtype=x.dtype, device=x.device)
    rows = x.numel() // k
    if rows == 0 or n == 0:
        return output
    lib = _lib.load()
    with torch.cuda.device(x.device):
        _lib.check(lib.sageb200_sph_linear(
            x.data_ptr(), packed_codes.data_ptr(), radius_extra.data_ptr(), radius_scales.data_ptr(),
            radius_mins.data_ptr(), codebook.data_ptr(), output.data_ptr(), rows, n, k,
            torch.cuda.current_stream(x.device).cuda_stream))
    return output


def _op(x: torch.Tensor, packed_codes: torch.Tensor, radius_extra: torch.Tensor, radius_scales: torch.Tensor,
        radius_mins: torch.Tensor, codebook: torch.Tensor) -> torch.Tensor:
    return sph_gemv_forward(x, packed_codes, radius_extra, radius_scales, radius_mins, codebook, 128)


def _fake(x, packed_codes, radius_extra, radius_scales, radius_mins, codebook):
    return x.new_empty((*x.shape[:-1], packed_codes.shape[0]))


def _register(namespace: str):
    op = torch.library.custom_op(f"{namespace}::sphquant", mutates_args=(), device_types="cuda")(_op)
    op.register_fake(_fake)
    return op


try:
    sphquant = _register("wvq")
except RuntimeError:  # the reference package already owns wvq::sphquant in this process
    sphquant = _register("sage_b200")


def sph_dequantize(packed_codes, radius_extra, radius_scales, radius_mins, codebook) -> torch.Tensor:
    """Dense FP16 weight [N, K] = fp16(the reference decode's FP32 weight), bit for bit."""
    n, k = packed_codes.shape[0], packed_codes.shape[1] * 8
    weight = torch.empty((n, k), dtype=torch.float16, device=packed_codes.device)
    lib = _lib.load()
    with torch.cuda.device(weight.device):
        _lib.check(lib.sageb200_sph_dequant(
            packed_codes.data_ptr(), radius_extra.data_ptr(), radius_scales.data_ptr(), radius_mins.data_ptr(),
            codebook.data_ptr(), weight.data_ptr(), n, k, torch.cuda.current_stream(weight.device).cuda_stream))
    return weight


class SPHQuantLinear(nn.Module):
    """SPHQuant 64/4 packed linear (row-major codes, no permutation)."""

    def __init__(self, packed: dict[str, torch.Tensor], bias: torch.Tensor | None = None):
        super().__init__()
        self.out_features = packed["packed_codes"].shape[0]
        self.in_features = packed["packed_codes"].shape[1] * 8
        for name in ("packed_codes", "radius_extra", "radius_scales", "radius_mins", "codebook"):
            self.register_buffer(name, packed[name])
        self.register_buffer("bias", bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        output = sphquant(x.to(torch.float16).contiguous(), self.packed_codes, self.radius_extra,
                          self.radius_scales, self.radius_mins, self.codebook).to(x.dtype)
        return output if self.bias is None else output + self.bias

    def dequantize(self) -> torch.Tensor:
        return sph_dequantize(self.packed_codes, self.radius_extra, self.radius_scales, self.radius_mins,
                              self.codebook)
