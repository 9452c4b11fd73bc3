"""Packed SAGE linear module with the reference's constructor and buffer names.

Mirrors `SAGELinear` (weight_vq/inference/linear.py:274-309 in the reference): buffers
`packed_codes`, `radius_codes`, `radius_grid`, `codebook`, `permutation`, `bias` are
registered under those names, so a reference state_dict loads with no missing or
unexpected keys; `out_features` excludes tile padding; `in_features` comes from the code
tensor's group count.  Unlike the reference, the input-channel gather is never hoisted
out of the operator: the kernels fold it into their activation loads for every shape.
"""

from __future__ import annotations

import torch
from torch import nn

from .ops import sage, sage_dequantize


class SAGELinear(nn.Module):
    """SAGE 64/4, 128/3 or 256/2 packed linear."""

    permutation: torch.Tensor

    def __init__(
        self, packed: dict[str, torch.Tensor], out_features: int, bias: torch.Tensor | None = None
    ):
        super().__init__()
        self.out_features = out_features
        self.in_features = packed["packed_codes"].shape[1] * 128
        for name in ("packed_codes", "radius_codes", "radius_grid", "codebook", "permutation"):
            self.register_buffer(name, packed[name])
        self.register_buffer("bias", bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        output = sage(
            x.to(torch.float16).contiguous(),
            self.packed_codes,
            self.radius_codes,
            self.radius_grid,
            self.codebook,
            self.permutation,
            self.out_features,
        ).to(x.dtype)
        return output if self.bias is None else output + self.bias

    def dequantize(self) -> torch.Tensor:
        """Dense FP16 weight [out_features, in_features] in original channel order."""
        return sage_dequantize(
            self.packed_codes, self.radius_codes, self.radius_grid, self.codebook,
            self.permutation, self.out_features,
        )

    def extra_repr(self) -> str:
        return (
            f"in_features={self.in_features}, out_features={self.out_features}, "
            f"entries={self.codebook.shape[1]}, permuted={self.permutation.numel() > 0}"
        )
