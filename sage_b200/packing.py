"""Trained spherical state -> packed SAGE / SPHQuant buffers, packed on the GPU.

Mirrors the reference's exporter `pack_spherical(state, *, sage)`
(weight_vq/sphquant/packing.py:7-77): same state keys, same checks and messages, same
returned buffers.  The per-weight work (grid fitting, radius-code selection, sign / index /
radius bit packing, SAGE's tiling and row padding) runs in one CUDA kernel through
`sageb200_pack_spherical`; the two small float tensors the exporter derives first are
computed here with torch on the state's device, as the reference does:

  * radii = softplus(radius_logits)                       (packing.py:34)
  * the direction codebook from its seven angular logits  (`direction_codebook_from_logits`,
    defined by the reference in patches/paroquant/0002-...patch:368-389: hyperspherical
    angles in (0, pi/2) -> a non-negative unit 8-vector)

There is no CPU path: the state must live on a CUDA device.
"""

from __future__ import annotations

import ctypes
import math

import torch

from . import _lib

ANGLE_EPS = 1e-4


def direction_codebook_from_logits(angle_logits: torch.Tensor, *, angle_eps: float = ANGLE_EPS) -> torch.Tensor:
    """[entries, 7] angular logits -> [entries, 8] non-negative unit directions (FP32)."""
    if angle_logits.shape[-1] != 7:
        raise ValueError(f"Expected seven angular logits, got {angle_logits.shape}")
    theta = angle_eps + (math.pi / 2 - 2 * angle_eps) * torch.sigmoid(angle_logits.float())
    sin_theta, cos_theta = torch.sin(theta), torch.cos(theta)
    prefix = torch.cumprod(sin_theta, dim=-1)
    components = [cos_theta[..., :1]]
    for index in range(1, 7):
        components.append(prefix[..., index - 1 : index] * cos_theta[..., index : index + 1])
    components.append(prefix[..., -1:])
    directions = torch.cat(components, dim=-1)
    return directions / directions.norm(dim=-1, keepdim=True).clamp_min(1e-12)


def pack_spherical_radii(signs: torch.Tensor, direction_indices: torch.Tensor, radius: torch.Tensor,
                         entries: int, *, sage: bool) -> dict[str, torch.Tensor]:
    """The kernel call: signs int8 [n, k] (+1/-1), indices [n, k/8], FP32 radii [n, k/8] ->
    the packed code / radius / grid buffers (everything of the packed dict except the codebook
    and the permutation)."""
    if not signs.is_cuda:
        raise RuntimeError("sage_b200 packs on a CUDA device; there is no CPU path")
    n, k = signs.shape
    if k % 128:
        raise ValueError("packed spherical inference requires input width divisible by 128")
    device = signs.device
    groups = k // 128
    signs = signs.to(torch.int8).contiguous()
    indices = direction_indices.to(device=device, dtype=torch.int32).reshape(n, k // 8).contiguous()
    radius = radius.to(device=device, dtype=torch.float32).reshape(n, k // 8).contiguous()
    lib = _lib.load()
    vp = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    with torch.cuda.device(device):
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        if sage:
            tiles = (n + 15) // 16
            out = {
                "packed_codes": torch.empty(tiles, groups, 16, 8, dtype=torch.int32, device=device),
                "radius_codes": torch.empty(tiles, groups, 16, dtype=torch.int32, device=device),
                "radius_grid": torch.empty(tiles, groups, 16, 2, dtype=torch.float16, device=device),
            }
            status = lib.sageb200_pack_spherical(
                vp(signs), vp(indices), vp(radius), vp(out["packed_codes"]), vp(out["radius_codes"]),
                vp(out["radius_grid"]), None, n, k, entries, 1, stream)
        else:
            out = {
                "packed_codes": torch.empty(n, k // 8, dtype=torch.int16, device=device),
                "radius_extra": torch.empty(n, groups, dtype=torch.int32, device=device),
                "radius_scales": torch.empty(n, groups, dtype=torch.float16, device=device),
                "radius_mins": torch.empty(n, groups, dtype=torch.float16, device=device),
            }
            status = lib.sageb200_pack_spherical(
                vp(signs), vp(indices), vp(radius), vp(out["packed_codes"]), vp(out["radius_extra"]),
                vp(out["radius_scales"]), vp(out["radius_mins"]), n, k, entries, 0, stream)
    if status:
        raise RuntimeError(f"sageb200_pack_spherical: {lib.sageb200_status_string(status).decode()}")
    return out


@torch.no_grad()
def pack_spherical(state: dict[str, torch.Tensor], *, sage: bool) -> dict[str, torch.Tensor]:
    """Pack frozen signs/indices and trained radii/angles, without refitting
    (reference weight_vq/sphquant/packing.py:7-77; same keys in, same buffers out)."""
    if sage != ("sage_version" in state):
        raise ValueError("spherical checkpoint method does not match the export configuration")
    entries = state["angle_logits"].shape[0]
    bits = entries.bit_length() - 1
    if entries not in ((64, 128, 256) if sage else (64,)):
        raise ValueError("packed SPHQuant requires 64/4; packed SAGE requires 64/4, 128/3 or 256/2")
    if int(state["group_size"]) != 128 or int(state["radius_bits"]) != 10 - bits:
        raise ValueError("checkpoint does not use the spherical kernel's 128-group bit split")
    n, k = state["signs"].shape
    if k % 128:
        raise ValueError("packed spherical inference requires input width divisible by 128")
    codebook = direction_codebook_from_logits(state["angle_logits"]).half()
    radius = torch.nn.functional.softplus(state["radius_logits"].float())
    packed = pack_spherical_radii(state["signs"], state["direction_indices"], radius, entries, sage=sage)
    if not sage:
        packed["codebook"] = codebook.contiguous()
        return packed
    packed["codebook"] = codebook.reshape(entries, 4, 2).permute(1, 0, 2).contiguous()
    # the checkpoint stores the inverse channel permutation; inference gathers with the forward one
    permutation = state["channel_unpermutation"].argsort().int()
    if torch.equal(permutation, torch.arange(k, device=permutation.device, dtype=torch.int32)):
        permutation = torch.empty(0, device=permutation.device, dtype=torch.int32)
    packed["permutation"] = permutation.to(packed["packed_codes"].device)
    return packed
