"""Generates tests/golden/pack_cases.npz by running the REFERENCE's own exporter.

    python tests/golden/make_golden_pack.py [--reference DIR]

Runs `weight_vq.sphquant.packing.pack_spherical` of the reference checkout on small seeded
trained-state dictionaries (the construction of the reference's own test,
tests/inference/test_spherical_export.py:30-50: random signs / indices / logits, a
constant-radius group and an FP16-underflow group, a padded last row tile, permuted or not)
and stores inputs, intermediate radii and every packed buffer.  The exporter imports one
function from an un-vendored training package, `paroquant.optim.sphlinear.
direction_codebook_from_logits`; its definition is part of the reference itself
(patches/paroquant/0002-...patch:368-389) and is supplied here as a stand-in module so the
exporter runs unmodified.  The checkout is read only; nothing of it is copied into the
fixtures except the numbers its code produces.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import pathlib
import sys
import types

import numpy as np
import torch


def codebook_from_logits(angle_logits, *, angle_eps=1e-4):
    theta = angle_eps + (math.pi / 2 - 2 * angle_eps) * torch.sigmoid(angle_logits.float())
    sin_theta, cos_theta = torch.sin(theta), torch.cos(theta)
    prefix = torch.cumprod(sin_theta, dim=-1)
    parts = [cos_theta[..., :1]]
    for i in range(1, 7):
        parts.append(prefix[..., i - 1 : i] * cos_theta[..., i : i + 1])
    parts.append(prefix[..., -1:])
    directions = torch.cat(parts, dim=-1)
    return directions / directions.norm(dim=-1, keepdim=True).clamp_min(1e-12)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument(
        "--reference",
        default=os.environ.get("SAGE_REFERENCE_DIR", str(pathlib.Path(__file__).resolve().parents[3] / "reference")),
        help="checkout of the reference project (default: $SAGE_REFERENCE_DIR, else ../reference beside this repository)",
    )
    args = parser.parse_args()
    sys.path.insert(0, args.reference)
    stand_in = types.ModuleType("paroquant.optim.sphlinear")
    stand_in.direction_codebook_from_logits = codebook_from_logits
    for name in ("paroquant", "paroquant.optim"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["paroquant.optim.sphlinear"] = stand_in
    from weight_vq.sphquant.packing import pack_spherical

    arrays, index = {}, []
    for sage, bits, permuted, n, k in [
        (False, 6, False, 19, 256), (True, 6, False, 19, 256), (True, 6, True, 19, 256),
        (True, 7, True, 19, 256), (True, 8, False, 33, 384), (True, 8, True, 48, 512),
    ]:
        torch.manual_seed(17 + bits + 10 * permuted + n)
        state = {
            "signs": torch.randint(0, 2, (n, k), dtype=torch.int8) * 2 - 1,
            "direction_indices": torch.randint(0, 1 << bits, (n, k // 8)),
            "radius_logits": torch.randn(n, k // 8),
            "angle_logits": torch.randn(1 << bits, 7),
            "radius_bits": torch.tensor(10 - bits),
            "group_size": torch.tensor(128),
            "sphquant_version": torch.tensor(1),
        }
        state["radius_logits"][0, :16] = 0.125  # a constant-radius group
        state["radius_logits"][0, 16:] = -40    # an FP16-underflow group: zero step
        if sage:
            order = torch.randperm(k) if permuted else torch.arange(k)
            state.update(channel_unpermutation=order.argsort(), sage_version=torch.tensor(1))
        packed = pack_spherical(state, sage=sage)
        name = f"{'sage' if sage else 'sph'}_b{bits}_{'perm' if permuted else 'plain'}_{n}x{k}"
        index.append({"name": name, "sage": sage, "bits": bits, "permuted": permuted, "n": n, "k": k})
        for key in ("signs", "direction_indices", "radius_logits", "angle_logits"):
            arrays[f"{name}/state/{key}"] = state[key].numpy()
        if sage:
            arrays[f"{name}/state/channel_unpermutation"] = state["channel_unpermutation"].numpy()
        arrays[f"{name}/radius"] = torch.nn.functional.softplus(state["radius_logits"].float()).numpy()
        for key, value in packed.items():
            data = value.numpy()
            arrays[f"{name}/packed/{key}"] = data.view(np.uint16) if data.dtype == np.float16 else data
    arrays["index_json"] = np.frombuffer(json.dumps(index).encode(), dtype=np.uint8)
    target = pathlib.Path(__file__).resolve().parent / "pack_cases.npz"
    np.savez_compressed(target, **arrays)
    print(f"wrote {target} ({target.stat().st_size} bytes, {len(index)} cases)")


if __name__ == "__main__":
    main()
