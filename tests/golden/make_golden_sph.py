"""Generate SPHQuant golden vectors from the reference project's own Python code.

    python tests/golden/make_golden_sph.py --reference /path/to/reference

Calls the reference's `synthetic_sphquant` (weight_vq/checkpoint.py:35-51) for packed inputs
and `decode_sphquant` (tests/inference/reference.py:16-22) to decode them; writes
`sph_cases.npz` (small cases: the five buffers, decoded FP32 weight, an FP16 input and the FP32
output `x.float() @ W.T` of tests/inference/test_ops.py:22) and `sph_hashes.json` (SHA-256 of
buffers and decoded weights for benchmark-sized shapes).  Tests only read those two files.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
SMALL_CASES = [(128, 1, 42), (128, 9, 0), (256, 17, 42), (2560, 9, 42), (1024, 33, 7)]  # (K, N, seed)
HASH_CASES = [(2560, 9728, 0), (9728, 2560, 1), (4096, 2560, 2)]
KEYS = ("packed_codes", "radius_extra", "radius_scales", "radius_mins", "codebook")


def raw(tensor: torch.Tensor) -> np.ndarray:
    array = tensor.numpy()
    return array.view(np.uint16) if tensor.dtype == torch.float16 else array


def sha(array: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument(
        "--reference",
        default=os.environ.get("SAGE_REFERENCE_DIR", str(pathlib.Path(__file__).resolve().parents[3] / "reference")),
        help="checkout of the reference project (default: $SAGE_REFERENCE_DIR, else ../reference beside this repository)",
    )
    args = parser.parse_args()
    sys.path.insert(0, args.reference)
    from tests.inference.reference import decode_sphquant  # type: ignore
    from weight_vq.checkpoint import synthetic_sphquant  # type: ignore

    arrays: dict[str, np.ndarray] = {}
    index = []
    for k, n, seed in SMALL_CASES:
        name = f"k{k}_n{n}_s{seed}"
        packed = synthetic_sphquant(k, n, seed=seed)
        weight = decode_sphquant(packed)
        x = torch.randn(3, k, generator=torch.Generator().manual_seed(43), dtype=torch.float16)
        for key in KEYS:
            arrays[f"{name}/{key}"] = raw(packed[key])
        arrays[f"{name}/weight_fp32"] = weight.numpy()
        arrays[f"{name}/x_fp16_bits"] = x.numpy().view(np.uint16)
        arrays[f"{name}/y_fp32"] = (x.float() @ weight.T).numpy()
        index.append({"name": name, "k": k, "n": n, "seed": seed})
    arrays["index_json"] = np.frombuffer(json.dumps(index).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "sph_cases.npz", **arrays)

    hashes = []
    for k, n, seed in HASH_CASES:
        packed = synthetic_sphquant(k, n, seed=seed)
        weight = decode_sphquant(packed)
        hashes.append({
            "k": k, "n": n, "seed": seed,
            "packed_sha256": {key: sha(raw(packed[key]).view(np.uint8)) for key in KEYS},
            "weight_fp32_sha256": sha(weight.numpy().view(np.uint32)),
            "weight_fp16_sha256": sha(weight.half().numpy().view(np.uint16)),
        })
    (HERE / "sph_hashes.json").write_text(json.dumps({
        "generator": "tests/golden/make_golden_sph.py", "torch": torch.__version__, "cases": hashes}, indent=1) + "\n")
    print("wrote", HERE / "sph_cases.npz", HERE / "sph_hashes.json")


if __name__ == "__main__":
    main()
