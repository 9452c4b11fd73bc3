"""Generate golden vectors from the reference project's own Python code.

Run where the reference checkout is available (it is imported, never copied):

    python tests/golden/make_golden.py --reference /path/to/reference

It calls the reference's `synthetic_sage` (weight_vq/checkpoint.py:54-89) to make
packed inputs and the reference's `decode_sage` (tests/inference/reference.py:39-49)
to decode them, and writes

  sage_cases.npz   small cases: every packed buffer, the decoded FP16 weight bits
                   and the FP32 `F.linear(x.float(), W.half().float())` output
  sage_hashes.json SHA-256 of packed buffers and decoded FP16 weights for
                   benchmark-sized shapes (the arrays themselves are too large
                   to commit)

The GPU box has no reference checkout, so tests only read these two files.
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

# (K, N, seed, permuted): seeds 0/1/2 select 256/128/64 codebook entries.
SMALL_CASES = [
    (128, 1, 0, False),
    (128, 1, 2, True),
    (256, 17, 0, True),
    (256, 17, 1, False),
    (512, 129, 2, False),
    (2560, 33, 1, True),
    (4096, 48, 2, True),
    (1024, 16, 0, True),
]
HASH_CASES = [
    (2560, 9728, 0, True),
    (2560, 9728, 1, True),
    (2560, 9728, 2, True),
    (9728, 2560, 0, True),
    (4096, 2560, 1, False),
    (2560, 1024, 2, True),
]
KEYS = ("packed_codes", "radius_codes", "radius_grid", "codebook", "permutation")


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
    from tests.inference.reference import decode_sage, unpack_sage  # type: ignore
    from weight_vq.checkpoint import synthetic_sage  # type: ignore

    arrays: dict[str, np.ndarray] = {}
    index = []
    for k, n, seed, permuted in SMALL_CASES:
        name = f"k{k}_n{n}_s{seed}_p{int(permuted)}"
        packed = synthetic_sage(k, n, seed=seed, permuted=permuted)
        weight = decode_sage(packed, n)
        x = torch.randn(3, k, generator=torch.Generator().manual_seed(43), dtype=torch.float16)
        y = torch.nn.functional.linear(x.float(), weight.half().float())
        signs, indices, radii = unpack_sage(packed, n)
        for key in KEYS:
            arrays[f"{name}/{key}"] = packed[key].numpy().view(
                np.uint16 if packed[key].dtype == torch.float16 else packed[key].numpy().dtype
            )
        arrays[f"{name}/weight_fp16_bits"] = weight.half().numpy().view(np.uint16)
        arrays[f"{name}/x_fp16_bits"] = x.numpy().view(np.uint16)
        arrays[f"{name}/y_fp32"] = y.numpy()
        arrays[f"{name}/field_index"] = indices.numpy().astype(np.int16)
        arrays[f"{name}/field_radius"] = radii.numpy().astype(np.int8)
        arrays[f"{name}/field_sign_bits"] = (
            ((signs.numpy() < 0).astype(np.int64) << np.arange(8)).sum(-1).astype(np.uint8)
        )
        index.append({"name": name, "k": k, "n": n, "seed": seed, "permuted": permuted})
    arrays["index_json"] = np.frombuffer(json.dumps(index).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "sage_cases.npz", **arrays)

    hashes = []
    for k, n, seed, permuted in HASH_CASES:
        packed = synthetic_sage(k, n, seed=seed, permuted=permuted)
        weight = decode_sage(packed, n).half()
        x = torch.randn(1, k, generator=torch.Generator().manual_seed(43), dtype=torch.float16)
        y = torch.nn.functional.linear(x.float(), weight.float())
        hashes.append(
            {
                "k": k,
                "n": n,
                "seed": seed,
                "permuted": permuted,
                "entries": int(packed["codebook"].shape[1]),
                "packed_sha256": {key: sha(packed[key].numpy().view(np.uint8)) for key in KEYS},
                "weight_fp16_sha256": sha(weight.numpy().view(np.uint16)),
                "y_fp32_first8": [float(v) for v in y[0, :8]],
                "y_fp32_norm": float(y.norm()),
            }
        )
    meta = {
        "generator": "tests/golden/make_golden.py",
        "torch": torch.__version__,
        "numpy": np.__version__,
        "cases": hashes,
    }
    (HERE / "sage_hashes.json").write_text(json.dumps(meta, indent=1) + "\n")
    print("wrote", HERE / "sage_cases.npz", HERE / "sage_hashes.json")


if __name__ == "__main__":
    main()
