"""SPHQuant 64/4 packed linear on the GPU, through the C ABI: the reference's own test cases
(tests/inference/test_ops.py) with this build's tighter gate, dense dequantisation bit-exact
against the oracle and the golden hashes."""

import hashlib
import json
import pathlib

import numpy as np
import pytest
import torch

from oracle import sph_oracle
from sage_b200 import SPHQuantLinear, sph_dequantize, synthetic_sphquant

pytestmark = pytest.mark.gpu
GOLDEN = pathlib.Path(__file__).parent / "golden"
GATE = 1e-3  # relative Frobenius error against the FP32 matmul on the oracle's decoded weight
REFERENCE_GATE = 5e-3  # the reference's own bound (tests/inference/test_ops.py:33); used where the
#                        output has so few elements that one FP16 rounding decides the ratio


def relative_error(actual: torch.Tensor, expected: np.ndarray) -> float:
    a = actual.float().cpu().numpy().reshape(expected.shape)
    return float(np.linalg.norm(a - expected) / max(np.linalg.norm(expected), 1e-30))


@pytest.mark.parametrize("shape,n", [((128,), 1), ((4, 256), 17), ((2, 3, 2560), 9), ((1, 9728), 17),
                                     ((1, 16384), 9), ((1, 2560), 9728), ((8, 4096), 2560), ((21, 1024), 333)])
def test_matches_oracle(shape, n):
    cpu_packed = synthetic_sphquant(shape[-1], n, seed=42)
    layer = SPHQuantLinear({key: tensor.cuda() for key, tensor in cpu_packed.items()})
    x = torch.randn(shape, generator=torch.Generator().manual_seed(43), dtype=torch.float16)
    with torch.inference_mode():
        actual = layer(x.cuda())
    assert actual.shape == (*shape[:-1], n) and actual.dtype == torch.float16
    expected = sph_oracle.linear_fp32(x, cpu_packed)
    assert relative_error(actual, expected) < (GATE if actual.numel() >= 64 else REFERENCE_GATE)


@pytest.mark.parametrize("rows,k,n", [(33, 256, 129), (257, 1024, 640), (300, 2560, 333), (512, 2560, 4096),
                                      (513, 1280, 2560), (2048, 4096, 2560)])
def test_prompt_rows_on_the_tensor_core_path_match_oracle(rows, k, n):
    """33 rows and more run the tcgen05 GEMM with this format's decode (row-major codes, n not
    padded to 16, several token blocks and both accumulators): same gate as the decode kernel,
    and every output row equal to the 8-row decode path's to FP16 rounding."""
    cpu_packed = synthetic_sphquant(k, n, seed=rows)
    layer = SPHQuantLinear({key: tensor.cuda() for key, tensor in cpu_packed.items()})
    x = torch.randn(rows, k, generator=torch.Generator().manual_seed(rows + 1), dtype=torch.float16)
    with torch.inference_mode():
        actual = layer(x.cuda())
        few = layer(x[:8].cuda())  # the decode kernel on the first rows
    expected = sph_oracle.linear_fp32(x, cpu_packed)
    assert relative_error(actual, expected) < GATE
    row_error = (actual[:8].float() - few.float()).norm() / few.float().norm()
    assert float(row_error) < 2e-3
    # one-hot rows: a token routed to the wrong block or accumulator shows as a wrong row
    hot = torch.zeros(rows, k, dtype=torch.float16)
    columns = torch.arange(rows) % k
    hot[torch.arange(rows), columns] = 1.0
    with torch.inference_mode():
        picked = layer(hot.cuda()).float().cpu()
    dense = torch.from_numpy(np.asarray(sph_oracle.decode_fp16(cpu_packed), dtype=np.float32))  # [n, k]
    assert torch.equal(picked, dense[:, columns].T.contiguous())  # x = 1 picks a weight: bit-exact


def test_zero_and_constant_grid():
    packed = synthetic_sphquant(128, 9)
    packed["radius_scales"].zero_()
    packed["radius_mins"].zero_()
    packed["radius_mins"][1:].fill_(0.25)
    layer = SPHQuantLinear({k: v.cuda() for k, v in packed.items()})
    x = torch.ones(4, 128, dtype=torch.float16)
    actual = layer(x.cuda())
    assert torch.count_nonzero(actual[:, 0]) == 0
    assert relative_error(actual, sph_oracle.linear_fp32(x, packed)) < GATE


def test_graph_state_dict_bias_and_odd_offsets():
    cpu_packed = synthetic_sphquant(256, 17)
    packed = {k: v.cuda() for k, v in cpu_packed.items()}
    x = torch.randn(2, 256, device="cuda", dtype=torch.float16)
    layer = SPHQuantLinear(packed, torch.ones(17, device="cuda", dtype=torch.float16))
    restored = SPHQuantLinear(cpu_packed, torch.zeros(17).half())
    restored.load_state_dict(layer.state_dict())
    restored = restored.cuda()
    with torch.inference_mode():
        expected = layer(x)
        assert torch.equal(restored(x), expected)
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(3):
                layer(x)
        torch.cuda.current_stream().wait_stream(stream)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            output = layer(x)
        graph.replay()
        assert torch.equal(output, expected)
        assert torch.equal(layer(x.T.contiguous().T), expected)  # layout conversion inside the module
        storage = torch.zeros(2 * 256 + 1, device="cuda", dtype=torch.float16)
        shifted = storage[1:].view(2, 256)  # 2-byte aligned only
        shifted.copy_(x)
        assert torch.equal(layer(shifted), expected)
        assert torch.equal(layer(x.float()).half(), expected) and layer(x.float()).dtype == torch.float32


def test_argument_checks_and_opcheck():
    packed = {k: v.cuda() for k, v in synthetic_sphquant(256, 5).items()}
    layer = SPHQuantLinear(packed)
    with pytest.raises(RuntimeError, match="invalid SPH input dimension"):
        layer(torch.zeros(1, 192, device="cuda", dtype=torch.float16))
    with pytest.raises(RuntimeError, match="invalid SPH packed code shape"):
        layer(torch.zeros(1, 384, device="cuda", dtype=torch.float16))
    from sage_b200.sphquant import sphquant

    x = torch.randn(3, 256, device="cuda", dtype=torch.float16)
    torch.library.opcheck(sphquant, (x, *[packed[k] for k in sph_oracle.KEYS]),
                          test_utils=("test_schema", "test_faketensor"))
    assert layer(torch.zeros(0, 256, device="cuda", dtype=torch.float16)).shape == (0, 5)


def test_dequantisation_is_bit_exact():
    data = np.load(GOLDEN / "sph_cases.npz")
    for case in json.loads(bytes(data["index_json"]).decode()):
        name = case["name"]
        packed = {key: data[f"{name}/{key}"] for key in sph_oracle.KEYS}
        device = {key: torch.from_numpy(packed[key].view(np.float16) if packed[key].dtype == np.uint16 else packed[key]).cuda()
                  for key in sph_oracle.KEYS}
        weight = sph_dequantize(*[device[key] for key in sph_oracle.KEYS]).cpu().numpy()
        want = data[f"{name}/weight_fp32"].astype(np.float16)
        assert np.array_equal(weight.view(np.uint16), want.view(np.uint16)), name


@pytest.mark.parametrize("case", json.loads((GOLDEN / "sph_hashes.json").read_text())["cases"],
                         ids=lambda c: f"k{c['k']}_n{c['n']}_s{c['seed']}")
def test_dequantisation_hashes_at_benchmark_sizes(case):
    packed = {k: v.cuda() for k, v in synthetic_sphquant(case["k"], case["n"], case["seed"]).items()}
    weight = sph_dequantize(*[packed[key] for key in sph_oracle.KEYS]).cpu().numpy()
    assert hashlib.sha256(np.ascontiguousarray(weight.view(np.uint16)).tobytes()).hexdigest() == case["weight_fp16_sha256"]
