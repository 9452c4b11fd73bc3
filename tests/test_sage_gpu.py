"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle.

Modelled on the reference's kernel tests (tests/inference/test_sage.py:66-203 there):
same shape list, both permutation settings, the three bit splits, three input scales,
misaligned storage offsets, zero/constant grids, state_dict round trip, side streams,
CUDA-graph replay, bias and opcheck.

Gates:
  dense dequantisation        bit-exact FP16 (integer compare)
  matmul output               relative Frobenius error <= 1e-3 against an FP32 matmul on the
                              oracle's FP16 weights, and max-abs / RMS < 5e-3 (the reference's
                              own second gate, tests/inference/test_sage.py:11-19)
"""

import ctypes

import numpy as np
import pytest
import torch

from oracle import c_oracle, sage_oracle
from sage_b200 import SAGELinear, _lib, sage, sage_dequantize, sage_grouped, synthetic_sage

pytestmark = pytest.mark.gpu

REL_FROBENIUS = 1e-3
MAX_OVER_RMS = 5e-3


def to_cuda(packed):
    return {k: v.cuda() for k, v in packed.items()}


def expected_output(x, cpu_packed, n):
    """FP32 matmul on the oracle's FP16 dequantised weight (computed on the GPU in FP32)."""
    weight = torch.from_numpy(c_oracle.decode_fp16(cpu_packed, n)).cuda()
    return x.float() @ weight.float().T


def assert_output(actual, expected):
    if actual.numel() == 0:
        return {}
    error = actual.float() - expected.float()
    norm = expected.float().norm().clamp_min(1e-30)
    rms = expected.float().square().mean().sqrt().clamp_min(1e-30)
    metrics = {
        "relative_frobenius": (error.norm() / norm).item(),
        "max_absolute_over_rms": (error.abs().max() / rms).item(),
    }
    assert metrics["relative_frobenius"] <= REL_FROBENIUS, metrics
    assert metrics["max_absolute_over_rms"] < MAX_OVER_RMS, metrics
    return metrics


# ---------------------------------------------------------------- dense dequantisation


@pytest.mark.parametrize(
    "k,n", [(128, 1), (256, 17), (512, 129), (2560, 33), (4096, 48), (9728, 32), (16384, 9)]
)
@pytest.mark.parametrize("permuted", [False, True])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_dequant_bit_exact(k, n, permuted, seed):
    cpu = synthetic_sage(k, n, seed=seed, permuted=permuted)
    gpu = to_cuda(cpu)
    args = [gpu[key] for key in ("packed_codes", "radius_codes", "radius_grid", "codebook", "permutation")]
    got = sage_dequantize(*args, n).cpu().numpy().view(np.uint16)
    np.testing.assert_array_equal(got, c_oracle.decode_fp16(cpu, n).view(np.uint16))
    quantised = sage_dequantize(*args, n, original_order=False).cpu().numpy().view(np.uint16)
    np.testing.assert_array_equal(
        quantised, c_oracle.decode_fp16(cpu, n, apply_permutation=False).view(np.uint16)
    )


def test_dequant_golden_cases(golden_cases):
    """Against the weights the reference's own decoder produced."""
    for case in golden_cases:
        gpu = {k: torch.from_numpy(np.ascontiguousarray(v)).cuda() for k, v in case["packed"].items()}
        got = sage_dequantize(
            gpu["packed_codes"], gpu["radius_codes"], gpu["radius_grid"], gpu["codebook"],
            gpu["permutation"], case["n"],
        )
        np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), case["weight_fp16_bits"])


def test_dequant_all_code_values():
    """Every 16-bit code value, the three bit splits (reference test_sage.py:46-63)."""
    for seed in (0, 1, 2):
        cpu = synthetic_sage(128, 4096, seed=seed, permuted=False)
        words = torch.arange(65536).reshape(4096, 16)
        cpu["packed_codes"] = (words[:, ::2] | (words[:, 1::2] << 16)).int().reshape(256, 1, 16, 8)
        cpu["radius_codes"].fill_(int(torch.tensor(0xE4E4E4E4).int()))
        gpu = to_cuda(cpu)
        got = sage_dequantize(
            gpu["packed_codes"], gpu["radius_codes"], gpu["radius_grid"], gpu["codebook"],
            gpu["permutation"], 4096,
        )
        np.testing.assert_array_equal(
            got.cpu().numpy().view(np.uint16), c_oracle.decode_fp16(cpu, 4096).view(np.uint16)
        )


def test_dequant_benchmark_shape_hashes(golden_hashes):
    """Benchmark-sized matrices against SHA-256 of the reference decoder's output."""
    import hashlib

    for case in golden_hashes:
        cpu = synthetic_sage(case["k"], case["n"], seed=case["seed"], permuted=case["permuted"])
        gpu = to_cuda(cpu)
        got = sage_dequantize(
            gpu["packed_codes"], gpu["radius_codes"], gpu["radius_grid"], gpu["codebook"],
            gpu["permutation"], case["n"],
        )
        digest = hashlib.sha256(got.cpu().numpy().view(np.uint16).tobytes()).hexdigest()
        assert digest == case["weight_fp16_sha256"], (case["k"], case["n"], case["seed"])


# ---------------------------------------------------------------- matmul against the oracle

REFERENCE_SHAPES = [
    ((128,), 1),
    ((4, 256), 17),
    ((2, 3, 2560), 9),
    ((1, 9728), 33),
    ((1, 16384), 9),
    ((128, 256), 32),
    ((16, 128), 1),
    ((17, 256), 17),
    ((65, 2560), 33),
    ((256, 128), 16),
    ((16, 512), 129),
    ((31, 2560), 257),
    ((32, 4096), 256),
    ((129, 9728), 65),
    ((1, 4096), 1024),
    ((1, 4096), 1025),
    ((2, 3, 4352), 33),
    ((15, 4096), 1025),
    ((1, 2560), 4096),
    ((1, 2560), 1024),
    ((1, 2560), 9728),
    ((1, 4096), 2560),
    ((1, 9728), 2560),
    ((0, 128), 17),
]


@pytest.mark.parametrize("shape,n", REFERENCE_SHAPES)
@pytest.mark.parametrize("permuted", [False, True])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_linear_against_oracle(shape, n, permuted, seed):
    cpu = synthetic_sage(shape[-1], n, seed=seed, permuted=permuted)
    layer = SAGELinear(to_cuda(cpu), n)
    base = torch.randn(shape, generator=torch.Generator().manual_seed(43), dtype=torch.float16).cuda()
    weight = torch.from_numpy(c_oracle.decode_fp16(cpu, n)).cuda().float()
    for scale in (0.03125, 1.0, 32.0):
        x = base * scale
        # a contiguous tensor can sit at an odd (2-byte) storage offset
        storage = torch.empty(x.numel() + 1, device="cuda", dtype=x.dtype)
        shifted = storage[1:].view(shape).copy_(x)
        actual = layer(shifted)
        assert torch.equal(actual, layer(x))
        assert actual.shape == (*shape[:-1], n)
        assert_output(actual, x.float() @ weight.T)


@pytest.mark.parametrize("rows", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("bits", [6, 7, 8])
@pytest.mark.parametrize(
    "k,n", [(2560, 4096), (2560, 1024), (4096, 2560), (2560, 9728), (9728, 2560)]
)
def test_qwen3_4b_layer_shapes(k, n, rows, bits):
    """The decoder-layer shapes at batch 1..16 with every bit split forced."""
    cpu = synthetic_sage(k, n, seed=100 + bits, permuted=True, direction_bits=bits)
    layer = SAGELinear(to_cuda(cpu), n)
    x = torch.randn(rows, k, generator=torch.Generator().manual_seed(7), dtype=torch.float16).cuda()
    assert_output(layer(x), expected_output(x, cpu, n))


def test_one_hot_rows_reproduce_weight_columns():
    """x = e_j selects column j of the weight: checks the permutation fold and the row
    mapping element by element (not only in norm)."""
    k, n = 512, 48
    cpu = synthetic_sage(k, n, seed=1, permuted=True)
    layer = SAGELinear(to_cuda(cpu), n)
    weight = torch.from_numpy(c_oracle.decode_fp16(cpu, n)).cuda()
    for start in range(0, k, 16):
        x = torch.zeros(16, k, dtype=torch.float16, device="cuda")
        x[torch.arange(16), torch.arange(start, start + 16)] = 1.0
        got = layer(x)  # [16, n]; got[m] ~ weight[:, start+m]
        want = weight[:, start : start + 16].T.float()
        assert torch.allclose(got.float(), want, rtol=2e-3, atol=1e-6)


def test_full_size_against_gpu_dequant():
    """At the benchmark's full size: matmul against an FP32 matmul on the kernel-made dense
    weight (itself pinned bit-exactly by the hash test), plus linearity of the operator."""
    k, n = 2560, 9728
    for seed in (0, 1, 2):
        gpu = to_cuda(synthetic_sage(k, n, seed=seed, permuted=True))
        layer = SAGELinear(gpu, n)
        weight = layer.dequantize().float()
        x = torch.randn(16, k, generator=torch.Generator().manual_seed(seed), dtype=torch.float16).cuda()
        for rows in (1, 3, 8, 16):
            assert_output(layer(x[:rows]), x[:rows].float() @ weight.T)
        a, b = layer(x[:1]).float(), layer(x[1:2]).float()
        both = layer((x[:1].float() + x[1:2].float()).half()).float()
        assert ((a + b - both).norm() / both.norm()).item() < 3e-3


# ---------------------------------------------------------------- module behaviour


@pytest.mark.parametrize("rows,k", [(2, 256), (65, 256), (32, 4096), (1, 2560), (1, 4096), (1, 9728)])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_grids_state_streams_graph_bias_opcheck(rows, k, seed):
    cpu = synthetic_sage(k, 17, seed=seed)
    cpu["radius_grid"][..., 1].zero_()
    cpu["radius_grid"][..., 0].fill_(0.25)
    cpu["radius_grid"][0, :, 0].zero_()
    layer = SAGELinear(to_cuda(cpu), 17)
    restored = SAGELinear({key: torch.zeros_like(value) for key, value in cpu.items()}, 17)
    missing, unexpected = restored.load_state_dict(layer.state_dict())
    assert not missing and not unexpected
    restored.cuda()
    x = torch.randn(rows, k, device="cuda", dtype=torch.float16)
    expected = layer(x)
    assert torch.count_nonzero(expected[:, 0]) == 0
    assert_output(expected, expected_output(x, cpu, 17))
    assert torch.equal(restored(x), expected)
    assert torch.equal(layer(x.T.contiguous().T), expected)
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
    graph.replay()
    assert torch.equal(output, expected)
    layer.bias = torch.ones(17, device="cuda", dtype=torch.float16)
    assert torch.equal(layer(x), expected + 1)
    torch.library.opcheck(
        sage,
        (x, layer.packed_codes, layer.radius_codes, layer.radius_grid, layer.codebook, layer.permutation, 17),
    )


def test_dtype_boundary_and_repeatability():
    cpu = synthetic_sage(2560, 40, seed=0)
    layer = SAGELinear(to_cuda(cpu), 40)
    x = torch.randn(3, 2560, device="cuda", dtype=torch.bfloat16)
    out = layer(x)
    assert out.dtype == torch.bfloat16
    reference = expected_output(x.half(), cpu, 40)
    assert ((out.float() - reference).norm() / reference.norm()).item() < 5e-3
    first = layer(x.half())
    for _ in range(20):
        assert torch.equal(layer(x.half()), first)


def test_validation_errors():
    cpu = synthetic_sage(256, 17, seed=0)
    gpu = to_cuda(cpu)
    layer = SAGELinear(gpu, 17)
    with pytest.raises(RuntimeError, match="contiguous CUDA FP16"):
        sage(torch.zeros(2, 256, device="cuda"), *[gpu[k] for k in gpu], 17)
    with pytest.raises(RuntimeError, match="Invalid SAGE packed layout"):
        sage(torch.zeros(2, 256, device="cuda", dtype=torch.float16), *[gpu[k] for k in gpu], 33)
    with pytest.raises(RuntimeError, match="divisible by 128"):
        sage(torch.zeros(2, 200, device="cuda", dtype=torch.float16), *[gpu[k] for k in gpu], 17)
    bad = dict(gpu)
    bad["codebook"] = torch.zeros(4, 32, 2, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match="codebook"):
        sage(torch.zeros(2, 256, device="cuda", dtype=torch.float16), *[bad[k] for k in bad], 17)
    assert layer(torch.zeros(0, 256, device="cuda", dtype=torch.float16)).shape == (0, 17)


# ---------------------------------------------------------------- the C ABI directly


def test_c_abi_status_codes_and_host_entry():
    lib = _lib.load()
    k, n, rows = 2560, 1024, 4
    cpu = synthetic_sage(k, n, seed=2)
    gpu = to_cuda(cpu)
    entries = cpu["codebook"].shape[1]
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    x = torch.randn(rows, k, dtype=torch.float16)
    y = torch.empty(rows, n, dtype=torch.float16)
    staging_bytes = lib.sageb200_host_staging_bytes(rows, n, k)
    staging = torch.zeros(staging_bytes, dtype=torch.uint8, device="cuda")
    launches = lib.sageb200_launch_count()
    for pinned in (False, True):
        xh = x.pin_memory() if pinned else x
        yh = y.pin_memory() if pinned else y
        status = lib.sageb200_linear_host(
            ctypes.c_void_p(xh.data_ptr()), ptr(gpu["packed_codes"]), ptr(gpu["radius_codes"]),
            ptr(gpu["radius_grid"]), ptr(gpu["codebook"]), ptr(gpu["permutation"]),
            ctypes.c_void_p(yh.data_ptr()), ptr(staging), staging_bytes, rows, n, k, entries, stream,
        )
        assert status == 0, lib.sageb200_status_string(status)
        assert_output(yh.cuda(), expected_output(x.cuda(), cpu, n))
    assert lib.sageb200_launch_count() >= launches + 2
    # error paths return codes, never raise or launch
    dev_x = x.cuda()
    dev_y = torch.empty(rows, n, dtype=torch.float16, device="cuda")
    common = (ptr(gpu["packed_codes"]), ptr(gpu["radius_codes"]), ptr(gpu["radius_grid"]), ptr(gpu["codebook"]), ptr(gpu["permutation"]))
    assert lib.sageb200_linear(ptr(dev_x), *common, ptr(dev_y), None, 0, rows, n, 200, entries, stream) == -1
    assert lib.sageb200_linear(ptr(dev_x), *common, ptr(dev_y), None, 0, rows, n, k, 100, stream) == -1
    assert lib.sageb200_linear(ptr(dev_x), *common, ptr(dev_y), None, 0, 70000, n, k, entries, stream) == -3
    assert lib.sageb200_linear(ptr(dev_x), *common, ptr(dev_y), None, 0, rows, n, k, entries, stream) == -4
    misaligned = ctypes.c_void_p(gpu["radius_grid"].data_ptr() + 2)
    assert lib.sageb200_linear(
        ptr(dev_x), common[0], common[1], misaligned, common[3], common[4], ptr(dev_y), None, 0, rows, n, k, entries, stream
    ) == -2
    assert lib.sageb200_linear(ptr(dev_x), *common, ptr(dev_y), None, 0, 0, n, k, entries, stream) == 0
    assert lib.sageb200_gemv_fuses_permutation(n, 16384) == 1


def test_grouped_launch_matches_oracle_and_is_repeatable():
    """q/k/v-style grouped launch: one kernel for three linears that share an input.  The
    grouped launch plans its CTAs jointly, so sums may associate differently from single
    launches; each output must pass the oracle gate and repeat bit for bit."""
    k = 2560
    shapes = [(4096, 0), (1024, 1), (1024, 2)]
    for rows in (1, 5, 16):
        x = torch.randn(rows, k, generator=torch.Generator().manual_seed(rows), dtype=torch.float16).cuda()
        cpus = [synthetic_sage(k, n, seed=s) for n, s in shapes]
        layers = [SAGELinear(to_cuda(cpu), n) for cpu, (n, _) in zip(cpus, shapes)]
        problems = [(x, l.packed_codes, l.radius_codes, l.radius_grid, l.codebook, l.permutation) for l in layers]
        grouped = sage_grouped(problems, [n for n, _ in shapes])
        again = sage_grouped(problems, [n for n, _ in shapes])
        for cpu, (n, _), many, repeat, layer in zip(cpus, shapes, grouped, again, layers):
            assert_output(many, expected_output(x, cpu, n))
            assert torch.equal(many, repeat)
            single = layer(x)
            assert ((many.float() - single.float()).norm() / single.float().norm()).item() < 1e-3


@pytest.mark.parametrize("blocks", [(16, 8), (12, 12), (16, 16), (9, 8)])
def test_grouped_launch_of_row_blocks_with_given_outputs(blocks):
    """Row blocks of several linears in one grouped launch, written into row ranges of one output
    tensor per linear (`outputs=`).  Blocks of more than eight rows next to blocks of at most eight
    need different kernel shapes; the library then runs the group as two launches instead of
    failing.  Every output passes the oracle gate."""
    k = 2560
    shapes = [(4096, 0), (1024, 1), (1024, 2)]
    rows = sum(blocks)
    x = torch.randn(rows, k, generator=torch.Generator().manual_seed(rows), dtype=torch.float16).cuda()
    cpus = [synthetic_sage(k, n, seed=s) for n, s in shapes]
    layers = [SAGELinear(to_cuda(cpu), n) for cpu, (n, _) in zip(cpus, shapes)]
    outs = [torch.full((rows, n), float("nan"), dtype=torch.float16, device="cuda") for n, _ in shapes]
    problems, widths, targets = [], [], []
    for layer, (n, _), out in zip(layers, shapes, outs):
        first = 0
        for count in blocks:
            problems.append((x[first:first + count], layer.packed_codes, layer.radius_codes, layer.radius_grid,
                             layer.codebook, layer.permutation))
            widths.append(n)
            targets.append(out[first:first + count])
            first += count
    returned = sage_grouped(problems, widths, outputs=targets)
    assert all(r.data_ptr() == t.data_ptr() for r, t in zip(returned, targets))
    for cpu, (n, _), out in zip(cpus, shapes, outs):
        assert_output(out, expected_output(x, cpu, n))
    with pytest.raises(RuntimeError):
        sage_grouped(problems, widths, outputs=[t[:, :-1] for t in targets])


def test_tuning_knob_sweep_stays_within_tolerance():
    """Every launch geometry the knob can select gives the same answer within the gate."""
    lib = _lib.load()
    k, n = 4096, 2560
    cpu = synthetic_sage(k, n, seed=1)
    layer = SAGELinear(to_cuda(cpu), n)
    try:
        for rows in (1, 12):
            x = torch.randn(rows, k, generator=torch.Generator().manual_seed(3), dtype=torch.float16).cuda()
            want = expected_output(x, cpu, n)
            for warps, slices, ctas_per_sm, mode in [
                (1, 1, 1, 1), (8, 1, 2, 2), (4, 4, 2, 0), (3, 5, 4, 1), (16, 8, 1, 0), (2, 2, 8, 2),
                (5, 3, 1, 1), (16, 1, 1, 1), (16, 1, 1, 2), (7, 1, 3, 2),
            ]:
                assert lib.sageb200_set_tuning(warps, slices, ctas_per_sm, mode) == 0
                assert_output(layer(x), want)
    finally:
        lib.sageb200_set_tuning(0, 0, 0, 0)


def test_reference_cuda_kernels_agree_when_built():
    """If the reference project's own kernels were compiled (oracle/_ref), both
    implementations must agree within the output gate on the same inputs."""
    ref = c_oracle.reference_kernels()
    if ref is None:
        pytest.skip("oracle/_ref/libsage_ref.so not built on this machine")
    vp = ctypes.c_void_p
    stream = vp(torch.cuda.current_stream().cuda_stream)
    for (k, n, rows, seed) in [(2560, 9728, 1, 0), (4096, 2560, 4, 1), (2560, 1024, 15, 2), (9728, 2560, 1, 0)]:
        cpu = synthetic_sage(k, n, seed=seed)
        gpu = to_cuda(cpu)
        layer = SAGELinear(gpu, n)
        x = torch.randn(rows, k, generator=torch.Generator().manual_seed(5), dtype=torch.float16).cuda()
        ours = layer(x)
        fused = ref.sage_ref_fuses_permutation(n, k)
        xin = x if fused else x.index_select(-1, gpu["permutation"].long()).contiguous()
        theirs = torch.empty(rows, n, dtype=torch.float16, device="cuda")
        status = ref.sage_ref_gemv(
            vp(xin.data_ptr()), vp(gpu["packed_codes"].data_ptr()), vp(gpu["radius_codes"].data_ptr()),
            vp(gpu["radius_grid"].data_ptr()), vp(gpu["codebook"].data_ptr()), vp(theirs.data_ptr()),
            vp(gpu["permutation"].data_ptr()) if fused else None, rows, n, k, cpu["codebook"].shape[1], stream,
        )
        assert status == 0
        torch.cuda.synchronize()
        want = expected_output(x, cpu, n)
        assert_output(theirs, want)
        assert_output(ours, want)


@pytest.mark.parametrize("rows", [1, 5])
@pytest.mark.parametrize("permuted", [True, False])
def test_fused_producers_match_separate_kernels(rows, permuted):
    """Residual add + RMSNorm and SwiGLU fused into the grouped launch against the
    stand-alone glue kernels followed by the plain grouped launch."""
    lib = _lib.load()
    vp = ctypes.c_void_p
    stream = vp(torch.cuda.current_stream().cuda_stream)
    k = 2560
    gen = torch.Generator(device="cuda").manual_seed(rows)
    residual = torch.randn(rows, k, generator=gen, device="cuda").half()
    delta = torch.randn(rows, k, generator=gen, device="cuda").half()
    weight = (1 + 0.1 * torch.randn(k, generator=gen, device="cuda")).half()
    cpus = [synthetic_sage(k, n, seed=s, permuted=permuted) for n, s in [(1024, 0), (4096, 1)]]
    layers = [SAGELinear(to_cuda(cpu), n) for cpu, n in zip(cpus, (1024, 4096))]
    problem = lambda x: [(x, l.packed_codes, l.radius_codes, l.radius_grid, l.codebook, l.permutation) for l in layers]  # noqa: E731
    outs = [1024, 4096]
    # separate kernels
    h = residual.clone()
    x = torch.empty_like(h)
    assert lib.sageb200_glue_add_rmsnorm(vp(h.data_ptr()), vp(delta.data_ptr()), vp(weight.data_ptr()),
                                         vp(x.data_ptr()), rows, k, 1e-6, stream) == 0
    want = sage_grouped(problem(x), outs)
    # fused
    new_residual = torch.zeros_like(residual)
    got = sage_grouped(problem(residual), outs, (1, 1e-6, residual, delta, weight, new_residual))
    assert torch.equal(new_residual, h)
    for a, b in zip(got, want):
        assert ((a.float() - b.float()).norm() / b.float().norm()).item() < 1e-3
    got_none = sage_grouped(problem(residual), outs, (1, 1e-6, residual, None, weight, new_residual))
    assert torch.equal(new_residual, residual)
    assert all(torch.isfinite(t).all() for t in got_none)
    # SwiGLU
    gate = torch.randn(rows, k, generator=gen, device="cuda").half()
    up = torch.randn(rows, k, generator=gen, device="cuda").half()
    act = torch.empty_like(gate)
    assert lib.sageb200_glue_swiglu(vp(gate.data_ptr()), vp(up.data_ptr()), vp(act.data_ptr()), gate.numel(), stream) == 0
    want = sage_grouped(problem(act), outs)
    got = sage_grouped(problem(gate), outs, (2, 0.0, gate, up, None, None))
    for a, b in zip(got, want):
        assert ((a.float() - b.float()).norm() / b.float().norm()).item() < 1e-3


@pytest.mark.parametrize("k,n,rows", [(5120, 25600, 1), (5120, 25600, 5), (25600, 5120, 1), (25600, 2560, 2)])
def test_shares_larger_than_shared_memory_stream_through_rings(k, n, rows):
    """Qwen3-32B-sized matrices: a CTA's share no longer fits its shared memory and is streamed
    through per-warp rings (and through further waves of CTAs when that is switched off); both
    against an FP32 matmul on the kernel-made dense weight, and the fused producers on the same
    sizes against the separate kernels."""
    lib = _lib.load()
    gpu = to_cuda(synthetic_sage(k, n, seed=rows, permuted=True))
    layer = SAGELinear(gpu, n)
    weight = layer.dequantize().float()
    x = torch.randn(rows, k, generator=torch.Generator().manual_seed(k + rows), dtype=torch.float16).cuda()
    want = x.float() @ weight.T
    del weight
    streamed = layer(x)
    assert_output(streamed, want)
    assert torch.equal(layer(x), streamed)  # repeatable
    assert lib.sageb200_set_tuning(0, 0, 0, 3) == 0  # no rings: several waves of CTAs
    try:
        assert_output(layer(x), want)
    finally:
        assert lib.sageb200_set_tuning(0, 0, 0, 0) == 0
    if rows == 1:  # fused SwiGLU and fused residual add + RMSNorm feeding the same matrix
        vp = ctypes.c_void_p
        stream = vp(torch.cuda.current_stream().cuda_stream)
        gen = torch.Generator(device="cuda").manual_seed(n)
        problem = lambda t: [(t, layer.packed_codes, layer.radius_codes, layer.radius_grid, layer.codebook,  # noqa: E731
                              layer.permutation)]
        gate = torch.randn(1, k, generator=gen, device="cuda").half()
        up = torch.randn(1, k, generator=gen, device="cuda").half()
        act = torch.empty_like(gate)
        assert lib.sageb200_glue_swiglu(vp(gate.data_ptr()), vp(up.data_ptr()), vp(act.data_ptr()), gate.numel(),
                                        stream) == 0
        (plain,) = sage_grouped(problem(act), [n])
        (fused,) = sage_grouped(problem(gate), [n], (2, 0.0, gate, up, None, None))
        assert ((fused.float() - plain.float()).norm() / plain.float().norm()).item() < 1e-3
        if k > 24576:  # wider than the stand-alone norm kernel takes (no model norms such a row)
            return
        norm_weight = (1 + 0.1 * torch.randn(k, generator=gen, device="cuda")).half()
        h, normed, new_residual = gate.clone(), torch.empty_like(gate), torch.zeros_like(gate)
        assert lib.sageb200_glue_add_rmsnorm(vp(h.data_ptr()), vp(up.data_ptr()), vp(norm_weight.data_ptr()),
                                             vp(normed.data_ptr()), 1, k, 1e-6, stream) == 0
        (plain,) = sage_grouped(problem(normed), [n])
        (fused,) = sage_grouped(problem(gate), [n], (1, 1e-6, gate, up, norm_weight, new_residual))
        assert torch.equal(new_residual, h)
        assert ((fused.float() - plain.float()).norm() / plain.float().norm()).item() < 1e-3


# ---------------------------------------------------------------- tcgen05 GEMM on real grids


def _gemm_case(k, n, rows, seed, permuted, bits=None):
    kwargs = {} if bits is None else {"direction_bits": bits}
    cpu = synthetic_sage(k, n, seed=seed, permuted=permuted, **kwargs)
    layer = SAGELinear(to_cuda(cpu), n)
    x = torch.randn(rows, k, generator=torch.Generator().manual_seed(rows + n), dtype=torch.float16).cuda()
    return cpu, layer, x


@pytest.mark.parametrize("rows", [33, 257, 300, 513])
@pytest.mark.parametrize("k,n", [(256, 129), (640, 1025), (2560, 1024), (1280, 2560)])
@pytest.mark.parametrize("permuted", [False, True])
def test_gemm_multi_cta_grids_against_oracle(rows, k, n, permuted):
    """The tensor-core path on grids of several 128-row blocks and several token blocks
    (rows > 256), N not a multiple of 128 and rows not a multiple of 16, against the C
    oracle's FP16 weights."""
    cpu, layer, x = _gemm_case(k, n, rows, seed=rows % 3, permuted=permuted)
    assert_output(layer(x), expected_output(x, cpu, n))


@pytest.mark.parametrize("bits", [6, 7, 8])
@pytest.mark.parametrize("k,n", [(2560, 9728), (9728, 2560), (4096, 2560), (2560, 1024)])
def test_gemm_qwen3_4b_shapes_against_oracle(k, n, bits):
    """Prompt-sized row counts on the Qwen3-4B shapes, every bit split, against the oracle."""
    cpu = synthetic_sage(k, n, seed=200 + bits, permuted=True, direction_bits=bits)
    layer = SAGELinear(to_cuda(cpu), n)
    weight = torch.from_numpy(c_oracle.decode_fp16(cpu, n)).cuda().float()
    for rows in (33, 257, 512, 2048):
        x = torch.randn(rows, k, generator=torch.Generator().manual_seed(rows), dtype=torch.float16).cuda()
        assert_output(layer(x), x.float() @ weight.T)


def test_gemm_qwen3_32b_gate_at_2048_rows():
    """5120 -> 25600 at 2048 rows: an FP32 matmul on the kernel-made dense weight (pinned bit
    for bit against the reference decoder by the hash tests) keeps the host time down."""
    k, n, rows = 5120, 25600, 2048
    gpu = to_cuda(synthetic_sage(k, n, seed=4, permuted=True))
    layer = SAGELinear(gpu, n)
    x = torch.randn(rows, k, generator=torch.Generator().manual_seed(9), dtype=torch.float16).cuda()
    got = layer(x)
    weight = layer.dequantize().float()
    for begin in range(0, rows, 512):  # in slices: the FP32 product of the whole is 210 MB
        assert_output(got[begin : begin + 512], x[begin : begin + 512].float() @ weight.T)


@pytest.mark.parametrize("rows", [300, 513])
def test_gemm_one_hot_rows_across_token_blocks(rows):
    """x[m] = e_(m mod K) picks weight column (m mod K) for token m: a wrong token-block offset,
    TMA coordinate or store guard fails element by element, not only in norm."""
    k, n = 512, 200
    cpu = synthetic_sage(k, n, seed=2, permuted=True)
    layer = SAGELinear(to_cuda(cpu), n)
    weight = torch.from_numpy(c_oracle.decode_fp16(cpu, n)).cuda()
    x = torch.zeros(rows, k, dtype=torch.float16, device="cuda")
    columns = torch.arange(rows, device="cuda") * 7 % k
    x[torch.arange(rows, device="cuda"), columns] = 1.0
    got = layer(x)
    want = weight[:, columns].T.float()
    assert torch.allclose(got.float(), want, rtol=2e-3, atol=1e-6)


def test_gemm_maximum_rows_and_split_k_repeatability():
    """65535 activation rows (the interface's maximum: 256 token blocks) checked at the first, a
    middle and the last rows through the one-hot property, one more row refused; and a shape whose
    K is split over several CTAs per tile gives the same bits on every call (the splits are added in
    index order whoever arrives last)."""
    k, n = 256, 129
    cpu = synthetic_sage(k, n, seed=5, permuted=True)
    layer = SAGELinear(to_cuda(cpu), n)
    weight = torch.from_numpy(c_oracle.decode_fp16(cpu, n)).cuda().float()
    rows = 65535
    x = torch.zeros(rows, k, dtype=torch.float16, device="cuda")
    columns = torch.arange(rows, device="cuda") * 5 % k
    x[torch.arange(rows, device="cuda"), columns] = 1.0
    got = layer(x)
    for block in (slice(0, 300), slice(32700, 33000), slice(rows - 300, rows)):
        assert torch.allclose(got[block].float(), weight[:, columns[block]].T, rtol=2e-3, atol=1e-6)
    with pytest.raises(RuntimeError):
        layer(torch.zeros(rows + 1, k, dtype=torch.float16, device="cuda"))
    del x, got
    # K split: 9728 -> 2560 at 512 rows runs six CTAs per output tile
    cpu = synthetic_sage(9728, 2560, seed=6, permuted=True)
    layer = SAGELinear(to_cuda(cpu), 2560)
    x = torch.randn(512, 9728, generator=torch.Generator().manual_seed(7), dtype=torch.float16).cuda()
    first = layer(x).clone()
    for _ in range(5):
        assert torch.equal(layer(x), first)
    assert_output(first, expected_output(x, cpu, 2560))


# ---------------------------------------------------------------- traceability (torch.compile)


@pytest.mark.parametrize("k,n", [(2560, 4096), (2560, 9728), (4096, 2560), (9728, 2560)])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_compiled_module_matches_oracle(k, n, seed):
    """`torch.compile(fullgraph=True, mode="reduce-overhead")` traces through the operator's fake
    kernel and replays it under Inductor's CUDA graphs (reference tests/inference/test_sage.py:
    135-151: the four Qwen3-4B shapes, three seeds, three input scales)."""
    torch.compiler.reset()
    cpu = synthetic_sage(k, n, seed=seed)
    layer = SAGELinear(to_cuda(cpu), n)
    weight = torch.from_numpy(c_oracle.decode_fp16(cpu, n)).cuda().float()
    compiled = torch.compile(layer, fullgraph=True, dynamic=False, mode="reduce-overhead")
    x = torch.randn(1, k, generator=torch.Generator().manual_seed(43), dtype=torch.float16).cuda()
    try:
        for scale in (0.03125, 1.0, 32.0):
            scaled = x * scale
            for _ in range(3):  # warm-up, capture, replay
                got = compiled(scaled).clone()
            assert_output(got, scaled.float() @ weight.T)
            assert torch.equal(got, layer(scaled))
    finally:
        torch.compiler.reset()


def test_compiled_module_with_rows_and_bias():
    """The plain `fullgraph` compile of the module at several rows (decode kernel and tensor-core
    GEMM), with a bias (reference tests/inference/test_sage.py:187-191)."""
    torch.compiler.reset()
    cpu = synthetic_sage(256, 17, seed=1)
    layer = SAGELinear(to_cuda(cpu), 17, bias=torch.ones(17, device="cuda", dtype=torch.float16))
    compiled = torch.compile(layer, fullgraph=True)
    try:
        for rows in (2, 65):
            x = torch.randn(rows, 256, device="cuda", dtype=torch.float16)
            assert_output(compiled(x) - 1, expected_output(x, cpu, 17))
    finally:
        torch.compiler.reset()
