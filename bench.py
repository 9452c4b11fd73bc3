"""Benchmark of the SAGE packed-weight decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode_model|decode_linears|prompt|tp32b|ep30b|report|linear:K:N:M|sph:K:N:M|
                               gemm_roles:K:N:M|skinny_phases:K:N:M|mega_phases] [--prompt P]

A step is one decoded token of the full Qwen3-4B architecture at batch 1 (synthetic seeded
packed weights, ABS split cycling 6/7/8 direction bits per matrix; `decode_linears` times the
252 packed matmuls of a step alone).  Rank 0 prints ONE
JSON line.  `value` is whole-job tok/s with everything resident in HBM, timed with CUDA
events around K CUDA-graph replays; `e2e` is the same through the public module API with
the step's input copied from pinned host memory and its result read back every step.

`--impl reference` times the reference's CPU path for the same workload (dequantise,
round to FP16, FP32 matmul - tests/inference/reference.py:39-49 and
tests/inference/test_sage.py:113-122 in the reference project) on the host cores, using
this repo's C restatement of it (oracle/), one decoder layer per step.

Multi-GPU (`--gpus N` under torchrun): the decode path has no cross-sequence exchange, so
every rank decodes its own sequence with its own copy of the weights (weak scaling, no
collective on the data path); the timed region is bracketed by barriers and the slowest
rank's time is used.
"""

from __future__ import annotations

import argparse
import json
import os
import pathlib
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "qwen3_4b_sage_2.25bpw_batch1_decode_tok_s"
UNIT = "tok/s"

# Qwen3-4B decoder layer, (name, in K, out N), in execution order
QWEN3_4B_LAYERS = 36
QWEN3_4B_LINEARS = [
    ("q_proj", 2560, 4096),
    ("k_proj", 2560, 1024),
    ("v_proj", 2560, 1024),
    ("o_proj", 4096, 2560),
    ("gate_proj", 2560, 9728),
    ("up_proj", 2560, 9728),
    ("down_proj", 9728, 2560),
]


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def all_peaks() -> dict:
    """HBM copy GB/s and dense BF16 TFLOP/s (burst) of this pool's B200s, measured where the
    file exists, else the earlier measurement used as the stated fallback."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data.get("bf16_tflops", 1590.0)), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, index: int):
        self.index = index
        self.process = None
        self.lines: list[str] = []
        self.thread = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _pump(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        return False

    def summary(self) -> dict:
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                maxima.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        clocks.sort()
        return {
            "sm_mhz": clocks[len(clocks) // 2],
            "sm_max_mhz": max(maxima),
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


# ------------------------------------------------------------------ reference (CPU) arm


_CPU_LAYER = None
_CPU_HEAD = None
QWEN3_4B_VOCAB = 151936


def decode_workload_text(prompt_length: int) -> str:
    """The default workload in words; both arms print it."""
    return (f"Qwen3-4B (36 layers, hidden 2560, 32/8 heads, inter 9728, vocab 151936), "
            f"random-init, all 252 linears SAGE-packed (2.25 bpw), FP16 KV cache, batch 1, "
            f"greedy decode after a {prompt_length}-token prompt; one step = one token "
            f"(packed linears + norms + RoPE + attention + lm_head + argmax, one CUDA graph)")


def cpu_layer_seconds(repeats: int, threads: int) -> tuple[float, int]:
    """Best time of the reference CPU path over one Qwen3-4B decoder layer at batch 1."""
    import torch

    from oracle import c_oracle
    from sage_b200.synthetic import synthetic_sage

    cores = threads if threads > 0 else (os.cpu_count() or 1)
    global _CPU_LAYER
    if _CPU_LAYER is None:
        _CPU_LAYER = []
        for index, (_, k, n) in enumerate(QWEN3_4B_LINEARS):
            packed = synthetic_sage(k, n, seed=index, permuted=True)
            x = torch.randn(1, k, generator=torch.Generator().manual_seed(43), dtype=torch.float16)
            _CPU_LAYER.append((x, packed, n))
    layer = _CPU_LAYER
    best = float("inf")
    for _ in range(repeats):
        begin = time.perf_counter()
        for x, packed, n in layer:
            c_oracle.linear_fp32(x, packed, n, threads=cores)
        best = min(best, time.perf_counter() - begin)
    return best, cores


def cpu_head_seconds(repeats: int, threads: int) -> float:
    """Best time of the token's unpacked tail on the host cores: the 151936 x 2560 lm_head
    product and the argmax (torch, FP32 copy of the FP16 matrix, all threads)."""
    import torch

    global _CPU_HEAD
    if threads > 0:
        torch.set_num_threads(threads)
    if _CPU_HEAD is None:
        gen = torch.Generator().manual_seed(7)
        head = (torch.randn(QWEN3_4B_VOCAB, 2560, generator=gen) * 0.02).half().float()
        x = torch.randn(2560, generator=gen).half().float()
        _CPU_HEAD = (head, x)
    head, x = _CPU_HEAD
    best = float("inf")
    for _ in range(repeats):
        begin = time.perf_counter()
        int(torch.argmax(torch.mv(head, x)))
        best = min(best, time.perf_counter() - begin)
    return best


def cpu_token_rate(layer_seconds: float, head_seconds: float) -> float:
    """Tokens per second of the CPU path: 36 decoder layers' packed linears plus the lm_head."""
    return 1.0 / (layer_seconds * QWEN3_4B_LAYERS + head_seconds)


CPU_SAMPLE = ("packed linears of one decoder layer (7 matmuls, M=1, dequantise + FP32 product) timed and scaled by "
              "36 layers, plus the FP16 lm_head product and argmax timed once per token; norms, RoPE and "
              "attention over the cache are not included (they favour the CPU number)")


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    for _ in range(max(args.warmup, 1)):
        cpu_layer_seconds(1, cores)
        cpu_head_seconds(1, cores)
    begin = time.perf_counter()
    times = [(cpu_layer_seconds(1, cores)[0], cpu_head_seconds(1, cores)) for _ in range(args.steps)]
    wall = time.perf_counter() - begin
    layer_seconds = sum(t[0] for t in times) / len(times)
    head_seconds = sum(t[1] for t in times) / len(times)
    value = cpu_token_rate(layer_seconds, head_seconds)
    prompt_length = args.prompt if args.prompt else 512
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": 1000.0 * wall / args.steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f16 weights, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": decode_workload_text(prompt_length), "prompt_tokens": prompt_length,
                   "parallelism": "host cores of rank 0",
                   "note": "the reference's CPU implementation of the path (dequantise, FP32 matmul: "
                           "tests/inference/reference.py:25-49) restated in C with OpenMP (oracle/); each step "
                           "times a bounded sample of one token: " + CPU_SAMPLE,
                   "ms_per_token_estimate": 1000.0 / value},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": CPU_SAMPLE},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ our arm


def build_decode_linears(device):
    """All 252 packed linears of Qwen3-4B with fixed FP16 inputs; returns modules and bytes."""
    import torch

    from sage_b200 import SAGELinear
    from sage_b200.synthetic import linear_algorithmic_bytes, synthetic_sage_device

    layers, total_bytes = [], 0
    seed = 0
    for _ in range(QWEN3_4B_LAYERS):
        modules = []
        for _, k, n in QWEN3_4B_LINEARS:
            packed = synthetic_sage_device(k, n, seed, device, permuted=True)
            modules.append(SAGELinear(packed, n))
            total_bytes += linear_algorithmic_bytes(1, n, k, packed["codebook"].shape[1], True)
            seed += 1
        layers.append(modules)
    gen = torch.Generator(device=device).manual_seed(43)
    inputs = {
        2560: torch.randn(1, 2560, generator=gen, device=device, dtype=torch.float16),
        4096: torch.randn(1, 4096, generator=gen, device=device, dtype=torch.float16),
        9728: torch.randn(1, 9728, generator=gen, device=device, dtype=torch.float16),
    }
    return layers, inputs, total_bytes



def time_linear(k: int, n: int, rows: int, device, steps: int = 5, reference: bool = False):
    """Microseconds per call of one packed-linear shape on cold weights: enough distinct weight
    copies to exceed L2, all copies back to back in ONE CUDA graph, CUDA events around `steps`
    replays.  `reference`: the reference project's own kernels compiled for sm_100a
    (oracle/_ref/libsage_ref.so, dispatch of csrc/bindings.cpp:49-76) instead of this library;
    None when that comparator was not built."""
    import ctypes

    import torch

    from sage_b200 import SAGELinear
    from sage_b200.synthetic import linear_algorithmic_bytes, synthetic_sage_device

    one = linear_algorithmic_bytes(rows, n, k, 256, True)
    copies = max(2, int(200e6 // one) + 1)
    layers = [SAGELinear(synthetic_sage_device(k, n, 3 * i, device, direction_bits=8), n) for i in range(copies)]
    x = torch.randn(rows, k, device=device, dtype=torch.float16)
    if reference:
        from oracle import c_oracle  # the comparator lives with the checker code

        ref = c_oracle.reference_kernels()
        if ref is None:
            return None
        vp = ctypes.c_void_p
        sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        fused = rows < 16 and ref.sage_ref_fuses_permutation(n, k)
        parts = ref.sage_ref_gemm_splits(rows, n, k, sm_count) if rows >= 16 else 1
        workspace = torch.empty(max(parts * rows * n, 1), dtype=torch.float32, device=device)
        out = torch.empty(rows, n, dtype=torch.float16, device=device)

        def call(layer):
            stream = vp(torch.cuda.current_stream(device).cuda_stream)
            # (the reference gathers with index_select when its kernel does not fuse the permutation)
            xin = x if fused else x.index_select(-1, layer.permutation.long())
            common = (vp(xin.data_ptr()), vp(layer.packed_codes.data_ptr()), vp(layer.radius_codes.data_ptr()),
                      vp(layer.radius_grid.data_ptr()), vp(layer.codebook.data_ptr()), vp(out.data_ptr()))
            if rows < 16:
                ref.sage_ref_gemv(*common, vp(layer.permutation.data_ptr()) if fused else None, rows, n, k, 256, stream)
            else:
                ref.sage_ref_gemm(*common, vp(workspace.data_ptr()), parts, rows, n, k, 256, stream)
    else:
        def call(layer):
            layer(x)

    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        for layer in layers:
            call(layer)
    torch.cuda.current_stream(device).wait_stream(side)
    torch.cuda.synchronize(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for layer in layers:
            call(layer)
    for _ in range(3):
        graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        graph.replay()
    stop.record()
    torch.cuda.synchronize(device)
    return {"us": start.elapsed_time(stop) * 1000.0 / (steps * copies), "bytes": one, "copies": copies}


def kernel_records(device, peaks: dict) -> dict:
    """The per-kernel figures the headline line carries beside the model number: the batch-1
    GEMV and a 16-row decode call on the Qwen3-4B gate_proj shape (HBM roofline), the prompt GEMM
    on two shapes (tensor roofline, activation gather included), and the reference project's own
    kernels on the same inputs where that comparator was built."""
    hbm, tensor = peaks["hbm_gbs"], peaks["bf16_tflops"]
    records = {}
    for name, (k, n, rows) in {"gemv_2560x9728_m1": (2560, 9728, 1), "gemv_9728x2560_m1": (9728, 2560, 1),
                               "skinny_2560x9728_m16": (2560, 9728, 16)}.items():
        ours = time_linear(k, n, rows, device)
        theirs = time_linear(k, n, rows, device, reference=True)
        gbs = ours["bytes"] / ours["us"] / 1e3
        records[name] = {"us": round(ours["us"], 3), "gb_s": round(gbs, 1), "frac_of_hbm_peak": round(gbs / hbm, 4),
                         "reference_kernel_us": round(theirs["us"], 3) if theirs else None}
    for name, (k, n, rows) in {"gemm_2560x9728_m512": (2560, 9728, 512), "gemm_5120x25600_m2048": (5120, 25600, 2048)}.items():
        ours = time_linear(k, n, rows, device, steps=3)
        theirs = time_linear(k, n, rows, device, steps=3, reference=True)
        tflops = 2.0 * rows * k * n / ours["us"] / 1e6
        records[name] = {"us": round(ours["us"], 2), "tflop_s": round(tflops, 1),
                         "frac_of_tensor_peak": round(tflops / tensor, 4), "gather_pass_included": True,
                         "reference_kernel_us": round(theirs["us"], 2) if theirs else None}
    return records

def run_single_linear(args) -> None:
    """`--workload linear:K:N:M` - one packed-linear shape cycled over enough distinct weight
    copies to exceed L2, one CUDA graph of all copies per step.  This is the small case used for
    profiler captures; it prints achieved GB/s (algorithmic bytes per call / time per call)."""
    import torch

    from sage_b200 import SAGELinear, _lib
    from sage_b200.synthetic import linear_algorithmic_bytes, synthetic_sage_device

    _, k, n, rows = args.workload.split(":")
    k, n, rows = int(k), int(n), int(rows)
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    lib = _lib.load()
    one = linear_algorithmic_bytes(rows, n, k, 256, True)
    copies = max(2, int(200e6 // one) + 1)
    layers = [SAGELinear(synthetic_sage_device(k, n, 3 * i, device, direction_bits=8), n) for i in range(copies)]
    x = torch.randn(rows, k, device=device, dtype=torch.float16)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(max(args.warmup, 1)):
            for layer in layers:
                layer(x)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()  # all copies back to back, no host launch cost in the timing
    before = lib.sageb200_launch_count()
    with torch.cuda.graph(graph):
        for layer in layers:
            layer(x)
    per_replay = lib.sageb200_launch_count() - before
    graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    launches = per_replay * args.steps
    seconds = start.elapsed_time(stop) / 1000.0 / (args.steps * copies)
    peak, kind = measured_peaks()
    print(json.dumps({
        "metric": "sage_linear_hbm_gbs", "value": one / seconds / 1e9, "unit": "GB/s",
        "config": {"workload": args.workload, "copies": copies, "launch": "one CUDA graph of all copies"},
        "us_per_call": seconds * 1e6, "bytes_per_call": one, "frac": one / seconds / 1e9 / peak,
        "peak_kind": f"of {kind}", "gpu_launches": int(launches),
    }), flush=True)


def run_sph_linear(args) -> None:
    """`--workload sph:K:N:M` - one SPHQuant 64/4 shape (the `wvq::sphquant` kernel) cycled over
    enough distinct weight copies to exceed L2, one CUDA graph of all copies per step."""
    import torch

    from sage_b200 import SPHQuantLinear, synthetic_sphquant
    from sage_b200.synthetic import sph_algorithmic_bytes

    _, k, n, rows = args.workload.split(":")
    k, n, rows = int(k), int(n), int(rows)
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    one = sph_algorithmic_bytes(rows, n, k)
    copies = max(2, int(200e6 // one) + 1)
    layers = [SPHQuantLinear({key: t.to(device) for key, t in synthetic_sphquant(k, n, i).items()}) for i in range(copies)]
    x = torch.randn(rows, k, device=device, dtype=torch.float16)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for layer in layers:
            layer(x)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for layer in layers:
            layer(x)
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    passes = (rows + 7) // 8
    seconds = start.elapsed_time(stop) / 1000.0 / (args.steps * copies)
    peak, kind = measured_peaks()
    print(json.dumps({
        "metric": "sphquant_linear_hbm_gbs", "value": one / seconds / 1e9, "unit": "GB/s",
        "config": {"workload": args.workload, "copies": copies, "launch": "one CUDA graph of all copies"},
        "us_per_call": seconds * 1e6, "bytes_per_call": one, "frac": one / seconds / 1e9 / peak,
        "peak_kind": f"of {kind}", "gpu_launches": int(args.steps * copies * passes),
    }), flush=True)


def run_model(args) -> None:
    """Default workload: full Qwen3-4B, random-init, every linear SAGE-packed, batch 1,
    greedy decoding after a `--prompt`-token prompt (BASELINE.json configs[2])."""
    import torch
    import torch.distributed as dist

    from sage_b200 import _lib
    from sage_b200.qwen3 import QWEN3_4B, PackedQwen3

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: sage_b200 has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    lib = _lib.load()
    warmup = max(args.warmup, 3)
    prompt_length = args.prompt
    model = PackedQwen3(QWEN3_4B, device, seed=rank, max_seq=prompt_length + 2 * (args.steps + warmup) + 64,
                        batch=1, max_new=2 * (args.steps + warmup) + 16)
    model.capture()
    prompt = torch.randint(3, QWEN3_4B.vocab, (1, prompt_length),
                           generator=torch.Generator().manual_seed(1000 + rank))
    model.prefill(prompt)  # warm-up of the prompt path (tensor-core GEMM plans, tensor maps)
    torch.cuda.synchronize()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    model.prefill(prompt)
    p1.record()
    torch.cuda.synchronize()
    prefill_ms = p0.elapsed_time(p1)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        model.graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local) as sampler:
        start.record()
        for _ in range(args.steps):
            model.graph.replay()
        stop.record()
        barrier()
        elapsed_ms = start.elapsed_time(stop)
        if elapsed_ms < 1500:  # keep the GPU under the same load long enough for several clock samples
            hold = model.positions.clone()
            for _ in range(int((1500 - elapsed_ms) / max(elapsed_ms / args.steps, 1e-3))):
                model.positions.copy_(hold)  # stay inside the KV cache
                model.graph_no_head.replay()
            model.positions.copy_(hold)
            torch.cuda.synchronize()
    clocks = sampler.summary()
    context = prompt_length + warmup + args.steps // 2

    # the packed-linear kernels alone, live in this process: a graph of only the model's
    # SAGE launches (same weights, fixed inputs), timed with CUDA events
    inputs = {}
    def sage_only():
        for layer in model.layers:
            for names in (("q", "k", "v"), ("o",), ("gate", "up"), ("down",)):
                k = layer[names[0]].k
                if k not in inputs:
                    inputs[k] = torch.randn(1, k, device=device, dtype=torch.float16)
                model._linears(layer, names, inputs[k])
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        sage_only()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    sage_graph = torch.cuda.CUDAGraph()
    before = lib.sageb200_launch_count()
    with torch.cuda.graph(sage_graph):
        sage_only()
    sage_launches = lib.sageb200_launch_count() - before
    for _ in range(3):
        sage_graph.replay()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(20):
        sage_graph.replay()
    k1.record()
    torch.cuda.synchronize()
    sage_seconds = k0.elapsed_time(k1) / 1000.0 / (20 * sage_launches)

    # end to end through the public generation loop: token id from pinned host memory in,
    # next token read back on the host, every step
    host_token = torch.zeros(1, dtype=torch.int64).pin_memory()
    host_next = torch.zeros(1, dtype=torch.int64).pin_memory()
    host_token.copy_(model.tokens)
    for _ in range(3):
        model.tokens.copy_(host_token, non_blocking=True)
        model.graph.replay()
        host_next.copy_(model.tokens, non_blocking=True)
        torch.cuda.synchronize()
        host_token.copy_(host_next)
    barrier()
    e2e_begin = time.perf_counter()
    for _ in range(args.steps):
        model.tokens.copy_(host_token, non_blocking=True)
        model.graph.replay()
        host_next.copy_(model.tokens, non_blocking=True)
        torch.cuda.synchronize()
        host_token.copy_(host_next)
    e2e_ms = 1000.0 * (time.perf_counter() - e2e_begin)
    barrier()

    times = torch.tensor([elapsed_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = (float(v) for v in times.tolist())
    # figures that explain the headline, measured in this same process (rank 0's GPU)
    kernels, batch8, sharded = None, None, None
    packed_bytes, launches_per_step = model.packed_bytes, (model.sage_launches_per_step, model.glue_launches_per_step)
    step_bytes = model.bytes_per_token(context)
    del model, sage_graph
    torch.cuda.empty_cache()
    if rank == 0 and not args.quick:
        kernels = kernel_records(device, all_peaks())
        many = PackedQwen3(QWEN3_4B, device, seed=0, max_seq=160, batch=8, max_new=96)
        many.capture()
        many.prefill(torch.randint(3, QWEN3_4B.vocab, (8, 64), generator=torch.Generator().manual_seed(5)))
        for _ in range(3):
            many.graph.replay()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(32):
            many.graph.replay()
        b1.record()
        torch.cuda.synchronize()
        batch8 = {"ms_per_step": b0.elapsed_time(b1) / 32, "tok_s": 8 * 32 * 1000.0 / b0.elapsed_time(b1),
                  "note": "Qwen3-4B, 8 sequences decoded together after 64-token prompts, one CUDA graph per step"}
        del many
        torch.cuda.empty_cache()
    if world > 1 and not args.quick:
        # the sharded configurations in the same job: tensor parallel (Qwen3-32B shape) and expert
        # parallel (Qwen3-30B-A3B shape) over all ranks, and rank 0's own one-GPU runs of the same
        # models for the strong-scaling efficiency
        cpu_group = dist.new_group(backend="gloo")
        sharded = {}
        for kind, batch in (("tp32b", 1), ("ep30b", 1), ("ep30b", 32)):
            # (a sub-record that fails is reported as such; the headline line is printed either way)
            many_gpus, one_gpu, failure = None, None, None
            try:
                many_gpus = measure_sharded(kind, args, device, dist.group.WORLD, cpu_group, world, rank, batch=batch)
                torch.cuda.synchronize()
            except Exception as error:  # noqa: BLE001
                failure = f"{type(error).__name__}: {error}"
            dist.barrier(group=cpu_group)
            if rank == 0 and failure is None:
                try:
                    one_gpu = measure_sharded(kind, args, device, None, None, 1, 0, batch=batch)
                except Exception as error:  # noqa: BLE001
                    failure = f"one-GPU run: {type(error).__name__}: {error}"
            dist.barrier(group=cpu_group)
            if rank == 0:
                if failure is None:
                    many_gpus["one_gpu_tok_s"] = one_gpu["value"]
                    many_gpus["one_gpu_ms_per_step"] = one_gpu["ms_per_step"]
                    many_gpus["strong_scaling_efficiency"] = many_gpus["value"] / one_gpu["value"] / world
                    sharded[f"{kind}_batch{batch}"] = many_gpus
                else:
                    sharded[f"{kind}_batch{batch}"] = {"error": failure[:300]}
    if rank == 0:
        ms_per_step = elapsed_ms / args.steps
        peak, peak_kind = measured_peaks()
        achieved = (packed_bytes / sage_launches) / sage_seconds / 1e9
        cpu_seconds, cores = cpu_layer_seconds(3, 0)
        cpu_head = cpu_head_seconds(3, 0)
        line = {
            "metric": METRIC,
            "value": world * 1000.0 / ms_per_step,
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": warmup,
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f16 products, f32 accumulate",
            "data": "synthetic",
            "config": {
                "workload": decode_workload_text(prompt_length),
                "prompt_tokens": prompt_length,
                "prefill_ms": prefill_ms,
                "prefill_note": "whole prompt through each layer at once (packed linears on the tcgen05 GEMM "
                                "path), first token included; not part of the timed decode steps",
                "context_at_midpoint": context,
                "step_hbm_bytes": step_bytes,
                "step_hbm_gbs": step_bytes / (ms_per_step / 1000.0) / 1e9,
                "kernels_per_step": {"sage_linear": int(launches_per_step[0]), "glue": int(launches_per_step[1])},
                "timed_steps_note": f"{args.steps} consecutive decode steps timed (the configuration's 256-token "
                                    "generation is a matter of --steps 256); the context grows by one position per step",
                "l2_policy": "inputs larger than L2: 1.92 GB of weights stream per step",
                "parallelism": f"replicas x{world}" if world > 1 else "single GPU",
            },
            "roofline": {
                "bound": "hbm",
                "achieved": achieved,
                "peak": peak,
                "unit": "GB/s",
                "frac": achieved / peak,
                # DRAM bytes per launch: the ncu capture of one gate_proj launch read 1.003 x its
                # algorithmic bytes and wrote none (profiles/); scaled to this graph's average launch
                "traffic": 1.003 * packed_bytes / sage_launches,
                "traffic_how": "ncu dram__bytes_read+write of one 2560->9728 M=1 launch = 1.003 x algorithmic, scaled by bytes",
                "kernel": "sage_skinny_kernel",
                "peak_kind": f"of {peak_kind}",
                "bytes_per_launch": packed_bytes / sage_launches,
                "us_per_launch": sage_seconds * 1e6,
                "how": "CUDA events around 20 replays of a graph holding only the model's packed-linear launches",
            },
            "kernels": kernels,
            "decode_batch8": batch8,
            "sharded": sharded,
            "cpu_baseline": {
                "value": cpu_token_rate(cpu_seconds, cpu_head),
                "unit": UNIT,
                "cores": cores,
                "kind": "port",
                "sample": CPU_SAMPLE + " (best of 3)",
            },
            "e2e": {
                "value": world * 1000.0 * args.steps / e2e_ms,
                "unit": UNIT,
                "h2d_bytes_per_step": 8,
                "d2h_bytes_per_step": 8,
            },
            "gpu_launches": int((launches_per_step[0] + launches_per_step[1]) * args.steps),
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        if sharded is None:
            dist.destroy_process_group()
        else:  # no NCCL teardown under live CUDA graphs that captured collectives (see run_tp)
            sys.stdout.flush()
            dist.barrier(group=cpu_group)
            os._exit(0)


def run_report(args) -> None:
    """`--workload report`: Qwen3-4B, prompt `--prompt`, 256 generated tokens, measured and
    written in the reference benchmark's schema (JSON + CSV under `--output`, default ./reports)."""
    import torch

    from sage_b200.harness import measure, write_report
    from sage_b200.qwen3 import QWEN3_4B, PackedQwen3

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    decode = 256
    model = PackedQwen3(QWEN3_4B, device, seed=0, max_seq=args.prompt + decode + 16, batch=1, max_new=decode + 16)
    model.capture()
    prompt = torch.randint(3, QWEN3_4B.vocab, (1, args.prompt), generator=torch.Generator().manual_seed(0))
    result, rows = measure(model, prompt, decode, samples=max(3, min(args.steps, 10)), warmup=2)
    folder = pathlib.Path(args.output)
    path, csv_path = write_report(result, rows, folder, f"qwen3-4b-sage-prefill{args.prompt}-decode{decode}")
    print(json.dumps({"report": str(path), "csv": str(csv_path),
                      "rows": [[m, p, metric, round(value, 3), unit] for m, p, metric, value, unit in rows]}), flush=True)


def measure_sharded(kind: str, args, device, group, cpu_group, world: int, rank: int, batch: int = 1,
                    prompt_pass: bool = False):
    """One strong-scaling measurement: `kind` "tp32b" (Qwen3-32B shape, column/row tensor
    parallel, NCCL all-reduce) or "ep30b" (Qwen3-30B-A3B shape, expert parallel) on the ranks of
    `group` (None: this GPU alone), batch-`batch` greedy decode.  Returns the record of rank 0's
    line (every rank gets the timing fields)."""
    import torch
    import torch.distributed as dist

    from sage_b200.qwen3 import QWEN3_30B_A3B, QWEN3_32B, PackedQwen3

    expert_parallel = kind == "ep30b"
    config = QWEN3_30B_A3B if expert_parallel else QWEN3_32B
    sharded = group is not None and world > 1
    warmup = max(args.warmup, 3)
    prompt_length = min(args.prompt, 64)
    steps = args.steps
    # Expert parallelism beyond 16 sequences: every rank decodes its own share of the sequences and
    # the (token, expert) slots travel by all-to-all; up to 16 every rank decodes all of them and the
    # expert outputs are summed by all-reduce.  `batch` is the whole job's either way.
    exchange = expert_parallel and batch > 16
    local_batch = batch // world if exchange and sharded else batch
    # `prompt_pass` (the tp32b workload on its own): the dense-MLP model also times a 512-token prompt
    # pass; its longer KV cache costs the decode step a few per cent, so the default record leaves it out
    long_prompt = 512 if prompt_pass and not expert_parallel and batch == 1 else 0
    model = PackedQwen3(config, device, seed=0, max_seq=max(prompt_length + 2 * (steps + warmup), long_prompt) + 16,
                        batch=local_batch, max_new=2 * (steps + warmup) + 16,
                        tp_group=group if sharded and not expert_parallel else None,
                        perm_blocks=1 if expert_parallel else 8,
                        ep_group=group if sharded and expert_parallel else None,
                        ep_mode="all_to_all" if exchange else "all_reduce")
    model.capture()
    prompt = torch.randint(3, config.vocab, (local_batch, prompt_length),
                           generator=torch.Generator().manual_seed(7 + (rank if exchange else 0)))
    model.prefill(prompt)

    def barrier():
        torch.cuda.synchronize()
        if sharded:
            dist.barrier(group=cpu_group)
        torch.cuda.synchronize()

    for _ in range(warmup):
        model.graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(device.index) as sampler:
        start.record()
        for _ in range(steps):
            model.graph.replay()
        stop.record()
        barrier()
    clocks = sampler.summary()
    tokens = model.log[0, : warmup + steps + 1].tolist()
    # end to end: token ids from pinned host memory in, next tokens read back, every step
    host_token = torch.zeros(local_batch, dtype=torch.int64).pin_memory()
    host_next = torch.zeros(local_batch, dtype=torch.int64).pin_memory()
    host_token.copy_(model.tokens)
    barrier()
    e2e_begin = time.perf_counter()
    for _ in range(steps):
        model.tokens.copy_(host_token, non_blocking=True)
        model.graph.replay()
        host_next.copy_(model.tokens, non_blocking=True)
        torch.cuda.synchronize()
        host_token.copy_(host_next)
    e2e_ms = 1000.0 * (time.perf_counter() - e2e_begin)
    barrier()
    prompt_ms = 0.0
    if long_prompt:
        # a 512-token prompt pass of the same model (rows through the tcgen05 GEMM path; under tensor
        # parallelism the partial sums of o/down are reduced by the one-kernel all-reduce)
        long = torch.randint(3, config.vocab, (local_batch, long_prompt), generator=torch.Generator().manual_seed(11))
        model.prefill(long)
        barrier()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        model.prefill(long)
        end.record()
        barrier()
        prompt_ms = begin.elapsed_time(end)
    times = torch.tensor([start.elapsed_time(stop), e2e_ms, prompt_ms], dtype=torch.float64)
    if sharded:
        dist.all_reduce(times, op=dist.ReduceOp.MAX, group=cpu_group)
    ms_per_step = float(times[0]) / steps
    peak, peak_kind = measured_peaks()
    step_bytes = model.bytes_per_token(prompt_length + warmup + steps // 2)
    collective = "none"
    calls = 0
    if sharded and expert_parallel:
        collective = model.ep_collective
        calls = model.collective_calls_per_step
    elif sharded:
        collective, calls = model.tp_collective, 2 * config.layers + 1
    record = {
        "metric": ("qwen3_30b_a3b" if expert_parallel else "qwen3_32b") + f"_sage_2.25bpw_batch{batch}_decode_tok_s",
        "value": batch * 1000.0 / ms_per_step,
        "unit": UNIT,
        "n_gpus": world if sharded else 1,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": ms_per_step,
        "batch": batch,
        "parallelism": (f"ep{world}" if expert_parallel else f"tp{world}") if sharded else "single GPU",
        "collective": collective,
        "collective_note": getattr(model, "peer_error", "") or None,
        "collective_calls_per_step": calls,
        "prompt_pass_ms_512_tokens": float(times[2]) if long_prompt else None,
        "prompt_pass_batched": bool(long_prompt and (not sharded or model._tp_prompt_ok())) if long_prompt else None,
        "per_rank_hbm_bytes_per_step": step_bytes,
        "per_rank_hbm_gbs": step_bytes / (ms_per_step / 1000.0) / 1e9,
        "hbm_frac": step_bytes / (ms_per_step / 1000.0) / 1e9 / peak,
        "peak_kind": f"of {peak_kind}",
        "e2e_tok_s": batch * 1000.0 * steps / float(times[1]),
        "first_tokens": tokens[:8],
        "gpu_launches": int((model.sage_launches_per_step + model.glue_launches_per_step) * steps),
        "clocks": clocks,
    }
    del model
    torch.cuda.empty_cache()
    return record


def run_tp(args) -> None:
    """`--workload tp32b` / `ep30b`: the strong-scaling runs on their own (one sequence for the
    whole job).  Qwen3-32B shape: q/k/v/gate/up column-parallel, o/down row-parallel + NCCL
    all-reduce, vocabulary-parallel lm_head + all-gather.  Qwen3-30B-A3B shape: expert parallel."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    group = cpu_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD
        # Host-side barriers and the max-over-ranks reduction go through a gloo group: an eager
        # NCCL collective issued after NCCL collectives were captured into CUDA graphs did not
        # return on this software stack (seen with a 2-GPU run), a CPU group does.
        cpu_group = dist.new_group(backend="gloo")
    expert_parallel = args.workload == "ep30b"
    record = measure_sharded(args.workload, args, device, group, cpu_group, world, rank, batch=args.batch,
                             prompt_pass=True)
    if rank == 0:
        line = dict(record)
        line.update({
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 products, f32 accumulate", "data": "synthetic",
            "config": {
                "workload": ("Qwen3-30B-A3B shape (48 layers, hidden 2048, 32/4 heads, 128 experts top-8, "
                             "moe_inter 768), random-init, attention and expert linears SAGE-packed, FP16 router, "
                             "greedy decode, expert parallel (attention and router replicated, each rank runs its "
                             "block of experts)"
                             if expert_parallel else
                             "Qwen3-32B shape (64 layers, hidden 5120, 64/8 heads, inter 25600), random-init, "
                             "SAGE-packed, greedy decode, tensor parallel"),
                "parallelism": record["parallelism"], "batch": record["batch"],
                "row_parallel_permutation": "block permutation, 8 blocks (each rank gathers inside its slice)",
            },
            "e2e": {"value": record["e2e_tok_s"], "unit": UNIT, "h2d_bytes_per_step": 8 * record["batch"],
                    "d2h_bytes_per_step": 8 * record["batch"]},
        })
        print(json.dumps(line), flush=True)
    if world > 1:
        # leave without tearing the NCCL communicator down under live graphs (see above)
        dist.barrier(group=cpu_group)
        sys.stdout.flush()
        os._exit(0)


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from sage_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: sage_b200 has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    lib = _lib.load()

    layers, inputs, step_bytes = build_decode_linears(device)
    hidden = inputs[2560]

    def step(h):
        # the packed linears of one token, in execution order; inputs are fixed FP16
        # vectors of the right width (h feeds the first projections)
        out = None
        for modules in layers:
            q, k, v, o, gate, up, down = modules
            q(h)
            k(h)
            v(h)
            o(inputs[4096])
            gate(h)
            up(h)
            out = down(inputs[9728])
        return out

    # warm-up outside the graph (library init, workspace allocation), then capture
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step(hidden)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    before_capture = lib.sageb200_launch_count()
    with torch.cuda.graph(graph):
        result = step(hidden)
    launches_per_step = lib.sageb200_launch_count() - before_capture

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local) as sampler:
        start.record()
        for _ in range(args.steps):
            graph.replay()
        stop.record()
        barrier()
        elapsed_ms = start.elapsed_time(stop)
        if elapsed_ms < 400:  # keep the sampler alive long enough for a few samples
            extra = torch.cuda.Event(enable_timing=True)
            for _ in range(int(400 / max(elapsed_ms / args.steps, 1e-3))):
                graph.replay()
            extra.record()
            torch.cuda.synchronize()
    clocks = sampler.summary()

    # end to end: pinned host input -> device, the step, result -> host, every step
    host_in = hidden.cpu().pin_memory()
    host_out = torch.empty_like(result, device="cpu").pin_memory()
    for _ in range(3):
        hidden.copy_(host_in, non_blocking=True)
        graph.replay()
        host_out.copy_(result, non_blocking=True)
        torch.cuda.synchronize()
    barrier()
    e2e_begin = time.perf_counter()
    for _ in range(args.steps):
        hidden.copy_(host_in, non_blocking=True)
        graph.replay()
        host_out.copy_(result, non_blocking=True)
        torch.cuda.synchronize()
    e2e_ms = 1000.0 * (time.perf_counter() - e2e_begin)
    barrier()

    times = torch.tensor([elapsed_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = (float(v) for v in times.tolist())

    if rank == 0:
        ms_per_step = elapsed_ms / args.steps
        value = world * 1000.0 / ms_per_step
        peak, peak_kind = measured_peaks()
        launch_seconds = (elapsed_ms / 1000.0) / (args.steps * launches_per_step)
        achieved = (step_bytes / launches_per_step) / launch_seconds / 1e9
        cpu_seconds, cores = cpu_layer_seconds(3, 0)
        cpu_value = 1.0 / (cpu_seconds * QWEN3_4B_LAYERS)
        line = {
            "metric": METRIC,
            "value": value,
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f16 products, f32 accumulate",
            "data": "synthetic",
            "config": {
                "workload": "qwen3-4b batch-1 decode step, packed SAGE linears only "
                            "(36 layers x q,k,v,o,gate,up,down = 252 matmuls, M=1); "
                            "attention, norms and lm_head are not in this step",
                "packed_bytes_per_step": step_bytes,
                "l2_policy": "inputs larger than L2: 1.14 GB of packed weights per step",
                "parallelism": f"replicas x{world}" if world > 1 else "single GPU",
            },
            "roofline": {
                "bound": "hbm",
                "achieved": achieved,
                "peak": peak,
                "unit": "GB/s",
                "frac": achieved / peak,
                "traffic": None,
                "kernel": "sage_skinny_kernel",
                "peak_kind": f"of {peak_kind}",
                "bytes_per_launch": step_bytes / launches_per_step,
                "us_per_launch": launch_seconds * 1e6,
            },
            "cpu_baseline": {
                "value": cpu_value,
                "unit": UNIT,
                "cores": cores,
                "kind": "port",
                "sample": "one decoder layer (7 packed linears, M=1), best of 3, scaled by 36 layers",
            },
            "e2e": {
                "value": world * 1000.0 * args.steps / e2e_ms,
                "unit": UNIT,
                "h2d_bytes_per_step": host_in.numel() * 2,
                "d2h_bytes_per_step": host_out.numel() * 2,
            },
            "gpu_launches": int(launches_per_step * args.steps),
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_prompt(args) -> None:
    """`--workload prompt`: the batched prompt pass of Qwen3-4B (`--prompt` tokens through every
    layer at once: packed linears on the tcgen05 GEMM path, tensor-core causal attention, first
    token included), timed with CUDA events over `--steps` passes after `--warmup`."""
    import torch

    from sage_b200.qwen3 import QWEN3_4B, PackedQwen3

    device = torch.device("cuda", 0)
    model = PackedQwen3(QWEN3_4B, device, seed=0, max_seq=args.prompt + 16, max_new=8)
    model.capture()
    prompt = torch.randint(3, QWEN3_4B.vocab, (1, args.prompt), generator=torch.Generator().manual_seed(1))
    lib = model.lib
    for _ in range(max(args.warmup, 1)):
        model.prefill(prompt)
    torch.cuda.synchronize(device)
    before = lib.sageb200_launch_count() + lib.sageb200_glue_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        model.prefill(prompt)
    stop.record()
    torch.cuda.synchronize(device)
    ms = start.elapsed_time(stop) / args.steps
    print(json.dumps({
        "metric": "qwen3_4b_sage_2.25bpw_prompt_pass_ms", "value": ms, "unit": "ms", "higher_is_better": False,
        "prompt_tokens": args.prompt, "prompt_tok_s": args.prompt * 1000.0 / ms, "steps": args.steps,
        "warmup": args.warmup,
        "gpu_launches": int(lib.sageb200_launch_count() + lib.sageb200_glue_launch_count() - before),
        "config": {"workload": f"Qwen3-4B prompt pass, {args.prompt} tokens, batch 1, host-side reset and token "
                               "copy included"},
    }), flush=True)


def run_decode_batch(args) -> None:
    """`--workload decode_batch` with `--batch N` (2..64): N sequences of Qwen3-4B decoded together
    after `--prompt`-token prompts, one CUDA graph per step, timed with CUDA events over `--steps`
    steps after `--warmup`.  One more step runs between cudaProfilerStart/Stop, so a profiler
    started with its capture off records exactly one step."""
    import torch

    from sage_b200.qwen3 import QWEN3_4B, PackedQwen3

    device = torch.device("cuda", 0)
    batch = args.batch
    model = PackedQwen3(QWEN3_4B, device, seed=0, max_seq=args.prompt + args.steps + args.warmup + 8, batch=batch,
                        max_new=args.steps + args.warmup + 8)
    model.capture()
    model.prefill(torch.randint(3, QWEN3_4B.vocab, (batch, args.prompt), generator=torch.Generator().manual_seed(5)))
    lib = model.lib
    for _ in range(max(args.warmup, 1)):
        model.graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        model.graph.replay()
    stop.record()
    torch.cuda.synchronize(device)
    ms = start.elapsed_time(stop) / args.steps
    torch.cuda.profiler.start()
    model.graph.replay()
    torch.cuda.synchronize(device)
    torch.cuda.profiler.stop()
    print(json.dumps({
        "metric": "qwen3_4b_sage_2.25bpw_batched_decode_tok_s", "value": batch * 1000.0 / ms, "unit": "tok/s",
        "higher_is_better": True, "batch": batch, "ms_per_step": ms, "steps": args.steps, "warmup": args.warmup,
        "prompt_tokens": args.prompt,
        "kernels_per_step": {"sage_linear": model.sage_launches_per_step, "glue": model.glue_launches_per_step},
        "config": {"workload": f"Qwen3-4B, {batch} sequences decoded together after {args.prompt}-token prompts, "
                               "one CUDA graph per step"},
    }), flush=True)


def run_gemm_roles(args) -> None:
    """`--workload gemm_roles:K:N:M` (profiling build of the library only: SAGEB200_LIBRARY =
    libsage_b200_trace.so): one tcgen05 GEMM call with the per-role clock sums of its CTAs -
    how long the decode warps wait for a free stage and decode, how long the MMA thread waits
    for a full stage, the epilogue - as mean SM cycles per CTA and per 64-channel stage."""
    import ctypes

    import torch

    from sage_b200 import SAGELinear, _lib
    from sage_b200.synthetic import synthetic_sage_device

    _, k, n, rows = args.workload.split(":")
    k, n, rows = int(k), int(n), int(rows)
    lib = _lib.load()
    device = torch.device("cuda", 0)
    layer = SAGELinear(synthetic_sage_device(k, n, 3, device, direction_bits=8), n)
    x = torch.randn(rows, k, device=device, dtype=torch.float16)
    for _ in range(3):
        layer(x)
    torch.cuda.synchronize(device)
    trace = torch.zeros(1024 * 16, dtype=torch.int64, device=device)
    lib.sageb200_debug_trace(ctypes.c_void_p(trace.data_ptr()))
    layer(x)
    torch.cuda.synchronize(device)
    lib.sageb200_debug_trace(None)
    records = trace.view(-1, 16).cpu()
    records = records[records[:, 2] != 0].double()
    if records.numel() == 0:
        print(json.dumps({"workload": args.workload, "error": "no clock sums: load the profiling build "
                          "(python -m sage_b200.build --trace; SAGEB200_LIBRARY=sage_b200/libsage_b200_trace.so)"}))
        return
    names = ["decode_thread0_wait_free_stage", "decode_thread0_decode_store_arrive", "decode_thread0_main_loop",
             "decode_last_thread_wait_free_stage", "decode_last_thread_decode_store_arrive",
             "decode_last_thread_main_loop", "epilogue", "tma_thread_wait_free_stage", "mma_thread_wait_full_stage",
             "mma_thread_main_loop", "decode_thread0_decode_and_store", "decode_thread0_proxy_fence",
             "epilogue_wait_for_accumulator", "split_epilogue_write_tiles", "split_epilogue_fence_and_barriers",
             "split_epilogue_reduce_parts"]
    print(json.dumps({"workload": args.workload, "tiles_traced": int(records.shape[0]), "k_stages_total": k // 64,
                      "mean_sm_cycles_per_cta": {name: float(records[:, i].mean()) for i, name in enumerate(names)}}),
          flush=True)


def run_skinny_phases(args) -> None:
    """`--workload skinny_phases:K:N:M` (profiling build only): one decode-kernel call (M <= 16 rows)
    with the SM clock read at each phase boundary by every CTA; prints the median duration of each
    phase over the CTAs in microseconds (at the device's SM clock) and the call's CUDA-event time."""
    import ctypes

    import torch

    from sage_b200 import SAGELinear, _lib
    from sage_b200.synthetic import synthetic_sage_device

    _, k, n, rows = args.workload.split(":")
    k, n, rows = int(k), int(n), int(rows)
    lib = _lib.load()
    device = torch.device("cuda", 0)
    layer = SAGELinear(synthetic_sage_device(k, n, 3, device, direction_bits=8), n)
    x = torch.randn(rows, k, device=device, dtype=torch.float16)
    for _ in range(3):
        layer(x)
    torch.cuda.synchronize(device)
    trace = torch.zeros(64 * 512 * 16, dtype=torch.int64, device=device)
    lib.sageb200_debug_trace(ctypes.c_void_p(trace.data_ptr()))
    layer(x)
    torch.cuda.synchronize(device)
    lib.sageb200_debug_trace(None)
    records = trace.view(64, 512, 16)[0].cpu()
    records = records[records[:, 0] != 0].double()
    if records.numel() == 0:
        print(json.dumps({"workload": args.workload, "error": "no phase clocks: load the profiling build "
                          "(python -m sage_b200.build --trace; SAGEB200_LIBRARY=sage_b200/libsage_b200_trace.so)"}))
        return
    mhz = torch.cuda.clock_rate() if hasattr(torch.cuda, "clock_rate") else 1965
    order = [0, 11, 12, 1, 14, 2, 3, 4, 5, 6, 7, 8, 9, 10]
    names = ["partition_arithmetic", "barrier_init_and_bulk_copies", "tile_tables", "wait_for_previous_kernel",
             "activation_staging", "barrier", "permutation_gather", "wait_for_weight_bytes", "main_loop", "barrier_2",
             "combine_warps_and_store", "shared_tile_fix_up", "counter_reset"]
    phases = {}
    for i, name in enumerate(names):
        live = (records[:, order[i + 1]] != 0) & (records[:, order[i]] != 0)  # (phases a launch kind skips stay 0)
        if not bool(live.any()):
            continue
        delta = records[live][:, order[i + 1]] - records[live][:, order[i]]
        phases[name] = {"median_us": float(delta.median()) / mhz, "max_us": float(delta.max()) / mhz}
    last = torch.where(records[:, 10] != 0, records[:, 10], records[:, 8])
    total = last - records[:, 0]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(20):
        layer(x)
    stop.record()
    torch.cuda.synchronize(device)
    print(json.dumps({"workload": args.workload, "ctas": int(records.shape[0]), "sm_mhz": mhz, "phases": phases,
                      "cta_total_us": {"median": float(total.median()) / mhz, "max": float(total.max()) / mhz},
                      "eager_call_us_warm_weights": start.elapsed_time(stop) * 1000.0 / 20}), flush=True)


def run_mega_phases(args) -> None:
    """`--workload mega_phases` (profiling build only): one Qwen3-4B token through the one-kernel
    decode step with %globaltimer stamps at every phase boundary of every CTA; prints the median
    duration of each phase over CTAs and layers, in microseconds, and the graph-replay time."""
    import ctypes
    import statistics

    import torch

    from sage_b200 import _lib
    from sage_b200.qwen3 import QWEN3_4B, PackedQwen3

    lib = _lib.load()
    device = torch.device("cuda", 0)
    model = PackedQwen3(QWEN3_4B, device, seed=0, max_seq=args.prompt + 64, max_new=64)
    if model.mega is None:
        print(json.dumps({"workload": args.workload, "error": "the one-kernel step does not fit this model"}))
        return
    model.use_mega = True
    model.capture()
    prompt = torch.randint(3, QWEN3_4B.vocab, (1, args.prompt), generator=torch.Generator().manual_seed(1))
    model.prefill(prompt)
    for _ in range(5):
        model.graph.replay()
    torch.cuda.synchronize(device)
    ctas = model.sm_count
    trace = torch.zeros(ctas * 2048, dtype=torch.int64, device=device)
    lib.sageb200_debug_trace(ctypes.c_void_p(trace.data_ptr()))
    model.step(head=True)
    torch.cuda.synchronize(device)
    lib.sageb200_debug_trace(None)
    stamps = trace.view(ctas, 2048).cpu()
    count = int((stamps[0] != 0).sum())
    names = ["linear0.staging", "linear0.main_loops", "linear0.combine_and_prefetch", "barrier_to_attention",
             "attention.partial", "barrier_to_combine", "attention.combine", "barrier_to_linear1", "linear1.staging",
             "linear1.main_loops", "linear1.combine_and_prefetch", "barrier_to_linear2", "linear2.staging",
             "linear2.main_loops", "linear2.combine_and_prefetch", "barrier_to_linear3", "linear3.staging",
             "linear3.main_loops", "linear3.combine_and_prefetch"]
    per_layer = len(names) + 1
    layers = QWEN3_4B.layers
    if count < 1 + layers * per_layer:
        print(json.dumps({"workload": args.workload, "error": "no phase stamps: load the profiling build "
                          "(python -m sage_b200.build --trace; SAGEB200_LIBRARY=sage_b200/libsage_b200_trace.so)"}))
        return
    microseconds = (stamps[:, :count] - stamps[:, 0].min()).double() / 1000.0
    phases = {}
    for i, name in enumerate(names):
        values = [float((microseconds[:, 1 + layer * per_layer + i + 1] - microseconds[:, 1 + layer * per_layer + i]).median())
                  for layer in range(2, layers)]
        phases[name] = statistics.mean(values)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(50):
        model.graph.replay()
    stop.record()
    torch.cuda.synchronize(device)
    print(json.dumps({"workload": args.workload, "prompt_tokens": args.prompt,
                      "phase_us_median_over_ctas_mean_over_layers": phases,
                      "layer_us": sum(phases.values()),
                      "token_us_traced": float(microseconds[:, count - 1].max()),
                      "graph_replay_ms_per_token": start.elapsed_time(stop) / 50}), flush=True)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--workload", default="decode_model")
    parser.add_argument("--prompt", type=int, default=512)
    parser.add_argument("--batch", type=int, default=1, help="sequences decoded together (tp32b / ep30b / decode_batch workloads)")
    parser.add_argument("--output", default="reports", help="folder for the files of --workload report")
    parser.add_argument("--quick", action="store_true",
                        help="headline measurement only: skip the per-kernel, batch-8 and sharded sub-records")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload.startswith("linear:"):
        run_single_linear(args)
    elif args.workload.startswith("gemm_roles:"):
        run_gemm_roles(args)
    elif args.workload.startswith("skinny_phases:"):
        run_skinny_phases(args)
    elif args.workload == "mega_phases":
        run_mega_phases(args)
    elif args.workload == "prompt":
        run_prompt(args)
    elif args.workload == "decode_batch":
        run_decode_batch(args)
    elif args.workload.startswith("sph:"):
        run_sph_linear(args)
    elif args.workload == "report":
        run_report(args)
    elif args.workload == "decode_model":
        run_model(args)
    elif args.workload in ("tp32b", "ep30b"):
        run_tp(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
