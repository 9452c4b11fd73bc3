"""Generation measurements in the reference benchmark's report schema.

The reference's `benchmarks/model.py:283-355` reduces per-phase samples to rows
`(method, phase, metric, value, unit)` and writes them as a CSV beside a raw JSON file
(`:361-392`).  This module produces the same rows for `PackedQwen3`, so that a run here can be
laid beside the reference's tables:

  phase "prefill"      forward_latency [ms] (median), input_throughput [tokens/s]
  phase "decode"       forward_tpot [ms/token] (median window / steps), output_throughput [tokens/s]
  phase "end_to_end"   generate_latency [ms] (median), output_throughput [tokens/s],
                       ttft [ms] (median, GPU time to the first token), tpot [ms/token]

A decode window is `decode - 1` steps after the prompt, as in the reference (the first token
comes out of the prefill).  Times are synchronised wall-clock milliseconds, ttft is measured
with CUDA events; warm-up windows are discarded.
"""

from __future__ import annotations

import csv
import json
import pathlib
import time
from statistics import median

import torch

PHASES = ("prefill", "decode", "end_to_end")


def _window(model, prompt: torch.Tensor, phase: str, decode: int) -> dict:
    """One measured window of `phase`; the cache is rebuilt by the prefill each time."""
    device = model.device
    steps = decode - 1
    if phase == "decode":  # untimed prompt, then the timed token loop
        model.prefill(prompt)
        torch.cuda.synchronize(device)
    first, done = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin_event = torch.cuda.Event(enable_timing=True)
    begin = time.perf_counter()
    begin_event.record()
    first_cpu = None
    if phase in ("prefill", "end_to_end"):
        model.prefill(prompt)
        first.record()
        if phase == "end_to_end":
            first.synchronize()  # the first token is on the host's side of the stream now
            first_cpu = 1000.0 * (time.perf_counter() - begin)
    if phase in ("decode", "end_to_end"):
        for _ in range(steps):
            model.graph.replay()
    done.record()
    torch.cuda.synchronize(device)
    sample = {"synchronized_wall_ms": 1000.0 * (time.perf_counter() - begin)}
    if phase == "end_to_end":
        sample["gpu_ttft_ms"] = begin_event.elapsed_time(first)
        sample["first_token_cpu_ms"] = first_cpu
    return sample


def reduce_samples(method: str, phase: str, samples: list[dict], batch: int, prefill: int, decode: int):
    """The reference's reduction of one phase's samples to report rows."""
    times = [sample["synchronized_wall_ms"] for sample in samples]
    rows = []
    if phase == "decode":
        steps = decode - 1
        if steps:
            rows.append((method, phase, "forward_tpot", median(times) / steps, "ms/token"))
            rows.append((method, phase, "output_throughput", batch * steps * len(times) * 1000 / sum(times), "tokens/s"))
        return rows
    rows.append((method, phase, "forward_latency" if phase == "prefill" else "generate_latency", median(times), "ms"))
    tokens = prefill if phase == "prefill" else decode
    rows.append((method, phase, "input_throughput" if phase == "prefill" else "output_throughput",
                 batch * tokens * len(times) * 1000 / sum(times), "tokens/s"))
    if phase == "end_to_end":
        rows.append((method, phase, "ttft", median(sample["gpu_ttft_ms"] for sample in samples), "ms"))
        if decode > 1:
            rows.append((method, phase, "tpot",
                         median((sample["synchronized_wall_ms"] - sample["first_token_cpu_ms"]) / (decode - 1)
                                for sample in samples), "ms/token"))
    return rows


def measure(model, prompt: torch.Tensor, decode: int, *, samples: int = 5, warmup: int = 2,
            method: str = "sage", phases=PHASES):
    """Measure `phases` on `model` (a captured `PackedQwen3`); returns (result dict, rows)."""
    if decode > model.max_new:
        raise ValueError("decode exceeds the model's max_new")
    batch, prefill = prompt.shape
    result = {"method": method, "batch_size": batch, "prefill": prefill, "decode": decode,
              "samples": {phase: [] for phase in phases}}
    rows = []
    for phase in phases:
        for index in range(-warmup, samples):
            sample = _window(model, prompt, phase, decode)
            if index >= 0:
                result["samples"][phase].append(sample)
        rows.extend(reduce_samples(method, phase, result["samples"][phase], batch, prefill, decode))
    return result, rows


def write_report(result: dict, rows, directory, name: str) -> tuple[pathlib.Path, pathlib.Path]:
    """Raw JSON and the summary CSV with the reference's header and three-decimal values."""
    directory = pathlib.Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    path = directory / f"{name}.json"
    path.write_text(json.dumps(result, indent=2, default=str) + "\n")
    csv_path = path.with_suffix(".csv")
    with csv_path.open("w", newline="", encoding="utf-8") as stream:
        writer = csv.writer(stream)
        writer.writerow(("method", "phase", "metric", "value", "unit"))
        writer.writerows((m, p, metric, f"{value:.3f}", unit) for m, p, metric, value, unit in rows)
    return path, csv_path
