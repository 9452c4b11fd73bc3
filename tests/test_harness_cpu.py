"""The report schema of `sage_b200.harness` (no GPU): the reductions and the CSV follow the
reference benchmark's (benchmarks/model.py:283-355, :361-378; its own checks are in
tests/benchmark/test_model.py)."""

import csv
import json

from sage_b200.harness import reduce_samples, write_report


def test_decode_rows():
    samples = [{"synchronized_wall_ms": 30.0}, {"synchronized_wall_ms": 20.0}, {"synchronized_wall_ms": 40.0}]
    rows = reduce_samples("sage", "decode", samples, batch=2, prefill=8, decode=11)
    assert rows[0] == ("sage", "decode", "forward_tpot", 3.0, "ms/token")  # median 30 ms / 10 steps
    assert rows[1][:3] == ("sage", "decode", "output_throughput")
    assert abs(rows[1][3] - 2 * 10 * 3 * 1000 / 90.0) < 1e-9 and rows[1][4] == "tokens/s"
    assert reduce_samples("sage", "decode", samples, batch=1, prefill=8, decode=1) == []


def test_prefill_and_end_to_end_rows():
    prefill = reduce_samples("sage", "prefill", [{"synchronized_wall_ms": 10.0}, {"synchronized_wall_ms": 30.0}],
                             batch=1, prefill=512, decode=4)
    assert prefill[0] == ("sage", "prefill", "forward_latency", 20.0, "ms")
    assert prefill[1] == ("sage", "prefill", "input_throughput", 512 * 2 * 1000 / 40.0, "tokens/s")
    samples = [
        {"synchronized_wall_ms": 100.0, "gpu_ttft_ms": 40.0, "first_token_cpu_ms": 41.0},
        {"synchronized_wall_ms": 110.0, "gpu_ttft_ms": 42.0, "first_token_cpu_ms": 43.0},
        {"synchronized_wall_ms": 90.0, "gpu_ttft_ms": 38.0, "first_token_cpu_ms": 39.0},
    ]
    rows = {row[2]: row for row in reduce_samples("sage", "end_to_end", samples, batch=1, prefill=512, decode=4)}
    assert rows["generate_latency"][3] == 100.0 and rows["ttft"][3] == 40.0
    assert abs(rows["tpot"][3] - (100.0 - 41.0) / 3) < 1e-9
    assert abs(rows["output_throughput"][3] - 4 * 3 * 1000 / 300.0) < 1e-9


def test_report_files(tmp_path):
    rows = [("sage", "decode", "forward_tpot", 2.04567, "ms/token")]
    path, csv_path = write_report({"method": "sage"}, rows, tmp_path, "unit")
    assert json.loads(path.read_text()) == {"method": "sage"}
    with csv_path.open() as stream:
        assert list(csv.reader(stream)) == [["method", "phase", "metric", "value", "unit"],
                                            ["sage", "decode", "forward_tpot", "2.046", "ms/token"]]
