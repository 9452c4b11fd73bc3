"""CPU-only checks of the C-ABI library: it loads without a GPU, exports every symbol the
header declares, and its host-side planning/validation behaves (no compute is launched)."""

import ctypes
import pathlib
import re

import pytest

from sage_b200 import _lib, build

ROOT = pathlib.Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def declared_symbols(header="sage_b200.h"):
    text = (ROOT / "include" / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sageb200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), name
    assert set(names) == set(_lib.EXPORTED) | {n for n in names if n not in _lib.EXPORTED}
    for name in _lib.EXPORTED:
        assert name in names, f"{name} bound in Python but not declared in the header"


def test_decode_header_symbols_are_exported(lib):
    names = declared_symbols("sage_b200_decode.h")
    assert set(names) == set(_lib.EXPORTED_DECODE)
    for name in names:
        assert hasattr(lib, name), name


def test_debug_header_symbols_are_exported(lib):
    names = declared_symbols("sage_b200_debug.h")
    assert set(names) == set(_lib.EXPORTED_DEBUG)
    for name in names:
        assert hasattr(lib, name), name


def test_peer_header_symbols_are_exported(lib):
    names = declared_symbols("sage_b200_peer.h")
    assert set(names) == set(_lib.EXPORTED_PEER)
    for name in names:
        assert hasattr(lib, name), name
    # sizes only (no device work): header, flags, two slots per rank
    assert lib.sageb200_peer_exchange_bytes(2, 5120) == 8192 + 2 * 2 * 5120 * 2
    assert lib.sageb200_peer_exchange_bytes(1, 5120) == 0
    assert lib.sageb200_peer_exchange_bytes(9, 5120) == 0
    assert lib.sageb200_peer_exchange_bytes(2, 5121) == 0


def test_version_and_status_strings(lib):
    assert lib.sageb200_version() >= 100
    assert lib.sageb200_status_string(0) == b"ok"
    for code in range(-8, 0):
        assert lib.sageb200_status_string(code) not in (b"ok", b"unknown status")
    assert lib.sageb200_status_string(-99) == b"unknown status"


def test_planning_is_deterministic_and_sane(lib):
    assert lib.sageb200_gemv_fuses_permutation(9728, 16384) == 1
    shapes = [(2560, 4096), (2560, 1024), (4096, 2560), (2560, 9728), (9728, 2560), (128, 1), (16384, 9)]
    for k, n in shapes:
        for rows in (1, 2, 8, 16, 17, 300):
            splits = lib.sageb200_gemm_splits(rows, n, k, 148)
            assert 1 <= splits <= min(8, k // 128)
            need = lib.sageb200_workspace_bytes(rows, n, k)
            assert need == lib.sageb200_workspace_bytes(rows, n, k)
            assert need % 256 == 0
            staging = lib.sageb200_host_staging_bytes(rows, n, k)
            assert staging >= rows * (k + n) * 2 + need
    assert lib.sageb200_workspace_bytes(0, 16, 128) == 0
    assert lib.sageb200_workspace_bytes(1, 16, 100) == 0


def _gemm_plan(lib, rows, n, k, allow_split=1, sm_count=148):
    fields = (ctypes.c_int * 10)()
    assert lib.sageb200_debug_gemm_plan(rows, n, k, sm_count, allow_split, fields) == 0
    names = ("tokens", "token_blocks", "row_blocks", "accumulators", "pair", "k_splits", "groups_per_split",
             "stages", "shared_bytes", "partial_kib")
    return dict(zip(names, fields))


def test_gemm_planner_choices(lib):
    """The tcgen05 GEMM's tile plan (host arithmetic): big grids take 256 tokens x 2 accumulators on
    CTA pairs without a K split; grids that would leave most of 148 SMs idle split K within one
    wave; without scratch nothing is split; every plan fits the kernel's shared memory."""
    gate = _gemm_plan(lib, 512, 9728, 2560)
    assert (gate["tokens"], gate["accumulators"], gate["pair"], gate["k_splits"]) == (256, 2, 1, 1)
    assert gate["row_blocks"] == 76 and gate["stages"] >= 3
    big = _gemm_plan(lib, 2048, 25600, 5120)
    assert (big["tokens"], big["accumulators"], big["pair"], big["k_splits"], big["partial_kib"]) == (256, 2, 1, 1, 0)
    down = _gemm_plan(lib, 512, 2560, 9728)
    assert down["k_splits"] > 1 and down["partial_kib"] > 0
    tiles = down["row_blocks"] * -(-down["token_blocks"] // down["accumulators"])
    assert tiles * down["k_splits"] <= 148                      # the split grid is one wave
    assert down["groups_per_split"] * down["k_splits"] >= 9728 // 128
    assert down["groups_per_split"] * (down["k_splits"] - 1) < 9728 // 128  # no empty split
    assert _gemm_plan(lib, 512, 2560, 9728, allow_split=0)["k_splits"] == 1
    odd = _gemm_plan(lib, 300, 1152, 640)                       # nine row blocks: no pairs
    assert odd["row_blocks"] == 9 and odd["pair"] == 0
    for rows, n, k in [(33, 129, 256), (257, 640, 1024), (513, 2560, 1280), (4096, 9728, 2560), (65535, 129, 256)]:
        for allow in (0, 1):
            plan = _gemm_plan(lib, rows, n, k, allow)
            assert plan["tokens"] % 16 == 0 and 16 <= plan["tokens"] <= 256
            assert plan["token_blocks"] * plan["tokens"] >= rows
            assert plan["shared_bytes"] <= 226 * 1024 and 2 <= plan["stages"] <= 6
            assert plan["pair"] in (0, 1) and (not plan["pair"] or plan["row_blocks"] % 2 == 0)
    assert lib.sageb200_debug_gemm_plan(16, 128, 128, 148, 1, (ctypes.c_int * 10)()) == -1


def test_invalid_arguments_are_rejected_without_a_device(lib):
    null = ctypes.c_void_p(None)
    one = ctypes.c_void_p(256)  # never dereferenced: validation fails first
    assert lib.sageb200_linear(one, null, one, one, one, null, one, null, 0, 1, 16, 128, 256, null) == -1
    assert lib.sageb200_linear(one, one, one, one, one, null, one, null, 0, 1, 16, 100, 256, null) == -1
    assert lib.sageb200_linear(one, one, one, one, one, null, one, null, 0, 1, 16, 128, 99, null) == -1
    assert lib.sageb200_linear(one, one, one, one, one, null, one, null, 0, 70000, 16, 128, 256, null) == -3
    odd = ctypes.c_void_p(258)
    assert lib.sageb200_linear(one, one, one, odd, one, null, one, null, 0, 1, 16, 128, 256, null) == -2
    assert lib.sageb200_dequant(one, one, one, one, null, null, 16, 128, 256, null) == -1
    assert lib.sageb200_set_tuning(17, 0, 0, 0) == -1
    assert lib.sageb200_set_tuning(0, 9, 0, 0) == -1
    assert lib.sageb200_set_tuning(0, 0, 0, 4) == -1
    assert lib.sageb200_set_tuning(0, 0, 0, 0) == 0
    assert lib.sageb200_linear_grouped(None, 1, null, 0, null) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_handle", None)
    monkeypatch.setattr(_lib, "LIBRARY", tmp_path / "libsage_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def _plan(lib, rows, n, k, act_kind=0, sm_count=148):
    import ctypes

    fields = (ctypes.c_int * 8)()
    assert lib.sageb200_debug_plan(rows, n, k, sm_count, act_kind, fields) == 0
    names = ("ctas", "slices", "whole", "ring", "slots", "warps", "shared", "scratch")
    return dict(zip(names, fields))


def test_decode_planner_choices():
    """Host arithmetic of the decode kernel's work split (no GPU): resident shares for the
    Qwen3-4B shapes, ring streaming in one resident wave for shares larger than shared memory,
    K slices only where several rows cannot keep their activations in shared memory."""
    from sage_b200 import _lib

    lib = _lib.load()
    assert lib.sageb200_set_tuning(0, 0, 0, 0) == 0
    for k, n in [(2560, 9728), (2560, 4096), (4096, 2560), (9728, 2560)]:  # Qwen3-4B, one row
        for kind in (0, 1, 2):
            plan = _plan(lib, 1, n, k, kind)
            assert plan["ring"] == 0 and plan["slices"] == 1 and plan["ctas"] <= 148, (k, n, kind, plan)
            assert plan["shared"] <= 184 * 1024 and plan["slots"] <= 192
    gate = _plan(lib, 1, 25600, 5120, 1)  # Qwen3-32B gate_proj: 433 units per SM against 192 slots
    assert gate["ring"] == 4 and gate["ctas"] <= 148 and gate["slices"] == 1 and gate["slots"] == 16 * 3 * 4
    down = _plan(lib, 1, 5120, 25600, 2)  # K = 25600: unsliced for one row, smaller ring stages
    assert down["slices"] == 1 and down["ctas"] <= 148 and down["ring"] in (1, 2) and down["shared"] <= 184 * 1024
    assert lib.sageb200_set_tuning(0, 0, 0, 3) == 0  # rings off: further waves of CTAs instead
    try:
        waves = _plan(lib, 1, 25600, 5120, 1)
        assert waves["ring"] == 0 and waves["ctas"] > 148 and waves["slots"] <= 192
    finally:
        assert lib.sageb200_set_tuning(0, 0, 0, 0) == 0
    rows8 = _plan(lib, 8, 2560, 9728)  # eight rows of K = 9728 do not fit: K is cut into slices
    assert rows8["slices"] > 1 and rows8["ring"] == 0 and rows8["scratch"] == 1
    rows16 = _plan(lib, 16, 25600, 5120)  # two column blocks never stream through rings
    assert rows16["ring"] == 0
    # several rows that fit beside whole tiles run without K slices and without scratch: 8 rows of
    # K = 2560 / 4096, 16 rows of K = 2560
    for rows, k, n in [(8, 2560, 9728), (8, 2560, 4096), (8, 4096, 2560), (16, 2560, 9728), (16, 2560, 4096)]:
        plan = _plan(lib, rows, n, k)
        assert plan["slices"] == 1 and plan["whole"] == 1 and plan["scratch"] == 0, (rows, k, n, plan)
        assert plan["shared"] <= 184 * 1024
    import ctypes

    assert lib.sageb200_debug_plan(17, 16, 128, 148, 0, (ctypes.c_int * 8)()) == -1


def test_grouped_scratch_of_a_group_that_runs_as_two_launches():
    """Host arithmetic only.  Row blocks of Qwen3-4B's q, k and v in one grouped call: blocks of 16
    rows (two MMA column blocks) next to blocks of 8 (one column block, which may stream through
    rings under a small CTA share) cannot share a launch - the library runs the group as its first
    and its second half, and the scratch it asks for is the larger half's, not the sum."""
    from sage_b200 import _lib

    lib = _lib.load()
    assert lib.sageb200_set_tuning(0, 0, 0, 0) == 0

    def need(blocks):
        array = (_lib.Problem * len(blocks))()
        for i, (rows, n, k) in enumerate(blocks):
            array[i] = _lib.Problem(None, None, None, None, None, 1, None, rows, n, k, 256)  # (a permutation is present)
        return lib.sageb200_grouped_workspace_bytes(array, len(blocks))

    mixed = [(rows, n, 2560) for n in (4096, 1024, 1024) for rows in (16, 8)]
    assert need(mixed) == max(need(mixed[:3]), need(mixed[3:])) > 0
    even = [(rows, n, 2560) for n in (4096, 1024, 1024) for rows in (12, 12)]  # one launch: the sum of the needs
    assert need(even) > max(need(even[:3]), need(even[3:]))
    assert need(even) == need(even) and need(mixed) % 256 == 0
    assert need([(17, 4096, 2560)]) == 0  # more than 16 rows: not a grouped problem
