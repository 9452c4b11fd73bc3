"""The allocation-free decode entry point against the regular one (GPU).

`sageb200_linear_static` exists for hosts that cannot give the library a workspace because
they must not allocate device memory while serving (a fixed start-up memory plan, a plugin
that only receives pointers and a stream, a token loop that cannot afford an allocator's
device-wide stall).  Its scratch is a static array inside the library, so the things to
check are: same numbers as `sageb200_linear` with caller scratch, still the same on a second
call in a row (the array keeps the previous call's contents), no dependence on what ran
before in the process, and a clean refusal of shapes the array cannot hold.

This file sorts last on purpose: a run that stops at the first failure has by then run
every other test.
"""

import ctypes

import pytest
import torch

from sage_b200 import _lib, synthetic_sage

pytestmark = pytest.mark.gpu

REL_FROBENIUS = 1e-3  # the gate the other GPU tests use for matmul outputs
STATIC_BYTES = 8 * 1024 * 1024


def _pointers(gpu):
    vp = ctypes.c_void_p
    perm = gpu["permutation"]
    return (
        vp(gpu["packed_codes"].data_ptr()),
        vp(gpu["radius_codes"].data_ptr()),
        vp(gpu["radius_grid"].data_ptr()),
        vp(gpu["codebook"].data_ptr()),
        vp(perm.data_ptr()) if perm.numel() else None,
    )


# shapes that exercise every kind of scratch: shared output tiles (partial sums + arrival
# counters), several rows with a permutation (gathered activations), and none at all
CASES = [
    (9728, 2560, 1, 0, True),
    (9728, 2560, 8, 1, True),
    (4096, 2560, 16, 2, True),
    (2560, 9728, 1, 0, True),
    (2560, 1024, 5, 1, False),
    (256, 17, 3, 2, True),
]


@pytest.mark.parametrize("k,n,rows,seed,permuted", CASES)
def test_static_scratch_matches_caller_scratch_twice(k, n, rows, seed, permuted):
    lib = _lib.load()
    vp = ctypes.c_void_p
    cpu = synthetic_sage(k, n, seed=seed, permuted=permuted)
    gpu = {key: value.cuda() for key, value in cpu.items()}
    entries = cpu["codebook"].shape[1]
    stream = vp(torch.cuda.current_stream().cuda_stream)
    x = torch.randn(rows, k, generator=torch.Generator().manual_seed(11), dtype=torch.float16).cuda()

    need = lib.sageb200_workspace_bytes(rows, n, k)
    assert need <= STATIC_BYTES
    workspace = torch.zeros(max(need, 256), dtype=torch.uint8, device="cuda")
    want = torch.empty(rows, n, dtype=torch.float16, device="cuda")
    status = lib.sageb200_linear(
        vp(x.data_ptr()), *_pointers(gpu), vp(want.data_ptr()), vp(workspace.data_ptr()),
        workspace.numel(), rows, n, k, entries, stream,
    )
    assert status == 0, lib.sageb200_status_string(status)

    for call in range(2):  # the second call finds the first call's leftovers in the array
        got = torch.full((rows, n), float("nan"), dtype=torch.float16, device="cuda")
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        reserved_before = torch.cuda.memory_reserved()
        status = lib.sageb200_linear_static(
            vp(x.data_ptr()), *_pointers(gpu), vp(got.data_ptr()), rows, n, k, entries, stream
        )
        assert status == 0, lib.sageb200_status_string(status)
        torch.cuda.synchronize()
        if call == 1:  # past the first call's one-off set-up: the device's free memory did not move
            assert torch.cuda.mem_get_info()[0] == free_before
            assert torch.cuda.memory_reserved() == reserved_before
        assert torch.isfinite(got).all(), f"call {call}: output not fully written"
        error = (got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-30)
        assert error.item() <= REL_FROBENIUS, (call, error.item())
        # same kernel, same launch plan: in fact the bits agree
        assert torch.equal(got, want), call


def test_static_scratch_refuses_what_it_cannot_hold():
    lib = _lib.load()
    vp = ctypes.c_void_p
    stream = vp(torch.cuda.current_stream().cuda_stream)
    fake = vp(1 << 20)  # aligned, never dereferenced: the call must fail before any launch
    launches = lib.sageb200_launch_count()
    # more than 16 rows is outside the decode range this entry point serves
    assert lib.sageb200_linear_static(fake, fake, fake, fake, fake, None, fake, 17, 1024, 1024, 256, stream) == -8
    # a shape whose partial sums and gathered rows exceed the static array
    k, n, rows = 32768, 131072, 16
    assert lib.sageb200_workspace_bytes(rows, n, k) > STATIC_BYTES
    assert lib.sageb200_linear_static(fake, fake, fake, fake, fake, fake, fake, rows, n, k, 256, stream) == -8
    assert b"static" in lib.sageb200_status_string(-8)
    # ordinary argument errors are reported as usual
    assert lib.sageb200_linear_static(fake, fake, fake, fake, fake, None, fake, 1, 1024, 1000, 256, stream) == -1
    assert lib.sageb200_linear_static(fake, fake, fake, fake, fake, None, fake, 0, 1024, 1024, 256, stream) == 0
    assert lib.sageb200_launch_count() == launches
    torch.cuda.synchronize()
