"""GPU: the export-side packing kernel (through the C ABI) against the reference exporter's
golden vectors and the CPU oracle, bit for bit, and the pack -> dense dequantisation round trip
(reference tests/inference/test_spherical_export.py:30-80)."""

import numpy as np
import pytest
import torch

from oracle import pack_oracle
from sage_b200 import sage_dequantize, sph_dequantize
from sage_b200.packing import direction_codebook_from_logits, pack_spherical, pack_spherical_radii
from test_pack_oracle import CASES, packed_of

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_kernel_reproduces_the_reference_exporter(case):
    want = packed_of(case)
    got = pack_spherical_radii(torch.from_numpy(case["state/signs"]).cuda(),
                               torch.from_numpy(case["state/direction_indices"]).cuda(),
                               torch.from_numpy(case["radius"]).cuda(), 1 << case["bits"], sage=case["sage"])
    for key, value in got.items():
        data = value.cpu().numpy()
        assert data.shape == want[key].shape and data.dtype == want[key].dtype, key
        np.testing.assert_array_equal(data.view(np.uint8), want[key].view(np.uint8), err_msg=key)


@pytest.mark.parametrize("sage,bits", [(False, 6), (True, 6), (True, 7), (True, 8)])
@pytest.mark.parametrize("permuted", [False, True])
@pytest.mark.parametrize("n,k", [(19, 256), (4096, 2560)])
def test_pack_then_dequantise_is_exact(sage, bits, permuted, n, k):
    """The state dictionary through `pack_spherical` and the dense dequantisation kernel:
    weight == fp16(signs * fp16 codebook[index] * (min + code * step)) exactly, channels back in
    original order; the packed buffers equal the CPU oracle's on the same radii."""
    gen = torch.Generator().manual_seed(bits * 100 + n)
    state = {
        "signs": (torch.randint(0, 2, (n, k), generator=gen, dtype=torch.int8) * 2 - 1).cuda(),
        "direction_indices": torch.randint(0, 1 << bits, (n, k // 8), generator=gen).cuda(),
        "radius_logits": torch.randn(n, k // 8, generator=gen).cuda(),
        "angle_logits": torch.randn(1 << bits, 7, generator=gen).cuda(),
        "radius_bits": torch.tensor(10 - bits),
        "group_size": torch.tensor(128),
        "sphquant_version": torch.tensor(1),
    }
    state["radius_logits"][0, :16] = 0.125
    state["radius_logits"][0, 16:] = -40
    if sage:
        order = torch.randperm(k, generator=gen) if permuted else torch.arange(k)
        state.update(channel_unpermutation=order.argsort().cuda(), sage_version=torch.tensor(1))
    elif permuted:
        pytest.skip("SPHQuant has no channel permutation")
    packed = pack_spherical(state, sage=sage)
    assert all(t.is_contiguous() for t in packed.values())
    radius = torch.nn.functional.softplus(state["radius_logits"].float())
    want = pack_oracle.pack_radii(state["signs"].cpu().numpy(), state["direction_indices"].cpu().numpy(),
                                  radius.cpu().numpy(), 1 << bits, sage)
    for key, value in want.items():
        np.testing.assert_array_equal(packed[key].cpu().numpy().view(np.uint8), value.view(np.uint8), err_msg=key)
    # expected dense weight from the packed grid itself
    book = direction_codebook_from_logits(state["angle_logits"]).half().float()
    if sage:
        grid = packed["radius_grid"].permute(0, 2, 1, 3).reshape(-1, k // 128, 2)[:n].float()
        minimum, step = grid[..., 0], grid[..., 1]
        high = packed["radius_codes"].permute(0, 2, 1).reshape(-1, k // 128)[:n]
        words = packed["packed_codes"].permute(0, 2, 1, 3).reshape(-1, k // 128, 8)[:n].long() & 0xFFFFFFFF
        codes16 = torch.stack((words & 0xFFFF, words >> 16), dim=-1).reshape(n, k // 128, 16)
    else:
        minimum, step = packed["radius_mins"].float(), packed["radius_scales"].float()
        high = packed["radius_extra"]
        codes16 = (packed["packed_codes"].long() & 0xFFFF).reshape(n, k // 128, 16)
    shifts = 2 * torch.arange(16, device="cuda")
    code = (codes16 >> (8 + bits)) | ((((high.long() & 0xFFFFFFFF)[..., None] >> shifts) & 3) << (8 - bits))
    radii = minimum[..., None] + code.float() * step[..., None]                # FP32, as the kernels
    assert torch.count_nonzero(step[0]) == 0
    expected = (state["signs"].reshape(n, -1, 8).float() * book[state["direction_indices"]]
                * radii.reshape(n, -1)[..., None]).half().reshape(n, k)
    if sage:
        expected = expected[:, state["channel_unpermutation"]]
        got = sage_dequantize(packed["packed_codes"], packed["radius_codes"], packed["radius_grid"],
                              packed["codebook"], packed["permutation"], n)
        assert bool(packed["permutation"].numel()) == permuted
        if n % 16:
            assert torch.count_nonzero(packed["packed_codes"][-1, :, n % 16:]) == 0
            assert torch.count_nonzero(packed["radius_grid"][-1, :, n % 16:]) == 0
    else:
        got = sph_dequantize(packed["packed_codes"], packed["radius_extra"], packed["radius_scales"],
                             packed["radius_mins"], packed["codebook"])
    assert torch.equal(got.view(torch.int16), expected.view(torch.int16))


def test_pack_rejects_what_the_reference_rejects():
    state = {
        "signs": torch.ones(16, 256, dtype=torch.int8, device="cuda"),
        "direction_indices": torch.zeros(16, 32, dtype=torch.long, device="cuda"),
        "radius_logits": torch.zeros(16, 32, device="cuda"),
        "angle_logits": torch.zeros(128, 7, device="cuda"),
        "radius_bits": torch.tensor(3), "group_size": torch.tensor(128),
    }
    with pytest.raises(ValueError, match="does not match"):
        pack_spherical(state, sage=True)
    with pytest.raises(ValueError, match="64/4"):
        pack_spherical(state, sage=False)
    state["sage_version"] = torch.tensor(1)
    state["radius_bits"] = torch.tensor(4)
    with pytest.raises(ValueError, match="bit split"):
        pack_spherical(state, sage=True)
