"""GPU: the one-kernel decode step (`sageb200_mega_step`) against the per-launch path and the
dense oracle model.

The persistent kernel runs the same arithmetic as the grouped packed-linear launches and the
glue kernels, with sums associating in another fixed order, so logits agree to the matmul gate's
order of magnitude and greedy tokens are those of the dense oracle (FP16 matmuls on the
dequantised weights)."""

import pytest
import torch

from sage_b200.qwen3 import PackedQwen3, Qwen3Config

pytestmark = pytest.mark.gpu

CONFIGS = {
    # leftover-only splits (fewer tiles than CTAs), two query heads per kv head
    "tiny": Qwen3Config(layers=2, hidden=256, heads=2, kv_heads=1, intermediate=512, vocab=1024),
    # the lockstep test's small model
    "small": Qwen3Config(layers=4, hidden=512, heads=4, kv_heads=2, intermediate=1024, vocab=8192),
    # whole tiles plus a shared-out remainder in every phase, four query heads per kv head, 8 per kv for the last
    "mid": Qwen3Config(layers=3, hidden=2560, heads=16, kv_heads=4, intermediate=4864, vocab=4099),
    "wide_group": Qwen3Config(layers=2, hidden=1024, heads=16, kv_heads=2, intermediate=2048, vocab=2048),
}


def run_path(config, use_mega, tokens, max_seq):
    model = PackedQwen3(config, "cuda", seed=7, max_seq=max_seq, max_new=tokens.numel() + 4)
    assert model.mega is not None, "the model does not fit the one-kernel step"
    model.use_mega = use_mega
    model.capture()
    model.reset()
    logits, picks = [], []
    for i in range(tokens.numel()):
        model.tokens.copy_(tokens[i : i + 1])
        model.graph.replay()
        logits.append(model.logits[0].float().clone())
        picks.append(int(model.tokens))
    torch.cuda.synchronize()
    cache = [(layer["k_cache"].float().clone(), layer["v_cache"].float().clone()) for layer in model.layers]
    return torch.stack(logits), picks, cache, int(model.positions), int(model.step_counter), model.log.clone()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_one_kernel_step_matches_the_per_launch_path(name):
    config = CONFIGS[name]
    steps, max_seq = 40, 48
    tokens = torch.randint(3, config.vocab, (steps,), generator=torch.Generator().manual_seed(5)).cuda()
    want, want_picks, want_cache, _, _, _ = run_path(config, False, tokens, max_seq)
    got, got_picks, got_cache, position, step, log = run_path(config, True, tokens, max_seq)
    assert position == steps and step == steps
    assert log[0, :steps].tolist() == got_picks
    for i in range(steps):
        error = ((got[i] - want[i]).norm() / want[i].norm()).item()
        assert error < 1e-2, (i, error)
        if got_picks[i] != want_picks[i]:  # only a near tie of the per-launch logits may flip
            margin = (want[i][want_picks[i]] - want[i][got_picks[i]]).item()
            assert 0 <= margin <= 0.02 * want[i].std().item(), (i, margin)
    for (k_got, v_got), (k_want, v_want) in zip(got_cache, want_cache):
        assert ((k_got - k_want).norm() / k_want.norm()).item() < 5e-3
        assert ((v_got - v_want).norm() / v_want.norm()).item() < 5e-3
        assert torch.equal(k_got[:, :, steps:], k_want[:, :, steps:])  # nothing beyond the tokens fed


def test_one_kernel_step_is_repeatable_and_stops_at_a_full_cache():
    config = CONFIGS["small"]
    steps, max_seq = 20, 16  # the last four steps find the cache full: no append, finite logits
    tokens = torch.randint(3, config.vocab, (steps,), generator=torch.Generator().manual_seed(9)).cuda()
    first = run_path(config, True, tokens, max_seq)
    second = run_path(config, True, tokens, max_seq)
    assert torch.equal(first[0], second[0]) and first[1] == second[1]
    assert torch.isfinite(first[0]).all()
    for (k1, v1), (k2, v2) in zip(first[2], second[2]):
        assert torch.equal(k1, k2) and torch.equal(v1, v2)


def test_models_outside_the_kernels_range_use_the_per_launch_path():
    from sage_b200 import _lib

    lib = _lib.load()
    import ctypes

    def nbytes(**changes):
        fields = dict(layers=2, hidden=512, heads=4, kv_heads=2, head_dim=128, intermediate=1024, vocab=1000,
                      max_seq=64)
        fields.update(changes)
        model = _lib.MegaModel(*[fields[k] for k in ("layers", "hidden", "heads", "kv_heads", "head_dim",
                                                     "intermediate", "vocab", "max_seq")], 1e-6, 0, 0, 0, 0, 0)
        return lib.sageb200_mega_workspace_bytes(ctypes.byref(model), 148)

    assert nbytes() > 0
    assert nbytes(head_dim=64) == 0
    assert nbytes(heads=18, kv_heads=2) == 0       # nine query heads per kv head
    assert nbytes(hidden=500) == 0
    assert nbytes(intermediate=1 << 20) == 0       # a row that does not fit shared memory
    moe = Qwen3Config(layers=1, hidden=256, heads=2, kv_heads=1, intermediate=512, vocab=512, experts=4, top_k=2,
                      moe_intermediate=128)
    assert PackedQwen3(moe, "cuda", seed=1, max_seq=32).mega is None
    assert PackedQwen3(CONFIGS["tiny"], "cuda", seed=1, max_seq=32, batch=2).mega is None
