"""GPU: packed checkpoints loaded through native Hugging Face `from_pretrained` and run
(after the reference's tests/inference/test_hf_cuda.py:54-123): one random Qwen3 layer at the
production projection shapes, packed with seeded synthetic buffers, saved, loaded straight to
the GPU and via the CPU, prefill + two decode steps on a StaticCache, `generate`; the packed
model against the same model holding the dense dequantised weights; and the external dtype
boundary of both packed modules."""

import gc

import pytest
import torch

transformers = pytest.importorskip("transformers")

from oracle import c_oracle, sph_oracle  # noqa: E402
from sage_b200 import SAGELinear, SPHQuantLinear, integrations, synthetic_sage, synthetic_sphquant  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def real_width_model():
    config = transformers.Qwen3Config(
        vocab_size=32, hidden_size=2560, intermediate_size=9728, num_hidden_layers=1, num_attention_heads=32,
        num_key_value_heads=8, head_dim=128, pad_token_id=0, bos_token_id=1, eos_token_id=None)
    torch.manual_seed(9)
    return config


def load(destination, device):
    try:
        return transformers.AutoModelForCausalLM.from_pretrained(
            destination, device_map=device, dtype="auto", attn_implementation="sdpa", local_files_only=True).eval()
    except (ImportError, ValueError):  # no `accelerate`: load on the CPU and move
        model = transformers.AutoModelForCausalLM.from_pretrained(
            destination, dtype="auto", attn_implementation="sdpa", local_files_only=True).eval()
        return model.to(device)


@pytest.mark.skipif(not integrations.REGISTERED, reason='another package owns the "wvq" quantizer name')
@pytest.mark.parametrize("method", ["sage", "sphquant"])
@torch.inference_mode()
def test_loaded_model_prefill_decode_generate(real_width_model, tmp_path, method):
    from transformers import StaticCache

    source = transformers.AutoModelForCausalLM.from_config(real_width_model, dtype=torch.float16).eval()
    quantization = integrations.pack_synthetic(source, method, seed=44)
    assert len(quantization.modules) == 7
    destination = tmp_path / "packed"
    source.save_pretrained(destination, safe_serialization=True)
    direct = load(destination, "cuda")
    moved = load(destination, "cpu")
    moved.to(device="cuda")
    kind = SAGELinear if method == "sage" else SPHQuantLinear
    packed_modules = [m for m in direct.modules() if isinstance(m, kind)]
    assert len(packed_modules) == 7 and all(m.packed_codes.is_cuda for m in packed_modules)
    # the same architecture holding the kernel-dequantised dense weights: the model-level oracle
    dense = transformers.AutoModelForCausalLM.from_config(real_width_model, dtype=torch.float16).eval().cuda()
    state = {k: v for k, v in direct.state_dict().items()
             if not any(tag in k for tag in ("packed_codes", "radius_", "codebook", "permutation"))}
    for name in quantization.modules:
        state[name + ".weight"] = direct.get_submodule(name).dequantize()
    missing, unexpected = dense.load_state_dict(state, strict=False)
    assert not unexpected and all("lm_head" in m or "rotary" in m for m in missing), (missing, unexpected)

    tokens = torch.tensor([[1, 3, 5, 7]], device="cuda")
    models = (direct, moved, dense)
    caches = [StaticCache(config=model.config, max_cache_len=8) for model in models]
    try:
        for step in range(3):
            inputs = tokens if step == 0 else tokens[:, -1:]
            results = [model(inputs, past_key_values=cache, use_cache=True).logits
                       for model, cache in zip(models, caches)]
            assert all(torch.isfinite(result).all() for result in results)
            torch.testing.assert_close(results[0], results[1], rtol=2e-3, atol=2e-3)
            error = (results[0].float() - results[2].float()).norm() / results[2].float().norm()
            assert error.item() < 5e-3, (step, error.item())  # the reference's model-level gate
            assert all(cache.get_seq_length() == 4 + step for cache in caches)
        generated = direct.generate(tokens, max_new_tokens=3, do_sample=False, eos_token_id=None)
        assert generated.shape == (1, 7)
        assert torch.equal(generated[:, :4], tokens)
        assert not any(name.endswith(".dense") for name in direct.state_dict())
    finally:
        del direct, moved, dense, caches
        gc.collect()
        torch.cuda.empty_cache()


@pytest.mark.parametrize("method", ["sage", "sphquant"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@torch.inference_mode()
def test_spherical_external_dtype_boundary(method, dtype):
    if method == "sage":
        packed = synthetic_sage(256, 32, seed=2)
        layer = SAGELinear({k: v.cuda() for k, v in packed.items()}, 32)
        weight = torch.from_numpy(c_oracle.decode_fp16(packed, 32)).cuda()
    else:
        packed = synthetic_sphquant(256, 32, seed=2)
        layer = SPHQuantLinear({k: v.cuda() for k, v in packed.items()})
        weight = torch.from_numpy(sph_oracle.decode_fp16(packed)).cuda()
    for rows in (1, 17, 40):
        x = torch.randn(rows, 256, generator=torch.Generator().manual_seed(43)).to(dtype).cuda()
        actual = layer(x)
        expected = torch.nn.functional.linear(x.half(), weight).to(dtype)
        assert actual.dtype == dtype
        error = (actual.float() - expected.float()).norm() / expected.float().norm()
        assert error.item() < 5e-3
