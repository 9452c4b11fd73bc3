"""Hugging Face save/load round trips of packed checkpoints without CUDA, after the reference's
tests/inference/test_checkpoint.py:56-100: a tiny Qwen3 is packed with seeded synthetic
buffers, saved with `save_pretrained`, and read back by plain `from_pretrained` through the
registered "wvq" quantizer."""

import json

import pytest
import torch

transformers = pytest.importorskip("transformers")

from sage_b200 import SAGELinear, SPHQuantLinear, integrations  # noqa: E402
from sage_b200.synthetic import synthetic_sage, synthetic_sphquant  # noqa: E402


def tiny_model(dtype):
    config = transformers.Qwen3Config(
        vocab_size=16, hidden_size=128, intermediate_size=256, num_hidden_layers=1, num_attention_heads=4,
        num_key_value_heads=4, head_dim=32, tie_word_embeddings=True, attention_bias=True, pad_token_id=0,
        bos_token_id=1, eos_token_id=2)
    torch.manual_seed(9)
    return transformers.AutoModelForCausalLM.from_config(config).to(dtype).eval()


@pytest.mark.skipif(not integrations.REGISTERED, reason='another package owns the "wvq" quantizer name')
@pytest.mark.parametrize("method", ["sage", "sphquant"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_round_trip(tmp_path, method, dtype):
    model = tiny_model(dtype)
    quantization = integrations.pack_synthetic(model, method, seed=5)
    assert len(quantization.modules) == 7
    destination = tmp_path / "packed"
    model.save_pretrained(destination, safe_serialization=True)
    stored = json.loads((destination / "config.json").read_text())["quantization_config"]
    assert stored["quant_method"] == "wvq" and stored["method"] == method and stored["synthetic_seed"] == 5
    assert stored["format_version"] == 1 and len(stored["modules"]) == 7

    loaded, info = transformers.AutoModelForCausalLM.from_pretrained(
        destination, dtype="auto", local_files_only=True, output_loading_info=True)
    assert not info["missing_keys"] and not info["unexpected_keys"]
    kind = SAGELinear if method == "sage" else SPHQuantLinear
    generate = synthetic_sage if method == "sage" else synthetic_sphquant
    checked = 0
    for index, (name, module) in enumerate(list(model.named_modules())):
        if name not in quantization.modules:
            continue
        got = loaded.get_submodule(name)
        assert isinstance(got, kind)
        fresh = generate(got.in_features, got.out_features, 5 + index)
        for key, want in fresh.items():
            tensor = getattr(got, key)
            assert tensor.dtype == want.dtype and tensor.device.type == "cpu", (name, key)  # dtype="auto" left them alone
            assert torch.equal(tensor, want), (name, key)
        if module.bias is None:  # the MLP projections have none
            assert got.bias is None
        else:
            assert got.bias.dtype == dtype and torch.equal(got.bias, module.bias)
        checked += 1
    assert checked == 7
    assert loaded.lm_head.weight is loaded.model.embed_tokens.weight


def test_rejects_other_methods_and_versions():
    with pytest.raises(ValueError):
        integrations.WVQConfig(method="qtip")
    with pytest.raises(ValueError):
        integrations.WVQConfig(format_version=2)
