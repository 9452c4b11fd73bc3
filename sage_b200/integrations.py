"""Load packed SAGE / SPHQuant checkpoints through native Hugging Face `from_pretrained`.

Drop-in for the reference's `weight_vq/integrations/transformers.py:29-169` restricted to the
two packed formats this package runs: the on-disk format is the one the reference writes
(safetensors buffers named `<module>.packed_codes` ..., and `config.json` ->
`quantization_config = {"quant_method": "wvq", "method": "sage" | "sphquant", "modules":
{name: {"codebook_bits": 6|7|8, "permuted": bool}}, "format_version": 1, "synthetic_seed": ...}`),
so a directory exported by the reference loads onto `sage_b200.SAGELinear` /
`SPHQuantLinear` unchanged, and one written here loads in the reference.

Import this module before `AutoModelForCausalLM.from_pretrained`.  If the reference's
integration was imported first and already owns the "wvq" name, nothing is registered
(`REGISTERED` is False) and the reference's loader keeps building its own modules.

Beyond the reference: `model_type` "qwen3_moe" is accepted as well - every module named in
`modules` must be an `nn.Linear` of the native architecture (attention projections; experts
kept as fused tensors by the architecture are not linears and stay dense).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
from torch import nn
from transformers.quantizers import auto as _auto
from transformers.quantizers.base import HfQuantizer
from transformers.utils.quantization_config import QuantizationConfigMixin

from .linear import SAGELinear
from .sphquant import SPHQuantLinear
from .synthetic import synthetic_sage, synthetic_sphquant

METHODS = ("sage", "sphquant")
MODEL_TYPES = ("qwen3", "qwen3_moe")


@dataclass
class WVQConfig(QuantizationConfigMixin):
    """The inference ABI's metadata: which modules are packed and, for SAGE, each module's bit
    split and whether it carries a permutation (module sizes come from the architecture)."""

    method: str = "sage"
    modules: dict = field(default_factory=dict)
    format_version: int = 1
    synthetic_seed: int | None = None
    quant_method: str = "wvq"

    def __post_init__(self):
        if self.format_version != 1:
            raise ValueError(f"Unsupported weight-vq format version: {self.format_version}")
        if self.method not in METHODS:
            raise ValueError(f"sage_b200 loads the methods {METHODS}, not {self.method!r}")


def packed_linear(method: str, packed: dict, out_features: int, bias=None) -> nn.Module:
    if method == "sage":
        return SAGELinear(packed, out_features, bias)
    if method == "sphquant":
        return SPHQuantLinear(packed, bias)
    raise ValueError(f"Unsupported weight-vq method: {method}")


def skeleton(method: str, k: int, n: int, spec: dict) -> dict:
    """Empty buffers of one packed linear with the ABI's shapes and dtypes (on the current
    default device - the loader calls this under `torch.device("meta")`)."""
    if method == "sage":
        entries = 1 << int(spec["codebook_bits"])
        if entries not in (64, 128, 256):
            raise ValueError("SAGE codebook_bits must be 6, 7 or 8")
        tiles, groups = (n + 15) // 16, k // 128
        return {
            "packed_codes": torch.empty(tiles, groups, 16, 8, dtype=torch.int32),
            "radius_codes": torch.empty(tiles, groups, 16, dtype=torch.int32),
            "radius_grid": torch.empty(tiles, groups, 16, 2, dtype=torch.float16),
            "codebook": torch.empty(4, entries, 2, dtype=torch.float16),
            "permutation": torch.empty(k if spec["permuted"] else 0, dtype=torch.int32),
        }
    return {
        "packed_codes": torch.empty(n, k // 8, dtype=torch.int16),
        "radius_extra": torch.empty(n, k // 128, dtype=torch.int32),
        "radius_scales": torch.empty(n, k // 128, dtype=torch.float16),
        "radius_mins": torch.empty(n, k // 128, dtype=torch.float16),
        "codebook": torch.empty(64, 8, dtype=torch.float16),
    }


class WVQQuantizer(HfQuantizer):
    """Swaps the named `nn.Linear`s for packed modules before the weights are read, so the
    safetensors buffers land in them with their own dtypes (int32 / int16 / fp16 survive
    `dtype="auto"`); no dense weight is ever allocated."""

    requires_calibration = True

    def _process_model_before_weight_loading(self, model, **kwargs):
        if model.config.model_type not in MODEL_TYPES:
            raise ValueError(f"packed loading supports the model types {MODEL_TYPES}")
        config = self.quantization_config
        for name, spec in config.modules.items():
            linear = model.get_submodule(name)
            if not isinstance(linear, nn.Linear):
                raise ValueError(f"{name} is not an nn.Linear of the native architecture")
            k, n = linear.in_features, linear.out_features
            if k % 128:
                raise ValueError(f"{name}: in_features must be a multiple of 128")
            with torch.device("meta"):
                replacement = packed_linear(config.method, skeleton(config.method, k, n, spec), n, linear.bias)
            model.set_submodule(name, replacement)

    def _process_model_after_weight_loading(self, model, **kwargs):
        return model  # the packed buffers are complete as stored: nothing derived to rebuild

    def is_serializable(self, *args, **kwargs) -> bool:
        return True

    @property
    def is_trainable(self) -> bool:
        return False

    @property
    def is_compileable(self) -> bool:
        return True


def _register() -> bool:
    if "wvq" in _auto.AUTO_QUANTIZATION_CONFIG_MAPPING or "wvq" in _auto.AUTO_QUANTIZER_MAPPING:
        return False
    _auto.register_quantization_config("wvq")(WVQConfig)
    _auto.register_quantizer("wvq")(WVQQuantizer)
    return True


REGISTERED = _register()


def pack_synthetic(model: nn.Module, method: str = "sage", seed: int = 0) -> WVQConfig:
    """Replace every `nn.Linear` under `model.layers.` by a packed linear with seeded synthetic
    contents and record the metadata on `model.config` - the reference's synthetic export
    (weight_vq/checkpoint.py:193-216): per-module seed = seed + index in `named_modules()`."""
    generate = {"sage": synthetic_sage, "sphquant": synthetic_sphquant}[method]
    quantization = WVQConfig(method=method, synthetic_seed=seed)
    for index, (name, module) in enumerate(list(model.named_modules())):
        if not name.startswith("model.layers.") or not isinstance(module, nn.Linear):
            continue
        packed = generate(module.in_features, module.out_features, seed + index)
        spec = {}
        if method == "sage":
            spec = {"codebook_bits": packed["codebook"].shape[1].bit_length() - 1,
                    "permuted": bool(packed["permutation"].numel())}
        quantization.modules[name] = spec
        model.set_submodule(name, packed_linear(method, packed, module.out_features, module.bias))
    model.config.quantization_config = quantization
    return quantization
