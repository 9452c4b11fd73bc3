"""ctypes binding of libsage_b200.so (the C ABI declared in include/sage_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
import pathlib

PACKAGE = pathlib.Path(__file__).resolve().parent
# SAGEB200_LIBRARY selects another build of the same library (the profiling build that
# `python -m sage_b200.build --trace` writes beside the product one)
LIBRARY = pathlib.Path(os.environ.get("SAGEB200_LIBRARY", PACKAGE / "libsage_b200.so"))

OK = 0
MAX_GROUPED = 16

# every symbol include/sage_b200.h declares
EXPORTED = (
    "sageb200_version",
    "sageb200_status_string",
    "sageb200_gemv_fuses_permutation",
    "sageb200_gemm_splits",
    "sageb200_workspace_bytes",
    "sageb200_linear",
    "sageb200_linear_grouped",
    "sageb200_grouped_workspace_bytes",
    "sageb200_fused_workspace_bytes",
    "sageb200_linear_grouped_fused",
    "sageb200_experts_workspace_bytes",
    "sageb200_experts",
    "sageb200_expert_blocks_workspace_bytes",
    "sageb200_expert_blocks",
    "sageb200_dequant",
    "sageb200_pack_spherical",
    "sageb200_host_staging_bytes",
    "sageb200_linear_host",
    "sageb200_set_tuning",
    "sageb200_sph_linear",
    "sageb200_sph_dequant",
    "sageb200_linear_static",
    "sageb200_clear_status",
    "sageb200_launch_count",
    "sageb200_glue_launch_count",
)

# every symbol include/sage_b200_debug.h declares (tuning and profiling aids)
EXPORTED_DEBUG = (
    "sageb200_debug_plan",
    "sageb200_set_pdl",
    "sageb200_debug_trace",
    "sageb200_debug_gemm_pairs",
    "sageb200_debug_gemm_plan",
)


# every symbol include/sage_b200_decode.h declares
EXPORTED_DECODE = (
    "sageb200_glue_embed",
    "sageb200_glue_add_rmsnorm",
    "sageb200_glue_add_rmsnorm_permuted",
    "sageb200_glue_swiglu_permuted",
    "sageb200_glue_qk_norm_rope_cache",
    "sageb200_glue_attention_scratch_bytes",
    "sageb200_glue_attention_decode",
    "sageb200_glue_attention_step",
    "sageb200_glue_attention_step_permuted",
    "sageb200_glue_prefill_qk_norm_rope_cache",
    "sageb200_glue_prefill_attention",
    "sageb200_glue_lm_head_step_scratch_bytes",
    "sageb200_glue_lm_head_step",
    "sageb200_glue_moe_route",
    "sageb200_glue_moe_mix",
    "sageb200_glue_dispatch_plan",
    "sageb200_glue_dispatch_rows",
    "sageb200_glue_combine_rows",
    "sageb200_glue_swiglu",
    "sageb200_glue_lm_head",
    "sageb200_glue_argmax_advance",
    "sageb200_mega_workspace_bytes",
    "sageb200_mega_prepare",
    "sageb200_mega_step",
)


# every symbol include/sage_b200_peer.h declares
EXPORTED_PEER = (
    "sageb200_peer_exchange_bytes",
    "sageb200_peer_create",
    "sageb200_peer_open",
    "sageb200_peer_close",
    "sageb200_peer_destroy",
    "sageb200_peer_all_reduce",
)
PEER_MAX_WORLD = 8
PEER_HANDLE_BYTES = 64


class Activation(ctypes.Structure):
    """struct sageb200_activation."""

    _fields_ = [
        ("kind", ctypes.c_int),
        ("eps", ctypes.c_float),
        ("a", ctypes.c_void_p),
        ("b", ctypes.c_void_p),
        ("weight", ctypes.c_void_p),
        ("residual_out", ctypes.c_void_p),
    ]


class ExpertStack(ctypes.Structure):
    """struct sageb200_expert_stack."""

    _fields_ = [
        ("codes", ctypes.c_void_p),
        ("radii", ctypes.c_void_p),
        ("grid", ctypes.c_void_p),
        ("book", ctypes.c_void_p),
        ("perm", ctypes.c_void_p),
        ("experts", ctypes.c_int),
        ("first_expert", ctypes.c_int),
        ("n", ctypes.c_int),
        ("k", ctypes.c_int),
        ("entries", ctypes.c_int),
    ]


class MegaLinear(ctypes.Structure):
    """struct sageb200_mega_linear."""

    _fields_ = [
        ("codes", ctypes.c_void_p),
        ("radii", ctypes.c_void_p),
        ("grid", ctypes.c_void_p),
        ("book", ctypes.c_void_p),
        ("perm", ctypes.c_void_p),
        ("n", ctypes.c_int),
        ("k", ctypes.c_int),
        ("entries", ctypes.c_int),
    ]


class MegaLayer(ctypes.Structure):
    """struct sageb200_mega_layer."""

    _fields_ = [(name, MegaLinear) for name in ("q", "k", "v", "o", "gate", "up", "down")] + [
        (name, ctypes.c_void_p) for name in ("input_norm", "post_norm", "q_norm", "k_norm", "k_cache", "v_cache")
    ]


class MegaModel(ctypes.Structure):
    """struct sageb200_mega_model."""

    _fields_ = [(name, ctypes.c_int) for name in ("layers", "hidden", "heads", "kv_heads", "head_dim",
                                                  "intermediate", "vocab", "max_seq")] + [
        ("eps", ctypes.c_float)] + [
        (name, ctypes.c_void_p) for name in ("embed", "lm_head", "final_norm", "cos_table", "sin_table")]


class Problem(ctypes.Structure):
    """struct sageb200_problem."""

    _fields_ = [
        ("x", ctypes.c_void_p),
        ("codes", ctypes.c_void_p),
        ("radii", ctypes.c_void_p),
        ("grid", ctypes.c_void_p),
        ("book", ctypes.c_void_p),
        ("perm", ctypes.c_void_p),
        ("y", ctypes.c_void_p),
        ("rows", ctypes.c_int),
        ("n", ctypes.c_int),
        ("k", ctypes.c_int),
        ("entries", ctypes.c_int),
    ]


_handle: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _handle
    if _handle is not None:
        return _handle
    if not LIBRARY.exists():
        raise RuntimeError(
            f"{LIBRARY} is missing: build it with `python -m sage_b200.build` "
            "(sage_b200 has no CPU or PyTorch fallback)"
        )
    lib = ctypes.CDLL(str(LIBRARY))
    vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.sageb200_version.restype = ci
    lib.sageb200_version.argtypes = []
    lib.sageb200_status_string.restype = ctypes.c_char_p
    lib.sageb200_status_string.argtypes = [ci]
    lib.sageb200_gemv_fuses_permutation.restype = ci
    lib.sageb200_gemv_fuses_permutation.argtypes = [ci, ci]
    lib.sageb200_gemm_splits.restype = ci
    lib.sageb200_gemm_splits.argtypes = [ci, ci, ci, ci]
    lib.sageb200_workspace_bytes.restype = sz
    lib.sageb200_workspace_bytes.argtypes = [ci, ci, ci]
    lib.sageb200_linear.restype = ci
    lib.sageb200_linear.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, sz, ci, ci, ci, ci, vp]
    lib.sageb200_grouped_workspace_bytes.restype = sz
    lib.sageb200_grouped_workspace_bytes.argtypes = [ctypes.POINTER(Problem), ci]
    lib.sageb200_fused_workspace_bytes.restype = sz
    lib.sageb200_fused_workspace_bytes.argtypes = [ctypes.POINTER(Problem), ci]
    lib.sageb200_linear_grouped_fused.restype = ci
    lib.sageb200_linear_grouped_fused.argtypes = [ctypes.POINTER(Problem), ci, ctypes.POINTER(Activation), vp, sz, vp]
    lib.sageb200_experts_workspace_bytes.restype = sz
    lib.sageb200_experts_workspace_bytes.argtypes = [ctypes.POINTER(ExpertStack), ci, ci]
    lib.sageb200_experts.restype = ci
    lib.sageb200_experts.argtypes = [vp, ctypes.c_longlong, ctypes.POINTER(ExpertStack), ctypes.POINTER(vp), ci, vp, ci, vp, sz, vp]
    lib.sageb200_linear_grouped.restype = ci
    lib.sageb200_linear_grouped.argtypes = [ctypes.POINTER(Problem), ci, vp, sz, vp]
    lib.sageb200_dequant.restype = ci
    lib.sageb200_dequant.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci, vp]
    lib.sageb200_host_staging_bytes.restype = sz
    lib.sageb200_host_staging_bytes.argtypes = [ci, ci, ci]
    lib.sageb200_linear_host.restype = ci
    lib.sageb200_linear_host.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, sz, ci, ci, ci, ci, vp]
    lib.sageb200_set_tuning.restype = ci
    lib.sageb200_set_tuning.argtypes = [ci, ci, ci, ci]
    lib.sageb200_linear_static.restype = ci
    lib.sageb200_linear_static.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]
    lib.sageb200_sph_linear.restype = ci
    lib.sageb200_sph_linear.argtypes = [vp] * 7 + [ci] * 3 + [vp]
    lib.sageb200_sph_dequant.restype = ci
    lib.sageb200_sph_dequant.argtypes = [vp] * 6 + [ci] * 2 + [vp]
    lib.sageb200_debug_plan.restype = ci
    lib.sageb200_debug_plan.argtypes = [ci] * 5 + [ctypes.POINTER(ci)]
    lib.sageb200_expert_blocks_workspace_bytes.restype = sz
    lib.sageb200_expert_blocks_workspace_bytes.argtypes = [ctypes.POINTER(ExpertStack), ci, ci]
    lib.sageb200_expert_blocks.restype = ci
    lib.sageb200_expert_blocks.argtypes = [vp, ctypes.POINTER(ExpertStack), ctypes.POINTER(vp), ci, vp, ci, ci, vp, sz, vp]
    lib.sageb200_pack_spherical.restype = ci
    lib.sageb200_pack_spherical.argtypes = [vp] * 7 + [ci] * 4 + [vp]
    lib.sageb200_clear_status.restype = ci
    lib.sageb200_clear_status.argtypes = []
    lib.sageb200_set_pdl.restype = ci
    lib.sageb200_set_pdl.argtypes = [ci]
    lib.sageb200_debug_trace.restype = ci
    lib.sageb200_debug_trace.argtypes = [vp]
    lib.sageb200_debug_gemm_pairs.restype = ci
    lib.sageb200_debug_gemm_pairs.argtypes = [ci]
    lib.sageb200_debug_gemm_plan.restype = ci
    lib.sageb200_debug_gemm_plan.argtypes = [ci] * 5 + [ctypes.POINTER(ci)]
    lib.sageb200_launch_count.restype = ctypes.c_ulonglong
    lib.sageb200_launch_count.argtypes = []
    lib.sageb200_glue_launch_count.restype = ctypes.c_ulonglong
    lib.sageb200_glue_launch_count.argtypes = []
    # decode glue (include/sage_b200_decode.h)
    fl, ll = ctypes.c_float, ctypes.c_longlong
    lib.sageb200_glue_embed.restype = ci
    lib.sageb200_glue_embed.argtypes = [vp, vp, vp, ci, ci, ci, vp]
    lib.sageb200_glue_add_rmsnorm.restype = ci
    lib.sageb200_glue_add_rmsnorm.argtypes = [vp, vp, vp, vp, ci, ci, fl, vp]
    lib.sageb200_glue_add_rmsnorm_permuted.restype = ci
    lib.sageb200_glue_add_rmsnorm_permuted.argtypes = [vp, vp, vp, vp, ctypes.POINTER(vp), ctypes.POINTER(vp), ci, ci, ci, fl, vp]
    lib.sageb200_glue_swiglu_permuted.restype = ci
    lib.sageb200_glue_swiglu_permuted.argtypes = [vp, vp, vp, vp, ci, ci, ci, vp]
    lib.sageb200_glue_qk_norm_rope_cache.restype = ci
    lib.sageb200_glue_qk_norm_rope_cache.argtypes = [vp] * 10 + [ci] * 5 + [fl, vp]
    lib.sageb200_glue_attention_scratch_bytes.restype = sz
    lib.sageb200_glue_attention_scratch_bytes.argtypes = [ci, ci, ci]
    lib.sageb200_glue_attention_step.restype = ci
    lib.sageb200_glue_attention_step.argtypes = [vp] * 11 + [ci] * 6 + [ctypes.c_float, vp]
    lib.sageb200_glue_attention_step_permuted.restype = ci
    lib.sageb200_glue_attention_step_permuted.argtypes = [vp] * 12 + [ci] * 6 + [ctypes.c_float, vp]
    lib.sageb200_glue_prefill_qk_norm_rope_cache.restype = ci
    lib.sageb200_glue_prefill_qk_norm_rope_cache.argtypes = [vp] * 10 + [ci] * 6 + [ctypes.c_float, vp]
    lib.sageb200_glue_prefill_attention.restype = ci
    lib.sageb200_glue_prefill_attention.argtypes = [vp] * 5 + [ci] * 6 + [vp]
    lib.sageb200_glue_moe_route.restype = ci
    lib.sageb200_glue_moe_route.argtypes = [vp] * 7 + [ci] * 4 + [ctypes.c_float, vp]
    lib.sageb200_glue_dispatch_plan.restype = ci
    lib.sageb200_glue_dispatch_plan.argtypes = [vp, vp, vp, ci, ci, ci, ci, ci, vp]
    lib.sageb200_glue_dispatch_rows.restype = ci
    lib.sageb200_glue_dispatch_rows.argtypes = [vp, vp, vp, ci, ci, ci, ci, vp]
    lib.sageb200_glue_combine_rows.restype = ci
    lib.sageb200_glue_combine_rows.argtypes = [vp, vp, vp, ci, ci, ci, vp]
    lib.sageb200_glue_moe_mix.restype = ci
    lib.sageb200_glue_moe_mix.argtypes = [vp] * 3 + [ci] * 3 + [vp]
    lib.sageb200_glue_lm_head_step_scratch_bytes.restype = sz
    lib.sageb200_glue_lm_head_step_scratch_bytes.argtypes = [ci, ci]
    lib.sageb200_glue_lm_head_step.restype = ci
    lib.sageb200_glue_lm_head_step.argtypes = [vp] * 11 + [ci] * 3 + [ctypes.c_float, ci, ci, vp]
    lib.sageb200_glue_attention_decode.restype = ci
    lib.sageb200_glue_attention_decode.argtypes = [vp] * 6 + [ci] * 6 + [vp]
    lib.sageb200_glue_swiglu.restype = ci
    lib.sageb200_glue_swiglu.argtypes = [vp, vp, vp, ll, vp]
    lib.sageb200_glue_lm_head.restype = ci
    lib.sageb200_glue_lm_head.argtypes = [vp, vp, vp, ci, ci, ci, ci, vp]
    lib.sageb200_glue_argmax_advance.restype = ci
    lib.sageb200_glue_argmax_advance.argtypes = [vp] * 5 + [ci, ci, ci, vp]
    lib.sageb200_mega_workspace_bytes.restype = sz
    lib.sageb200_mega_workspace_bytes.argtypes = [ctypes.POINTER(MegaModel), ci]
    lib.sageb200_mega_prepare.restype = ci
    lib.sageb200_mega_prepare.argtypes = [ctypes.POINTER(MegaModel), ctypes.POINTER(MegaLayer), vp, sz, vp]
    lib.sageb200_mega_step.restype = ci
    lib.sageb200_mega_step.argtypes = [ctypes.POINTER(MegaModel), vp, vp, vp, vp, vp, vp, ci, vp]
    # all-reduce over peer memory (include/sage_b200_peer.h)
    lib.sageb200_peer_exchange_bytes.restype = sz
    lib.sageb200_peer_exchange_bytes.argtypes = [ci, ll]
    lib.sageb200_peer_create.restype = ci
    lib.sageb200_peer_create.argtypes = [ci, ll, ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_ubyte)]
    lib.sageb200_peer_open.restype = ci
    lib.sageb200_peer_open.argtypes = [ctypes.POINTER(ctypes.c_ubyte), ctypes.POINTER(vp)]
    lib.sageb200_peer_close.restype = ci
    lib.sageb200_peer_close.argtypes = [vp]
    lib.sageb200_peer_destroy.restype = ci
    lib.sageb200_peer_destroy.argtypes = [vp]
    lib.sageb200_peer_all_reduce.restype = ci
    lib.sageb200_peer_all_reduce.argtypes = [ctypes.POINTER(vp), ci, ci, ll, vp, ll, vp]
    if "SAGEB200_PDL" in os.environ:  # debug switch: which kernel families launch dependently
        lib.sageb200_set_pdl(int(os.environ["SAGEB200_PDL"]))
    _handle = lib
    return lib


def check(status: int) -> None:
    """Raise RuntimeError (as the reference's TORCH_CHECK does) on a non-zero status."""
    if status != OK:
        text = load().sageb200_status_string(status).decode()
        raise RuntimeError(f"sage_b200: {text} (status {status})")
