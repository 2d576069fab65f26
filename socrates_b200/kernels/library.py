"""Load the CUDA library and declare its C entry points.

The library is reached through ctypes: every entry point takes raw device pointers,
sizes and a stream, so it needs no Python or torch headers and builds in seconds.
If the library cannot be built or loaded, `library()` raises: there is no fallback
path (the reference fails at start-up in the same way,
model/kernels/__init__.py:82-92 require_cuda_kernel).
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_void_p
from typing import Optional

from .build import BuildError, build_core


class KernelError(RuntimeError):
    """A kernel refused its arguments or failed to launch."""


_lib: Optional[ctypes.CDLL] = None
_lib_path: Optional[str] = None

P, I, F, LL = c_void_p, c_int, c_float, c_longlong

_SIGNATURES = {
    "sb_abi_version": [],
    "sb_set_dependent_launch": [I],
    "sb_embed": [P, P, P, I, I, I, I, P, F, P],
    "sb_add_rmsnorm": [P, P, I, LL, P, P, P, I, I, F, I, P],
    "sb_qk_norm_rope_kvwrite": [P, P, I, LL, P, P, P, P, P, P, I, P, P, P, I, I, F, I, I, I, I, I, I, I, I, I, P, I, F, I, P],
    "sb_silu_mul": [P, P, I, I, I, I, P],
    "sb_sample": [P, P, P, P, P, I, I, P, P],
    "sb_sample_slices": [I],
    "sb_gemm_simt": [P, P, P, I, I, I, I, I, I, I, P],
    "sb_attention_simt": [P, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, I, I, P],
    "sb_gemm_tcgen05": [P, P, P, I, I, I, I, P, P, I, I, P, LL, P],
    "sb_gemm_tcgen05_splits": [I, I],
    "sb_gemm_tcgen05_shares_parts": [I, I, I],
    "sb_attention_mma_supports": [I, I, I, I, I],
    "sb_attention_prefill_mma": [P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, P],
    "sb_attention_decode_mma": [P, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, I, I, P],
    "sb_attention_decode_mma_blocks_per_sm": [I, I],
    "sb_attention_decode_mma_kernels": [I],
    "sb_attention_decode_stream_supports": [I, I, I, I],
    "sb_attention_decode_stream": [P, P, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, I, I, I, P],
    "sb_attention_tcgen05_supports": [I, I, I, I],
    "sb_attention_prefill_tcgen05": [P, P, P, P, I, P, I, P, P, P, I, I, I, I, I, I, I, F, P, P, LL, I, I, F, I, P, P],
    "sb_fold_rmsnorm": [P, P, I, LL, P, P, F, P, P, P, P, P, I, I, F, I, P],
    "sb_normed_mean": [P, P, I, LL, P, P, I, LL, P, I, I, F, F, P],
    "sb_bias_act": [P, P, P, I, LL, P, I, I, I, I, P],
    "sb_short_conv": [P, LL, P, P, P, I, P, I, I, I, P, P, P, I, I, I, P, P, P, P, P, P, P, I, P],
    "sb_short_conv_tail": [P, P, LL, P, I, I, P, P, I, I, P],
    "sb_retention": [P, LL, I, I, I, I, P, P, P, P, I, P, P, P, P, I, I, I, I, F, F, I, I, P, LL, I, P],
    "sb_retention_chunk": [I, I],
    "sb_selective_scan": [P, LL, P, LL, P, P, P, LL, P, P, P, P, P, P, I, I, I, I, P, LL, I, P],
    "sb_attention_bias_tile_supports": [I, I, I, I, I],
    "sb_delta_rule_supports": [I, I],
    "sb_delta_rule": [P, P, LL, I, I, I, P, LL, I, I, I, P, P, P, P, P, P, I, I, I, I, I, F, F, I, P, I, P],
    "sb_moe_logits": [P, P, P, I, I, I, I, P],
    "sb_moe_route": [P, P, P, P, P, I, I, I, I, I, P],
    "sb_moe_scale": [P, P, I, I, I, I, I, P],
    "sb_moe_passthrough": [P, P, P, I, I, I, I, I, P],
    "sb_attention_bias_tile": [P, P, P, P, P, I, P, P, P, I, P, LL, P, I, I, I, I, I, I, I, I, F, F, I, I, I, F, P],
    "sb_softcap": [P, LL, F, P],
    "sb_diff_combine": [P, P, I, I, I, F, F, F, I, P],
    "sb_moe_table": [P, P, P, P, I, I, I, I, P],
    "sb_attention_diff": [P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, I, F, F, F, F, I, P, P, I, P],
    "sb_attention_diff_tile_supports": [I, I, I, I, I],
    "sb_attention_diff_tile": [P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, I, F, F, F, F, I, P],
    "sb_hyper_fold_norm": [P, P, I, I, P, I, LL, F, P, I, LL, F, P, P, P, F, P, P, F, I, P, P, P, I, I, P],
    "sb_min_gru": [P, P, LL, P, P, P, P, P, I, I, I, I, P],
    "sb_gated_linear_attention_supports": [I, I],
    "sb_gated_linear_attention_segments": [I],
    "sb_gated_linear_attention": [P, P, LL, I, I, I, P, P, P, P, P, P, I, I, I, I, F, I, P, I, I, P, P],
    "sb_glu_clamp": [P, P, P, I, LL, P, P, I, I, F, F, F, I, P],
    "sb_scale": [P, LL, F, P],
    "sb_segment_norm": [P, LL, I, P, P, P, P, P, P, P, P, P, F, I, I, P],
    "sb_head_matmul": [P, LL, I, I, P, LL, I, I, P, I, I, I, I, I, I, I, P],
    "sb_latent_write": [P, LL, I, I, I, I, P, F, P, I, P, I, F, P, P, P, I, I, P, P, I, I, P],
    "sb_attention_talk_tile": [I, I, I, I],
    "sb_attention_talk_dense": [I, P, P, P, P, P, P, P, P, P, P, P, P, LL, P, I, I, I, I, I, I, I, I, I, I, I, F, P],
    "sb_attention_talk": [P, P, P, P, P, I, P, P, P, I, P, P, LL, I, I, I, I, I, I, I, F, I, I, P, P, I, P],
    "sb_attention_bias": [P, P, P, P, P, I, P, P, P, LL, P, I, I, I, I, I, I, I, I, F, F, I, P, P, I, I, I, F, P],
}


def declare(lib: ctypes.CDLL, signatures: dict) -> None:
    for name, argtypes in signatures.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    if hasattr(lib, "sb_selective_scan_scratch"):
        lib.sb_selective_scan_scratch.argtypes = [c_int, c_int, c_int, c_int]
        lib.sb_selective_scan_scratch.restype = c_longlong
    lib.sb_last_error.argtypes = []
    lib.sb_last_error.restype = c_char_p


def library() -> ctypes.CDLL:
    """The loaded CUDA library; built at first call.  Raises if that is not possible."""
    global _lib, _lib_path
    if _lib is None:
        try:
            path = build_core()
            lib = ctypes.CDLL(str(path))
        except (BuildError, OSError) as e:
            raise KernelError(
                f"the socrates_b200 CUDA library is unavailable and there is no fallback: {e}") from e
        declare(lib, _SIGNATURES)
        _lib, _lib_path = lib, str(path)
    return _lib


def library_path() -> Optional[str]:
    return _lib_path


class Counters:
    """Kernels launched through the entry points since import.  A launch recorded into a
    CUDA graph counts once here; every replay launches the same kernels again."""
    launches = 0


def check(lib: ctypes.CDLL, code: int, what: str, kernels: int = 1) -> None:
    Counters.launches += kernels
    if code != 0:
        msg = lib.sb_last_error().decode(errors="replace")
        raise KernelError(f"{what}: {msg} (code {code})")
