"""ctypes binding of ``libpie_kernels.so`` (the sm_100a kernel library).

The library is built in-tree by :mod:`pie_b200._build`. On a machine with a GPU the
kernels are the only path: if the library is missing or a symbol cannot be resolved the
ops raise instead of falling back to PyTorch. On a CPU-only machine the ops use their
PyTorch reference implementations (``pie_b200.ops.reference``).
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

import torch

_LIB = None
_LOCK = threading.Lock()
_LIB_PATH = Path(__file__).resolve().parent.parent / "_C" / "libpie_kernels.so"

p = C.c_void_p
i32 = C.c_int
i64 = C.c_long
f32 = C.c_float

_SIGNATURES = {
    "pie_embed_gather": [p, p, p, i32, i32, i32, i32, p],
    "pie_rmsnorm": [p, p, p, p, p, i32, i32, f32, f32, p],
    "pie_swiglu": [p, p, i64, i32, p],
    "pie_glu_interleaved": [p, p, i64, i32, i32, p],
    "pie_dequant_fp8_rowblock": [p, p, p, i64, i32, p],
    "pie_quant_act_fp8": [p, i32, p, p, i32, i32, p],
    "pie_gemm_fp8_blockscaled": [p, p, p, p, p, p, i32, i32, i32, i32, i32, i32, p, i32, p],
    "pie_qk_norm_rope_kvwrite": [p, p, p, p, p, p, p, p, i32, i32, i32, i32, i32, f32, i32, p],
    "pie_qk_bias_norm_rope_kvwrite": [p, p, p, p, p, p, p, p, p, p, i32, i32, i32, i32, i32, f32, i32, p],
    "pie_qk_norm_rope_kvwrite_kv8": [p, p, p, p, p, p, p, p, p, i32, i32, i32, i32, i32, f32, i32, p],
    "pie_paged_decode_attn_kv8": [p, p, p, p, p, p, p, p, p, p, p, p, i32, i32, i32, i32, i32, i32, f32, i32, i32, p, p],
    "pie_dequant_kv_pages": [p, p, p, p, i32, i32, i32, i32, p],
    "pie_gather_rows": [p, p, p, i32, i32, p],
    "pie_copy_pages": [p, p, p, i32, i32, i64, i64, p],
    "pie_brle_expand": [p, p, p, i32, i32, i32, p],
    "pie_brle_expand_ragged": [p, p, p, p, p, i32, i32, i32, p],
    "pie_set_status_word": [p],
    "pie_paged_decode_attn": [p, p, p, p, p, p, p, p, p, p, p, i32, i32, i32, i32, i32, i32, f32, i32, i32, p],
    "pie_moe_bias_glu": [p, p, p, p, i32, i32, f32, p],
    "pie_moe_row_bias": [p, p, p, i32, i32, p],
    "pie_paged_decode_attn_window": [p, p, p, p, p, p, p, p, p, p, p, i32, i32, i32, i32, i32, i32, f32, i32, i32, i32, p, p],
    "pie_paged_decode_attn_softcap": [p, p, p, p, p, p, p, p, p, p, p, i32, i32, i32, i32, i32, i32, f32, i32, i32, i32, p, f32, p],
    "pie_paged_prefill_attn_softcap": [p, p, p, p, p, p, p, p, i32, p, p, p, p, i32, i32, i32, i32, f32, i32, p, f32, p],
    "pie_paged_decode_attn_cascade": [p, p, p, p, p, p, p, p, p, p, p, i32, i32, i32, i32, i32, i32, f32, i32, p, p, p, p, p],
    "pie_paged_prefill_attn": [p, p, p, p, p, p, p, p, i32, p, p, p, p, i32, i32, i32, i32, f32, i32, p, p],
    "pie_prefill_tile_tokens": [i32],
    "pie_prefill_attn_tc_supported": [i32, i32, i32, i32],
    "pie_paged_prefill_attn_tc": [p, p, p, p, p, p, p, p, i32, p, p, p, p, i32, i32, i32, i32, i32, f32, i32, i32, p, p, p],
    "pie_paged_prefill_attn_tc_softcap": [p, p, p, p, p, p, p, p, i32, p, p, p, p, i32, i32, i32, i32, i32, f32, i32, i32, p, p, f32, p],
    "pie_sample": [p, i64, i32, i32, p, p, p, p, p, p, p, i32, p, p],
    "pie_tp_sample_max_grid": [i32],
    "pie_tp_sample": [p, p, i64, i32, p, p, p, p, p, p, p, i32, p, i32, p],
    "pie_row_stats": [p, i64, i32, i32, p, p],
    "pie_feed_tokens": [p, p, p, i32, p],
    "pie_validate_indices": [p, i32, i32, i32, i32, p, p],
    "pie_gdn_mixer": [p, i32, p, p, p, p, p, p, p, p, p, p, p, p, i32, i32, i32, i32, i32, i32, i32, f32, p],
    "pie_gdn_copy_slot": [p, i64, i64, i32, i32, i32, p],
    "pie_mamba2_mixer": [p, i32, p, p, p, p, p, p, p, p, p, p, p, p, p, i32, i32, i32, i32, i32, i32, p],
    "pie_gemm_set_workspace": [i32, p, i64, p, i32],
    "pie_gemm_set_pairs": [i32],
    "pie_gemm_set_swap": [i32],
    "pie_set_pdl": [i32],
    "pie_gemm_bf16": [p, p, p, p, i32, i32, i32, i32, i32, i32, i32, i32, i32, p, i32, p],
    "pie_grouped_gemm_bf16": [p, p, p, p, i32, i32, i32, i32, i32, i32, i32, p, i32, p],
    "pie_moe_route": [p, i32, i32, i32, i32, i32, i32, i32, i32, p, p, p, p, p],
    "pie_moe_combine_rs": [p, p, p, i32, i32, i32, p, i32, p],
    "pie_moe_align": [p, i32, i32, p, p, p, p],
    "pie_moe_permute": [p, i32, p, p, p, i32, i32, i32, p, p, p],
    "pie_moe_combine": [p, p, p, p, i32, i32, i32, i32, p, i32, p],
}
_RESTYPES = {"pie_decode_attn_scratch_floats": i64}


class KernelLibraryError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def load(required: bool = True):
    """Return the loaded kernel library (building nothing). Raises when absent and required."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        if not _LIB_PATH.exists():
            if required:
                raise KernelLibraryError(
                    f"{_LIB_PATH} is missing: run `python -m pie_b200._build` (needs nvcc) first")
            return None
        lib = C.CDLL(str(_LIB_PATH))
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name, None)
            if fn is None:
                continue  # resolved lazily by `fn()` so that a stale library fails loudly on use
            fn.argtypes = argtypes
            fn.restype = i32
        for name, rt in _RESTYPES.items():
            f = getattr(lib, name, None)
            if f is not None:
                f.restype = rt
        _LIB = lib
        return _LIB


def fn(name: str):
    lib = load(required=True)
    f = getattr(lib, name, None)
    if f is None:
        raise KernelLibraryError(f"symbol {name} not found in {_LIB_PATH}; rebuild the kernel library")
    return f


def declare(name: str, argtypes, restype=i32):
    """Declare the signature of a symbol added after the table above (multi-GPU kernels)."""
    f = fn(name)
    f.argtypes = argtypes
    f.restype = restype
    return f


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


LAUNCHES = 0   # native launcher calls made through this module (each is >= 1 kernel launch)


def check(err: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if err != 0:
        raise KernelLibraryError(f"{what}: CUDA error code {err}")


def use_cuda(t: torch.Tensor) -> bool:
    """True when `t` lives on a GPU, in which case the native kernels must be used."""
    return t.is_cuda
