"""ctypes binding of ``lib/libaptserve_b200.so`` (the C ABI in
``include/aptserve_b200.h``).

There is no fallback: if the library is missing, every operator of this package
raises.  Build it with ``python -m apt_serve_b200.build``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libaptserve_b200.so"

APS_OK = 0
APS_ERR_NULL_POINTER = 1
APS_ERR_MISALIGNED = 2
APS_ERR_DTYPE = 3
APS_ERR_SHAPE = 4
APS_ERR_UNSUPPORTED = 5
APS_ERR_WORKSPACE = 6
APS_ERR_CUDA = 7
APS_ERR_DEVICE = 8

DTYPE_ENUM = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

# name -> (restype, argtypes); kept in step with include/aptserve_b200.h
PROTOTYPES = {
    "aps_last_error": (c_char_p, []),
    "aps_version": (c_char_p, []),
    "aps_reshape_and_cache": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_int, c_int, c_int64,
                                                       c_int64, c_int64, c_int, c_void_p]),
    "aps_hidden_to_cache": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_int64, c_int64, c_int,
                                                     c_void_p]),
    "aps_cache_to_hidden": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_int64, c_int64, c_int,
                                                     c_void_p]),
    "aps_mixed_kv_to_cache": (c_int, [c_void_p] * 10 + [c_int64, c_int64, c_int, c_int, c_int,
                                                        c_int64, c_int64, c_int64, c_int64, c_int,
                                                        c_void_p]),
    "aps_prefill_cache_write": (c_int, [c_void_p] * 8 + [c_int64, c_void_p, c_int64] + [c_int] * 4 +
                                [c_int64] * 5 + [c_int, c_void_p]),
    "aps_copy_blocks": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64, c_void_p]),
    "aps_swap_blocks": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                c_int64, c_int, c_void_p, c_void_p]),
    "aps_attention_workspace_bytes": (c_size_t, [c_int] * 5),
    "aps_paged_decode_attention": (c_int, [c_void_p] * 6 + [c_int] * 5 + [c_int64] * 3 +
                                   [c_float, c_void_p, c_size_t, c_int, c_void_p]),
    "aps_paged_decode_attention_static": (c_int, [c_void_p] * 6 + [c_int] * 5 + [c_int64] * 3 +
                                          [c_float, c_int, c_void_p]),
    "aps_hybrid_decode_attention": (c_int, [c_void_p] * 12 + [c_int] * 6 + [c_int64] * 6 +
                                    [c_float, c_void_p, c_size_t, c_int, c_void_p]),
    "aps_kv_reprojection": (c_int, [c_void_p] * 3 + [c_int64] + [c_void_p] * 4 + [c_int] * 3 +
                            [c_int64] * 4 + [c_int, c_void_p, c_void_p]),
    "aps_decode_layer_step": (c_int, [c_void_p] * 15 + [c_int] * 6 + [c_int64] * 9 +
                              [c_float, c_void_p, c_size_t, c_int, c_void_p]),
    "aps_attention_status": (c_int, [c_void_p, c_void_p, c_void_p]),
    "aps_reprojection_cycles": (c_int, [c_void_p, c_void_p, c_void_p]),
    "aps_cache_ops_status": (c_int, [c_void_p, c_void_p]),
    "aps_selftest_bounded_wait": (c_int, [c_void_p, c_size_t, ctypes.c_longlong, c_void_p] + [c_int] * 5 +
                                  [c_int64, c_int, c_void_p]),
    "aps_set_profile_events": (c_int, [c_int, c_void_p, c_void_p]),
    "aps_absorbed_hidden_attention": (c_int, [c_void_p] * 9 + [c_int] * 5 + [c_int64, c_int64, c_int, c_void_p]),
    "aps_tp_unique_id": (c_int, [c_void_p]),
    "aps_tp_init": (c_int, [c_void_p, c_void_p, c_int, c_int]),
    "aps_tp_allreduce": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "aps_tp_world_size": (c_int, [c_void_p, c_void_p]),
    "aps_tp_destroy": (c_int, [c_void_p]),
    "aps_decode_metadata_scratch_bytes": (c_size_t, [c_int]),
    "aps_expand_decode_metadata": (c_int, [c_void_p] * 4 + [c_int] * 3 + [c_void_p] * 8 +
                                   [c_int64, c_int64, c_void_p, c_void_p, c_size_t, c_void_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA extension has not been built "
                "(run `python -m apt_serve_b200.build`). There is no CPU or PyTorch fallback.")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int) -> None:
    """Turn a non-zero ``aps_status`` into the exception the reference would
    raise: ``ValueError`` for unsupported head / block sizes and dtypes
    (aptserve_flash_attn.py:40-41, 278-288), ``RuntimeError`` otherwise
    (``TORCH_CHECK`` in mixed_cache.cu:202)."""
    if status == APS_OK:
        return
    msg = lib().aps_last_error().decode("utf-8", "replace")
    if status in (APS_ERR_UNSUPPORTED, APS_ERR_DTYPE):
        raise ValueError(f"aptserve_b200: {msg} (status {status})")
    raise RuntimeError(f"aptserve_b200: {msg} (status {status})")


def dtype_enum(t: torch.Tensor) -> int:
    try:
        return DTYPE_ENUM[t.dtype]
    except KeyError:
        raise ValueError(f"aptserve_b200: dtype {t.dtype} is not supported") from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("aptserve_b200 operators run on CUDA tensors only "
                               "(there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("aptserve_b200: tensors live on different devices")
    return dev


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream
