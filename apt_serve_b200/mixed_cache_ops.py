"""Drop-in for the reference's ``mixed_cache_ops`` torch extension
(additional_designs/mixed_cache_kernels/mixed_cache.cu:233-237): same three
function names, same positional arguments, in-place on the caller's tensors,
enqueued on the current CUDA stream, returning ``None``.

Unlike the reference launchers (mixed_cache.cu:137,167 use the legacy default
stream) every op here runs on the current torch stream, and bf16 is accepted
next to fp32 / fp16.
"""
from __future__ import annotations

import torch

from . import _native as N


def _idx(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int64:
        raise RuntimeError(f"{name} must be an int64 tensor (got {t.dtype})")
    return t if t.is_contiguous() else t.contiguous()


def _rows(t: torch.Tensor, name: str):
    """A 2-D (or [T, H, D]) tensor whose rows are contiguous; returns the row stride."""
    if t.dim() < 2:
        raise RuntimeError(f"{name} must have at least 2 dimensions")
    inner = t[0]
    if t.shape[0] > 0 and not inner.is_contiguous():
        raise RuntimeError(f"{name}: rows must be contiguous")
    return t.stride(0)


def hidden_to_cache(hidden: torch.Tensor, paged_cache: torch.Tensor, slot_mapping: torch.Tensor,
                    src_idx: torch.Tensor, target_slot_idx: torch.Tensor) -> None:
    """``paged_cache`` row ``slot_mapping[target_slot_idx[i]]`` := ``hidden[src_idx[i]]``
    (mixed_cache.cu:119-147).  ``paged_cache`` is the layer's ``[2, NB, BS, H, D]``
    tensor, addressed as flat rows of ``paged_cache.stride(2)`` elements."""
    dev = N.require_cuda(hidden, paged_cache, slot_mapping, src_idx, target_slot_idx)
    if hidden.dtype != paged_cache.dtype:
        raise RuntimeError("hidden_to_cache: hidden and paged_cache dtypes differ")
    n = src_idx.size(0)
    with torch.cuda.device(dev):
        N.check(N.lib().aps_hidden_to_cache(
            N.ptr(hidden), N.ptr(paged_cache), N.ptr(_idx(slot_mapping, "slot_mapping")),
            N.ptr(_idx(src_idx, "src_idx")), N.ptr(_idx(target_slot_idx, "target_slot_idx")),
            n, hidden.size(1), _rows(hidden, "hidden"), paged_cache.stride(2),
            N.dtype_enum(hidden), N.current_stream(dev)))


def cache_to_hidden(hidden: torch.Tensor, paged_cache: torch.Tensor, slot_mapping: torch.Tensor,
                    dst_idx: torch.Tensor) -> None:
    """``hidden[t] := paged_cache`` row ``slot_mapping[t]`` for ``t`` in ``dst_idx``
    (mixed_cache.cu:150-176)."""
    dev = N.require_cuda(hidden, paged_cache, slot_mapping, dst_idx)
    if hidden.dtype != paged_cache.dtype:
        raise RuntimeError("cache_to_hidden: hidden and paged_cache dtypes differ")
    with torch.cuda.device(dev):
        N.check(N.lib().aps_cache_to_hidden(
            N.ptr(hidden), N.ptr(paged_cache), N.ptr(_idx(slot_mapping, "slot_mapping")),
            N.ptr(_idx(dst_idx, "dst_idx")), dst_idx.size(0), hidden.size(1),
            _rows(hidden, "hidden"), paged_cache.stride(2), N.dtype_enum(hidden),
            N.current_stream(dev)))


def mixed_kv_to_cache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, shared_k_cache: torch.Tensor,
                      shared_v_cache: torch.Tensor, slot_mapping: torch.Tensor,
                      slot_mapping_shared: torch.Tensor, kv_cache_use_tot: torch.Tensor,
                      hidden_cache_use_tot: torch.Tensor) -> None:
    """Dual-destination K/V scatter of a hybrid decode batch (mixed_cache.cu:179-230).
    ``key`` / ``value``: ``[N_tot, H, D]``; caches ``[NB, BS, H, D]`` and
    ``[2 NB, BS, H, D]``."""
    dev = N.require_cuda(key, value, k_cache, v_cache, shared_k_cache, shared_v_cache,
                         slot_mapping, slot_mapping_shared, kv_cache_use_tot,
                         hidden_cache_use_tot)
    if k_cache.stride(0) != v_cache.stride(0):  # TORCH_CHECK at mixed_cache.cu:202
        raise RuntimeError("mixed_kv_to_cache: k_cache.stride(0) != v_cache.stride(0)")
    if shared_k_cache.stride(0) != shared_v_cache.stride(0):
        raise RuntimeError("mixed_kv_to_cache: shared cache strides differ")
    with torch.cuda.device(dev):
        N.check(N.lib().aps_mixed_kv_to_cache(
            N.ptr(key), N.ptr(value), N.ptr(k_cache), N.ptr(v_cache), N.ptr(shared_k_cache),
            N.ptr(shared_v_cache), N.ptr(_idx(slot_mapping, "slot_mapping")),
            N.ptr(_idx(slot_mapping_shared, "slot_mapping_shared")),
            N.ptr(_idx(kv_cache_use_tot, "kv_cache_use_tot")),
            N.ptr(_idx(hidden_cache_use_tot, "hidden_cache_use_tot")),
            kv_cache_use_tot.size(0), slot_mapping_shared.size(0), key.size(1), key.size(2),
            k_cache.size(1), _rows(key, "key"), _rows(value, "value"), k_cache.stride(0),
            shared_k_cache.stride(0), N.dtype_enum(key), N.current_stream(dev)))
