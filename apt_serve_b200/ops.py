"""The three ``vllm._custom_ops`` entry points the reference's attention backend
calls (additional_designs/attention/backends/aptserve_flash_attn.py:44-65,
338-385), with vLLM 0.5.0's signatures."""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from . import _native as N


def reshape_and_cache_flash(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor,
                            value_cache: torch.Tensor, slot_mapping: torch.Tensor,
                            kv_cache_dtype: str = "auto") -> None:
    """``key_cache[slot // BS, slot % BS] = key[t]`` (and value) for ``slot >= 0``.
    ``key`` / ``value``: ``[T, H, D]``; caches ``[NB, BS, H, D]``."""
    if kv_cache_dtype != "auto":  # aptserve_flash_attn.py:311-312: no FP8 cache here
        raise ValueError(f"kv_cache_dtype {kv_cache_dtype!r} is not supported")
    dev = N.require_cuda(key, value, key_cache, value_cache, slot_mapping)
    if slot_mapping.dtype != torch.int64:
        raise RuntimeError("slot_mapping must be int64")
    if key.dtype != key_cache.dtype or value.dtype != value_cache.dtype or key.dtype != value.dtype:
        raise RuntimeError("reshape_and_cache_flash: dtypes differ")
    if key_cache.stride(0) != value_cache.stride(0):
        raise RuntimeError("reshape_and_cache_flash: cache block strides differ")
    if key.shape[0] > 0 and not (key[0].is_contiguous() and value[0].is_contiguous()):
        raise RuntimeError("reshape_and_cache_flash: token rows must be contiguous")
    with torch.cuda.device(dev):
        N.check(N.lib().aps_reshape_and_cache(
            N.ptr(key), N.ptr(value), N.ptr(key_cache), N.ptr(value_cache),
            N.ptr(slot_mapping.contiguous()), slot_mapping.size(0), key.size(1), key.size(2),
            key_cache.size(1), key.stride(0), value.stride(0), key_cache.stride(0),
            N.dtype_enum(key), N.current_stream(dev)))


def prefill_cache_write(key: Optional[torch.Tensor], value: Optional[torch.Tensor],
                        hidden_states: Optional[torch.Tensor], kv_cache: Optional[torch.Tensor],
                        hidden_cache: Optional[torch.Tensor], slot_mapping: torch.Tensor,
                        kv_cache_use_tot: Optional[torch.Tensor],
                        hidden_cache_use_input: Optional[torch.Tensor]) -> None:
    """One launch for a prefill batch's cache writes: K/V rows of the K/V-designated
    prompt tokens (``kv_cache_use_tot``) into ``kv_cache``, layer-input rows of the
    hidden-designated ones (``hidden_cache_use_input``) into the flat rows of
    ``hidden_cache``; every token's slot is ``slot_mapping[token]``.  Stands in for
    ``hidden_to_cache`` + ``reshape_and_cache_flash(key[kv_cache_use_tot], ...)``
    (aptserve_opt.py:108-109, aptserve_flash_attn.py:347-355) without the gathered copies.
    ``key`` / ``value``: ``[T, H, D]``; ``hidden_states``: ``[T, E]``.  Either half may be left
    out (``None`` tensors and index list): only the other kind of row is written."""
    dev = N.require_cuda(key, value, hidden_states, kv_cache, hidden_cache, slot_mapping,
                         kv_cache_use_tot, hidden_cache_use_input)
    has_kv = kv_cache_use_tot is not None and kv_cache_use_tot.numel() > 0
    has_hid = hidden_cache_use_input is not None and hidden_cache_use_input.numel() > 0
    if not has_kv and not has_hid:
        return
    if has_kv and (key is None or value is None or kv_cache is None):
        raise RuntimeError("prefill_cache_write: K/V rows listed without key / value / kv_cache")
    if has_hid and (hidden_states is None or hidden_cache is None):
        raise RuntimeError("prefill_cache_write: hidden rows listed without hidden_states / hidden_cache")
    for t, name in ((slot_mapping, "slot_mapping"), (kv_cache_use_tot, "kv_cache_use_tot"),
                    (hidden_cache_use_input, "hidden_cache_use_input")):
        if t is not None and t.dtype != torch.int64:
            raise RuntimeError(f"{name} must be int64")
    used = [t for t in ((key, value, kv_cache) if has_kv else ()) + ((hidden_states, hidden_cache) if has_hid else ())]
    if any(t.dtype != used[0].dtype for t in used):
        raise RuntimeError("prefill_cache_write: dtypes differ")
    heads, head_size, block_size = ((key.size(1), key.size(2), kv_cache.size(2)) if has_kv
                                    else (1, 1, hidden_cache.size(2)))
    with torch.cuda.device(dev):
        N.check(N.lib().aps_prefill_cache_write(
            N.ptr(key) if has_kv else 0, N.ptr(value) if has_kv else 0, N.ptr(hidden_states) if has_hid else 0,
            N.ptr(kv_cache[0]) if has_kv else 0, N.ptr(kv_cache[1]) if has_kv else 0,
            N.ptr(hidden_cache) if has_hid else 0, N.ptr(slot_mapping.contiguous()),
            N.ptr(kv_cache_use_tot.contiguous()) if has_kv else 0, kv_cache_use_tot.numel() if has_kv else 0,
            N.ptr(hidden_cache_use_input.contiguous()) if has_hid else 0,
            hidden_cache_use_input.numel() if has_hid else 0, heads, head_size,
            hidden_states.size(1) if has_hid else 1, block_size,
            key.stride(0) if has_kv else 0, value.stride(0) if has_kv else 0,
            hidden_states.stride(0) if has_hid else 0, kv_cache.stride(1) if has_kv else 0,
            hidden_cache.stride(2) if has_hid else 0, N.dtype_enum(used[0]), N.current_stream(dev)))


def copy_blocks(key_caches: List[torch.Tensor], value_caches: List[torch.Tensor],
                block_mapping: torch.Tensor) -> None:
    """Copy-on-write block copies for every layer; ``block_mapping`` is an int64
    ``[n, 2]`` device tensor of ``(src, dst)`` block numbers."""
    if len(key_caches) != len(value_caches):
        raise RuntimeError("copy_blocks: key / value cache lists differ in length")
    if not key_caches or block_mapping.numel() == 0:
        return
    dev = N.require_cuda(block_mapping, *key_caches, *value_caches)
    if block_mapping.dtype != torch.int64:
        raise RuntimeError("copy_blocks: block_mapping must be int64")
    first = key_caches[0]
    block_bytes = first.stride(0) * first.element_size()
    for t in list(key_caches) + list(value_caches):
        if t.stride(0) * t.element_size() != block_bytes or not t[0].is_contiguous():
            raise RuntimeError("copy_blocks: every cache must have the same contiguous block layout")
    n = len(key_caches)
    karr = (ctypes.c_void_p * n)(*[t.data_ptr() for t in key_caches])
    varr = (ctypes.c_void_p * n)(*[t.data_ptr() for t in value_caches])
    with torch.cuda.device(dev):
        N.check(N.lib().aps_copy_blocks(karr, varr, n, N.ptr(block_mapping.contiguous()),
                                        block_mapping.size(0), block_bytes,
                                        N.current_stream(dev)))


def swap_blocks(src: torch.Tensor, dst: torch.Tensor, src_to_dst: torch.Tensor) -> int:
    """GPU <-> pinned-CPU block moves (aptserve_flash_attn.py:44-56): ``dst[d] = src[s]`` for
    every row ``(s, d)`` of ``src_to_dst`` (a CPU int64 tensor, as the reference passes it).
    ``src`` / ``dst`` are one plane ``[NB, BS, H, D]`` of a cache.  The copies are enqueued on the
    current stream of the CUDA side from a native loop (``aps_swap_blocks``), runs of consecutive
    blocks as one copy.  Returns the number of copies issued."""
    if src.is_cuda and dst.is_cuda:
        kind, dev = 2, src.device
    elif src.is_cuda:
        kind, dev = 1, src.device
    elif dst.is_cuda:
        kind, dev = 0, dst.device
    else:
        # both sides in host memory (the cache engine's bookkeeping exercised without a GPU):
        # a host copy per pair, no device work to enqueue
        pairs = src_to_dst.tolist()
        for s_id, d_id in pairs:
            dst[d_id].copy_(src[s_id])
        return len(pairs)
    if src.dtype != dst.dtype or src.shape[1:] != dst.shape[1:]:
        raise RuntimeError("swap_blocks: the two caches must hold blocks of the same shape and type")
    if not (src[0].is_contiguous() and dst[0].is_contiguous()):
        raise RuntimeError("swap_blocks: blocks must be contiguous")
    pairs = src_to_dst.detach().to("cpu", torch.int64).contiguous()
    if pairs.numel() == 0:
        return 0
    es = src.element_size()
    issued = ctypes.c_int64(0)
    with torch.cuda.device(dev):
        N.check(N.lib().aps_swap_blocks(
            src.data_ptr(), dst.data_ptr(), pairs.data_ptr(), pairs.size(0), src[0].numel() * es,
            src.stride(0) * es, dst.stride(0) * es, src.size(0), dst.size(0), kind,
            ctypes.addressof(issued), N.current_stream(dev)))
    return issued.value
