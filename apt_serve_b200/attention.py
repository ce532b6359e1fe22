"""Attention backend of the hybrid-cache path, with the interface of the
reference's ``additional_designs/attention/backends/aptserve_flash_attn.py``
(``FlashAttentionBackend``, ``FlashAttentionMetadata``, ``FlashAttentionImpl``)
and ``additional_designs/attention/aptserve_layer.py`` (``Attention``), so the
reference's model code, cache engine and model runner can call it unchanged.

Two ways in:

* ``FlashAttentionImpl.forward`` keeps the reference's argument list and its op
  sequence (cache-write branch selection of aptserve_flash_attn.py:331-387,
  decode attention of :449-475); each op behind it is one of this package's
  kernels.
* ``hybrid_decode_attention`` / ``FlashAttentionImpl.forward_hybrid_decode`` is
  the fused call: K/V requests stream their private K/V blocks, hidden requests
  are re-projected from their hidden blocks inside the kernel, and neither the
  ``hidden_holder`` buffer nor the shared cache is touched.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, List, Optional, Tuple, Type

import torch

from . import _native as N
from . import mixed_cache_ops, ops
from .metadata import derive_private_block_tables

# ----------------------------------------------------------------------------- #
# scratch
# ----------------------------------------------------------------------------- #
_workspaces: Dict[torch.device, torch.Tensor] = {}


def attention_workspace(device: torch.device, batch: int, max_blocks: int, block_size: int,
                        heads: int, head_size: int) -> torch.Tensor:
    """A per-device scratch tensor large enough for the given batch (grown on
    demand, reused by later calls on the same stream)."""
    need = N.lib().aps_attention_workspace_bytes(batch, max_blocks, block_size, heads, head_size)
    ws = _workspaces.get(device)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[device] = ws
    return ws


def attention_status(workspace: torch.Tensor) -> int:
    """Status word left by the last attention call that used ``workspace``
    (0 = fine).  Synchronises the current stream."""
    import ctypes
    host = ctypes.c_int(0)
    dev = workspace.device
    with torch.cuda.device(dev):
        N.check(N.lib().aps_attention_status(N.ptr(workspace), ctypes.addressof(host),
                                             N.current_stream(dev)))
    return host.value


def reprojection_cycles(workspace: torch.Tensor) -> int:
    """SM clock cycles CTA 0 of the re-projection kernel spent in the last hybrid call that
    used ``workspace``.  Synchronises the current stream."""
    import ctypes
    host = ctypes.c_ulonglong(0)
    dev = workspace.device
    with torch.cuda.device(dev):
        N.check(N.lib().aps_reprojection_cycles(N.ptr(workspace), ctypes.addressof(host),
                                                N.current_stream(dev)))
    return host.value


def raise_on_device_status(workspace: Optional[torch.Tensor] = None,
                           device: Optional[torch.device] = None) -> None:
    """Raise ``RuntimeError`` if the last attention call on ``workspace`` (default: the
    per-device workspace of ``device``) left a non-zero status word: 1..7 = a bounded wait
    of the re-projection kernel ran out and the call's output is NaN, 8 = K/V-cached
    requests in a batch that was given no K/V cache.  Synchronises the current stream, so
    call it where a synchronisation is cheap (once per engine step, beside the sampler's
    device-to-host copy), not per layer."""
    if workspace is None:
        workspace = _workspaces.get(torch.device(device) if device is not None
                                    else torch.device("cuda", torch.cuda.current_device()))
        if workspace is None:
            return
    code = attention_status(workspace)
    if code != 0:
        what = ("a bounded device-side wait ran out; the output was filled with NaN" if code < 8 else
                "the batch holds K/V-cached requests but no K/V cache was passed; their rows are zero")
        raise RuntimeError(f"aptserve_b200: attention status {code}: {what}")


def _i32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int32:
        raise RuntimeError(f"{name} must be int32 (got {t.dtype})")
    return t if t.is_contiguous() else t.contiguous()


# ----------------------------------------------------------------------------- #
# functional entry points
# ----------------------------------------------------------------------------- #
def paged_decode_attention(query: torch.Tensor, key_cache: torch.Tensor,
                           value_cache: torch.Tensor, block_tables: torch.Tensor,
                           seq_lens: torch.Tensor, scale: float,
                           out: Optional[torch.Tensor] = None,
                           workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode attention over K/V blocks: ``query [B, H*D]``, caches
    ``[NB, BS, H, D]``, ``block_tables`` int32 ``[B, max_blocks]``, ``seq_lens``
    int32 ``[B]`` -> ``[B, H*D]`` (the ``flash_attn_with_kvcache`` call of
    aptserve_flash_attn.py:452-461)."""
    dev = N.require_cuda(query, key_cache, value_cache, block_tables, seq_lens)
    b = query.shape[0]
    _, bs, h, d = key_cache.shape
    if out is None:
        out = torch.empty_like(query)
    if b == 0:
        return out
    if key_cache.stride(0) != value_cache.stride(0):
        raise RuntimeError("paged_decode_attention: cache block strides differ")
    bt = _i32(block_tables, "block_tables")
    sl = _i32(seq_lens, "seq_lens")
    if workspace is None:
        workspace = attention_workspace(dev, b, bt.shape[1], bs, h, d)
    with torch.cuda.device(dev):
        N.check(N.lib().aps_paged_decode_attention(
            N.ptr(out), N.ptr(query), N.ptr(key_cache), N.ptr(value_cache), N.ptr(bt), N.ptr(sl),
            b, bt.shape[1], h, d, bs, query.stride(0), out.stride(0), key_cache.stride(0),
            float(scale), N.ptr(workspace), workspace.numel(), N.dtype_enum(query),
            N.current_stream(dev)))
    return out


def hybrid_decode_attention(query: torch.Tensor, kv_cache: Optional[torch.Tensor],
                            hidden_cache: torch.Tensor, w_k: torch.Tensor,
                            b_k: Optional[torch.Tensor], w_v: torch.Tensor,
                            b_v: Optional[torch.Tensor], block_tables: torch.Tensor,
                            seq_lens: torch.Tensor, cache_type: torch.Tensor, scale: float,
                            num_heads: Optional[int] = None, head_size: Optional[int] = None,
                            out: Optional[torch.Tensor] = None,
                            workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Fused hybrid decode attention.

    ``kv_cache``: the layer's ``[2, NB, BS, H, D]`` tensor (``None`` when every
    request is hidden-cached); ``hidden_cache``: the tensor whose flat rows of
    ``stride(2)`` elements hold the hidden states -- the same tensor as
    ``kv_cache`` for the reference layout, a ``[2, NB, BS, 1, E]`` tensor under
    tensor parallelism; ``w_k`` / ``w_v``: ``[H*D, E]`` (rows of this rank's
    heads); ``block_tables``: int32 ``[B, max_blocks]`` *private* tables (a hidden
    request's odd logical blocks carry V-plane ids >= NB); ``cache_type``: int32
    ``[B]``, non-zero for hidden-cached requests.
    """
    dev = N.require_cuda(query, kv_cache, hidden_cache, w_k, b_k, w_v, b_v, block_tables,
                         seq_lens, cache_type)
    b = query.shape[0]
    if out is None:
        out = torch.empty_like(query)
    if b == 0:
        return out
    if kv_cache is not None:
        _, _, bs, h, d = kv_cache.shape
        kc, vc, block_stride = kv_cache[0], kv_cache[1], kv_cache.stride(1)
    else:
        if num_heads is None or head_size is None:
            raise RuntimeError("hybrid_decode_attention: num_heads / head_size needed without kv_cache")
        bs, h, d = hidden_cache.shape[2], num_heads, head_size
        kc = vc = None
        block_stride = bs * h * d
    e = w_k.shape[1]
    if w_k.shape != w_v.shape or w_k.stride(0) != w_v.stride(0) or w_k.stride(1) != 1:
        raise RuntimeError("hybrid_decode_attention: W_k / W_v must be row-major with equal strides")
    if w_k.shape[0] != h * d:
        raise RuntimeError("hybrid_decode_attention: W_k has %d rows, expected H*D = %d"
                           % (w_k.shape[0], h * d))
    row_stride = hidden_cache.stride(2)
    n_rows = hidden_cache.numel() // row_stride
    bt = _i32(block_tables, "block_tables")
    sl = _i32(seq_lens, "seq_lens")
    ct = _i32(cache_type, "cache_type")
    if workspace is None:
        workspace = attention_workspace(dev, b, bt.shape[1], bs, h, d)
    with torch.cuda.device(dev):
        N.check(N.lib().aps_hybrid_decode_attention(
            N.ptr(out), N.ptr(query), N.ptr(kc), N.ptr(vc), N.ptr(hidden_cache), N.ptr(w_k),
            N.ptr(b_k), N.ptr(w_v), N.ptr(b_v), N.ptr(bt), N.ptr(sl), N.ptr(ct), b, bt.shape[1],
            h, d, e, bs, query.stride(0), out.stride(0), block_stride, row_stride, n_rows,
            w_k.stride(0), float(scale), N.ptr(workspace), workspace.numel(),
            N.dtype_enum(query), N.current_stream(dev)))
    return out


def decode_layer_step(query: torch.Tensor, hidden_states: Optional[torch.Tensor],
                      new_key: Optional[torch.Tensor], new_value: Optional[torch.Tensor],
                      kv_cache: Optional[torch.Tensor], hidden_cache: torch.Tensor,
                      w_k: torch.Tensor, b_k: Optional[torch.Tensor], w_v: torch.Tensor,
                      b_v: Optional[torch.Tensor], block_tables: torch.Tensor,
                      seq_lens: torch.Tensor, cache_type: torch.Tensor, scale: float,
                      num_heads: Optional[int] = None, head_size: Optional[int] = None,
                      out: Optional[torch.Tensor] = None,
                      workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One decode layer-step in one native call (``aps_decode_layer_step``): the new token's
    cache writes -- ``hidden_states[r]`` into the hidden cache for hidden-cached requests
    (aptserve_opt.py:108-109), ``new_key[r]`` / ``new_value[r]`` into the K/V planes for
    K/V-cached requests (aptserve_flash_attn.py:338-345, 363-373) -- addressed from the
    private block tables, then ``hybrid_decode_attention`` over the batch.  ``new_key`` /
    ``new_value``: ``[B, H*D]`` (or ``[B, H, D]``) with any row stride; rows of requests of
    the other cache type are ignored.  ``None`` skips that kind of write."""
    dev = N.require_cuda(query, hidden_states, new_key, new_value, kv_cache, hidden_cache, w_k, b_k,
                         w_v, b_v, block_tables, seq_lens, cache_type)
    b = query.shape[0]
    if out is None:
        out = torch.empty_like(query)
    if b == 0:
        return out
    if kv_cache is not None:
        _, _, bs, h, d = kv_cache.shape
        kc, vc, block_stride = kv_cache[0], kv_cache[1], kv_cache.stride(1)
    else:
        if num_heads is None or head_size is None:
            raise RuntimeError("decode_layer_step: num_heads / head_size needed without kv_cache")
        bs, h, d = hidden_cache.shape[2], num_heads, head_size
        kc = vc = None
        block_stride = bs * h * d
        new_key = new_value = None
    e = w_k.shape[1]
    if w_k.shape != w_v.shape or w_k.stride(0) != w_v.stride(0) or w_k.stride(1) != 1:
        raise RuntimeError("decode_layer_step: W_k / W_v must be row-major with equal strides")
    if w_k.shape[0] != h * d:
        raise RuntimeError("decode_layer_step: W_k has %d rows, expected H*D = %d" % (w_k.shape[0], h * d))
    if (new_key is None) != (new_value is None):
        raise RuntimeError("decode_layer_step: new_key and new_value go together")
    for name, t in (("hidden_states", hidden_states), ("new_key", new_key), ("new_value", new_value)):
        if t is not None and (t.shape[0] != b or t.stride(-1) != 1):
            raise RuntimeError(f"decode_layer_step: {name} must hold one contiguous row per request")
    row_stride = hidden_cache.stride(2)
    n_rows = hidden_cache.numel() // row_stride
    bt = _i32(block_tables, "block_tables")
    sl = _i32(seq_lens, "seq_lens")
    ct = _i32(cache_type, "cache_type")
    if workspace is None:
        workspace = attention_workspace(dev, b, bt.shape[1], bs, h, d)
    with torch.cuda.device(dev):
        N.check(N.lib().aps_decode_layer_step(
            N.ptr(out), N.ptr(query), N.ptr(hidden_states), N.ptr(new_key), N.ptr(new_value),
            N.ptr(kc), N.ptr(vc), N.ptr(hidden_cache), N.ptr(w_k), N.ptr(b_k), N.ptr(w_v), N.ptr(b_v),
            N.ptr(bt), N.ptr(sl), N.ptr(ct), b, bt.shape[1], h, d, e, bs, query.stride(0), out.stride(0),
            0 if hidden_states is None else hidden_states.stride(0),
            0 if new_key is None else new_key.stride(0), 0 if new_value is None else new_value.stride(0),
            block_stride, row_stride, n_rows, w_k.stride(0), float(scale), N.ptr(workspace),
            workspace.numel(), N.dtype_enum(query), N.current_stream(dev)))
    return out


def absorbed_supported(num_heads: int, hidden_size: int, dtype: torch.dtype) -> bool:
    """Whether ``hybrid_decode_attention_absorbed`` takes this shape: fp16 / bf16, the head
    count padded to a multiple of 16 must be 16, 32, 48 or 80, hidden size a multiple of 512."""
    hp = (num_heads + 15) // 16 * 16
    return (dtype in (torch.float16, torch.bfloat16) and hp in (16, 32, 48, 80)
            and hidden_size % 512 == 0)


_absorbed_scratch: Dict[torch.device, Dict[str, torch.Tensor]] = {}


def _scratch(dev: torch.device, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
    """A per-device buffer that only grows (the scores / absorbed-query / weighted-sum scratch)."""
    bufs = _absorbed_scratch.setdefault(dev, {})
    t = bufs.get(name)
    if t is None or t.numel() < numel or t.dtype != dtype:
        t = torch.empty(numel, dtype=dtype, device=dev)
        bufs[name] = t
    return t[:numel]


def hybrid_decode_attention_absorbed(query: torch.Tensor, kv_cache: Optional[torch.Tensor],
                                     hidden_cache: torch.Tensor, w_k: torch.Tensor,
                                     b_k: Optional[torch.Tensor], w_v: torch.Tensor,
                                     b_v: Optional[torch.Tensor], block_tables: torch.Tensor,
                                     seq_lens: torch.Tensor, cache_type: torch.Tensor, scale: float,
                                     hidden_rows: Optional[torch.Tensor] = None,
                                     num_heads: Optional[int] = None, head_size: Optional[int] = None,
                                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Hybrid decode attention with the projections of hidden-cached requests absorbed into
    the query and the output instead of re-projecting every cached row: same arguments and
    result as ``hybrid_decode_attention`` (``b_k`` cancels in the softmax and is unused).

    ``scores = X (W_k,h^T q)``, ``z = softmax(scores)^T X``, ``out_h = W_v,h z + b_v``: the fold
    and the unfold are one batched GEMM each (library calls), the two passes over the cached
    hidden rows are ``aps_absorbed_hidden_attention``.  K/V-cached requests take the K/V
    streaming path.  ``hidden_rows``: the batch rows of the hidden-cached requests
    (``hidden_cache_use_input`` of the metadata); derived from ``cache_type`` with a host
    synchronisation when absent.
    """
    dev = N.require_cuda(query, kv_cache, hidden_cache, w_k, w_v, b_v, block_tables, seq_lens, cache_type)
    b = query.shape[0]
    if out is None:
        out = torch.empty_like(query)
    if b == 0:
        return out
    if kv_cache is not None:
        _, _, bs, h, d = kv_cache.shape
    else:
        if num_heads is None or head_size is None:
            raise RuntimeError("hybrid_decode_attention_absorbed: num_heads / head_size needed without kv_cache")
        bs, h, d = hidden_cache.shape[2], num_heads, head_size
    e = w_k.shape[1]
    if query.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("hybrid_decode_attention_absorbed: fp16 or bf16 only")
    bt = _i32(block_tables, "block_tables")
    sl = _i32(seq_lens, "seq_lens")
    ct = _i32(cache_type, "cache_type")
    if hidden_rows is None:
        hidden_rows = torch.nonzero(ct, as_tuple=False).flatten()
    n_h = int(hidden_rows.shape[0])
    max_tokens = bt.shape[1] * bs
    # K/V-cached requests: the streaming path over the whole batch, hidden requests with length 0
    if kv_cache is not None and n_h < b:
        paged_decode_attention(query, kv_cache[0], kv_cache[1], bt, torch.where(ct != 0, torch.zeros_like(sl), sl),
                               scale, out=out)
    if n_h == 0:
        return out
    rows64 = hidden_rows.to(torch.int64)
    # longest requests first: the kernels' CTAs are dispatched in request order and a CTA's
    # run time grows with its request's length
    rows64 = rows64[torch.argsort(sl.index_select(0, rows64), descending=True)]
    rows32 = rows64.to(torch.int32)
    hp = (h + 15) // 16 * 16
    log2e = 1.4426950408889634
    with torch.cuda.device(dev):
        # fold: qa[h][i] = scale * log2(e) * W_k,h^T q[i][h]  (one batched GEMM over the heads,
        # written in place: the kernels take the head-major layout)
        q_h = (query.index_select(0, rows64).view(n_h, h, d).transpose(0, 1).float() * (scale * log2e)).to(query.dtype)
        qa = _scratch(dev, "qa", hp * n_h * e, query.dtype).view(hp, n_h, e)
        if hp != h:
            qa[h:].zero_()
        torch.bmm(q_h, w_k.view(h, d, e), out=qa[:h])
        lens = sl.index_select(0, rows64).clamp(max=max_tokens).to(torch.int64)
        tok_offset = torch.zeros(n_h + 1, dtype=torch.int64, device=dev)
        torch.cumsum(lens, 0, out=tok_offset[1:])
        scores = _scratch(dev, "scores", n_h * max_tokens * hp, torch.float32)
        probs = _scratch(dev, "probs", n_h * max_tokens * hp, query.dtype)
        z = _scratch(dev, "z", hp * n_h * e, query.dtype).view(hp, n_h, e)
        row_stride = hidden_cache.stride(2)
        N.check(N.lib().aps_absorbed_hidden_attention(
            N.ptr(z), N.ptr(scores), N.ptr(probs), N.ptr(hidden_cache), N.ptr(qa), N.ptr(bt), N.ptr(sl), N.ptr(rows32),
            N.ptr(tok_offset), n_h, bt.shape[1], bs, e, hp, row_stride, hidden_cache.numel() // row_stride,
            N.dtype_enum(query), N.current_stream(dev)))
        # unfold: out[i][h] = W_v,h z[i][h] + b_v
        o = torch.bmm(z[:h], w_v.view(h, d, e).transpose(1, 2))                          # [h, n_h, d]
        if b_v is not None:
            o = o + b_v.view(h, 1, d)
        out.index_copy_(0, rows64, o.transpose(0, 1).reshape(n_h, h * d).to(out.dtype))
    return out


def kv_reprojection(x: torch.Tensor, w_k: torch.Tensor, b_k: Optional[torch.Tensor],
                    w_v: torch.Tensor, b_v: Optional[torch.Tensor], head_size: int,
                    block_ids: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``kv = [X W_k^T + b_k | X W_v^T + b_v]`` on the tensor cores (the
    ``kv_only`` projection of aptserve_linear.py:123-130).  ``x`` is a dense
    ``[N, E]`` matrix, or -- with ``block_ids`` (int32) -- a paged cache
    ``[2, NB, BS, H, D]`` whose flat rows of ``stride(2)`` elements are read in
    16-row blocks."""
    dev = N.require_cuda(x, w_k, b_k, w_v, b_v, block_ids)
    hd, e = w_k.shape
    if block_ids is None:
        if x.dim() != 2:
            raise RuntimeError("kv_reprojection: dense input must be [N, E]")
        rows_total, row_stride = x.shape[0], x.stride(0)
        n = rows_total if n_rows is None else n_rows
    else:
        row_stride = x.stride(2) if x.dim() == 5 else x.stride(-2)
        rows_total = x.numel() // row_stride
        n = block_ids.numel() * 16 if n_rows is None else n_rows
        block_ids = _i32(block_ids, "block_ids")
    if out is None:
        out = torch.empty(n, 2 * hd, dtype=x.dtype, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        N.check(N.lib().aps_kv_reprojection(
            N.ptr(out), N.ptr(x), N.ptr(block_ids), n, N.ptr(w_k), N.ptr(b_k), N.ptr(w_v),
            N.ptr(b_v), hd // head_size, head_size, e, row_stride, rows_total, w_k.stride(0),
            out.stride(0), N.dtype_enum(x), N.ptr(status), N.current_stream(dev)))
    return out


# ----------------------------------------------------------------------------- #
# backend classes (reference interface)
# ----------------------------------------------------------------------------- #
class FlashAttentionBackend:
    """Static API of aptserve_flash_attn.py:15-65."""

    @staticmethod
    def get_supported_head_sizes() -> List[int]:
        # what the decode kernels take (the reference's flash-attn list, aptserve_flash_attn.py:19,
        # also names 96, 160, 192, 224; OPT uses 64 and 128)
        return [32, 64, 128, 256]

    @staticmethod
    def get_name() -> str:
        return "flash-attn"

    @staticmethod
    def get_impl_cls() -> Type["FlashAttentionImpl"]:
        return FlashAttentionImpl

    @staticmethod
    def make_metadata(*args, **kwargs) -> "FlashAttentionMetadata":
        return FlashAttentionMetadata(*args, **kwargs)

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int,
                           head_size: int) -> Tuple[int, ...]:
        if block_size % 16 != 0:
            raise ValueError("Block size must be a multiple of 16.")
        return (2, num_blocks, block_size, num_kv_heads, head_size)

    @staticmethod
    def swap_blocks(src_kv_cache: torch.Tensor, dst_kv_cache: torch.Tensor,
                    src_to_dst: torch.Tensor) -> None:
        for plane in (0, 1):
            ops.swap_blocks(src_kv_cache[plane], dst_kv_cache[plane], src_to_dst)

    @staticmethod
    def copy_blocks(kv_caches: List[torch.Tensor], src_to_dists: torch.Tensor) -> None:
        ops.copy_blocks([c[0] for c in kv_caches], [c[1] for c in kv_caches], src_to_dists)


@dataclass
class FlashAttentionMetadata:
    """Field names, order and meaning of aptserve_abstract.py:55-80 followed by
    aptserve_flash_attn.py:68-125."""
    num_prefills: int
    num_prefill_tokens: int
    num_decode_tokens: int
    num_hidden_cache_tokens: int
    num_tot_tokens: int
    slot_mapping: torch.Tensor
    slot_mapping_shared: torch.Tensor
    hidden_cache_use_tot: torch.Tensor
    kv_cache_use_tot: torch.Tensor
    hidden_cache_use_input: torch.Tensor
    hidden_cache_store_tot: torch.Tensor
    hidden_holder_upd: torch.Tensor
    hidden_holder_pull: torch.Tensor
    seq_lens: Optional[List[int]]
    seq_lens_tensor: Optional[torch.Tensor]
    max_query_len: Optional[int]
    max_prefill_seq_len: int
    max_decode_seq_len: int
    query_start_loc: Optional[torch.Tensor]
    seq_start_loc: Optional[torch.Tensor]
    context_lens_tensor: Optional[torch.Tensor]
    block_tables: Optional[torch.Tensor]
    use_cuda_graph: bool
    _cached_prefill_metadata: Optional["FlashAttentionMetadata"] = None
    _cached_decode_metadata: Optional["FlashAttentionMetadata"] = None

    @property
    def prefill_metadata(self) -> Optional["FlashAttentionMetadata"]:
        """The prefill slice of a batch (aptserve_flash_attn.py:127-177)."""
        if self.num_prefills == 0:
            return None
        if self._cached_prefill_metadata is None:
            n, t = self.num_prefills, self.num_prefill_tokens
            self._cached_prefill_metadata = replace(
                self, num_decode_tokens=0, slot_mapping=self.slot_mapping[:t],
                seq_lens=self.seq_lens[:n], seq_lens_tensor=self.seq_lens_tensor[:n],
                max_decode_seq_len=0, query_start_loc=self.query_start_loc[:n + 1],
                seq_start_loc=self.seq_start_loc[:n + 1],
                context_lens_tensor=self.context_lens_tensor[:n],
                block_tables=self.block_tables[:n], use_cuda_graph=False,
                _cached_prefill_metadata=None, _cached_decode_metadata=None)
        return self._cached_prefill_metadata

    @property
    def decode_metadata(self) -> Optional["FlashAttentionMetadata"]:
        """The decode slice of a batch (aptserve_flash_attn.py:179-222)."""
        if self.num_decode_tokens == 0:
            return None
        if self._cached_decode_metadata is None:
            n, t = self.num_prefills, self.num_prefill_tokens
            self._cached_decode_metadata = replace(
                self, num_prefills=0, num_prefill_tokens=0, slot_mapping=self.slot_mapping[t:],
                seq_lens=None, seq_lens_tensor=self.seq_lens_tensor[n:], max_query_len=None,
                max_prefill_seq_len=0, query_start_loc=None, seq_start_loc=None,
                context_lens_tensor=None, block_tables=self.block_tables[n:],
                _cached_prefill_metadata=None, _cached_decode_metadata=None)
        return self._cached_decode_metadata

    @classmethod
    def from_decode(cls, meta) -> "FlashAttentionMetadata":
        """Wrap a ``metadata.DecodeMetadata`` (decode-only batch)."""
        return cls(num_prefills=0, num_prefill_tokens=0, num_decode_tokens=meta.num_decode_tokens,
                   num_hidden_cache_tokens=meta.num_hidden_cache_tokens,
                   num_tot_tokens=meta.num_tot_tokens, slot_mapping=meta.slot_mapping,
                   slot_mapping_shared=meta.slot_mapping_shared,
                   hidden_cache_use_tot=meta.hidden_cache_use_tot,
                   kv_cache_use_tot=meta.kv_cache_use_tot,
                   hidden_cache_use_input=meta.hidden_cache_use_input,
                   hidden_cache_store_tot=meta.hidden_cache_store_tot,
                   hidden_holder_upd=meta.hidden_holder_upd,
                   hidden_holder_pull=meta.hidden_holder_pull, seq_lens=meta.seq_lens,
                   seq_lens_tensor=meta.seq_lens_tensor, max_query_len=1, max_prefill_seq_len=0,
                   max_decode_seq_len=meta.max_decode_seq_len, query_start_loc=None,
                   seq_start_loc=None, context_lens_tensor=None, block_tables=meta.block_tables,
                   use_cuda_graph=False)

    @classmethod
    def from_prefill(cls, meta) -> "FlashAttentionMetadata":
        """Wrap a ``metadata.PrefillMetadata`` (prefill-only batch, no prefix cache)."""
        dev = meta.slot_mapping.device
        lens = torch.tensor(meta.seq_lens, dtype=torch.int32, device=dev)
        return cls(num_prefills=meta.num_prefills, num_prefill_tokens=meta.num_prefill_tokens,
                   num_decode_tokens=0, num_hidden_cache_tokens=meta.num_hidden_cache_tokens,
                   num_tot_tokens=meta.num_tot_tokens, slot_mapping=meta.slot_mapping,
                   slot_mapping_shared=meta.slot_mapping_shared,
                   hidden_cache_use_tot=meta.hidden_cache_use_tot,
                   kv_cache_use_tot=meta.kv_cache_use_tot,
                   hidden_cache_use_input=meta.hidden_cache_use_input,
                   hidden_cache_store_tot=meta.hidden_cache_store_tot,
                   hidden_holder_upd=meta.hidden_holder_upd,
                   hidden_holder_pull=meta.hidden_holder_pull, seq_lens=meta.seq_lens,
                   seq_lens_tensor=lens, max_query_len=meta.max_prefill_seq_len,
                   max_prefill_seq_len=meta.max_prefill_seq_len, max_decode_seq_len=0,
                   query_start_loc=meta.seq_start_loc, seq_start_loc=meta.seq_start_loc,
                   context_lens_tensor=torch.zeros_like(lens),
                   block_tables=torch.zeros(meta.num_prefills, 0, dtype=torch.int32, device=dev),
                   use_cuda_graph=False)


def _varlen_prefill_attention(q, k, v, seq_start_loc, max_len, scale):
    """Causal var-len self-attention over packed prompts.  Prefill attention is
    not one of the rewritten kernels: it stays a library call, as in the
    reference (flash_attn_varlen_func, aptserve_flash_attn.py:414-426)."""
    try:
        from flash_attn import flash_attn_varlen_func
        if q.dtype in (torch.float16, torch.bfloat16):
            return flash_attn_varlen_func(q, k, v, cu_seqlens_q=seq_start_loc,
                                          cu_seqlens_k=seq_start_loc, max_seqlen_q=max_len,
                                          max_seqlen_k=max_len, softmax_scale=scale, causal=True)
    except ImportError:
        pass
    out = torch.empty_like(q)
    bounds = seq_start_loc.tolist()
    for a, b in zip(bounds[:-1], bounds[1:]):
        o = torch.nn.functional.scaled_dot_product_attention(
            q[a:b].transpose(0, 1)[None], k[a:b].transpose(0, 1)[None],
            v[a:b].transpose(0, 1)[None], is_causal=True, scale=scale)
        out[a:b] = o[0].transpose(0, 1)
    return out


def _prefix_prefill_attention(query, key_cache, value_cache, query_start_loc, seq_lens,
                              block_tables, scale):
    """Prefix-enabled prefill (aptserve_flash_attn.py:432-447): the new prompt tokens of each
    sequence attend to the sequence's whole context, read through its block table from the
    cache the step has just written; causal with the query rows aligned to the END of the
    context.  Like the prefill attention without a prefix it stays a composition of library
    calls (a gather by block id and scaled_dot_product_attention per sequence); the reference
    calls flash_attn_varlen_func with ``block_table``."""
    out = torch.empty_like(query)
    bounds = query_start_loc.tolist()
    bs = key_cache.shape[1]
    for i, (a, b) in enumerate(zip(bounds[:-1], bounds[1:])):
        n_q, n_ctx = b - a, int(seq_lens[i])
        if n_q == 0:
            continue
        ids = block_tables[i, :(n_ctx + bs - 1) // bs].long()
        k = key_cache.index_select(0, ids).flatten(0, 1)[:n_ctx]
        v = value_cache.index_select(0, ids).flatten(0, 1)[:n_ctx]
        pos = torch.arange(n_ctx, device=query.device)
        mask = pos[None, :] <= (n_ctx - n_q + torch.arange(n_q, device=query.device))[:, None]
        o = torch.nn.functional.scaled_dot_product_attention(
            query[a:b].transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None],
            attn_mask=mask, scale=scale)
        out[a:b] = o[0].transpose(0, 1)
    return out


class FlashAttentionImpl:
    """Same constructor and ``forward`` signature as aptserve_flash_attn.py:251-299."""

    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int,
                 alibi_slopes: Optional[List[float]], sliding_window: Optional[int],
                 kv_cache_dtype: str, blocksparse_params: Optional[Dict[str, Any]] = None) -> None:
        assert blocksparse_params is None, ValueError(
            "FlashAttention does not support block-sparse attention.")
        self.num_heads = num_heads
        self.head_size = head_size
        self.scale = float(scale)
        self.num_kv_heads = num_kv_heads
        if alibi_slopes is not None:
            raise ValueError("alibi slopes are not supported by the hybrid-cache kernels "
                             "(OPT uses none)")
        self.alibi_slopes = None
        self.sliding_window = (-1, -1)
        self.kv_cache_dtype = kv_cache_dtype
        assert self.num_heads % self.num_kv_heads == 0
        self.num_queries_per_kv = self.num_heads // self.num_kv_heads
        if self.num_queries_per_kv != 1:
            raise ValueError("grouped-query attention is not supported: the hybrid cache "
                             "slices the fused QKV weight in thirds (MHA only)")
        if sliding_window is not None:
            raise ValueError("Sliding window is not supported in FlashAttention.")
        supported = FlashAttentionBackend.get_supported_head_sizes()
        if head_size not in supported:
            raise ValueError(f"Head size {head_size} is not supported by FlashAttention. "
                             f"Supported head sizes are: {supported}.")

    # -- reference op sequence ------------------------------------------------- #
    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                kv_cache: Optional[torch.Tensor], shared_cache: Optional[torch.Tensor],
                attn_metadata: FlashAttentionMetadata, kv_scale: float = 1.0) -> torch.Tensor:
        """``query [T, H*D]``; ``key`` / ``value`` ``[T or N_tot, H*D]``;
        ``kv_cache [2, NB, BS, H, D]``; ``shared_cache [2, 2NB, BS, H, D]``
        -> ``[T, H*D]``.  Follows the reference step by step: which cache-write op
        runs (aptserve_flash_attn.py:331-387), var-len attention for prompts
        (:405-447), paged attention for decode tokens (:449-475)."""
        assert kv_scale == 1.0, "kv_scale is not supported in FlashAttention."
        num_tokens, hidden_size = query.shape
        query = query.view(-1, self.num_heads, self.head_size)
        key = key.view(-1, self.num_kv_heads, self.head_size)
        value = value.view(-1, self.num_kv_heads, self.head_size)
        m = attn_metadata
        n_hidden, n_prefill, n_decode = (m.num_hidden_cache_tokens, m.num_prefill_tokens,
                                         m.num_decode_tokens)
        if n_hidden == 0:
            assert key.shape[0] == n_prefill + n_decode
            assert value.shape[0] == n_prefill + n_decode

        shared_k = shared_v = None
        if kv_cache is not None:
            key_cache, value_cache = kv_cache[0], kv_cache[1]
            if n_hidden == 0:
                ops.reshape_and_cache_flash(key, value, key_cache, value_cache, m.slot_mapping,
                                            self.kv_cache_dtype)
            elif n_prefill != 0:
                # K/V are cached for the K/V-designated prompt tokens only: the rows listed in
                # kv_cache_use_tot go straight from the packed tensors to their slots, which
                # writes exactly what the reference's index-select copy
                # (reshape_and_cache_flash(key[kv_cache_use_tot], ...)) writes, without
                # materialising the gathered tensors
                ops.prefill_cache_write(key, value, None, kv_cache, None, m.slot_mapping,
                                        m.kv_cache_use_tot, None)
            else:
                shared_k, shared_v = shared_cache[0], shared_cache[1]
                if m.num_tot_tokens != len(m.slot_mapping_shared):
                    mixed_cache_ops.mixed_kv_to_cache(
                        key, value, key_cache, value_cache, shared_k, shared_v, m.slot_mapping,
                        m.slot_mapping_shared, m.kv_cache_use_tot, m.hidden_cache_use_tot)
                else:
                    ops.reshape_and_cache_flash(key, value, shared_k, shared_v,
                                                m.slot_mapping_shared, self.kv_cache_dtype)

        output = torch.empty_like(query)
        decode_query = query[n_prefill:]
        query, key, value = query[:n_prefill], key[:n_prefill], value[:n_prefill]
        assert query.shape[0] == n_prefill
        assert decode_query.shape[0] == n_decode

        if (prefill_meta := m.prefill_metadata) is not None:
            if (kv_cache is None or prefill_meta.block_tables is None
                    or prefill_meta.block_tables.numel() == 0):
                output[:n_prefill] = _varlen_prefill_attention(
                    query, key, value, prefill_meta.seq_start_loc,
                    prefill_meta.max_prefill_seq_len, self.scale)
            else:
                # prefix-enabled attention over the K/V cache (aptserve_flash_attn.py:432-447)
                assert prefill_meta.seq_lens is not None
                output[:n_prefill] = _prefix_prefill_attention(
                    query, key_cache, value_cache, prefill_meta.query_start_loc,
                    prefill_meta.seq_lens, prefill_meta.block_tables, self.scale)

        if (decode_meta := m.decode_metadata) is not None:
            kc, vc = (key_cache, value_cache) if n_hidden == 0 else (shared_k, shared_v)
            q2 = decode_query.reshape(n_decode, self.num_heads * self.head_size)
            o2 = output[n_prefill:].view(n_decode, self.num_heads * self.head_size)
            paged_decode_attention(q2, kc, vc, decode_meta.block_tables,
                                   decode_meta.seq_lens_tensor, self.scale, out=o2)
        return output.view(num_tokens, hidden_size)

    # -- fused decode ------------------------------------------------------------ #
    def forward_hybrid_decode(self, query: torch.Tensor, kv_cache: Optional[torch.Tensor],
                              hidden_cache: torch.Tensor, w_k: torch.Tensor,
                              b_k: Optional[torch.Tensor], w_v: torch.Tensor,
                              b_v: Optional[torch.Tensor],
                              attn_metadata, block_size: Optional[int] = None) -> torch.Tensor:
        """Decode attention of a batch that contains hidden-cached requests, fed
        from the reference's unchanged metadata: the private block tables and the
        cache-type mask are derived on device from ``slot_mapping``,
        ``hidden_holder_upd``, ``hidden_cache_use_input`` and ``seq_lens_tensor``
        unless the metadata already carries them."""
        tables = getattr(attn_metadata, "private_block_tables", None)
        ctype = getattr(attn_metadata, "cache_type", None)
        if tables is None or ctype is None:
            bs = block_size if block_size is not None else hidden_cache.shape[2]
            tables, ctype = derive_private_block_tables(attn_metadata, bs)
        return hybrid_decode_attention(query, kv_cache, hidden_cache, w_k, b_k, w_v, b_v, tables,
                                       attn_metadata.seq_lens_tensor, ctype, self.scale,
                                       num_heads=self.num_heads, head_size=self.head_size)


class Attention(torch.nn.Module):
    """``nn.Module`` wrapper with the reference's extra ``shared_cache`` argument
    (aptserve_layer.py:81-90)."""

    def __init__(self, num_heads: int, head_size: int, scale: float,
                 num_kv_heads: Optional[int] = None, alibi_slopes: Optional[List[float]] = None,
                 cache_config=None, quant_config=None, blocksparse_params=None) -> None:
        super().__init__()
        kv_cache_dtype = getattr(cache_config, "cache_dtype", "auto") if cache_config else "auto"
        sliding_window = getattr(cache_config, "sliding_window", None) if cache_config else None
        self._kv_scale = 1.0
        self.impl = FlashAttentionImpl(num_heads, head_size, scale,
                                       num_heads if num_kv_heads is None else num_kv_heads,
                                       alibi_slopes, sliding_window, kv_cache_dtype,
                                       blocksparse_params)

    def forward(self, query, key, value, kv_cache, shared_cache, attn_metadata) -> torch.Tensor:
        return self.impl.forward(query, key, value, kv_cache, shared_cache, attn_metadata,
                                 self._kv_scale)

    def extra_repr(self) -> str:
        return (f"head_size={self.impl.head_size}, num_heads={self.impl.num_heads}, "
                f"num_kv_heads={self.impl.num_kv_heads}, scale={self.impl.scale}, "
                f"backend={self.impl.__class__.__name__}")
