"""Model-side callers of the hybrid-cache ops, mirroring the attention part of
the reference's OPT model (additional_designs/model_executor/models/
aptserve_opt.py:60-134) and the two linear layers it relies on
(additional_designs/model_executor/layers/aptserve_linear.py:102-132, 315-328,
815-839).

The projections that are not part of the rewritten path (Q, fused QKV for
K/V-only batches, o_proj) stay ``F.linear`` library GEMMs; the tensor-parallel
reduction is one NCCL all-reduce issued through ``torch.distributed``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import mixed_cache_ops, ops
from .attention import (Attention, absorbed_supported, decode_layer_step, hybrid_decode_attention,
                        hybrid_decode_attention_absorbed)
from .metadata import derive_private_block_tables


def tensor_model_parallel_all_reduce(x: torch.Tensor, group=None) -> torch.Tensor:
    """Sum over the tensor-parallel group (the call at aptserve_linear.py:828-829).
    A no-op without an initialised process group or with a single rank.  Goes through
    the library's own communicator (``tp_comm.install``) when one is installed."""
    from . import tp_comm
    comm = tp_comm.installed()
    if comm is not None and group is None:
        return x if comm.world_size == 1 else comm.all_reduce(x)
    import torch.distributed as dist
    if not dist.is_available() or not dist.is_initialized():
        return x
    if dist.get_world_size(group) == 1:
        return x
    dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
    return x


class QKVParallelLinear(torch.nn.Module):
    """Fused QKV projection holding this rank's rows ``[q | k | v]``.
    ``forward(x, q_only, kv_only)`` slices the weight in thirds exactly like
    aptserve_linear.py:102-132 and returns ``(output, None)``."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor]):
        super().__init__()
        assert weight.shape[0] % 3 == 0
        self.weight = torch.nn.Parameter(weight, requires_grad=False)
        self.bias = None if bias is None else torch.nn.Parameter(bias, requires_grad=False)

    def slices(self):
        s = self.weight.shape[0] // 3
        b = self.bias
        return ((self.weight[:s], None if b is None else b[:s]),
                (self.weight[s:2 * s], None if b is None else b[s:2 * s]),
                (self.weight[2 * s:], None if b is None else b[2 * s:]))

    def forward(self, input_: torch.Tensor, q_only: bool = False, kv_only: bool = False):
        if q_only and kv_only:
            raise NotImplementedError
        s = self.weight.shape[0] // 3
        if q_only:
            w, b = self.weight[:s], None if self.bias is None else self.bias[:s]
        elif kv_only:
            w, b = self.weight[s:], None if self.bias is None else self.bias[s:]
        else:
            w, b = self.weight, self.bias
        return F.linear(input_, w, b), None


class RowParallelLinear(torch.nn.Module):
    """o_proj: this rank's columns of W_o; partial GEMM, all-reduce, then the bias
    once (aptserve_linear.py:815-839)."""

    def __init__(self, weight_shard: torch.Tensor, bias: Optional[torch.Tensor], group=None):
        super().__init__()
        self.weight = torch.nn.Parameter(weight_shard, requires_grad=False)
        self.bias = None if bias is None else torch.nn.Parameter(bias, requires_grad=False)
        self.group = group

    def forward(self, input_: torch.Tensor):
        out = tensor_model_parallel_all_reduce(F.linear(input_, self.weight), self.group)
        if self.bias is not None:
            out = out + self.bias
        return out, None


class OPTAttention(torch.nn.Module):
    """The reference's ``OPTAttention.forward(hidden_states, kv_cache,
    shared_cache, attn_metadata)`` (aptserve_opt.py:99-134).

    ``fused=True`` (default) collapses the decode branch with hidden-cached
    requests -- hidden_holder fill, ``cache_to_hidden`` gather, ``kv_only``
    projection, ``mixed_kv_to_cache`` scatter, paged attention over the shared
    cache -- into: Q projection, the new token's K/V projection and cache write
    for K/V requests, the new token's hidden row write for hidden requests, one
    hybrid decode attention call; a prefill batch with hidden-designated prompts
    writes both kinds of cache rows with one launch.  ``fused="absorbed"`` is the same with
    the hidden requests attended through absorbed projections (fp16 / bf16; shapes the absorbed
    kernels do not take -- see ``attention.absorbed_supported`` -- fall back to the re-projecting
    kernel).  ``fused=False`` runs the reference's op sequence literally on this package's kernels.

    Under tensor parallelism ``hidden_cache`` must be given (a
    ``[2, NB, BS, 1, E]`` tensor replicated per rank); with one rank it defaults
    to ``kv_cache``, the reference's aliasing layout.
    """

    def __init__(self, embed_dim: int, num_heads: int, qkv_weight: torch.Tensor,
                 qkv_bias: Optional[torch.Tensor], o_weight: torch.Tensor,
                 o_bias: Optional[torch.Tensor], tp_size: int = 1, group=None,
                 fused=True):
        super().__init__()
        assert num_heads % tp_size == 0
        self.embed_dim = embed_dim
        self.num_heads = num_heads // tp_size
        self.head_dim = embed_dim // num_heads
        self.scaling = self.head_dim ** -0.5
        self.qkv_proj = QKVParallelLinear(qkv_weight, qkv_bias)
        self.out_proj = RowParallelLinear(o_weight, o_bias, group)
        self.attn = Attention(self.num_heads, self.head_dim, scale=self.scaling)
        self.fused = fused

    def forward(self, hidden_states: torch.Tensor, kv_cache: torch.Tensor,
                shared_cache: Optional[torch.Tensor], attn_metadata,
                hidden_cache: Optional[torch.Tensor] = None) -> torch.Tensor:
        m = attn_metadata
        hcache = kv_cache if hidden_cache is None else hidden_cache
        if (self.fused and m.num_hidden_cache_tokens != 0 and m.num_decode_tokens == 0
                and kv_cache is not None):
            # prefill with hidden-designated prompts: one launch writes the K/V rows of the
            # K/V-designated tokens and the layer-input rows of the hidden-designated ones;
            # the attention below then runs without a cache (nothing left to write)
            qkv, _ = self.qkv_proj(hidden_states)
            q, k, v = qkv.chunk(chunks=3, dim=-1)
            ops.prefill_cache_write(k.view(-1, self.num_heads, self.head_dim),
                                    v.view(-1, self.num_heads, self.head_dim), hidden_states,
                                    kv_cache, hcache, m.slot_mapping, m.kv_cache_use_tot,
                                    m.hidden_cache_use_input)
            attn_output = self.attn(q, k, v, None, shared_cache, m)
            output, _ = self.out_proj(attn_output)
            return output
        if m.num_hidden_cache_tokens != 0:
            if m.num_decode_tokens != 0 and self.fused:
                # the new token's hidden rows are written by the fused step itself
                return self._fused_decode(hidden_states, kv_cache, hcache, m)
            mixed_cache_ops.hidden_to_cache(hidden_states, hcache, m.slot_mapping,
                                            m.hidden_cache_use_input, m.hidden_cache_store_tot)
            if m.num_decode_tokens != 0:
                holder = torch.zeros(m.num_tot_tokens, hidden_states.shape[1],
                                     device=hidden_states.device, dtype=hidden_states.dtype)
                q, _ = self.qkv_proj(hidden_states, q_only=True)
                holder[m.hidden_holder_upd] = hidden_states
                mixed_cache_ops.cache_to_hidden(holder, hcache, m.slot_mapping,
                                                m.hidden_cache_use_tot)
                kv, _ = self.qkv_proj(holder, kv_only=True)
                k, v = kv.chunk(chunks=2, dim=-1)
            else:
                qkv, _ = self.qkv_proj(hidden_states)
                q, k, v = qkv.chunk(chunks=3, dim=-1)
        else:
            qkv, _ = self.qkv_proj(hidden_states)
            q, k, v = qkv.chunk(chunks=3, dim=-1)
        attn_output = self.attn(q, k, v, kv_cache, shared_cache, m)
        output, _ = self.out_proj(attn_output)
        return output

    def use_absorbed(self, dtype: torch.dtype) -> bool:
        """``fused="absorbed"`` takes the absorbed kernels only for the shapes they are
        instantiated for; everything else runs the re-projecting kernel."""
        return self.fused == "absorbed" and absorbed_supported(self.num_heads, self.embed_dim, dtype)

    def _fused_decode(self, hidden_states, kv_cache, hidden_cache, m) -> torch.Tensor:
        (w_q, b_q), (w_k, b_k), (w_v, b_v) = self.qkv_proj.slices()
        tables = getattr(m, "private_block_tables", None)
        ctype = getattr(m, "cache_type", None)
        if tables is None or ctype is None:
            tables, ctype = derive_private_block_tables(m, kv_cache.shape[2])
        q = F.linear(hidden_states, w_q, b_q)
        k_new = v_new = None
        if m.kv_cache_use_tot.numel() != 0:
            # new token of every K/V request: K/V projection of the step's rows (the rows of
            # hidden requests are projected too and ignored by the write)
            hd = self.num_heads * self.head_dim
            kv = F.linear(hidden_states, self.qkv_proj.weight[hd:],
                          None if self.qkv_proj.bias is None else self.qkv_proj.bias[hd:])
            k_new, v_new = kv[:, :hd], kv[:, hd:]
        if self.use_absorbed(q.dtype):
            mixed_cache_ops.hidden_to_cache(hidden_states, hidden_cache, m.slot_mapping,
                                            m.hidden_cache_use_input, m.hidden_cache_store_tot)
            if k_new is not None:
                slots = torch.where(ctype != 0, torch.full_like(m.hidden_holder_upd, -1),
                                    m.slot_mapping[m.hidden_holder_upd])
                ops.reshape_and_cache_flash(k_new.view(-1, self.num_heads, self.head_dim),
                                            v_new.view(-1, self.num_heads, self.head_dim),
                                            kv_cache[0], kv_cache[1], slots, "auto")
            attn_output = hybrid_decode_attention_absorbed(
                q, kv_cache, hidden_cache, w_k, b_k, w_v, b_v, tables, m.seq_lens_tensor, ctype,
                self.scaling, hidden_rows=m.hidden_cache_use_input)
        else:
            # cache writes of the new tokens + attention in one native call
            attn_output = decode_layer_step(q, hidden_states, k_new, v_new, kv_cache, hidden_cache,
                                            w_k, b_k, w_v, b_v, tables, m.seq_lens_tensor, ctype,
                                            self.scaling)
        output, _ = self.out_proj(attn_output)
        return output
