"""The reference's decode op chain on the GPU, run with the kernels the reference
itself runs (TEST INFRASTRUCTURE ONLY -- the checker of the GPU parity tests and the
``--impl reference`` arm of ``bench.py``; nothing in the product imports this).

For a decode batch with hidden-cached requests the reference executes, per layer
(additional_designs/model_executor/models/aptserve_opt.py:106-124 and
additional_designs/attention/backends/aptserve_flash_attn.py:356-387, 462-473):

    mixed_cache_ops.hidden_to_cache      new token's layer input -> hidden block
    torch.zeros hidden_holder, holder[hidden_holder_upd] = hidden_states
    mixed_cache_ops.cache_to_hidden      every cached hidden row -> holder
    F.linear(holder, W_kv, b_kv)         kv_only projection (cuBLAS)
    mixed_cache_ops.mixed_kv_to_cache    (mixed batch)  or
    ops.reshape_and_cache_flash          (all-hidden batch) -> shared cache
    flash_attn_with_kvcache              paged attention over the shared cache

Each step here is that very kernel:

* ``mixed_cache_ops`` is the reference's own ``mixed_cache.cu`` compiled unmodified by
  ``oracle/build_ref.py`` into ``oracle/_ref/``;
* the projection is ``torch.nn.functional.linear`` as in the reference
  (aptserve_linear.py:123-130);
* ``reshape_and_cache_flash`` is vLLM's ``_custom_ops`` op (the installed vLLM is newer
  than the 0.5.0.post1 the reference patches: the op takes two extra scale tensors, the
  layout and semantics are the same);
* the paged attention is vLLM's flash-attention build (``vllm.vllm_flash_attn``, the
  descendant of the ``vllm_flash_attn`` wheel the reference imports), which takes the
  reference's block size of 16; the stand-alone ``flash_attn`` package only accepts
  paged blocks of 256 tokens and serves as the fallback for caches laid out that way.

``mixed_kv_to_cache`` of the reference indexes its hidden tokens with
``blockIdx.x % (2 * n_kv)`` (mixed_cache.cu:88), which equals the intended index only
while the number of cached hidden TOKENS is at most twice the number of K/V-cached
REQUESTS; outside that envelope hidden tokens alias (the accesses stay in bounds:
the index is below 2 * n_kv <= N_h).  Parity cases with a mixed batch stay inside the
envelope; all-hidden batches take the ``reshape_and_cache_flash`` branch and have no
such limit.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.nn.functional as F


def _load_mixed_cache_ops():
    from . import build_ref
    if not build_ref.module_path().exists():
        raise ImportError("oracle/_ref/mixed_cache_ops is not built (python -m oracle.build_ref)")
    return build_ref.load()


def _resolve_paged_attention() -> Tuple[Callable, str, int]:
    """(function(q [B,H,D], k_cache, v_cache, block_tables, seq_lens, scale) -> [B,H,D],
    its name, the block-size granularity it accepts)."""
    try:
        from vllm.vllm_flash_attn import flash_attn_varlen_func

        def run(q, kc, vc, bt, lens, scale):
            b = q.shape[0]
            cu_q = torch.arange(b + 1, dtype=torch.int32, device=q.device)
            return flash_attn_varlen_func(q, kc, vc, max_seqlen_q=1, cu_seqlens_q=cu_q,
                                          max_seqlen_k=int(bt.shape[1] * kc.shape[1]), seqused_k=lens,
                                          softmax_scale=scale, causal=True, block_table=bt)
        return run, "vllm.vllm_flash_attn.flash_attn_varlen_func (paged, one query token per request)", 16
    except Exception:
        pass
    from flash_attn import flash_attn_with_kvcache

    def run256(q, kc, vc, bt, lens, scale):
        return flash_attn_with_kvcache(q.unsqueeze(1), kc, vc, block_table=bt, cache_seqlens=lens,
                                       softmax_scale=scale, causal=True).squeeze(1)
    return run256, "flash_attn.flash_attn_with_kvcache (paged blocks of 256 tokens)", 256


def _resolve_reshape_and_cache():
    from vllm import _custom_ops as vops

    def run(key, value, key_cache, value_cache, slot_mapping):
        one = torch.ones(1, dtype=torch.float32, device=key.device)
        vops.reshape_and_cache_flash(key, value, key_cache, value_cache, slot_mapping, "auto", one, one)
    return run


class LiteralChain:
    """Holds the resolved kernels; ``LiteralChain.create()`` returns ``(chain, None)`` or
    ``(None, reason)`` when a piece is missing on this machine."""

    def __init__(self, mixed_cache_ops, paged_attention, attention_name, block_granularity,
                 reshape_and_cache):
        self.mixed_cache_ops = mixed_cache_ops
        self.paged_attention = paged_attention
        self.attention_name = attention_name
        self.block_granularity = block_granularity
        self.reshape_and_cache = reshape_and_cache

    @classmethod
    def create(cls):
        try:
            mco = _load_mixed_cache_ops()
        except Exception as exc:
            return None, f"reference extension unavailable: {exc}"
        try:
            attn, name, gran = _resolve_paged_attention()
        except Exception as exc:
            return None, f"no third-party paged flash attention importable: {exc}"
        try:
            rac = _resolve_reshape_and_cache()
        except Exception as exc:
            return None, f"vllm._custom_ops.reshape_and_cache_flash unavailable: {exc}"
        return cls(mco, attn, name, gran, rac), None

    # -- aptserve_flash_attn.py:452-461 / 464-473 ---------------------------------- #
    def decode_attention(self, query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                         block_tables: torch.Tensor, seq_lens: torch.Tensor, scale: float) -> torch.Tensor:
        """``query [B, H*D]`` -> ``[B, H*D]`` over caches ``[NB, BS, H, D]``."""
        h, d = key_cache.shape[2], key_cache.shape[3]
        out = self.paged_attention(query.view(-1, h, d), key_cache, value_cache, block_tables, seq_lens, scale)
        return out.reshape(query.shape[0], h * d)

    # -- aptserve_opt.py:106-124 + aptserve_flash_attn.py:356-387, 462-473 ----------- #
    def hybrid_decode_layer(self, hidden_states: torch.Tensor, query: torch.Tensor, w_kv: torch.Tensor,
                            b_kv: Optional[torch.Tensor], kv_cache: torch.Tensor,
                            shared_cache: torch.Tensor, meta, scale: float,
                            holder: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The chain for a decode batch that holds hidden-cached requests.  ``w_kv`` /
        ``b_kv`` are the K and V thirds of the fused QKV weight (``weight[HD:]``,
        aptserve_linear.py:123-125); ``meta`` carries the reference's index tensors.
        ``holder``: optional pre-allocated ``[N_tot, E]`` buffer (zero-filled here, as the
        reference's ``torch.zeros`` does).  Returns the attention output ``[B, H*D]``."""
        mco = self.mixed_cache_ops
        n_heads, d = kv_cache.shape[3], kv_cache.shape[4]
        mco.hidden_to_cache(hidden_states, kv_cache, meta.slot_mapping, meta.hidden_cache_use_input,
                            meta.hidden_cache_store_tot)
        if holder is None:
            holder = torch.zeros(meta.num_tot_tokens, hidden_states.shape[1], device=hidden_states.device,
                                 dtype=hidden_states.dtype)
        else:
            holder.zero_()
        holder[meta.hidden_holder_upd] = hidden_states
        mco.cache_to_hidden(holder, kv_cache, meta.slot_mapping, meta.hidden_cache_use_tot)
        kv = F.linear(holder, w_kv, b_kv)
        k, v = kv.chunk(chunks=2, dim=-1)
        k = k.view(-1, n_heads, d)
        v = v.view(-1, n_heads, d)
        if meta.num_tot_tokens != meta.slot_mapping_shared.numel():
            mco.mixed_kv_to_cache(k, v, kv_cache[0], kv_cache[1], shared_cache[0], shared_cache[1],
                                  meta.slot_mapping, meta.slot_mapping_shared, meta.kv_cache_use_tot,
                                  meta.hidden_cache_use_tot)
        else:
            self.reshape_and_cache(k, v, shared_cache[0], shared_cache[1], meta.slot_mapping_shared)
        return self.decode_attention(query, shared_cache[0], shared_cache[1], meta.block_tables,
                                     meta.seq_lens_tensor, scale)

    def inside_mixed_envelope(self, meta) -> bool:
        """Whether ``mixed_kv_to_cache``'s hidden-token index equals the intended one for
        this batch (all-hidden batches do not call it)."""
        n_hid_tok = int(meta.slot_mapping_shared.numel())
        n_kv = int(meta.kv_cache_use_tot.numel())
        return n_kv == 0 or n_hid_tok <= 2 * n_kv
