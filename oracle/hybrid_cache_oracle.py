"""CPU oracle for Apt-Serve's hybrid-cache data path (TEST INFRASTRUCTURE ONLY).

This file restates, in plain PyTorch on the CPU, what the reference computes on
the hybrid-cache hot path.  It exists to check the CUDA kernels; the product
never imports it.  Only the test-suite, the smoke check and the CPU-baseline /
reference legs of the benchmark may call it.

Parity status: the reference ships no tests, golden vectors or fixtures for this
path, and its arithmetic lives in un-vendored third-party code (vLLM 0.5.0.post1
``_custom_ops``, its ``vllm_flash_attn`` wheel, cuBLAS through ``F.linear``).
The three ``mixed_cache_ops`` kernels are pinned against the reference's own
CUDA source built unmodified (see ``oracle/build_ref.py`` and the GPU test that
compares it with this file); everything else is **parity unpinned**: it follows
the semantics visible at the reference's call sites, cited per function below.

Reference files cited (paths inside the reference project):
  mc.cu   additional_designs/mixed_cache_kernels/mixed_cache.cu
  fa.py   additional_designs/attention/backends/aptserve_flash_attn.py
  opt.py  additional_designs/model_executor/models/aptserve_opt.py
  lin.py  additional_designs/model_executor/layers/aptserve_linear.py
  ce.py   additional_designs/worker/aptserve_cache_engine.py
  mr.py   additional_designs/worker/aptserve_model_runner.py
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


# --------------------------------------------------------------------------- #
# layout helpers
# --------------------------------------------------------------------------- #
def flat_rows(paged_cache: torch.Tensor) -> torch.Tensor:
    """View a paged cache as flat rows of ``stride(2)`` elements.

    mc.cu:24,50,129 address the whole ``[2, NB, BS, H, D]`` tensor as
    ``data[slot * paged_cache.stride(2) + i]``; slots below ``NB*BS`` land in the
    K plane, the rest in the V plane.
    """
    assert paged_cache.dim() == 5
    row = paged_cache.stride(2)
    n_rows = paged_cache.numel() // row
    return torch.as_strided(paged_cache, (n_rows, row), (row, 1),
                            paged_cache.storage_offset())


# --------------------------------------------------------------------------- #
# cache writes (bit-exact data movement)
# --------------------------------------------------------------------------- #
def reshape_and_cache_flash(key: torch.Tensor, value: torch.Tensor,
                            key_cache: torch.Tensor, value_cache: torch.Tensor,
                            slot_mapping: torch.Tensor) -> None:
    """``cache[slot // BS, slot % BS] = x[t]`` for every token with ``slot >= 0``.

    Third-party op (vLLM 0.5.0.post1); semantics from its call sites fa.py:338-355,
    fa.py:378-385 and the pad-slot convention mr.py:32,493 (``_PAD_SLOT_ID = -1``).
    key/value: [T, H, D]; caches: [NB, BS, H, D]; slot_mapping: [T] int64.
    """
    bs = key_cache.shape[1]
    slots = slot_mapping.tolist()
    for t, slot in enumerate(slots):
        if slot < 0:
            continue
        key_cache[slot // bs, slot % bs] = key[t]
        value_cache[slot // bs, slot % bs] = value[t]


def hidden_to_cache(hidden: torch.Tensor, paged_cache: torch.Tensor,
                    slot_mapping: torch.Tensor, src_idx: torch.Tensor,
                    target_slot_idx: torch.Tensor) -> None:
    """mc.cu:31-53 / 119-147: row ``src_idx[i]`` of ``hidden`` goes to the flat
    cache row ``slot_mapping[target_slot_idx[i]]`` (skipped when negative)."""
    rows = flat_rows(paged_cache)
    e = hidden.shape[1]
    for i in range(src_idx.numel()):
        slot = int(slot_mapping[int(target_slot_idx[i])])
        if slot < 0:
            continue
        rows[slot, :e] = hidden[int(src_idx[i])]


def cache_to_hidden(hidden: torch.Tensor, paged_cache: torch.Tensor,
                    slot_mapping: torch.Tensor, dst_idx: torch.Tensor) -> None:
    """mc.cu:6-28 / 150-176: ``hidden[t] = flat_row(slot_mapping[t])`` for every
    ``t`` in ``dst_idx`` (skipped when the slot is negative)."""
    rows = flat_rows(paged_cache)
    e = hidden.shape[1]
    idx = dst_idx.long()
    slots = slot_mapping[idx]
    ok = slots >= 0
    hidden[idx[ok]] = rows[slots[ok], :e]


def mixed_kv_to_cache(key, value, k_cache, v_cache, shared_k_cache, shared_v_cache,
                      slot_mapping, slot_mapping_shared, kv_cache_use_tot,
                      hidden_cache_use_tot, literal_index: bool = False) -> None:
    """mc.cu:56-116 / 179-230, three ranges of the launch grid:

    * ``[0, n_kv)``      token ``kv_cache_use_tot[b]`` -> private cache at ``slot_mapping[tok]``
    * ``[n_kv, 2 n_kv)`` the same token -> shared cache at the same slot
    * ``[2 n_kv, ...)``  token ``hidden_cache_use_tot[j]`` -> shared cache at
      ``slot_mapping_shared[j]``.

    The reference computes ``j = blockIdx.x % (2 n_kv)`` (mc.cu:88), which equals
    the intended ``blockIdx.x - 2 n_kv`` only while ``n_hidden <= 2 n_kv``.
    ``literal_index=True`` reproduces the modulo; the default is the intent.
    """
    bs = k_cache.shape[1]
    n_kv = kv_cache_use_tot.numel()
    n_h = slot_mapping_shared.numel()

    def put(cache_k, cache_v, tok, slot):
        if slot < 0:
            return
        cache_k[slot // bs, slot % bs] = key[tok]
        cache_v[slot // bs, slot % bs] = value[tok]

    for b in range(n_kv):
        tok = int(kv_cache_use_tot[b])
        slot = int(slot_mapping[tok])
        put(k_cache, v_cache, tok, slot)
        put(shared_k_cache, shared_v_cache, tok, slot)
    for jj in range(n_h):
        j = ((2 * n_kv + jj) % (2 * n_kv)) if (literal_index and n_kv > 0) else jj
        put(shared_k_cache, shared_v_cache,
            int(hidden_cache_use_tot[j]), int(slot_mapping_shared[j]))


def copy_blocks(key_caches: Sequence[torch.Tensor], value_caches: Sequence[torch.Tensor],
                src_to_dists: torch.Tensor) -> None:
    """Third-party op; call site fa.py:58-65.  For every layer and every
    ``(src, dst)`` row: ``cache[dst] = cache[src]`` for the K and the V plane."""
    pairs = src_to_dists.tolist()
    for kc, vc in zip(key_caches, value_caches):
        for src, dst in pairs:
            kc[dst] = kc[src].clone()
            vc[dst] = vc[src].clone()


def swap_blocks(src: torch.Tensor, dst: torch.Tensor, src_to_dst: torch.Tensor) -> None:
    """Third-party op; call site fa.py:44-56: ``dst[d] = src[s]`` per ``(s, d)`` row."""
    for s, d in src_to_dst.tolist():
        dst[d] = src[s]


# --------------------------------------------------------------------------- #
# projections (lin.py)
# --------------------------------------------------------------------------- #
def qkv_slices(qkv_weight: torch.Tensor, qkv_bias: Optional[torch.Tensor]):
    """lin.py:115-130: the fused ``[3*HD, E]`` weight cut in thirds (MHA only):
    ``q_only`` uses ``weight[:HD]``, ``kv_only`` uses ``weight[HD:]``;
    opt.py:124 chunks the KV output into K then V."""
    s = qkv_weight.shape[0] // 3
    w_q, w_k, w_v = qkv_weight[:s], qkv_weight[s:2 * s], qkv_weight[2 * s:]
    if qkv_bias is None:
        return (w_q, None), (w_k, None), (w_v, None)
    return (w_q, qkv_bias[:s]), (w_k, qkv_bias[s:2 * s]), (w_v, qkv_bias[2 * s:])


def linear_fp32(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    y = x.float() @ w.float().t()
    if b is not None:
        y = y + b.float()
    return y


# --------------------------------------------------------------------------- #
# hybrid decode attention (intended semantics)
# --------------------------------------------------------------------------- #
def request_slots(block_table_row: torch.Tensor, seq_len: int, block_size: int) -> torch.Tensor:
    pos = torch.arange(seq_len)
    return block_table_row[pos // block_size].long() * block_size + pos % block_size


def hybrid_decode_attention(query: torch.Tensor, kv_cache: torch.Tensor,
                            hidden_cache: torch.Tensor,
                            w_k: torch.Tensor, b_k: Optional[torch.Tensor],
                            w_v: torch.Tensor, b_v: Optional[torch.Tensor],
                            block_tables: torch.Tensor, seq_lens: torch.Tensor,
                            cache_type: torch.Tensor, scale: float,
                            round_kv_to: Optional[torch.dtype] = None,
                            requests: Optional[Sequence[int]] = None) -> torch.Tensor:
    """fp32 decode attention over a ragged batch whose requests are K/V-cached
    (``cache_type == 0``) or hidden-cached (``cache_type == 1``).

    * K/V request: K/V rows are read from ``kv_cache[0]`` / ``kv_cache[1]``
      (fa.py:332-333, layout ce.py:61-80) through the request's private block
      table (the decode call fa.py:452-461).
    * hidden request: hidden rows are read from the flat rows of ``hidden_cache``
      (mc.cu:24) through the request's private table, whose odd logical blocks
      carry V-plane ids ``>= NB``; K = X W_k^T + b_k, V = X W_v^T + b_v
      (opt.py:120-124, lin.py:123-130).
    * ``out[r, h] = softmax(scale * q[r, h] . K[:, h]) @ V[:, h]`` (opt.py:78,
      fa.py:452-473), all in fp32.

    ``round_kv_to`` rounds the re-projected K/V to the model dtype first, which is
    what the reference's cuBLAS output does.  ``requests`` restricts the result to
    a subset of batch rows (rows not listed stay zero).
    """
    b, hd = query.shape
    bs = kv_cache.shape[2]
    d = kv_cache.shape[4]
    n_heads = hd // d
    e = w_k.shape[1]
    out = torch.zeros(b, hd, dtype=torch.float32)
    k_plane = kv_cache[0].reshape(-1, kv_cache.shape[3], d)
    v_plane = kv_cache[1].reshape(-1, kv_cache.shape[3], d)
    h_rows = flat_rows(hidden_cache)
    todo = range(b) if requests is None else requests
    for r in todo:
        s = int(seq_lens[r])
        slots = request_slots(block_tables[r], s, bs)
        if int(cache_type[r]) != 0:
            x = h_rows[slots, :e]
            k = linear_fp32(x, w_k, b_k)
            v = linear_fp32(x, w_v, b_v)
            if round_kv_to is not None:
                k = k.to(round_kv_to).float()
                v = v.to(round_kv_to).float()
            k = k.view(s, n_heads, d)
            v = v.view(s, n_heads, d)
        else:
            k = k_plane[slots].float()
            v = v_plane[slots].float()
        q = query[r].float().view(n_heads, d)
        logits = torch.einsum("hd,thd->ht", q, k) * scale
        p = torch.softmax(logits, dim=-1)
        out[r] = torch.einsum("ht,thd->hd", p, v).reshape(hd)
    return out


def paged_decode_attention(query, key_cache, value_cache, block_tables, seq_lens,
                           scale: float) -> torch.Tensor:
    """Decode attention over K/V blocks only: the third-party
    ``flash_attn_with_kvcache`` as called at fa.py:452-461 (one query token per
    request, ``causal=True`` is a no-op, no alibi for OPT)."""
    b, hd = query.shape
    bs, n_heads, d = key_cache.shape[1:]
    k_plane = key_cache.reshape(-1, n_heads, d)
    v_plane = value_cache.reshape(-1, n_heads, d)
    out = torch.zeros(b, hd, dtype=torch.float32)
    for r in range(b):
        s = int(seq_lens[r])
        slots = request_slots(block_tables[r], s, bs)
        k = k_plane[slots].float()
        v = v_plane[slots].float()
        q = query[r].float().view(n_heads, d)
        p = torch.softmax(torch.einsum("hd,thd->ht", q, k) * scale, dim=-1)
        out[r] = torch.einsum("ht,thd->hd", p, v).reshape(hd)
    return out


# --------------------------------------------------------------------------- #
# reference-literal composition of one hybrid decode layer
# --------------------------------------------------------------------------- #
def literal_decode_layer(hidden_states: torch.Tensor, qkv_weight: torch.Tensor,
                         qkv_bias: Optional[torch.Tensor], kv_cache: torch.Tensor,
                         shared_cache: torch.Tensor, meta, scale: float) -> torch.Tensor:
    """Chain the reference's own op sequence for a decode batch that contains
    hidden-cached requests: opt.py:106-124 then fa.py:356-387 and fa.py:462-473.

    ``meta`` carries the index tensors of mr.py:515-668 (see
    ``apt_serve_b200.metadata.DecodeMetadata``).  Returns the attention output
    ``[B, H*D]`` in fp32.  For hidden requests this equals
    :func:`hybrid_decode_attention`; for K/V requests it reads the *shared* cache
    through private ids, which only ever holds tokens mirrored by
    ``mixed_kv_to_cache`` (a reference quirk, so the two differ there).
    """
    dtype = hidden_states.dtype
    (w_q, b_q), (w_k, b_k), (w_v, b_v) = qkv_slices(qkv_weight, qkv_bias)
    # opt.py:108-109
    hidden_to_cache(hidden_states, kv_cache, meta.slot_mapping,
                    meta.hidden_cache_use_input, meta.hidden_cache_store_tot)
    # opt.py:112-121
    holder = torch.zeros(meta.num_tot_tokens, hidden_states.shape[1], dtype=dtype)
    q = linear_fp32(hidden_states, w_q, b_q).to(dtype)
    holder[meta.hidden_holder_upd] = hidden_states
    cache_to_hidden(holder, kv_cache, meta.slot_mapping, meta.hidden_cache_use_tot)
    # opt.py:123-124
    w_kv = qkv_weight[qkv_weight.shape[0] // 3:]
    b_kv = None if qkv_bias is None else qkv_bias[qkv_bias.shape[0] // 3:]
    kv = linear_fp32(holder, w_kv, b_kv).to(dtype)
    k, v = kv.chunk(2, dim=-1)
    n_heads, d = kv_cache.shape[3], kv_cache.shape[4]
    k = k.reshape(-1, n_heads, d)
    v = v.reshape(-1, n_heads, d)
    # fa.py:356-385
    if meta.num_tot_tokens != meta.slot_mapping_shared.numel():
        mixed_kv_to_cache(k, v, kv_cache[0], kv_cache[1], shared_cache[0], shared_cache[1],
                          meta.slot_mapping, meta.slot_mapping_shared,
                          meta.kv_cache_use_tot, meta.hidden_cache_use_tot)
    else:
        reshape_and_cache_flash(k, v, shared_cache[0], shared_cache[1],
                                meta.slot_mapping_shared)
    # fa.py:464-473
    return paged_decode_attention(q, shared_cache[0], shared_cache[1],
                                  meta.block_tables, meta.seq_lens_tensor, scale)


# --------------------------------------------------------------------------- #
# tensor parallelism (lin.py:545-569, 764-765, 815-839)
# --------------------------------------------------------------------------- #
def shard_heads(t: torch.Tensor, rank: int, tp: int, dim: int = 0) -> torch.Tensor:
    n = t.shape[dim] // tp
    return t.narrow(dim, rank * n, n)


def out_proj_tp(attn_out_per_rank: List[torch.Tensor], w_o: torch.Tensor,
                b_o: Optional[torch.Tensor]) -> torch.Tensor:
    """Row-parallel o_proj: ``y = sum_r A_r W_o[:, cols_r]^T + b_o``; the bias is
    added once, after the all-reduce (lin.py:827-834)."""
    tp = len(attn_out_per_rank)
    y = None
    for r, a in enumerate(attn_out_per_rank):
        part = a.float() @ shard_heads(w_o, r, tp, dim=1).float().t()
        y = part if y is None else y + part
    if b_o is not None:
        y = y + b_o.float()
    return y


def decode_layer_step(hidden_states, q, new_k, new_v, kv_cache, hidden_cache,
                      w_k, b_k, w_v, b_v, meta, scale,
                      round_kv_to: Optional[torch.dtype] = None,
                      requests: Optional[Sequence[int]] = None) -> torch.Tensor:
    """One layer-step of the measured path: the new token's cache write for every
    request (K/V rows for K/V requests, fa.py:334-345; the layer-input row for
    hidden requests, opt.py:108-109) followed by hybrid decode attention."""
    kv_rows = meta.kv_request_rows
    if kv_rows.numel():
        n_heads, d = kv_cache.shape[3], kv_cache.shape[4]
        reshape_and_cache_flash(new_k[kv_rows].view(-1, n_heads, d),
                                new_v[kv_rows].view(-1, n_heads, d), kv_cache[0], kv_cache[1],
                                meta.slot_mapping[meta.kv_cache_use_tot])
    if meta.hidden_cache_use_input.numel():
        hidden_to_cache(hidden_states, hidden_cache, meta.slot_mapping,
                        meta.hidden_cache_use_input, meta.hidden_cache_store_tot)
    return hybrid_decode_attention(q, kv_cache, hidden_cache, w_k, b_k, w_v, b_v,
                                   meta.private_block_tables, meta.seq_lens_tensor,
                                   meta.cache_type, scale, round_kv_to, requests)


def profit_coefficient_literal(token_counts, seconds, block_size: int) -> float:
    """The scheduler's profit coefficient as the reference computes it from its timing
    sweep (aptserve_llm_engine.py:336-346): prepend the origin, floor-divide the token
    counts by the block size with a minimum of one block for non-empty samples, fit
    scikit-learn's ``LinearRegression`` and return slope / 5."""
    import numpy as np
    from sklearn.linear_model import LinearRegression

    x = np.array([0] + list(token_counts))
    x = x // block_size
    x[1:][x[1:] == 0] = 1
    y = np.array([0] + list(seconds))
    model = LinearRegression()
    model.fit(x.reshape(-1, 1), y)
    return float(model.coef_[0] / 5)
