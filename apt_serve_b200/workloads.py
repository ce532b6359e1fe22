"""Seeded synthetic workloads for the hybrid-cache path.

The reference measures end to end on dataset traces through a live server;
here one decoder layer is driven with synthetic tensors whose shapes, length
distributions and value distributions are fixed per configuration:

  1  OPT-125m layer, fp32, 8 decode requests, U{32..512}, even rows hidden-cached
  2  OPT-13B layer, fp16, 256 decode requests, lognormal(700, 0.6) in [16, 2048],
     a seeded half hidden-cached
  3  config 2's decode part with 224 requests, plus 32 prefill requests
     U{64..2048} (seeded half hidden-designated) and a 5 % block copy
  4  OPT-66B layer, bf16, 512 decode requests, lognormal(900, 0.5), 40 % hidden,
     heads sharded over 1/2/4/8 ranks
  5  OPT-13B layer, fp16, 64 decode requests U{1536..2048}, hidden fraction swept

A drawn length is the request's sequence length *including* the token being
decoded.  Lengths and cache types come from ``numpy.random.default_rng(seed)``
(seed = 1000 + config id unless given), values from a ``torch.Generator`` on the
device the tensors are created on; whoever needs the same numbers elsewhere
copies the tensors.

Block ids follow the reference block manager (see ``metadata.BlockPool``); the
layer's cache is ``[2, NB, BS, H, D]`` as the reference's cache engine allocates
it (additional_designs/worker/aptserve_cache_engine.py:61-86).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .metadata import (BlockPool, DecodeMetadata, PrefillMetadata, blocks_needed,
                       build_decode_metadata, build_prefill_metadata)


@dataclass(frozen=True)
class LayerShape:
    name: str
    num_heads: int      # total heads (un-sharded)
    head_dim: int
    hidden: int
    dtype: torch.dtype
    block_size: int = 16

    @property
    def es(self) -> int:
        return torch.empty(0, dtype=self.dtype).element_size()


OPT_125M = LayerShape("opt-125m", 12, 64, 768, torch.float32)
OPT_13B = LayerShape("opt-13b", 40, 128, 5120, torch.float16)
OPT_66B = LayerShape("opt-66b", 72, 128, 9216, torch.bfloat16)

CONFIG_SHAPES: Dict[int, LayerShape] = {1: OPT_125M, 2: OPT_13B, 3: OPT_13B, 4: OPT_66B, 5: OPT_13B}


def _lognormal_lengths(rng, n, median, sigma, lo=16, hi=2048):
    x = rng.lognormal(mean=math.log(median), sigma=sigma, size=n)
    return np.clip(np.rint(x), lo, hi).astype(np.int64)


def _seeded_fraction(rng, n, frac):
    k = int(round(n * frac))
    mask = np.zeros(n, dtype=bool)
    mask[rng.permutation(n)[:k]] = True
    return mask


def draw_decode_batch(config: int, seed: Optional[int] = None, batch: Optional[int] = None,
                      hidden_fraction: Optional[float] = None) -> Tuple[List[int], List[bool]]:
    """Sequence lengths and cache types of a configuration's decode batch."""
    rng = np.random.default_rng(1000 + config if seed is None else seed)
    if config == 1:
        n = 8 if batch is None else batch
        lens = rng.integers(32, 513, size=n)
        hid = (np.arange(n) % 2 == 0)
    elif config in (2, 3):
        n = (256 if config == 2 else 224) if batch is None else batch
        lens = _lognormal_lengths(rng, n, 700, 0.6)
        hid = _seeded_fraction(rng, n, 0.5 if hidden_fraction is None else hidden_fraction)
    elif config == 4:
        n = 512 if batch is None else batch
        lens = _lognormal_lengths(rng, n, 900, 0.5)
        hid = _seeded_fraction(rng, n, 0.4 if hidden_fraction is None else hidden_fraction)
    elif config == 5:
        n = 64 if batch is None else batch
        lens = rng.integers(1536, 2049, size=n)
        hid = _seeded_fraction(rng, n, 0.5 if hidden_fraction is None else hidden_fraction)
    else:
        raise ValueError(f"unknown config {config}")
    return [int(x) for x in lens], [bool(x) for x in hid]


def draw_prefill_batch(seed: Optional[int] = None, n: int = 32, lo: int = 64, hi: int = 2048):
    """Config 3's prefill part: ``n`` prompts U{lo..hi}, a seeded half hidden-designated."""
    rng = np.random.default_rng(1003 + 7919 if seed is None else seed)
    lens = rng.integers(lo, hi + 1, size=n)
    hid = _seeded_fraction(rng, n, 0.5)
    return [int(x) for x in lens], [bool(x) for x in hid]


@dataclass
class DecodeWorkload:
    shape: LayerShape
    tp_rank: int
    tp_size: int
    num_blocks: int
    kv_cache: torch.Tensor            # [2, NB, BS, H_rank, D]
    hidden_cache: torch.Tensor        # aliases kv_cache when H_rank*D == E, else [2, NB, BS, 1, E]
    shared_cache: Optional[torch.Tensor]
    qkv_weight: torch.Tensor          # [3*H_rank*D, E]   (q rows, k rows, v rows of this rank)
    qkv_bias: torch.Tensor            # [3*H_rank*D]
    o_weight: torch.Tensor            # [E, H_rank*D]
    o_bias: torch.Tensor              # [E]
    hidden_states: torch.Tensor       # [B, E]  layer input of the token being decoded
    query: torch.Tensor               # [B, H_rank*D]
    new_key: torch.Tensor             # [B, H_rank*D]
    new_value: torch.Tensor           # [B, H_rank*D]
    meta: DecodeMetadata
    seq_lens: List[int]
    use_hidden: List[bool]
    block_tables: List[List[int]]
    block_tables_4_shared: List[List[int]]
    prefill: Optional["PrefillWriteWorkload"] = None   # configuration 3 only
    copy_pairs: Optional[torch.Tensor] = None          # [n, 2] int64 (src, dst) block ids

    @property
    def heads(self) -> int:
        return self.shape.num_heads // self.tp_size

    @property
    def scale(self) -> float:
        return self.shape.head_dim ** -0.5

    def kv_weights(self):
        hd = self.heads * self.shape.head_dim
        w, b = self.qkv_weight, self.qkv_bias
        return w[hd:2 * hd], b[hd:2 * hd], w[2 * hd:], b[2 * hd:]

    @property
    def t_kv(self) -> int:
        return sum(s for s, h in zip(self.seq_lens, self.use_hidden) if not h)

    @property
    def t_hidden(self) -> int:
        return sum(s for s, h in zip(self.seq_lens, self.use_hidden) if h)

    def cpu(self) -> "DecodeWorkload":
        return self.to("cpu")

    def to(self, device) -> "DecodeWorkload":
        kv = self.kv_cache.to(device)
        alias = self.hidden_cache.data_ptr() == self.kv_cache.data_ptr()
        kw = dict(self.__dict__)
        for k, v in kw.items():
            if torch.is_tensor(v):
                kw[k] = v.to(device)
        kw["kv_cache"] = kv
        kw["hidden_cache"] = kv if alias else self.hidden_cache.to(device)
        kw["meta"] = self.meta.to(device)
        if self.prefill is not None:
            pf = self.prefill
            kw["prefill"] = PrefillWriteWorkload(pf.hidden_states.to(device), pf.key.to(device),
                                                 pf.value.to(device), pf.meta.to(device),
                                                 pf.block_tables, pf.prompt_lens, pf.use_hidden)
        return DecodeWorkload(**kw)


def make_decode_workload(shape: LayerShape, seq_lens: Sequence[int], use_hidden: Sequence[bool],
                         seed: int, device="cpu", tp_rank: int = 0, tp_size: int = 1,
                         with_shared_cache: bool = False, spare_blocks: int = 8,
                         kv_from_projection: bool = False,
                         prefill: Optional[Tuple[Sequence[int], Sequence[bool]]] = None,
                         copy_fraction: float = 0.0) -> DecodeWorkload:
    """Allocate and fill one layer's caches, weights and step inputs.

    Every rank of a tensor-parallel group calls this with the same ``seed``: the
    full-width tensors are drawn identically and each rank keeps its head slice,
    so the ranks' K/V planes, W_q/W_k/W_v rows and W_o columns are consistent
    (additional_designs/model_executor/layers/aptserve_linear.py:545-569, 764-765).

    ``prefill=(prompt_lens, use_hidden)`` adds configuration 3's prefill part: packed
    prompt tokens (layer inputs and K/V rows) whose blocks come from the same pool;
    ``copy_fraction`` adds copy-on-write pairs for that share of the blocks in use.
    """
    assert shape.num_heads % tp_size == 0
    bs, d, e = shape.block_size, shape.head_dim, shape.hidden
    h_rank = shape.num_heads // tp_size
    hd_rank = h_rank * d
    rng = np.random.default_rng(seed)
    nb = blocks_needed(seq_lens, use_hidden, bs) + spare_blocks
    if prefill is not None:
        nb += blocks_needed(prefill[0], prefill[1], bs)
    n_copy = 0
    if copy_fraction > 0:
        n_copy = max(1, int(round(copy_fraction * (nb - spare_blocks))))
        nb += n_copy
    pool = BlockPool(nb, rng)
    tables = [pool.table_for(s, bs, h) for s, h in zip(seq_lens, use_hidden)]
    shared_tables = [pool.shared_table_for(s, bs) if h else []
                     for s, h in zip(seq_lens, use_hidden)]
    meta = build_decode_metadata(seq_lens, use_hidden, tables, shared_tables, bs)
    prefill_tables = None
    if prefill is not None:
        prefill_tables = [pool.table_for(s, bs, h) for s, h in zip(prefill[0], prefill[1])]
    copy_pairs = None
    if n_copy:
        # copy-on-write pairs: sources among the blocks in use, destinations fresh blocks
        used = sorted({b % nb for t in tables for b in t})
        src = rng.choice(used, size=n_copy, replace=len(used) < n_copy)
        dst = [pool.allocate() for _ in range(n_copy)]
        copy_pairs = np.stack([np.asarray(src, dtype=np.int64), np.asarray(dst, dtype=np.int64)], axis=1)

    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)

    def randn(*size, std=1.0, dtype=shape.dtype):
        # drawn in fp32 then rounded, in slabs, so the stream does not depend on dtype
        out = torch.empty(*size, dtype=dtype, device=dev)
        flat = out.view(-1)
        step = 1 << 26
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            flat[i:i + n] = (torch.randn(n, generator=gen, device=dev, dtype=torch.float32)
                             * std).to(dtype)
        return out

    hd_full = shape.num_heads * d
    # weights: full-width draw, then this rank's slice (q rows | k rows | v rows)
    w_full = randn(3 * hd_full, e, std=0.02)
    b_full = randn(3 * hd_full, std=0.02)
    rows = torch.cat([torch.arange(hd_rank, device=dev) + j * hd_full + tp_rank * hd_rank
                      for j in range(3)])
    qkv_weight = w_full[rows].contiguous()
    qkv_bias = b_full[rows].contiguous()
    del w_full, b_full
    o_full = randn(e, hd_full, std=0.02)
    o_weight = o_full[:, tp_rank * hd_rank:(tp_rank + 1) * hd_rank].contiguous()
    del o_full
    o_bias = randn(e, std=0.02)

    kv_std = 0.02 * math.sqrt(e)
    alias = hd_rank == e
    # K/V planes: drawn per plane and per slab of blocks at FULL width, then cut to this
    # rank's heads, so that every tensor-parallel size sees the same numbers
    kv_cache = torch.empty(2, nb, bs, h_rank, d, dtype=shape.dtype, device=dev)
    slab = max(1, (1 << 26) // (bs * hd_full))
    for p in range(2):
        for i in range(0, nb, slab):
            n = min(slab, nb - i)
            full = randn(n, bs, shape.num_heads, d, std=kv_std)
            kv_cache[p, i:i + n] = full[:, :, tp_rank * h_rank:(tp_rank + 1) * h_rank]
            del full
    if alias:
        hidden_cache = kv_cache
    else:
        hidden_cache = torch.zeros(2, nb, bs, 1, e, dtype=shape.dtype, device=dev)
    # hidden-request blocks hold layer inputs ~ N(0, 1)
    hid_ids = sorted({b for t, h in zip(tables, use_hidden) if h for b in t if b < nb})
    if hid_ids:
        ids = torch.tensor(hid_ids, device=dev, dtype=torch.long)
        step = max(1, (1 << 26) // (bs * e))
        for i in range(0, ids.numel(), step):
            sel = ids[i:i + step]
            for p in range(2):
                hidden_cache[p].view(nb, bs, e)[sel] = randn(sel.numel(), bs, e)

    hidden_states = randn(len(seq_lens), e)
    q_full = randn(len(seq_lens), hd_full)
    k_full = randn(len(seq_lens), hd_full, std=kv_std)
    v_full = randn(len(seq_lens), hd_full, std=kv_std)
    sl = slice(tp_rank * hd_rank, (tp_rank + 1) * hd_rank)
    query, new_key, new_value = (x[:, sl].contiguous() for x in (q_full, k_full, v_full))

    if kv_from_projection:
        # K/V blocks hold projections of seeded hidden states, like the hidden blocks' data
        hd = hd_rank
        w_k, b_k, w_v, b_v = (qkv_weight[hd:2 * hd], qkv_bias[hd:2 * hd],
                              qkv_weight[2 * hd:], qkv_bias[2 * hd:])
        for r, (s, h) in enumerate(zip(seq_lens, use_hidden)):
            if h:
                continue
            x = randn(s, e)
            k = (x.float() @ w_k.float().t() + b_k.float()).to(shape.dtype).view(s, h_rank, d)
            v = (x.float() @ w_v.float().t() + b_v.float()).to(shape.dtype).view(s, h_rank, d)
            pos = torch.arange(s, device=dev)
            blk = torch.tensor(tables[r], device=dev, dtype=torch.long)[pos // bs]
            kv_cache[0][blk, pos % bs] = k
            kv_cache[1][blk, pos % bs] = v

    shared_cache = None
    if with_shared_cache:
        shared_cache = torch.zeros(2, 2 * nb, bs, h_rank, d, dtype=shape.dtype, device=dev)

    prefill_part = None
    if prefill is not None:
        p_lens, p_hid = [int(x) for x in prefill[0]], [bool(x) for x in prefill[1]]
        t = sum(p_lens)
        pk = randn(t, hd_full, std=kv_std)[:, sl].contiguous().view(t, h_rank, d)
        pv = randn(t, hd_full, std=kv_std)[:, sl].contiguous().view(t, h_rank, d)
        prefill_part = PrefillWriteWorkload(
            hidden_states=randn(t, e), key=pk, value=pv,
            meta=build_prefill_metadata(p_lens, p_hid, prefill_tables, bs).to(dev),
            block_tables=prefill_tables, prompt_lens=p_lens, use_hidden=p_hid)
    copy_t = None if copy_pairs is None else torch.from_numpy(copy_pairs).to(dev)

    return DecodeWorkload(prefill=prefill_part, copy_pairs=copy_t, shape=shape, tp_rank=tp_rank, tp_size=tp_size, num_blocks=nb,
                          kv_cache=kv_cache, hidden_cache=hidden_cache,
                          shared_cache=shared_cache, qkv_weight=qkv_weight, qkv_bias=qkv_bias,
                          o_weight=o_weight, o_bias=o_bias, hidden_states=hidden_states,
                          query=query, new_key=new_key, new_value=new_value,
                          meta=meta.to(dev), seq_lens=[int(s) for s in seq_lens],
                          use_hidden=[bool(h) for h in use_hidden], block_tables=tables,
                          block_tables_4_shared=shared_tables)


def make_config_workload(config: int, device="cpu", seed: Optional[int] = None,
                         batch: Optional[int] = None, hidden_fraction: Optional[float] = None,
                         tp_rank: int = 0, tp_size: int = 1, max_len: Optional[int] = None,
                         **kw) -> DecodeWorkload:
    """The decode workload of configuration ``config`` (optionally with a smaller
    batch or capped lengths, for CPU-sized parity cases)."""
    seed = 1000 + config if seed is None else seed
    lens, hid = draw_decode_batch(config, seed, batch, hidden_fraction)
    if max_len is not None:
        lens = [min(s, max_len) for s in lens]
    return make_decode_workload(CONFIG_SHAPES[config], lens, hid, seed, device,
                                tp_rank=tp_rank, tp_size=tp_size, **kw)


@dataclass
class PrefillWriteWorkload:
    """Config 3's prefill part: packed prompt tokens and where they are cached."""
    hidden_states: torch.Tensor   # [T, E]
    key: torch.Tensor             # [T, H, D]
    value: torch.Tensor           # [T, H, D]
    meta: PrefillMetadata
    block_tables: List[List[int]]
    prompt_lens: List[int]
    use_hidden: List[bool]


def algorithmic_work(shape: LayerShape, seq_lens: Sequence[int], use_hidden: Sequence[bool],
                     tp_size: int = 1) -> Dict[str, float]:
    """Algorithmic bytes / FLOPs of one layer-step on one rank: K and V rows read
    once for K/V requests; hidden rows and W_k|W_v read once plus
    ``2 * T_h * E * 2*H*D`` FLOPs for hidden requests; new-token cache writes
    counted as read + write of their payload."""
    h = shape.num_heads // tp_size
    hd, e, es = h * shape.head_dim, shape.hidden, shape.es
    t_kv = sum(s for s, u in zip(seq_lens, use_hidden) if not u)
    t_h = sum(s for s, u in zip(seq_lens, use_hidden) if u)
    n_kv = sum(1 for u in use_hidden if not u)
    n_h = len(seq_lens) - n_kv
    return {
        "t_kv": t_kv, "t_hidden": t_h,
        "kv_attention_bytes": t_kv * 2 * hd * es + n_kv * 2 * hd * es,
        "hidden_bytes": t_h * e * es + 2 * e * hd * es,
        "reprojection_flops": 2.0 * t_h * e * 2 * hd,
        "cache_write_bytes": 2 * (n_kv * 2 * hd * es + n_h * e * es),
    }
