"""Index tensors of the hybrid-cache path, built the way the reference's model
runner builds them (additional_designs/worker/aptserve_model_runner.py:515-668),
plus the block-id conventions of its block manager
(additional_designs/core/aptserve_block_manager.py:176-199, 530-540, 739-752).

This is host logic: everything here is integer bookkeeping done with numpy and
handed to the kernels as int64 / int32 tensors.  The names and dtypes of the
fields are the reference's (additional_designs/attention/backends/
aptserve_abstract.py:65-80, aptserve_flash_attn.py:68-125); three derived
fields (``private_block_tables``, ``cache_type``, ``kv_request_rows``) feed the
fused decode call and can be recomputed from the reference fields on device
(see :func:`derive_private_block_tables`).
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import List, Optional, Sequence

import numpy as np
import torch

PAD_SLOT_ID = -1  # aptserve_model_runner.py:32


# --------------------------------------------------------------------------- #
# block-id conventions
# --------------------------------------------------------------------------- #
class BlockPool:
    """Hands out block ids with the reference block manager's conventions.

    * private ids live in ``[0, NB)``; a K/V request takes one per logical block;
    * a hidden request takes a fresh id ``p`` for every even logical block and
      ``p + NB`` for the following odd one, i.e. the V plane of the same physical
      block (aptserve_block_manager.py:530-540, 739-752);
    * shared ids live in ``[NB, 2 NB)`` (aptserve_block_manager.py:176-199).
    """

    def __init__(self, num_blocks: int, rng: np.random.Generator):
        self.num_blocks = int(num_blocks)
        self._free = list(rng.permutation(self.num_blocks))
        self._free_shared = list(self.num_blocks + rng.permutation(self.num_blocks))

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise ValueError("Out of memory! No free blocks are available.")
        return int(self._free.pop())

    def allocate_shared(self) -> int:
        if not self._free_shared:
            raise ValueError("Out of memory! No free shared blocks are available.")
        return int(self._free_shared.pop())

    def table_for(self, seq_len: int, block_size: int, use_hidden: bool) -> List[int]:
        n_logical = -(-seq_len // block_size)
        table: List[int] = []
        for i in range(n_logical):
            if not use_hidden or i % 2 == 0:
                table.append(self.allocate())
            else:
                table.append(table[-1] + self.num_blocks)
        return table

    def shared_table_for(self, seq_len: int, block_size: int) -> List[int]:
        return [self.allocate_shared() for _ in range(-(-seq_len // block_size))]


def blocks_needed(seq_lens: Sequence[int], use_hidden: Sequence[bool], block_size: int) -> int:
    """Smallest ``NB`` that holds a batch: one physical block per logical block
    for K/V requests, one per *pair* of logical blocks for hidden requests -- and
    at least as many as the hidden requests' logical blocks, because the shared
    id range ``[NB, 2 NB)`` hands out one id per logical block of a hidden request."""
    n = shared = 0
    for s, h in zip(seq_lens, use_hidden):
        logical = -(-int(s) // block_size)
        n += (logical + 1) // 2 if h else logical
        shared += logical if h else 0
    return max(n, shared)


# --------------------------------------------------------------------------- #
# metadata containers
# --------------------------------------------------------------------------- #
@dataclass
class DecodeMetadata:
    """Decode-batch index tensors (all int64 unless noted).

    Expanded token space: request by request, ``S_r`` entries for a hidden
    request and one entry for a K/V request (aptserve_model_runner.py:527,555).
    """
    slot_mapping: torch.Tensor            # [N_tot]
    slot_mapping_shared: torch.Tensor     # [N_h]
    hidden_cache_use_tot: torch.Tensor    # [N_h]
    kv_cache_use_tot: torch.Tensor        # [n_kv]
    hidden_holder_upd: torch.Tensor       # [B]
    hidden_holder_pull: torch.Tensor      # [N_tot - B]
    hidden_cache_store_tot: torch.Tensor  # [n_h]
    hidden_cache_use_input: torch.Tensor  # [n_h]
    block_tables: torch.Tensor            # [B, max_blocks] int32, pad 0
    seq_lens_tensor: torch.Tensor         # [B] int32
    seq_lens: List[int]
    num_hidden_cache_tokens: int
    num_tot_tokens: int
    num_prefills: int = 0
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0
    max_decode_seq_len: int = 0
    # derived, for the fused decode call
    private_block_tables: Optional[torch.Tensor] = None  # [B, max_blocks] int32
    cache_type: Optional[torch.Tensor] = None            # [B] int32, 1 = hidden
    kv_request_rows: Optional[torch.Tensor] = None       # [n_kv] int64 batch rows

    def to(self, device, non_blocking: bool = False) -> "DecodeMetadata":
        kw = {}
        for f in fields(self):
            v = getattr(self, f.name)
            kw[f.name] = v.to(device, non_blocking=non_blocking) if torch.is_tensor(v) else v
        return DecodeMetadata(**kw)

    def pin_memory(self) -> "DecodeMetadata":
        kw = {}
        for f in fields(self):
            v = getattr(self, f.name)
            kw[f.name] = v.pin_memory() if torch.is_tensor(v) else v
        return DecodeMetadata(**kw)

    def tensor_bytes(self) -> int:
        return sum(getattr(self, f.name).numel() * getattr(self, f.name).element_size()
                   for f in fields(self) if torch.is_tensor(getattr(self, f.name)))


@dataclass
class PrefillMetadata:
    """Prefill-batch index tensors: one entry per prompt token
    (aptserve_model_runner.py:541-566, 651-666)."""
    slot_mapping: torch.Tensor            # [T]
    hidden_cache_use_input: torch.Tensor  # token rows of hidden requests
    hidden_cache_use_tot: torch.Tensor    # same tensor
    hidden_cache_store_tot: torch.Tensor  # same tensor
    kv_cache_use_tot: torch.Tensor        # the other token rows
    slot_mapping_shared: torch.Tensor     # empty
    hidden_holder_upd: torch.Tensor       # empty
    hidden_holder_pull: torch.Tensor      # empty
    seq_start_loc: torch.Tensor           # [n+1] int32
    seq_lens: List[int]
    num_hidden_cache_tokens: int
    num_tot_tokens: int
    num_prefills: int
    num_prefill_tokens: int
    num_decode_tokens: int = 0
    max_prefill_seq_len: int = 0

    def to(self, device, non_blocking: bool = False) -> "PrefillMetadata":
        kw = {}
        for f in fields(self):
            v = getattr(self, f.name)
            kw[f.name] = v.to(device, non_blocking=non_blocking) if torch.is_tensor(v) else v
        return PrefillMetadata(**kw)


def _pad_tables(tables: Sequence[Sequence[int]]) -> np.ndarray:
    width = max(1, max(len(t) for t in tables))
    out = np.zeros((len(tables), width), dtype=np.int32)  # pad = 0, model_runner:601-609
    for r, t in enumerate(tables):
        out[r, :len(t)] = t
    return out


def build_decode_metadata(seq_lens: Sequence[int], use_hidden: Sequence[bool],
                          block_tables: Sequence[Sequence[int]],
                          block_tables_4_shared: Sequence[Sequence[int]],
                          block_size: int) -> DecodeMetadata:
    """Restates the decode branch of ``_prepare_model_input``
    (aptserve_model_runner.py:515-564 for the per-request loop, :613-648 for the
    boolean-mask to index conversion, :601-609 and :707-709 for block tables and
    sequence lengths).  ``seq_lens[r]`` includes the token being decoded."""
    bs = block_size
    slot_chunks, shared_chunks = [], []
    use_tot_mask, upd_mask = [], []
    tables_out = []
    for r, (s, hid) in enumerate(zip(seq_lens, use_hidden)):
        s = int(s)
        priv = np.asarray(block_tables[r], dtype=np.int64)
        if hid:
            pos = np.arange(s, dtype=np.int64)
            shared = np.asarray(block_tables_4_shared[r], dtype=np.int64)
            slot_chunks.append(priv[pos // bs] * bs + pos % bs)
            shared_chunks.append(shared[pos // bs] * bs + pos % bs)
            use_tot_mask.append(np.ones(s, dtype=bool))
            m = np.zeros(s, dtype=bool)
            m[-1] = True
            upd_mask.append(m)
            tables_out.append(list(block_tables_4_shared[r]))  # model_runner:415-418
        else:
            i = s - 1
            slot_chunks.append(np.asarray([priv[i // bs] * bs + i % bs], dtype=np.int64))
            use_tot_mask.append(np.zeros(1, dtype=bool))
            upd_mask.append(np.ones(1, dtype=bool))
            tables_out.append(list(block_tables[r]))
    slot_mapping = np.concatenate(slot_chunks) if slot_chunks else np.zeros(0, np.int64)
    slot_shared = np.concatenate(shared_chunks) if shared_chunks else np.zeros(0, np.int64)
    use_tot = np.concatenate(use_tot_mask) if use_tot_mask else np.zeros(0, bool)
    upd = np.concatenate(upd_mask) if upd_mask else np.zeros(0, bool)
    idx = np.arange(use_tot.size, dtype=np.int64)
    use_hidden_arr = np.asarray(list(use_hidden), dtype=bool)
    rows = np.arange(use_hidden_arr.size, dtype=np.int64)

    t = torch.from_numpy
    meta = DecodeMetadata(
        slot_mapping=t(slot_mapping),
        slot_mapping_shared=t(slot_shared),
        hidden_cache_use_tot=t(idx[use_tot]),
        kv_cache_use_tot=t(idx[~use_tot]),
        hidden_holder_upd=t(idx[upd]),
        hidden_holder_pull=t(idx[~upd]),
        hidden_cache_store_tot=t(idx[use_tot & upd]),
        hidden_cache_use_input=t(rows[use_hidden_arr]),
        block_tables=t(_pad_tables(tables_out)),
        seq_lens_tensor=torch.tensor([int(s) for s in seq_lens], dtype=torch.int32),
        seq_lens=[int(s) for s in seq_lens],
        num_hidden_cache_tokens=int(use_hidden_arr.sum()),
        num_tot_tokens=int(use_tot.size),
        num_decode_tokens=len(seq_lens),
        max_decode_seq_len=max([int(s) for s in seq_lens], default=0),
        private_block_tables=t(_pad_tables(block_tables)),
        cache_type=t(use_hidden_arr.astype(np.int32)),
        kv_request_rows=t(rows[~use_hidden_arr]),
    )
    return meta


def build_prefill_metadata(prompt_lens: Sequence[int], use_hidden: Sequence[bool],
                           block_tables: Sequence[Sequence[int]],
                           block_size: int) -> PrefillMetadata:
    """Restates the prefill branch (aptserve_model_runner.py:541-566, 651-666):
    one slot per prompt token through the private table; hidden-designated token
    rows in ``hidden_cache_use_input`` (= ``use_tot`` = ``store_tot``), the others
    in ``kv_cache_use_tot``."""
    bs = block_size
    slots, mask = [], []
    for r, (s, hid) in enumerate(zip(prompt_lens, use_hidden)):
        s = int(s)
        priv = np.asarray(block_tables[r], dtype=np.int64)
        pos = np.arange(s, dtype=np.int64)
        slots.append(priv[pos // bs] * bs + pos % bs)
        mask.append(np.full(s, bool(hid)))
    slot_mapping = np.concatenate(slots) if slots else np.zeros(0, np.int64)
    m = np.concatenate(mask) if mask else np.zeros(0, bool)
    idx = np.arange(m.size, dtype=np.int64)
    t = torch.from_numpy
    hid_idx = t(idx[m])
    empty = torch.zeros(0, dtype=torch.int64)
    start = np.zeros(len(prompt_lens) + 1, dtype=np.int32)
    start[1:] = np.cumsum(np.asarray(prompt_lens, dtype=np.int64))
    return PrefillMetadata(
        slot_mapping=t(slot_mapping),
        hidden_cache_use_input=hid_idx,
        hidden_cache_use_tot=hid_idx,
        hidden_cache_store_tot=hid_idx,
        kv_cache_use_tot=t(idx[~m]),
        slot_mapping_shared=empty,
        hidden_holder_upd=empty,
        hidden_holder_pull=empty,
        seq_start_loc=t(start),
        seq_lens=[int(s) for s in prompt_lens],
        num_hidden_cache_tokens=int(m.sum()),
        num_tot_tokens=int(m.size),
        num_prefills=len(prompt_lens),
        num_prefill_tokens=int(m.size),
        max_prefill_seq_len=max([int(s) for s in prompt_lens], default=0),
    )


def derive_private_block_tables(meta: DecodeMetadata, block_size: int):
    """Recover, with tensor ops only (no host sync), what the fused decode call
    needs from the *unchanged* reference metadata.

    A hidden request's ``block_tables`` row is its shared table, useless once the
    shared cache is bypassed; its private slots are the request's segment of
    ``slot_mapping`` (ending at ``hidden_holder_upd[r]``), so its private block
    ids are ``slot_mapping[start + BS*j] // BS``.  K/V requests keep their row.
    Returns ``(private_block_tables int32 [B, max_blocks], cache_type int32 [B])``.
    """
    dev = meta.block_tables.device
    b, width = meta.block_tables.shape
    cache_type = torch.zeros(b, dtype=torch.int32, device=dev)
    if meta.hidden_cache_use_input.numel() == 0:
        return meta.block_tables, cache_type
    cache_type[meta.hidden_cache_use_input] = 1
    lens = meta.seq_lens_tensor.long()
    start = meta.hidden_holder_upd - (lens - 1) * cache_type.long()
    j = torch.arange(width, device=dev, dtype=torch.int64)[None, :] * block_size
    valid = (j < lens[:, None]) & (cache_type[:, None] != 0)
    pos = torch.where(valid, start[:, None] + j, torch.zeros_like(j))
    ids = (meta.slot_mapping[pos] // block_size).to(torch.int32)
    tables = torch.where(valid, ids, meta.block_tables)
    tables = torch.where((cache_type[:, None] != 0) & ~valid, torch.zeros_like(tables), tables)
    return tables, cache_type
