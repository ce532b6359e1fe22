"""Decode-batch index tensors expanded on the device.

The reference's model runner builds ``slot_mapping``, ``slot_mapping_shared`` and the
index lists of a decode batch with a Python loop over every cached position of every
hidden-cached request and copies them to the GPU each step
(additional_designs/worker/aptserve_model_runner.py:515-564, 613-648).  Here the host
only ships the two block tables, the sequence lengths and the cache types;
``aps_expand_decode_metadata`` writes the eight tensors on the device, bit-identical
to ``metadata.build_decode_metadata``.

``python -m apt_serve_b200.device_metadata`` times both constructions on configuration 2.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from . import _native as N
from .metadata import DecodeMetadata, _pad_tables


def expand_decode_metadata(seq_lens: Sequence[int], use_hidden: Sequence[bool],
                           block_tables: Sequence[Sequence[int]],
                           block_tables_4_shared: Sequence[Sequence[int]], block_size: int,
                           device) -> DecodeMetadata:
    """Same arguments and result as ``metadata.build_decode_metadata``, with the tensors
    created on ``device`` by the expansion kernels.  Host work is O(number of blocks):
    padding the two block tables."""
    dev = torch.device(device)
    b = len(seq_lens)
    lens = [int(s) for s in seq_lens]
    if any(s < 1 for s in lens):
        # the kernels count a length below 1 as 1; the host counts must agree with them
        raise ValueError("expand_decode_metadata: every sequence length must be >= 1 "
                         "(it includes the token being decoded)")
    hid = np.asarray(list(use_hidden), dtype=bool)
    n_tot = int(sum(s if h else 1 for s, h in zip(lens, hid)))
    n_hid_tok = int(sum(s for s, h in zip(lens, hid) if h))
    n_h = int(hid.sum())
    n_kv = b - n_h
    priv = _pad_tables(block_tables)
    width = priv.shape[1]
    shared = np.zeros_like(priv)
    for r, t in enumerate(block_tables_4_shared):
        if hid[r]:
            shared[r, :len(t)] = t
    host = {
        "priv": torch.from_numpy(priv), "shared": torch.from_numpy(shared),
        "lens": torch.tensor(lens, dtype=torch.int32), "ctype": torch.from_numpy(hid.astype(np.int32)),
    }
    d = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
    i64 = dict(dtype=torch.int64, device=dev)
    out = {
        "slot_mapping": torch.empty(n_tot, **i64), "slot_mapping_shared": torch.empty(n_hid_tok, **i64),
        "hidden_cache_use_tot": torch.empty(n_hid_tok, **i64), "kv_cache_use_tot": torch.empty(n_kv, **i64),
        "hidden_holder_upd": torch.empty(b, **i64), "hidden_holder_pull": torch.empty(n_tot - b, **i64),
        "hidden_cache_store_tot": torch.empty(n_h, **i64), "hidden_cache_use_input": torch.empty(n_h, **i64),
    }
    scratch = torch.empty(max(1, N.lib().aps_decode_metadata_scratch_bytes(b) // 4), dtype=torch.int32,
                          device=dev)
    with torch.cuda.device(dev):
        N.check(N.lib().aps_expand_decode_metadata(
            N.ptr(d["priv"]), N.ptr(d["shared"]), N.ptr(d["lens"]), N.ptr(d["ctype"]), b, width,
            block_size, N.ptr(out["slot_mapping"]), N.ptr(out["slot_mapping_shared"]),
            N.ptr(out["hidden_cache_use_tot"]), N.ptr(out["kv_cache_use_tot"]),
            N.ptr(out["hidden_holder_upd"]), N.ptr(out["hidden_holder_pull"]),
            N.ptr(out["hidden_cache_store_tot"]), N.ptr(out["hidden_cache_use_input"]), n_tot,
            n_hid_tok, None, N.ptr(scratch), scratch.numel() * 4, N.current_stream(dev)))
    # block_tables of the reference metadata: shared table for hidden requests, private otherwise
    ref_tables = torch.where(d["ctype"][:, None] != 0, d["shared"], d["priv"])
    rows = torch.arange(b, device=dev, dtype=torch.int64)
    return DecodeMetadata(
        block_tables=ref_tables, seq_lens_tensor=d["lens"], seq_lens=lens,
        num_hidden_cache_tokens=n_h, num_tot_tokens=n_tot, num_decode_tokens=b,
        max_decode_seq_len=max(lens, default=0), private_block_tables=d["priv"],
        cache_type=d["ctype"], kv_request_rows=rows[d["ctype"] == 0], **out)


def _time_both(config: int = 2, repeats: int = 5):
    import time
    from .metadata import BlockPool, blocks_needed, build_decode_metadata
    from .workloads import draw_decode_batch
    lens, hid = draw_decode_batch(config)
    rng = np.random.default_rng(0)
    pool = BlockPool(blocks_needed(lens, hid, 16) + 8, rng)
    tables = [pool.table_for(s, 16, h) for s, h in zip(lens, hid)]
    shared = [pool.shared_table_for(s, 16) if h else [] for s, h in zip(lens, hid)]
    dev = torch.device("cuda")
    for _ in range(2):
        expand_decode_metadata(lens, hid, tables, shared, 16, dev)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(repeats):
        m = expand_decode_metadata(lens, hid, tables, shared, 16, dev)
    torch.cuda.synchronize()
    t_dev = (time.perf_counter() - t0) / repeats
    t0 = time.perf_counter()
    for _ in range(repeats):
        h = build_decode_metadata(lens, hid, tables, shared, 16).to(dev)
    torch.cuda.synchronize()
    t_host = (time.perf_counter() - t0) / repeats
    # the reference's own construction: a Python loop appending two slots per cached position
    t0 = time.perf_counter()
    sm, sms = [], []
    for r, (s, u) in enumerate(zip(lens, hid)):
        if u:
            for j in range(s):
                sms.append(shared[r][j // 16] * 16 + j % 16)
                sm.append(tables[r][j // 16] * 16 + j % 16)
        else:
            sm.append(tables[r][(s - 1) // 16] * 16 + (s - 1) % 16)
    torch.tensor(sm, dtype=torch.long, device=dev); torch.tensor(sms, dtype=torch.long, device=dev)
    torch.cuda.synchronize()
    t_loop = time.perf_counter() - t0
    same = all(torch.equal(getattr(m, f), getattr(h, f)) for f in (
        "slot_mapping", "slot_mapping_shared", "hidden_cache_use_tot", "kv_cache_use_tot",
        "hidden_holder_upd", "hidden_holder_pull", "hidden_cache_store_tot", "hidden_cache_use_input"))
    bytes_dev = sum(v.numel() * v.element_size() for v in (m.private_block_tables, m.block_tables,
                                                           m.seq_lens_tensor, m.cache_type))
    print(f"config {config}: {len(lens)} requests, N_tot={m.num_tot_tokens}; identical={same}; "
          f"device expansion {t_dev * 1e3:.3f} ms per step ({bytes_dev} bytes host->device), "
          f"numpy construction + copy {t_host * 1e3:.3f} ms ({h.tensor_bytes()} bytes), "
          f"per-position Python loop (slot lists only) + copy {t_loop * 1e3:.1f} ms")


if __name__ == "__main__":
    _time_both()
