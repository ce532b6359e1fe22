"""Host logic: index tensors and block-id conventions (no GPU)."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from apt_serve_b200.metadata import (BlockPool, blocks_needed, build_decode_metadata,
                                     build_prefill_metadata, derive_private_block_tables)

NB = 100
BS = 16


def test_worked_example_decode():
    # r0 hidden-cached, S=3, private table [7], shared table [NB+2];
    # r1 K/V-cached, S=5, private table [4]  (traced through the reference's model runner)
    m = build_decode_metadata([3, 5], [True, False], [[7], [4]], [[NB + 2], []], BS)
    assert m.slot_mapping.tolist() == [112, 113, 114, 68]
    assert m.slot_mapping_shared.tolist() == [(NB + 2) * 16 + i for i in range(3)]
    assert m.hidden_cache_use_tot.tolist() == [0, 1, 2]
    assert m.kv_cache_use_tot.tolist() == [3]
    assert m.hidden_holder_upd.tolist() == [2, 3]
    assert m.hidden_holder_pull.tolist() == [0, 1]
    assert m.hidden_cache_store_tot.tolist() == [2]
    assert m.hidden_cache_use_input.tolist() == [0]
    assert m.block_tables.tolist() == [[NB + 2], [4]]
    assert m.seq_lens_tensor.tolist() == [3, 5]
    assert m.block_tables.dtype == torch.int32 and m.seq_lens_tensor.dtype == torch.int32
    assert m.num_tot_tokens == 4 and m.num_hidden_cache_tokens == 1 and m.num_decode_tokens == 2
    assert m.cache_type.tolist() == [1, 0] and m.kv_request_rows.tolist() == [1]


def test_hidden_request_uses_v_plane_for_odd_blocks():
    rng = np.random.default_rng(0)
    pool = BlockPool(NB, rng)
    t = pool.table_for(50, BS, use_hidden=True)  # 4 logical blocks -> 2 physical
    assert len(t) == 4
    assert t[1] == t[0] + NB and t[3] == t[2] + NB
    assert 0 <= t[0] < NB and 0 <= t[2] < NB and t[0] != t[2]
    assert pool.num_free == NB - 2
    s = pool.shared_table_for(50, BS)
    assert len(s) == 4 and all(NB <= x < 2 * NB for x in s)
    assert blocks_needed([50, 50], [True, False], BS) == 2 + 4
    assert blocks_needed([50, 50], [True, True], BS) == 8  # shared ids: one per logical block


def test_pool_exhaustion_raises():
    pool = BlockPool(1, np.random.default_rng(0))
    pool.allocate()
    with pytest.raises(ValueError):
        pool.allocate()


def _random_batch(seed, n, max_len):
    rng = np.random.default_rng(seed)
    lens = rng.integers(1, max_len + 1, size=n).tolist()
    hid = (rng.random(n) < 0.5).tolist()
    nb = blocks_needed(lens, hid, BS) + 3
    pool = BlockPool(nb, rng)
    tables = [pool.table_for(s, BS, h) for s, h in zip(lens, hid)]
    shared = [pool.shared_table_for(s, BS) if h else [] for s, h in zip(lens, hid)]
    return lens, hid, nb, tables, shared


@settings(max_examples=40, deadline=None)
@given(st.integers(0, 10_000), st.integers(1, 12), st.integers(1, 100))
def test_decode_invariants(seed, n, max_len):
    lens, hid, nb, tables, shared = _random_batch(seed, n, max_len)
    m = build_decode_metadata(lens, hid, tables, shared, BS)
    n_tot = sum(s if h else 1 for s, h in zip(lens, hid))
    n_h = sum(s for s, h in zip(lens, hid) if h)
    # the commented checks of the reference's model runner
    assert m.slot_mapping.numel() == n_tot == m.num_tot_tokens
    assert m.hidden_cache_use_tot.numel() + m.kv_cache_use_tot.numel() == n_tot
    assert m.hidden_holder_upd.numel() == n == m.num_decode_tokens
    assert m.hidden_holder_upd.numel() + m.hidden_holder_pull.numel() == n_tot
    assert m.slot_mapping_shared.numel() == n_h
    assert m.slot_mapping_shared.numel() == m.hidden_holder_pull.numel() + m.num_hidden_cache_tokens
    assert m.hidden_cache_store_tot.numel() == m.num_hidden_cache_tokens == sum(hid)
    # slots are unique and in range; hidden slots may reach the V plane
    slots = m.slot_mapping.tolist()
    assert len(set(slots)) == len(slots)
    assert all(0 <= s < 2 * nb * BS for s in slots)
    assert all(nb * BS <= s < 2 * nb * BS for s in m.slot_mapping_shared.tolist())
    # the fused call's inputs can be recovered from the reference fields alone
    tables_d, ctype = derive_private_block_tables(m, BS)
    assert ctype.tolist() == [int(h) for h in hid]
    for r, (s, t) in enumerate(zip(lens, tables)):
        nblk = -(-s // BS)
        assert tables_d[r, :nblk].tolist() == t[:nblk]


def test_prefill_metadata():
    m = build_prefill_metadata([5, 20], [True, False], [[3], [8, 2]], BS)
    assert m.slot_mapping.tolist() == [48 + i for i in range(5)] + \
        [128 + i for i in range(16)] + [32 + i for i in range(4)]
    assert m.hidden_cache_use_input.tolist() == list(range(5))
    assert m.hidden_cache_use_tot is m.hidden_cache_use_input
    assert m.kv_cache_use_tot.tolist() == list(range(5, 25))
    assert m.seq_start_loc.tolist() == [0, 5, 25]
    assert m.slot_mapping_shared.numel() == 0 and m.hidden_holder_upd.numel() == 0
    assert m.num_hidden_cache_tokens == 5 and m.num_prefill_tokens == 25
