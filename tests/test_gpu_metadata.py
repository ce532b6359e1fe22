"""Device-side expansion of the decode index tensors: bit-identical to the host
construction (which restates the reference's model runner)."""
import numpy as np
import pytest
import torch

from apt_serve_b200.device_metadata import expand_decode_metadata
from apt_serve_b200.metadata import BlockPool, blocks_needed, build_decode_metadata
from apt_serve_b200.workloads import draw_decode_batch

pytestmark = pytest.mark.gpu

FIELDS = ("slot_mapping", "slot_mapping_shared", "hidden_cache_use_tot", "kv_cache_use_tot",
          "hidden_holder_upd", "hidden_holder_pull", "hidden_cache_store_tot",
          "hidden_cache_use_input", "block_tables", "seq_lens_tensor", "private_block_tables",
          "cache_type", "kv_request_rows")


def batch(lens, hid, seed=0, bs=16):
    rng = np.random.default_rng(seed)
    pool = BlockPool(blocks_needed(lens, hid, bs) + 5, rng)
    tables = [pool.table_for(s, bs, h) for s, h in zip(lens, hid)]
    shared = [pool.shared_table_for(s, bs) if h else [] for s, h in zip(lens, hid)]
    return tables, shared


def check(lens, hid, bs=16, seed=0):
    tables, shared = batch(lens, hid, seed, bs)
    host = build_decode_metadata(lens, hid, tables, shared, bs)
    dev = expand_decode_metadata(lens, hid, tables, shared, bs, "cuda")
    torch.cuda.synchronize()
    for f in FIELDS:
        a, b = getattr(dev, f).cpu(), getattr(host, f)
        assert a.dtype == b.dtype and torch.equal(a, b), f
    assert dev.num_tot_tokens == host.num_tot_tokens
    assert dev.num_hidden_cache_tokens == host.num_hidden_cache_tokens


def test_worked_example():
    check([3, 5], [True, False])


@pytest.mark.parametrize("lens,hid", [
    ([1, 1, 1], [True, False, True]),
    ([16, 17, 2048, 5], [True, True, True, True]),      # no K/V request
    ([40, 700, 33], [False, False, False]),             # no hidden request
    ([129, 1, 64, 300, 16, 15], [False, True, False, True, True, False]),
])
def test_edge_batches(lens, hid):
    check(lens, hid)


def test_block_size_32_and_many_requests():
    rng = np.random.default_rng(5)
    lens = rng.integers(1, 400, size=1500).tolist()    # more requests than scan threads
    hid = (rng.random(1500) < 0.4).tolist()
    check(lens, hid, bs=32, seed=5)


def test_config2_and_config4_batches():
    for cfg in (2, 4):
        lens, hid = draw_decode_batch(cfg)
        check(lens, hid, seed=cfg)
