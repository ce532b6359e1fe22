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


def test_counts_that_disagree_with_the_device_side_batch_write_nothing():
    """The caller sizes (and may NULL) the outputs from its own counts.  When the device-side
    cache types / lengths disagree with them the kernels must not store anything: every
    output keeps its sentinel, and the counts word shows what the device saw.  Two cases:
    all-hidden counts with a K/V row on the device (kv_cache_use_tot is NULL), and a
    sequence length of 0, which the device counts as 1."""
    from apt_serve_b200 import _native as N
    dev = torch.device("cuda")
    bs, width = 16, 4
    cases = [
        # (device-side lens, device-side cache types, claimed N_tot, claimed N_h)
        ([20, 7, 33], [1, 0, 1], 60, 60),     # claim: all three hidden
        ([20, 0, 33], [1, 1, 1], 53, 53),     # claim: host counted the empty request as 0 tokens
    ]
    for lens, ctype, n_tot, n_hid in cases:
        b = len(lens)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        tables = torch.arange(b * width, dtype=torch.int32, device=dev).view(b, width)
        sent = -7
        full = lambda n: torch.full((max(n, 1),), sent, dtype=torch.int64, device=dev)
        out = {"slot_mapping": full(n_tot), "slot_mapping_shared": full(n_hid), "use_tot": full(n_hid),
               "upd": full(b), "pull": full(n_tot - b), "store": full(b), "use_input": full(b)}
        counts = torch.zeros(4, dtype=torch.int64, device=dev)
        scratch = torch.empty(N.lib().aps_decode_metadata_scratch_bytes(b) // 4, dtype=torch.int32, device=dev)
        st = N.lib().aps_expand_decode_metadata(
            N.ptr(tables), N.ptr(tables), N.ptr(i32(lens)), N.ptr(i32(ctype)), b, width, bs,
            N.ptr(out["slot_mapping"]), N.ptr(out["slot_mapping_shared"]), N.ptr(out["use_tot"]),
            None,                                   # kv_cache_use_tot: empty for an all-hidden claim
            N.ptr(out["upd"]), N.ptr(out["pull"]), N.ptr(out["store"]), N.ptr(out["use_input"]),
            n_tot, n_hid, N.ptr(counts), N.ptr(scratch), scratch.numel() * 4, N.current_stream(dev))
        assert st == N.APS_OK
        torch.cuda.synchronize()
        for name, t in out.items():
            assert bool((t == sent).all()), f"{name} was written despite the mismatch"
        seen = counts.tolist()
        assert seen[0] != n_tot or seen[1] != n_hid


def test_zero_length_is_refused_on_the_host():
    with pytest.raises(ValueError, match=">= 1"):
        expand_decode_metadata([5, 0], [True, False], [[0], [1]], [[2], []], 16, "cuda")
