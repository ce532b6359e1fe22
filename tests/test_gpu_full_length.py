"""Full-length parity cases of every configuration against the fp32 CPU oracle.

Requests of a batch are independent, so the oracle is evaluated for a subset of each
batch (the ``requests`` argument) that always holds the longest and the shortest request
of each cache type; the cache contents are compared over the whole cache, bit for bit.

Tolerance: |x - ref| <= 2e-2 + 2e-2 * |ref| for the attention output (fp16 / bf16).
"""
import numpy as np
import pytest
import torch

from oracle import hybrid_cache_oracle as O
from apt_serve_b200 import attention as A
from apt_serve_b200 import mixed_cache_ops, ops
from apt_serve_b200.workloads import (CONFIG_SHAPES, OPT_66B, draw_decode_batch, draw_prefill_batch,
                                      make_decode_workload)

from helpers import assert_close

pytestmark = pytest.mark.gpu


def extremes(lens, hid, extra=0, seed=0):
    """Longest and shortest request of each cache type, plus ``extra`` seeded picks."""
    pick = set()
    for kind in (True, False):
        rows = sorted((r for r, h in enumerate(hid) if h == kind), key=lambda r: lens[r])
        if rows:
            pick |= {rows[0], rows[-1]}
    rest = [r for r in range(len(lens)) if r not in pick]
    if extra and rest:
        rng = np.random.default_rng(seed)
        pick |= set(int(x) for x in rng.choice(rest, min(extra, len(rest)), replace=False))
    return sorted(pick)


def fused_step(w):
    wk, bk, wv, bv = w.kv_weights()
    out = A.decode_layer_step(w.query, w.hidden_states, w.new_key, w.new_value, w.kv_cache, w.hidden_cache,
                              wk, bk, wv, bv, w.meta.private_block_tables, w.meta.seq_lens_tensor,
                              w.meta.cache_type, w.scale)
    A.raise_on_device_status()
    return out


def oracle_step(cpu, requests):
    return O.decode_layer_step(cpu.hidden_states, cpu.query, cpu.new_key, cpu.new_value, cpu.kv_cache,
                               cpu.hidden_cache, *cpu.kv_weights(), cpu.meta, cpu.scale, requests=requests)


@pytest.mark.parametrize("fraction", [0.0, 0.5, 1.0])
def test_config5_full_length_requests(fraction):
    """Configuration 5: OPT-13B shapes, requests of 1536..2048 tokens, hidden fraction 0 / 50 /
    100 %; eight requests of the configuration's own draw, every one checked."""
    lens, hid = draw_decode_batch(5, hidden_fraction=fraction)
    rows = extremes(lens, hid, extra=8 - len(extremes(lens, hid)), seed=5)
    lens, hid = [lens[r] for r in rows], [hid[r] for r in rows]
    assert min(lens) >= 1536 and len(lens) == 8
    w = make_decode_workload(CONFIG_SHAPES[5], lens, hid, seed=1005, device="cuda")
    cpu = w.cpu()
    out = fused_step(w)
    ref = oracle_step(cpu, None)
    assert torch.equal(w.kv_cache.cpu().view(torch.uint8), cpu.kv_cache.view(torch.uint8))
    assert_close(out, ref, f"config 5 at {fraction:.0%} hidden, lengths {lens}")


@pytest.mark.parametrize("tp_size,tp_rank", [(1, 0), (8, 6)])
def test_config4_uncapped_lengths(tp_size, tp_rank):
    """Configuration 4 (OPT-66B shapes, bf16): the longest and the shortest request of each
    cache type of the configuration's 512-request draw, whole (tp = 1) and as one rank's
    head slice of tp = 8 (dedicated replicated hidden tensor)."""
    lens, hid = draw_decode_batch(4)
    rows = extremes(lens, hid)
    lens, hid = [lens[r] for r in rows], [hid[r] for r in rows]
    assert max(lens) == 2048
    w = make_decode_workload(OPT_66B, lens, hid, seed=1004, device="cuda", tp_rank=tp_rank, tp_size=tp_size)
    if tp_size > 1:
        # a rank's hidden tensor is a replica of the full-width layer's hidden rows
        full = make_decode_workload(OPT_66B, lens, hid, seed=1004, device="cuda")
        w.hidden_cache.view(-1, 9216).copy_(full.hidden_cache.view(-1, 9216))
        del full
    cpu = w.cpu()
    out = fused_step(w)
    ref = oracle_step(cpu, None)
    assert torch.equal(w.kv_cache.cpu().view(torch.uint8), cpu.kv_cache.view(torch.uint8))
    assert torch.equal(w.hidden_cache.cpu().view(torch.uint8), cpu.hidden_cache.view(torch.uint8))
    assert_close(out, ref, f"config 4 tp {tp_size} rank {tp_rank}, lengths {lens}")


def test_config3_whole_step():
    """Configuration 3 as ONE step at full size: the prefill cache writes of 32 packed prompts
    (K/V rows or layer-input rows by designation), the copy-on-write block copies, the new-token
    writes of the 224 decode requests and the hybrid decode attention, in that order, on the
    GPU and in the oracle.  The whole cache is compared bit for bit; the attention output of a
    subset (extremes of each cache type + 8 seeded requests) within tolerance."""
    from apt_serve_b200.attention import FlashAttentionBackend
    lens, hid = draw_decode_batch(3)
    w = make_decode_workload(CONFIG_SHAPES[3], lens, hid, seed=1003, device="cuda",
                             prefill=draw_prefill_batch(), copy_fraction=0.05)
    cpu = w.cpu()
    # ---- GPU ----
    pf, pm = w.prefill, w.prefill.meta
    slots = torch.full_like(pm.slot_mapping, -1)
    slots[pm.kv_cache_use_tot] = pm.slot_mapping[pm.kv_cache_use_tot]
    ops.reshape_and_cache_flash(pf.key, pf.value, w.kv_cache[0], w.kv_cache[1], slots, "auto")
    mixed_cache_ops.hidden_to_cache(pf.hidden_states, w.hidden_cache, pm.slot_mapping,
                                    pm.hidden_cache_use_input, pm.hidden_cache_store_tot)
    FlashAttentionBackend.copy_blocks([w.kv_cache], w.copy_pairs)
    out = fused_step(w)
    # ---- oracle ----
    cf, cm = cpu.prefill, cpu.prefill.meta
    O.reshape_and_cache_flash(cf.key[cm.kv_cache_use_tot], cf.value[cm.kv_cache_use_tot], cpu.kv_cache[0],
                              cpu.kv_cache[1], cm.slot_mapping[cm.kv_cache_use_tot])
    O.hidden_to_cache(cf.hidden_states, cpu.hidden_cache, cm.slot_mapping, cm.hidden_cache_use_input,
                      cm.hidden_cache_store_tot)
    O.copy_blocks([cpu.kv_cache[0]], [cpu.kv_cache[1]], cpu.copy_pairs)
    rows = extremes(lens, hid, extra=8, seed=3)
    ref = oracle_step(cpu, rows)
    assert torch.equal(w.kv_cache.cpu().view(torch.uint8), cpu.kv_cache.view(torch.uint8)), \
        "cache contents after the step differ from the oracle's"
    assert_close(out[rows], ref[rows], f"config 3 whole step, requests {rows}")


def test_config3_fused_prefill_write_gives_the_same_cache():
    """The one-launch prefill write (aps_prefill_cache_write) leaves the same bits as the two
    separate launches on configuration 3's prefill part."""
    lens, hid = draw_decode_batch(3, batch=8)
    base = make_decode_workload(CONFIG_SHAPES[3], lens, hid, seed=1003, device="cuda",
                                prefill=draw_prefill_batch())
    pf, pm = base.prefill, base.prefill.meta
    a, b = base.kv_cache.clone(), base.kv_cache.clone()
    slots = torch.full_like(pm.slot_mapping, -1)
    slots[pm.kv_cache_use_tot] = pm.slot_mapping[pm.kv_cache_use_tot]
    ops.reshape_and_cache_flash(pf.key, pf.value, a[0], a[1], slots, "auto")
    mixed_cache_ops.hidden_to_cache(pf.hidden_states, a, pm.slot_mapping, pm.hidden_cache_use_input,
                                    pm.hidden_cache_store_tot)
    ops.prefill_cache_write(pf.key, pf.value, pf.hidden_states, b, b, pm.slot_mapping, pm.kv_cache_use_tot,
                            pm.hidden_cache_use_input)
    assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    assert not torch.equal(a.view(torch.uint8), base.kv_cache.view(torch.uint8))
