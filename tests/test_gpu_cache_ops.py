"""Paged cache writes on the GPU against the CPU oracle: bit-exact."""
import numpy as np
import pytest
import torch

from oracle import hybrid_cache_oracle as O
from apt_serve_b200 import mixed_cache_ops, ops
from apt_serve_b200.attention import FlashAttentionBackend
from apt_serve_b200.metadata import build_prefill_metadata, BlockPool, blocks_needed

from helpers import small_workload

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def bits(t: torch.Tensor) -> torch.Tensor:
    return t.detach().cpu().contiguous().view(torch.uint8)


def rand(*shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,head_dim", [(2, 64), (5, 128), (3, 24)])
def test_reshape_and_cache_flash(dtype, heads, head_dim):
    nb, bs, t = 7, 16, 37
    key = rand(t, heads, head_dim, dtype=dtype, seed=1)
    value = rand(t, heads, head_dim, dtype=dtype, seed=2)
    kc = rand(nb, bs, heads, head_dim, dtype=dtype, seed=3)
    vc = rand(nb, bs, heads, head_dim, dtype=dtype, seed=4)
    slots = torch.randperm(nb * bs, generator=torch.Generator().manual_seed(5))[:t]
    slots[::5] = -1  # padded tokens are skipped
    kc_ref, vc_ref = kc.clone(), vc.clone()
    O.reshape_and_cache_flash(key, value, kc_ref, vc_ref, slots)
    kc_d, vc_d = kc.cuda(), vc.cuda()
    ops.reshape_and_cache_flash(key.cuda(), value.cuda(), kc_d, vc_d, slots.cuda(), "auto")
    assert torch.equal(bits(kc_d), bits(kc_ref)) and torch.equal(bits(vc_d), bits(vc_ref))


def test_reshape_and_cache_strided_inputs_and_empty():
    # key / value are column slices of a fused qkv output: row stride 3*H*D
    t, h, d = 20, 4, 128
    qkv = rand(t, 3 * h * d, dtype=torch.float16, seed=7)
    q, k, v = qkv.chunk(3, dim=-1)
    kc = torch.zeros(4, 16, h, d, dtype=torch.float16)
    vc = torch.zeros_like(kc)
    slots = torch.arange(t) + 3
    O.reshape_and_cache_flash(k.reshape(t, h, d), v.reshape(t, h, d), kc, vc, slots)
    qkv_d = qkv.cuda()
    _, k_d, v_d = qkv_d.chunk(3, dim=-1)
    kc_d, vc_d = torch.zeros_like(kc).cuda(), torch.zeros_like(vc).cuda()
    ops.reshape_and_cache_flash(k_d.view(t, h, d), v_d.view(t, h, d), kc_d, vc_d, slots.cuda())
    assert torch.equal(bits(kc_d), bits(kc)) and torch.equal(bits(vc_d), bits(vc))
    ops.reshape_and_cache_flash(k_d.view(t, h, d)[:0], v_d.view(t, h, d)[:0], kc_d, vc_d,
                                slots.cuda()[:0])
    assert torch.equal(bits(kc_d), bits(kc))


@pytest.mark.parametrize("dtype", DTYPES)
def test_hidden_to_cache_and_back(dtype):
    w = small_workload(dtype=dtype, heads=3, head_dim=64, lens=(5, 40, 17, 33, 64),
                       hidden=(True, False, True, True, False))
    m = w.meta
    ref = w.kv_cache.clone()
    O.hidden_to_cache(w.hidden_states, ref, m.slot_mapping, m.hidden_cache_use_input,
                      m.hidden_cache_store_tot)
    dev = w.to("cuda")
    mixed_cache_ops.hidden_to_cache(dev.hidden_states, dev.kv_cache, dev.meta.slot_mapping,
                                    dev.meta.hidden_cache_use_input, dev.meta.hidden_cache_store_tot)
    assert torch.equal(bits(dev.kv_cache), bits(ref))
    # gather every cached hidden row; rows of K/V requests keep their previous content
    holder = rand(m.num_tot_tokens, w.shape.hidden, dtype=dtype, seed=11)
    holder_ref = holder.clone()
    O.cache_to_hidden(holder_ref, ref, m.slot_mapping, m.hidden_cache_use_tot)
    holder_d = holder.cuda()
    mixed_cache_ops.cache_to_hidden(holder_d, dev.kv_cache, dev.meta.slot_mapping,
                                    dev.meta.hidden_cache_use_tot)
    assert torch.equal(bits(holder_d), bits(holder_ref))


def test_hidden_to_cache_prefill_rows_and_negative_slots():
    nb, bs, h, d = 6, 16, 2, 64
    pool = BlockPool(nb, np.random.default_rng(0))
    lens, hid = [20, 9, 33], [True, False, True]
    tables = [pool.table_for(s, bs, u) for s, u in zip(lens, hid)]
    m = build_prefill_metadata(lens, hid, tables, bs)
    x = rand(sum(lens), h * d, dtype=torch.float16, seed=1)
    cache = rand(2, nb, bs, h, d, dtype=torch.float16, seed=2)
    slot_mapping = m.slot_mapping.clone()
    slot_mapping[3] = -1
    ref = cache.clone()
    O.hidden_to_cache(x, ref, slot_mapping, m.hidden_cache_use_input, m.hidden_cache_store_tot)
    cache_d = cache.cuda()
    mixed_cache_ops.hidden_to_cache(x.cuda(), cache_d, slot_mapping.cuda(),
                                    m.hidden_cache_use_input.cuda(), m.hidden_cache_store_tot.cuda())
    assert torch.equal(bits(cache_d), bits(ref))
    assert not torch.equal(bits(ref), bits(cache))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("lens,hidden", [
    ((5, 40, 17, 33), (True, False, True, False)),
    ((70, 3, 90), (True, False, True)),          # n_hidden > 2 * n_kv: the reference's modulo would alias
    ((12, 20), (True, True)),                    # no K/V request at all
])
def test_mixed_kv_to_cache(dtype, lens, hidden):
    w = small_workload(dtype=dtype, heads=2, head_dim=64, lens=lens, hidden=hidden,
                       with_shared_cache=True)
    m = w.meta
    h, d = 2, 64
    key = rand(m.num_tot_tokens, h, d, dtype=dtype, seed=21)
    value = rand(m.num_tot_tokens, h, d, dtype=dtype, seed=22)
    kv_ref, sh_ref = w.kv_cache.clone(), w.shared_cache.clone()
    O.mixed_kv_to_cache(key, value, kv_ref[0], kv_ref[1], sh_ref[0], sh_ref[1], m.slot_mapping,
                        m.slot_mapping_shared, m.kv_cache_use_tot, m.hidden_cache_use_tot)
    dev = w.to("cuda")
    dm = dev.meta
    mixed_cache_ops.mixed_kv_to_cache(key.cuda(), value.cuda(), dev.kv_cache[0], dev.kv_cache[1],
                                      dev.shared_cache[0], dev.shared_cache[1], dm.slot_mapping,
                                      dm.slot_mapping_shared, dm.kv_cache_use_tot,
                                      dm.hidden_cache_use_tot)
    assert torch.equal(bits(dev.kv_cache), bits(kv_ref))
    assert torch.equal(bits(dev.shared_cache), bits(sh_ref))


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_copy_blocks_all_layers(dtype):
    layers, nb, bs, h, d = 3, 12, 16, 2, 64
    caches = [rand(2, nb, bs, h, d, dtype=dtype, seed=30 + i) for i in range(layers)]
    pairs = torch.tensor([[0, 5], [1, 7], [0, 9], [11, 2]])
    ref = [c.clone() for c in caches]
    O.copy_blocks([c[0] for c in ref], [c[1] for c in ref], pairs)
    dev = [c.cuda() for c in caches]
    FlashAttentionBackend.copy_blocks(dev, pairs.cuda())
    for a, b in zip(dev, ref):
        assert torch.equal(bits(a), bits(b))
    FlashAttentionBackend.copy_blocks(dev, pairs.cuda()[:0])  # empty mapping is a no-op
    for a, b in zip(dev, ref):
        assert torch.equal(bits(a), bits(b))


def test_copy_blocks_more_layers_than_one_launch_holds():
    layers, nb = 70, 4
    caches = [rand(2, nb, 16, 1, 32, dtype=torch.float16, seed=100 + i) for i in range(layers)]
    pairs = torch.tensor([[3, 0], [2, 1]])
    ref = [c.clone() for c in caches]
    O.copy_blocks([c[0] for c in ref], [c[1] for c in ref], pairs)
    dev = [c.cuda() for c in caches]
    FlashAttentionBackend.copy_blocks(dev, pairs.cuda())
    for a, b in zip(dev, ref):
        assert torch.equal(bits(a), bits(b))


def test_swap_blocks_roundtrip():
    src = rand(2, 6, 16, 2, 64, dtype=torch.float16, seed=5).cuda()
    host = torch.zeros(2, 6, 16, 2, 64, dtype=torch.float16).pin_memory()
    FlashAttentionBackend.swap_blocks(src, host, torch.tensor([[1, 4], [5, 0]]))
    torch.cuda.synchronize()
    assert torch.equal(host[0, 4], src[0, 1].cpu()) and torch.equal(host[1, 0], src[1, 5].cpu())
    back = torch.zeros_like(src)
    FlashAttentionBackend.swap_blocks(host, back, torch.tensor([[4, 2]]))
    torch.cuda.synchronize()
    assert torch.equal(back[1, 2].cpu(), src[1, 1].cpu())


def test_swap_blocks_merges_runs_and_matches_the_oracle():
    """Swap-out then swap-in of a block list with runs (consecutive source AND destination ids
    become one copy), against the oracle's block moves, both planes."""
    src = rand(2, 12, 16, 2, 64, dtype=torch.float16, seed=6)
    host_ref = torch.zeros(2, 10, 16, 2, 64, dtype=torch.float16)
    pairs = torch.tensor([[0, 3], [1, 4], [2, 5], [7, 0], [9, 9], [10, 1], [11, 2]])
    for plane in range(2):
        O.swap_blocks(src[plane], host_ref[plane], pairs)
    dev = src.cuda()
    host = torch.zeros_like(host_ref).pin_memory()
    issued = [ops.swap_blocks(dev[plane], host[plane], pairs) for plane in range(2)]
    torch.cuda.synchronize()
    assert issued == [4, 4]          # runs 0-2 -> 3-5, 7 -> 0, 9 -> 9, 10-11 -> 1-2
    assert torch.equal(bits(host), bits(host_ref))
    back = torch.zeros_like(dev)
    back_pairs = torch.tensor([[3, 6], [4, 7], [5, 8], [0, 0]])
    n = ops.swap_blocks(host[0], back[0], back_pairs)
    torch.cuda.synchronize()
    assert n == 2
    assert torch.equal(back[0, 6:9].cpu(), src[0, 0:3]) and torch.equal(back[0, 0].cpu(), src[0, 7])
    # device to device, and a pair outside the destination is refused before anything is copied
    other = torch.zeros_like(dev)
    assert ops.swap_blocks(dev[1], other[1], torch.tensor([[2, 2], [3, 3]])) == 1
    torch.cuda.synchronize()
    assert torch.equal(other[1, 2:4].cpu(), src[1, 2:4])
    with pytest.raises(RuntimeError):
        ops.swap_blocks(dev[0], host[0], torch.tensor([[0, 10]]))


def test_full_size_prefill_write_roundtrip():
    """Config-3-sized prefill write (OPT-13B rows): write every token of 8 long
    prompts into hidden or K/V blocks, gather the hidden rows back and compare
    with the source; a checksum over the K/V planes checks the scatter."""
    rng = np.random.default_rng(1003)
    bs, h, d = 16, 40, 128
    lens = rng.integers(512, 2049, size=8).tolist()
    hid = [i % 2 == 0 for i in range(8)]
    nb = blocks_needed(lens, hid, bs) + 4
    pool = BlockPool(nb, rng)
    tables = [pool.table_for(s, bs, u) for s, u in zip(lens, hid)]
    m = build_prefill_metadata(lens, hid, tables, bs).to("cuda")
    t = sum(lens)
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(t, h * d, generator=g, device="cuda", dtype=torch.float16)
    k = torch.randn(t, h, d, generator=g, device="cuda", dtype=torch.float16)
    v = torch.randn(t, h, d, generator=g, device="cuda", dtype=torch.float16)
    cache = torch.zeros(2, nb, bs, h, d, device="cuda", dtype=torch.float16)
    mixed_cache_ops.hidden_to_cache(x, cache, m.slot_mapping, m.hidden_cache_use_input,
                                    m.hidden_cache_store_tot)
    slots = torch.full_like(m.slot_mapping, -1)
    slots[m.kv_cache_use_tot] = m.slot_mapping[m.kv_cache_use_tot]
    ops.reshape_and_cache_flash(k, v, cache[0], cache[1], slots)
    back = torch.zeros_like(x)
    mixed_cache_ops.cache_to_hidden(back, cache, m.slot_mapping, m.hidden_cache_use_tot)
    hid_rows = m.hidden_cache_use_input
    assert torch.equal(back[hid_rows], x[hid_rows])
    assert back[m.kv_cache_use_tot].abs().sum() == 0
    kv_rows = m.kv_cache_use_tot
    sl = m.slot_mapping[kv_rows]
    assert torch.equal(cache[0].view(-1, h, d)[sl], k[kv_rows])
    assert torch.equal(cache[1].view(-1, h, d)[sl], v[kv_rows])
    # nothing else was touched: total mass equals the mass of what was written
    total = cache.double().abs().sum()
    want = x[hid_rows].double().abs().sum() + k[kv_rows].double().abs().sum() + v[kv_rows].double().abs().sum()
    assert torch.allclose(total, want, rtol=1e-9)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_cache_write_one_launch(dtype):
    """The fused prefill write against the oracle's two ops (hidden rows + K/V rows of the
    K/V-designated tokens), bit-exact, including tokens with a padded slot."""
    nb, bs, h, d = 20, 16, 3, 64
    pool = BlockPool(nb, np.random.default_rng(1))
    lens, hid = [20, 9, 33, 50, 1], [True, False, True, False, True]
    tables = [pool.table_for(s, bs, u) for s, u in zip(lens, hid)]
    m = build_prefill_metadata(lens, hid, tables, bs)
    t = sum(lens)
    x = rand(t, h * d, dtype=dtype, seed=1)
    qkv = rand(t, 3 * h * d, dtype=dtype, seed=2)          # K and V are column slices of a fused output
    _, k, v = qkv.chunk(3, dim=-1)
    cache = rand(2, nb, bs, h, d, dtype=dtype, seed=3)
    slot_mapping = m.slot_mapping.clone()
    slot_mapping[[2, 25]] = -1
    ref = cache.clone()
    O.hidden_to_cache(x, ref, slot_mapping, m.hidden_cache_use_input, m.hidden_cache_store_tot)
    O.reshape_and_cache_flash(k.reshape(t, h, d)[m.kv_cache_use_tot], v.reshape(t, h, d)[m.kv_cache_use_tot],
                              ref[0], ref[1], slot_mapping[m.kv_cache_use_tot])
    cache_d, qkv_d = cache.cuda(), qkv.cuda()
    _, k_d, v_d = qkv_d.chunk(3, dim=-1)
    ops.prefill_cache_write(k_d.view(t, h, d), v_d.view(t, h, d), x.cuda(), cache_d, cache_d,
                            slot_mapping.cuda(), m.kv_cache_use_tot.cuda(), m.hidden_cache_use_input.cuda())
    assert torch.equal(bits(cache_d), bits(ref))
    assert not torch.equal(bits(ref), bits(cache))
    # only hidden-designated, only K/V-designated, and empty batches
    for kv_idx, hid_idx in ((m.kv_cache_use_tot[:0], m.hidden_cache_use_input),
                            (m.kv_cache_use_tot, m.hidden_cache_use_input[:0]),
                            (m.kv_cache_use_tot[:0], m.hidden_cache_use_input[:0])):
        c2, r2 = cache.cuda(), cache.clone()
        O.hidden_to_cache(x, r2, slot_mapping, hid_idx, hid_idx)
        O.reshape_and_cache_flash(k.reshape(t, h, d)[kv_idx], v.reshape(t, h, d)[kv_idx], r2[0], r2[1],
                                  slot_mapping[kv_idx])
        ops.prefill_cache_write(k_d.view(t, h, d), v_d.view(t, h, d), x.cuda(), c2, c2,
                                slot_mapping.cuda(), kv_idx.cuda(), hid_idx.cuda())
        assert torch.equal(bits(c2), bits(r2))
