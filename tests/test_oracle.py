"""The CPU oracle on hand-checkable cases, and its internal consistency."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import hybrid_cache_oracle as O
from apt_serve_b200.metadata import build_decode_metadata
from apt_serve_b200.workloads import make_config_workload, make_decode_workload

from helpers import assert_close, small_workload, tiny_shape


def test_reshape_and_cache_single_block():
    kc = torch.zeros(3, 16, 2, 4)
    vc = torch.zeros(3, 16, 2, 4)
    k = torch.arange(3 * 8, dtype=torch.float32).view(3, 2, 4)
    v = -k
    O.reshape_and_cache_flash(k, v, kc, vc, torch.tensor([17, -1, 47]))
    assert torch.equal(kc[1, 1], k[0]) and torch.equal(vc[1, 1], v[0])
    assert torch.equal(kc[2, 15], k[2])
    assert kc.abs().sum() == k[0].abs().sum() + k[2].abs().sum()  # padded token skipped


def test_hidden_rows_land_in_k_then_v_plane():
    nb, bs, h, d = 4, 16, 2, 4
    cache = torch.zeros(2, nb, bs, h, d)
    hidden = torch.arange(2 * h * d, dtype=torch.float32).view(2, h * d) + 1
    # slot 5 -> K plane block 0 row 5; slot nb*bs + 3 -> V plane block 0 row 3
    slot_mapping = torch.tensor([5, nb * bs + 3])
    O.hidden_to_cache(hidden, cache, slot_mapping, torch.tensor([0, 1]), torch.tensor([0, 1]))
    assert torch.equal(cache[0, 0, 5].reshape(-1), hidden[0])
    assert torch.equal(cache[1, 0, 3].reshape(-1), hidden[1])
    back = torch.zeros(2, h * d)
    O.cache_to_hidden(back, cache, slot_mapping, torch.tensor([0, 1]))
    assert torch.equal(back, hidden)
    # negative slot is skipped in both directions
    O.hidden_to_cache(hidden, cache, torch.tensor([-1]), torch.tensor([1]), torch.tensor([0]))
    assert cache[0].abs().sum() == hidden[0].abs().sum()


def test_mixed_kv_to_cache_ranges_and_literal_index():
    nb, bs, h, d = 4, 16, 1, 2
    n_tot = 5  # tokens 0..2 hidden request (3 positions), 3 and 4 K/V requests
    key = torch.arange(n_tot * h * d, dtype=torch.float32).view(n_tot, h, d) + 1
    val = key * 10
    caches = [torch.zeros(nb, bs, h, d) for _ in range(2)] + [torch.zeros(2 * nb, bs, h, d) for _ in range(2)]
    slot_mapping = torch.tensor([0, 1, 2, 20, 37])
    shared = torch.tensor([(nb + 1) * bs + i for i in range(3)])
    O.mixed_kv_to_cache(key, val, *caches, slot_mapping, shared, torch.tensor([3, 4]),
                        torch.tensor([0, 1, 2]))
    kc, vc, sk, sv = caches
    assert torch.equal(kc[1, 4], key[3]) and torch.equal(sk[1, 4], key[3])   # mirrored
    assert torch.equal(vc[2, 5], val[4]) and torch.equal(sv[2, 5], val[4])
    for i in range(3):
        assert torch.equal(sk[nb + 1, i], key[i]) and torch.equal(sv[nb + 1, i], val[i])
    assert kc.count_nonzero() == 2 * h * d  # hidden tokens never reach the private cache
    # the reference's modulo index aliases once n_hidden > 2 * n_kv
    caches2 = [torch.zeros_like(c) for c in caches]
    O.mixed_kv_to_cache(key, val, *caches2, slot_mapping, shared, torch.tensor([3]),
                        torch.tensor([0, 1, 2]), literal_index=True)
    assert not torch.equal(caches2[2][nb + 1, 2], key[2])


def test_copy_and_swap_blocks():
    kc = [torch.randn(4, 16, 2, 4) for _ in range(2)]
    vc = [torch.randn(4, 16, 2, 4) for _ in range(2)]
    ref = [c.clone() for c in kc + vc]
    O.copy_blocks(kc, vc, torch.tensor([[0, 3], [1, 2]]))
    for c, r in zip(kc + vc, ref):
        assert torch.equal(c[3], r[0]) and torch.equal(c[2], r[1]) and torch.equal(c[0], r[0])
    dst = torch.zeros(4, 16, 2, 4)
    O.swap_blocks(kc[0], dst, torch.tensor([[3, 1]]))
    assert torch.equal(dst[1], kc[0][3])


def test_single_token_attention_returns_value_row():
    shape = tiny_shape(heads=2, head_dim=32)
    w = make_decode_workload(shape, [1, 1], [True, False], seed=1)
    wk, bk, wv, bv = w.kv_weights()
    out = O.hybrid_decode_attention(w.query, w.kv_cache, w.hidden_cache, wk, bk, wv, bv,
                                    w.meta.private_block_tables, w.meta.seq_lens_tensor,
                                    w.meta.cache_type, w.scale)
    x = O.flat_rows(w.hidden_cache)[w.block_tables[0][0] * 16, :shape.hidden]
    assert_close(out[0], x @ wv.t() + bv, "hidden request, one token", 1e-5, 1e-5)
    assert_close(out[1], w.kv_cache[1, w.block_tables[1][0], 0].reshape(-1), "kv request", 1e-6, 1e-6)


def test_literal_reference_sequence_matches_fused_for_hidden_requests():
    """opt.py:106-124 + fa.py:356-387,462-473 chained through the shared cache give,
    for hidden-cached requests, what the fused definition gives; K/V requests differ
    because the reference reads the shared cache through private ids."""
    w = small_workload(dtype=torch.float32, heads=2, head_dim=32, lens=(5, 40, 17, 33),
                       hidden=(True, False, True, False), with_shared_cache=True)
    lit = O.literal_decode_layer(w.hidden_states, w.qkv_weight, w.qkv_bias, w.kv_cache.clone(),
                                 w.shared_cache, w.meta, w.scale)
    kvc = w.kv_cache.clone()
    wk, bk, wv, bv = w.kv_weights()
    (w_q, b_q), _, _ = O.qkv_slices(w.qkv_weight, w.qkv_bias)
    q = O.linear_fp32(w.hidden_states, w_q, b_q)
    O.hidden_to_cache(w.hidden_states, kvc, w.meta.slot_mapping, w.meta.hidden_cache_use_input,
                      w.meta.hidden_cache_store_tot)
    fused = O.hybrid_decode_attention(q, kvc, kvc, wk, bk, wv, bv, w.meta.private_block_tables,
                                      w.meta.seq_lens_tensor, w.meta.cache_type, w.scale)
    assert_close(lit[0], fused[0], "hidden request 0", 1e-4, 1e-4)
    assert_close(lit[2], fused[2], "hidden request 2", 1e-4, 1e-4)
    assert not torch.allclose(lit[1], fused[1], atol=1e-3)


def test_tensor_parallel_heads_sum_to_unsharded():
    shape = tiny_shape(heads=4, head_dim=32)
    lens, hid = [20, 35, 7], [True, False, True]
    full = make_decode_workload(shape, lens, hid, seed=9)
    wk, bk, wv, bv = full.kv_weights()
    ref = O.hybrid_decode_attention(full.query, full.kv_cache, full.hidden_cache, wk, bk, wv, bv,
                                    full.meta.private_block_tables, full.meta.seq_lens_tensor,
                                    full.meta.cache_type, full.scale)
    y_ref = ref @ full.o_weight.float().t() + full.o_bias.float()
    parts = []
    for r in range(2):
        w = make_decode_workload(shape, lens, hid, seed=9, tp_rank=r, tp_size=2)
        # hidden rows are replicated: copy them from the unsharded layout
        O.flat_rows(w.hidden_cache)[:, :shape.hidden] = O.flat_rows(full.hidden_cache)
        a, b, c, d = w.kv_weights()
        parts.append(O.hybrid_decode_attention(w.query, w.kv_cache, w.hidden_cache, a, b, c, d,
                                               w.meta.private_block_tables, w.meta.seq_lens_tensor,
                                               w.meta.cache_type, w.scale))
    assert_close(torch.cat(parts, dim=1), ref, "head shards", 1e-5, 1e-5)
    y = O.out_proj_tp(parts, full.o_weight, full.o_bias)
    assert_close(y, y_ref, "row-parallel o_proj", 1e-4, 1e-4)


def test_config1_runs_end_to_end_on_cpu():
    w = make_config_workload(1, kv_from_projection=True)
    assert w.shape.num_heads == 12 and w.shape.head_dim == 64 and w.shape.dtype == torch.float32
    assert len(w.seq_lens) == 8 and all(32 <= s <= 512 for s in w.seq_lens)
    assert w.use_hidden == [True, False] * 4
    wk, bk, wv, bv = w.kv_weights()
    out = O.decode_layer_step(w.hidden_states, w.query, w.new_key, w.new_value, w.kv_cache,
                              w.hidden_cache, wk, bk, wv, bv, w.meta, w.scale)
    assert out.shape == (8, 768) and torch.isfinite(out).all()


def test_projection_absorption_gives_the_same_attention():
    """The algebra behind the next step noted in the design: for a hidden-cached request
    softmax(q.(W_k x_t + b_k)) . (W_v x_t + b_v) over t equals W_v (sum_t p_t x_t) + b_v with
    p = softmax((W_k^T q) . x_t): the bias term of the scores is constant over t."""
    import torch
    from helpers import small_workload
    w = small_workload(dtype=torch.float32, heads=3, head_dim=32, lens=(37, 5, 130), hidden=(True, True, True))
    wk, bk, wv, bv = w.kv_weights()
    ref = O.hybrid_decode_attention(w.query, w.kv_cache, w.hidden_cache, wk, bk, wv, bv,
                                    w.meta.private_block_tables, w.meta.seq_lens_tensor,
                                    w.meta.cache_type, w.scale)
    rows = O.flat_rows(w.hidden_cache)
    h, d = w.heads, w.shape.head_dim
    bs = w.shape.block_size
    out = torch.empty_like(ref)
    for r, s in enumerate(w.seq_lens):
        pos = torch.arange(s)
        blk = w.meta.private_block_tables[r, pos // bs].long()
        x = rows[blk * bs + pos % bs].float()                                   # [s, E]
        q = w.query[r].view(h, d).float()
        q_abs = torch.einsum("hd,hde->he", q, wk.float().view(h, d, -1)) * w.scale   # W_k^T q per head
        p = torch.softmax(x @ q_abs.t(), dim=0)                                  # [s, h]
        z = p.t() @ x                                                           # [h, E]
        out[r] = (torch.einsum("he,hde->hd", z, wv.float().view(h, d, -1)) + bv.float().view(h, d)).reshape(-1)
    assert torch.allclose(out, ref, atol=2e-5, rtol=2e-5)
