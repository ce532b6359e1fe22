"""Hybrid decode attention with absorbed projections against the fp32 oracle and against the
re-projecting kernel.  Tolerance as for the other attention tests: |x - ref| <= 2e-2 + 2e-2 |ref|."""
import numpy as np
import pytest
import torch

from oracle import hybrid_cache_oracle as O
from apt_serve_b200 import attention as A
from apt_serve_b200.workloads import make_config_workload

from helpers import assert_close, small_workload

pytestmark = pytest.mark.gpu


def oracle_out(w):
    wk, bk, wv, bv = w.kv_weights()
    return O.hybrid_decode_attention(w.query, w.kv_cache, w.hidden_cache, wk, bk, wv, bv,
                                     w.meta.private_block_tables, w.meta.seq_lens_tensor,
                                     w.meta.cache_type, w.scale)


def absorbed(dev, **kw):
    wk, bk, wv, bv = dev.kv_weights()
    return A.hybrid_decode_attention_absorbed(dev.query, dev.kv_cache, dev.hidden_cache, wk, bk, wv, bv,
                                              dev.meta.private_block_tables, dev.meta.seq_lens_tensor,
                                              dev.meta.cache_type, dev.scale, **kw)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_absorbed_small(dtype):
    w = small_workload(dtype=dtype, heads=4, head_dim=128,
                       lens=(5, 40, 17, 129, 300, 16, 128, 1, 64, 65),
                       hidden=(True, False, True, False, True, False, True, True, True, True))
    ref = oracle_out(w)
    out = absorbed(w.to("cuda"))
    assert_close(out, ref, f"absorbed small {dtype}")


@pytest.mark.parametrize("hidden_all", [True, False])
def test_absorbed_pure_batches(hidden_all):
    w = small_workload(heads=4, head_dim=128, lens=[33, 200, 77, 512], hidden=[hidden_all] * 4)
    ref = oracle_out(w)
    out = absorbed(w.to("cuda"))
    assert_close(out, ref, f"absorbed pure {hidden_all}")


def test_absorbed_garbage_beyond_seq_len_does_not_leak():
    w = small_workload(heads=4, head_dim=128, lens=(21, 150), hidden=(True, True))
    rows = O.flat_rows(w.hidden_cache)
    for r, s in enumerate((21, 150)):
        last = w.block_tables[r][(s - 1) // 16]
        rows[last * 16 + s % 16: last * 16 + 16] = float("nan")
    ref = oracle_out(w)
    out = absorbed(w.to("cuda"))
    assert_close(out, ref, "absorbed garbage tail")


def test_absorbed_opt13b_shapes_and_agreement_with_the_reprojecting_kernel():
    w = make_config_workload(2, device="cuda", batch=16, max_len=700)
    ref = oracle_out(w.cpu())
    out = absorbed(w, hidden_rows=w.meta.hidden_cache_use_input)
    assert_close(out, ref, "absorbed OPT-13B shapes")
    wk, bk, wv, bv = w.kv_weights()
    other = A.hybrid_decode_attention(w.query, w.kv_cache, w.hidden_cache, wk, bk, wv, bv,
                                      w.meta.private_block_tables, w.meta.seq_lens_tensor,
                                      w.meta.cache_type, w.scale)
    assert_close(out, other.float(), "absorbed vs re-projecting kernel")
    again = absorbed(w, hidden_rows=w.meta.hidden_cache_use_input)
    assert torch.equal(out, again)


@pytest.mark.parametrize("seed", range(6))
def test_absorbed_ragged_sweep(seed):
    rng = np.random.default_rng(7300 + seed)
    batch = int(rng.integers(1, 20))
    edges = (1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 257)
    lens = [int(rng.choice(edges)) if rng.random() < 0.7 else int(rng.integers(1, 600)) for _ in range(batch)]
    hidden = [bool(v) for v in rng.random(batch) < 0.6]
    dtype = (torch.float16, torch.bfloat16)[seed % 2]
    w = small_workload(dtype=dtype, heads=4, head_dim=128, lens=lens, hidden=hidden, seed=seed)
    ref = oracle_out(w)
    out = absorbed(w.to("cuda"))
    assert_close(out, ref, f"absorbed sweep {seed}: lens={lens} hidden={hidden}")


def test_opt_attention_with_absorbed_projections_matches_the_fused_layer():
    from apt_serve_b200.layers import OPTAttention
    w = small_workload(heads=4, head_dim=128, lens=(33, 70, 150, 9, 260), hidden=(True, False, True, False, True),
                       device="cuda", with_shared_cache=True)
    meta = A.FlashAttentionMetadata.from_decode(w.meta)
    args = (w.shape.hidden, 4, w.qkv_weight, w.qkv_bias, w.o_weight, w.o_bias)
    kv1, kv2 = w.kv_cache.clone(), w.kv_cache.clone()
    y1 = OPTAttention(*args, fused=True)(w.hidden_states, kv1, None, meta)
    y2 = OPTAttention(*args, fused="absorbed")(w.hidden_states, kv2, None, meta)
    assert torch.equal(kv1, kv2)                          # the same cache writes
    assert_close(y2, y1.float(), "OPTAttention absorbed vs fused", 3e-2, 3e-2)


def test_absorbed_opt66b_bf16_tensor_parallel_slice():
    """Config-4 shapes at tp = 8: 9 heads per rank (padded to 16), E = 9216, dedicated hidden
    tensor; the rank's output equals its slice of the full-width oracle result."""
    from apt_serve_b200.workloads import OPT_66B, draw_decode_batch, make_decode_workload
    lens, hid = draw_decode_batch(4, batch=6)
    lens = [min(s, 400) for s in lens]
    hid[0], hid[1] = True, False
    full = make_decode_workload(OPT_66B, lens, hid, seed=1004, device="cuda")
    ref_full = oracle_out(full.cpu())
    rank = 5
    w = make_decode_workload(OPT_66B, lens, hid, seed=1004, device="cuda", tp_rank=rank, tp_size=8)
    w.hidden_cache.view(-1, 9216).copy_(full.hidden_cache.view(-1, 9216))   # replicated hidden rows
    out = absorbed(w)
    sl = slice(rank * 9 * 128, (rank + 1) * 9 * 128)
    assert_close(out, ref_full[:, sl], "absorbed, tp rank 5")
