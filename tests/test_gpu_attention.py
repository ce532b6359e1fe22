"""Decode attention on the GPU against the fp32 CPU oracle.

Tolerance (stated once): |x - ref| <= 2e-2 + 2e-2 * |ref| for fp16 / bf16 runs,
1e-4 for fp32 runs."""
import numpy as np
import pytest
import torch

from oracle import hybrid_cache_oracle as O
from apt_serve_b200 import attention as A
from apt_serve_b200.layers import OPTAttention
from apt_serve_b200.workloads import (LayerShape, OPT_13B, draw_decode_batch, make_config_workload,
                                      make_decode_workload)

from helpers import assert_close, small_workload

pytestmark = pytest.mark.gpu


def oracle_out(w, requests=None, round_kv_to=None):
    wk, bk, wv, bv = w.kv_weights()
    return O.hybrid_decode_attention(w.query, w.kv_cache, w.hidden_cache, wk, bk, wv, bv,
                                     w.meta.private_block_tables, w.meta.seq_lens_tensor,
                                     w.meta.cache_type, w.scale, round_kv_to, requests)


def gpu_hybrid(dev):
    wk, bk, wv, bv = dev.kv_weights()
    out = A.hybrid_decode_attention(dev.query, dev.kv_cache, dev.hidden_cache, wk, bk, wv, bv,
                                    dev.meta.private_block_tables, dev.meta.seq_lens_tensor,
                                    dev.meta.cache_type, dev.scale)
    ws = A.attention_workspace(out.device, 1, 1, 16, 1, 1)
    assert A.attention_status(ws) == 0, "a bounded device-side wait ran out"
    return out


# --------------------------------------------------------------------------- #
# K/V path
# --------------------------------------------------------------------------- #
@pytest.mark.parametrize("dtype,heads,head_dim", [
    (torch.float16, 4, 128), (torch.bfloat16, 3, 128), (torch.float32, 12, 64),
    (torch.float16, 5, 64), (torch.float32, 2, 128), (torch.bfloat16, 2, 256),
    (torch.float16, 2, 32), (torch.float32, 3, 32),
])
def test_paged_decode_attention(dtype, heads, head_dim):
    lens = [1, 15, 16, 17, 127, 128, 129, 300, 1000, 2048]
    shape = LayerShape("t", heads, head_dim, heads * head_dim, dtype)
    w = make_decode_workload(shape, lens, [False] * len(lens), seed=5)
    ref = O.paged_decode_attention(w.query, w.kv_cache[0], w.kv_cache[1], w.meta.block_tables,
                                   w.meta.seq_lens_tensor, w.scale)
    dev = w.to("cuda")
    out = A.paged_decode_attention(dev.query, dev.kv_cache[0], dev.kv_cache[1],
                                   dev.meta.block_tables, dev.meta.seq_lens_tensor, dev.scale)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert_close(out, ref, f"paged decode {dtype} H{heads} D{head_dim}", tol, tol)


@pytest.mark.parametrize("bs", [32, 64, 256])
def test_paged_decode_attention_larger_blocks_and_garbage_tail(bs):
    # larger cache blocks; slots past seq_len inside the last block hold NaN and must not leak
    shape = LayerShape("t", 2, 128, 256, torch.float16, block_size=bs)
    lens = [5, 33, 70, 300, 257]
    w = make_decode_workload(shape, lens, [False] * len(lens), seed=8)
    for r, s in enumerate(lens):
        blk = w.block_tables[r][-1]
        w.kv_cache[:, blk, s % bs or bs:] = float("nan")
    ref = O.paged_decode_attention(w.query, w.kv_cache[0], w.kv_cache[1], w.meta.block_tables,
                                   w.meta.seq_lens_tensor, w.scale)
    dev = w.to("cuda")
    out = A.paged_decode_attention(dev.query, dev.kv_cache[0], dev.kv_cache[1],
                                   dev.meta.block_tables, dev.meta.seq_lens_tensor, dev.scale)
    assert_close(out, ref, f"block size {bs}")


def test_paged_decode_attention_padded_block_stride():
    """Cache blocks that are not laid out back to back (a view with 128 bytes of padding after
    every block): the tensor-copy kernel does not apply and the CUDA-core kernel takes over."""
    shape = LayerShape("t", 3, 128, 384, torch.float16)
    lens = [1, 17, 130, 700]
    w = make_decode_workload(shape, lens, [False] * len(lens), seed=12)
    ref = O.paged_decode_attention(w.query, w.kv_cache[0], w.kv_cache[1], w.meta.block_tables,
                                   w.meta.seq_lens_tensor, w.scale)
    dev = w.to("cuda")
    nb, bs, h, d = dev.kv_cache.shape[1:]
    padded = torch.zeros(2, nb, bs * h * d + 64, dtype=torch.float16, device="cuda")
    padded[:, :, :bs * h * d] = dev.kv_cache.view(2, nb, -1)
    kc, vc = (padded[p, :, :bs * h * d].view(nb, bs, h, d) for p in (0, 1))
    assert kc.stride(0) == bs * h * d + 64
    out = A.paged_decode_attention(dev.query, kc, vc, dev.meta.block_tables, dev.meta.seq_lens_tensor, dev.scale)
    assert_close(out, ref, "padded block stride")


def test_unsupported_head_size_raises():
    q = torch.zeros(1, 2 * 96, dtype=torch.float16, device="cuda")
    kc = torch.zeros(2, 16, 2, 96, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        A.paged_decode_attention(q, kc, kc, torch.zeros(1, 1, dtype=torch.int32, device="cuda"),
                                 torch.ones(1, dtype=torch.int32, device="cuda"), 0.1)


# --------------------------------------------------------------------------- #
# re-projection on its own
# --------------------------------------------------------------------------- #
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n_rows,heads,hidden", [(128, 1, 128), (300, 2, 256), (1000, 3, 832)])
def test_kv_reprojection_dense(dtype, n_rows, heads, hidden):
    g = torch.Generator().manual_seed(n_rows)
    x = torch.randn(n_rows, hidden, generator=g).to(dtype)
    hd = heads * 128
    wk = (torch.randn(hd, hidden, generator=g) * 0.05).to(dtype)
    wv = (torch.randn(hd, hidden, generator=g) * 0.05).to(dtype)
    bk = torch.randn(hd, generator=g).to(dtype)
    bv = torch.randn(hd, generator=g).to(dtype)
    ref = torch.cat([O.linear_fp32(x, wk, bk), O.linear_fp32(x, wv, bv)], dim=1)
    out = A.kv_reprojection(x.cuda(), wk.cuda(), bk.cuda(), wv.cuda(), bv.cuda(), 128)
    torch.cuda.synchronize()
    assert_close(out, ref, f"kv_reprojection {dtype} {n_rows}x{hidden}")


def test_kv_reprojection_paged_blocks_no_bias():
    g = torch.Generator().manual_seed(0)
    cache = torch.randn(2, 10, 16, 2, 128, generator=g).to(torch.float16)  # rows of 256
    ids = torch.tensor([13, 2, 7, 19, 0], dtype=torch.int32)            # incl. V-plane ids
    wk = (torch.randn(256, 256, generator=g) * 0.05).to(torch.float16)
    wv = (torch.randn(256, 256, generator=g) * 0.05).to(torch.float16)
    rows = (ids.long()[:, None] * 16 + torch.arange(16)[None]).reshape(-1)
    x = O.flat_rows(cache)[rows]
    n = 70  # last block partly used
    ref = torch.cat([O.linear_fp32(x, wk, None), O.linear_fp32(x, wv, None)], dim=1)[:n]
    out = A.kv_reprojection(cache.cuda(), wk.cuda(), None, wv.cuda(), None, 128,
                            block_ids=ids.cuda(), n_rows=n)
    assert_close(out, ref, "paged kv_reprojection")


# --------------------------------------------------------------------------- #
# hybrid decode attention
# --------------------------------------------------------------------------- #
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_hybrid_small(dtype):
    w = small_workload(dtype=dtype, heads=2, head_dim=128,
                       lens=(5, 40, 17, 129, 300, 16, 128, 1), hidden=(True, False, True, False,
                                                                        True, False, True, True))
    ref = oracle_out(w)
    out = gpu_hybrid(w.to("cuda"))
    assert_close(out, ref, f"hybrid small {dtype}")


@pytest.mark.parametrize("bs,heads,head_dim", [(32, 2, 128), (64, 2, 128), (32, 4, 64)])
def test_hybrid_larger_cache_blocks(bs, heads, head_dim):
    """Cache blocks of 32 / 64 tokens: a hidden request's 16-row sub-blocks then sit at offsets
    inside a block, K/V groups likewise."""
    shape = LayerShape("t", heads, head_dim, 256, torch.float16, block_size=bs)
    lens, hid = [5, 40, 17, 129, 300, 64, 65], [True, False, True, False, True, True, False]
    w = make_decode_workload(shape, lens, hid, seed=4)
    ref = oracle_out(w)
    out = gpu_hybrid(w.to("cuda"))
    assert_close(out, ref, f"hybrid, block size {bs}, {heads} x {head_dim}")


@pytest.mark.parametrize("hidden_fraction", [0.0, 1.0])
def test_hybrid_pure_batches(hidden_fraction):
    lens = [33, 200, 77, 512]
    w = small_workload(heads=3, head_dim=128, lens=lens, hidden=[hidden_fraction > 0] * 4)
    ref = oracle_out(w)
    out = gpu_hybrid(w.to("cuda"))
    assert_close(out, ref, f"hybrid pure {hidden_fraction}")


def test_hybrid_garbage_beyond_seq_len_does_not_leak():
    w = small_workload(heads=2, head_dim=128, lens=(21, 150), hidden=(True, True))
    rows = O.flat_rows(w.hidden_cache)
    for r, s in enumerate((21, 150)):
        last = w.block_tables[r][(s - 1) // 16]
        rows[last * 16 + s % 16: last * 16 + 16] = float("nan")
    ref = oracle_out(w)
    out = gpu_hybrid(w.to("cuda"))
    assert_close(out, ref, "garbage tail")


def test_hybrid_opt13b_shapes_reduced_batch():
    # OPT-13B layer shapes (40 x 128, E = 5120), 12 requests of the config-2 distribution
    w = make_config_workload(2, device="cuda", batch=12, max_len=600)
    cpu = w.cpu()
    ref = oracle_out(cpu)
    out = gpu_hybrid(w)
    assert_close(out, ref, "OPT-13B shapes")


def test_hybrid_full_config2_subset_oracle_and_permutation_invariance():
    """Full config 2 (256 requests): a seeded subset of requests is checked against
    the oracle; the whole batch is checked by size-independent properties:
    reversing the request order permutes the output rows, and a repeated call
    returns the same bits."""
    w = make_config_workload(2, device="cuda")
    out = gpu_hybrid(w)
    assert torch.isfinite(out.float()).all()
    rng = np.random.default_rng(0)
    hid = [r for r, h in enumerate(w.use_hidden) if h]
    kv = [r for r, h in enumerate(w.use_hidden) if not h]
    # always the longest and the shortest request of each cache type, plus a seeded draw
    by_len = lambda rows: sorted(rows, key=lambda r: w.seq_lens[r])
    pick = {by_len(hid)[0], by_len(hid)[-1], by_len(kv)[0], by_len(kv)[-1]}
    pick |= set(rng.choice(hid, 2, replace=False).tolist()) | set(rng.choice(kv, 2, replace=False).tolist())
    pick = sorted(pick)
    assert max(w.seq_lens[r] for r in pick if w.use_hidden[r]) >= 1500
    cpu = w.cpu()
    ref = oracle_out(cpu, requests=pick)
    assert_close(out[pick], ref[pick], "config 2 subset")
    perm = torch.arange(len(w.seq_lens) - 1, -1, -1, device="cuda")
    wk, bk, wv, bv = w.kv_weights()
    out2 = A.hybrid_decode_attention(w.query[perm].contiguous(), w.kv_cache, w.hidden_cache, wk, bk,
                                     wv, bv, w.meta.private_block_tables[perm].contiguous(),
                                     w.meta.seq_lens_tensor[perm].contiguous(),
                                     w.meta.cache_type[perm].contiguous(), w.scale)
    # M tiles are packed across requests, so the order changes which rows share a partial:
    # the permuted result agrees to rounding, and a given order is reproducible bit for bit
    assert_close(out2, out[perm].float(), "request permutation", 2e-3, 2e-3)
    assert torch.equal(gpu_hybrid(w), out)


def test_hybrid_opt66b_bf16_tensor_parallel_slices():
    # config-4 shapes at tp = 8: 9 heads per rank, E = 9216, dedicated hidden tensor
    lens, hid = draw_decode_batch(4, batch=6)
    lens = [min(s, 400) for s in lens]
    hid[0], hid[1] = True, False
    from apt_serve_b200.workloads import OPT_66B
    full = make_decode_workload(OPT_66B, lens, hid, seed=1004, device="cuda")
    ref_full = oracle_out(full.cpu())
    for rank in (0, 5):
        w = make_decode_workload(OPT_66B, lens, hid, seed=1004, device="cuda", tp_rank=rank, tp_size=8)
        assert w.hidden_cache.shape[-1] == 9216 and w.kv_cache.shape[3] == 9
        O_rows = w.hidden_cache.view(-1, 9216)
        O_rows.copy_(full.hidden_cache.view(-1, 9216))  # replicated hidden rows
        out = gpu_hybrid(w)
        sl = slice(rank * 9 * 128, (rank + 1) * 9 * 128)
        assert_close(out, ref_full[:, sl], f"tp rank {rank}")


# --------------------------------------------------------------------------- #
# CUDA-core re-projection (fp32, other head sizes)
# --------------------------------------------------------------------------- #
def test_config1_full_on_gpu_fp32():
    """Configuration 1 (OPT-125m layer, fp32, 12 heads x 64, 8 requests): the whole
    layer-step on the GPU against the CPU oracle; fp32 tolerance 1e-3."""
    from apt_serve_b200 import mixed_cache_ops, ops
    w = make_config_workload(1, device="cuda", kv_from_projection=True)
    cpu = w.cpu()
    ref = O.decode_layer_step(cpu.hidden_states, cpu.query, cpu.new_key, cpu.new_value, cpu.kv_cache,
                              cpu.hidden_cache, *cpu.kv_weights(), cpu.meta, cpu.scale)
    m, h, d = w.meta, w.heads, w.shape.head_dim
    rows = m.kv_request_rows
    ops.reshape_and_cache_flash(w.new_key[rows].view(-1, h, d), w.new_value[rows].view(-1, h, d),
                                w.kv_cache[0], w.kv_cache[1], m.slot_mapping[m.kv_cache_use_tot])
    mixed_cache_ops.hidden_to_cache(w.hidden_states, w.hidden_cache, m.slot_mapping,
                                    m.hidden_cache_use_input, m.hidden_cache_store_tot)
    out = gpu_hybrid(w)
    assert torch.equal(w.kv_cache.cpu().view(torch.uint8), cpu.kv_cache.view(torch.uint8))
    assert_close(out, ref, "config 1 on the GPU", 1e-3, 1e-3)


@pytest.mark.parametrize("dtype,heads,head_dim", [(torch.float16, 3, 64), (torch.bfloat16, 2, 32),
                                                  (torch.float32, 2, 128)])
def test_hybrid_cuda_core_reprojection_shapes(dtype, heads, head_dim):
    w = small_workload(dtype=dtype, heads=heads, head_dim=head_dim, lens=(5, 40, 17, 129, 200, 16),
                       hidden=(True, False, True, False, True, True))
    ref = oracle_out(w)
    out = gpu_hybrid(w.to("cuda"))
    tol = 1e-3 if dtype == torch.float32 else 2e-2
    assert_close(out, ref, f"CUDA-core re-projection {dtype} D{head_dim}", tol, tol)


@pytest.mark.parametrize("dtype,heads,head_dim", [(torch.float16, 2, 64), (torch.bfloat16, 6, 64),
                                                  (torch.float16, 4, 32), (torch.bfloat16, 12, 32)])
def test_hybrid_tensor_core_reprojection_small_heads(dtype, heads, head_dim):
    """Head sizes 64 and 32 with heads x head size a multiple of 128: two / four adjacent heads
    share one accumulator tile of the tensor-core kernel, each with its own softmax."""
    w = small_workload(dtype=dtype, heads=heads, head_dim=head_dim,
                       lens=(5, 40, 17, 129, 300, 16, 128, 1, 260),
                       hidden=(True, False, True, False, True, False, True, True, True))
    ref = oracle_out(w)
    out = gpu_hybrid(w.to("cuda"))
    assert_close(out, ref, f"tensor-core re-projection {dtype} {heads} x {head_dim}")


@pytest.mark.parametrize("name,heads,hidden,dtype", [("opt-125m", 12, 768, torch.float16),
                                                     ("opt-350m", 16, 1024, torch.bfloat16),
                                                     ("opt-1.3b", 32, 2048, torch.float16)])
def test_hybrid_small_opt_models_head_size_64(name, heads, hidden, dtype):
    """The OPT sizes with 64-element heads, in the 16-bit types the serving path runs."""
    rng = np.random.default_rng(heads)
    lens = [int(x) for x in rng.integers(1, 700, size=14)] + [2048, 16]
    hid = [bool(b) for b in rng.random(len(lens)) < 0.5]
    hid[-2] = True
    w = make_decode_workload(LayerShape(name, heads, 64, hidden, dtype), lens, hid, seed=heads)
    ref = oracle_out(w)
    out = gpu_hybrid(w.to("cuda"))
    assert_close(out, ref, f"{name} {dtype}")


def test_cuda_core_and_tensor_core_reprojection_agree_head_size_64():
    w = small_workload(heads=4, head_dim=64, lens=(70, 300, 129, 2), hidden=(True, True, False, True)).to("cuda")
    tensor = gpu_hybrid(w).clone()
    wk, bk, wv, bv = (t.float() for t in w.kv_weights())
    simt = A.hybrid_decode_attention(w.query.float(), w.kv_cache.float(), w.hidden_cache.float(), wk, bk,
                                     wv, bv, w.meta.private_block_tables, w.meta.seq_lens_tensor,
                                     w.meta.cache_type, w.scale)
    assert_close(simt, tensor.float(), "CUDA-core vs tensor-core path, head size 64", 5e-3, 5e-3)


def test_kv_reprojection_head_size_64_and_32():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(300, 256, generator=g).to(torch.float16)
    wk = (torch.randn(256, 256, generator=g) * 0.05).to(torch.float16)
    wv = (torch.randn(256, 256, generator=g) * 0.05).to(torch.float16)
    bk = torch.randn(256, generator=g).to(torch.float16)
    bv = torch.randn(256, generator=g).to(torch.float16)
    ref = torch.cat([O.linear_fp32(x, wk, bk), O.linear_fp32(x, wv, bv)], dim=1)
    for head_size in (64, 32):
        out = A.kv_reprojection(x.cuda(), wk.cuda(), bk.cuda(), wv.cuda(), bv.cuda(), head_size)
        assert_close(out, ref, f"kv_reprojection, head size {head_size}")


def test_cuda_core_and_tensor_core_reprojection_agree():
    """The same fp16 values through the tcgen05 kernel (fp16 tensors) and through the
    CUDA-core kernel (the same values held as fp32 tensors)."""
    w = small_workload(heads=2, head_dim=128, lens=(70, 300, 129), hidden=(True, True, False)).to("cuda")
    tensor = gpu_hybrid(w).clone()
    wk, bk, wv, bv = (t.float() for t in w.kv_weights())
    simt = A.hybrid_decode_attention(w.query.float(), w.kv_cache.float(), w.hidden_cache.float(), wk, bk,
                                     wv, bv, w.meta.private_block_tables, w.meta.seq_lens_tensor,
                                     w.meta.cache_type, w.scale)
    assert_close(simt, tensor.float(), "CUDA-core vs tensor-core path", 5e-3, 5e-3)


# --------------------------------------------------------------------------- #
# device status word
# --------------------------------------------------------------------------- #
def test_kv_requests_without_kv_cache_set_the_status_and_give_zero_rows():
    """A batch with K/V-cached requests but no K/V cache: the call succeeds on the host
    (it cannot see the cache types), the status word reads 8, the K/V requests' rows are
    zero (no stale partials are merged) and the hidden requests' rows are right."""
    w = small_workload(heads=2, head_dim=128, lens=(40, 9, 150, 64), hidden=(True, False, True, False))
    ref = oracle_out(w)
    dev = w.to("cuda")
    gpu_hybrid(dev)   # leaves valid partials of every request in the workspace
    wk, bk, wv, bv = dev.kv_weights()
    out = A.hybrid_decode_attention(dev.query, None, dev.hidden_cache, wk, bk, wv, bv,
                                    dev.meta.private_block_tables, dev.meta.seq_lens_tensor,
                                    dev.meta.cache_type, dev.scale, num_heads=2, head_size=128)
    ws = A.attention_workspace(out.device, 1, 1, 16, 1, 1)
    assert A.attention_status(ws) == 8
    with pytest.raises(RuntimeError, match="status 8"):
        A.raise_on_device_status(ws)
    assert_close(out[[0, 2]], ref[[0, 2]], "hidden requests without a K/V cache")
    assert float(out[[1, 3]].abs().max()) == 0.0
    assert A.attention_status(A.attention_workspace(out.device, 1, 1, 16, 1, 1)) == 8
    gpu_hybrid(dev)   # the next complete call resets the word
    A.raise_on_device_status(ws)


def test_reprojection_cycle_count_is_at_least_the_tensor_bound():
    """aps_reprojection_cycles after a hybrid call: CTA 0's cycles cover at least the 512 cycles
    per 64-element slab its tile pairs need on the tensor cores, and not absurdly more."""
    w = make_config_workload(5, device="cuda", batch=8, hidden_fraction=1.0)
    out = gpu_hybrid(w)
    assert torch.isfinite(out.float()).all()
    ws = A.attention_workspace(out.device, 1, 1, 16, 1, 1)
    cycles = A.reprojection_cycles(ws)
    subs = sum((s + 15) // 16 for s in w.seq_lens)
    units = ((subs + 7) // 8 + 1) // 2
    pairs = torch.cuda.get_device_properties(0).multi_processor_count // 2
    rounds = -(-units * OPT_13B.num_heads // pairs)
    need = rounds * (OPT_13B.hidden // 64) * 512
    assert need <= cycles <= 1.5 * need + 200_000, (cycles, need)


def test_bounded_wait_that_runs_out_marks_the_output():
    """A wait nobody satisfies gives up after its clock budget and leaves code 7; the
    combine step then writes NaN instead of numbers; the next call works as before."""
    from apt_serve_b200 import _native as N
    w = small_workload(heads=2, head_dim=128, lens=(40, 9, 150), hidden=(True, False, True)).to("cuda")
    good = gpu_hybrid(w).clone()
    ws = A.attention_workspace(good.device, 1, 1, 16, 1, 1)
    out = torch.zeros_like(good)
    bt = w.meta.private_block_tables
    N.check(N.lib().aps_selftest_bounded_wait(N.ptr(ws), ws.numel(), 200000, N.ptr(out), 3, bt.shape[1], 2, 128,
                                              16, out.stride(0), N.dtype_enum(out), N.current_stream(out.device)))
    assert A.attention_status(ws) == 7
    assert torch.isnan(out.float()).all()
    with pytest.raises(RuntimeError, match="status 7"):
        A.raise_on_device_status(ws)
    assert torch.equal(gpu_hybrid(w), good)


# --------------------------------------------------------------------------- #
# the layer-step in one call
# --------------------------------------------------------------------------- #
@pytest.mark.parametrize("case", ["fp16 aliased", "bf16 tensor-parallel slice", "fp32 config 1"])
def test_decode_layer_step_equals_separate_ops(case):
    """aps_decode_layer_step (new-token writes addressed from the block tables + attention)
    against the three separate calls fed from the index tensors: same cache bits, same
    output bits, and both within tolerance of the oracle's layer-step."""
    from apt_serve_b200 import mixed_cache_ops, ops
    if case == "fp16 aliased":
        w = small_workload(heads=2, head_dim=128, lens=(5, 40, 17, 129, 300, 16, 128, 1),
                           hidden=(True, False, True, False, True, False, True, True), device="cuda")
        tol = 2e-2
    elif case == "bf16 tensor-parallel slice":
        from apt_serve_b200.workloads import OPT_66B
        w = make_decode_workload(OPT_66B, [33, 200, 16, 310], [True, False, False, True], seed=11,
                                 device="cuda", tp_rank=3, tp_size=8)
        tol = 2e-2
    else:
        w = make_config_workload(1, device="cuda", kv_from_projection=True)
        tol = 1e-3
    cpu = w.cpu()
    ref = O.decode_layer_step(cpu.hidden_states, cpu.query, cpu.new_key, cpu.new_value, cpu.kv_cache,
                              cpu.hidden_cache, *cpu.kv_weights(), cpu.meta, cpu.scale)
    m, h, d = w.meta, w.heads, w.shape.head_dim
    alias = w.hidden_cache.data_ptr() == w.kv_cache.data_ptr()
    kv_a, kv_b = w.kv_cache.clone(), w.kv_cache.clone()
    hid_a = kv_a if alias else w.hidden_cache.clone()
    hid_b = kv_b if alias else w.hidden_cache.clone()
    wk, bk, wv, bv = w.kv_weights()
    # separate ops
    rows = m.kv_request_rows
    ops.reshape_and_cache_flash(w.new_key[rows].view(-1, h, d), w.new_value[rows].view(-1, h, d),
                                kv_a[0], kv_a[1], m.slot_mapping[m.kv_cache_use_tot])
    mixed_cache_ops.hidden_to_cache(w.hidden_states, hid_a, m.slot_mapping, m.hidden_cache_use_input,
                                    m.hidden_cache_store_tot)
    out_a = A.hybrid_decode_attention(w.query, kv_a, hid_a, wk, bk, wv, bv, m.private_block_tables,
                                      m.seq_lens_tensor, m.cache_type, w.scale).clone()
    # one call
    out_b = A.decode_layer_step(w.query, w.hidden_states, w.new_key, w.new_value, kv_b, hid_b, wk, bk,
                                wv, bv, m.private_block_tables, m.seq_lens_tensor, m.cache_type, w.scale)
    A.raise_on_device_status()
    assert torch.equal(kv_a.view(torch.uint8), kv_b.view(torch.uint8))
    assert torch.equal(hid_a.view(torch.uint8), hid_b.view(torch.uint8))
    assert torch.equal(kv_b.cpu().view(torch.uint8), cpu.kv_cache.view(torch.uint8))
    assert torch.equal(out_a, out_b)
    assert_close(out_b, ref, f"decode_layer_step {case}", tol, tol)


# --------------------------------------------------------------------------- #
# model-side callers
# --------------------------------------------------------------------------- #
def test_opt_attention_fused_matches_literal_and_oracle():
    w = small_workload(heads=2, head_dim=128, lens=(40, 9, 150, 64), hidden=(True, False, True, False),
                       with_shared_cache=True, device="cuda")
    meta = A.FlashAttentionMetadata.from_decode(w.meta)
    cpu = w.cpu()
    kv_ref = cpu.kv_cache.clone()
    (w_q, b_q), (w_k, b_k), (w_v, b_v) = O.qkv_slices(cpu.qkv_weight, cpu.qkv_bias)
    hs = cpu.hidden_states
    q = O.linear_fp32(hs, w_q, b_q).half()
    k_new = O.linear_fp32(hs, w_k, b_k).half()
    v_new = O.linear_fp32(hs, w_v, b_v).half()
    attn_ref = O.decode_layer_step(hs, q, k_new, v_new, kv_ref, kv_ref, w_k, b_k, w_v, b_v,
                                   cpu.meta, cpu.scale)
    y_ref = attn_ref @ cpu.o_weight.float().t() + cpu.o_bias.float()

    fused = OPTAttention(w.shape.hidden, 2, w.qkv_weight, w.qkv_bias, w.o_weight, w.o_bias, fused=True)
    kv1 = w.kv_cache.clone()
    y1 = fused(w.hidden_states, kv1, None, meta)           # reference metadata only
    assert_close(y1, y_ref, "fused OPTAttention", 3e-2, 3e-2)
    # cache contents after the step: the new hidden rows are copies (bit-exact); the new
    # K/V rows come from a GPU GEMM, so they match the CPU projection to rounding only
    rows1, rows_ref = O.flat_rows(kv1.cpu()), O.flat_rows(kv_ref)
    hid_slots = cpu.meta.slot_mapping[cpu.meta.hidden_cache_store_tot]
    assert torch.equal(rows1[hid_slots], rows_ref[hid_slots])
    assert torch.allclose(kv1.cpu().float(), kv_ref.float(), atol=4e-3, rtol=4e-3)

    literal = OPTAttention(w.shape.hidden, 2, w.qkv_weight, w.qkv_bias, w.o_weight, w.o_bias, fused=False)
    kv2, shared = w.kv_cache.clone(), w.shared_cache.clone()
    y2 = literal(w.hidden_states, kv2, shared, meta)
    hid_rows = [0, 2]
    assert_close(y2[hid_rows], y_ref[hid_rows], "literal op sequence, hidden requests", 3e-2, 3e-2)


def test_flash_attention_impl_kv_only_decode_and_prefill_write():
    w = small_workload(heads=2, head_dim=128, lens=(40, 9, 150), hidden=(False, False, False),
                       device="cuda")
    impl = A.FlashAttentionImpl(2, 128, w.scale, 2, None, None, "auto")
    meta = A.FlashAttentionMetadata.from_decode(w.meta)
    cpu = w.cpu()
    kv_ref = cpu.kv_cache.clone()
    ref = O.decode_layer_step(cpu.hidden_states, cpu.query, cpu.new_key, cpu.new_value, kv_ref,
                              kv_ref, *cpu.kv_weights(), cpu.meta, cpu.scale)
    kv = w.kv_cache.clone()
    out = impl.forward(w.query, w.new_key, w.new_value, kv, None, meta)
    assert_close(out, ref, "FlashAttentionImpl decode")
    assert torch.equal(kv.cpu().view(torch.uint8), kv_ref.view(torch.uint8))


def test_flash_attention_impl_prefix_cached_prefill():
    """Prefill whose prompts continue a cached prefix (aptserve_flash_attn.py:432-447): the new
    tokens' K/V go to their slots, then each new token attends to the whole context through the
    block table, causally aligned to the context's end."""
    g = torch.Generator().manual_seed(11)
    heads, d, bs, nb = 2, 64, 16, 32
    ctx, new = [32, 48, 0], [10, 5, 20]
    tables = [[3, 7, 9, 0], [1, 4, 12, 15], [20, 21, 0, 0]]
    kv = (torch.randn(2, nb, bs, heads, d, generator=g) * 0.5).to(torch.float16)
    n = sum(new)
    q, k, v = ((torch.randn(n, heads * d, generator=g) * 0.5).to(torch.float16) for _ in range(3))
    slots, starts = [], [0]
    for c, m, t in zip(ctx, new, tables):
        slots += [t[p // bs] * bs + p % bs for p in range(c, c + m)]
        starts.append(starts[-1] + m)
    seq_lens = [c + m for c, m in zip(ctx, new)]
    # expected: fp32 attention over [cached prefix ; new tokens] per sequence
    ref = torch.empty(n, heads * d)
    kv_ref = kv.clone()
    flat_k, flat_v = kv_ref[0].view(nb * bs, heads, d), kv_ref[1].view(nb * bs, heads, d)
    flat_k[slots] = k.view(n, heads, d)
    flat_v[slots] = v.view(n, heads, d)
    scale = d ** -0.5
    for i, (c, m, t) in enumerate(zip(ctx, new, tables)):
        rows = [t[p // bs] * bs + p % bs for p in range(c + m)]
        kk, vv = flat_k[rows].float(), flat_v[rows].float()
        qq = q[starts[i]:starts[i + 1]].view(m, heads, d).float()
        sc = torch.einsum("qhd,khd->hqk", qq, kk) * scale
        mask = torch.arange(c + m)[None, :] <= (c + torch.arange(m))[:, None]
        sc = sc.masked_fill(~mask[None], float("-inf"))
        ref[starts[i]:starts[i + 1]] = torch.einsum("hqk,khd->qhd", sc.softmax(-1), vv).reshape(m, heads * d)
    dev = "cuda"
    empty = torch.zeros(0, dtype=torch.int64, device=dev)
    cum = [0]
    for s_ in seq_lens:
        cum.append(cum[-1] + s_)
    meta = A.FlashAttentionMetadata(
        num_prefills=3, num_prefill_tokens=n, num_decode_tokens=0, num_hidden_cache_tokens=0,
        num_tot_tokens=n, slot_mapping=torch.tensor(slots, dtype=torch.int64, device=dev),
        slot_mapping_shared=empty, hidden_cache_use_tot=empty, kv_cache_use_tot=empty,
        hidden_cache_use_input=empty, hidden_cache_store_tot=empty, hidden_holder_upd=empty,
        hidden_holder_pull=empty, seq_lens=seq_lens,
        seq_lens_tensor=torch.tensor(seq_lens, dtype=torch.int32, device=dev), max_query_len=max(new),
        max_prefill_seq_len=max(seq_lens), max_decode_seq_len=0,
        query_start_loc=torch.tensor(starts, dtype=torch.int32, device=dev),
        seq_start_loc=torch.tensor(cum, dtype=torch.int32, device=dev),
        context_lens_tensor=torch.tensor(ctx, dtype=torch.int32, device=dev),
        block_tables=torch.tensor(tables, dtype=torch.int32, device=dev), use_cuda_graph=False)
    impl = A.FlashAttentionImpl(heads, d, scale, heads, None, None, "auto")
    kv_dev = kv.to(dev)
    out = impl.forward(q.to(dev), k.to(dev), v.to(dev), kv_dev, None, meta)
    assert torch.equal(kv_dev.cpu().view(torch.uint8), kv_ref.view(torch.uint8))
    assert_close(out, ref, "prefix-cached prefill")


def test_opt_attention_prefill_fused_write_matches_literal():
    """A prefill batch with hidden-designated prompts through both forms of OPTAttention:
    same cache contents bit for bit, same attention output."""
    from apt_serve_b200.metadata import BlockPool, build_prefill_metadata
    rng = np.random.default_rng(4)
    heads, d, bs = 2, 128, 16
    e = heads * d
    lens, hid = [30, 17, 64], [True, False, True]
    nb = 16
    pool = BlockPool(nb, rng)
    tables = [pool.table_for(s, bs, u) for s, u in zip(lens, hid)]
    meta = A.FlashAttentionMetadata.from_prefill(build_prefill_metadata(lens, hid, tables, bs).to("cuda"))
    g = torch.Generator(device="cuda").manual_seed(2)
    hs = torch.randn(sum(lens), e, generator=g, device="cuda", dtype=torch.float16)
    w = (torch.randn(3 * e, e, generator=g, device="cuda") * 0.05).half()
    b = torch.randn(3 * e, generator=g, device="cuda").half()
    wo = (torch.randn(e, e, generator=g, device="cuda") * 0.05).half()
    bo = torch.randn(e, generator=g, device="cuda").half()
    outs, caches = [], []
    for fused in (True, False):
        layer = OPTAttention(e, heads, w, b, wo, bo, fused=fused)
        cache = torch.zeros(2, nb, bs, heads, d, device="cuda", dtype=torch.float16)
        outs.append(layer(hs, cache, None, meta))
        caches.append(cache)
    assert torch.equal(caches[0], caches[1])
    assert caches[0].abs().sum() > 0
    assert_close(outs[0], outs[1].float(), "prefill output", 1e-3, 1e-3)


def test_decode_layer_step_replays_from_a_cuda_graph():
    """The layer-step enqueues kernels and nothing else (no allocation, no synchronisation, no
    host read of device data), so it can be captured in a CUDA graph -- the reference itself
    cannot (it must run with --enforce-eager).  A captured step is replayed on new inputs
    written into the captured buffers and compared, bit for bit, with an eager call."""
    w = small_workload(heads=2, head_dim=128, lens=(5, 40, 17, 129, 300, 16, 128, 1),
                       hidden=(True, False, True, False, True, False, True, True), device="cuda")
    m = w.meta
    wk, bk, wv, bv = w.kv_weights()
    ws = A.attention_workspace(w.query.device, len(w.seq_lens), m.private_block_tables.shape[1], 16, 2, 128)
    kv_graph, kv_eager = w.kv_cache.clone(), w.kv_cache.clone()
    q, hs, nk, nv = w.query.clone(), w.hidden_states.clone(), w.new_key.clone(), w.new_value.clone()
    out_graph = torch.empty_like(q)

    def step(kv, out):
        return A.decode_layer_step(q, hs, nk, nv, kv, kv, wk, bk, wv, bv, m.private_block_tables,
                                   m.seq_lens_tensor, m.cache_type, w.scale, out=out, workspace=ws)
    step(w.kv_cache.clone(), torch.empty_like(q))       # first call: kernel attributes, tensor maps
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step(kv_graph, out_graph)
    for seed in (1, 2):
        gen = torch.Generator(device="cuda").manual_seed(seed)
        for t in (q, hs, nk, nv):
            t.copy_(torch.randn(t.shape, device="cuda", generator=gen).to(t.dtype))
        g.replay()
        ref = step(kv_eager, torch.empty_like(q))
        torch.cuda.synchronize()
        A.raise_on_device_status(ws)
        assert torch.equal(out_graph, ref)
        assert torch.equal(kv_graph.view(torch.uint8), kv_eager.view(torch.uint8))


# --------------------------------------------------------------------------- #
# seeded sweep over ragged batch compositions (tile packing, segments, edges)
# --------------------------------------------------------------------------- #
EDGE_LENS = (1, 2, 15, 16, 17, 31, 32, 33, 47, 48, 127, 128, 129, 143, 144, 145, 255, 256, 257, 511, 513)


@pytest.mark.parametrize("seed", range(10))
def test_hybrid_ragged_batches_sweep(seed):
    """Random batches whose lengths sit on and next to the 16-token block and 128-row tile
    boundaries, so that requests share tiles, span tiles and end exactly on their edges;
    cache types, head counts, dtype and batch size vary with the seed."""
    rng = np.random.default_rng(7000 + seed)
    batch = int(rng.integers(1, 28))
    lens = [int(rng.choice(EDGE_LENS)) if rng.random() < 0.7 else int(rng.integers(1, 700))
            for _ in range(batch)]
    mode = seed % 5
    hidden = ([True] * batch if mode == 0 else [False] * batch if mode == 1
              else [bool(b) for b in rng.random(batch) < (0.25, 0.5, 0.75)[mode - 2]])
    heads = int(rng.integers(1, 4))
    dtype = (torch.float16, torch.bfloat16)[seed % 2]
    w = small_workload(dtype=dtype, heads=heads, head_dim=128, lens=lens, hidden=hidden, seed=seed)
    ref = oracle_out(w)
    dev = w.to("cuda")
    out = gpu_hybrid(dev)
    assert_close(out, ref, f"sweep seed {seed}: B={batch} heads={heads} {dtype} lens={lens} hidden={hidden}")
    again = gpu_hybrid(dev)
    assert torch.equal(out, again), "two runs on the same inputs differ"


@pytest.mark.parametrize("seed", range(6))
def test_hybrid_ragged_batches_sweep_small_heads_tensor_path(seed):
    """The ragged sweep on the tensor-core kernel with two (head size 64) and four (head
    size 32) heads per accumulator tile."""
    rng = np.random.default_rng(7200 + seed)
    batch = int(rng.integers(1, 24))
    lens = [int(rng.choice(EDGE_LENS)) if rng.random() < 0.7 else int(rng.integers(1, 700))
            for _ in range(batch)]
    hidden = [bool(b) for b in rng.random(batch) < (0.5, 1.0, 0.75)[seed % 3]]
    head_dim = (64, 32)[seed % 2]
    heads = (128 // head_dim) * int(rng.integers(1, 4))
    dtype = (torch.float16, torch.bfloat16)[(seed // 2) % 2]
    w = small_workload(dtype=dtype, heads=heads, head_dim=head_dim, lens=lens, hidden=hidden, seed=seed)
    ref = oracle_out(w)
    dev = w.to("cuda")
    out = gpu_hybrid(dev)
    assert_close(out, ref, f"sweep seed {seed}: B={batch} {heads} x {head_dim} {dtype} lens={lens} hidden={hidden}")
    assert torch.equal(out, gpu_hybrid(dev)), "two runs on the same inputs differ"


@pytest.mark.parametrize("seed", range(4))
def test_hybrid_ragged_batches_sweep_cuda_core_path(seed):
    """The same sweep on the fp32 CUDA-core re-projection (head sizes 64 and 32)."""
    rng = np.random.default_rng(7100 + seed)
    batch = int(rng.integers(1, 12))
    lens = [int(rng.choice(EDGE_LENS[:16])) if rng.random() < 0.7 else int(rng.integers(1, 300))
            for _ in range(batch)]
    hidden = [bool(b) for b in rng.random(batch) < 0.6]
    head_dim = (64, 32)[seed % 2]
    w = small_workload(dtype=torch.float32, heads=int(rng.integers(1, 5)), head_dim=head_dim, lens=lens,
                       hidden=hidden, seed=seed)
    ref = oracle_out(w)
    out = gpu_hybrid(w.to("cuda"))
    assert_close(out, ref, f"fp32 sweep seed {seed}: lens={lens} hidden={hidden}", atol=1e-4, rtol=1e-4)


def test_more_requests_than_plan_threads():
    """1300 short requests: the plan kernel's threads own two requests each, so its list
    filling runs two rounds; K/V and hidden requests alternate in runs of three."""
    rng = np.random.default_rng(42)
    batch = 1300
    lens = [int(v) for v in rng.integers(1, 41, size=batch)]
    hidden = [(r // 3) % 2 == 0 for r in range(batch)]
    w = small_workload(dtype=torch.float16, heads=1, head_dim=128, lens=lens, hidden=hidden, seed=9)
    ref = oracle_out(w)
    out = gpu_hybrid(w.to("cuda"))
    assert_close(out, ref, "1300 requests")
