"""Cache allocation and block moves without the shared cache
(aptserve_cache_engine.py:15-119, aptserve_block_manager.py:535-540)."""
import pytest
import torch

from apt_serve_b200.cache_engine import CacheEngine, physical_block_map


def test_physical_block_map_folds_the_v_plane_ids():
    nb_src, nb_dst = 10, 6
    pairs = [(3, 1), (13, 7), (4, 2), (9, 0)]           # (13, 7) = V halves of (3, 1)
    assert physical_block_map(pairs, nb_src, nb_dst) == [(3, 1), (4, 2), (9, 0)]


def test_physical_block_map_rejects_maps_that_split_a_block():
    with pytest.raises(ValueError):
        physical_block_map([(3, 1), (13, 8)], 10, 6)     # halves of block 3 to different blocks
    with pytest.raises(ValueError):
        physical_block_map([(3, 1), (4, 1)], 10, 6)      # two sources onto one block
    with pytest.raises(ValueError):
        physical_block_map([(3, 7)], 10, 6)              # K half onto a V half
    with pytest.raises(ValueError):
        physical_block_map([(20, 0)], 10, 6)


def test_block_budget_without_the_shared_cache():
    # OPT-13B, fp16: 40 layers x 2 planes x 16 tokens x 5120 x 2 B = 13 107 200 B per block
    args = (40, 40, 128, 16, torch.float16)
    assert CacheEngine.get_cache_block_size(*args) == 40 * 2 * 16 * 5120 * 2
    budget = 100 << 30
    with_shared = CacheEngine.num_blocks_for_budget(budget, *args, with_shared_cache=True)
    without = CacheEngine.num_blocks_for_budget(budget, *args)
    # the shared cache costs two single-layer blocks per block: 2/40 of a 40-layer block
    assert without == budget // 13107200
    assert with_shared == budget // (13107200 + 2 * 327680)
    assert without > with_shared


def test_tensor_parallel_rank_pays_for_dedicated_hidden_rows():
    full = CacheEngine.get_cache_block_size(64, 72, 128, 16, torch.bfloat16, hidden_size=9216)
    rank = CacheEngine.get_cache_block_size(64, 9, 128, 16, torch.bfloat16, hidden_size=9216)
    assert full == 64 * 2 * 16 * 9216 * 2
    assert rank == 64 * (2 * 16 * 9 * 128 + 2 * 16 * 9216) * 2


def test_allocation_and_host_side_moves():
    e = CacheEngine(2, 4, 32, 16, num_gpu_blocks=6, num_cpu_blocks=5, dtype=torch.float32, device="cpu",
                    pin_memory=False)
    assert e.shared_cache is None and e.aliased_hidden
    assert e.gpu_cache[0].shape == (2, 6, 16, 4, 32) and e.cpu_cache[1].shape == (2, 5, 16, 4, 32)
    for c in e.gpu_cache:
        c.copy_(torch.randn_like(c))
    before = [c.clone() for c in e.gpu_cache]
    e.swap_out(torch.tensor([[1, 4], [5, 0]]))
    for g, c in zip(before, e.cpu_cache):
        assert torch.equal(c[:, 4], g[:, 1]) and torch.equal(c[:, 0], g[:, 5])
    for c in e.gpu_cache:
        c.zero_()
    e.swap_in(torch.tensor([[4, 2], [0, 3]]))
    for g, c in zip(before, e.gpu_cache):
        assert torch.equal(c[:, 2], g[:, 1]) and torch.equal(c[:, 3], g[:, 5])
    legacy = CacheEngine(1, 4, 32, 16, 6, 1, torch.float32, device="cpu", with_shared_cache=True,
                         pin_memory=False)
    assert legacy.shared_cache.shape == (2, 12, 16, 4, 32)
    with pytest.raises(ValueError):
        CacheEngine(1, 4, 32, 8, 1, 1, torch.float32, device="cpu")


@pytest.mark.gpu
def test_hidden_requests_survive_a_swap_out_and_in():
    """A hidden-cached batch is swapped out to pinned host memory block by block, its GPU
    blocks are wiped, and it comes back into OTHER physical blocks: the fused attention
    over the re-pointed block tables gives bit-identical results."""
    from apt_serve_b200 import attention as A
    from helpers import small_workload
    w = small_workload(dtype=torch.float16, device="cuda", seed=11)
    m = w.meta
    nb = w.kv_cache.shape[1]
    wk, bk, wv, bv = w.kv_weights()
    ref = A.hybrid_decode_attention(w.query, w.kv_cache, w.hidden_cache, wk, bk, wv, bv,
                                    m.private_block_tables, m.seq_lens_tensor, m.cache_type, w.scale).clone()
    e = CacheEngine(1, w.heads, w.shape.head_dim, w.shape.block_size, nb, nb, torch.float16)
    e.gpu_cache[0].copy_(w.kv_cache)
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(3))
    ids = torch.arange(nb)
    e.swap_out(torch.stack([ids, perm], dim=1))            # block i -> host block perm[i]
    e.gpu_cache[0].zero_()
    perm2 = torch.randperm(nb, generator=torch.Generator().manual_seed(4))
    e.swap_in(torch.stack([perm, perm2], dim=1))           # host block perm[i] -> GPU block perm2[i]
    torch.cuda.synchronize()
    # re-point the tables: physical id p -> perm2[p], V-plane ids keep their + NB
    t = m.private_block_tables.cpu().long()
    moved = (perm2[t % nb] + (t // nb) * nb).to(torch.int32).cuda()
    out = A.hybrid_decode_attention(w.query, e.gpu_cache[0], e.gpu_cache[0], wk, bk, wv, bv, moved,
                                    m.seq_lens_tensor, m.cache_type, w.scale)
    assert torch.equal(out, ref)


@pytest.mark.gpu
def test_copy_moves_both_halves_of_a_physical_block():
    e = CacheEngine(3, 4, 64, 16, num_gpu_blocks=8, num_cpu_blocks=1, dtype=torch.float16)
    for c in e.gpu_cache:
        c.copy_(torch.randn(c.shape, device="cuda").half())
    before = [c.clone() for c in e.gpu_cache]
    e.copy(torch.tensor([[1, 5], [2, 7]], device="cuda"))
    torch.cuda.synchronize()
    for g, c in zip(before, e.gpu_cache):
        assert torch.equal(c[:, 5], g[:, 1]) and torch.equal(c[:, 7], g[:, 2])
        assert torch.equal(c[:, :5], g[:, :5]) and torch.equal(c[:, 6], g[:, 6])
