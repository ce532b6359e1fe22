"""Tensor-parallel host logic on CPU ranks (gloo, world size 2): head sharding of
the workload generator, the row-parallel o_proj with its all-reduce, and bias
added once after the reduce.  The attention of each shard comes from the oracle,
so no GPU is involved."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import hybrid_cache_oracle as O
        from apt_serve_b200.layers import RowParallelLinear, tensor_model_parallel_all_reduce
        from apt_serve_b200.workloads import LayerShape, make_decode_workload

        shape = LayerShape("t", 4, 32, 128, torch.float32)
        lens, hid = [20, 35, 7, 50], [True, False, True, False]
        w = make_decode_workload(shape, lens, hid, seed=11, tp_rank=rank, tp_size=world)
        assert w.kv_cache.shape[3] == 4 // world
        assert w.hidden_cache.shape[-1] == shape.hidden and w.hidden_cache.shape[3] == 1
        # index tensors are identical on every rank (the reference broadcasts them)
        sig = torch.cat([w.meta.slot_mapping, w.meta.block_tables.flatten().long()])
        gathered = [torch.empty_like(sig) for _ in range(world)]
        dist.all_gather(gathered, sig)
        assert all(torch.equal(g, sig) for g in gathered)
        # replicated hidden rows are identical too
        chk = O.flat_rows(w.hidden_cache).double().sum().reshape(1)
        both = [torch.empty_like(chk) for _ in range(world)]
        dist.all_gather(both, chk)
        assert torch.equal(both[0], both[1])

        wk, bk, wv, bv = w.kv_weights()
        attn = O.hybrid_decode_attention(w.query, w.kv_cache, w.hidden_cache, wk, bk, wv, bv,
                                         w.meta.private_block_tables, w.meta.seq_lens_tensor,
                                         w.meta.cache_type, w.scale)
        layer = RowParallelLinear(w.o_weight, w.o_bias)
        y, _ = layer(attn)

        # unsharded result, computed locally from the full-width draw
        full = make_decode_workload(shape, lens, hid, seed=11)
        fk, fbk, fv, fbv = full.kv_weights()
        ref = O.hybrid_decode_attention(full.query, full.kv_cache, full.hidden_cache, fk, fbk, fv,
                                        fbv, full.meta.private_block_tables,
                                        full.meta.seq_lens_tensor, full.meta.cache_type, full.scale)
        hd = attn.shape[1]
        assert torch.allclose(attn, ref[:, rank * hd:(rank + 1) * hd], atol=1e-5)
        y_ref = ref @ full.o_weight.t() + full.o_bias
        assert torch.allclose(y, y_ref, atol=1e-4), float((y - y_ref).abs().max())
        # a rank count that does not divide the heads is refused
        try:
            make_decode_workload(shape, lens, hid, seed=11, tp_rank=0, tp_size=3)
            raise SystemExit("expected an assertion for 4 heads over 3 ranks")
        except AssertionError:
            pass
        x = torch.ones(3) * (rank + 1)
        assert torch.equal(tensor_model_parallel_all_reduce(x), torch.ones(3) * 3)
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_row_parallel_attention_block_two_cpu_ranks(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_all_reduce_is_identity_without_a_group():
    from apt_serve_b200.layers import tensor_model_parallel_all_reduce
    x = torch.arange(4.0)
    assert torch.equal(tensor_model_parallel_all_reduce(x), x)
