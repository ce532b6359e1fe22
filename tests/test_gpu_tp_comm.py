"""The library's NCCL communicator (aps_tp_*): the all-reduce after o_proj
(aptserve_linear.py:827-829) through the C ABI."""
import ctypes
import multiprocessing as mp
import os
import time

import pytest
import torch

from apt_serve_b200 import _native


def test_argument_checks_need_no_device():
    lib = _native.lib()
    assert lib.aps_tp_destroy(None) == _native.APS_OK
    assert lib.aps_tp_allreduce(None, None, 4, 1, None) == _native.APS_ERR_NULL_POINTER
    assert lib.aps_tp_unique_id(None) == _native.APS_ERR_NULL_POINTER
    handle = ctypes.c_void_p()
    uid = ctypes.create_string_buffer(128)
    assert lib.aps_tp_init(ctypes.byref(handle), ctypes.cast(uid, ctypes.c_void_p), 2, 2) == _native.APS_ERR_SHAPE
    assert b"rank 2 of 2" in lib.aps_last_error()


@pytest.mark.gpu
def test_single_rank_communicator_round_trip():
    from apt_serve_b200 import layers, tp_comm
    comm = tp_comm.TensorParallelComm(0, 1, tp_comm.new_unique_id())
    try:
        assert comm.size() == 1
        for dtype in (torch.float32, torch.float16, torch.bfloat16):
            x = torch.randn(512, 768, device="cuda").to(dtype)
            want = x.clone()
            assert comm.all_reduce(x) is x
            torch.cuda.synchronize()
            assert torch.equal(x, want)
        with pytest.raises(ValueError):
            comm.all_reduce(torch.zeros(4, 4, device="cuda").t()[1:])
        with pytest.raises(ValueError):
            comm.all_reduce(torch.zeros(4, device="cuda", dtype=torch.int32))
        tp_comm.install(comm)
        y = torch.ones(8, device="cuda")
        assert layers.tensor_model_parallel_all_reduce(y) is y
    finally:
        comm.destroy()
    assert tp_comm.installed() is None
    with pytest.raises(RuntimeError):
        comm.all_reduce(torch.zeros(4, device="cuda"))


def _rank_main(rank, world, id_path, out_path):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    from apt_serve_b200 import tp_comm
    torch.cuda.set_device(rank)
    if rank == 0:
        uid = tp_comm.new_unique_id()
        with open(id_path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(id_path + ".tmp", id_path)
    else:
        deadline = time.time() + 60
        while not os.path.exists(id_path):
            if time.time() > deadline:
                raise RuntimeError("rank 0 never published the id")
            time.sleep(0.05)
        with open(id_path, "rb") as f:
            uid = f.read()
    comm = tp_comm.TensorParallelComm(rank, world, uid)
    ok = comm.size() == world
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        g = torch.Generator(device="cuda").manual_seed(5)
        base = torch.randn(512, 9216, device="cuda", generator=g).to(dtype)   # same on every rank
        x = (base * (rank + 1)).contiguous()
        comm.all_reduce(x)
        torch.cuda.synchronize()
        want = sum((base * (r + 1)).float() for r in range(world))
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        ok = ok and torch.allclose(x.float(), want, atol=tol, rtol=tol)
    comm.destroy()
    with open(f"{out_path}.{rank}", "w") as f:
        f.write("ok" if ok else "mismatch")


@pytest.mark.gpu
def test_all_reduce_over_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    id_path, out_path = str(tmp_path / "nccl_id"), str(tmp_path / "result")
    procs = [ctx.Process(target=_rank_main, args=(r, world, id_path, out_path)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    for p in procs:
        if p.is_alive():          # a rank that never came back: end exactly that process
            p.kill()
            pytest.fail("a rank did not finish")
    for r in range(world):
        assert procs[r].exitcode == 0
        assert open(f"{out_path}.{r}").read() == "ok"
