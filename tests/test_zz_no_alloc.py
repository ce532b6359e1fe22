"""The allocation-free decode attention entry point, called through the C ABI.

``aps_paged_decode_attention_static`` keeps its scratch in a 32 MiB array inside the
library's device image, for hosts that cannot allocate device memory at decode time
(a worker whose cache engine already owns all free HBM, or a host language without a
device-memory pool).  It must give what ``aps_paged_decode_attention`` gives with a
caller-provided workspace -- here on two calls in a row with different batches, so
that whatever the first call left in the shared array is shown not to matter.

This file is named to be collected last: it must pass both on its own in a fresh
process and after every other GPU test has run in the same process.
"""
import pytest
import torch

from apt_serve_b200 import _native as N
from apt_serve_b200.workloads import LayerShape, make_decode_workload

from helpers import assert_close

pytestmark = pytest.mark.gpu


def _args(w, out):
    kc, vc = w.kv_cache[0], w.kv_cache[1]
    bt, sl = w.meta.block_tables, w.meta.seq_lens_tensor
    _, bs, h, d = kc.shape
    head = [N.ptr(out), N.ptr(w.query), N.ptr(kc), N.ptr(vc), N.ptr(bt), N.ptr(sl),
            w.query.shape[0], bt.shape[1], h, d, bs, w.query.stride(0), out.stride(0),
            kc.stride(0), float(w.scale)]
    return head, (w.query.shape[0], bt.shape[1], bs, h, d)


def _both_ways(w):
    lib = N.lib()
    dev = w.query.device
    stream = N.current_stream(dev)
    dtype = N.dtype_enum(w.query)
    out_ws = torch.zeros_like(w.query)
    out_static = torch.zeros_like(w.query)
    head, dims = _args(w, out_ws)
    need = lib.aps_attention_workspace_bytes(*dims)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    N.check(lib.aps_paged_decode_attention(*head, N.ptr(ws), ws.numel(), dtype, stream))
    head2, _ = _args(w, out_static)
    N.check(lib.aps_paged_decode_attention_static(*head2, dtype, stream))
    torch.cuda.synchronize()
    return out_ws, out_static


def test_static_scratch_matches_workspace_version_twice_in_a_row():
    first = make_decode_workload(LayerShape("a", 8, 128, 1024, torch.float16),
                                 [300, 17, 2048, 129, 640, 1], [False] * 6, seed=21, device="cuda")
    second = make_decode_workload(LayerShape("b", 12, 64, 768, torch.float32),
                                  [45, 512, 33], [False] * 3, seed=22, device="cuda")
    for w, tol in ((first, 2e-2), (second, 1e-4), (first, 2e-2)):
        out_ws, out_static = _both_ways(w)
        assert torch.isfinite(out_static.float()).all()
        assert_close(out_static, out_ws.float(), "static scratch vs caller workspace", tol, tol)
        assert torch.equal(out_static, out_ws)  # same kernels, same order of operations


def test_static_scratch_rejects_batches_beyond_its_size():
    lib = N.lib()
    w = make_decode_workload(LayerShape("a", 8, 128, 1024, torch.float16), [40, 50], [False] * 2,
                             seed=3, device="cuda")
    out = torch.zeros_like(w.query)
    head, _ = _args(w, out)
    # claim a batch of 4096 requests with 128-block tables: far more than 32 MiB of partials
    head[6], head[7] = 4096, 128
    st = lib.aps_paged_decode_attention_static(*head, N.dtype_enum(w.query), N.current_stream(out.device))
    assert st == N.APS_ERR_WORKSPACE
    msg = lib.aps_last_error().decode()
    assert "built-in" in msg and "aps_paged_decode_attention" in msg
    torch.cuda.synchronize()
    assert out.abs().sum() == 0  # nothing was launched
