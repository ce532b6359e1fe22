"""Shared helpers of the test-suite."""
import numpy as np
import torch

from apt_serve_b200.metadata import BlockPool, blocks_needed, build_decode_metadata
from apt_serve_b200.workloads import LayerShape, make_decode_workload

ATOL = RTOL = 2e-2  # |x - ref| <= 2e-2 + 2e-2 * |ref| against the fp32 oracle


def assert_close(x: torch.Tensor, ref: torch.Tensor, what: str = "", atol=ATOL, rtol=RTOL):
    x = x.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert torch.isfinite(x).all(), f"{what}: non-finite values"
    err = (x - ref).abs()
    bound = atol + rtol * ref.abs()
    bad = err > bound
    assert not bad.any(), (f"{what}: {int(bad.sum())} / {bad.numel()} outside tolerance, "
                           f"max abs err {float(err.max()):.4g}")


def tiny_shape(dtype=torch.float32, heads=4, head_dim=32, hidden=None) -> LayerShape:
    return LayerShape("tiny", heads, head_dim, heads * head_dim if hidden is None else hidden, dtype)


def small_workload(dtype=torch.float16, heads=2, head_dim=128, lens=(5, 40, 17, 129, 300, 16),
                   hidden=(True, False, True, False, True, False), seed=3, device="cpu", **kw):
    shape = LayerShape("small", heads, head_dim, heads * head_dim, dtype)
    return make_decode_workload(shape, list(lens), list(hidden), seed, device, **kw)
