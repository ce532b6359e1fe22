"""Profit coefficient of the hybrid-cache scheduler, calibrated from the fused path.

The reference derives the coefficient its scheduler charges per hidden block
(aptserve_scheduler.py:586, 634: ``profit - U * coef * n_blocks``) by timing the K/V
re-projection GEMM ``F.linear(x, w_qkv)`` of every layer for 1, 101, ..., 4001 tokens,
regressing the times on the block counts and dividing the slope by five
(aptserve_llm_engine.py:316-354).  Here the re-projection happens inside the hybrid
decode attention kernel, so the quantity to time is that kernel on hidden-cached
requests; the regression and its post-processing are kept as the reference has them
so that the scheduler's inequality keeps its meaning.

``fit_profit_coefficient`` is the host arithmetic (numpy only); ``probe_profit_coefficient``
produces its inputs by timing the fused path on the current CUDA device.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence, Tuple

import numpy as np

# the reference's sweep: range(1, 4101, 100) tokens (aptserve_llm_engine.py:326)
DEFAULT_TOKEN_COUNTS = tuple(range(1, 4101, 100))
# the slope is divided by this constant (aptserve_llm_engine.py:346)
SLOPE_DIVISOR = 5.0


def block_counts(token_counts: Sequence[int], block_size: int) -> np.ndarray:
    """Token counts -> regressor values: whole blocks, at least one for a non-empty
    sample, with the origin prepended (aptserve_llm_engine.py:336-340)."""
    x = np.asarray([0] + list(token_counts), dtype=np.int64) // int(block_size)
    tail = x[1:]
    tail[tail == 0] = 1
    return x


def fit_profit_coefficient(token_counts: Sequence[int], seconds: Sequence[float],
                           block_size: int) -> float:
    """Ordinary least squares with intercept of ``[0] + seconds`` on the block counts;
    returns slope / 5 (aptserve_llm_engine.py:336-346)."""
    if len(token_counts) != len(seconds):
        raise ValueError("one time per token count is required")
    if len(token_counts) < 2:
        raise ValueError("at least two samples are needed for a slope")
    x = block_counts(token_counts, block_size).astype(np.float64)
    y = np.asarray([0.0] + list(seconds), dtype=np.float64)
    xc = x - x.mean()
    denom = float(np.dot(xc, xc))
    if denom == 0.0:
        raise ValueError("all samples fall into the same number of blocks")
    slope = float(np.dot(xc, y - y.mean())) / denom
    return slope / SLOPE_DIVISOR


def probe_profit_coefficient(num_heads: int, head_size: int, hidden_size: int, num_layers: int,
                             block_size: int, dtype=None, device="cuda",
                             token_counts: Sequence[int] = DEFAULT_TOKEN_COUNTS,
                             repeats: int = 3, seed: int = 0,
                             timer: Optional[Callable[[int], float]] = None
                             ) -> Tuple[float, np.ndarray]:
    """Time the fused hidden path for each token count and fit the coefficient.

    One sample is one hidden-cached request of ``n`` tokens attended by all heads of a
    layer, timed with CUDA events (the fastest of ``repeats``) and multiplied by
    ``num_layers`` -- the reference times ``num_layers`` back-to-back GEMMs of one layer's
    weights (aptserve_llm_engine.py:330-331).  Returns ``(coef, seconds)``.

    ``timer(n) -> seconds`` replaces the GPU measurement (tests, or a caller who times the
    whole model instead of one layer).
    """
    if timer is None:
        timer = _fused_path_timer(num_heads, head_size, hidden_size, block_size, dtype, device,
                                  max(token_counts), repeats, seed)
        scale = float(num_layers)
    else:
        scale = 1.0
    seconds = np.asarray([timer(int(n)) * scale for n in token_counts], dtype=np.float64)
    return fit_profit_coefficient(token_counts, seconds, block_size), seconds


def _fused_path_timer(num_heads, head_size, hidden_size, block_size, dtype, device, max_tokens,
                      repeats, seed) -> Callable[[int], float]:
    import torch

    from . import attention as A

    dtype = dtype or torch.float16
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("the probe times the CUDA path; there is no CPU path to time")
    hd = num_heads * head_size
    if hd != hidden_size:
        raise ValueError("the probe lays hidden rows into the K/V planes, which needs H*D == E")
    gen = torch.Generator(device=dev).manual_seed(seed)
    n_logical = (max_tokens + block_size - 1) // block_size
    n_phys = (n_logical + 1) // 2
    kv_cache = torch.randn((2, n_phys, block_size, num_heads, head_size), device=dev, dtype=dtype,
                           generator=gen)
    w = [torch.randn((hd, hidden_size), device=dev, dtype=dtype, generator=gen) * 0.02 for _ in range(2)]
    b = [torch.zeros(hd, device=dev, dtype=dtype) for _ in range(2)]
    query = torch.randn((1, hd), device=dev, dtype=dtype, generator=gen)
    # logical block 2i -> physical block i, logical block 2i+1 -> i + NB (its V plane)
    table = torch.tensor([[(j // 2) + (n_phys if j % 2 else 0) for j in range(n_logical)]],
                         device=dev, dtype=torch.int32)
    cache_type = torch.ones(1, device=dev, dtype=torch.int32)
    scale = head_size ** -0.5

    def time_one(n: int) -> float:
        seq = torch.tensor([n], device=dev, dtype=torch.int32)
        best = float("inf")
        for _ in range(repeats + 1):   # the first run also warms the kernel up
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            A.hybrid_decode_attention(query, kv_cache, kv_cache, w[0], b[0], w[1], b[1], table, seq,
                                      cache_type, scale)
            stop.record()
            stop.synchronize()
            best = min(best, start.elapsed_time(stop) * 1e-3)
        return best

    return time_one


if __name__ == "__main__":
    import argparse
    import json

    import torch

    from .workloads import OPT_13B

    ap = argparse.ArgumentParser(description="profit coefficient of the fused hidden path")
    ap.add_argument("--layers", type=int, default=40)
    args = ap.parse_args()
    s = OPT_13B
    coef, secs = probe_profit_coefficient(s.num_heads, s.head_dim, s.hidden, args.layers, s.block_size,
                                          dtype=s.dtype)
    print(json.dumps({"model": s.name, "layers": args.layers, "profit_coefficient": coef,
                      "seconds_at_1_token": secs[0], "seconds_at_4001_tokens": secs[-1],
                      "device": torch.cuda.get_device_name(0)}))
