"""Profit coefficient (aptserve_llm_engine.py:316-354): the host arithmetic against the
oracle's literal restatement, and the probe's plumbing with an injected timer."""
import numpy as np
import pytest

from apt_serve_b200 import cost_model as C
from oracle import hybrid_cache_oracle as O


def test_block_counts_follow_the_reference_rounding():
    x = C.block_counts([1, 15, 16, 17, 101, 4001], 16)
    assert x.tolist() == [0, 1, 1, 1, 1, 6, 250]


@pytest.mark.parametrize("block_size", [16, 32])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_fit_matches_the_literal_regression(block_size, seed):
    rng = np.random.default_rng(seed)
    tokens = list(C.DEFAULT_TOKEN_COUNTS)
    secs = 3e-4 + 2.5e-6 * np.asarray(tokens) + rng.normal(0, 2e-5, len(tokens))
    ours = C.fit_profit_coefficient(tokens, secs, block_size)
    ref = O.profit_coefficient_literal(tokens, secs, block_size)
    assert np.isclose(ours, ref, rtol=1e-10, atol=0)


def test_exact_line_gives_slope_over_five():
    tokens = [16 * k for k in range(1, 40)]
    secs = [1e-3 * (t // 16) for t in tokens]          # exactly 1 ms per block, through the origin
    assert np.isclose(C.fit_profit_coefficient(tokens, secs, 16), 1e-3 / 5, rtol=1e-12)


def test_fit_rejects_degenerate_input():
    with pytest.raises(ValueError):
        C.fit_profit_coefficient([1, 2], [1.0], 16)
    with pytest.raises(ValueError):
        C.fit_profit_coefficient([5], [1.0], 16)


def test_probe_uses_the_injected_timer():
    calls = []

    def timer(n):
        calls.append(n)
        return 2e-6 * n

    coef, secs = C.probe_profit_coefficient(40, 128, 5120, 40, 16, timer=timer)
    assert calls == list(C.DEFAULT_TOKEN_COUNTS)
    assert np.isclose(coef, O.profit_coefficient_literal(C.DEFAULT_TOKEN_COUNTS, secs, 16), rtol=1e-10)


@pytest.mark.gpu
def test_probe_times_the_fused_path():
    import torch
    coef, secs = C.probe_profit_coefficient(12, 64, 768, 12, 16, dtype=torch.float16,
                                            token_counts=(1, 257, 513, 1025), repeats=2)
    assert secs.shape == (4,) and np.all(secs > 0)
    assert np.isfinite(coef)
    # four times the tokens cannot be cheaper than a single token
    assert secs[-1] >= secs[0] * 0.5
