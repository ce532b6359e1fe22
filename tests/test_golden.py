"""Known-answer vectors of configuration 1 (tests/golden/config1_layer_step.npz, made by
tests/golden/make_golden.py from the CPU oracle): the oracle and the workload generator
must still reproduce them, and the GPU path must hit them."""
import os

import numpy as np
import pytest
import torch

from apt_serve_b200.workloads import make_config_workload
from oracle import hybrid_cache_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "config1_layer_step.npz")


def load():
    return np.load(GOLDEN)


def magnitude_sum(t: torch.Tensor) -> float:
    return t.double().abs().sum().item()


def test_workload_generator_reproduces_the_golden_batch():
    g = load()
    w = make_config_workload(1, kv_from_projection=True)
    assert np.array_equal(g["seq_lens"], np.asarray(w.seq_lens, dtype=np.int32))
    assert np.array_equal(g["use_hidden"], np.asarray(w.use_hidden))
    assert np.array_equal(g["private_block_tables"], w.meta.private_block_tables.numpy())
    assert np.array_equal(g["slot_mapping_head"], w.meta.slot_mapping[:64].numpy())
    assert np.isclose(float(g["cache_sum_before"]), magnitude_sum(w.kv_cache), rtol=1e-6)


def test_oracle_reproduces_the_golden_output():
    g = load()
    w = make_config_workload(1, kv_from_projection=True)
    cache = w.kv_cache.clone()
    out = O.decode_layer_step(w.hidden_states, w.query, w.new_key, w.new_value, cache, cache,
                              *w.kv_weights(), w.meta, w.scale)
    assert np.allclose(out.numpy(), g["attention_output"], atol=1e-5, rtol=1e-5)
    assert np.isclose(float(g["cache_sum_after"]), magnitude_sum(cache), rtol=1e-6)


@pytest.mark.gpu
def test_gpu_layer_step_hits_the_golden_output():
    from apt_serve_b200 import attention as A, mixed_cache_ops, ops
    g = load()
    w = make_config_workload(1, kv_from_projection=True).to("cuda")
    m, h, d = w.meta, w.heads, w.shape.head_dim
    rows = m.kv_request_rows
    ops.reshape_and_cache_flash(w.new_key[rows].view(-1, h, d), w.new_value[rows].view(-1, h, d),
                                w.kv_cache[0], w.kv_cache[1], m.slot_mapping[m.kv_cache_use_tot])
    mixed_cache_ops.hidden_to_cache(w.hidden_states, w.hidden_cache, m.slot_mapping,
                                    m.hidden_cache_use_input, m.hidden_cache_store_tot)
    wk, bk, wv, bv = w.kv_weights()
    out = A.hybrid_decode_attention(w.query, w.kv_cache, w.hidden_cache, wk, bk, wv, bv,
                                    m.private_block_tables, m.seq_lens_tensor, m.cache_type, w.scale)
    torch.cuda.synchronize()
    assert np.allclose(out.cpu().numpy(), g["attention_output"], atol=1e-3, rtol=1e-3)
    assert np.isclose(float(g["cache_sum_after"]), magnitude_sum(w.kv_cache.cpu()), rtol=1e-6)
    # bit for bit against the oracle's cache writes on this machine's copy of the workload
    wc = make_config_workload(1, kv_from_projection=True)
    cache = wc.kv_cache.clone()
    O.decode_layer_step(wc.hidden_states, wc.query, wc.new_key, wc.new_value, cache, cache,
                        *wc.kv_weights(), wc.meta, wc.scale)
    assert torch.equal(w.kv_cache.cpu(), cache)
    new_slots = m.slot_mapping[m.hidden_holder_upd][m.cache_type != 0]
    written = O.flat_rows(w.kv_cache.cpu())[new_slots.cpu()][:, :8].numpy()
    assert np.array_equal(written, g["written_rows"])
