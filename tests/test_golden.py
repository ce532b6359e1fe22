"""Known-answer vectors.

tests/golden/config1_layer_step.npz (made by tests/golden/make_golden.py from the CPU oracle,
configuration 1): the oracle and the workload generator must still reproduce them, and the
GPU path must hit them.

tests/golden/reference_chain_decode.npz (made by tests/golden/make_reference_chain_golden.py
on a B200 from the REFERENCE's own op chain: its mixed_cache.cu unmodified, cuBLAS, vLLM's
cache write and flash-attention paged decode): the CPU oracle must agree with what the
reference computed, and so must this package's kernels."""
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


# --------------------------------------------------------------------------- #
# outputs of the reference's own op chain, recorded on a B200
# --------------------------------------------------------------------------- #
CHAIN_GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_chain_decode.npz")


def _chain_cases():
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "make_reference_chain_golden",
        os.path.join(os.path.dirname(CHAIN_GOLDEN), "make_reference_chain_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _fp16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.float16).copy())


def _close(x: torch.Tensor, ref: torch.Tensor, tol: float, what: str):
    err = (x.float() - ref.float()).abs()
    bound = tol + tol * ref.float().abs()
    assert bool((err <= bound).all()), f"{what}: max abs err {err.max().item():.3e}"


@pytest.mark.parametrize("case", ["all_hidden", "mixed", "kv_only"])
def test_oracle_matches_the_recorded_reference_chain(case):
    """The CPU oracle against what the reference's own kernels produced for the same seeded
    inputs (mixed_cache.cu unmodified + cuBLAS + vLLM's cache write and flash-attention paged
    decode, recorded by tests/golden/make_reference_chain_golden.py on a B200).  Tolerance:
    |x - ref| <= 4e-3 + 4e-3 |ref| (fp32 oracle with K/V rounded to fp16 like the GEMM's
    output, against fp16 tensor-core arithmetic); rows that are plain copies are bit-exact."""
    g = np.load(CHAIN_GOLDEN)
    w = _chain_cases().build_case(case)
    assert np.array_equal(g[case + "/seq_lens"], np.asarray(w.seq_lens, dtype=np.int32))
    ref = _fp16(g[case + "/out"])
    if case == "kv_only":
        out = O.paged_decode_attention(w.query, w.kv_cache[0], w.kv_cache[1], w.meta.block_tables,
                                       w.meta.seq_lens_tensor, w.scale)
        _close(out, ref, 4e-3, "oracle vs recorded paged decode")
        return
    m = w.meta
    O.hidden_to_cache(w.hidden_states, w.kv_cache, m.slot_mapping, m.hidden_cache_use_input,
                      m.hidden_cache_store_tot)
    slots = m.slot_mapping[m.hidden_cache_store_tot]
    assert torch.equal(O.flat_rows(w.kv_cache)[slots].view(torch.int16),
                       torch.from_numpy(g[case + "/new_hidden_rows"].view(np.int16).copy()))
    wk, bk, wv, bv = w.kv_weights()
    out = O.hybrid_decode_attention(w.query, w.kv_cache, w.kv_cache, wk, bk, wv, bv,
                                    m.private_block_tables, m.seq_lens_tensor, m.cache_type, w.scale,
                                    torch.float16)
    rows = [r for r, h in enumerate(w.use_hidden) if h]    # the chain's rows of hidden requests
    _close(out[rows], ref[rows], 4e-3, f"oracle vs recorded chain ({case})")


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["all_hidden", "mixed", "kv_only"])
def test_gpu_kernels_match_the_recorded_reference_chain(case):
    """This package's kernels against the recorded outputs of the reference's chain (needs
    none of the third-party kernels on the box).  |x - ref| <= 2e-2 + 2e-2 |ref|."""
    from apt_serve_b200 import attention as A
    g = np.load(CHAIN_GOLDEN)
    w = _chain_cases().build_case(case).to("cuda")
    ref = _fp16(g[case + "/out"])
    if case == "kv_only":
        out = A.paged_decode_attention(w.query, w.kv_cache[0], w.kv_cache[1], w.meta.block_tables,
                                       w.meta.seq_lens_tensor, w.scale)
        _close(out.cpu(), ref, 2e-2, "paged decode vs recorded chain")
        return
    wk, bk, wv, bv = w.kv_weights()
    out = A.decode_layer_step(w.query, w.hidden_states, w.new_key, w.new_value, w.kv_cache, w.hidden_cache,
                              wk, bk, wv, bv, w.meta.private_block_tables, w.meta.seq_lens_tensor,
                              w.meta.cache_type, w.scale)
    A.raise_on_device_status()
    m = w.meta
    slots = m.slot_mapping[m.hidden_cache_store_tot]
    assert torch.equal(O.flat_rows(w.kv_cache)[slots].cpu().view(torch.int16),
                       torch.from_numpy(g[case + "/new_hidden_rows"].view(np.int16).copy()))
    rows = [r for r, h in enumerate(w.use_hidden) if h]
    _close(out.cpu()[rows], ref[rows], 2e-2, f"fused layer-step vs recorded chain ({case})")


@pytest.mark.parametrize("case", ["ops_inside", "ops_outside"])
def test_oracle_cache_ops_match_the_recorded_reference_build(case):
    """hidden_to_cache, cache_to_hidden and mixed_kv_to_cache of the oracle against what the
    reference's own extension (mixed_cache.cu compiled unmodified) wrote for the same seeded
    inputs, bit for bit.  "ops_outside" has more hidden tokens than twice the K/V requests:
    there the reference re-reads the first 2 * n_kv hidden tokens (mixed_cache.cu:88), which the
    oracle restates with literal_index=True."""
    g = np.load(CHAIN_GOLDEN)
    w, key, value, holder = _chain_cases().build_ops_case(case)
    m = w.meta
    inside = m.slot_mapping_shared.numel() <= 2 * m.kv_cache_use_tot.numel()
    assert inside == (case == "ops_inside")
    kv, shared = w.kv_cache, w.shared_cache
    O.hidden_to_cache(w.hidden_states, kv, m.slot_mapping, m.hidden_cache_use_input, m.hidden_cache_store_tot)
    O.cache_to_hidden(holder, kv, m.slot_mapping, m.hidden_cache_use_tot)
    O.mixed_kv_to_cache(key, value, kv[0], kv[1], shared[0], shared[1], m.slot_mapping,
                        m.slot_mapping_shared, m.kv_cache_use_tot, m.hidden_cache_use_tot,
                        literal_index=True)

    def same(t, name):
        return np.array_equal(t.contiguous().view(torch.int16).numpy().view(np.uint16), g[case + "/" + name])

    assert same(kv, "kv_cache"), "private cache differs from the reference build's"
    assert same(holder, "hidden_holder"), "gathered hidden rows differ from the reference build's"
    assert same(shared, "shared_cache"), "shared cache differs from the reference build's"
    if inside:
        # inside the envelope the literal index is the intended one
        w2, key2, value2, _ = _chain_cases().build_ops_case(case)
        m2 = w2.meta
        O.hidden_to_cache(w2.hidden_states, w2.kv_cache, m2.slot_mapping, m2.hidden_cache_use_input,
                          m2.hidden_cache_store_tot)
        O.mixed_kv_to_cache(key2, value2, w2.kv_cache[0], w2.kv_cache[1], w2.shared_cache[0], w2.shared_cache[1],
                            m2.slot_mapping, m2.slot_mapping_shared, m2.kv_cache_use_tot, m2.hidden_cache_use_tot)
        assert torch.equal(w2.shared_cache.view(torch.int16), shared.view(torch.int16))


def test_oracle_reshape_and_cache_flash_matches_the_recorded_vllm_op():
    """The oracle's paged K/V scatter against what vLLM's `_custom_ops.reshape_and_cache_flash`
    wrote (the third-party op behind aptserve_flash_attn.py:338-345): strided inputs, -1 slots."""
    g = np.load(CHAIN_GOLDEN)
    key, value, slots, cache = _chain_cases().build_cache_write_case()
    O.reshape_and_cache_flash(key, value, cache[0], cache[1], slots)
    assert np.array_equal(cache.view(torch.int16).numpy().view(np.uint16), g["reshape_and_cache_flash/cache"])


@pytest.mark.gpu
def test_gpu_reshape_and_cache_flash_matches_the_recorded_vllm_op():
    from apt_serve_b200 import ops
    g = np.load(CHAIN_GOLDEN)
    key, value, slots, cache = _chain_cases().build_cache_write_case()
    c = cache.cuda()
    ops.reshape_and_cache_flash(key.cuda(), value.cuda(), c[0], c[1], slots.cuda(), "auto")
    torch.cuda.synchronize()
    assert np.array_equal(c.cpu().view(torch.int16).numpy().view(np.uint16), g["reshape_and_cache_flash/cache"])
