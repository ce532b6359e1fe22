"""Parity of the decode attention kernels against the reference's REAL op chain on the
GPU: the reference's own ``mixed_cache.cu`` (compiled unmodified into ``oracle/_ref``),
``torch.nn.functional.linear`` for the ``kv_only`` projection, vLLM's
``reshape_and_cache_flash`` / ``copy_blocks`` and vLLM's flash-attention paged decode --
the kernels aptserve_opt.py:106-124 and aptserve_flash_attn.py:356-387, 452-473 call.

This is the pin of the oracle for the attention / re-projection rows: the same inputs go
through (a) that chain, (b) the CPU oracle, (c) this package's kernels.

Tolerances, stated once:
  kernel vs chain        |x - ref| <= 2e-2 + 2e-2 * |ref|      (the path's stated bound)
  oracle vs chain        |x - ref| <= 4e-3 + 4e-3 * |ref|      (fp32 oracle with K/V rounded
                                                               to fp16 like the chain's GEMM output,
                                                               against fp16 tensor-core arithmetic)
  cache contents         bit-exact where only copies are involved
"""
import numpy as np
import pytest
import torch

from oracle import hybrid_cache_oracle as O
from oracle.literal_chain_gpu import LiteralChain
from apt_serve_b200 import attention as A
from apt_serve_b200 import ops
from apt_serve_b200.workloads import LayerShape, OPT_13B, make_decode_workload

from helpers import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def chain():
    c, why = LiteralChain.create()
    if c is None:
        pytest.skip(why)
    return c


def kv_weight_rows(w):
    hd = w.heads * w.shape.head_dim
    return w.qkv_weight[hd:], w.qkv_bias[hd:]


def run_chain(chain, w):
    """The reference's chain on a device workload (mutates its caches); attention output."""
    w_kv, b_kv = kv_weight_rows(w)
    return chain.hybrid_decode_layer(w.hidden_states, w.query, w_kv, b_kv, w.kv_cache, w.shared_cache,
                                     w.meta, w.scale)


def run_ours(w):
    """This package's fused layer-step on a device workload (mutates its caches)."""
    wk, bk, wv, bv = w.kv_weights()
    out = A.decode_layer_step(w.query, w.hidden_states, w.new_key, w.new_value, w.kv_cache, w.hidden_cache,
                              wk, bk, wv, bv, w.meta.private_block_tables, w.meta.seq_lens_tensor,
                              w.meta.cache_type, w.scale)
    A.raise_on_device_status()
    return out


def block_size_for(chain, want=16):
    return want if want % chain.block_granularity == 0 else chain.block_granularity


def test_kv_only_batch_against_third_party_paged_attention(chain):
    """aptserve_flash_attn.py:452-461: a K/V-only decode batch over the private cache."""
    # one (dtype, head size) only: the third-party kernel is compiled for this GPU at its first
    # call per instantiation, which takes about a minute each; the other dtypes and head sizes
    # of the K/V path are checked against the CPU oracle in test_gpu_attention.py
    bs = block_size_for(chain)
    for dtype, heads, d in ((torch.float16, 4, 128),):
        shape = LayerShape("t", heads, d, heads * d, dtype, block_size=bs)
        lens = [1, 15, 16, 17, 127, 128, 129, 300, 1000, 2048]
        w = make_decode_workload(shape, lens, [False] * len(lens), seed=5, device="cuda")
        ref = chain.decode_attention(w.query, w.kv_cache[0], w.kv_cache[1], w.meta.block_tables,
                                     w.meta.seq_lens_tensor, w.scale)
        out = A.paged_decode_attention(w.query, w.kv_cache[0], w.kv_cache[1], w.meta.block_tables,
                                       w.meta.seq_lens_tensor, w.scale)
        assert_close(out, ref, f"paged decode vs {chain.attention_name} ({dtype}, {heads}x{d})")
        cpu = w.cpu()
        orc = O.paged_decode_attention(cpu.query, cpu.kv_cache[0], cpu.kv_cache[1], cpu.meta.block_tables,
                                       cpu.meta.seq_lens_tensor, cpu.scale)
        tol = 4e-3 if dtype == torch.float16 else 1.6e-2   # bf16 output rounding: 2^-8 relative
        assert_close(orc, ref, f"oracle vs {chain.attention_name} ({dtype})", tol, tol)


def test_mixed_batch_inside_the_reference_envelope(chain):
    """A hybrid batch whose hidden tokens number at most twice its K/V requests, where the
    reference's mixed_kv_to_cache index is the intended one: hidden requests' rows of the
    chain's output against this package's fused step and against the oracle."""
    bs = block_size_for(chain)
    shape = LayerShape("t", 4, 128, 512, torch.float16, block_size=bs)
    lens = [30, 17, 33] + [int(x) for x in np.random.default_rng(1).integers(1, 400, size=40)]
    hid = [True] * 3 + [False] * 40
    w = make_decode_workload(shape, lens, hid, seed=21, device="cuda", with_shared_cache=True,
                             kv_from_projection=True)
    assert chain.inside_mixed_envelope(w.meta)
    cpu = w.cpu()
    ours = run_ours(cpu.to("cuda"))        # on a copy: both runs start from the same caches
    ref = run_chain(chain, w)
    rows = [0, 1, 2]
    assert_close(ours[rows], ref[rows], "fused step vs the reference chain, hidden requests")
    # the oracle over the same query, with the new hidden rows written and K/V rounded to
    # fp16 as the chain's GEMM output is
    wk, bk, wv, bv = cpu.kv_weights()
    O.hidden_to_cache(cpu.hidden_states, cpu.kv_cache, cpu.meta.slot_mapping, cpu.meta.hidden_cache_use_input,
                      cpu.meta.hidden_cache_store_tot)
    orc = O.hybrid_decode_attention(cpu.query, cpu.kv_cache, cpu.kv_cache, wk, bk, wv, bv,
                                    cpu.meta.private_block_tables, cpu.meta.seq_lens_tensor,
                                    cpu.meta.cache_type, cpu.scale, torch.float16)
    assert_close(orc[rows], ref[rows], "oracle vs the reference chain, hidden requests", 4e-3, 4e-3)
    # the private cache after the chain: the new hidden rows are copies, bit-exact against the
    # oracle's cache; the K/V requests' new rows come from the GEMM
    hid_slots = cpu.meta.slot_mapping[cpu.meta.hidden_cache_store_tot]
    assert torch.equal(O.flat_rows(w.kv_cache.cpu())[hid_slots], O.flat_rows(cpu.kv_cache)[hid_slots])


@pytest.mark.parametrize("dtype,lens", [
    (torch.float16, (5, 129, 300, 16, 1, 700)),
    (torch.float16, (2048, 1536, 1900)),          # full-length requests (configuration 5's range)
])
def test_all_hidden_batch_any_length(chain, dtype, lens):
    """All requests hidden-cached: the reference scatters the projected K/V with
    reshape_and_cache_flash (aptserve_flash_attn.py:378-385), so no length limit applies."""
    bs = block_size_for(chain)
    shape = LayerShape("t", 4, 128, 512, dtype, block_size=bs)
    w = make_decode_workload(shape, list(lens), [True] * len(lens), seed=33, device="cuda",
                             with_shared_cache=True)
    cpu = w.cpu()
    ours = run_ours(cpu.to("cuda"))
    ref = run_chain(chain, w)
    assert_close(ours, ref, f"fused step vs the reference chain, all hidden {lens}")
    wk, bk, wv, bv = cpu.kv_weights()
    O.hidden_to_cache(cpu.hidden_states, cpu.kv_cache, cpu.meta.slot_mapping, cpu.meta.hidden_cache_use_input,
                      cpu.meta.hidden_cache_store_tot)
    orc = O.hybrid_decode_attention(cpu.query, cpu.kv_cache, cpu.kv_cache, wk, bk, wv, bv,
                                    cpu.meta.private_block_tables, cpu.meta.seq_lens_tensor,
                                    cpu.meta.cache_type, cpu.scale, dtype)
    assert_close(orc, ref, f"oracle vs the reference chain, all hidden {lens}", 4e-3, 4e-3)


def test_opt13b_shapes_all_hidden_against_the_chain(chain):
    """OPT-13B layer shapes (40 heads x 128, E = 5120): four hidden-cached requests of
    configuration 2's length range through the reference chain and the fused step."""
    bs = block_size_for(chain)
    shape = LayerShape(OPT_13B.name, OPT_13B.num_heads, OPT_13B.head_dim, OPT_13B.hidden, OPT_13B.dtype, bs)
    lens = [2048, 700, 131, 16]
    w = make_decode_workload(shape, lens, [True] * 4, seed=1002, device="cuda", with_shared_cache=True)
    w2 = make_decode_workload(shape, lens, [True] * 4, seed=1002, device="cuda")
    ours = run_ours(w2)
    ref = run_chain(chain, w)
    assert_close(ours, ref, "OPT-13B shapes vs the reference chain")


def test_cache_write_ops_against_vllm_ops(chain):
    """reshape_and_cache_flash and copy_blocks bit for bit against vLLM's own ops (the
    third-party ops behind aptserve_flash_attn.py:63-65, 338-345)."""
    from vllm import _custom_ops as vops
    g = torch.Generator(device="cuda").manual_seed(3)
    for dtype, heads, d, bs in ((torch.float16, 40, 128, 16), (torch.bfloat16, 9, 128, 16),
                                (torch.float16, 3, 64, 32), (torch.float32, 12, 64, 16)):
        nb, t = 64, 300
        key = torch.randn(t, heads, d, device="cuda", generator=g).to(dtype)
        value = torch.randn(t, heads, d, device="cuda", generator=g).to(dtype)
        slots = torch.randperm(nb * bs, device="cuda", generator=g)[:t].to(torch.int64)
        slots[::7] = -1
        a = torch.zeros(2, nb, bs, heads, d, device="cuda", dtype=dtype)
        b = torch.zeros_like(a)
        chain.reshape_and_cache(key, value, a[0], a[1], slots)
        ops.reshape_and_cache_flash(key, value, b[0], b[1], slots, "auto")
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), f"reshape_and_cache_flash {dtype}"
        assert a.abs().sum() > 0
        # copy-on-write pairs over two "layers"
        layers_a = [a.clone(), a.clone().mul_(2)]
        layers_b = [x.clone() for x in layers_a]
        pairs = torch.tensor([[1, 40], [5, 41], [5, 42], [63, 0]], dtype=torch.int64, device="cuda")
        if hasattr(vops, "copy_blocks"):
            vops.copy_blocks([x[0] for x in layers_a], [x[1] for x in layers_a], pairs)
        else:
            # this vLLM build no longer exports the op: the same copies as plain tensor assignments
            for x in layers_a:
                for src, dst in pairs.tolist():
                    x[:, dst] = x[:, src]
        ops.copy_blocks([x[0] for x in layers_b], [x[1] for x in layers_b], pairs)
        for x, y in zip(layers_a, layers_b):
            assert torch.equal(x.view(torch.uint8), y.view(torch.uint8)), f"copy_blocks {dtype}"
