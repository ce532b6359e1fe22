"""The reference's own CUDA extension (built unmodified by oracle/build_ref.py)
against the CPU oracle and against this package's kernels: the pin for the three
``mixed_cache_ops``.  The reference build dispatches fp32 / fp64 / fp16 only and
its hidden-token index is only right while n_hidden <= 2 * n_kv, so the cases stay
inside that envelope."""
import pytest
import torch

from oracle import build_ref, hybrid_cache_oracle as O
from apt_serve_b200 import mixed_cache_ops

from helpers import small_workload

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_ext():
    if not build_ref.module_path().exists():
        pytest.skip("reference extension not prebuilt (python -m oracle.build_ref)")
    return build_ref.load()


def bits(t):
    return t.detach().cpu().contiguous().view(torch.uint8)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_three_ops_agree_with_reference_build(ref_ext, dtype):
    w = small_workload(dtype=dtype, heads=2, head_dim=64, lens=(3, 40, 17, 4, 64, 9),
                       hidden=(True, False, False, True, False, False), with_shared_cache=True)
    m = w.meta
    assert m.slot_mapping_shared.numel() <= 2 * m.kv_cache_use_tot.numel()
    g = torch.Generator().manual_seed(1)
    key = torch.randn(m.num_tot_tokens, 2, 64, generator=g).to(dtype)
    value = torch.randn(m.num_tot_tokens, 2, 64, generator=g).to(dtype)
    holder = torch.randn(m.num_tot_tokens, w.shape.hidden, generator=g).to(dtype)

    # CPU oracle
    kv_o, sh_o, holder_o = w.kv_cache.clone(), w.shared_cache.clone(), holder.clone()
    O.hidden_to_cache(w.hidden_states, kv_o, m.slot_mapping, m.hidden_cache_use_input,
                      m.hidden_cache_store_tot)
    O.cache_to_hidden(holder_o, kv_o, m.slot_mapping, m.hidden_cache_use_tot)
    O.mixed_kv_to_cache(key, value, kv_o[0], kv_o[1], sh_o[0], sh_o[1], m.slot_mapping,
                        m.slot_mapping_shared, m.kv_cache_use_tot, m.hidden_cache_use_tot)

    def run(mod):
        d = w.to("cuda")
        dm = d.meta
        hold = holder.cuda()
        mod.hidden_to_cache(d.hidden_states, d.kv_cache, dm.slot_mapping,
                            dm.hidden_cache_use_input, dm.hidden_cache_store_tot)
        torch.cuda.synchronize()
        mod.cache_to_hidden(hold, d.kv_cache, dm.slot_mapping, dm.hidden_cache_use_tot)
        torch.cuda.synchronize()
        mod.mixed_kv_to_cache(key.cuda(), value.cuda(), d.kv_cache[0], d.kv_cache[1],
                              d.shared_cache[0], d.shared_cache[1], dm.slot_mapping,
                              dm.slot_mapping_shared, dm.kv_cache_use_tot, dm.hidden_cache_use_tot)
        torch.cuda.synchronize()
        return d.kv_cache, d.shared_cache, hold

    kv_r, sh_r, hold_r = run(ref_ext)
    kv_n, sh_n, hold_n = run(mixed_cache_ops)
    for name, a, b, c in (("kv_cache", kv_r, kv_n, kv_o), ("shared_cache", sh_r, sh_n, sh_o),
                          ("hidden_holder", hold_r, hold_n, holder_o)):
        assert torch.equal(bits(a), bits(c)), f"{name}: reference build != oracle"
        assert torch.equal(bits(b), bits(c)), f"{name}: this package != oracle"
