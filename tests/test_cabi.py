"""The C-ABI library: loads, exports every declared symbol, validates arguments
without touching a GPU."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

from apt_serve_b200 import _native as N

HEADER = Path(__file__).resolve().parents[1] / "include" / "aptserve_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(aps_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = N.lib()
    names = declared_symbols()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(names) == set(N.PROTOTYPES), "ctypes prototypes out of step with the header"


def test_version_and_workspace_size():
    lib = N.lib()
    assert b"sm_100a" in lib.aps_version()
    small = lib.aps_attention_workspace_bytes(8, 32, 16, 12, 64)
    big = lib.aps_attention_workspace_bytes(256, 128, 16, 40, 128)
    assert 0 < small < big
    # partial accumulators dominate: batch * chunks * heads * (D + 2) floats
    assert big >= 256 * 16 * 40 * 130 * 4
    assert lib.aps_attention_workspace_bytes(0, 32, 16, 12, 64) == 0


def test_argument_validation_returns_status_codes():
    lib = N.lib()
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) // 16 * 16
    # null pointer
    assert lib.aps_hidden_to_cache(0, p, p, p, p, 1, 8, 8, 8, 1, 0) == N.APS_ERR_NULL_POINTER
    assert b"null" in lib.aps_last_error()
    # unknown dtype
    assert lib.aps_hidden_to_cache(p, p, p, p, p, 1, 8, 8, 8, 7, 0) == N.APS_ERR_DTYPE
    # row stride shorter than a row
    assert lib.aps_cache_to_hidden(p, p, p, p, 1, 8, 4, 8, 1, 0) == N.APS_ERR_SHAPE
    # empty launches succeed without touching the device
    assert lib.aps_reshape_and_cache(0, 0, 0, 0, 0, 0, 2, 8, 16, 16, 16, 256, 1, 0) == N.APS_OK
    assert lib.aps_copy_blocks(0, 0, 0, 0, 0, 64, 0) == N.APS_OK
    # unsupported head size / block size
    st = lib.aps_paged_decode_attention(p16, p16, p16, p16, p16, p16, 1, 4, 2, 96, 16, 192, 192,
                                        16 * 192, 1.0, p16, 4096, 1, 0)
    assert st == N.APS_ERR_UNSUPPORTED
    st = lib.aps_paged_decode_attention(p16, p16, p16, p16, p16, p16, 1, 4, 2, 64, 8, 128, 128,
                                        8 * 128, 1.0, p16, 4096, 1, 0)
    assert st == N.APS_ERR_UNSUPPORTED
    # workspace too small
    st = lib.aps_paged_decode_attention(p16, p16, p16, p16, p16, p16, 4, 4, 2, 64, 16, 128, 128,
                                        16 * 128, 1.0, (p + 255) // 256 * 256, 16, 1, 0)
    assert st == N.APS_ERR_WORKSPACE
    # misaligned query
    st = lib.aps_paged_decode_attention(p16, p16 + 2, p16, p16, p16, p16, 4, 4, 2, 64, 16, 128, 128,
                                        16 * 128, 1.0, (p + 255) // 256 * 256, 1 << 30, 1, 0)
    assert st == N.APS_ERR_MISALIGNED
    # a head size no re-projection kernel takes is refused with a clear code
    ws = (p + 255) // 256 * 256
    st = lib.aps_hybrid_decode_attention(p16, p16, p16, p16, p16, p16, 0, p16, 0, p16, p16, p16,
                                         1, 1, 2, 96, 192, 16, 192, 192, 16 * 192, 192, 64, 192,
                                         1.0, ws, 1 << 30, 1, 0)
    assert st == N.APS_ERR_UNSUPPORTED


def test_swap_blocks_argument_checks():
    lib = N.lib()
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    pairs = (ctypes.c_int64 * 4)(0, 1, 5, 0)
    n = ctypes.c_int64(-1)
    # nothing to do: no copy, no device needed
    assert lib.aps_swap_blocks(p, p, ctypes.addressof(pairs), 0, 256, 256, 256, 4, 4, 1, ctypes.addressof(n), 0) == N.APS_OK
    assert n.value == 0
    # a block id outside the source, an unknown direction, a stride shorter than a block
    assert lib.aps_swap_blocks(p, p, ctypes.addressof(pairs), 2, 256, 256, 256, 4, 4, 1, 0, 0) == N.APS_ERR_SHAPE
    assert lib.aps_swap_blocks(p, p, ctypes.addressof(pairs), 1, 256, 256, 256, 4, 4, 5, 0, 0) == N.APS_ERR_SHAPE
    assert lib.aps_swap_blocks(p, p, ctypes.addressof(pairs), 1, 256, 128, 256, 4, 4, 1, 0, 0) == N.APS_ERR_SHAPE
    assert lib.aps_swap_blocks(0, p, ctypes.addressof(pairs), 1, 256, 256, 256, 4, 4, 1, 0, 0) == N.APS_ERR_NULL_POINTER


def test_status_and_cycle_readers_check_their_pointers():
    lib = N.lib()
    host = ctypes.c_ulonglong(0)
    assert lib.aps_reprojection_cycles(0, ctypes.addressof(host), 0) == N.APS_ERR_NULL_POINTER
    assert lib.aps_attention_status(0, ctypes.addressof(host), 0) == N.APS_ERR_NULL_POINTER
    buf = (ctypes.c_char * 512)()
    assert lib.aps_reprojection_cycles(ctypes.addressof(buf), 0, 0) == N.APS_ERR_NULL_POINTER


def test_python_shims_refuse_cpu_tensors_and_map_errors():
    from apt_serve_b200 import mixed_cache_ops, ops
    z = torch.zeros(2, 8)
    i = torch.zeros(1, dtype=torch.long)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        mixed_cache_ops.cache_to_hidden(z, torch.zeros(2, 2, 16, 1, 8), i, i)
    with pytest.raises(ValueError):
        ops.reshape_and_cache_flash(z, z, z, z, i, "fp8")
    with pytest.raises(ValueError):
        N.check(N.APS_ERR_UNSUPPORTED)
    with pytest.raises(RuntimeError):
        N.check(N.APS_ERR_SHAPE)


def test_backend_static_api():
    from apt_serve_b200.attention import FlashAttentionBackend, FlashAttentionImpl
    assert FlashAttentionBackend.get_kv_cache_shape(10, 16, 4, 128) == (2, 10, 16, 4, 128)
    with pytest.raises(ValueError):
        FlashAttentionBackend.get_kv_cache_shape(10, 8, 4, 128)
    assert FlashAttentionBackend.get_impl_cls() is FlashAttentionImpl
    with pytest.raises(ValueError):
        FlashAttentionImpl(4, 100, 0.1, 4, None, None, "auto")
    with pytest.raises(ValueError):
        FlashAttentionImpl(4, 128, 0.1, 4, None, 1024, "auto")


def test_advertised_head_sizes_are_the_ones_the_kernels_take():
    """Every head size the backend advertises passes the decode attention's argument check for
    fp16, and the sizes of the reference's list that the kernels do not take are refused."""
    from apt_serve_b200.attention import FlashAttentionBackend
    lib = N.lib()
    buf = (ctypes.c_char * 8192)()
    p = (ctypes.addressof(buf) + 255) // 256 * 256
    sizes = FlashAttentionBackend.get_supported_head_sizes()
    assert sizes == [32, 64, 128, 256]
    for d in (32, 64, 96, 128, 160, 192, 224, 256):
        # batch 1 with a far too small workspace: a supported size gets as far as the workspace check
        st = lib.aps_paged_decode_attention(p, p, p, p, p, p, 1, 4, 2, d, 16, 2 * d, 2 * d, 32 * d, 1.0,
                                            p, 16, 1, 0)
        assert st == (N.APS_ERR_WORKSPACE if d in sizes else N.APS_ERR_UNSUPPORTED), d


def test_absorbed_variant_falls_back_for_shapes_it_is_not_built_for():
    from apt_serve_b200.attention import absorbed_supported
    from apt_serve_b200.layers import OPTAttention
    assert absorbed_supported(40, 5120, torch.float16)          # OPT-13B
    assert absorbed_supported(72, 9216, torch.bfloat16)         # OPT-66B, padded to 80 heads
    assert absorbed_supported(9, 9216, torch.bfloat16)          # OPT-66B at tp = 8
    assert not absorbed_supported(56, 7168, torch.float16)      # OPT-30B: 56 heads pad to 64
    assert not absorbed_supported(12, 768, torch.float32)       # fp32
    assert not absorbed_supported(12, 768, torch.float16)       # hidden size not a multiple of 512
    e, h = 7168, 56
    z = torch.zeros
    layer = OPTAttention(e, h, z(3 * e, 8), None, z(8, e), None, fused="absorbed")
    assert not layer.use_absorbed(torch.float16)
    layer = OPTAttention(5120, 40, z(3 * 5120, 8), None, z(8, 5120), None, fused="absorbed")
    assert layer.use_absorbed(torch.float16) and not layer.use_absorbed(torch.float32)
    assert not OPTAttention(5120, 40, z(3 * 5120, 8), None, z(8, 5120), None, fused=True).use_absorbed(torch.float16)


def test_decode_layer_step_argument_checks():
    lib = N.lib()
    buf = (ctypes.c_char * 8192)()
    p = (ctypes.addressof(buf) + 255) // 256 * 256
    args = dict(batch=1, max_blocks=4, heads=2, d=128, e=256, bs=16)

    def call(cache_type=p, new_key=p, new_value=p, key_cache=p, value_cache=p, hs_stride=256):
        return lib.aps_decode_layer_step(p, p, p, new_key, new_value, key_cache, value_cache, p, p, 0, p, 0,
                                         p, p, cache_type, 1, 4, 2, 128, 256, 16, 256, 256, hs_stride, 256, 256,
                                         16 * 256, 256, 64, 256, 1.0, p, 16, 1, 0)
    assert call() == N.APS_ERR_WORKSPACE               # everything else is in order
    assert call(cache_type=0) == N.APS_ERR_WORKSPACE   # (the workspace check comes first)
    big = 1 << 30

    def call_ws(**kw):
        a = dict(cache_type=p, new_key=p, new_value=p, key_cache=p, value_cache=p, hs_stride=256)
        a.update(kw)
        return lib.aps_decode_layer_step(p, p, p, a["new_key"], a["new_value"], a["key_cache"], a["value_cache"],
                                         p, p, 0, p, 0, p, p, a["cache_type"], 1, 4, 2, 128, 256, 16, 256, 256,
                                         a["hs_stride"], 256, 256, 16 * 256, 256, 64, 256, 1.0, p, big, 1, 0)
    assert call_ws(cache_type=0) == N.APS_ERR_NULL_POINTER
    assert call_ws(value_cache=0) == N.APS_ERR_NULL_POINTER      # one cache plane without the other
    assert call_ws(hs_stride=8) == N.APS_ERR_SHAPE
