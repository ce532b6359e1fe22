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
