"""B200-native hybrid-cache data path with Apt-Serve's operator interface.

Modules
  mixed_cache_ops  the reference's three-op torch extension (same names / arguments)
  ops              reshape_and_cache_flash, copy_blocks, swap_blocks (vLLM 0.5.0 signatures)
  attention        FlashAttentionBackend / Metadata / Impl, Attention, fused hybrid decode
  layers           OPTAttention, QKVParallelLinear (q_only / kv_only), RowParallelLinear
  metadata         index tensors as the reference's model runner builds them
  workloads        seeded synthetic configurations

Everything that touches data runs in ``lib/libaptserve_b200.so`` (CUDA, sm_100a);
there is no CPU or PyTorch fallback.
"""
from . import _native, attention, layers, metadata, mixed_cache_ops, ops, workloads  # noqa: F401

__all__ = ["attention", "layers", "metadata", "mixed_cache_ops", "ops", "workloads"]
__version__ = "0.1"
