"""Per-worker cache allocation and block moves, without the shared cache.

Mirror of the reference's ``CacheEngine`` (aptserve_cache_engine.py:15-119) for the
fused decode path.  The reference allocates, next to the per-layer ``[2, NB, BS, H, D]``
caches, ONE ``[2, 2*NB, BS, H, D]`` shared cache (aptserve_cache_engine.py:81-85) that
holds the re-projected K/V of hidden-cached requests between ``mixed_kv_to_cache`` and
the attention call.  The fused hybrid decode attention keeps those K/V on chip, so the
shared cache is only allocated on request (``with_shared_cache=True``, for callers that
still run the legacy three-op sequence) and its bytes go to cache blocks instead:
``num_blocks_for_budget`` does that arithmetic.

Hidden blocks live in the K/V planes of their layer (a physical block holds two hidden
blocks, ids ``p`` and ``p + NB``, aptserve_block_manager.py:535-540), which needs
``H * D == E``.  Under tensor parallelism a rank's planes are narrower than a hidden row,
so each layer gets a dedicated ``[2, NB, BS, 1, E]`` hidden cache with the same slot
numbering.  Block moves address PHYSICAL blocks, both planes at once, so a swap or a copy
of physical block ``p`` carries the hidden blocks ``p`` and ``p + NB`` with it;
``physical_block_map`` folds a map written in logical ids.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import ops


def physical_block_map(pairs: Sequence[Tuple[int, int]], num_src_blocks: int,
                       num_dst_blocks: int) -> List[Tuple[int, int]]:
    """Fold ``(src, dst)`` pairs that may name V-plane ids (``p + NB``) into unique
    pairs of physical ids, keeping first-seen order.  Raises if one physical source
    would go to two destinations or two sources to one destination (the two halves
    of a physical block move together)."""
    out: List[Tuple[int, int]] = []
    src_seen, dst_seen = {}, {}
    for s, d in pairs:
        s, d = int(s), int(d)
        if not (0 <= s < 2 * num_src_blocks and 0 <= d < 2 * num_dst_blocks):
            raise ValueError(f"block pair ({s}, {d}) is out of range")
        if (s >= num_src_blocks) != (d >= num_dst_blocks):
            raise ValueError(f"block pair ({s}, {d}) moves a K-plane half onto a V-plane half")
        ps, pd = s % num_src_blocks, d % num_dst_blocks
        if src_seen.get(ps, pd) != pd or dst_seen.get(pd, ps) != ps:
            raise ValueError(f"block pair ({s}, {d}) splits a physical block")
        if ps not in src_seen:
            out.append((ps, pd))
        src_seen[ps], dst_seen[pd] = pd, ps
    return out


class CacheEngine:
    """Allocates the GPU and CPU caches of one worker and moves blocks between them
    (aptserve_cache_engine.py:23-59: same attributes ``gpu_cache``, ``cpu_cache``,
    ``shared_cache``; same methods ``swap_in``, ``swap_out``, ``copy``)."""

    def __init__(self, num_layers: int, num_kv_heads: int, head_size: int, block_size: int,
                 num_gpu_blocks: int, num_cpu_blocks: int, dtype: torch.dtype,
                 device="cuda", hidden_size: Optional[int] = None,
                 with_shared_cache: bool = False, pin_memory: Optional[bool] = None):
        if block_size % 16 != 0:
            raise ValueError("Block size must be a multiple of 16.")   # aptserve_flash_attn.py:40-41
        self.num_layers, self.num_kv_heads, self.head_size = num_layers, num_kv_heads, head_size
        self.block_size, self.dtype = block_size, dtype
        self.num_gpu_blocks, self.num_cpu_blocks = num_gpu_blocks, num_cpu_blocks
        self.hidden_size = hidden_size if hidden_size is not None else num_kv_heads * head_size
        self.device = torch.device(device)
        if pin_memory is None:
            pin_memory = torch.cuda.is_available()
        self.gpu_cache = self._allocate(num_gpu_blocks, self.device, False)
        self.cpu_cache = self._allocate(num_cpu_blocks, torch.device("cpu"), pin_memory)
        # hidden rows of a layer: its K/V planes when they are as wide as a hidden row,
        # else a dedicated tensor with the same [2, NB, BS] slot numbering
        self.aliased_hidden = self.hidden_size == num_kv_heads * head_size
        if self.aliased_hidden:
            self.gpu_hidden_cache, self.cpu_hidden_cache = self.gpu_cache, self.cpu_cache
        else:
            self.gpu_hidden_cache = self._allocate(num_gpu_blocks, self.device, False, hidden=True)
            self.cpu_hidden_cache = self._allocate(num_cpu_blocks, torch.device("cpu"), pin_memory, hidden=True)
        self.shared_cache = None
        if with_shared_cache:
            self.shared_cache = torch.zeros(self.kv_cache_shape(2 * num_gpu_blocks), dtype=dtype,
                                            device=self.device)

    # ---- shapes and sizes ---------------------------------------------------------
    def kv_cache_shape(self, num_blocks: int) -> Tuple[int, ...]:
        """``(2, NB, BS, H, D)`` (aptserve_flash_attn.py:33-42)."""
        return (2, num_blocks, self.block_size, self.num_kv_heads, self.head_size)

    def _allocate(self, num_blocks, device, pin, hidden=False) -> List[torch.Tensor]:
        shape = ((2, num_blocks, self.block_size, 1, self.hidden_size) if hidden
                 else self.kv_cache_shape(num_blocks))
        # zero-filled like the reference's (aptserve_cache_engine.py:72-80): the null
        # block must read as zeros
        return [torch.zeros(shape, dtype=self.dtype, device=device,
                            pin_memory=bool(pin) and device.type == "cpu")
                for _ in range(self.num_layers)]

    @staticmethod
    def get_cache_block_size(num_layers: int, num_kv_heads: int, head_size: int, block_size: int,
                             dtype: torch.dtype, hidden_size: Optional[int] = None) -> int:
        """Bytes of one physical block over all layers (aptserve_cache_engine.py:101-119),
        plus the dedicated hidden rows when the planes cannot hold them."""
        es = torch.empty((), dtype=dtype).element_size()
        per_layer = 2 * block_size * num_kv_heads * head_size
        if hidden_size is not None and hidden_size != num_kv_heads * head_size:
            per_layer += 2 * block_size * hidden_size
        return es * num_layers * per_layer

    @staticmethod
    def num_blocks_for_budget(budget_bytes: int, num_layers: int, num_kv_heads: int, head_size: int,
                              block_size: int, dtype: torch.dtype, hidden_size: Optional[int] = None,
                              with_shared_cache: bool = False) -> int:
        """Physical blocks that fit into ``budget_bytes``.  With the shared cache every
        block also pays for two shared blocks of one layer's width
        (aptserve_cache_engine.py:81-85); without it that memory holds cache blocks."""
        es = torch.empty((), dtype=dtype).element_size()
        per_block = CacheEngine.get_cache_block_size(num_layers, num_kv_heads, head_size, block_size,
                                                     dtype, hidden_size)
        if with_shared_cache:
            per_block += es * 2 * (2 * block_size * num_kv_heads * head_size)
        return int(budget_bytes // per_block)

    # ---- block moves ----------------------------------------------------------------
    def _swap(self, src, dst, src_hidden, dst_hidden, src_to_dst: torch.Tensor) -> None:
        for i in range(self.num_layers):
            for plane in (0, 1):                                   # K then V (aptserve_flash_attn.py:50-56)
                ops.swap_blocks(src[i][plane], dst[i][plane], src_to_dst)
                if not self.aliased_hidden:
                    ops.swap_blocks(src_hidden[i][plane], dst_hidden[i][plane], src_to_dst)

    def swap_in(self, src_to_dst: torch.Tensor) -> None:
        """CPU -> GPU, physical block ids (aptserve_cache_engine.py:88-91)."""
        self._swap(self.cpu_cache, self.gpu_cache, self.cpu_hidden_cache, self.gpu_hidden_cache, src_to_dst)

    def swap_out(self, src_to_dst: torch.Tensor) -> None:
        """GPU -> CPU, physical block ids (aptserve_cache_engine.py:93-96)."""
        self._swap(self.gpu_cache, self.cpu_cache, self.gpu_hidden_cache, self.cpu_hidden_cache, src_to_dst)

    def copy(self, src_to_dsts: torch.Tensor) -> None:
        """Copy-on-write block copies in every layer (aptserve_cache_engine.py:98-99)."""
        ops.copy_blocks([c[0] for c in self.gpu_cache], [c[1] for c in self.gpu_cache], src_to_dsts)
        if not self.aliased_hidden:
            ops.copy_blocks([c[0] for c in self.gpu_hidden_cache], [c[1] for c in self.gpu_hidden_cache],
                            src_to_dsts)
