"""The library's own tensor-parallel communicator (``aps_tp_*``): one NCCL communicator
per process, created through the C ABI, with the unique id handed from rank 0 to the
other ranks over whatever channel the host already has.

``layers.tensor_model_parallel_all_reduce`` uses it once ``install`` has been called
and falls back to ``torch.distributed`` otherwise -- both end in the same NCCL
all-reduce (aptserve_linear.py:827-829); the communicator here exists so that a host
that is not PyTorch can drive the exchange step through the same C ABI as the kernels.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Optional

import torch

from . import _native

UNIQUE_ID_BYTES = 128

_installed: Optional["TensorParallelComm"] = None


def new_unique_id() -> bytes:
    """Rank 0 calls this and ships the bytes to every other rank."""
    buf = ctypes.create_string_buffer(UNIQUE_ID_BYTES)
    _native.check(_native.lib().aps_tp_unique_id(ctypes.cast(buf, ctypes.c_void_p)))
    return buf.raw


class TensorParallelComm:
    """``TensorParallelComm(rank, world_size, unique_id)`` joins the communicator on the
    current CUDA device; every rank must call it with the same ``unique_id``."""

    def __init__(self, rank: int, world_size: int, unique_id: bytes):
        if len(unique_id) != UNIQUE_ID_BYTES:
            raise ValueError(f"a unique id has {UNIQUE_ID_BYTES} bytes")
        if not torch.cuda.is_available():
            raise RuntimeError("aptserve_b200: the communicator needs a CUDA device")
        self.rank, self.world_size = rank, world_size
        self.device = torch.device("cuda", torch.cuda.current_device())
        handle = ctypes.c_void_p()
        idbuf = ctypes.create_string_buffer(unique_id, UNIQUE_ID_BYTES)
        _native.check(_native.lib().aps_tp_init(ctypes.byref(handle), ctypes.cast(idbuf, ctypes.c_void_p),
                                                rank, world_size))
        self._handle = handle

    @classmethod
    def from_exchange(cls, rank: int, world_size: int,
                      broadcast_bytes: Callable[[Optional[bytes]], bytes]) -> "TensorParallelComm":
        """``broadcast_bytes(payload_or_None) -> payload``: the host's channel; rank 0
        passes the id, the others pass ``None`` and receive it."""
        uid = broadcast_bytes(new_unique_id() if rank == 0 else None)
        return cls(rank, world_size, uid)

    @classmethod
    def from_torch_distributed(cls, group=None) -> "TensorParallelComm":
        """Bootstrap over an initialised ``torch.distributed`` group (any backend)."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)

        def bcast(payload):
            box = [payload]
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0,
                                       group=group)
            return box[0]

        return cls.from_exchange(rank, world, bcast)

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """In-place sum over the ranks, on the current stream; returns ``x``."""
        if self._handle is None:
            raise RuntimeError("aptserve_b200: the communicator has been destroyed")
        _native.require_cuda(x)
        if not x.is_contiguous():
            raise ValueError("aptserve_b200: all_reduce needs a contiguous tensor")
        _native.check(_native.lib().aps_tp_allreduce(self._handle, _native.ptr(x), x.numel(),
                                                     _native.dtype_enum(x),
                                                     _native.current_stream(x.device)))
        return x

    def size(self) -> int:
        n = ctypes.c_int(0)
        _native.check(_native.lib().aps_tp_world_size(self._handle, ctypes.byref(n)))
        return n.value

    def destroy(self) -> None:
        global _installed
        if self._handle is not None:
            torch.cuda.synchronize(self.device)
            _native.check(_native.lib().aps_tp_destroy(self._handle))
            self._handle = None
        if _installed is self:
            _installed = None


def install(comm: Optional[TensorParallelComm]) -> None:
    """Make ``comm`` the one ``layers.tensor_model_parallel_all_reduce`` uses
    (``None`` goes back to ``torch.distributed``)."""
    global _installed
    _installed = comm


def installed() -> Optional[TensorParallelComm]:
    return _installed
