"""Symmetric device buffers for a world of one-process-per-GPU ranks.

`World` is the host-side plumbing the fused operators need around them: every rank allocates
the same set of named buffers, the ranks exchange CUDA IPC handles through a
`torch.distributed` process group (NCCL or gloo: only python objects travel), and each rank
ends up with the device address of every peer's copy -- the `peer_*` pointer arrays of the
operator parameter records.  No collective runs on the data path.

With world_size == 1 (or `local=True`, used to emulate several ranks on one GPU) the buffers
are ordinary torch tensors and every "peer" address is local."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch

from . import _native as N


class _RawBuffer:
    """A cudaMalloc allocation presented to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2, "strides": None}


def exchange(objects, group=None):
    """All-gather of one python object per rank (thin wrapper, testable with gloo on CPU)."""
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [objects]
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, objects, group=group)
    return out


@dataclass
class SymmetricBuffer:
    name: str
    nbytes: int
    local: torch.Tensor                      # uint8 view of this rank's copy
    peer_ptrs: list = field(default_factory=list)  # device address of every rank's copy

    def view(self, dtype, *shape):
        return self.local.view(dtype).view(*shape) if shape else self.local.view(dtype)


class World:
    def __init__(self, rank: int = 0, world_size: int = 1, device: int = 0, group=None):
        self.rank, self.world_size, self.device, self.group = rank, world_size, device, group
        self.buffers: dict[str, SymmetricBuffer] = {}
        self._opened: list[int] = []
        self._owned: list[int] = []

    def allocate(self, specs: dict[str, int]) -> dict[str, SymmetricBuffer]:
        """specs: name -> bytes (same on every rank).  Collective over the group."""
        torch.cuda.set_device(self.device)
        if self.world_size == 1:
            for name, nbytes in specs.items():
                t = torch.zeros(nbytes, dtype=torch.uint8, device=f"cuda:{self.device}")
                self.buffers[name] = SymmetricBuffer(name, nbytes, t, [t.data_ptr()])
            return self.buffers
        lib = N.lib()
        handles = {}
        for name, nbytes in specs.items():
            ptr = C.c_void_p()
            handle = C.create_string_buffer(64)
            rc = lib.fuse_b200_symmetric_alloc(nbytes, C.byref(ptr), handle)
            if rc != 0:
                raise RuntimeError(f"symmetric_alloc({name}, {nbytes}) -> cudaError {rc}")
            self._owned.append(ptr.value)
            t = torch.as_tensor(_RawBuffer(ptr.value, nbytes), device=f"cuda:{self.device}")
            self.buffers[name] = SymmetricBuffer(name, nbytes, t, [0] * self.world_size)
            handles[name] = handle.raw
        gathered = exchange(handles, self.group)
        for name in specs:
            buf = self.buffers[name]
            for peer in range(self.world_size):
                if peer == self.rank:
                    buf.peer_ptrs[peer] = buf.local.data_ptr()
                    continue
                ptr = C.c_void_p()
                rc = lib.fuse_b200_symmetric_open(gathered[peer][name], C.byref(ptr))
                if rc != 0:
                    raise RuntimeError(f"symmetric_open({name}, peer {peer}) -> cudaError {rc}")
                self._opened.append(ptr.value)
                buf.peer_ptrs[peer] = ptr.value
        return self.buffers

    def close(self):
        torch.cuda.synchronize()
        lib = N.lib()
        for ptr in self._opened:
            lib.fuse_b200_symmetric_close(ptr)
        self._opened.clear()
        self.buffers.clear()
        for ptr in self._owned:
            lib.fuse_b200_symmetric_free(ptr)
        self._owned.clear()


def shard_plan(world_size: int, rank: int, global_seq: int, q_heads: int, kv_heads: int):
    """Which rows and heads a rank owns under Ulysses context parallelism: a contiguous
    sequence shard before the all-to-all, contiguous head shards after it
    (include/fuse/layout/ulysses.h:95-104 of the reference)."""
    if global_seq % world_size or q_heads % world_size or kv_heads % world_size:
        raise ValueError("sequence and heads must divide by the world size")
    seq_local = global_seq // world_size
    return {"seq_local": seq_local, "row_begin": rank * seq_local, "row_end": (rank + 1) * seq_local,
            "q_heads": (rank * q_heads // world_size, (rank + 1) * q_heads // world_size),
            "kv_heads": (rank * kv_heads // world_size, (rank + 1) * kv_heads // world_size)}
