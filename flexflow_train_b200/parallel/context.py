"""Per-rank distributed context: process group plumbing plus NVLink peer memory.

One process per GPU (``torch.distributed``, NCCL) provides bootstrap, object exchange and the baseline
collectives.  The product path uses *symmetric buffers*: every rank allocates the same buffer, publishes its
CUDA IPC handle and maps all peers' buffers, so kernels address remote memory with ordinary pointers
(loads/stores over NVLink 5 / NVSwitch).  The reference's counterpart is the per-device handle with its NCCL
communicator (lib/kernels/src/kernels/managed_per_device_ff_handle.cc:7-48) and Realm's instance copies
(lib/realm-execution/src/realm-execution/realm_context.cc:157-225).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops import kernels as K

NUM_FLAGS = 4096  # 64-bit flags per rank


class _DevMem:
    """Exposes a raw device pointer through __cuda_array_interface__ so torch can wrap it without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _wrap(ptr: int, nbytes: int, device) -> torch.Tensor:
    return torch.as_tensor(_DevMem(ptr, nbytes), device=device)


class SymmetricBuffer:
    """The same `nbytes` region on every rank; ``local`` is this rank's tensor (uint8), ``peer_ptrs[r]`` the
    address of rank r's region as seen from this rank (``peer_ptrs[rank]`` is the local address)."""

    def __init__(self, ctx: "DistContext", nbytes: int):
        lib = K.lib()
        lib.ffk_symm_alloc.restype = ctypes.c_void_p
        lib.ffk_symm_alloc.argtypes = [ctypes.c_longlong]
        lib.ffk_ipc_get_handle.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.ffk_ipc_get_handle.restype = ctypes.c_int
        lib.ffk_ipc_open.restype = ctypes.c_void_p
        lib.ffk_ipc_open.argtypes = [ctypes.c_void_p]
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.ctx = ctx
        ptr = lib.ffk_symm_alloc(self.nbytes)
        if not ptr:
            raise RuntimeError(f"symmetric allocation of {self.nbytes} bytes failed")
        self.local_ptr = int(ptr)
        handle = ctypes.create_string_buffer(64)
        rc = lib.ffk_ipc_get_handle(ptr, handle)
        if rc != 0:
            raise RuntimeError(f"cudaIpcGetMemHandle failed with {rc}")
        handles: List[Optional[bytes]] = [None] * ctx.world_size
        dist.all_gather_object(handles, bytes(handle.raw), group=ctx.group)
        self.peer_ptrs: List[int] = []
        for r, h in enumerate(handles):
            if r == ctx.rank:
                self.peer_ptrs.append(self.local_ptr)
            else:
                p = lib.ffk_ipc_open(ctypes.create_string_buffer(h, 64))
                if not p:
                    raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed (peer access unavailable?)")
                self.peer_ptrs.append(int(p))
        self.local = _wrap(self.local_ptr, self.nbytes, ctx.device)
        self.ptr_array = (ctypes.c_void_p * ctx.world_size)(*self.peer_ptrs)

    def view(self, dtype, shape=None, byte_offset: int = 0, numel: Optional[int] = None) -> torch.Tensor:
        es = torch.empty((), dtype=dtype).element_size()
        n = numel if numel is not None else (self.nbytes - byte_offset) // es
        t = self.local[byte_offset:byte_offset + n * es].view(dtype)
        return t.view(shape) if shape is not None else t

    def peer_ptr_array(self, byte_offset: int = 0):
        return (ctypes.c_void_p * self.ctx.world_size)(*[p + byte_offset for p in self.peer_ptrs])


class DistContext:
    def __init__(self, rank: int, world_size: int, local_rank: Optional[int] = None, group=None):
        self.rank = rank
        self.world_size = world_size
        self.local_rank = rank if local_rank is None else local_rank
        self.group = group
        self.device = torch.device("cuda", self.local_rank)
        self._subgroups: Dict[Tuple[int, ...], object] = {}
        self.flags = SymmetricBuffer(self, NUM_FLAGS * 8)
        self._next_flag = 0
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._syncs: List[torch.Tensor] = []
        dist.barrier(group=group)

    # ---- resources
    def alloc_flags(self, n: int) -> int:
        base = self._next_flag
        if base + n > NUM_FLAGS:
            raise RuntimeError("out of peer flags")
        self._next_flag += n
        return base

    def new_sync(self) -> torch.Tensor:
        """16 bytes of local state for one collective call site: epoch (u64), started, blocks_done (u32)."""
        t = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._syncs.append(t)
        return t

    def symmetric(self, nbytes: int) -> SymmetricBuffer:
        return SymmetricBuffer(self, nbytes)

    def subgroup(self, ranks: Sequence[int]):
        key = tuple(ranks)
        if key == tuple(range(self.world_size)):
            return self.group
        if key not in self._subgroups:
            self._subgroups[key] = dist.new_group(list(key))
        return self._subgroups[key]

    def check_status(self):
        """Raise if a device-side bounded wait on a peer ran out (reads one int from the device)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            from ..utils.failure import CommTimeoutError
            raise CommTimeoutError(f"rank {self.rank}: a peer did not answer within the device-side wait limit (code {code})")
