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

    def sub(self, ranks: Sequence[int]) -> "GroupContext":
        """The same resources seen by a subset of the ranks (one axis of a device mesh): kernels and fused operators given
        this object address only the members' memory and count only the members.  Every rank of the job must call this
        with the group *it* belongs to at the same point of the program (allocations behind it exchange handles across the
        whole job)."""
        ranks = tuple(int(r) for r in ranks)
        if ranks == tuple(range(self.world_size)):
            return self
        key = ("sub",) + ranks
        if key not in self._subgroups:
            self._subgroups[key] = GroupContext(self, ranks)
        return self._subgroups[key]

    def make_mesh_groups(self, outer: int, inner: int):
        """Rank r = o * inner + i of an outer x inner mesh: returns (group of the ranks that share r's inner index, i.e. the
        outer axis; group of the ranks that share r's outer index, i.e. the inner axis).  The library process groups of
        every row and column are created on every rank, as torch.distributed requires."""
        if outer * inner != self.world_size:
            raise ValueError(f"a {outer} x {inner} mesh does not cover {self.world_size} ranks")
        mine_outer = mine_inner = None
        for i in range(inner):
            members = [o * inner + i for o in range(outer)]
            g = self.subgroup(members) if outer > 1 else None
            if self.rank in members:
                mine_outer = (members, g)
        for o in range(outer):
            members = [o * inner + i for i in range(inner)]
            g = self.subgroup(members) if inner > 1 else None
            if self.rank in members:
                mine_inner = (members, g)
        return self.sub(mine_outer[0]), self.sub(mine_inner[0])

    def check_status(self):
        """Raise if a device-side bounded wait on a peer ran out (reads one int from the device)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            from ..utils.failure import CommTimeoutError
            raise CommTimeoutError(f"rank {self.rank}: a peer did not answer within the device-side wait limit (code {code})")


class _GroupBuffer:
    """A symmetric buffer as one rank group sees it: pointers of the members only, in group order."""

    def __init__(self, base: SymmetricBuffer, g: "GroupContext"):
        self.base, self.ctx = base, g
        self.nbytes = base.nbytes
        self.local_ptr = base.local_ptr
        self.local = base.local
        self.peer_ptrs = [base.peer_ptrs[r] for r in g.members]
        self.ptr_array = (ctypes.c_void_p * g.world_size)(*self.peer_ptrs)

    def view(self, dtype, shape=None, byte_offset: int = 0, numel: Optional[int] = None) -> torch.Tensor:
        return self.base.view(dtype, shape, byte_offset, numel)

    def peer_ptr_array(self, byte_offset: int = 0):
        return (ctypes.c_void_p * self.ctx.world_size)(*[p + byte_offset for p in self.peer_ptrs])


class GroupContext:
    """A DistContext restricted to `members` (global ranks): ``rank`` is the position inside the group and ``world_size``
    the group's size, so the peer-memory collectives and fused operators run unchanged on one axis of a mesh.  Flags,
    status word and call-site state are the parent's; symmetric allocations go through the parent (every rank of the job
    allocates at the same time, each for its own group) and expose the members' addresses only."""

    def __init__(self, parent: DistContext, members: Sequence[int]):
        if parent.rank not in members:
            raise ValueError("a rank can only hold the groups it belongs to")
        self.parent = parent
        self.members = tuple(members)
        self.rank = self.members.index(parent.rank)
        self.world_size = len(self.members)
        self.local_rank = parent.local_rank
        self.device = parent.device
        self.group = parent.subgroup(self.members) if self.world_size > 1 else None
        self.flags = _GroupBuffer(parent.flags, self)
        self.status = parent.status

    def alloc_flags(self, n: int) -> int:
        return self.parent.alloc_flags(n)

    def new_sync(self) -> torch.Tensor:
        return self.parent.new_sync()

    def symmetric(self, nbytes: int) -> _GroupBuffer:
        return _GroupBuffer(self.parent.symmetric(nbytes), self)

    def subgroup(self, ranks: Sequence[int]):
        return self.parent.subgroup(ranks)

    def check_status(self):
        self.parent.check_status()
