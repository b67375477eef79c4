"""Allocators and tensor accessors of the runtime.

``Allocator`` is what a task body allocates through (``TaskArgumentAccessor.allocate``): ``LocalCPUAllocator`` and
``LocalCudaAllocator`` own what they hand out and release it on ``close`` (or when a tensor is given back),
``TrackedAllocator`` wraps any of them and counts current and peak bytes -- the measured cost estimator reports an
operator's memory from it.  Counterparts: lib/kernels/include/kernels/allocation.h, local_cpu_allocator.h,
local_cuda_allocator.h (src/cuda/local_cuda_allocator.cc:7-35) and lib/local-execution's tracked allocator.

``TensorAccessor`` is a typed read or read-write view of a tensor with its shape, dtype and device
(lib/kernels/include/kernels/accessor.h:22-140): ``at`` reads one element on the host, and the helper functions
copy, fill, compare and format accessor contents (lib/kernels/src/kernels/{copy_tensor_accessor,
tensor_accessor_binary_ops,format_accessor_contents}.cc), including the naive reference matmul used as an oracle.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


class Allocator:
    """Interface: ``allocate`` / ``deallocate``; ``__call__`` has the signature TaskArgumentAccessor.allocate expects."""
    device = "cpu"

    def allocate(self, shape: Sequence[int], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        raise NotImplementedError

    def deallocate(self, t: torch.Tensor) -> None:
        raise NotImplementedError

    def __call__(self, shape, dtype=torch.float32):
        return self.allocate(shape, dtype)


class _OwningAllocator(Allocator):
    def __init__(self, device: str):
        self.device = device
        self._live: Dict[int, torch.Tensor] = {}

    def allocate(self, shape, dtype=torch.float32):
        t = torch.empty(list(shape), dtype=dtype, device=self.device)
        self._live[t.data_ptr() if t.numel() else id(t)] = t
        return t

    def deallocate(self, t):
        key = t.data_ptr() if t.numel() else id(t)
        if key not in self._live:
            raise ValueError("deallocate: this allocator did not hand out that tensor (or it was already released)")
        del self._live[key]

    @property
    def num_live(self) -> int:
        return len(self._live)

    def close(self):
        """Release everything still held (the reference's allocator frees its tracked pointers in its destructor)."""
        self._live.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class LocalCPUAllocator(_OwningAllocator):
    def __init__(self):
        super().__init__("cpu")


class LocalCudaAllocator(_OwningAllocator):
    def __init__(self, device_idx: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("LocalCudaAllocator needs a GPU")
        super().__init__(f"cuda:{device_idx}")


class TrackedAllocator(Allocator):
    """Counts the bytes allocated through it: ``current_bytes``, ``peak_bytes``, ``total_allocated_bytes``."""

    def __init__(self, inner: Allocator):
        self.inner = inner
        self.device = inner.device
        self.current_bytes = 0
        self.peak_bytes = 0
        self.total_allocated_bytes = 0
        self._sizes: Dict[int, int] = {}

    def allocate(self, shape, dtype=torch.float32):
        t = self.inner.allocate(shape, dtype)
        n = _nbytes(t)
        self._sizes[t.data_ptr() if t.numel() else id(t)] = n
        self.current_bytes += n
        self.total_allocated_bytes += n
        self.peak_bytes = max(self.peak_bytes, self.current_bytes)
        return t

    def deallocate(self, t):
        key = t.data_ptr() if t.numel() else id(t)
        self.current_bytes -= self._sizes.pop(key)
        self.inner.deallocate(t)


# ------------------------------------------------------------------------------------------ accessors
@dataclass
class TensorAccessor:
    """A tensor with its shape, dtype and device; ``writable`` distinguishes the W from the R accessor."""
    tensor: torch.Tensor
    writable: bool = False

    @property
    def shape(self) -> List[int]:
        return list(self.tensor.shape)

    @property
    def dtype(self) -> torch.dtype:
        return self.tensor.dtype

    @property
    def device_type(self) -> str:
        return "GPU" if self.tensor.is_cuda else "CPU"

    @property
    def ptr(self) -> int:
        return self.tensor.data_ptr()

    def at(self, *coord: int):
        """One element, host tensors only (the reference's accessor.at<DT>(coord) is CPU-only as well)."""
        if self.tensor.is_cuda:
            raise RuntimeError("at() reads on the host: copy the accessor to the CPU first")
        if len(coord) != self.tensor.dim():
            raise IndexError(f"{len(coord)} indices for a {self.tensor.dim()}-d accessor")
        return self.tensor[tuple(coord)].item()

    def set(self, value, *coord: int):
        if not self.writable:
            raise PermissionError("read-only accessor")
        if self.tensor.is_cuda:
            raise RuntimeError("set() writes on the host")
        self.tensor[tuple(coord)] = value


def read_only(a: TensorAccessor) -> TensorAccessor:
    return TensorAccessor(a.tensor, False)


def copy_accessor_data_to_l_from_r(dst: TensorAccessor, src: TensorAccessor) -> None:
    if not dst.writable:
        raise PermissionError("destination accessor is read-only")
    if dst.shape != src.shape or dst.dtype != src.dtype:
        raise ValueError(f"copy between accessors of different shape or dtype: {dst.shape} {dst.dtype} <- {src.shape} {src.dtype}")
    dst.tensor.copy_(src.tensor)


def copy_tensor_accessor(src: TensorAccessor, allocator: Allocator) -> TensorAccessor:
    """A writable copy of `src` in memory from `allocator` (which may live on another device)."""
    out = TensorAccessor(allocator.allocate(src.shape, src.dtype), True)
    out.tensor.copy_(src.tensor)
    return out


def fill_with_zeros(a: TensorAccessor) -> None:
    if not a.writable:
        raise PermissionError("read-only accessor")
    a.tensor.zero_()


def accessors_are_equal(a: TensorAccessor, b: TensorAccessor) -> bool:
    return a.shape == b.shape and a.dtype == b.dtype and bool(torch.equal(a.tensor.cpu(), b.tensor.cpu()))


def format_accessor_contents(a: TensorAccessor, max_elements: int = 64) -> str:
    t = a.tensor.detach().cpu()
    flat = t.reshape(-1)
    shown = flat[:max_elements].tolist()
    tail = "" if flat.numel() <= max_elements else f", ... ({flat.numel() - max_elements} more)"
    return f"<{a.device_type} {str(a.dtype).replace('torch.', '')} {a.shape}> [{', '.join(repr(v) for v in shown)}{tail}]"


def tensor_accessor_matmul(a: TensorAccessor, b: TensorAccessor, allocator: Optional[Allocator] = None) -> TensorAccessor:
    """Naive reference product of two 2-d host accessors, accumulated in fp64 one element at a time (an oracle for
    small cases, not a kernel; lib/kernels/src/kernels/tensor_accessor_binary_ops.cc:111-141)."""
    if a.tensor.is_cuda or b.tensor.is_cuda:
        raise RuntimeError("the reference matmul runs on host accessors")
    if a.tensor.dim() != 2 or b.tensor.dim() != 2 or a.shape[1] != b.shape[0]:
        raise ValueError(f"matmul of shapes {a.shape} and {b.shape}")
    alloc = allocator or LocalCPUAllocator()
    out = TensorAccessor(alloc.allocate([a.shape[0], b.shape[1]], a.dtype), True)
    A, B = a.tensor.double().tolist(), b.tensor.double().tolist()
    for i in range(a.shape[0]):
        for j in range(b.shape[1]):
            s = 0.0
            for k in range(a.shape[1]):
                s += A[i][k] * B[k][j]
            out.tensor[i, j] = s
    return out
