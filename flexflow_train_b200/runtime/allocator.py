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


# ------------------------------------------------------------------------------------------ accessor utilities
# Host-side helpers over accessors, the vocabulary the reference's kernel tests are written in
# (lib/kernels/include/kernels/{map_tensor_accessors,compare_tensor_accessors,tensor_accessor_reductions,
# tensor_accessor_unary_ops,reduce_tensor_accessor,create_accessor_with_contents}.h).  They work on CPU and GPU accessors
# alike (the work runs as torch operators on the accessor's device); functions given as Python callables are applied
# element by element on the host.
def _out(alloc: Optional[Allocator], shape, dtype, like: torch.Tensor) -> TensorAccessor:
    if alloc is None:
        return TensorAccessor(torch.empty(list(shape), dtype=dtype, device=like.device), True)
    return TensorAccessor(alloc.allocate(list(shape), dtype), True)


def _need_writable(a: TensorAccessor):
    if not a.writable:
        raise PermissionError("read-only accessor")


def create_accessor_with_contents(contents, dtype: torch.dtype = torch.float32, allocator: Optional[Allocator] = None,
                                  writable: bool = True) -> TensorAccessor:
    """An accessor holding the nested list `contents` (1-d to 4-d in the reference; any rank here).  Ragged input is an error."""
    try:
        t = torch.tensor(contents, dtype=dtype)
    except (ValueError, TypeError) as e:
        raise ValueError(f"contents are not a rectangular nested list: {e}") from None
    out = _out(allocator, t.shape, dtype, t)
    out.tensor.copy_(t)
    return TensorAccessor(out.tensor, writable)


def map_tensor_accessor(a: TensorAccessor, f, allocator: Optional[Allocator] = None, out_dtype: Optional[torch.dtype] = None) -> TensorAccessor:
    """A new accessor with f applied to every element."""
    flat = a.tensor.detach().cpu().reshape(-1).tolist()
    vals = [f(v) for v in flat]
    dt = out_dtype or a.dtype
    out = _out(allocator, a.shape, dt, a.tensor)
    out.tensor.copy_(torch.tensor(vals, dtype=dt).reshape(a.shape))
    return out


def map_tensor_accessor_inplace(a: TensorAccessor, f) -> None:
    _need_writable(a)
    a.tensor.copy_(map_tensor_accessor(a, f).tensor)


def map_tensor_accessors2(lhs: TensorAccessor, rhs: TensorAccessor, f, allocator: Optional[Allocator] = None,
                          out_dtype: Optional[torch.dtype] = None) -> TensorAccessor:
    """f(l, r) element by element over two accessors of the same shape."""
    if lhs.shape != rhs.shape:
        raise ValueError(f"map over accessors of different shapes: {lhs.shape} and {rhs.shape}")
    lv, rv = lhs.tensor.detach().cpu().reshape(-1).tolist(), rhs.tensor.detach().cpu().reshape(-1).tolist()
    dt = out_dtype or lhs.dtype
    out = _out(allocator, lhs.shape, dt, lhs.tensor)
    out.tensor.copy_(torch.tensor([f(x, y) for x, y in zip(lv, rv)], dtype=dt).reshape(lhs.shape))
    return out


def _compare(op):
    def run(lhs: TensorAccessor, rhs: TensorAccessor, allocator: Optional[Allocator] = None) -> TensorAccessor:
        if lhs.shape != rhs.shape or lhs.dtype != rhs.dtype:
            raise ValueError(f"comparison of accessors of different shape or dtype: {lhs.shape} {lhs.dtype} and {rhs.shape} {rhs.dtype}")
        out = _out(allocator, lhs.shape, torch.bool, lhs.tensor)
        out.tensor.copy_(op(lhs.tensor, rhs.tensor.to(lhs.tensor.device)))
        return out
    return run


compare_tensor_accessors_lt = _compare(torch.lt)
compare_tensor_accessors_le = _compare(torch.le)
compare_tensor_accessors_gt = _compare(torch.gt)
compare_tensor_accessors_ge = _compare(torch.ge)
compare_tensor_accessors_eq = _compare(torch.eq)
compare_tensor_accessors_ne = _compare(torch.ne)


def tensor_accessor_all(a: TensorAccessor) -> bool:
    if a.dtype != torch.bool:
        raise TypeError("tensor_accessor_all wants a BOOL accessor")
    return bool(a.tensor.all().item())


def tensor_accessor_any(a: TensorAccessor) -> bool:
    if a.dtype != torch.bool:
        raise TypeError("tensor_accessor_any wants a BOOL accessor")
    return bool(a.tensor.any().item())


def tensor_accessor_scale_by_constant(a: TensorAccessor, constant: float, allocator: Optional[Allocator] = None) -> TensorAccessor:
    out = _out(allocator, a.shape, a.dtype, a.tensor)
    out.tensor.copy_(a.tensor * constant)
    return out


def tensor_accessor_scale_by_constant_inplace(a: TensorAccessor, constant: float) -> None:
    _need_writable(a)
    a.tensor.mul_(constant)


def tensor_accessor_relu(a: TensorAccessor, allocator: Optional[Allocator] = None) -> TensorAccessor:
    out = _out(allocator, a.shape, a.dtype, a.tensor)
    out.tensor.copy_(torch.relu(a.tensor))
    return out


def tensor_accessor_broadcast(a: TensorAccessor, target_shape: Sequence[int], allocator: Optional[Allocator] = None) -> TensorAccessor:
    """numpy broadcasting to `target_shape` (rank promotion at the front, size-1 dims expanded)."""
    try:
        b = a.tensor.expand(list(target_shape))
    except RuntimeError:
        raise ValueError(f"{a.shape} does not broadcast to {list(target_shape)}") from None
    out = _out(allocator, target_shape, a.dtype, a.tensor)
    out.tensor.copy_(b)
    return out


def tensor_accessor_transpose(a: TensorAccessor, allocator: Optional[Allocator] = None) -> TensorAccessor:
    if a.tensor.dim() != 2:
        raise ValueError("transpose of a 2-d accessor")
    out = _out(allocator, [a.shape[1], a.shape[0]], a.dtype, a.tensor)
    out.tensor.copy_(a.tensor.t())
    return out


def reduce_tensor_accessor_in_dims(a: TensorAccessor, dims: Sequence[int], f, allocator: Optional[Allocator] = None) -> TensorAccessor:
    """Folds f(acc, element) over the given dims (which disappear from the shape); the first element seeds acc."""
    dims = sorted(set(int(d) for d in dims))
    if any(d < 0 or d >= a.tensor.dim() for d in dims):
        raise ValueError(f"reduce dims {dims} outside a {a.tensor.dim()}-d accessor")
    keep = [d for d in range(a.tensor.dim()) if d not in dims]
    moved = a.tensor.detach().cpu().permute(keep + dims).reshape([a.shape[d] for d in keep] + [-1])
    rows = moved.reshape(-1, moved.shape[-1]).tolist()
    vals = []
    for row in rows:
        acc = row[0]
        for v in row[1:]:
            acc = f(acc, v)
        vals.append(acc)
    out = _out(allocator, [a.shape[d] for d in keep], a.dtype, a.tensor)
    out.tensor.copy_(torch.tensor(vals, dtype=a.dtype).reshape([a.shape[d] for d in keep]))
    return out


def tensor_accessor_reduce(a: TensorAccessor, dim: int, allocator: Optional[Allocator] = None) -> TensorAccessor:
    """Sum over one dim."""
    return reduce_tensor_accessor_in_dims(a, [dim], lambda x, y: x + y, allocator)
