"""Per-device handle and stream objects of the runtime.

A task body gets from its ``DeviceHandle`` everything that is per device rather than per operator: the device, the
allocator its long-lived buffers come from, the one fp32 workspace every operator's scratch needs are folded into, the
tf32 policy and -- with several GPUs -- the peer-memory context that plays the communicator's role.  The reference keeps
the same things in ``PerDeviceFFHandle`` (library handles, ``workSpace`` / ``workSpaceSize``,
``allowTensorOpMathConversion``, ``ncclComm``: lib/kernels/include/kernels/ff_handle.h) behind an owning wrapper with
``initialize_single_gpu_handle`` / ``initialize_multi_gpu_handle`` (managed_per_device_ff_handle.h) and a
``device_handle_t`` that is empty on the CPU (device_handle_t.h).  There is no cuDNN / cuBLAS handle here: the kernels
are this package's own and take a stream.

The workspace is sized in two steps because the executor learns its operators' needs while it builds the plan:
operators call ``reserve_workspace`` during set-up, ``materialize_workspace`` allocates once afterwards; a fixed
``workspace_bytes`` given at creation is a floor.

``ManagedStream`` owns a CUDA stream (managed_ff_stream.h); ``DeviceStream`` is the value a task sees: a CUDA stream or
the CPU's "no stream" (device_stream_t.h).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .allocator import Allocator, LocalCPUAllocator, LocalCudaAllocator, TrackedAllocator


@dataclass(frozen=True)
class DeviceStream:
    """A CUDA stream handle (``cuda_stream`` is the raw ``cudaStream_t`` value) or, on the CPU, nothing."""
    cuda_stream: Optional[int] = None

    @property
    def is_gpu(self) -> bool:
        return self.cuda_stream is not None


class ManagedStream:
    """Owns one CUDA stream of a device; ``raw_stream`` is what the kernel entry points take."""

    def __init__(self, device_index: int = 0):
        self._stream = torch.cuda.Stream(device=device_index)

    @property
    def torch_stream(self) -> "torch.cuda.Stream":
        return self._stream

    def raw_stream(self) -> DeviceStream:
        return DeviceStream(self._stream.cuda_stream)

    def synchronize(self):
        self._stream.synchronize()


@dataclass
class DeviceHandle:
    device: torch.device
    device_index: int
    allocator: TrackedAllocator
    workspace_bytes: int = 0                       # reserved so far (a floor before planning, the maximum asked afterwards)
    allow_tensor_op_math_conversion: bool = True   # fp32 matrix products may run on the tensor cores as tf32
    num_ranks: int = 1
    my_rank: int = 0
    dist: object = None                            # parallel.context.DistContext: peer pointers, flags, process groups
    workspace: Optional[torch.Tensor] = field(default=None, repr=False)

    @property
    def is_gpu(self) -> bool:
        return self.device.type == "cuda"

    def stream(self) -> DeviceStream:
        """The stream kernels launched now go to (the current stream of the device; a capture stream during capture)."""
        return DeviceStream(torch.cuda.current_stream(self.device_index).cuda_stream) if self.is_gpu else DeviceStream()

    def reserve_workspace(self, nbytes: int) -> None:
        if self.workspace is not None and nbytes > self.workspace.numel() * 4:
            raise RuntimeError(f"workspace of {self.workspace.numel() * 4} bytes is already allocated; {nbytes} bytes were asked for")
        self.workspace_bytes = max(self.workspace_bytes, int(nbytes))

    def materialize_workspace(self) -> torch.Tensor:
        if self.workspace is None:
            self.workspace = self.allocator.allocate([max((self.workspace_bytes + 3) // 4, 1)], torch.float32)
        return self.workspace

    def describe(self) -> str:
        return (f"<DeviceHandle {self.device.type}:{self.device_index} rank {self.my_rank}/{self.num_ranks} workspace "
                f"{self.workspace_bytes} bytes tf32 {'on' if self.allow_tensor_op_math_conversion else 'off'}>")


def _make(device: torch.device, workspace_bytes: int, allow_tf32: bool, num_ranks: int, my_rank: int, dist, allocator: Optional[Allocator]) -> DeviceHandle:
    gpu = device.type == "cuda"
    # "cuda" without an index means the process's current device (one process per GPU sets it before compiling)
    index = device.index if device.index is not None else (torch.cuda.current_device() if gpu else 0)
    inner = allocator or (LocalCudaAllocator(index) if gpu else LocalCPUAllocator())
    tracked = inner if isinstance(inner, TrackedAllocator) else TrackedAllocator(inner)
    return DeviceHandle(device=device, device_index=index, allocator=tracked, workspace_bytes=int(workspace_bytes),
                        allow_tensor_op_math_conversion=allow_tf32, num_ranks=num_ranks, my_rank=my_rank, dist=dist)


def create_local_handle_for_device(device="cuda", workspace_bytes: int = 0, allow_tensor_op_math_conversion: bool = True,
                                   allocator: Optional[Allocator] = None) -> DeviceHandle:
    """One process, one device (``initialize_single_gpu_handle`` / the CPU's empty handle)."""
    return _make(torch.device(device), workspace_bytes, allow_tensor_op_math_conversion, 1, 0, None, allocator)


def create_multi_gpu_handle(dist, workspace_bytes: int = 0, allow_tensor_op_math_conversion: bool = True,
                            allocator: Optional[Allocator] = None) -> DeviceHandle:
    """This rank's handle in a job of ``dist.world_size`` processes (``initialize_multi_gpu_handle(num_ranks, my_rank, ...)``):
    the distributed context carries what the communicator carries upstream."""
    dev = torch.device("cuda", getattr(dist, "local_rank", 0)) if torch.cuda.is_available() else torch.device("cpu")
    return _make(dev, workspace_bytes, allow_tensor_op_math_conversion, int(dist.world_size), int(dist.rank), dist, allocator)
