"""Runtime-agnostic access to the arguments of one lowered task.

A lowered training graph is a list of invocations (``runtime/lowering.py``): each names a task kind (FWD / BWD /
UPD / LOSS / COPY), the operator, and its input and output *values*, a value being (producer node, slot, role,
shard) with role FWD (activation or weight), GRAD, or OPT:<state>.  ``TaskArgumentAccessor`` resolves those
values against whatever holds the tensors -- a dict for the CPU interpreter, the executor's value table on the
GPU -- so a task body is written once against this interface.

Counterpart of the reference's ``ITaskArgumentAccessor`` (lib/task-spec/include/task-spec/task_argument_accessor/
itask_argument_accessor.h:21-41): tensors by (slot, role), operator / loss / optimizer attributes, device index,
profiling settings.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..utils.profiling import ProfilingSettings

TensorKey = Tuple[int, str, str, Optional[int]]  # (node, slot, role, shard)


def value_key(v: dict) -> TensorKey:
    return (int(v["node"]), str(v["slot"]), str(v["role"]), v.get("shard"))


@dataclass
class TaskArgumentAccessor:
    invocation: dict
    tensors: Dict[TensorKey, torch.Tensor]
    op_attrs: dict = field(default_factory=dict)
    loss_attrs: Optional[dict] = None
    optimizer_attrs: Optional[dict] = None
    device_idx: int = 0
    profiling: ProfilingSettings = field(default_factory=ProfilingSettings)
    allocate: Optional[Callable[[List[int], torch.dtype], torch.Tensor]] = None

    # ---- identity of the task
    @property
    def task_type(self) -> str:
        return self.invocation["task"]

    @property
    def op_type(self) -> str:
        return self.invocation["op_type"]

    @property
    def name(self) -> str:
        return self.invocation.get("name") or ""

    # ---- tensors
    def _find(self, values: List[dict], slot: str, role: str) -> Optional[dict]:
        for v in values:
            if v.get("as", v["slot"]) == slot and v["role"] == role:
                return v
        return None

    def has(self, slot: str, role: str = "FWD") -> bool:
        return self._find(self.invocation["inputs"], slot, role) is not None

    def get_tensor(self, slot: str, role: str = "FWD") -> torch.Tensor:
        """Input tensor bound to operator slot `slot` (e.g. "INPUT", "WEIGHT") in the given role."""
        v = self._find(self.invocation["inputs"], slot, role)
        if v is None:
            raise KeyError(f"task {self.task_type} of {self.op_type} has no input ({slot}, {role})")
        return self.tensors[value_key(v)]

    def get_output(self, slot: str = "OUTPUT", role: Optional[str] = None) -> torch.Tensor:
        outs = self.invocation["outputs"]
        for v in outs:
            if v.get("as", v["slot"]) == slot and (role is None or v["role"] == role):
                return self.tensors[value_key(v)]
        raise KeyError(f"task {self.task_type} of {self.op_type} has no output ({slot}, {role})")

    def set_output(self, tensor: torch.Tensor, slot: str = "OUTPUT", role: Optional[str] = None):
        for v in self.invocation["outputs"]:
            if v.get("as", v["slot"]) == slot and (role is None or v["role"] == role):
                self.tensors[value_key(v)] = tensor
                return
        raise KeyError(f"task {self.task_type} of {self.op_type} has no output ({slot}, {role})")

    def optimizer_state(self, name: str) -> torch.Tensor:
        """Optimizer slot tensor of an UPD task ("m", "v", "momentum")."""
        for v in self.invocation["inputs"]:
            if v["role"] == f"OPT:{name}":
                return self.tensors[value_key(v)]
        raise KeyError(f"no optimizer state {name}")

    def new_tensor(self, shape, dtype=torch.float32) -> torch.Tensor:
        if self.allocate is not None:
            return self.allocate(list(shape), dtype)
        return torch.empty(list(shape), dtype=dtype)


def run_invocations(invocations: List[dict], bodies: Dict[Tuple[str, str], Callable[[TaskArgumentAccessor], None]], tensors=None,
                    op_attrs_of: Optional[Callable[[int], dict]] = None, **accessor_kw) -> Dict[TensorKey, torch.Tensor]:
    """Execute lowered invocations in order with task bodies keyed by (task kind, operator type); a body keyed
    (task kind, "*") is the default for that kind.  Returns the tensor table."""
    table: Dict[TensorKey, torch.Tensor] = {} if tensors is None else tensors
    for inv in invocations:
        body = bodies.get((inv["task"], inv["op_type"])) or bodies.get((inv["task"], "*"))
        if body is None:
            raise NotImplementedError(f"no task body for {inv['task']} of {inv['op_type']}")
        attrs = op_attrs_of(inv["node"]) if op_attrs_of is not None else {}
        body(TaskArgumentAccessor(inv, table, op_attrs=attrs, **accessor_kw))
    return table
