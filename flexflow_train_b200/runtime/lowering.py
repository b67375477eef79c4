"""Python surface of the lowering passes (C++: csrc/core/lowering.cc)."""
from __future__ import annotations

from typing import Optional

from .. import _ffcore as core

make_dynamic_graph = core.make_dynamic_graph
perform_pass_expansion = core.perform_pass_expansion
perform_loss_insertion = core.perform_loss_insertion
perform_update_insertion = core.perform_update_insertion
perform_copy_insertion = core.perform_copy_insertion
perform_shard_expansion = core.perform_shard_expansion
perform_machine_slicing = core.perform_machine_slicing


def lower(graph, machine=None, *, logit=None, loss: str = "sparse_categorical_crossentropy", optimizer: Optional[dict] = None,
          distributed: bool = False, device: Optional[int] = None):
    """All passes in the reference's order; optionally sliced to one device."""
    machine = machine or core.MachineSpecification(1, 1)
    if logit is None:  # default: the last sink that is an operator output
        kinds = {n["id"]: n["type"] for n in graph.nodes()}
        sinks = [tuple(v) for v in graph.sink_values() if kinds[v[0]] not in ("WEIGHT", "INPUT")]
        logit = sinks[-1] if sinks else None
    inv = core.lower_training_graph(graph, machine, logit, {"type": loss}, optimizer or {"type": "sgd"}, distributed)
    if device is not None:
        if not distributed:  # a single-device lowering is not shard-expanded: all of it belongs to device 0
            return inv if device == 0 else []
        inv = core.perform_machine_slicing(inv, device)
    return inv
