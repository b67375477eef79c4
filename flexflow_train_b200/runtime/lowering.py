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


def check_plan(executable, invocations) -> list:
    """Compare an executor's step plan with the lowered step.  Returns a list of human-readable violations (empty when the
    two agree):

    * every lowered invocation (FWD / LOSS / BWD / UPD of a node) is run by the plan, or is one the executor folds into
      a neighbour or leaves out: the backward of the loss operator (done by the fused loss kernel at the LOSS step), the
      backward of an operator none of whose inputs needs a gradient or that does not lead to the loss, and the update
      of a table that takes its sparse update inside the Embedding's backward;
    * the plan's order respects every read-after-write, write-after-read and write-after-write dependency of the lowered
      step (`runtime.dependency.dependency_graph`);
    * every FWD invocation reads exactly the values the executor's operator is wired to.
    """
    from .dependency import dependency_graph

    plan = executable.step_plan()
    pos = {}
    for i, key in enumerate(plan):
        pos.setdefault(key, i)
    loss_pos = next((i for i, (t, _) in enumerate(plan) if t == "LOSS"), None)
    problems = []

    # operators on a branch that does not lead to the loss value (an auxiliary head that is not trained) receive no
    # gradient: the lowered step still lists their backward, the executor leaves it out
    reaches_loss = set()
    if executable.loss_value is not None:
        stack = [executable.loss_value[0]]
        while stack:
            n = stack.pop()
            if n in reaches_loss:
                continue
            reaches_loss.add(n)
            stack.extend(executable.graph.predecessors(n))
    bwd_memo = {}

    def bwd_pos(node):
        """Where the backward of `node` happens: its own BWD step, the LOSS step for the loss operator (the loss kernel
        writes the gradient of that operator's input itself), and for an operator without a backward of its own (nothing
        upstream needs a gradient, or it was folded into a neighbour) just after the last backward among its consumers."""
        if node in bwd_memo:
            return bwd_memo[node]
        if ("BWD", node) in pos:
            r = pos[("BWD", node)]
        elif loss_pos is not None and executable.loss_value is not None and node == executable.loss_value[0]:
            r = loss_pos
        else:
            later = [bwd_pos(n) for n in executable.graph.successors(node)]
            later = [x for x in later if x is not None]
            r = (max(later) + 0.001) if later else (loss_pos if loss_pos is not None else 0)
        bwd_memo[node] = r
        return r

    def where(inv):
        key = (inv["task"], inv["node"])
        if key in pos:
            return pos[key]
        if inv["task"] == "BWD" and inv["node"] in executable.ops:
            if inv["node"] not in reaches_loss:
                return "untrained"
            return bwd_pos(inv["node"])
        if inv["task"] == "UPD" and inv["node"] in getattr(executable, "sparse_tables", {}):
            return len(plan)
        return None

    where_of = [where(inv) for inv in invocations]
    for inv, w in zip(invocations, where_of):
        if w is None:
            problems.append(f"{inv['task']} of node {inv['node']} ({inv['op_type']}) is in the lowered step but not in the plan")
    deps = dependency_graph(invocations)
    for i, ds in deps.items():
        for d in ds:
            a, b = where_of[d], where_of[i]
            if a is None or b is None or a == "untrained" or b == "untrained":
                continue
            if not a <= b or (a == b and invocations[d]["task"] == invocations[i]["task"] == "FWD"):
                problems.append(f"{invocations[i]['task']} of node {invocations[i]['node']} runs at {b}, before its dependency "
                                f"{invocations[d]['task']} of node {invocations[d]['node']} at {a}")
    for inv in invocations:
        if inv["task"] != "FWD":
            continue
        op = executable.ops.get(inv["node"])
        if op is None:
            problems.append(f"node {inv['node']} has no operator in the executor")
            continue
        want = {(v["node"], v["slot"]) for v in inv["inputs"]}
        have = {tuple(v) for v in op.inputs.values()}
        if want != have:
            problems.append(f"node {inv['node']} ({inv['op_type']}) reads {sorted(have)} in the executor and {sorted(want)} in the lowered step")
    return problems
