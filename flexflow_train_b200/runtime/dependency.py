"""Reader / writer dependency tracking over lowered invocations.

``DependencySet`` keeps, per tensor value, the last writer and the readers since: an invocation that reads a value
waits for its last writer (read after write); one that writes it waits for the readers since the last write (write
after read) and for that writer (write after write).  The reference's distributed executor orders its Realm task
launches and copies exactly so (lib/realm-execution/src/realm-execution/dependency_set.cc, used from
pcg_instance.cc:229-273).  Here the GPU executors run a static plan in stream order, so the tracker's job is
analysis: ``dependency_graph`` gives the true partial order of a lowered step, ``check_order`` verifies that a
sequential order respects it, and ``schedule_levels`` shows which invocations could run concurrently (what a
multi-stream plan may overlap: the parallel branches of an Inception block, the gradient all-reduce of a finished
bucket against the rest of backward).
"""
from __future__ import annotations

from typing import Dict, Hashable, Iterable, List, Sequence, Set, Tuple

from .task_accessor import value_key


class DependencySet:
    """Events are any hashable ids (here: positions in the invocation list)."""

    def __init__(self):
        self._writer: Dict[Hashable, Hashable] = {}
        self._readers: Dict[Hashable, List[Hashable]] = {}

    def add_reader(self, value: Hashable, event: Hashable) -> Set[Hashable]:
        """Register `event` as a reader of `value`; returns the events it must wait for."""
        deps = set()
        w = self._writer.get(value)
        if w is not None and w != event:
            deps.add(w)
        self._readers.setdefault(value, []).append(event)
        return deps

    def add_writer(self, value: Hashable, event: Hashable) -> Set[Hashable]:
        """Register `event` as the new writer of `value`; returns the events it must wait for."""
        deps = {r for r in self._readers.get(value, ()) if r != event}
        w = self._writer.get(value)
        if w is not None and w != event:
            deps.add(w)
        self._writer[value] = event
        self._readers[value] = []
        return deps


def _accumulates(inv: dict, v: dict) -> bool:
    """A gradient output is added into (read and written) when another invocation produced it before."""
    return v["role"] == "GRAD"


def dependency_graph(invocations: Sequence[dict]) -> Dict[int, Set[int]]:
    """invocation index -> indices it depends on (RAW, WAR and WAW over the values it reads and writes)."""
    ds = DependencySet()
    deps: Dict[int, Set[int]] = {}
    for i, inv in enumerate(invocations):
        d: Set[int] = set()
        for v in inv.get("inputs", ()):
            d |= ds.add_reader(value_key(v), i)
        for v in inv.get("outputs", ()):
            k = value_key(v)
            if _accumulates(inv, v):
                d |= ds.add_reader(k, i)
            d |= ds.add_writer(k, i)
        deps[i] = d
    return deps


def check_order(invocations: Sequence[dict], order: Iterable[int]) -> List[Tuple[int, int]]:
    """Pairs (invocation, dependency) that `order` runs the wrong way round; empty when the order is valid."""
    deps = dependency_graph(invocations)
    pos = {idx: p for p, idx in enumerate(order)}
    return [(i, j) for i, ds_ in deps.items() for j in ds_ if pos[j] > pos[i]]


def schedule_levels(invocations: Sequence[dict]) -> List[List[int]]:
    """Invocations grouped by the length of their longest dependency chain: members of one level are independent."""
    deps = dependency_graph(invocations)
    level: Dict[int, int] = {}
    for i in range(len(invocations)):  # the list order is a valid order, so dependencies have their level already
        level[i] = 1 + max((level[j] for j in deps[i]), default=-1)
    out: List[List[int]] = [[] for _ in range(max(level.values(), default=-1) + 1)]
    for i, l in level.items():
        out[l].append(i)
    return out
