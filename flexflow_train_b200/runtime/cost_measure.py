"""Measured operator costs for the search (the reference's LocalCostEstimator,
lib/local-execution/src/local-execution/cost_estimator/local_cost_estimator.cc:84-179).

Instead of building a one-operator graph per query, one profiled training step of the whole (single-device or
per-rank) graph times every operator's forward and backward with CUDA events; the timings are stored in the
C++ estimator under the operator's cost key, so later queries for the same operator and shapes are table hits.
"""
from __future__ import annotations

import json
from typing import Dict, Optional

from .. import _ffcore as core


def measure_into(estimator, executable, *, steps: int = 1) -> Dict[str, dict]:
    """Profile `executable` and record every operator's measured cost in `estimator`.  Returns the table."""
    table: Dict[str, dict] = {}
    acc: Dict[int, list] = {}
    for _ in range(max(1, steps)):
        prof = executable.profile_step()
        for (nid, phase), ms in prof["by_node"].items():
            if nid < 0:
                continue
            a = acc.setdefault(nid, [0.0, 0.0, 0])
            a[0 if phase == "fwd" else 1] += ms
    g = executable.graph
    for nid, (fwd, bwd, _) in acc.items():
        key = estimator.op_cost_key(g, nid)
        mem = sum(sh.piece_bytes for _, sh, _ in executable.nodes[nid]["outputs"])
        fwd, bwd = fwd / steps, bwd / steps
        estimator.set_measured(key, fwd, bwd, float(mem))
        table[key] = {"fwd_ms": fwd, "bwd_ms": bwd, "memory_bytes": float(mem), "type": executable.nodes[nid]["type"]}
    return table


def save_table(table: Dict[str, dict], path: str):
    with open(path, "w") as f:
        json.dump(table, f)


def load_table(estimator, path: str) -> int:
    with open(path) as f:
        table = json.load(f)
    for k, v in table.items():
        estimator.set_measured(k, v["fwd_ms"], v["bwd_ms"], v.get("memory_bytes", 0.0))
    return len(table)
