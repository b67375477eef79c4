"""sp-ization-benchmarking: compare the SP-ization algorithms on sample graphs under several cost distributions.

    python -m flexflow_train_b200.bin.sp_ization_benchmarking
    python -m flexflow_train_b200.bin.sp_ization_benchmarking --graphs nasnet_cell,random --repeat 20 --json

For every (graph, cost distribution, noise) it turns the DAG into a series-parallel tree with each technique and
reports, relative to the DAG itself, how much total work the tree performs (duplicating techniques re-execute
nodes) and how much longer its critical path is (synchronising techniques add barriers).  The algorithm picks
with the *noisy* costs; the result is judged with the *true* costs, which is how a cost-model error shows.

Counterpart of bin/sp-ization-benchmarking (src/sp-ization-benchmarking/main.cc: graph families, the Constant /
Uniform / Binary / Chooser distributions with uniform and Gaussian noise, and the output table).
"""
from __future__ import annotations

import argparse
import json
import random
import sys
from typing import Callable, Dict, List, Tuple

from .. import _ffcore as core


# ------------------------------------------------------------------------------------------ graph families
def _graph(n: int, edges: List[Tuple[int, int]]):
    g = core.DiGraph()
    for i in range(n):
        g.add_node(i)
    for a, b in edges:
        g.add_edge(a, b)
    return g


def make_linear(length: int = 8):
    return _graph(length, [(i, i + 1) for i in range(length - 1)])


def make_rhombus():
    return _graph(4, [(0, 1), (0, 2), (1, 3), (2, 3)])


def make_diamond():
    return _graph(6, [(0, 1), (0, 2), (1, 3), (2, 3), (2, 4), (3, 5), (4, 5)])


def make_fully_connected(layer_sizes=(1, 3, 3, 1)):
    edges, start = [], 0
    for a, b in zip(layer_sizes, layer_sizes[1:]):
        for i in range(a):
            for j in range(b):
                edges.append((start + i, start + a + j))
        start += a
    return _graph(sum(layer_sizes), edges)


def make_parallel_chains(chain_length: int = 8, chain_num: int = 4):
    edges, n = [], 1
    sink = 1 + chain_length * chain_num
    for _ in range(chain_num):
        prev = 0
        for _ in range(chain_length):
            edges.append((prev, n))
            prev = n
            n += 1
        edges.append((prev, sink))
    return _graph(sink + 1, edges)


def make_sample_dag():
    """A small non-SP DAG with crossing dependencies between two branches."""
    return _graph(9, [(0, 1), (0, 2), (1, 3), (1, 4), (2, 4), (2, 5), (3, 6), (4, 6), (4, 7), (5, 7), (6, 8), (7, 8)])


def make_nasnet_cell(blocks: int = 5, seed: int = 7):
    """NASNet-style cell: two cell inputs; every block combines two earlier hidden states through two operator
    nodes and an add; unused states are concatenated at the end."""
    rng = random.Random(seed)
    edges, states, used = [], [0, 1], set()
    n = 2
    for _ in range(blocks):
        a, b = rng.sample(states, 2) if len(states) > 1 else (states[0], states[0])
        op_a, op_b, add = n, n + 1, n + 2
        n += 3
        edges += [(a, op_a), (b, op_b), (op_a, add), (op_b, add)]
        used.update((a, b))
        states.append(add)
    concat = n
    n += 1
    for s in states:
        if s not in used and s > 1:
            edges.append((s, concat))
    src = n  # single source feeding both cell inputs keeps the graph 2-terminal
    n += 1
    edges += [(src, 0), (src, 1)]
    if not any(e[1] == concat for e in edges):
        edges.append((states[-1], concat))
    return _graph(n, edges)


def make_2_terminal_random_dag(num_nodes: int = 30, p: float = 0.15, step: int = 4, seed: int = 0):
    rng = random.Random(seed)
    edges = set()
    for i in range(1, num_nodes - 1):
        lo = max(0, i - step)
        preds = [j for j in range(lo, i) if rng.random() < p]
        if not preds:
            preds = [rng.randrange(lo, i)]
        for j in preds:
            edges.add((j, i))
    has_succ = {a for a, _ in edges}
    for i in range(num_nodes - 1):
        if i not in has_succ:
            edges.add((i, num_nodes - 1))
    return _graph(num_nodes, sorted(edges))


def model_graph(name: str):
    g = core.build_model(name, {})
    return g.digraph()


GRAPHS: Dict[str, Callable[[int], object]] = {
    "linear": lambda s: make_linear(),
    "rhombus": lambda s: make_rhombus(),
    "diamond": lambda s: make_diamond(),
    "fully_connected": lambda s: make_fully_connected(),
    "parallel_chains": lambda s: make_parallel_chains(),
    "sample_dag": lambda s: make_sample_dag(),
    "nasnet_cell": lambda s: make_nasnet_cell(seed=7 + s),
    "random": lambda s: make_2_terminal_random_dag(seed=s),
    "split_test": lambda s: model_graph("split_test"),
}


# ------------------------------------------------------------------------------------------ cost distributions
def Constant(c=1.0): return lambda rng: c
def Uniform(a=0.0, b=1.0): return lambda rng: rng.uniform(a, b)
def Binary(a=1.0, b=80.0, p=0.5): return lambda rng: a if rng.random() < p else b
def Chooser(values=(1.0, 20.0, 500.0)): return lambda rng: rng.choice(list(values))
def NoNoise(): return lambda rng: 1.0
def UniformNoise(lo=0.8, hi=1.25): return lambda rng: rng.uniform(lo, hi)
def GaussianNoise(mean=1.0, std=0.1): return lambda rng: max(rng.gauss(mean, std), 1e-3)


DISTRIBUTIONS = {"Constant(1)": Constant(1.0), "Uniform(0,1)": Uniform(0, 1), "Binary(1,80)": Binary(1, 80),
                 "Chooser({1,20,500})": Chooser()}
NOISES = {"": NoNoise(), "UniformNoise(0.8,1.25)": UniformNoise(), "GaussianNoise(1,0.1)": GaussianNoise()}


# ------------------------------------------------------------------------------------------ measurement
def _dag_costs(g, cost: Dict[int, float]) -> Tuple[float, float]:
    work = sum(cost[n] for n in g.nodes())
    longest: Dict[int, float] = {}
    for n in core.topological_ordering(g):
        longest[n] = cost[n] + max((longest[p] for p in g.predecessors(n)), default=0.0)
    return work, max(longest.values())


TECHNIQUES = {
    "stratum_sync": lambda g, noisy: core.naive_stratum_sync_sp_ization(g),
    "work_duplicating": lambda g, noisy: core.work_duplicating_sp_ization(g, False),
    "work_duplicating_coalesced": lambda g, noisy: core.work_duplicating_sp_ization(g, True),
    "escribano": lambda g, noisy: core.escribano_sp_ization(g),
    "flexible": lambda g, noisy: core.flexible_sp_ization(g, noisy),
}


def benchmark_graph(g, dist, noise, rng: random.Random, repeat: int = 1) -> Dict[str, dict]:
    acc = {t: {"work": 0.0, "cp": 0.0, "ok": True} for t in TECHNIQUES}
    for _ in range(repeat):
        true = {n: float(dist(rng)) for n in g.nodes()}
        noisy = {n: c * noise(rng) for n, c in true.items()}
        work0, cp0 = _dag_costs(g, true)
        for name, fn in TECHNIQUES.items():
            tree = fn(g, noisy)
            acc[name]["work"] += core.sp_work_cost(tree, true) / max(work0, 1e-12)
            acc[name]["cp"] += core.sp_critical_path_cost(tree, true) / max(cp0, 1e-12)
            acc[name]["ok"] = acc[name]["ok"] and bool(core.sp_preserves_dependencies(tree, g))
    return {t: {"relative_work_increase": v["work"] / repeat, "relative_critical_path_increase": v["cp"] / repeat,
                "dependencies_preserved": v["ok"]} for t, v in acc.items()}


def output_benchmark(title: str, result: Dict[str, dict], out=None):
    out = out or sys.stdout
    out.write(f"Benchmark for {title}\n")
    out.write("Technique | Work-Increase | Critical-Path-Increase | Dependencies-Preserved\n")
    for t, r in result.items():
        out.write(f"{t} | {r['relative_work_increase']:.3f} | {r['relative_critical_path_increase']:.3f} | "
                  f"{'yes' if r['dependencies_preserved'] else 'NO'}\n")
    out.write("\n")


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="sp-ization-benchmarking", description=__doc__.split("\n")[0])
    p.add_argument("--graphs", default="sample_dag,nasnet_cell,parallel_chains,random", help=f"comma list of {sorted(GRAPHS)}")
    p.add_argument("--repeat", type=int, default=10, help="cost samples per configuration (random graphs are regenerated)")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--json", action="store_true", help="one JSON object instead of the tables")
    a = p.parse_args(argv)
    rng = random.Random(a.seed)
    results = {}
    for gname in a.graphs.split(","):
        if gname not in GRAPHS:
            p.error(f"unknown graph family {gname}")
        for dname, dist in DISTRIBUTIONS.items():
            for nname, noise in NOISES.items():
                title = ", ".join(x for x in (gname, dname, nname) if x)
                if gname in ("random", "nasnet_cell"):
                    parts = [benchmark_graph(GRAPHS[gname](a.seed + i), dist, noise, rng, 1) for i in range(a.repeat)]
                    res = {t: {k: (all(q[t][k] for q in parts) if k == "dependencies_preserved" else sum(q[t][k] for q in parts) / len(parts))
                               for k in parts[0][t]} for t in parts[0]}
                else:
                    res = benchmark_graph(GRAPHS[gname](0), dist, noise, rng, a.repeat)
                results[title] = res
                if not a.json:
                    output_benchmark(title, res)
    if a.json:
        sys.stdout.write(json.dumps(results, indent=1) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
