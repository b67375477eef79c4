"""Strategy selection: from a computation graph to the parallel computation graph that will be executed.

``optimize`` is the counterpart of the reference's entry point
(lib/compiler/src/compiler/compiler.cc:10-38): it dispatches on the algorithm (Unity best-first search over
substitutions, MCMC over mapped PCGs, or plain data parallelism -- which the reference declares but leaves
unimplemented).  The search is seeded with the canonical strategies that the substitution rules can express
(pure data parallel, Megatron-style tensor parallel), each scored by the same machine-mapping DP, so a small
budget already returns a sensible plan on deep repeated-layer models where blind search would not.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Tuple

from .. import _ffcore as core


def machine_for(world: int, num_nodes: int = 1) -> "core.MachineSpecification":
    return core.MachineSpecification(num_nodes, max(world // num_nodes, 1))


def _rules_named(rules, pred: Callable[[str], bool]):
    return [r for r in rules if pred(r.name)]


def cancellation_rules(rules):
    return _rules_named(rules, lambda n: n.startswith("cancel"))


def data_parallel_rules(rules, degree: int):
    """Every generated rule that shards dim 0 (the sample dim) `degree` ways."""
    sfx = (f"_0_{degree}", f"_0_{degree}_bias", f"_0_{degree}_affine")

    def pred(n: str) -> bool:
        if n.startswith("partition_attention_combine_") or n.startswith("partition_conv2d_combine_"):
            return n.split("_")[3] == str(degree)
        return n.startswith("partition_") and "_combine" in n and n.endswith(sfx)

    return _rules_named(rules, pred)


def is_parameter_parallel_rule(name: str) -> bool:
    """Rules that shard an operator's weights (column / row parallel Linear, head-parallel attention)."""
    return name.startswith(("replicate_linear_combine", "partition_linear_reduce", "replicate_attention_reduce"))


def is_attribute_parallel_rule(name: str) -> bool:
    """Partition rules on a dim other than the sample dim (the reference's attribute parallelism)."""
    if not (name.startswith("partition_") and "_combine_" in name):
        return False
    parts = name.replace("_bias", "").replace("_affine", "").split("_")
    tail = parts[parts.index("combine") + 1:]
    if len(tail) < 2 or not all(t.isdigit() for t in tail[-2:]):
        return False  # rules without a dim in their name shard the sample dim
    return int(tail[-2]) != 0


def filter_rules(rules, enable_parameter_parallel: bool = True, enable_attribute_parallel: bool = True):
    return [r for r in rules
            if (enable_parameter_parallel or not is_parameter_parallel_rule(r.name))
            and (enable_attribute_parallel or not is_attribute_parallel_rule(r.name))]


def apply_where(graph, rule, pred: Callable, max_total_degree: int = 0, with_graph: bool = False):
    """Apply `rule` at every match whose first pattern node satisfies pred(node dict) -- or pred(graph, node dict)
    with ``with_graph``, for predicates that look at the node's neighbours in the current graph."""
    changed = True
    while changed:
        changed = False
        for m in core.find_pattern_matches(rule, graph):
            node = graph.node(m.nodes[0])
            if not (pred(graph, node) if with_graph else pred(node)):
                continue
            ng = core.apply_substitution(graph, rule, m)
            if ng is None:
                continue
            if max_total_degree and any(o[1].total_degree > max_total_degree for n in ng.nodes() for o in n["outputs"]):
                continue
            graph = ng
            changed = True
            break
    return graph


def data_parallel_strategy(cg, world: int, rules=None):
    ms = machine_for(world)
    rules = rules or core.get_substitution_set(ms)
    pcg = core.pcg_from_computation_graph(cg)
    sel = data_parallel_rules(rules, world) + cancellation_rules(rules)
    return core.apply_rules_exhaustively(pcg, sel, 100000, world)


def _on_table_side(graph, n) -> bool:
    """Is `n` an Embedding, the Reshape of one, or the Concat that stacks such lookups?"""
    t = n["type"]
    if t == "EMBEDDING":
        return True
    if t in ("RESHAPE", "FLAT"):
        return graph.node(tuple(n["inputs"][0][1])[0])["type"] == "EMBEDDING"
    if t == "CONCAT":
        prods = [graph.node(tuple(v)[0]) for _, v in n["inputs"]]
        return all(p["type"] != "CONCAT" and _on_table_side(graph, p) for p in prods)
    return False


def has_stacked_embeddings(cg) -> bool:
    return any(n["type"] == "CONCAT" and _on_table_side(cg, n) for n in cg.nodes())


def table_parallel_strategy(cg, world: int, rules=None):
    """Embedding tables model-parallel, everything else data-parallel (the recommendation-model layout).

    The lookups and the Concat that stacks them stay unpartitioned operators on whole tables -- placed on
    different devices, which is the reference's inter-operator parallelism over the parallel branches of the
    series-parallel decomposition (lib/compiler/src/compiler/machine_mapping/get_optimal_machine_mapping.cc:215-263)
    -- and every other operator is sharded over the sample dim.  The Repartition(0) that the first data-parallel
    consumer puts behind the Concat is the all-to-all from table owners to sample owners; no table is ever
    replicated, so no table-sized gradient crosses the links."""
    ms = machine_for(world)
    rules = rules or core.get_substitution_set(ms)
    g = core.pcg_from_computation_graph(cg)
    if not has_stacked_embeddings(g):
        raise ValueError("no stacked embedding lookups in this graph")
    for r in data_parallel_rules(rules, world):
        g = apply_where(g, r, lambda graph, n: not _on_table_side(graph, n), world, with_graph=True)
    g = core.apply_rules_exhaustively(g, cancellation_rules(rules), 100000, world)
    return core.merge_duplicate_parallel_ops(g)


def tensor_parallel_strategy(cg, world: int, rules=None, sequence_parallel: bool = True):
    """Megatron-style template expressed with the substitution rules: attention heads sharded
    (replicate-attention-reduce), the first Linear of each MLP column-parallel (replicate-linear-combine), the
    second row-parallel (partition-linear-reduce), the pointwise ops between them sharded on the feature dim.

    With ``sequence_parallel`` every operator the template leaves replicated (LayerNorm, residual add, dropout,
    embedding, the vocabulary projection and softmax) is then sharded over the sample dim with the data-parallel
    rules.  The activations between two tensor-parallel regions are thereby held as row shards: each Reduction is
    followed by a Repartition (together a reduce-scatter, fused into the producing GEMM) and each Replicate is
    preceded by a Combine (together an all-gather, fused into the consuming GEMM), and nothing is computed
    redundantly."""
    ms = machine_for(world)
    rules = rules or core.get_substitution_set(ms)
    by_name = {r.name: r for r in rules}
    g = core.pcg_from_computation_graph(cg)
    W = world
    for bias in ("", "_bias"):
        r = by_name.get(f"replicate_attention_reduce_{W}{bias}")
        if r is not None:
            g = apply_where(g, r, lambda n: True, W)
    # Linear layers: a Linear fed (through pointwise ops) by another Linear becomes row-parallel, its producer
    # column-parallel
    def producer_linear(graph, node):
        v = dict((s, tuple(x)) for s, x in node["inputs"]).get("INPUT")
        while v is not None:
            p = graph.node(v[0])
            if p["type"] == "LINEAR":
                return p
            if p["type"] in ("DROPOUT", "RELU", "GELU", "SIGMOID", "TANH", "CAST"):
                v = tuple(p["inputs"][0][1])
            else:
                return None
        return None

    pairs = []
    for n in g.nodes():
        if n["type"] == "LINEAR":
            p = producer_linear(g, n)
            if p is not None and len(g.consumers((p["id"], "OUTPUT"))) == 1:
                pairs.append((p["name"] or p["id"], n["name"] or n["id"]))
    firsts = {a for a, _ in pairs}
    seconds = {b for _, b in pairs}
    key = lambda n: n["name"] or n["id"]
    for bias in ("", "_bias"):
        rc = by_name.get(f"replicate_linear_combine_{W}{bias}")
        rr = by_name.get(f"partition_linear_reduce_{W}{bias}")
        if rc is not None:
            g = apply_where(g, rc, lambda n: key(n) in firsts, W)
        if rr is not None:
            g = apply_where(g, rr, lambda n: key(n) in seconds, W)
    # shard the pointwise ops between the two Linears on the (last) feature dim, then cancel Combine/Repartition pairs
    feature = [r for r in rules if r.name.startswith("partition_") and "_combine_" in r.name and
               any(r.name.startswith(f"partition_{op}_combine_") for op in ("DROPOUT", "RELU", "GELU", "SIGMOID", "TANH"))
               and r.name.endswith(f"_{W}") and not r.name.endswith(f"_0_{W}")]

    def between(rule_dim):
        def pred(n):
            v = tuple(n["inputs"][0][1])
            # only the feature (last) dim continues the column-parallel sharding of the producing Linear
            return g.node(v[0])["type"] == "COMBINE" and rule_dim == len(n["outputs"][0][1].sizes) - 1
        return pred

    for r in feature:
        g = apply_where(g, r, between(int(r.name.split("_")[-2])), W)
    g = core.apply_rules_exhaustively(g, cancellation_rules(rules), 100000, W)
    if sequence_parallel:
        g = shard_replicated_operators(g, W, rules)
    return core.merge_duplicate_parallel_ops(g)


def hybrid_strategy(cg, dp: int, tp: int, rules=None):
    """Data parallel of degree `dp` around tensor parallel of degree `tp` (dp * tp devices): the Megatron template at
    degree tp with replicated activations, then the sample-dim rules at degree dp on every operator.  The
    Combine(0, dp) that each data-parallel operator ends with is commuted past the template's Replicate / Reduction
    so that it meets the next operator's Repartition(0, dp) and cancels; what remains is one Repartition of the
    inputs, one Combine of the output and the tensor-parallel collectives inside each data-parallel replica.

    The distributed executor runs such a graph on a dp x tp device mesh (rank = i_dp * tp + i_tp)."""
    world = dp * tp
    ms = machine_for(world)
    rules = rules or core.get_substitution_set(ms)
    if dp == 1:
        return tensor_parallel_strategy(cg, tp, rules)
    if tp == 1:
        return data_parallel_strategy(cg, dp, rules)
    g = tensor_parallel_strategy(cg, tp, rules, sequence_parallel=False)
    g = core.apply_rules_exhaustively(g, data_parallel_rules(rules, dp) + cancellation_rules(rules), 100000, world)
    tidy = cancellation_rules(rules) + list(core.get_commute_rules())
    while True:
        n0 = len(g.nodes())
        g = core.apply_rules_exhaustively(core.merge_duplicate_parallel_ops(g), tidy, 100000, world)
        if len(g.nodes()) == n0:
            return g


def shard_replicated_operators(g, world: int, rules):
    """Apply the sample-dim (dim 0) partition rules to every operator whose activations are still unsharded,
    then cancel the Combine/Repartition pairs that meet."""
    weight_slots = ("WEIGHT", "BIAS", "GAMMA", "BETA", "FILTER", "INPUT_BIAS", "OUTPUT_BIAS")

    def unsharded(graph):
        def pred(n):
            if n["type"] in ("INPUT", "WEIGHT") or core.is_parallel_op(n["type"]):
                return False
            acts = [graph.shape(tuple(v)) for s, v in n["inputs"] if s not in weight_slots]
            outs = [o[1] for o in n["outputs"]]
            return all(sh.total_degree == 1 for sh in acts + outs) and all(sh.sizes[0] % world == 0 for sh in acts + outs)
        return pred

    for r in data_parallel_rules(rules, world):
        g = apply_where(g, r, unsharded(g), world)
    return core.apply_rules_exhaustively(g, cancellation_rules(rules), 100000, world)


def rule_families(rules, world: int) -> List[List[int]]:
    """Groups of rule indices that the Unity search may apply as one move: for every degree that divides the machine,
    all rules that shard the sample dimension that many ways."""
    names = [r.name for r in rules]
    fams = []
    d = 2
    while d <= world:
        if world % d == 0:
            members = {r.name for r in data_parallel_rules(rules, d)}
            fam = [i for i, n in enumerate(names) if n in members]
            if fam:
                fams.append(fam)
        d *= 2
    return fams


def optimize(cg, machine=None, *, world: Optional[int] = None, algorithm: str = "unity", budget: int = 0, alpha: float = 1.05,
             estimator=None, rules=None, seed: int = 0, mcmc_iterations: int = 200, mcmc_temperature: float = 0.02,
             substitution_frequency: float = 0.2, time_limit_s: float = 120.0, only_data_parallel: bool = False,
             enable_parameter_parallel: bool = True, enable_attribute_parallel: bool = True, score_hybrid: bool = False,
             start: str = "best_template") -> dict:
    """Search a strategy.  Returns ``{"pcg", "mapped_pcg", "runtime_ms", "memory_bytes", "stats", "candidates"}``.

    The hand-built templates (single device, data parallel, tensor parallel, table parallel) are always scored.  With
    ``budget > 0`` the Unity (or MCMC) search then runs from ``start``: ``"best_template"`` (the cheapest template) or
    ``"serial"`` (the unparallelised graph, as the reference's search starts,
    lib/compiler/src/compiler/unity_algorithm/unity_algorithm.cc:51-146); the cheaper of the search's result and the best
    template is returned.  ``mcmc_temperature`` is a fraction of the starting cost."""
    if machine is None:
        machine = machine_for(world or 1)
    W = machine.num_devices
    estimator = estimator or core.CostEstimator(machine)
    rules = rules or core.get_substitution_set(machine)
    t0 = time.time()
    base = core.pcg_from_computation_graph(cg)
    cands: Dict[str, object] = {"single_device": base}
    if W > 1:
        cands[f"dp{W}"] = data_parallel_strategy(cg, W, rules)
        if not only_data_parallel and algorithm != "data_parallel" and enable_parameter_parallel:
            try:
                cands[f"tp{W}"] = tensor_parallel_strategy(cg, W, rules)
            except Exception:  # a model without the pattern simply has no such candidate
                pass
            if has_stacked_embeddings(cg):
                cands[f"dp{W}+tables_mp{W}"] = table_parallel_strategy(cg, W, rules)
    # data x tensor parallel meshes (the executor runs them on a dp x tp device mesh)
    if W >= 4 and f"tp{W}" in cands and not only_data_parallel and (algorithm in ("unity", "mcmc") or "xtp" in algorithm):
        tp = 2
        while tp < W:
            if W % tp == 0:
                try:
                    cands[f"dp{W // tp}xtp{tp}"] = hybrid_strategy(cg, W // tp, tp, rules)
                except Exception:
                    pass
            tp *= 2
    scored = {k: core.evaluate_pcg(g, machine, estimator) for k, g in cands.items()}
    if algorithm == "data_parallel" or only_data_parallel:
        best_name = f"dp{W}" if W > 1 else "single_device"
    elif algorithm == "tensor_parallel":
        best_name = f"tp{W}" if f"tp{W}" in scored else min(scored, key=lambda k: scored[k]["runtime_ms"])
    elif algorithm == "table_parallel":
        best_name = f"dp{W}+tables_mp{W}" if f"dp{W}+tables_mp{W}" in scored else min(scored, key=lambda k: scored[k]["runtime_ms"])
    elif algorithm in scored:   # a template by name, e.g. "dp2xtp2": the mesh strategy as it is
        best_name = algorithm
    else:
        best_name = min(scored, key=lambda k: scored[k]["runtime_ms"])
    best = scored[best_name]
    template_best = best
    stats = {"candidates": {k: v["runtime_ms"] for k, v in scored.items()}, "seed_strategy": best_name}
    origin = scored["single_device"] if start == "serial" else best
    stats["search_start"] = "serial" if start == "serial" else best_name
    if algorithm == "unity" and budget > 0 and W > 1:
        use = rules if not only_data_parallel else data_parallel_rules(rules, W) + cancellation_rules(rules)
        use = filter_rules(use, enable_parameter_parallel, enable_attribute_parallel)
        r = core.unity_search(origin["pcg"], machine, estimator, use, alpha, budget, 100000, time_limit_s, True, True,
                              rule_families(use, W))
        stats["unity"] = dict(r["stats"], runtime_ms=r["runtime_ms"])
        if r["runtime_ms"] < best["runtime_ms"]:
            best = r
            stats["seed_strategy"] = ("serial" if start == "serial" else stats["seed_strategy"]) + "+unity"
    elif algorithm == "mcmc" and W > 1:
        r = core.mcmc_search(origin["pcg"], machine, estimator, filter_rules(rules, enable_parameter_parallel, enable_attribute_parallel),
                             mcmc_temperature, mcmc_iterations, substitution_frequency, seed, True)
        stats["mcmc"] = r["stats"]
        # MCMC scores with the simulator; re-score with the mapping DP for a comparable number
        rescored = core.evaluate_pcg(r["pcg"], machine, estimator)
        if rescored["runtime_ms"] < best["runtime_ms"]:
            best = rescored
            stats["seed_strategy"] += "+mcmc"
    stats["search_seconds"] = time.time() - t0
    out = dict(best)
    out["stats"] = stats
    # what to run if the executor cannot lower a strategy the search composed itself
    out["template_mapped_pcg"] = template_best["mapped_pcg"] if best is not template_best else None
    return out


def choose_strategy(cg, world: int, config, estimator=None) -> Tuple[object, dict]:
    """Strategy for `world` ranks under an FFConfig: imported from a file if given, searched otherwise."""
    if getattr(config, "import_strategy_file", None):
        with open(config.import_strategy_file) as f:
            return core.Graph.from_v1(f.read()), {"imported": config.import_strategy_file}
    algo = getattr(config, "search_algorithm", "unity")
    rules, extra = None, {}
    path = getattr(config, "substitution_json_path", None)
    if path:
        # legacy TASO-format rule collection (the reference's --substitution-json): the rules that convert are added
        # to the generated set, so the templates still find their rules by name and the search can apply the rest
        with open(path) as f:
            legacy, st = core.load_legacy_rules(f.read())
        rules = list(core.get_substitution_set(machine_for(world))) + [r for r in legacy if r.is_valid()]
        extra = {"substitution_json": {"path": path, "rules_in_file": st["num_rules"], "rules_loaded": st["num_converted"]}}
    r = optimize(cg, world=world, algorithm=algo, budget=getattr(config, "search_budget", 0),
                 alpha=getattr(config, "search_alpha", 1.05), seed=getattr(config, "seed", 0),
                 time_limit_s=getattr(config, "search_time_limit_s", 60.0), start=getattr(config, "search_start", "best_template"),
                 only_data_parallel=getattr(config, "only_data_parallel", False), rules=rules, estimator=estimator,
                 enable_parameter_parallel=getattr(config, "enable_parameter_parallel", True),
                 enable_attribute_parallel=getattr(config, "enable_attribute_parallel", True),
                 score_hybrid=getattr(config, "score_hybrid_strategies", False))
    stats = dict(r["stats"])
    stats.update(extra)
    if r.get("template_mapped_pcg") is not None:
        stats["_template_strategy"] = r["template_mapped_pcg"]
    return r["mapped_pcg"], stats
