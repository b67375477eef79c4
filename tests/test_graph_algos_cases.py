"""Digraph algorithms on the hand-worked cases of lib/utils/test/src/utils/graph/digraph/algorithms/*.cc (transitive
reduction / closure, dominators, post-dominators, longest paths, components, lowest common ancestors) and against a brute-force
oracle on random DAGs."""
import itertools
import random

import pytest

from flexflow_train_b200 import _ffcore as c


def G(edges, n=None):
    ns = sorted(set(x for e in edges for x in e) | set(range(n or 0)))
    return c.DiGraph(ns, edges)


@pytest.mark.parametrize("n,edges,kept", [
    (3, [(0, 1), (1, 2), (0, 2)], [(0, 1), (1, 2)]),
    (6, [(0, 1), (1, 2), (2, 3), (0, 3)], [(0, 1), (1, 2), (2, 3)]),
    (6, [(0, 1), (1, 2), (2, 3), (3, 4), (0, 3), (1, 4)], [(0, 1), (1, 2), (2, 3), (3, 4)]),
    (4, [(0, 1), (0, 2), (1, 3), (2, 3)], [(0, 1), (0, 2), (1, 3), (2, 3)]),            # a diamond has nothing to remove
    (5, [(0, 1), (0, 2), (1, 3), (2, 3), (0, 3), (3, 4), (0, 4), (1, 4)], [(0, 1), (0, 2), (1, 3), (2, 3), (3, 4)]),
    (4, [], []),
])
def test_transitive_reduction_cases(n, edges, kept):
    r = c.transitive_reduction(G(edges, n))
    assert sorted(r.edges()) == sorted(kept) and sorted(r.nodes()) == list(range(n))


@pytest.mark.parametrize("edges,closure", [
    ([(0, 1), (1, 2), (2, 3)], [(0, 1), (0, 2), (0, 3), (1, 2), (1, 3), (2, 3)]),
    ([(0, 1), (0, 2)], [(0, 1), (0, 2)]),
    ([(0, 2), (1, 2), (2, 3), (2, 4)], [(0, 2), (0, 3), (0, 4), (1, 2), (1, 3), (1, 4), (2, 3), (2, 4)]),
])
def test_transitive_closure_cases(edges, closure):
    assert sorted(c.transitive_closure(G(edges)).edges()) == sorted(closure)


def test_dominators_on_a_graph_with_a_join_and_a_side_entrance():
    #      0 -> 1 -> 3 -> 4
    #      0 -> 2 -> 3        5 -> 4   (a second source: only 4 and 5 itself are reachable from it)
    g = G([(0, 1), (0, 2), (1, 3), (2, 3), (3, 4), (5, 4)])
    dom = c.get_dominators(g)
    assert dom[0] == {0} and dom[1] == {0, 1} and dom[2] == {0, 2} and dom[3] == {0, 3}
    assert dom[4] == {4}      # reachable from two sources: no other node lies on every path
    pdom = c.get_post_dominators(g)
    assert pdom[0] == {0, 3, 4} and pdom[1] == {1, 3, 4} and pdom[5] == {5, 4} and pdom[4] == {4}
    assert c.get_imm_dominator(g, 3) == 0 and c.get_imm_dominator(g, 1) == 0 and c.get_imm_dominator(g, 4) is None


@pytest.mark.parametrize("edges,lengths", [
    ([(0, 1), (1, 2), (0, 2)], {0: 0, 1: 1, 2: 2}),
    ([(0, 1), (0, 2), (1, 3), (2, 3), (3, 4), (0, 4)], {0: 0, 1: 1, 2: 1, 3: 2, 4: 3}),
    ([(0, 1), (1, 2), (2, 3), (0, 3), (3, 4), (1, 4)], {0: 0, 1: 1, 2: 2, 3: 3, 4: 4}),
])
def test_longest_path_lengths_from_root_cases(edges, lengths):
    assert c.get_longest_path_lengths_from_root(G(edges)) == lengths


@pytest.mark.parametrize("edges,n,components", [
    ([(0, 1), (1, 2), (3, 4)], 6, [[0, 1, 2], [3, 4], [5]]),
    ([(0, 2), (1, 2)], 3, [[0, 1, 2]]),
    ([], 3, [[0], [1], [2]]),
])
def test_weakly_connected_components_cases(edges, n, components):
    got = sorted(sorted(s) for s in c.get_weakly_connected_components(G(edges, n)))
    assert got == components


def test_lowest_common_ancestor_cases():
    #        0
    #       / \
    #      1   2
    #     / \   \
    #    3   4   5
    tree = G([(0, 1), (0, 2), (1, 3), (1, 4), (2, 5)])
    assert c.get_lowest_common_ancestor(tree, {3, 4}) == 1
    assert c.get_lowest_common_ancestor(tree, {3, 5}) == 0
    assert c.get_lowest_common_ancestor(tree, {3}) == 3
    assert c.get_lowest_common_ancestor(tree, {1, 4}) == 1


# ------------------------------------------------------------------------------------------ random DAGs vs brute force
def random_dag(rng, n, p):
    return [(i, j) for i in range(n) for j in range(i + 1, n) if rng.random() < p]


def reach(n, edges):
    adj = {i: set() for i in range(n)}
    for a, b in edges:
        adj[a].add(b)
    r = {i: set() for i in range(n)}
    for i in reversed(range(n)):
        for j in adj[i]:
            r[i] |= {j} | r[j]
    return r


@pytest.mark.parametrize("seed", range(12))
def test_closure_reduction_descendants_against_brute_force(seed):
    rng = random.Random(seed)
    n = rng.randint(4, 11)
    edges = random_dag(rng, n, rng.choice([0.2, 0.4, 0.7]))
    g = G(edges, n)
    r = reach(n, edges)
    assert sorted(c.transitive_closure(g).edges()) == sorted((i, j) for i in range(n) for j in r[i])
    red = sorted(c.transitive_reduction(g).edges())
    # an edge survives iff no longer path connects its ends; the reduction keeps reachability
    want = sorted((a, b) for a, b in set(edges) if not any(b in r[k] for k in range(n) if k != b and (a, k) in set(edges)))
    assert red == want
    assert reach(n, red) == r
    for v in range(n):
        assert c.get_descendants(g, v) == r[v]
        assert c.get_ancestors(g, v) == {u for u in range(n) if v in r[u]}
    order = c.topological_ordering(g)
    pos = {v: i for i, v in enumerate(order)}
    assert all(pos[a] < pos[b] for a, b in edges)


@pytest.mark.parametrize("seed", range(8))
def test_dominators_against_path_enumeration(seed):
    rng = random.Random(100 + seed)
    n = rng.randint(4, 8)
    edges = [(0, j) for j in range(1, n) if rng.random() < 0.4] + random_dag(rng, n, 0.35)
    edges = sorted(set(edges) | {(0, j) for j in range(1, n) if not any(b == j for _, b in edges)})   # single source 0
    g = G(edges, n)
    adj = {i: [b for a, b in edges if a == i] for i in range(n)}

    def paths(u, v):
        if u == v:
            return [[v]]
        return [[u] + p for w in adj[u] for p in paths(w, v)]

    dom = c.get_dominators(g)
    for v in range(n):
        ps = paths(0, v)
        assert dom[v] == set.intersection(*[set(p) for p in ps]), (edges, v)


# ------------------------------------------------------------------ series-parallel decomposition of computation graphs
# cases of lib/compiler/test/src/compiler/series_parallel/computation_graph/get_computation_graph_series_parallel_decomposition.cc
from flexflow_train_b200 import _ffcore as core  # noqa: E402
def _norm(t):
    """SP tree with the children of parallel splits as frozensets (their order carries no meaning)."""
    if isinstance(t, int):
        return t
    kind, kids = t
    kids = [_norm(k) for k in kids]
    return (kind, frozenset(kids)) if kind == "P" else (kind, tuple(kids))


def _decompose(b):
    tree, exact = core.get_graph_sp_decomposition(b.graph)
    return _norm(tree), exact


def test_cg_sp_decomposition_empty_graph_and_single_input():
    tree, exact = core.get_graph_sp_decomposition(core.GraphBuilder().graph)
    assert core.sp_nodes(tree) == [] and not exact          # an empty graph has no series-parallel decomposition
    b = core.GraphBuilder()
    x = b.create_input([10, 12], "FLOAT", name="x")
    assert _decompose(b) == (x[0], True)


def test_cg_sp_decomposition_single_operator_with_input_and_weights():
    b = core.GraphBuilder()
    x = b.create_input([10, 12], "FLOAT", name="x")
    y = b.dense(x, 14, None, True)
    ids = {n["id"]: n["type"] for n in b.graph.nodes()}
    weights = [i for i, t in ids.items() if t == "WEIGHT"]
    assert len(weights) == 2
    assert _decompose(b) == (("S", (("P", frozenset([x[0]] + weights)), y[0])), True)


def test_cg_sp_decomposition_shared_input_with_private_weights():
    #   w1   input   w2        series-parallel without the weights, not with them as they stand: inputs and weights are
    #    \   /   \   /         gathered into one parallel stage in front (the decomposition's preprocessing)
    #     op1     op2
    b = core.GraphBuilder()
    x = b.create_input([10, 12], "FLOAT", name="x")
    y1 = b.dense(x, 14, None, False, name="op1")
    y2 = b.dense(x, 14, None, False, name="op2")
    weights = [n["id"] for n in b.graph.nodes() if n["type"] == "WEIGHT"]
    assert len(weights) == 2
    assert _decompose(b) == (("S", (("P", frozenset([x[0]] + weights)), ("P", frozenset([y1[0], y2[0]])))), True)


def test_cg_sp_decomposition_keeps_independent_chains_apart_when_no_preprocessing_is_needed():
    #   input1   input2
    #     |        |
    #    op1      op2
    b = core.GraphBuilder()
    x1 = b.create_input([10, 12], "FLOAT", name="x1")
    x2 = b.create_input([10, 12], "FLOAT", name="x2")
    r1 = b.unary("RELU", x1)
    r2 = b.unary("RELU", x2)
    assert _decompose(b) == (("P", frozenset([("S", (x1[0], r1[0])), ("S", (x2[0], r2[0]))])), True)


def test_cg_sp_decomposition_of_an_n_shaped_graph_is_not_exact():
    #      input            op4 reads op1 and op2, op3 reads op1 only: not series-parallel with or without weights.  The
    #      /   \            reference answers "none" here; this implementation SP-izes and says that it did (exact = False),
    #    op1   op2          and the result still orders every producer before its consumers
    #     | \   |
    #    op3  op4
    b = core.GraphBuilder()
    x = b.create_input([10, 12], "FLOAT", name="x")
    o1 = b.unary("RELU", x)
    o2 = b.unary("RELU", x)
    o3 = b.unary("RELU", o1)
    o4 = b.binary("EW_ADD", o1, o2)
    tree, exact = core.get_graph_sp_decomposition(b.graph)
    assert not exact and set(core.sp_nodes(tree)) >= {x[0], o1[0], o2[0], o3[0], o4[0]}
    order = core.sp_nodes(tree)                      # leaves in series order: every producer comes before its consumers
    first = {n: order.index(n) for n in set(order)}
    for a_, b_ in ((x[0], o1[0]), (x[0], o2[0]), (o1[0], o3[0]), (o1[0], o4[0]), (o2[0], o4[0])):
        assert first[a_] < max(i for i, n in enumerate(order) if n == b_)


# ------------------------------------------------------------------ more digraph algorithms
from hypothesis import given, settings, strategies as st  # noqa: E402
def _dg(edges, nodes=()):
    g = c.DiGraph()
    for n in nodes:
        g.add_node(n)
    for a, b in edges:
        g.add_edge(a, b)
    return g


def test_apply_contraction_reference_case():
    # lib/utils/test/src/utils/graph/digraph/algorithms/apply_contraction.cc
    g = _dg([(0, 1), (0, 2), (0, 4), (1, 3), (2, 4), (3, 0), (3, 4), (3, 5), (4, 5)])
    r = c.apply_contraction(g, {0: 3, 3: 2, 2: 2, 1: 4})
    assert sorted(r.nodes()) == [2, 4, 5]
    assert sorted(r.edges()) == [(2, 2), (2, 4), (2, 5), (4, 2), (4, 5)]
    one = c.contract_node(_dg([(0, 1), (1, 2)]), 1, 0)
    assert sorted(one.nodes()) == [0, 2] and sorted(one.edges()) == [(0, 0), (0, 2)]
    with pytest.raises(Exception):
        c.apply_contraction(g, {0: 1, 1: 0})


def test_flipped_and_dominator_variants():
    g = _dg([(0, 1), (0, 2), (1, 3), (2, 3), (3, 4)])
    assert sorted(c.flipped(g).edges()) == [(1, 0), (2, 0), (3, 1), (3, 2), (4, 3)]
    strict = c.get_strict_dominators(g)
    assert strict[0] == set() and strict[3] == {0} and strict[4] == {0, 3}
    assert c.get_imm_dominators_map(g) == {0: None, 1: 0, 2: 0, 3: 0, 4: 3}
    assert c.get_imm_post_dominator(g, 0) == 3 and c.get_imm_post_dominator(g, 4) is None
    assert c.get_imm_post_dominators_map(g) == {0: 3, 1: 3, 2: 3, 3: 4, 4: None}


def test_topological_rank_and_orderings():
    g = _dg([(0, 1), (0, 2), (1, 3), (2, 3), (3, 4), (5, 4)])
    rank = c.calculate_topo_rank(g)
    assert sorted(rank.values()) == list(range(6)) and all(rank[a] < rank[b] for a, b in g.edges())
    assert c.get_node_with_greatest_topo_rank({0, 1, 3}, g) == 3 and c.get_node_with_greatest_topo_rank(set(), g) is None
    assert c.get_topological_ordering_from_starting_node(g, 1) == [1, 3, 4]
    assert c.get_topological_ordering_from_starting_node(g, 4) == [4]
    order = c.get_edge_topological_ordering(g)
    assert sorted(order) == sorted(g.edges()) and [rank[a] for a, _ in order] == sorted(rank[a] for a, _ in order)
    with pytest.raises(Exception):
        c.get_topological_ordering_from_starting_node(_dg([(0, 1), (1, 0)]), 0)


def test_is_tree_and_complete_bipartite():
    assert c.is_tree(_dg([(0, 1), (0, 2), (2, 3)])) and c.is_tree(_dg([], nodes=[7]))
    assert not c.is_tree(_dg([(0, 1), (0, 2), (1, 3), (2, 3)]))          # a diamond: |E| = |V|
    assert not c.is_tree(_dg([(0, 1), (2, 3)]))                          # two roots
    with pytest.raises(Exception):
        c.is_tree(c.DiGraph())
    assert c.is_complete_bipartite_digraph(_dg([(0, 2), (0, 3), (1, 2), (1, 3)]))
    assert not c.is_complete_bipartite_digraph(_dg([(0, 2), (0, 3), (1, 2)]))            # 1 -> 3 is missing
    assert not c.is_complete_bipartite_digraph(_dg([(0, 1), (1, 2)]))                    # a middle node
    assert not c.is_complete_bipartite_digraph(_dg([(0, 1)], nodes=[5]))                 # an isolated node


def test_subgraph_edge_queries_and_dot():
    g = _dg([(0, 1), (0, 2), (1, 3), (2, 3), (3, 4)])
    assert c.get_edges_from_subgraph_to_subgraph(g, {0, 1}, {2, 3}) == {(0, 2), (1, 3)}
    assert c.get_edges_from_subgraph_to_subgraph(g, {4}, {0}) == set()
    with pytest.raises(Exception):
        c.get_edges_from_subgraph_to_subgraph(g, {0, 1}, {1, 2})
    assert c.get_subgraph_outgoing_edges(g, {0, 1}) == {(0, 2), (1, 3)} and c.get_subgraph_successors(g, {0, 1}) == {2, 3}
    assert c.get_subgraph_outgoing_edges(g, {0, 1, 2, 3, 4}) == set()
    dot = c.digraph_as_dot(g)
    assert dot.startswith("digraph {") and dot.count("->") == 5 and 'n3 [label="3"]' in dot


@settings(max_examples=60, deadline=None)
@given(st.integers(2, 9), st.integers(0, 10 ** 6))
def test_dominator_variants_agree_on_random_dags(n, seed):
    rng = random.Random(seed)
    g = _dg([(a, b) for a in range(n) for b in range(a + 1, n) if rng.random() < 0.35] + [(0, k) for k in range(1, n)])
    dom, strict, imm = c.get_dominators(g), c.get_strict_dominators(g), c.get_imm_dominators_map(g)
    for v in g.nodes():
        assert strict[v] == dom[v] - {v}
        if v == 0:
            assert imm[v] is None
        else:
            # the immediate dominator is the strict dominator that every other strict dominator dominates
            assert imm[v] in strict[v] and all(d in dom[imm[v]] for d in strict[v])
    f = c.flipped(c.flipped(g))
    assert sorted(f.edges()) == sorted(g.edges())


# ------------------------------------------------------------------ SP-ization golden cases
def _canon(t):
    """Order-free form of a decomposition: the children of a parallel split are a set."""
    if not isinstance(t, tuple):
        return t
    kind, kids = t
    kids = [_canon(k) for k in kids]
    return (kind, frozenset(kids)) if kind == "P" else (kind, tuple(kids))


def _S(*k):
    return ("S", list(k))


def _P(*k):
    return ("P", list(k))


def _graph_costs(edges, cost):
    """Work and critical path of the graph itself."""
    longest = {}
    order = sorted(cost)  # the cases number their nodes in a topological order
    for n in order:
        longest[n] = cost[n] + max([longest[a] for a, b in edges if b == n], default=0.0)
    return sum(cost.values()), max(longest.values())


_STRATUM_CASES = [
    # lib/utils/test/src/utils/graph/series_parallel/sp_ization/naive_stratum_sync.cc
    ("independent nodes", 4, [], {0: 1, 1: 5, 2: 2, 3: 3}, _P(0, 1, 2, 3), None),
    ("chain", 5, [(0, 1), (1, 2), (2, 3), (3, 4)], {0: 1, 1: 2, 2: 3, 3: 4, 4: 5}, _S(0, 1, 2, 3, 4), None),
    ("two layers, all to all", 5, [(0, 2), (0, 3), (0, 4), (1, 2), (1, 3), (1, 4)],
     {0: 2, 1: 3, 2: 5, 3: 7, 4: 11}, _S(_P(0, 1), _P(2, 3, 4)), None),
    ("barrier lengthens the critical path", 6, [(0, 1), (0, 2), (1, 3), (2, 5), (3, 4), (4, 5)],
     {0: 1, 1: 1, 2: 10, 3: 1, 4: 1, 5: 1}, None, (12.0, 14.0)),
    ("diamond with tail", 6, [(0, 1), (0, 2), (1, 3), (2, 4), (3, 5), (4, 5)],
     {n: 1 for n in range(6)}, _S(0, _P(1, 2), _P(3, 4), 5), None),
]


@pytest.mark.parametrize("name,n,edges,cost,expected,paths", _STRATUM_CASES, ids=[k[0] for k in _STRATUM_CASES])
def test_naive_stratum_sync_golden_cases(name, n, edges, cost, expected, paths):
    g = _dg(edges, range(n))
    cost = {k: float(v) for k, v in cost.items()}
    sp = c.naive_stratum_sync_sp_ization(g)
    if expected is not None:
        assert _canon(sp) == _canon(expected)
    work, critical = _graph_costs(edges, cost)
    assert c.sp_work_cost(sp, cost) == work
    if paths is None:
        assert c.sp_critical_path_cost(sp, cost) == critical
    else:
        assert (critical, c.sp_critical_path_cost(sp, cost)) == paths
    assert c.sp_preserves_dependencies(sp, g)


_ESCRIBANO_CASES = [
    # lib/utils/test/src/utils/graph/series_parallel/sp_ization/escribano_algo.cc
    ("single node", 1, [], 0),
    ("chain", 3, [(0, 1), (1, 2)], _S(0, 1, 2)),
    ("rhombus", 4, [(0, 1), (0, 2), (1, 3), (2, 3)], _S(0, _P(1, 2), 3)),
    ("sample 1", 6, [(0, 1), (0, 2), (1, 2), (1, 3), (2, 4), (3, 4), (3, 5), (4, 5)], _S(0, 1, _P(2, 3), 4, 5)),
    ("diamond without crossing", 6, [(0, 1), (0, 2), (1, 3), (2, 5), (3, 4), (4, 5)], _S(0, _P(_S(1, 3, 4), 2), 5)),
    ("diamond", 6, [(0, 1), (0, 2), (1, 4), (1, 3), (2, 4), (3, 5), (4, 5)], _S(0, _P(1, 2), _P(3, 4), 5)),
    ("sample 2", 10, [(0, 1), (0, 3), (1, 2), (1, 5), (1, 4), (2, 6), (3, 4), (3, 5), (3, 8), (4, 8), (5, 7), (7, 8),
                      (6, 9), (8, 9)],
     _S(0, _P(1, 3), _P(_S(2, 6), _S(_P(_S(5, 7), 4), 8)), 9)),
    # lib/utils/include/utils/graph/series_parallel/sp_ization/index.dox: strata 1 and 2 are joined in two local groups
    ("local joins", 8, [(0, 1), (0, 2), (0, 3), (1, 4), (1, 5), (2, 5), (3, 6), (4, 7), (5, 7), (6, 7)],
     _S(0, _P(_S(_P(1, 2), _P(4, 5)), _S(3, 6)), 7)),
    # several sources and sinks: not in the upstream cases, which want a two-terminal graph
    ("two sources, two sinks", 4, [(0, 2), (1, 2), (1, 3)], _S(_P(0, 1), _P(2, 3))),
    ("independent chains", 4, [(0, 1), (2, 3)], _P(_S(0, 1), _S(2, 3))),
]


@pytest.mark.parametrize("name,n,edges,expected", _ESCRIBANO_CASES, ids=[k[0] for k in _ESCRIBANO_CASES])
def test_escribano_golden_cases(name, n, edges, expected):
    g = _dg(edges, range(n))
    sp = c.escribano_sp_ization(g)
    assert c.sp_preserves_dependencies(sp, g)
    assert sorted(c.sp_nodes(sp)) == list(range(n))
    assert _canon(sp) == _canon(expected)


_SIX_DIAMOND = [(0, 1), (0, 2), (1, 3), (1, 4), (2, 4), (3, 5), (4, 5)]
_APPENDAGE = _SIX_DIAMOND + [(0, 6), (6, 5), (2, 7), (7, 5)]
_PAPER = [(0, 1), (0, 2), (1, 3), (1, 4), (2, 10), (2, 11), (2, 12), (3, 5), (3, 6), (4, 6), (4, 7), (4, 10), (5, 8),
          (6, 8), (6, 9), (7, 8), (8, 17), (9, 17), (10, 16), (11, 16), (12, 13), (12, 14), (13, 15), (14, 15),
          (15, 16), (16, 17)]
_FLEXIBLE_CASES = [
    # lib/utils/test/src/utils/graph/series_parallel/sp_ization/flexible_algo.cc
    ("single node", 1, [], {}, 0),
    ("rhombus", 4, [(0, 1), (0, 2), (1, 3), (2, 3)], {}, _S(0, _P(1, 2), 3)),
    ("chain", 4, [(0, 1), (1, 2), (2, 3)], {}, _S(0, 1, 2, 3)),
    ("six-node diamond, unit costs", 6, _SIX_DIAMOND, {}, _S(0, _P(1, 2), _P(3, 4), 5)),
    ("six-node diamond, heavy 3", 6, _SIX_DIAMOND, {2: 10, 3: 1000}, _S(0, 1, _P(_S(2, 4), 3), 5)),
    ("six-node diamond, heavy 2 and 3", 6, _SIX_DIAMOND, {2: 1000, 3: 1000}, _S(0, _P(_S(1, 3), 2), 4, 5)),
    ("parallel strands", 8, [(0, 1), (0, 2), (1, 3), (2, 4), (3, 5), (4, 6), (5, 7), (6, 7)], {},
     _S(0, _P(_S(1, 3, 5), _S(2, 4, 6)), 7)),
    ("diamond beside a strand", 7, [(0, 1), (0, 2), (1, 3), (1, 4), (2, 4), (3, 6), (4, 6), (0, 5), (5, 6)],
     {2: 100, 3: 100}, _S(0, _P(_S(_P(_S(1, 3), 2), 4), 5), 6)),
    ("appendage, unit costs", 8, _APPENDAGE, {}, _S(0, _P(6, _S(_P(1, 2), _P(3, 4, 7))), 5)),
    ("appendage, weighted", 8, _APPENDAGE, {1: 100, 7: 100}, _S(0, _P(6, _S(2, _P(7, _S(1, _P(3, 4))))), 5)),
    ("cut across unequal depths", 7, [(0, 1), (0, 2), (1, 3), (1, 4), (2, 5), (3, 6), (4, 5), (5, 6)],
     {3: 10, 5: 10}, _S(0, _P(_S(1, 4), 2), _P(3, 5), 6)),
    ("graph from the paper, unit costs", 18, _PAPER + [(10, 9)], {},
     _S(0, _P(_S(1, _P(3, 4)), _S(2, _P(11, 12))), _P(_S(_P(10, 5, 6, 7), _P(8, 9)), _S(_P(13, 14), 15)), 16, 17)),
    ("graph from the paper without 10->9", 18, _PAPER, {}, None),
    ("graph from the paper, mixed costs", 18, _PAPER,
     {1: 3, 2: 5, 3: 3, 4: 5, 5: 3, 6: 5, 8: 5, 9: 5, 10: 3, 11: 3, 13: 3, 14: 3}, None),
]


@pytest.mark.parametrize("name,n,edges,heavy,expected", _FLEXIBLE_CASES, ids=[k[0] for k in _FLEXIBLE_CASES])
def test_flexible_golden_cases(name, n, edges, heavy, expected):
    g = _dg(edges, range(n))
    cost = {k: float(heavy.get(k, 1)) for k in range(n)}
    sp = c.flexible_sp_ization(g, cost)
    assert c.sp_preserves_dependencies(sp, g)
    assert sorted(c.sp_nodes(sp)) == list(range(n))      # no work is duplicated
    if expected is not None:
        assert _canon(sp) == _canon(expected)
    # never worse than closing whole strata
    assert c.sp_critical_path_cost(sp, cost) <= c.sp_critical_path_cost(c.naive_stratum_sync_sp_ization(g), cost)


def test_flexible_picks_the_cut_that_suits_the_costs_on_the_n_graph():
    # a -> c, a -> d, b -> d between a common source 9 and sink 10: each of the three ways of closing the N is best
    # under one of these cost maps (lib/utils/include/utils/graph/series_parallel/sp_ization/index.dox)
    a, b, cc, d = 0, 1, 2, 3
    edges = [(9, a), (9, b), (a, cc), (a, d), (b, d), (cc, 10), (d, 10)]
    for costs, best in (((1, 1, 1, 1), 2.0), ((1, 3, 2, 1), 4.0), ((1, 2, 3, 1), 4.0)):
        g = _dg(edges, [a, b, cc, d, 9, 10])
        cost = {a: costs[0], b: costs[1], cc: costs[2], d: costs[3], 9: 0.0, 10: 0.0}
        sp = c.flexible_sp_ization(g, {k: float(v) for k, v in cost.items()})
        assert c.sp_preserves_dependencies(sp, g)
        assert c.sp_critical_path_cost(sp, {k: float(v) for k, v in cost.items()}) == best


@settings(max_examples=60, deadline=None)
@given(st.integers(2, 14), st.integers(0, 10 ** 6))
def test_escribano_and_flexible_on_random_dags(n, seed):
    # any DAG (several sources, sinks and components included): every dependency kept, every node exactly once,
    # and the locally-joining algorithms never lengthen the critical path beyond whole-stratum barriers
    rng = random.Random(seed)
    edges = random_dag(rng, n, rng.choice([0.15, 0.3, 0.6]))
    g = _dg(edges, range(n))
    cost = {k: float(rng.choice([1, 1, 2, 5, 20])) for k in range(n)}
    unit = {k: 1.0 for k in range(n)}
    esc = c.escribano_sp_ization(g)
    flex = c.flexible_sp_ization(g, cost)
    for sp in (esc, flex):
        assert c.sp_preserves_dependencies(sp, g)
        assert sorted(c.sp_nodes(sp)) == list(range(n))
    assert c.sp_critical_path_cost(esc, unit) <= c.sp_critical_path_cost(c.naive_stratum_sync_sp_ization(g), unit)


def _canon_multi(t):
    """Like _canon but a parallel split may hold equal children more than once (duplicated work)."""
    if not isinstance(t, tuple):
        return t
    kind, kids = t
    kids = [_canon_multi(k) for k in kids]
    return (kind, tuple(sorted(kids, key=repr))) if kind == "P" else (kind, tuple(kids))


_LOPSIDED = [(0, 1), (0, 2), (1, 3), (2, 5), (3, 4), (4, 5)]
_DUPLICATING_CASES = [
    # lib/utils/test/src/utils/graph/series_parallel/sp_ization/work_duplicating_sp_ization.cc
    ("chain", False, 3, [(0, 1), (1, 2)], _S(0, 1, 2)),
    ("rhombus", False, 4, [(0, 1), (0, 2), (1, 3), (2, 3)], _S(_P(_S(0, 1), _S(0, 2)), 3)),
    ("paths of different lengths", False, 6, _LOPSIDED, _S(_P(_S(0, 1, 3, 4), _S(0, 2)), 5)),
    ("rhombus, coalesced", True, 4, [(0, 1), (0, 2), (1, 3), (2, 3)], _S(0, _P(1, 2), 3)),
    ("paths of different lengths, coalesced", True, 6, _LOPSIDED, _S(0, _P(_S(1, 3, 4), 2), 5)),
    ("strands with cross edges, coalesced", True, 6,
     # upstream stops at S(0, 1, P(S(P(2, 3), 4), 3), 5), with node 3 still twice; the factoring here also merges that copy
     [(0, 1), (0, 2), (1, 2), (1, 3), (2, 4), (3, 4), (3, 5), (4, 5)], _S(0, 1, _P(2, 3), 4, 5)),
    ("transitive edges, coalesced", True, 5,
     [(0, 1), (0, 2), (0, 4), (1, 2), (1, 3), (1, 4), (2, 4), (3, 4)], _S(0, 1, _P(2, 3), 4)),
]


@pytest.mark.parametrize("name,coalesce,n,edges,expected", _DUPLICATING_CASES, ids=[k[0] for k in _DUPLICATING_CASES])
def test_work_duplicating_golden_cases(name, coalesce, n, edges, expected):
    g = _dg(edges, range(n))
    sp = c.work_duplicating_sp_ization(g, coalesce)
    assert c.sp_preserves_dependencies(sp, g)
    assert _canon_multi(sp) == _canon_multi(expected)
    # duplication buys an unchanged critical path
    unit = {k: 1.0 for k in range(n)}
    assert c.sp_critical_path_cost(sp, unit) == _graph_costs(edges, unit)[1]


def test_dependencies_are_maintained_cases():
    # lib/utils/test/src/utils/graph/series_parallel/sp_ization/dependencies_are_maintained.cc
    assert c.sp_preserves_dependencies(0, _dg([], [0]))
    chain = _dg([(0, 1), (1, 2)], range(3))
    assert c.sp_preserves_dependencies(_S(0, 1, 2), chain)
    assert not c.sp_preserves_dependencies(_S(0, 2, 1), chain)
    assert not c.sp_preserves_dependencies(_P(0, 1, 2), chain)
    assert not c.sp_preserves_dependencies(_S(0, 1), chain)          # a node is missing
    loose = _dg([], range(3))
    assert c.sp_preserves_dependencies(_P(0, 1, 2), loose)
    assert c.sp_preserves_dependencies(_S(0, 1, 2), loose)          # extra ordering is allowed
    rhombus = _dg([(0, 1), (0, 2), (1, 3), (2, 3)], range(4))
    assert c.sp_preserves_dependencies(_S(0, _P(1, 2), 3), rhombus)
    assert c.sp_preserves_dependencies(_S(0, 1, 2, 3), rhombus)
    assert c.sp_preserves_dependencies(_S(_P(_S(0, 1), _S(0, 2)), 3), rhombus)
    assert not c.sp_preserves_dependencies(_S(_P(0, 1), 2, 3), rhombus)
    diamond = _dg(_SIX_DIAMOND, range(6))
    assert c.sp_preserves_dependencies(_S(0, _P(1, 2), _P(3, 4), 5), diamond)
    assert c.sp_preserves_dependencies(_S(0, _P(_S(1, 3), 2), 4, 5), diamond)
    assert not c.sp_preserves_dependencies(_S(0, _P(_S(1, 3), _S(2, 4)), 5), diamond)   # 1 -> 4 is lost


def test_bridge_out_nodes_cases():
    # lib/utils/test/src/utils/graph/series_parallel/sp_ization/node_role.cc
    g = _dg([(0, 1), (1, 2), (1, 3), (2, 4), (3, 4)], range(5))
    r = c.bridge_out_nodes(g, {1, 2})
    assert sorted(r.nodes()) == [0, 3, 4]
    assert sorted(r.edges()) == [(0, 3), (0, 4), (3, 4)]
    g = _dg([(0, 1), (1, 2), (1, 3)], range(4))
    r = c.bridge_out_nodes(g, set())
    assert sorted(r.nodes()) == sorted(g.nodes()) and sorted(r.edges()) == sorted(g.edges())
    # a dropped source or sink simply goes
    r = c.bridge_out_nodes(g, {0, 3})
    assert sorted(r.nodes()) == [1, 2] and sorted(r.edges()) == [(1, 2)]


_DECOMPOSITION_CASES = [
    # lib/utils/test/src/utils/graph/series_parallel/get_series_parallel_decomposition.cc
    ("single node", 1, [], 0),
    ("two loose nodes", 2, [], _P(0, 1)),
    ("chain", 2, [(0, 1)], _S(0, 1)),
    ("fork", 3, [(0, 1), (0, 2)], _S(0, _P(1, 2))),
    ("two strands", 6, [(0, 1), (0, 2), (1, 3), (2, 4), (3, 5), (4, 5)], _S(0, _P(_S(1, 3), _S(2, 4)), 5)),
    ("all to all", 4, [(0, 2), (0, 3), (1, 2), (1, 3)], _S(_P(0, 1), _P(2, 3))),
    ("N graph", 4, [(0, 2), (1, 2), (1, 3)], None),
    ("needs transitive reduction", 4, [(0, 1), (0, 2), (1, 2), (1, 3), (2, 3)], _S(0, 1, 2, 3)),
]


@pytest.mark.parametrize("name,n,edges,expected", _DECOMPOSITION_CASES, ids=[k[0] for k in _DECOMPOSITION_CASES])
def test_series_parallel_decomposition_golden_cases(name, n, edges, expected):
    sp = c.get_series_parallel_decomposition(_dg(edges, range(n)))
    if expected is None:
        assert sp is None
    else:
        assert _canon(sp) == _canon(expected)


@pytest.mark.parametrize("tree,nodes,edges,sources,sinks", [
    # lib/utils/test/src/utils/graph/series_parallel/digraph_generation.cc
    (_S(1, 2, 3), 3, 2, 1, 1),
    (_P(1, 2, 3), 3, 0, 3, 3),
    (_S(1, _P(2, 3)), 3, 2, 1, 2),
    (_P(_S(1, 2), _S(3, 4)), 4, 2, 2, 2),
    (_S(1, _P(2, 3), 4), 4, 4, 1, 1),
    (_S(_P(_S(_P(1, 2), _P(3, 4), 5), _S(6, 7)), 8), 8, 9, 3, 1),
])
def test_digraph_from_sp_cases(tree, nodes, edges, sources, sinks):
    g = c.digraph_from_sp(tree)
    assert (len(g.nodes()), len(g.edges()), len(g.sources()), len(g.sinks())) == (nodes, edges, sources, sinks)
    if nodes > 1:
        assert _canon(c.get_series_parallel_decomposition(g)) == _canon(tree)     # the two are inverses


def test_sp_ancestors_cases():
    # lib/utils/test/src/utils/graph/series_parallel/get_ancestors.cc
    assert c.sp_ancestors(0, 0) == set()
    assert c.sp_ancestors(_S(0, 1, 2), 2) == {0, 1}
    assert c.sp_ancestors(_P(0, 1, 2), 1) == set()
    assert c.sp_ancestors(_S(0, _P(_S(1, 2), 3)), 2) == {0, 1}
    assert c.sp_ancestors(_S(0, _P(1, 2), 3), 3) == {0, 1, 2}
    sp = _S(0, _P(_S(1, _P(2, 3), 4), _S(5, 6)), 7)
    assert c.sp_ancestors(sp, 4) == {0, 1, 2, 3}
    assert c.sp_ancestors(sp, 3) == {0, 1}
    assert c.sp_ancestors(sp, 6) == {0, 5}
    assert c.sp_ancestors(sp, 7) == {0, 1, 2, 3, 4, 5, 6}
    with pytest.raises(Exception):
        c.sp_ancestors(sp, 99)
    # the tree's own view agrees with the graph it stands for
    g = c.digraph_from_sp(sp)
    for n in range(8):
        assert c.sp_ancestors(sp, n) == set(c.get_ancestors(g, n))


def test_sp_normalize_cases():
    # lib/utils/test/src/utils/graph/series_parallel/normalize_sp_decomposition.cc
    assert c.sp_normalize(1) == 1
    assert c.sp_normalize(_S(1)) == 1
    assert c.sp_normalize(_P(1)) == 1
    assert c.sp_normalize(_S(_P(1), 2)) == _S(1, 2)
    assert _canon(c.sp_normalize(_P(_S(1), 2))) == _canon(_P(1, 2))
    assert _canon(c.sp_normalize(_P(_S(_P(1, 2)), 3, _S()))) == _canon(_P(1, 2, 3))
    assert c.sp_normalize(_S(1, _S(2, _S(3, _P())), 4)) == _S(1, 2, 3, 4)
    with pytest.raises(Exception):
        c.sp_normalize(_S(_P(), _P()))
