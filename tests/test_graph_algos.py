"""Digraph algorithms, SP decomposition and SP-ization (reference: lib/utils/test/src/utils/graph/**)."""
import random

from flexflow_train_b200 import _ffcore as c


def G(edges, nodes=None):
    ns = sorted(set(x for e in edges for x in e) | set(nodes or []))
    return c.DiGraph(ns, edges)


def test_topological_ordering_and_acyclicity():
    g = G([(0, 1), (1, 2), (0, 2), (2, 3)])
    order = c.topological_ordering(g)
    assert order.index(0) < order.index(1) < order.index(2) < order.index(3)
    assert c.is_acyclic(g) and not c.is_acyclic(G([(0, 1), (1, 0)]))


def test_transitive_closure_and_reduction():
    g = G([(0, 1), (1, 2), (0, 2), (2, 3), (0, 3)])
    red = c.transitive_reduction(g)
    assert sorted(red.edges()) == [(0, 1), (1, 2), (2, 3)]
    clo = c.transitive_closure(g)
    assert sorted(clo.edges()) == [(0, 1), (0, 2), (0, 3), (1, 2), (1, 3), (2, 3)]


def test_dominators_lca_components_longest_path():
    g = G([(0, 1), (0, 2), (1, 3), (2, 3), (3, 4)])
    dom = c.get_dominators(g)
    assert dom[3] == {0, 3} and dom[4] == {0, 3, 4}
    pdom = c.get_post_dominators(g)
    assert pdom[0] == {0, 3, 4}
    assert c.get_imm_dominator(g, 3) == 0 and c.get_imm_dominator(g, 0) is None
    assert c.get_lowest_common_ancestor(g, {1, 2}) == 0
    assert c.get_longest_path_lengths_from_root(g) == {0: 0, 1: 1, 2: 1, 3: 2, 4: 3}
    comps = c.get_weakly_connected_components(G([(0, 1), (2, 3)], [4]))
    assert sorted(sorted(s) for s in comps) == [[0, 1], [2, 3], [4]]
    assert c.is_2_terminal_dag(g) and not c.is_2_terminal_dag(G([(0, 2), (1, 2)]))
    assert c.get_descendants(g, 1) == {3, 4} and c.get_ancestors(g, 3) == {0, 1, 2}


def test_sp_decomposition_of_sp_graphs():
    assert c.get_series_parallel_decomposition(G([(0, 1), (1, 2)])) == ("S", [0, 1, 2])
    t = c.get_series_parallel_decomposition(G([(0, 1), (0, 2), (1, 3), (2, 3)]))
    assert t[0] == "S" and t[1][0] == 0 and t[1][2] == 3 and t[1][1][0] == "P" and sorted(t[1][1][1]) == [1, 2]
    # transitive edges do not matter
    assert c.get_series_parallel_decomposition(G([(0, 1), (1, 2), (0, 2)])) == ("S", [0, 1, 2])
    # the N-graph is the canonical non-SP graph
    assert c.get_series_parallel_decomposition(G([(0, 2), (0, 3), (1, 3)])) is None


def test_binary_sp_trees_and_json():
    t = ("S", [0, ("P", [1, 2, 3]), 4])
    for f in (c.sp_balanced_binary, c.sp_left_associative_binary, c.sp_right_associative_binary):
        b = f(t)
        assert sorted(c.sp_nodes(b)) == [0, 1, 2, 3, 4]
        j = c.sp_to_json(b)
        assert j["type"] in ("series", "parallel") and {"left_child", "right_child"} <= set(j)
        assert c.sp_normalize(c.sp_from_json(j)) == c.sp_normalize(t) or sorted(c.sp_nodes(c.sp_from_json(j))) == [0, 1, 2, 3, 4]
    assert c.sp_to_json(7) == {"type": "leaf", "value": 7}
    assert c.sp_work_cost(t, {1: 2.0}) == 6.0 and c.sp_critical_path_cost(t, {1: 2.0}) == 4.0


def _random_dag(n, p, seed):
    rnd = random.Random(seed)
    edges = [(i, j) for i in range(n) for j in range(i + 1, n) if rnd.random() < p]
    return G(edges, range(n))


def test_sp_ization_preserves_dependencies_on_random_dags():
    for seed in range(12):
        g = _random_dag(9, 0.3, seed)
        for algo in (c.naive_stratum_sync_sp_ization, c.escribano_sp_ization, lambda d: c.work_duplicating_sp_ization(d, False),
                     lambda d: c.work_duplicating_sp_ization(d, True), lambda d: c.flexible_sp_ization(d, {})):
            t = algo(g)
            assert set(c.sp_nodes(t)) == set(g.nodes())
            assert c.sp_preserves_dependencies(t, g), (seed, t)


def test_sp_ization_quality_ordering():
    g = G([(0, 2), (0, 3), (1, 3)])  # N graph
    naive = c.naive_stratum_sync_sp_ization(g)
    dup = c.work_duplicating_sp_ization(g, False)
    assert c.sp_critical_path_cost(naive, {}) == 2.0
    assert c.sp_work_cost(dup, {}) >= c.sp_work_cost(naive, {})  # duplication trades work for dependencies
    assert len(c.sp_nodes(naive)) == 4 and len(c.sp_nodes(dup)) == 5


def test_model_graphs_are_series_parallel_after_preprocessing():
    for name in ("transformer", "bert", "split_test", "mlp", "dlrm", "candle_uno"):
        g = c.build_model(name, {"batch_size": 4})
        tree, exact = c.get_graph_sp_decomposition(g)
        assert exact, name
        assert set(c.sp_nodes(tree)) == set(g.node_ids())
