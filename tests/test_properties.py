"""Property-based tests (hypothesis) of the graph library, the SP machinery and parallel shape inference, plus a
hand-written golden file of the v1 format.  The reference tests these layers with rapidcheck generators
(lib/utils/test/src/utils/graph/**, lib/op-attrs/test/src/op-attrs/ops/*.cc); the properties here are the same kind:
invariants that must hold for every input, checked on random ones."""
import json

import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from flexflow_train_b200 import _ffcore as core

SETTINGS = dict(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])


# ---------------------------------------------------------------- random DAGs
@st.composite
def dags(draw, max_nodes=12):
    n = draw(st.integers(2, max_nodes))
    edges = []
    for b in range(1, n):
        for a in range(b):
            if draw(st.booleans()) and draw(st.integers(0, 2)) == 0:
                edges.append((a, b))
    return core.DiGraph(list(range(n)), edges)


def _reach(g):
    order = core.topological_ordering(g)
    r = {n: {n} for n in order}
    for n in reversed(order):
        for s in g.successors(n):
            r[n] |= r[s]
    return r


@given(dags())
@settings(**SETTINGS)
def test_transitive_reduction_keeps_reachability_and_is_minimal(g):
    red = core.transitive_reduction(g)
    assert _reach(red) == _reach(g)
    assert set(red.edges()) <= set(g.edges())
    for (a, b) in red.edges():   # removing any kept edge loses a path
        smaller = core.DiGraph(red.nodes(), [e for e in red.edges() if e != (a, b)])
        assert b not in _reach(smaller)[a]
    clo = core.transitive_closure(g)
    assert {(a, b) for a, rs in _reach(g).items() for b in rs if a != b} == set(clo.edges())


@given(dags())
@settings(**SETTINGS)
def test_topological_order_and_dominators(g):
    order = core.topological_ordering(g)
    pos = {n: i for i, n in enumerate(order)}
    assert sorted(order) == sorted(g.nodes()) and all(pos[a] < pos[b] for a, b in g.edges())
    dom = core.get_dominators(g)
    for n in g.nodes():
        assert n in dom[n]
        preds = g.predecessors(n)
        if preds:   # a node's dominators are itself plus what dominates all of its predecessors
            common = set.intersection(*[set(dom[p]) for p in preds])
            assert set(dom[n]) == common | {n}


@given(dags(10))
@settings(**SETTINGS)
def test_every_sp_ization_preserves_the_dependencies_of_the_dag(g):
    for tree in (core.naive_stratum_sync_sp_ization(g), core.escribano_sp_ization(g),
                 core.work_duplicating_sp_ization(g, coalesce=True), core.work_duplicating_sp_ization(g, coalesce=False)):
        assert core.sp_preserves_dependencies(tree, g)
        assert set(core.sp_nodes(tree)) == set(g.nodes())
    exact = core.get_series_parallel_decomposition(g)
    if exact is not None:   # an SP graph decomposes without adding or duplicating anything
        assert sorted(core.sp_nodes(exact)) == sorted(g.nodes())
        assert _reach(core.digraph_from_sp(exact)) == _reach(core.transitive_reduction(g))


# ---------------------------------------------------------------- random SP trees
@st.composite
def sp_trees(draw, depth=3, counter=None):
    counter = counter if counter is not None else [0]
    if depth == 0 or draw(st.integers(0, 3)) == 0:
        counter[0] += 1
        return counter[0] - 1
    kind = draw(st.sampled_from(["S", "P"]))
    k = draw(st.integers(2, 3))
    return (kind, [draw(sp_trees(depth - 1, counter)) for _ in range(k)])


@given(sp_trees())
@settings(**SETTINGS)
def test_decomposing_the_graph_of_an_sp_tree_gives_the_tree_back(tree):
    norm = core.sp_normalize(tree)
    if not isinstance(norm, tuple):
        return
    g = core.digraph_from_sp(norm)
    back = core.get_series_parallel_decomposition(g)
    assert back is not None
    assert _reach(core.digraph_from_sp(back)) == _reach(core.transitive_reduction(g))
    for binary in (core.sp_balanced_binary(norm), core.sp_left_associative_binary(norm), core.sp_right_associative_binary(norm)):
        assert sorted(core.sp_nodes(binary)) == sorted(core.sp_nodes(norm))
        assert _reach(core.digraph_from_sp(binary)) == _reach(g)
        assert core.sp_from_json(core.sp_to_json(binary)) == binary
    cost = {n: float(n % 5 + 1) for n in core.sp_nodes(norm)}
    assert core.sp_critical_path_cost(norm, cost) <= core.sp_work_cost(norm, cost) + 1e-9


# ---------------------------------------------------------------- parallel shapes
@given(st.integers(1, 4), st.integers(1, 6), st.integers(1, 6), st.sampled_from([1, 2, 4]), st.sampled_from([1, 2, 4]), st.integers(0, 1))
@settings(**SETTINGS)
def test_repartition_then_combine_is_the_identity_on_shapes_and_linear_follows_the_degrees(b, m, k, d0, d1, bias):
    rows, cols, out = 8 * b, 8 * m, 8 * k
    gb = core.GraphBuilder(parallel=True)
    x = gb.create_input([rows, cols], name="x")
    p = gb.parallel_partition(x, 0, d0)
    sh = gb.shape(p)
    assert list(sh.sizes) == [rows, cols] and list(sh.degrees) == [d0, 1] and list(sh.piece_sizes) == [rows // d0, cols]
    q = gb.parallel_combine(p, 0, d0)
    assert gb.shape(q) == gb.shape(x)
    r = gb.parallel_replicate(p, d1)
    assert gb.shape(r).discard_copy_degree == d1 and gb.shape(r).total_degree == d0 * d1
    y = gb.dense(p, out, None, bool(bias), None, None, "fc")
    ysh = gb.shape(y)
    assert list(ysh.sizes) == [rows, out] and ysh.degrees[0] == d0 and ysh.sum_degree == 1
    # the weight the builder created for the sample-parallel Linear is replicated d0 ways
    w = [n for n in gb.graph.nodes() if n["type"] == "WEIGHT" and n["name"] == "fc.weight"][0]
    final = w["id"]
    while True:
        succ = [s for s in gb.graph.successors(final) if core.is_parallel_op(gb.graph.node_type(s))]
        if not succ:
            break
        final = succ[0]
    wsh = gb.graph.node(final)["outputs"][0][1]
    assert list(wsh.sizes) == [out, cols] and wsh.total_degree == d0


# ---------------------------------------------------------------- v1 golden file
GOLDEN_V1 = {
    "raw_graph": {
        "node_labels": [
            [0, {"op_attrs": {"type": "input", "value": {"tensor_shape": {"dims": {"ff_ordered": [4, 8]}, "data_type": "FLOAT"}}}, "name": "x"}],
            [1, {"op_attrs": {"type": "weight", "value": {"tensor_shape": {"dims": {"ff_ordered": [3, 8]}, "data_type": "FLOAT"},
                                                           "initializer": {"type": "zero", "value": {}}}}, "name": "fc.weight"}],
            [2, {"op_attrs": {"type": "linear", "value": {"out_channels": 3, "use_bias": False, "data_type": "FLOAT", "activation": "RELU",
                                                           "regularizer": None}}, "name": "fc"}],
        ],
        "output_labels": [
            [{"node": 0, "slot_name": "OUTPUT"}, {"shape": {"dims": {"ff_ordered": [4, 8]}, "data_type": "FLOAT"}, "create_grad": "NO"}],
            [{"node": 1, "slot_name": "OUTPUT"}, {"shape": {"dims": {"ff_ordered": [3, 8]}, "data_type": "FLOAT"}, "create_grad": "YES"}],
            [{"node": 2, "slot_name": "OUTPUT"}, {"shape": {"dims": {"ff_ordered": [4, 3]}, "data_type": "FLOAT"}, "create_grad": "YES"}],
        ],
        "graph": {
            "nodes": [0, 1, 2],
            "edges": [{"srcNode": 0, "srcSlot": "OUTPUT", "dstNode": 2, "dstSlot": "INPUT"},
                      {"srcNode": 1, "srcSlot": "OUTPUT", "dstNode": 2, "dstSlot": "WEIGHT"}],
            "outputs": [{"node": 0, "slot_name": "OUTPUT"}, {"node": 1, "slot_name": "OUTPUT"}, {"node": 2, "slot_name": "OUTPUT"}],
        },
    }
}


def test_v1_reader_accepts_a_hand_written_file_with_the_reference_field_names():
    """Field names of lib/pcg/include/pcg/file_format/v1/graphs/*.dtg.toml (raw_graph / node_labels / output_labels /
    graph{nodes, edges{srcNode, srcSlot, dstNode, dstSlot}, outputs{node, slot_name}}), maps as [key, value] pair lists,
    FFOrdered as {"ff_ordered": [...]}, optionals as null, enums as their value names, variants as {type, value}: written
    here by hand, not produced by this repository's writer."""
    g = core.Graph.from_v1(json.dumps(GOLDEN_V1))
    nodes = {n["id"]: n for n in g.nodes()}
    assert [nodes[i]["type"] for i in (0, 1, 2)] == ["INPUT", "WEIGHT", "LINEAR"]
    assert nodes[2]["attrs"]["out_channels"] == 3 and nodes[2]["attrs"]["activation"] == "RELU" and nodes[2]["attrs"]["use_bias"] is False
    assert dict((s, tuple(v)) for s, v in nodes[2]["inputs"]) == {"INPUT": (0, "OUTPUT"), "WEIGHT": (1, "OUTPUT")}
    assert list(g.shape((2, "OUTPUT")).sizes) == [4, 3]
    # and the writer emits the same document (key for key) for this graph
    assert json.loads(g.to_v1_string()) == GOLDEN_V1


# ------------------------------------------------------------------------------------------ dataflow graphs
def _random_dataflow(data, n_inputs, n_nodes):
    """Builds an open dataflow graph from hypothesis draws; returns (graph, recipe) where recipe lets the same graph be
    rebuilt with its nodes added in another order."""
    d = core.dataflow
    g = d.OpenDataflowGraph()
    values = [g.add_input() for _ in range(n_inputs)]
    recipe = []
    for _ in range(n_nodes):
        k = data.draw(st.integers(0, min(3, len(values))))
        ins = [values[data.draw(st.integers(0, len(values) - 1))] for _ in range(k)]
        n_out = data.draw(st.integers(1, 2))
        node, outs = g.add_node(ins, n_out)
        recipe.append((ins, n_out, node))
        values.extend(outs)
    return g, recipe


@settings(max_examples=40, deadline=None)
@given(st.data())
def test_dataflow_graph_invariants(data):
    d = core.dataflow
    n_inputs = data.draw(st.integers(0, 3))
    g, recipe = _random_dataflow(data, n_inputs, data.draw(st.integers(1, 7)))
    nodes = sorted(g.get_nodes())
    assert len(nodes) == len(recipe)
    # every operand is an earlier value; uses and inputs mirror each other
    order = g.topological_ordering()
    pos = {n: i for i, n in enumerate(order)}
    for ins, n_out, node in recipe:
        assert g.get_inputs(node) == ins and len(g.get_outputs(node)) == n_out
        for slot, v in enumerate(ins):
            assert (node, slot) in g.get_uses(v)
            if v[0] != "input":
                assert pos[v[0]] < pos[node]
    used = {tuple(v) for ins, _, _ in recipe for v in ins}
    assert sorted(g.get_unused_outputs()) == sorted(o for _, _, node in recipe for o in g.get_outputs(node) if tuple(o) not in used)
    # a graph is isomorphic to itself, and the map is the identity when every node is distinguishable by position
    m = d.find_dataflow_isomorphism(g, g)
    assert m is not None and sorted(m) == nodes and sorted(m.values()) == nodes
    # copies are independent
    h = g.copy()
    h.add_node([], 1)
    assert len(h.get_nodes()) == len(nodes) + 1 and len(g.get_nodes()) == len(nodes)
    assert d.find_dataflow_isomorphism(g, h) is None


@settings(max_examples=40, deadline=None)
@given(st.data())
def test_open_subgraph_keeps_structure_and_cuts_the_rest_into_inputs(data):
    d = core.dataflow
    g, recipe = _random_dataflow(data, data.draw(st.integers(0, 2)), data.draw(st.integers(2, 7)))
    nodes = sorted(g.get_nodes())
    keep = {n for n in nodes if data.draw(st.booleans())} or {nodes[0]}
    sub, node_of, input_of = d.get_open_subgraph(g, keep)
    assert set(node_of) == keep and len(sub.get_nodes()) == len(keep)
    outside = {}
    for gi, v in input_of:
        outside[tuple(gi)] = tuple(v) if not isinstance(v, tuple) else v
    # distinct outside values get distinct graph inputs
    assert len(set(outside.values())) == len(outside)
    for n in keep:
        ins_full = g.get_inputs(n)
        ins_sub = sub.get_inputs(node_of[n])
        assert len(ins_full) == len(ins_sub)
        for vf, vs in zip(ins_full, ins_sub):
            if vf[0] != "input" and vf[0] in keep:
                assert vs == (node_of[vf[0]], vf[1])           # an edge inside the set stays an edge
            else:
                assert vs[0] == "input" and outside[tuple(vs)] == tuple(vf)   # a cut value became this graph input
    # taking everything changes nothing but the numbering
    whole, _, ins = d.get_open_subgraph(g, set(nodes))
    assert d.find_dataflow_isomorphism(g, whole) is not None or len(g.get_graph_inputs()) != len(whole.get_graph_inputs())
