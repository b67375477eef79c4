"""Dataflow graph family (open graphs, named slots, labels, subgraphs, isomorphism) and the declarative command-line spec of
the native core.  Models: lib/utils/test/src/utils/graph/dataflow_graph/*, open_dataflow_graph/*, lib/utils/test/src/utils/cli/*."""
import pytest

from flexflow_train_b200 import _ffcore as core
from flexflow_train_b200.bin import export_model_arch

d = core.dataflow


def diamond():
    g = d.OpenDataflowGraph()
    x = g.add_input()
    a, (a0, a1) = g.add_node([x], 2)
    b, (b0,) = g.add_node([a0], 1)
    c, (c0,) = g.add_node([a1, x], 1)
    e, (e0,) = g.add_node([b0, c0], 1)
    return g, x, (a, b, c, e), (a0, a1, b0, c0, e0)


def test_open_dataflow_graph_queries():
    g, x, (a, b, c, e), (a0, a1, b0, c0, e0) = diamond()
    assert sorted(g.get_nodes()) == [a, b, c, e]
    assert g.get_graph_inputs() == [x]
    assert g.get_inputs(c) == [a1, x]
    assert g.get_outputs(a) == [a0, a1]
    assert sorted(g.get_uses(x)) == [(a, 0), (c, 1)]
    assert g.get_unused_outputs() == [e0]
    order = g.topological_ordering()
    assert order.index(a) < order.index(b) < order.index(e) and order.index(c) < order.index(e)
    assert not g.is_closed()
    edges = g.query_edges(dst_nodes={e})
    assert sorted(edges) == [(b0, (e, 0)), (c0, (e, 1))]
    assert g.query_edges(src_nodes={a}, dst_nodes={b}) == [(a0, (b, 0))]


def test_copies_do_not_share_later_changes():
    g, x, nodes, outs = diamond()
    h = g.copy()
    h.add_node([outs[-1]], 1)
    assert len(h.get_nodes()) == 5 and len(g.get_nodes()) == 4


def test_open_subgraph_turns_cut_values_into_inputs():
    g, x, (a, b, c, e), (a0, a1, b0, c0, e0) = diamond()
    sub, node_of, input_of = d.get_open_subgraph(g, {c, e})
    assert len(sub.get_nodes()) == 2
    # c reads a1 and x, e reads b0: three distinct outside values, each bound to one new graph input
    assert {str(v) for _, v in input_of} == {str(a1), str(x), str(b0)}
    assert len(sub.get_graph_inputs()) == 3
    assert set(node_of) == {c, e} and set(node_of.values()) == set(sub.get_nodes())


def test_isomorphism_respects_operand_order():
    g, *_ = diamond()
    h, *_ = diamond()
    m = d.find_dataflow_isomorphism(g, h)
    assert m is not None and sorted(m) == sorted(g.get_nodes())
    # the same shape with e's operands swapped is a different dataflow graph
    k = d.OpenDataflowGraph()
    x = k.add_input()
    a, (a0, a1) = k.add_node([x], 2)
    b, (b0,) = k.add_node([a0], 1)
    c, (c0,) = k.add_node([a1, x], 1)
    k.add_node([c0, b0], 1)
    assert d.find_dataflow_isomorphism(g, k) is None
    # node numbering does not matter
    p = d.OpenDataflowGraph()
    x = p.add_input()
    a, (a0, a1) = p.add_node([x], 2)
    c, (c0,) = p.add_node([a1, x], 1)
    b, (b0,) = p.add_node([a0], 1)
    p.add_node([b0, c0], 1)
    m = d.find_dataflow_isomorphism(g, p)
    assert m is not None and m[1] == 2 and m[2] == 1


def test_kwarg_graph_names_its_slots():
    g = d.KwargDataflowGraph()
    n0, o0 = g.add_node({}, ["out"])
    n1, o1 = g.add_node({}, ["out"])
    n2, o2 = g.add_node({"lhs": o0["out"], "rhs": o1["out"]}, ["sum", "carry"])
    assert g.get_inputs(n2) == {"lhs": (n0, "out"), "rhs": (n1, "out")}
    assert sorted(g.get_output_slots(n2)) == ["carry", "sum"]
    pos = g.positional()  # slots in sorted order become positions
    assert pos.get_inputs(n2) == [(n0, 0), (n1, 0)]
    assert len(pos.get_outputs(n2)) == 2


def test_labelled_graph_keeps_labels_with_structure():
    g = d.LabelledOpenDataflowGraph()
    x = g.add_input({"shape": (4, 8)})
    n, (o,) = g.add_node("relu", [x], [{"shape": (4, 8)}])
    m, (p,) = g.add_node("linear", [o], [{"shape": (4, 2)}])
    assert g.node_label(m) == "linear" and g.value_label(p) == {"shape": (4, 2)} and g.value_label(x) == {"shape": (4, 8)}
    h = g.rewrite_node_labels(lambda node, label: label.upper())
    assert h.node_label(n) == "RELU" and g.node_label(n) == "relu"
    assert h.raw().get_inputs(m) == [o]


# ---------------------------------------------------------------------------------------------- command lines
def spec():
    s = d.empty_cli_spec()
    keys = dict(
        help=d.cli_add_help_flag(s),
        verbose=d.cli_add_flag(s, "verbose", "v", "say more"),
        mode=d.cli_add_positional_argument(s, "mode", ["fast", "slow"], "how to run"),
        path=d.cli_add_positional_argument(s, "path"),
    )
    return s, keys


def test_cli_parse_flags_and_positionals():
    s, k = spec()
    r = d.cli_parse(s, ["prog", "-v", "fast", "out.json"])
    assert d.cli_get_flag(r, k["verbose"]) and not d.cli_get_flag(r, k["help"])
    assert d.cli_get_argument(r, k["mode"]) == "fast" and d.cli_get_argument(r, k["path"]) == "out.json"
    r = d.cli_parse(s, ["prog", "slow", "--verbose", "x"])
    assert d.cli_get_flag(r, k["verbose"]) and d.cli_get_argument(r, k["path"]) == "x"
    r = d.cli_parse(s, ["prog", "slow", "x"])
    assert not d.cli_get_flag(r, k["verbose"])


@pytest.mark.parametrize("argv,msg", [
    (["prog", "fast"], "Not enough positional arguments: found 1, expected 2"),
    (["prog", "fast", "a", "b"], "Too many positional arguments: expected 2"),
    (["prog", "medium", "a"], 'Invalid option for positional argument "mode": "medium"'),
    (["prog", "--loud", "fast", "a"], "Encountered unknown flag --loud"),
])
def test_cli_parse_errors(argv, msg):
    s, _ = spec()
    with pytest.raises(ValueError, match=msg.replace("(", r"\(")):
        d.cli_parse(s, argv)


def test_cli_help_message_layout():
    s, _ = spec()
    text = d.cli_get_help_message("prog", s)
    lines = text.splitlines()
    assert lines[0] == "usage: prog [-h] [-v] {fast,slow} path"
    assert "positional arguments:" in lines and "options:" in lines
    assert "  {fast,slow}    how to run" in lines
    assert "  path" in lines  # no description: the key alone
    assert "  -h, --help     show this help message and exit" in lines
    assert "  -v, --verbose  say more" in lines
    # help is answered without the positionals
    r = d.cli_parse(s, ["prog", "--help"])
    assert r is not None
    # a long key pushes its description to the next line
    t = d.empty_cli_spec()
    d.cli_add_flag(t, "a-very-long-flag-name-indeed", None, "described below")
    out = d.cli_get_help_message("p", t).splitlines()
    assert out[-2] == "  --a-very-long-flag-name-indeed" and out[-1].strip() == "described below" and out[-1].startswith(" " * 24)


def test_export_model_arch_uses_the_native_spec(capsys):
    assert export_model_arch.main(["--help"]) == 0
    out = capsys.readouterr().out
    assert out.startswith("usage: export-model-arch [-h] [--sp-decomposition] [--dot] [--preprocessed-dot] {")
    assert export_model_arch.main(["no_such_model"]) == 2
    assert "Invalid option for positional argument" in capsys.readouterr().err


# ------------------------------------------------------------------ algorithms over open dataflow graphs
def test_source_nodes_unused_inputs_and_edges_between_nodes():
    g, x, (a, b, c, e), (a0, a1, b0, c0, e0) = diamond()
    assert d.get_source_nodes(g) == {a}                       # only `a` reads nothing but graph inputs
    assert d.get_unused_open_dataflow_graph_inputs(g) == set()
    y = g.add_input()
    assert d.get_unused_open_dataflow_graph_inputs(g) == {y[1]}
    assert d.get_dataflow_edges_from_node_to_node(g, a, c) == [(a1, (c, 0))]
    assert d.get_dataflow_edges_from_node_to_node(g, a, e) == [] and d.get_dataflow_edges_from_node_to_node(g, e, a) == []
    lone = d.OpenDataflowGraph()
    n, _ = lone.add_node([], 1)
    assert d.get_source_nodes(lone) == {n}


def test_subgraph_inputs_and_crossing_edges():
    g, x, (a, b, c, e), (a0, a1, b0, c0, e0) = diamond()
    assert sorted(d.get_subgraph_inputs(g, {b, c}), key=str) == sorted([a0, a1, x], key=str)
    assert d.get_subgraph_inputs(g, {a, b, c, e}) == [x]
    assert sorted(d.get_subgraph_incoming_edges(g, {b, c})) == [(a0, (b, 0)), (a1, (c, 0))]
    assert sorted(d.get_subgraph_outgoing_edges(g, {b, c})) == [(b0, (e, 0)), (c0, (e, 1))]
    assert d.get_subgraph_incoming_edges(g, {a}) == [] and d.get_subgraph_outgoing_edges(g, {e}) == []


def test_permutations_keep_the_graph_isomorphic():
    g, x, (a, b, c, e), outs = diamond()
    same = {n: n for n in (a, b, c, e)}
    assert d.is_isomorphic_under(g, g, same, {x[1]: x[1]})
    assert not d.is_isomorphic_under(g, g, {a: a, b: c, c: b, e: e}, {x[1]: x[1]})      # b and c read different operands
    h, got = d.permute_node_ids(g, {a: 3, b: 2, c: 1, e: 0})
    assert sorted(got) == [a, b, c, e] and d.is_isomorphic_under(g, h, got, {x[1]: h.get_graph_inputs()[0][1]})
    assert d.find_dataflow_isomorphism(g, h) is not None
    with pytest.raises(Exception):
        d.permute_node_ids(g, {a: 0, b: 0, c: 1, e: 2})
    with pytest.raises(Exception):
        d.permute_node_ids(g, {a: 0})
    # two inputs swapped: the graph is isomorphic to the original under the swapped input map only
    k = d.OpenDataflowGraph()
    p, q = k.add_input(), k.add_input()
    n, _ = k.add_node([p, q, q], 1)
    s = d.permute_input_ids(k, {p[1]: q[1], q[1]: p[1]})
    sn = s.get_nodes()[0]
    assert d.is_isomorphic_under(k, s, {n: sn}, {p[1]: q[1], q[1]: p[1]})
    assert not d.is_isomorphic_under(k, s, {n: sn}, {p[1]: p[1], q[1]: q[1]})
    with pytest.raises(Exception):
        d.permute_input_ids(k, {p[1]: 0, q[1]: 0})


def test_open_dataflow_graph_as_dot():
    g, x, (a, b, c, e), outs = diamond()
    dot = d.open_dataflow_graph_as_dot(g)
    assert dot.startswith("digraph {") and dot.rstrip().endswith("}")
    assert dot.count("[shape=box") == 1 and dot.count(" -> n") == 6          # 4 node-to-node uses + 2 uses of the input
    assert f'n{a} -> n{c} [label="1 -> 0"]' in dot and f'i{x[1]} -> n{c} [label="-> 1"]' in dot
