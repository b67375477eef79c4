"""Substitution engine (reference: lib/substitutions/test, lib/substitution-generator/test)."""
import json
import os

import pytest

from flexflow_train_b200 import _ffcore as c

MS = c.MachineSpecification(1, 4)


def mlp():
    return c.build_model("mlp", {"batch_size": 16, "input_dim": 32, "hidden": [64], "num_classes": 8})


def kinds(g):
    out = {}
    for n in g.nodes():
        out[n["type"]] = out.get(n["type"], 0) + 1
    return out


def test_rule_set_is_valid_and_sized():
    rules = c.get_substitution_set(MS)
    assert len(rules) > 100 and all(r.is_valid() for r in rules)
    names = {r.name for r in rules}
    for must in ("replicate_linear_combine_2", "partition_linear_combine_0_4_bias", "partition_attention_combine_2",
                 "replicate_attention_reduce_4_bias", "partition_conv2d_combine_2", "partition_softmax_combine_1_0_2",
                 "fuse_linear_RELU", "partition_linear_reduce_4", "cancel_combine_repartition"):
        assert must in names, must


def test_replicate_linear_combine_matches_hand_built_pcg():
    g = mlp()
    rule = c.create_replicate_linear_combine(2, True)
    ms = c.find_pattern_matches(rule, g)
    assert len(ms) == 2
    first = [m for m in ms if g.node(m.nodes[0])["name"] == "fc0"][0]
    g2 = c.apply_substitution(g, rule, first)
    lin = [n for n in g2.nodes() if n["name"] == "fc0"][0]
    ins = dict((s, tuple(v)) for s, v in lin["inputs"])
    assert g2.node(ins["INPUT"][0])["type"] == "REPLICATE"
    w = g2.node(ins["WEIGHT"][0])
    assert w["type"] == "REPARTITION" and w["attrs"]["repartition_dim"] == 0 and w["outputs"][0][1].degrees == [2, 1]
    assert lin["outputs"][0][1].degrees == [1, 2]
    cons = g2.consumers((lin["id"], "OUTPUT"))
    assert len(cons) == 1 and g2.node(cons[0][0])["type"] == "COMBINE"
    # the hand-built equivalent through the parallel builder has the same operator multiset
    pb = c.GraphBuilder(parallel=True)
    x = pb.create_input([16, 32], "FLOAT")
    y = pb.parallel_combine(pb.dense(pb.parallel_replicate(x, 2), 64, "RELU", True), -1, 2)
    assert kinds(pb.graph)["REPARTITION"] == 2 and kinds(pb.graph)["REPLICATE"] == 1 and pb.graph.shape(y).degrees == [1, 1]


def test_data_parallel_linear_and_cancellation():
    g = mlp()
    rules = c.get_substitution_set(MS)
    sel = [r for r in rules if r.name.startswith("partition_linear_combine_0_4") or r.name.startswith("cancel")]
    g2 = c.apply_rules_exhaustively(g, sel, 1000, 4)
    k = kinds(g2)
    # both Linears data parallel; the Combine/Repartition pair between them cancelled
    assert k["REPARTITION"] == 1 and k["COMBINE"] == 1 and k["REPLICATE"] == 4
    for n in g2.nodes():
        if n["type"] == "LINEAR":
            assert n["outputs"][0][1].degrees == [4, 1]


def test_row_parallel_linear_emits_reduction():
    g = mlp()
    rule = c.create_partition_linear_reduce(4, True)
    m = c.find_pattern_matches(rule, g)[0]
    g2 = c.apply_substitution(g, rule, m)
    lin = g2.node([n["id"] for n in g2.nodes() if n["type"] == "LINEAR" and n["outputs"][0][1].sum_degree == 4][0])
    cons = g2.consumers((lin["id"], "OUTPUT"))
    assert g2.node(cons[0][0])["type"] == "REDUCTION"


def test_fuse_linear_activation():
    b = c.GraphBuilder()
    x = b.create_input([8, 16], "FLOAT")
    y = b.unary("RELU", b.dense(x, 8, None, True))
    b.dense(y, 4)
    rule = c.create_fuse_linear_activation("RELU")
    ms = c.find_pattern_matches(rule, b.graph)
    assert len(ms) == 1
    g2 = c.apply_substitution(b.graph, rule, ms[0])
    assert kinds(g2).get("RELU", 0) == 0
    assert [n["attrs"]["activation"] for n in g2.nodes() if n["type"] == "LINEAR"].count("RELU") == 1


def test_interior_value_with_outside_use_blocks_the_match():
    b = c.GraphBuilder()
    x = b.create_input([8, 16], "FLOAT")
    h = b.dense(x, 8, None, True)
    r = b.unary("RELU", h)
    b.binary("EW_ADD", r, h)  # the Linear's output is also used outside the Linear->ReLU pattern
    rule = c.create_fuse_linear_activation("RELU")
    ms = c.find_pattern_matches(rule, b.graph)
    assert ms and c.apply_substitution(b.graph, rule, ms[0]) is None
    assert "outside" in c.why_not_applicable(b.graph, rule, ms[0])


def test_inapplicable_degree_is_rejected_by_shape_inference():
    g = c.build_model("mlp", {"batch_size": 6, "input_dim": 32, "hidden": [64], "num_classes": 8})
    rule = c.create_partition_linear_combine(0, 4, True)
    assert c.find_pattern_matches(rule, g) == []  # 6 rows are not divisible by 4


def test_attention_rules():
    g = c.build_model("transformer_lm", {"num_features": 64, "sequence_length": 16, "batch_size": 4, "dim_feedforward": 128,
                                         "num_heads": 4, "num_decoder_layers": 1, "dropout": 0.0, "vocab_size": 32})
    r = c.create_replicate_attention_reduce(4, False)
    m = c.find_pattern_matches(r, g)
    assert len(m) == 1
    g2 = c.apply_substitution(g, r, m[0])
    att = [n for n in g2.nodes() if n["type"] == "MULTIHEAD_ATTENTION"][0]
    assert att["outputs"][0][1].sum_degree == 4
    w = dict((s, tuple(v)) for s, v in att["inputs"])["WEIGHT"]
    assert g2.shape(w).degrees == [1, 4]
    r = c.create_partition_attention_combine(2, False)
    g3 = c.apply_substitution(g, r, c.find_pattern_matches(r, g)[0])
    att = [n for n in g3.nodes() if n["type"] == "MULTIHEAD_ATTENTION"][0]
    assert att["outputs"][0][1].degrees == [2, 1, 1]


# the reference checkout sits beside this repository (or where FF_REFERENCE_DIR points)
REF = os.path.join(os.environ.get("FF_REFERENCE_DIR") or
                   os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"), "substitutions")


@pytest.mark.skipif(not os.path.exists(REF), reason="legacy rule files not available")
def test_legacy_rule_collection_loads():
    rules, st = c.load_legacy_rules(open(os.path.join(REF, "test_subst.json")).read())
    assert st["num_rules"] == 1 and st["num_converted"] == 1 and rules[0].is_valid()
    rules, st = c.load_legacy_rules(open(os.path.join(REF, "graph_subst_3_v2.json")).read())
    assert st["num_rules"] == 640 and st["num_converted"] > 400
    assert st["op_histogram"]["OP_REPLICATE"] == 866 and st["op_histogram"]["OP_LINEAR"] == 562


def test_legacy_rule_inline_and_dot():
    rule = {"_t": "Rule", "name": "r", "srcOp": [{"_t": "Operator", "type": "OP_PARTITION", "input": [{"_t": "Tensor", "opId": -1, "tsId": 0}],
                                                  "para": [{"_t": "Parameter", "key": "PM_PARALLEL_DIM", "value": 1}, {"_t": "Parameter", "key": "PM_PARALLEL_DEGREE", "value": 2}]},
                                                 {"_t": "Operator", "type": "OP_COMBINE", "input": [{"_t": "Tensor", "opId": 0, "tsId": 0}],
                                                  "para": [{"_t": "Parameter", "key": "PM_PARALLEL_DIM", "value": 1}, {"_t": "Parameter", "key": "PM_PARALLEL_DEGREE", "value": 2}]}],
            "dstOp": [{"_t": "Operator", "type": "OP_RELU", "input": [{"_t": "Tensor", "opId": -1, "tsId": 0}], "para": []}],
            "mappedOutput": [{"_t": "MapOutput", "srcOpId": 1, "srcTsId": 0, "dstOpId": 0, "dstTsId": 0}]}
    rules, st = c.load_legacy_rules({"_t": "RuleCollection", "rule": [rule]})
    assert st["num_converted"] == 1
    assert "digraph" in rules[0].as_dot() and "OP_PARTITION" in c.legacy_rule_as_dot(rule)


# ------------------------------------------------------------------ one rule at a time on a hand-built graph
# (the structure the reference's lib/substitutions/test/src/substitutions/unity_substitution_set.cc builds by hand)
def _rule(name):
    return {r.name: r for r in c.get_substitution_set(MS)}[name]


def _apply_once(g, rule):
    ms = c.find_pattern_matches(rule, g)
    assert len(ms) == 1, len(ms)
    g2 = c.apply_substitution(g, rule, ms[0])
    assert g2 is not None
    return g2


def _producer(g, node, slot):
    ins = dict((s, tuple(v)) for s, v in node["inputs"])
    return g.node(ins[slot][0])


def _only(g, typ):
    ns = [n for n in g.nodes() if n["type"] == typ]
    assert len(ns) == 1, (typ, len(ns))
    return ns[0]


def test_partition_conv2d_combine_rule():
    b = c.GraphBuilder()
    x = b.create_input([8, 4, 16, 16], "FLOAT", name="image")
    b.conv2d(x, 6, 3, 3, 1, 1, 1, 1, None, 1, True, name="conv")
    g2 = _apply_once(b.graph, _rule("partition_conv2d_combine_2_bias"))
    conv = _only(g2, "CONV2D")
    rp = _producer(g2, conv, "INPUT")
    assert rp["type"] == "REPARTITION" and rp["attrs"]["repartition_dim"] == 0 and rp["attrs"]["repartition_degree"] == 2
    for slot in ("FILTER", "BIAS"):
        w = _producer(g2, conv, slot)
        assert w["type"] == "REPLICATE" and w["attrs"]["replicate_degree"] == 2 and g2.node(dict((s, tuple(v)) for s, v in w["inputs"])["INPUT"][0])["type"] == "WEIGHT"
    assert conv["outputs"][0][1].degrees == [2, 1, 1, 1]
    cons = g2.consumers((conv["id"], "OUTPUT"))
    comb = g2.node(cons[0][0])
    assert len(cons) == 1 and comb["type"] == "COMBINE" and comb["attrs"]["combine_dim"] == 0 and comb["attrs"]["combine_degree"] == 2
    assert comb["outputs"][0][1].degrees == [1, 1, 1, 1] and comb["outputs"][0][1].sizes == [8, 6, 16, 16]


def test_partition_softmax_combine_rule_cuts_a_dim_other_than_the_softmax_dim():
    b = c.GraphBuilder()
    x = b.create_input([8, 10], "FLOAT", name="logits")
    b.softmax(x, 1, name="prob")
    g = b.graph
    g2 = _apply_once(g, _rule("partition_softmax_combine_1_0_2"))       # softmax over dim 1, cut dim 0 in two
    sm = _only(g2, "SOFTMAX")
    rp = _producer(g2, sm, "INPUT")
    assert rp["type"] == "REPARTITION" and rp["attrs"]["repartition_dim"] == 0 and sm["outputs"][0][1].degrees == [2, 1]
    comb = g2.node(g2.consumers((sm["id"], "OUTPUT"))[0][0])
    assert comb["type"] == "COMBINE" and comb["attrs"]["combine_dim"] == 0
    # the rule that would cut the softmax dim itself does not exist, and one written for another softmax dim does not match
    names = {r.name for r in c.get_substitution_set(MS)}
    assert "partition_softmax_combine_1_1_2" not in names
    assert c.find_pattern_matches(_rule("partition_softmax_combine_0_1_2"), g) == []


def test_partition_add_combine_rule_cuts_both_operands():
    b = c.GraphBuilder()
    x = b.create_input([8, 10], "FLOAT", name="a")
    y = b.create_input([8, 10], "FLOAT", name="b")
    b.binary("EW_ADD", x, y, name="sum")
    g2 = _apply_once(b.graph, _rule("partition_EW_ADD_combine_1_2"))
    add = _only(g2, "EW_ADD")
    for slot in ("LHS_INPUT", "RHS_INPUT"):
        rp = _producer(g2, add, slot)
        assert rp["type"] == "REPARTITION" and rp["attrs"]["repartition_dim"] == 1 and rp["attrs"]["repartition_degree"] == 2
    assert add["outputs"][0][1].degrees == [1, 2]
    assert g2.node(g2.consumers((add["id"], "OUTPUT"))[0][0])["type"] == "COMBINE"


def test_partition_relu_combine_rule_and_its_cancellation_with_a_neighbour():
    b = c.GraphBuilder()
    x = b.create_input([8, 10], "FLOAT", name="x")
    r1 = b.unary("RELU", x, name="r1")
    b.unary("RELU", r1, name="r2")
    g = b.graph
    rule = _rule("partition_RELU_combine_0_2")
    assert len(c.find_pattern_matches(rule, g)) == 2
    both = c.apply_rules_exhaustively(g, [rule], 100, 4)
    k = kinds(both)
    assert k["REPARTITION"] == 2 and k["COMBINE"] == 2
    # Combine(0, 2) followed by Repartition(0, 2) between the two ReLUs cancels: one cut region remains
    merged = c.apply_rules_exhaustively(both, [r for r in c.get_substitution_set(MS) if r.name.startswith("cancel")], 100, 4)
    k = kinds(merged)
    assert k["REPARTITION"] == 1 and k["COMBINE"] == 1
    assert all(n["outputs"][0][1].degrees == [2, 1] for n in merged.nodes() if n["type"] == "RELU")
