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
