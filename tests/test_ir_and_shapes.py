"""IR, (parallel) shape inference and v1 file-format tests (reference: lib/op-attrs/test, lib/pcg/test)."""
import json

import pytest

from flexflow_train_b200 import _ffcore as c

PTS = c.ParallelTensorShape


def infer(op, attrs, inputs):
    r = c.infer_shapes(op, attrs, inputs)
    return dict(r["outputs"]), dict(r["weights"])


def test_enums_match_reference_sets():
    ops = c.operator_types()
    assert len(ops) == 83 and ops[0] == "NOOP" and "BATCHMATMUL" in ops and ops[-1] == "FUSED_PARALLEL"
    slots = c.slot_names()
    assert slots[:3] == ["INPUT", "OUTPUT", "FILTER"] and "INPUT_7" in slots and slots[-1] == "SCALE"


def test_linear_unparallel_shapes():
    out, w = infer("LINEAR", {"out_channels": 32, "use_bias": True}, [("INPUT", PTS([8, 5, 16]))])
    assert out["OUTPUT"].sizes == [8, 5, 32]
    assert w["WEIGHT"].sizes == [32, 16] and w["BIAS"].sizes == [32]


def test_linear_parallel_degree_algebra():
    # data parallel on dim 0, row parallel on the contracted dim, replicated input -> channel shards
    x = PTS([8, 16], "FLOAT", [2, 4], 1, 3)
    out, w = infer("LINEAR", {"out_channels": 30, "use_bias": True}, [("INPUT", x)])
    o = out["OUTPUT"]
    assert o.degrees == [2, 3] and o.sum_degree == 4 and o.discard_copy_degree == 1
    assert w["WEIGHT"].degrees == [3, 4] and w["WEIGHT"].discard_copy_degree == 2 and w["WEIGHT"].sum_degree == 1
    assert w["BIAS"].degrees == [3] and w["BIAS"].sum_degree == 4 and w["BIAS"].discard_copy_degree == 2


def test_parallel_ops_change_only_their_degree():
    x = PTS([8, 16])
    p = infer("REPARTITION", {"repartition_dim": 0, "repartition_degree": 4}, [("INPUT", x)])[0]["OUTPUT"]
    assert p.degrees == [4, 1] and p.piece_sizes == [2, 16]
    r = infer("REPLICATE", {"replicate_degree": 2}, [("INPUT", p)])[0]["OUTPUT"]
    assert r.discard_copy_degree == 2 and r.total_degree == 8
    cmb = infer("COMBINE", {"combine_dim": 0, "combine_degree": 2}, [("INPUT", p)])[0]["OUTPUT"]
    assert cmb.degrees == [2, 1]
    s = PTS([8, 16], "FLOAT", [1, 1], 4, 1)
    red = infer("REDUCTION", {"reduction_degree": 4}, [("INPUT", s)])[0]["OUTPUT"]
    assert red.sum_degree == 1
    with pytest.raises(c.CoreError):
        infer("COMBINE", {"combine_dim": 0, "combine_degree": 3}, [("INPUT", p)])
    with pytest.raises(c.CoreError):
        infer("REPARTITION", {"repartition_dim": 0, "repartition_degree": 3}, [("INPUT", x)])


def test_attention_shapes_and_head_parallelism():
    q = PTS([4, 10, 32])
    attrs = {"embed_dim": 32, "num_heads": 8, "kdim": 4, "vdim": 4, "dropout": 0.0, "bias": False}
    out, w = infer("MULTIHEAD_ATTENTION", attrs, [("QUERY", q), ("KEY", q), ("VALUE", q)])
    assert out["OUTPUT"].sizes == [4, 10, 32]
    assert w["WEIGHT"].sizes == [32 * 4 * 3 + 4 * 32, 8]
    qr = PTS([4, 10, 32], "FLOAT", [1, 1, 1], 1, 4)
    out, w = infer("MULTIHEAD_ATTENTION", attrs, [("QUERY", qr), ("KEY", qr), ("VALUE", qr)])
    assert out["OUTPUT"].sum_degree == 4 and w["WEIGHT"].degrees == [1, 4]
    qs = PTS([4, 10, 32], "FLOAT", [1, 2, 1])
    with pytest.raises(c.CoreError):
        infer("MULTIHEAD_ATTENTION", attrs, [("QUERY", qs), ("KEY", qs), ("VALUE", qs)])


def test_conv_pool_bn_shapes():
    x = PTS([2, 3, 32, 32])
    out, w = infer("CONV2D", {"out_channels": 8, "kernel_h": 3, "kernel_w": 3, "stride_h": 2, "stride_w": 2, "padding_h": 1,
                              "padding_w": 1, "groups": 1, "use_bias": True}, [("INPUT", x)])
    assert out["OUTPUT"].sizes == [2, 8, 16, 16] and w["FILTER"].sizes == [8, 3, 3, 3] and w["BIAS"].sizes == [8]
    out, _ = infer("POOL2D", {"kernel_h": 2, "kernel_w": 2, "stride_h": 2, "stride_w": 2, "padding_h": 0, "padding_w": 0,
                              "pool_type": "MAX"}, [("INPUT", x)])
    assert out["OUTPUT"].sizes == [2, 3, 16, 16]
    out, w = infer("BATCHNORM", {"relu": True, "affine": True, "eps": 1e-5}, [("INPUT", x)])
    assert out["OUTPUT"].sizes == [2, 3, 32, 32] and w["GAMMA"].sizes == [3]


def test_misc_shape_rules():
    x = PTS([4, 6, 8])
    assert infer("SOFTMAX", {"dim": 2}, [("INPUT", x)])[0]["OUTPUT"].sizes == [4, 6, 8]
    assert infer("FLAT", {"start_dim": 1, "end_dim": 2}, [("INPUT", x)])[0]["OUTPUT"].sizes == [4, 48]
    assert infer("TRANSPOSE", {"permutation": [0, 2, 1]}, [("INPUT", x)])[0]["OUTPUT"].sizes == [4, 8, 6]
    outs = infer("SPLIT", {"splits": [2, 4], "axis": 1}, [("INPUT", x)])[0]
    assert outs["OUTPUT_0"].sizes == [4, 2, 8] and outs["OUTPUT_1"].sizes == [4, 4, 8]
    cat = infer("CONCAT", {"axis": 2, "num_inputs": 2}, [("INPUT_0", x), ("INPUT_1", x)])[0]["OUTPUT"]
    assert cat.sizes == [4, 6, 16]
    red = infer("REDUCE_SUM", {"axes": [1], "op_type": "REDUCE_SUM", "keepdims": False}, [("INPUT", x)])[0]["OUTPUT"]
    assert red.sizes == [4, 8]
    tk = infer("TOPK", {"k": 3, "sorted": True}, [("INPUT", x)])[0]
    assert tk["OUTPUT"].sizes == [4, 6, 3] and tk["INDEX"].dtype == "INT32"
    bm = infer("BATCHMATMUL", {}, [("LHS_INPUT", PTS([2, 5, 7])), ("RHS_INPUT", PTS([2, 7, 3]))])[0]["OUTPUT"]
    assert bm.sizes == [2, 5, 3]
    emb, w = infer("EMBEDDING", {"num_entries": 100, "out_channels": 16, "aggr": "SUM", "data_type": "FLOAT"},
                   [("INPUT", PTS([4, 6, 1], "INT32"))])
    assert emb["OUTPUT"].sizes == [4, 6, 16] and w["WEIGHT"].sizes == [100, 16]
    with pytest.raises(c.CoreError):  # softmax dim cannot be sharded
        infer("SOFTMAX", {"dim": 2}, [("INPUT", PTS([4, 6, 8], "FLOAT", [1, 1, 2]))])


def test_builder_inserts_weights_and_parallel_weight_chains():
    b = c.GraphBuilder()
    x = b.create_input([8, 16], "FLOAT", name="x")
    y = b.dense(x, 32, "RELU", True, name="fc")
    g = b.graph
    types = [n["type"] for n in g.nodes()]
    assert types.count("WEIGHT") == 2 and types.count("LINEAR") == 1
    assert g.shape(y).sizes == [8, 32]
    pb = c.GraphBuilder(parallel=True)
    x = pb.create_input([8, 16], "FLOAT")
    xp = pb.parallel_partition(x, 0, 4)
    y = pb.dense(xp, 32, None, True)
    yc = pb.parallel_combine(y, 0, 4)
    assert pb.graph.shape(yc).degrees == [1, 1] and pb.graph.shape(y).degrees == [4, 1]
    types = [n["type"] for n in pb.graph.nodes()]
    assert types.count("REPLICATE") == 2  # weight and bias replicated over the 4 data-parallel shards
    with pytest.raises(c.CoreError):
        b.parallel_partition(x, 0, 2)  # not a parallel builder


def test_v1_json_round_trip_all_models():
    for name in c.model_names():
        g = c.build_model(name, {"batch_size": 4} if name != "single_operator" else None)
        text = g.to_v1_string()
        j = json.loads(text)
        raw = j["raw_graph"]
        assert set(raw) == {"node_labels", "output_labels", "graph"} and set(raw["graph"]) == {"nodes", "edges", "outputs"}
        e = raw["graph"]["edges"][0]
        assert set(e) == {"srcNode", "srcSlot", "dstNode", "dstSlot"}
        g2 = c.Graph.from_v1(text)
        assert g2.signature() == g.signature() and len(g2) == len(g)


def test_v1_parallel_and_mapped_round_trip():
    pb = c.GraphBuilder(parallel=True)
    x = pb.create_input([8, 16], "FLOAT")
    y = pb.dense(pb.parallel_partition(x, 0, 2), 4)
    g = pb.graph
    ms = c.MachineSpecification(1, 2)
    r = c.evaluate_pcg(g, ms, c.CostEstimator(ms))
    mp = r["mapped_pcg"]
    assert mp.is_mapped()
    j = mp.to_v1(parallel=True)
    assert "machine_views" in j
    shp = j["raw_graph"]["output_labels"][0][1]["shape"]
    assert set(shp["dims"]) == {"shard_dims", "replica_dims"}
    back = c.Graph.from_v1(j)
    assert back.is_mapped() and back.signature() == mp.signature()


def test_json_optional_is_null_and_parser_round_trip():
    g = c.build_model("single_operator", None)
    lin = [n for n in g.nodes() if n["type"] == "LINEAR"][0]
    assert lin["attrs"]["activation"] is None and lin["attrs"]["regularizer"] is None
    assert json.loads(c.json_roundtrip('{"a": [1, 2.5, null, true, "x\\n"], "b": {"c": -3}}')) == \
        {"a": [1, 2.5, None, True, "x\n"], "b": {"c": -3}}


# ------------------------------------------------------------------ v1 files against hand-written golden files
def _golden(name):
    import os
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name)) as f:
        return json.load(f)


def test_v1_computation_graph_matches_the_golden_file():
    # field names, variant tags ({"type", "value"}), [key, value] pairs for maps with non-string keys, null for empty
    # optionals and enum value names are pinned by a file written by hand from the format description
    b = c.GraphBuilder()
    x = b.create_input([4, 6], "FLOAT", name="x")
    b.dense(x, 3, "RELU", False, name="fc")
    gold = _golden("v1_computation_graph_linear_relu.json")
    assert b.graph.to_v1() == gold
    back = c.Graph.from_v1(gold)
    assert back.signature() == b.graph.signature() and back.to_v1() == gold
    lin = [n for n in back.nodes() if n["type"] == "LINEAR"][0]
    assert lin["attrs"]["activation"] == "RELU" and lin["attrs"]["use_bias"] is False and lin["name"] == "fc"


def test_v1_mapped_parallel_graph_matches_the_golden_file():
    pb = c.GraphBuilder(parallel=True)
    x = pb.create_input([8, 16], "FLOAT", name="x")
    pb.dense(pb.parallel_partition(x, 0, 2, name="cut"), 4, None, False, name="fc")
    ms = c.MachineSpecification(1, 2)
    mapped = c.evaluate_pcg(pb.graph, ms, c.CostEstimator(ms))["mapped_pcg"]
    gold = _golden("v1_mapped_pcg_partitioned_linear.json")
    assert mapped.to_v1(parallel=True) == gold
    back = c.Graph.from_v1(gold)
    assert back.is_mapped() and back.signature() == mapped.signature()
    # a file that names an unknown operator tag or lacks a label is refused with a message, not half-read
    bad = json.loads(json.dumps(gold))
    bad["raw_graph"]["node_labels"][4][1]["op_attrs"]["type"] = "no_such_operator"
    with pytest.raises(Exception):
        c.Graph.from_v1(bad)
    bad = json.loads(json.dumps(gold))
    del bad["raw_graph"]["output_labels"][4]
    with pytest.raises(Exception):
        c.Graph.from_v1(bad)


def test_sp_decomposition_json_form():
    # {"type": "series" | "parallel", "left_child", "right_child"} / {"type": "leaf", "value": n}, binary and left-associative
    # (lib/pcg/src/pcg/file_format/v1/v1_binary_sp_decomposition/json.cc)
    b = c.GraphBuilder()
    x = b.create_input([4, 6], "FLOAT", name="x")
    y = b.dense(x, 3, "RELU", True, name="fc")
    tree, exact = c.get_graph_sp_decomposition(b.graph)
    assert exact
    j = c.sp_to_json(c.sp_left_associative_binary(tree))     # the n-ary tree has a three-way parallel stage
    leaf = lambda n: {"type": "leaf", "value": n}   # noqa: E731
    assert j["type"] == "series" and j["right_child"] == leaf(y[0])
    par = j["left_child"]                            # ((input | weight) | bias), left-associative
    assert par["type"] == "parallel" and par["left_child"]["type"] == "parallel" and par["right_child"]["type"] == "leaf"
    leaves = {par["right_child"]["value"], par["left_child"]["left_child"]["value"], par["left_child"]["right_child"]["value"]}
    assert leaves == {n["id"] for n in b.graph.nodes() if n["type"] in ("INPUT", "WEIGHT")}
    assert c.sp_nodes(c.sp_from_json(j)) == c.sp_nodes(tree)
    for bad in ({"type": "leaf"}, {"type": "series", "left_child": leaf(0)}, {"type": "tree", "value": 1}):
        with pytest.raises(Exception):
            c.sp_from_json(bad)


# ------------------------------------------------------------------ graph queries (lib/pcg/include/pcg/computation_graph.h)
def _two_layer():
    b = c.GraphBuilder()
    x = b.create_input([4, 6], "FLOAT", name="x")
    h = b.dense(x, 5, "RELU", True, name="fc1")
    y = b.dense(h, 3, None, False, name="fc2")
    return b.graph, x, h, y


def test_graph_queries_by_name_and_role():
    g, x, h, y = _two_layer()
    fc1 = g.get_layer_by_name("fc1")
    assert fc1 == h[0] and g.node(fc1)["type"] == "LINEAR"
    with pytest.raises(Exception):
        g.get_layer_by_name("no such layer")
    assert g.get_incoming_inputs(fc1) == [x]
    weights = g.get_incoming_weights(fc1)
    assert len(weights) == 2 and all(g.node(w[0])["type"] == "WEIGHT" for w in weights)
    assert [s for s, _ in g.get_incoming_tensors(fc1)] == ["INPUT", "WEIGHT", "BIAS"]
    assert g.get_incoming_weights(x[0]) == [] and g.get_incoming_inputs(x[0]) == []
    assert g.get_outgoing_tensors(fc1) == [h] and g.get_source_layer(y) == y[0]
    assert sorted(g.get_all_tensors()) == sorted((n["id"], "OUTPUT") for n in g.nodes())


def test_graph_isomorphism_ignores_names_and_ids():
    g, x, h, y = _two_layer()
    bare = g.without_layer_names()
    assert all(n["name"] == "" for n in bare.nodes()) and bare.is_isomorphic_to(g) and g.get_layer_by_name("fc2") == y[0]
    # the same layers added in another order (weights first) get other ids and are still the same graph
    b = c.GraphBuilder()
    x2 = b.create_input([4, 6], "FLOAT", name="other")
    b.dense(b.dense(x2, 5, "RELU", True), 3, None, False)
    assert b.graph.is_isomorphic_to(g)
    b.unary("RELU", x2)
    assert not b.graph.is_isomorphic_to(g)
    wider = c.GraphBuilder()
    wider.dense(wider.dense(wider.create_input([4, 6], "FLOAT"), 7, "RELU", True), 3, None, False)
    assert not wider.graph.is_isomorphic_to(g)


def test_graph_subgraph_edges():
    g, x, h, y = _two_layer()
    sub = {h[0]}
    inc = g.get_subgraph_incoming_edges(sub)
    assert len(inc) == 3 and ((x[0], "OUTPUT"), (h[0], "INPUT")) in inc
    assert g.get_subgraph_outgoing_edges(sub) == [(h, (y[0], "INPUT"))]
    assert g.get_subgraph_successors(sub) == {y[0]} and g.get_subgraph_successors({y[0]}) == set()
    everything = {n["id"] for n in g.nodes()}
    assert g.get_subgraph_incoming_edges(everything) == [] and g.get_subgraph_outgoing_edges(everything) == []
