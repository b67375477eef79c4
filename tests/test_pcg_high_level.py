"""The high-level Python API over the C interface (frontend/pcg.py): operator overloading builds the same graph as
the pybind builder, the graph serialises / renders / round-trips, and the strategy search runs through the C call."""
import json

import pytest

from flexflow_train_b200 import _ffcore as core
from flexflow_train_b200.frontend import pcg


def test_operator_overloads_build_the_expected_graph():
    g = pcg.ComputationGraph()
    x = g.create_input([8, 16], name="x")
    y = g.create_input([8, 16], name="y")
    h = ((x + y) * 2.0 - y).relu()
    h = (h / 4.0).exp() + 1.0
    out = h.dense(32, activation="GELU", name="fc1").dense(4, name="fc2").softmax(name="prob")
    assert x.shape == [8, 16] and out.shape == [8, 4]
    text = g.to_json()
    ref = core.Graph.from_v1(text)
    types = [n["type"] for n in ref.nodes()]
    for t in ("EW_ADD", "SCALAR_MULTIPLY", "EW_SUB", "RELU", "SCALAR_TRUE_DIV", "EXP", "SCALAR_ADD", "LINEAR", "SOFTMAX"):
        assert t in types, (t, types)
    assert types.count("LINEAR") == 2 and types.count("WEIGHT") == 4
    # the same model through the pybind builder has the same signature
    b = core.GraphBuilder()
    bx, by = b.create_input([8, 16], name="x"), b.create_input([8, 16], name="y")
    t = b.unary("RELU", b.binary("EW_SUB", b.unary("SCALAR_MULTIPLY", b.binary("EW_ADD", bx, by), 2.0), by))
    t = b.unary("SCALAR_ADD", b.unary("EXP", b.unary("SCALAR_TRUE_DIV", t, 4.0)), 1.0)
    b.softmax(b.dense(b.dense(t, 32, activation="GELU", name="fc1"), 4, name="fc2"), name="prob")
    assert b.graph.signature() == ref.signature()
    snap = g.graph()
    assert snap.num_nodes == len(types) and snap.to_dot().lstrip().startswith("digraph")
    assert pcg.Graph.from_json(text).to_json() == text


def test_generic_layers_errors_and_search_through_the_c_api():
    g = pcg.ComputationGraph()
    x = g.create_input([4, 3, 8, 8], name="img")
    c = x.conv2d(8, (3, 3), padding=(1, 1), activation="RELU", name="conv")
    (p,) = g.add_layer("POOL2D", {"kernel_h": 2, "kernel_w": 2, "stride_h": 2, "stride_w": 2, "padding_h": 0, "padding_w": 0,
                                  "pool_type": "MAX", "activation": None}, [("INPUT", c)], name="pool")
    assert c.shape == [4, 8, 8, 8] and p.shape == [4, 8, 4, 4]
    w = g.create_weight([5], initializer={"type": "zero"}, name="w")
    assert w.shape == [5]
    with pytest.raises(pcg.FFIError):
        x.dense(4).add(p)                      # shapes that do not match
    other = pcg.ComputationGraph()
    with pytest.raises(ValueError):
        x.add(other.create_input([4, 3, 8, 8]))
    with pytest.raises(pcg.FFIError):
        pcg.Graph.from_json("{not json")
    model = pcg.Graph.from_model("mlp", {})
    strategy, ms = model.optimize(gpus_per_node=4, algorithm="data_parallel")
    assert ms > 0 and strategy.num_nodes > model.num_nodes
    mapped = core.Graph.from_v1(strategy.to_json(parallel=True))
    assert mapped.is_mapped() and any(n["type"] == "REPARTITION" for n in mapped.nodes())
    json.loads(strategy.to_json(parallel=True))
