"""Lowering passes: pass expansion, loss / update insertion, copy insertion, shard expansion, machine slicing
(reference: lib/task-spec/src/task-spec/dynamic_graph/*.cc and their tests under lib/task-spec/test)."""
from collections import Counter

from flexflow_train_b200 import _ffcore as core
from flexflow_train_b200.compiler import strategy as S
from flexflow_train_b200.runtime import lowering as L


def _mlp(batch=8):
    return core.build_model("mlp", {"batch_size": batch})


def test_dynamic_graph_has_one_forward_invocation_per_node():
    g = _mlp()
    inv = L.make_dynamic_graph(g)
    assert len(inv) == len(g.nodes())
    assert all(i["task"] == "FWD" for i in inv)


def test_pass_expansion_adds_backward_twins_with_grad_roles():
    g = _mlp()
    inv = L.perform_pass_expansion(g, L.make_dynamic_graph(g))
    fwd = [i for i in inv if i["task"] == "FWD"]
    bwd = [i for i in inv if i["task"] == "BWD"]
    assert len(fwd) == len(g.nodes())
    # inputs and weights have no backward task; every operator on a path to a weight has one
    assert {i["op_type"] for i in bwd}.isdisjoint({"INPUT", "WEIGHT"})
    assert {i["node"] for i in bwd} == {n["id"] for n in g.nodes() if n["type"] not in ("INPUT", "WEIGHT")}
    for b in bwd:
        assert any(x["role"] == "GRAD" for x in b["inputs"])
        assert all(x["role"] == "GRAD" for x in b["outputs"])
    # backward tasks come in reverse topological order
    pos = {n: k for k, n in enumerate(g.topological_order())}
    order = [pos[b["node"]] for b in bwd]
    assert order == sorted(order, reverse=True)


def test_loss_and_update_insertion():
    g = _mlp()
    inv = L.lower(g, optimizer={"type": "adam"})
    c = Counter(i["task"] for i in inv)
    weights = [n for n in g.nodes() if n["type"] == "WEIGHT"]
    assert c["LOSS"] == 1 and c["UPD"] == len(weights)
    tasks = [i["task"] for i in inv]
    assert tasks.index("LOSS") > max(k for k, t in enumerate(tasks) if t == "FWD")
    assert tasks.index("LOSS") < min(k for k, t in enumerate(tasks) if t == "BWD")
    upd = [i for i in inv if i["task"] == "UPD"][0]
    assert {x["role"] for x in upd["inputs"]} == {"FWD", "GRAD", "OPT:m", "OPT:v"}
    sgd = [i for i in L.lower(g, optimizer={"type": "sgd", "momentum": 0.9}) if i["task"] == "UPD"][0]
    assert {x["role"] for x in sgd["inputs"]} == {"FWD", "GRAD", "OPT:momentum"}
    plain = [i for i in L.lower(g, optimizer={"type": "sgd"}) if i["task"] == "UPD"][0]
    assert {x["role"] for x in plain["inputs"]} == {"FWD", "GRAD"}


def test_shard_expansion_and_machine_slicing_on_a_mapped_pcg():
    g = _mlp(batch=8)
    ms = core.MachineSpecification(1, 2)
    res = S.optimize(g, world=2, algorithm="data_parallel")
    pcg = res["mapped_pcg"]
    inv = L.lower(pcg, ms, optimizer={"type": "sgd"}, distributed=True)
    per_dev = Counter(i["device"] for i in inv if i["op_type"] in ("LINEAR", "SOFTMAX", "LOSS"))
    assert set(per_dev) == {0, 1}
    assert per_dev[0] == per_dev[1]  # both devices run the same operator tasks, each on its shard
    # unsharded sources (inputs, weights) have one task, on the device their view names
    assert Counter(i["device"] for i in inv if i["op_type"] == "WEIGHT" and i["task"] == "FWD") == {0: 6}
    sl0 = L.perform_machine_slicing(inv, 0)
    assert sl0 and all(i["device"] in (0, None) for i in sl0)
    # data parallelism needs exactly the gradient reductions as cross-device work: every weight gradient is
    # all-reduced; nothing else moves
    moved = [i for i in inv if i["task"] == "COPY"]
    assert all(i["op_type"] in ("REPARTITION", "COMBINE", "REPLICATE", "REDUCTION", "COPY") for i in moved)
