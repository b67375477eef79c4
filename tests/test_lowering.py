"""Lowering passes: pass expansion, loss / update insertion, copy insertion, shard expansion, machine slicing
(reference: lib/task-spec/src/task-spec/dynamic_graph/*.cc and their tests under lib/task-spec/test)."""
from collections import Counter

import pytest

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


def test_task_argument_accessor_runs_a_lowered_linear_layer_forward_backward_update():
    """Task bodies written against the accessor execute the lowered invocations of one Linear layer + loss + SGD
    and reproduce a plain PyTorch step."""
    import torch

    from flexflow_train_b200.runtime.task_accessor import TaskArgumentAccessor, run_invocations, value_key

    b = core.GraphBuilder()
    x = b.create_input([4, 6], name="x")
    y = b.dense(x, 3, use_bias=True, name="fc")
    g = b.graph
    nodes = {n["id"]: n for n in g.nodes()}
    inv = L.lower(g, logit=tuple(y), loss="mean_squared_error_avg_reduce", optimizer={"type": "sgd", "lr": 0.1})
    torch.manual_seed(0)
    xin, w0, b0, target = torch.randn(4, 6), torch.randn(3, 6), torch.randn(3), torch.randn(4, 3)
    table = {}

    def fwd_source(acc: TaskArgumentAccessor):
        data = {"x": xin, "fc.weight": w0.clone(), "fc.bias": b0.clone()}[acc.name]
        acc.set_output(data)

    def fwd_linear(acc):
        acc.set_output(acc.get_tensor("INPUT") @ acc.get_tensor("WEIGHT").t() + acc.get_tensor("BIAS"))

    def loss(acc):
        pred = acc.get_tensor("INPUT") if acc.has("INPUT") else list(acc.tensors.values())[-1]
        acc.set_output(2.0 * (pred - target) / pred.numel(), acc.invocation["outputs"][0]["slot"], "GRAD")

    def bwd_linear(acc):
        dy = acc.get_tensor("OUTPUT", "GRAD")
        for v in acc.invocation["outputs"]:
            slot = v.get("as", v["slot"])
            src = nodes[v["node"]]["name"]
            if src == "fc.weight":
                acc.tensors[value_key(v)] = dy.t() @ acc.get_tensor("INPUT")
            elif src == "fc.bias":
                acc.tensors[value_key(v)] = dy.sum(0)
            else:
                acc.tensors[value_key(v)] = dy @ acc.get_tensor("WEIGHT")

    def upd(acc):
        ins = acc.invocation["inputs"]
        w = acc.tensors[value_key(next(v for v in ins if v["role"] == "FWD"))]
        gr = acc.tensors[value_key(next(v for v in ins if v["role"] == "GRAD"))]
        w -= 0.1 * gr

    bodies = {("FWD", "INPUT"): fwd_source, ("FWD", "WEIGHT"): fwd_source, ("FWD", "LINEAR"): fwd_linear, ("LOSS", "*"): loss,
              ("BWD", "LINEAR"): bwd_linear, ("UPD", "*"): upd}
    run_invocations(inv, bodies, table, op_attrs_of=lambda n: nodes[n]["attrs"])
    wt = w0.clone().requires_grad_(True)
    bt = b0.clone().requires_grad_(True)
    ((xin @ wt.t() + bt - target) ** 2).mean().backward()
    got_w = next(t for k, t in table.items() if nodes[k[0]]["name"] == "fc.weight" and k[2] == "FWD")
    got_b = next(t for k, t in table.items() if nodes[k[0]]["name"] == "fc.bias" and k[2] == "FWD")
    assert torch.allclose(got_w, w0 - 0.1 * wt.grad, atol=1e-6)
    assert torch.allclose(got_b, b0 - 0.1 * bt.grad, atol=1e-6)


def test_passes_check_the_state_they_require():
    """Pass-state invariants at pass boundaries: a pass applied twice or out of order fails at once."""
    from flexflow_train_b200 import _ffcore as core

    cg = core.build_model("mlp", {})
    ms = core.MachineSpecification(1, 2)
    l0 = core.make_dynamic_graph(cg)
    l1 = core.perform_pass_expansion(cg, l0)
    with pytest.raises(core.CoreError, match="already has backward"):
        core.perform_pass_expansion(cg, l1)
    l2 = core.perform_update_insertion(cg, l1, {"type": "sgd"})
    with pytest.raises(core.CoreError, match="already has update"):
        core.perform_update_insertion(cg, l2, {"type": "sgd"})
    with pytest.raises(core.CoreError, match="shard-expanded first"):
        core.perform_machine_slicing(l2, 0)
    l3 = core.perform_copy_insertion(cg, l2, ms)
    l4 = core.perform_shard_expansion(cg, l3, ms)
    assert all(i["shard"] is not None and i["device"] is not None for i in l4)
    for fn in (lambda: core.perform_shard_expansion(cg, l4, ms), lambda: core.perform_copy_insertion(cg, l4, ms),
               lambda: core.perform_pass_expansion(cg, l4)):
        with pytest.raises(core.CoreError, match="shard|backward"):
            fn()
    assert len(core.perform_machine_slicing(l4, 0)) > 0


def test_optimizer_attrs_and_adam_bias_correction_schedule():
    import math

    from flexflow_train_b200 import _ffcore as core

    sgd = core.make_sgd_optimizer_attrs(0.1, momentum=0.9, nesterov=True, weight_decay=1e-4)
    assert sgd == {"type": "sgd", "lr": 0.1, "momentum": 0.9, "nesterov": True, "weight_decay": 1e-4}
    assert core.get_optimizer_attrs_for_next_iter(sgd) == sgd
    a = core.make_adam_optimizer_attrs(alpha=1e-3, beta1=0.9, beta2=0.999)
    assert a["beta_t"] == 1.0 and a["beta2_t"] == 1.0
    for t in range(1, 6):
        a = core.get_optimizer_attrs_for_next_iter(a)
        assert a["beta_t"] == pytest.approx(0.9 ** t) and a["beta2_t"] == pytest.approx(0.999 ** t)
        # the executors' closed form for step t
        assert a["alpha_t"] == pytest.approx(1e-3 * math.sqrt(1 - 0.999 ** t) / (1 - 0.9 ** t))
    with pytest.raises(core.CoreError):
        core.make_adam_optimizer_attrs(beta1=1.0)
    with pytest.raises(core.CoreError):
        core.make_sgd_optimizer_attrs(-1.0)
    # the update-insertion pass takes these attribute objects as they are
    cg = core.build_model("mlp", {})
    l = core.perform_update_insertion(cg, core.perform_pass_expansion(cg, core.make_dynamic_graph(cg)), a)
    assert any(i["task"] == "UPD" and any(v["role"] == "OPT:m" for v in i["inputs"]) for i in l)


SMALL_MODELS = {
    "mlp": {"batch_size": 8},
    "transformer": {"num_features": 32, "sequence_length": 8, "batch_size": 4, "dim_feedforward": 64, "num_heads": 2,
                    "num_encoder_layers": 1, "num_decoder_layers": 1, "vocab_size": 16},
    "transformer_lm": {"num_features": 32, "sequence_length": 8, "batch_size": 4, "dim_feedforward": 64, "num_heads": 2,
                       "num_decoder_layers": 2, "vocab_size": 16},
    "bert": {"token_ids": True, "batch_size": 4, "sequence_length": 8, "vocab_size": 32, "hidden_size": 32, "num_encoder_layers": 1,
             "num_heads": 2, "dim_feedforward": 64},
    "dlrm": {"batch_size": 8, "embedding_size": [50, 50], "embedding_dim": 8, "dense_arch_layer_sizes": [4, 8],
             "over_arch_layer_sizes": [16, 1]},
    "split_test": {"batch_size": 8},
    "candle_uno": {"batch_size": 4},
    "inception_v3": {"batch_size": 2, "num_classes": 10},
}


@pytest.mark.parametrize("model", sorted(SMALL_MODELS))
def test_executor_plan_agrees_with_the_lowered_step(model):
    """The kernel-library executor builds its step straight from the graph; the lowering passes build theirs through pass
    expansion, loss and update insertion.  For every model of the zoo the two must describe the same step: same
    invocations, every reader / writer dependency of the lowered step respected by the executor's stream order, same
    operands per operator.  (Planning needs no GPU: the executor is constructed with device='cpu'.)"""
    from flexflow_train_b200.runtime.executor import ExecConfig, Executable, OptimizerConfig
    from flexflow_train_b200.runtime.lowering import check_plan, lower

    cg = core.build_model(model, SMALL_MODELS[model])
    loss = "mean_squared_error_avg_reduce" if model in ("dlrm", "candle_uno") else "sparse_categorical_crossentropy"
    ex = Executable(cg, ExecConfig(device="cpu", compute_dtype="bf16" if model == "inception_v3" else "fp32", loss=loss,
                                   optimizer=OptimizerConfig(kind="sgd", lr=0.1)))
    inv = lower(cg, logit=ex.loss_value, loss=loss, optimizer={"type": "sgd"})
    assert len(inv) >= len(ex.step_plan()) - 1
    assert check_plan(ex, inv) == []
    # and the check does notice a wrong order: run the first Linear-like operator's backward before the loss
    plan = ex.step_plan()
    first_bwd = next(i for i, (t, _) in enumerate(plan) if t == "BWD")
    broken = plan[:]
    broken.insert(0, broken.pop(first_bwd))
    ex.step_plan = lambda: broken
    assert any("before its dependency" in p for p in check_plan(ex, inv))


def _two_relus_on(dev_first: int, dev_second: int):
    """x -> dense -> relu on a two-GPU machine: input, weight and dense on one device, the relu on the other."""
    b = core.GraphBuilder(parallel=True)
    x = b.create_input([4, 8], "FLOAT", name="x")
    r1 = b.dense(x, 8, None, False, name="fc")
    r2 = b.unary("RELU", r1, name="r2")
    view = lambda d: {"start": {"node_idx": 0, "device_idx": d, "device_type": "GPU"}, "dimensions": []}   # noqa: E731
    placement = {n["id"]: view(dev_first) for n in b.graph.nodes()}
    placement[r2[0]] = view(dev_second)
    return core.mapped_pcg_from_pcg_and_mapping(b.graph, placement), r1[0], r2[0]


def test_copy_insertion_same_placement_needs_no_copies():
    # the cases of lib/task-spec/test/src/task-spec/dynamic_graph/copy_insertion.cc: same mapping, no copies ...
    ms = core.MachineSpecification(1, 2)
    g, _, _ = _two_relus_on(0, 0)
    inv = core.perform_copy_insertion(g, core.perform_pass_expansion(g, core.make_dynamic_graph(g)), ms)
    assert [i for i in inv if i["task"] == "COPY"] == []


def test_copy_insertion_moves_a_tensor_between_differently_placed_operators():
    # ... and one tensor that has to move: forward from the producer's device to the consumer's, its gradient back
    ms = core.MachineSpecification(1, 2)
    g, r1, r2 = _two_relus_on(0, 1)
    before = core.perform_pass_expansion(g, core.make_dynamic_graph(g))
    inv = core.perform_copy_insertion(g, before, ms)
    copies = [i for i in inv if i["task"] == "COPY"]
    assert len(copies) == 2 and len(inv) == len(before) + 2
    roles = sorted((cp["inputs"][0]["role"], cp["src_devices"], cp["dst_devices"]) for cp in copies)
    assert roles == [("FWD", [0], [1]), ("GRAD", [1], [0])]
    # the forward copy sits right before the consumer's forward task, the gradient copy right before the producer's backward task
    pos = {(i["task"], i["node"], i["inputs"][0]["role"] if i["task"] == "COPY" else ""): k for k, i in enumerate(inv)}
    assert pos[("COPY", r2, "FWD")] + 1 == pos[("FWD", r2, "")] and pos[("COPY", r1, "GRAD")] + 1 == pos[("BWD", r1, "")]
    shard = core.perform_shard_expansion(g, inv, ms)
    placed = [(i["device"], i["op_type"]) for i in shard if i["task"] == "COPY"]
    assert len(placed) == 2
    on = {i["node"]: i["device"] for i in shard if i["task"] == "FWD" and i["node"] in (r1, r2)}
    assert on == {r1: 0, r2: 1}
    # each device's slice holds its own operator's forward and backward tasks
    for dev, node in ((0, r1), (1, r2)):
        sl = core.perform_machine_slicing(shard, dev)
        assert {i["task"] for i in sl if i.get("node") == node} >= {"FWD", "BWD"}
