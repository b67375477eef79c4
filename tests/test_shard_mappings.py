"""Operator task space -> tensor shard mappings, checked by arithmetic: a parallel Linear is executed one task at a
time -- every task reads the pieces of input, weight and bias that the mapping names and adds its product into the
output piece the mapping names -- and the assembled result must equal the unsharded layer.  Covers column-parallel
(replicated input), row-parallel (partial sums), data-parallel and hybrid layouts; plus the element-wise, transpose
and parallel-operator rules."""
import itertools

import pytest
import torch

from flexflow_train_b200 import _ffcore as core
from flexflow_train_b200.compiler import strategy as S


def _piece(full: torch.Tensor, shape, coord):
    """The shard `coord["shard"]` of a tensor with parallel shape `shape` (replicas of sum / discard-copy hold the same
    data here, except that only sum replica 0 of a partial-sum tensor carries the value)."""
    t = full
    for d, (deg, idx) in enumerate(zip(shape.degrees, coord["shard"])):
        n = t.shape[d] // deg
        t = t.narrow(d, idx * n, n)
    return t


def _run_linear(g, nid):
    node = g.node(nid)
    ins = {s: tuple(v) for s, v in node["inputs"]}
    xs, ws, ys = g.shape(ins["INPUT"]), g.shape(ins["WEIGHT"]), node["outputs"][0][1]
    assert xs.sum_degree == 1   # the test feeds whole inputs
    torch.manual_seed(0)
    x = torch.randn([int(v) for v in xs.sizes], dtype=torch.float64)
    w = torch.randn([int(v) for v in ws.sizes], dtype=torch.float64)
    b = torch.randn(int(ws.sizes[0]), dtype=torch.float64) if "BIAS" in ins else None
    bs = g.shape(ins["BIAS"]) if b is not None else None
    full = core.operator_full_task_degrees(g, nid)
    assert full == list(ys.degrees) + [ys.sum_degree, ys.discard_copy_degree]
    out = torch.zeros([int(v) for v in ys.sizes], dtype=torch.float64)
    tasks = 0
    for task in itertools.product(*[range(d) for d in full]):
        task = list(task)
        ci = core.operator_tensor_coord(g, nid, task, "INPUT", False)
        cw = core.operator_tensor_coord(g, nid, task, "WEIGHT", False)
        co = core.operator_tensor_coord(g, nid, task, "OUTPUT", True)
        assert ci["sum"] < xs.sum_degree and ci["discard_copy"] < xs.discard_copy_degree
        assert cw["discard_copy"] < ws.discard_copy_degree and cw["sum"] == 0
        y = _piece(x, xs, ci) @ _piece(w, ws, cw).t()
        if b is not None:
            cb = core.operator_tensor_coord(g, nid, task, "BIAS", False)
            assert cb["sum"] < bs.sum_degree and cb["discard_copy"] < bs.discard_copy_degree
            if task[-2] == 0:    # one task per output piece adds the bias: the one with sum component 0
                y = y + _piece(b, bs, cb)
        dst = _piece(out, ys, co)
        dst += y             # partial sums of different sum replicas land on the same output piece
        tasks += 1
    ref = x @ w.t() + (b if b is not None else 0)
    assert torch.allclose(out, ref, atol=1e-9), float((out - ref).abs().max())
    return tasks, full


def _first(g, typ, pred=lambda n: True):
    return next(n["id"] for n in g.nodes() if n["type"] == typ and pred(n))


def test_linear_tasks_assemble_to_the_full_layer_under_every_layout():
    cg = core.build_model("mlp", {"batch_size": 8})
    rules = core.get_substitution_set(core.MachineSpecification(1, 8))
    by_name = {r.name: r for r in rules}
    layouts = {}
    pcg = core.pcg_from_computation_graph(cg)
    for rule in ("replicate_linear_combine_4_bias", "partition_linear_reduce_4_bias", "partition_linear_combine_0_2_bias"):
        r = by_name[rule]
        m = core.find_pattern_matches(r, pcg)
        layouts[rule] = core.apply_substitution(pcg, r, m[0])
    layouts["hybrid"] = S.hybrid_strategy(cg, 2, 4, rules)
    seen = set()
    for name, g in layouts.items():
        for n in g.nodes():
            if n["type"] != "LINEAR" or n["outputs"][0][1].total_degree == 1:
                continue
            tasks, full = _run_linear(g, n["id"])
            seen.add((name, tuple(full)))
            assert tasks == n["outputs"][0][1].total_degree
    kinds = {f for _, f in seen}
    assert any(f[-2] > 1 for f in kinds) and any(f[-3] > 1 for f in kinds) and any(f[0] > 1 for f in kinds)  # row, column, batch
    assert any(f[0] > 1 and (f[-2] > 1 or f[-3] > 1) for f in kinds)                                         # hybrid


def test_elementwise_transpose_and_parallel_operator_mappings():
    cg = core.build_model("transformer_lm", {"num_features": 32, "sequence_length": 8, "batch_size": 8, "dim_feedforward": 64,
                                             "num_heads": 2, "num_decoder_layers": 1, "vocab_size": 32})
    g = S.data_parallel_strategy(cg, 4)
    rep = _first(g, "REPARTITION")
    full = core.operator_full_task_degrees(g, rep)
    k = int(g.node(rep)["attrs"]["repartition_degree"])
    for t in range(full[0]):
        task = [t] + [0] * (len(full) - 1)
        assert core.operator_tensor_coord(g, rep, task, "OUTPUT", True)["shard"][0] == t
        assert core.operator_tensor_coord(g, rep, task, "INPUT", False)["shard"][0] == t // k
    comb = _first(g, "COMBINE")
    fullc = core.operator_full_task_degrees(g, comb)
    kc = int(g.node(comb)["attrs"]["combine_degree"])
    last = [fullc[0] - 1] + [0] * (len(fullc) - 1)
    assert core.operator_tensor_coord(g, comb, last, "INPUT", False)["shard"][0] == fullc[0] - 1
    assert core.operator_tensor_coord(g, comb, last, "OUTPUT", True)["shard"][0] == (fullc[0] - 1) // kc
    rpl = _first(g, "REPLICATE")
    fr = core.operator_full_task_degrees(g, rpl)
    kr = int(g.node(rpl)["attrs"]["replicate_degree"])
    task = [0] * (len(fr) - 1) + [fr[-1] - 1]
    assert core.operator_tensor_coord(g, rpl, task, "INPUT", False)["discard_copy"] == (fr[-1] - 1) // kr
    add = _first(g, "EW_ADD")
    fa = core.operator_full_task_degrees(g, add)
    task = [fa[0] - 1] + [0] * (len(fa) - 1)
    for slot in ("LHS_INPUT", "RHS_INPUT"):
        assert core.operator_tensor_coord(g, add, task, slot, False)["shard"] == task[:-2]
    tp = S.tensor_parallel_strategy(cg, 2, sequence_parallel=False)
    red = _first(tp, "REDUCTION")
    fd = core.operator_full_task_degrees(tp, red)
    task = [0] * (len(fd) - 2) + [fd[-2] - 1, 0]
    assert core.operator_tensor_coord(tp, red, task, "OUTPUT", True)["sum"] == 0
    assert core.operator_tensor_coord(tp, red, task, "INPUT", False)["sum"] == fd[-2] - 1
    # transpose: output dim i is input dim perm[i]
    b = core.GraphBuilder()
    x = b.create_input([4, 6, 8], name="x")
    b.transpose(x, [0, 2, 1], name="t")
    pg = core.pcg_from_computation_graph(b.graph)
    tnode = _first(pg, "TRANSPOSE")
    assert core.operator_tensor_coord(pg, tnode, [0, 0, 0, 0, 0], "INPUT", False)["shard"] == [0, 0, 0]
    with pytest.raises(core.CoreError):
        core.operator_tensor_coord(pg, tnode, [1, 0, 0, 0, 0], "INPUT", False)      # outside the (all-ones) task space
    att = _first(g, "MULTIHEAD_ATTENTION")
    with pytest.raises(core.CoreError):   # no mapping for attention (nor in the reference)
        core.operator_tensor_coord(g, att, [0] * len(core.operator_full_task_degrees(g, att)), "QUERY", False)


def test_tensor_set_movement_lists_the_pieces_that_change_device():
    """Producer and consumer on the same view: nothing moves.  The consumer's view shifted to other devices: every
    piece travels once, from the device that made it to the device that reads it."""
    cg = core.build_model("mlp", {"batch_size": 8})
    ms = core.MachineSpecification(1, 8)
    est = core.CostEstimator(ms)
    g = S.data_parallel_strategy(cg, 4)
    rep = _first(g, "REPARTITION", lambda n: g.node(tuple(n["inputs"][0][1])[0])["type"] == "INPUT")
    lin = g.consumers((rep, "OUTPUT"))[0][0]
    assert g.node(lin)["type"] == "LINEAR"
    lo, hi = core.allowed_machine_views([4], 0, 8, ms)            # devices 0-3 and 4-7
    assert core.get_tensor_set_movement(g, rep, lo, lin, lo, ms) == []
    edges = core.get_tensor_set_movement(g, rep, lo, lin, hi, ms)
    piece = g.shape((rep, "OUTPUT")).piece_bytes
    assert sorted((e["src"], e["dst"]) for e in edges) == [(0, 4), (1, 5), (2, 6), (3, 7)]
    assert all(e["bytes"] == piece for e in edges)
    assert core.tensor_set_movement_cost_ms(g, rep, lo, lin, hi, ms, est) == pytest.approx(est.movement_cost_ms(piece, False))
    assert core.tensor_set_movement_cost_ms(g, rep, lo, lin, lo, ms, est) == 0.0
    # column-parallel Linear: replica c of the input feeds the task that computes output-channel shard c
    rules = core.get_substitution_set(ms)
    r = {x.name: x for x in rules}["replicate_linear_combine_4_bias"]
    pcg = core.pcg_from_computation_graph(cg)
    tp = core.apply_substitution(pcg, r, core.find_pattern_matches(r, pcg)[0])
    lin2 = _first(tp, "LINEAR", lambda n: n["outputs"][0][1].total_degree == 4)
    src = dict((s, tuple(v)) for s, v in tp.node(lin2)["inputs"])["INPUT"]
    assert tp.node(src[0])["type"] == "REPLICATE"
    assert core.get_tensor_set_movement(tp, src[0], lo, lin2, lo, ms) == []
    moved = core.get_tensor_set_movement(tp, src[0], lo, lin2, hi, ms)
    assert sorted((e["src"], e["dst"]) for e in moved) == [(0, 4), (1, 5), (2, 6), (3, 7)]


def test_strategies_evaluated_shard_by_shard_give_the_unsharded_result():
    """The PCG executed the way its degrees say (pieces cut by Repartition, copied by Replicate, added by Reduction,
    concatenated by Combine; one Linear product per task) reproduces the computation graph's output."""
    from flexflow_train_b200.runtime.spmd_sim import ShardedEvaluation
    from flexflow_train_b200.runtime.torch_oracle import TorchOracle

    cg = core.build_model("mlp", {"batch_size": 8})
    oracle = TorchOracle(cg, seed=5)
    params = {k: v.detach().double() for k, v in oracle.params.items()}
    torch.manual_seed(0)
    inputs = {n["name"]: torch.randn([int(v) for v in n["outputs"][0][1].sizes], dtype=torch.float64)
              for n in cg.nodes() if n["type"] == "INPUT"}
    ref = ShardedEvaluation(core.pcg_from_computation_graph(cg), params, inputs)
    sink = tuple(cg.sink_values()[-1])
    want = ref.assemble(sink)
    assert torch.allclose(want.float(), oracle.forward({k: v.float() for k, v in inputs.items()}).detach(), atol=1e-5)
    rules = core.get_substitution_set(core.MachineSpecification(1, 8))
    strategies = {"dp4": S.data_parallel_strategy(cg, 4, rules), "tp4": S.tensor_parallel_strategy(cg, 4, rules),
                  "tp4_replicated": S.tensor_parallel_strategy(cg, 4, rules, sequence_parallel=False),
                  "dp2xtp4": S.hybrid_strategy(cg, 2, 4, rules)}
    for name, g in strategies.items():
        ev = ShardedEvaluation(g, params, inputs)
        out_value = tuple(g.sink_values()[-1])
        got = ev.assemble(out_value)
        assert torch.allclose(got, want, atol=1e-9), (name, float((got - want).abs().max()))
        # the strategy really ran sharded: some Linear was computed in more than one task
        assert any(len(p) > 1 for (nid, _), p in ev.pieces.items() if ev.nodes[nid]["type"] == "LINEAR"), name
