"""Machine views, machine-mapping DP, Unity / MCMC search, simulator (reference: lib/compiler/test)."""
import itertools

import pytest

from flexflow_train_b200 import _ffcore as c
from flexflow_train_b200.compiler import strategy as S


def test_allowed_machine_views_are_contiguous_and_aligned():
    ms = c.MachineSpecification(1, 8)
    v = c.allowed_machine_views([4], 0, 8, ms)
    assert len(v) == 2
    assert [c.view_devices(x, [4], ms) for x in v] == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert c.view_devices(c.allowed_machine_views([2, 2], 4, 4, ms)[0], [2, 2], ms) == [4, 5, 6, 7]
    assert c.allowed_machine_views([16], 0, 8, ms) == []
    ms2 = c.MachineSpecification(2, 4)
    v = c.allowed_machine_views([2, 4], 0, 8, ms2)
    assert v[0]["dimensions"][0]["projection"] == "INTER_NODE" and v[0]["dimensions"][1]["projection"] == "INTRA_NODE"
    assert c.view_devices(v[0], [2, 4], ms2) == list(range(8))


def _chain(n_par, batch=64, width=256):
    """input -> n_par parallel dense branches -> sum: a graph with a parallel split in its SP tree."""
    b = c.GraphBuilder()
    x = b.create_input([batch, width], "FLOAT")
    ys = [b.dense(x, width, "RELU", False) for _ in range(n_par)]
    y = ys[0]
    for z in ys[1:]:
        y = b.binary("EW_ADD", y, z)
    b.softmax(y)
    return b.graph


@pytest.mark.parametrize("batch,width", [(64, 256), (8192, 8192)])
def test_mapping_dp_matches_brute_force_on_parallel_split(batch, width):
    g = _chain(2, batch, width)
    ms = c.MachineSpecification(1, 2)
    est = c.CostEstimator(ms)
    pts = c.get_optimal_machine_mapping(g, None, ms, est, 1)
    assert len(pts) == 1
    dp_cost = pts[0]["runtime_ms"]
    # brute force: either everything in series on one device, or the two branch Linears side by side on the two
    # devices, which costs one transfer of a branch output (forward) and of its gradient (backward)
    costs = {n["id"]: sum(est.op_cost(g, n["id"])[k] for k in ("fwd_ms", "bwd_ms")) for n in g.nodes()}
    lin = [n["id"] for n in g.nodes() if n["type"] == "LINEAR"]
    serial = sum(costs.values())
    move = 2 * est.movement_cost_ms(batch * width * 4, False)
    split = serial - min(costs[l] for l in lin) + 2 * move  # the branch input travels too
    assert abs(dp_cost - min(serial, split)) < 1e-6 * serial
    used = {tuple(c.view_devices(v, [], ms)) for v in pts[0]["views"].values()}
    assert used == ({(0,)} if serial <= split else {(0,), (1,)})


def test_memory_pareto_front():
    g = _chain(2)
    ms = c.MachineSpecification(1, 2)
    pts = c.get_optimal_machine_mapping(g, None, ms, c.CostEstimator(ms), 4)
    assert len(pts) >= 1
    for a, b_ in itertools.combinations(pts, 2):  # no point dominates another
        assert not (a["runtime_ms"] <= b_["runtime_ms"] and a["memory_bytes"] <= b_["memory_bytes"]) or a == b_


def test_unity_search_improves_mlp_and_respects_budget():
    g = c.build_model("mlp", {"batch_size": 4096, "input_dim": 4096, "hidden": [8192, 8192], "num_classes": 4096})
    ms = c.MachineSpecification(1, 4)
    est = c.CostEstimator(ms)
    rules = c.get_substitution_set(ms)
    base = c.evaluate_pcg(g, ms, est)["runtime_ms"]
    r0 = c.unity_search(g, ms, est, rules, 1.05, 0, 100000, 60.0)
    assert r0["runtime_ms"] == base and r0["stats"]["iterations"] == 0
    r = c.unity_search(g, ms, est, rules, 1.3, 6, 100000, 60.0)
    assert r["runtime_ms"] < base and r["stats"]["evaluated"] > 10
    assert any(n["type"] in ("REPARTITION", "REPLICATE") for n in r["pcg"].nodes())
    assert r["mapped_pcg"].is_mapped()


def test_mcmc_is_deterministic_under_a_seed():
    g = c.build_model("mlp", {"batch_size": 1024, "input_dim": 1024, "hidden": [2048], "num_classes": 1024})
    ms = c.MachineSpecification(1, 4)
    est = c.CostEstimator(ms)
    rules = c.get_substitution_set(ms)
    a = c.mcmc_search(g, ms, est, rules, 1.0, 40, 0.3, 0)
    b_ = c.mcmc_search(g, ms, est, rules, 1.0, 40, 0.3, 0)
    assert a["runtime_ms"] == b_["runtime_ms"] and a["stats"] == b_["stats"]
    assert a["pcg"].signature() == b_["pcg"].signature()
    d = c.mcmc_search(g, ms, est, rules, 1.0, 40, 0.3, 1)
    assert d["stats"]["iterations"] == 40


def test_simulator_forward_vs_forward_backward():
    g = _chain(2)
    ms = c.MachineSpecification(1, 2)
    est = c.CostEstimator(ms)
    m = c.evaluate_pcg(g, ms, est)["mapped_pcg"]
    f = c.simulate_task_graph(m, ms, est, False)
    fb = c.simulate_task_graph(m, ms, est, True)
    assert 0 < f < fb


def test_measured_costs_override_the_analytical_model():
    g = c.build_model("mlp", {"batch_size": 64})
    ms = c.MachineSpecification(1, 1)
    est = c.CostEstimator(ms)
    lin = [n["id"] for n in g.nodes() if n["type"] == "LINEAR"][0]
    before = est.op_cost(g, lin)["fwd_ms"]
    est.set_measured(est.op_cost_key(g, lin), 123.0, 456.0, 1.0)
    after = est.op_cost(g, lin)
    assert before != 123.0 and after["fwd_ms"] == 123.0 and after["bwd_ms"] == 456.0


def test_optimize_picks_data_parallel_for_large_transformer_and_exports():
    cfg = {"num_features": 1024, "sequence_length": 512, "batch_size": 16, "dim_feedforward": 4096, "num_heads": 8,
           "num_decoder_layers": 2, "dropout": 0.1, "vocab_size": 8192}
    g = c.build_model("transformer_lm", cfg)
    r = S.optimize(g, world=8, algorithm="unity", budget=0)
    assert r["stats"]["seed_strategy"].startswith("dp8")
    assert set(r["stats"]["candidates"]) == {"single_device", "dp8", "tp8", "dp4xtp2", "dp2xtp4"}
    text = r["mapped_pcg"].to_v1_string(parallel=True)
    back = c.Graph.from_v1(text)
    assert back.signature() == r["mapped_pcg"].signature()
    tp = S.tensor_parallel_strategy(g, 8)
    k = {}
    for n in tp.nodes():
        k[n["type"]] = k.get(n["type"], 0) + 1
    assert k["REDUCTION"] == 4 and k["REPLICATE"] >= 4  # attention + row-parallel FFN per layer


def test_data_parallel_strategy_shards_every_operator_of_every_model_family():
    """The sample-dim rules cover convolution stacks (conv, batch norm, pooling, concat, flat), recommendation
    models (embedding, cast, concat) and MLPs: no operator is left replicated, and activations cross ranks only at
    the model's inputs and outputs."""
    for name, cfg in (("inception_v3", {"batch_size": 8}), ("dlrm", {"batch_size": 16}), ("candle_uno", {"batch_size": 8}),
                      ("bert", {"batch_size": 4, "token_ids": True, "num_encoder_layers": 2})):
        cg = c.build_model(name, cfg)
        g = S.data_parallel_strategy(cg, 2)
        nodes = {n["id"]: n for n in g.nodes()}
        replicated = [n["type"] for n in g.nodes() if not c.is_parallel_op(n["type"]) and n["type"] not in ("WEIGHT", "INPUT")
                      and n["outputs"][0][1].total_degree == 1]
        assert replicated == [], (name, replicated)
        n_inputs = sum(1 for n in cg.nodes() if n["type"] == "INPUT")
        n_sinks = len([v for v in cg.sink_values() if nodes.get(v[0], {"type": ""})["type"] not in ("WEIGHT", "INPUT")])
        moves = [n for n in g.nodes() if n["type"] in ("REPARTITION", "COMBINE")
                 and nodes[n["inputs"][0][1][0]]["type"] != "WEIGHT" and not c.is_parallel_op(nodes[n["inputs"][0][1][0]]["type"])]
        assert len(moves) <= n_inputs + max(n_sinks, 2), (name, len(moves))


def test_table_parallel_strategy_keeps_lookups_whole_and_shards_the_rest():
    """Recommendation-model layout: Embeddings and the Concat stacking them stay unpartitioned (placed per table),
    one Repartition(0) hands the stack to the data-parallel rest, and no table is replicated."""
    cfg = {"batch_size": 64, "embedding_dim": 16, "embedding_bag_size": 1, "embedding_size": [500, 300, 200, 100],
           "dense_arch_layer_sizes": [13, 32, 16], "over_arch_layer_sizes": [48, 32, 1], "arch_interaction_op": "DOT",
           "embedding_data_type": "FLOAT"}
    cg = c.build_model("dlrm", cfg)
    assert S.has_stacked_embeddings(cg)
    g = S.table_parallel_strategy(cg, 4)
    nodes = {n["id"]: n for n in g.nodes()}
    embs = [n for n in nodes.values() if n["type"] == "EMBEDDING"]
    assert len(embs) == 4
    for e in embs:
        assert e["outputs"][0][1].total_degree == 1
        w = dict((s, tuple(v)) for s, v in e["inputs"])["WEIGHT"]
        assert nodes[w[0]]["type"] == "WEIGHT"  # no Replicate / Repartition between the table and its lookup
    stacks = [n for n in nodes.values() if n["type"] == "CONCAT" and n["outputs"][0][1].total_degree == 1]
    assert len(stacks) == 1
    cons = g.consumers((stacks[0]["id"], "OUTPUT"))
    assert len(cons) == 1 and nodes[cons[0][0]]["type"] == "REPARTITION"
    rep = nodes[cons[0][0]]
    assert rep["outputs"][0][1].degrees[0] == 4
    for n in nodes.values():
        if n["type"] == "LINEAR":
            assert n["outputs"][0][1].degrees[0] == 4
    # the search offers it as a candidate next to pure data parallelism, and it is far cheaper than replicating tables
    r = S.optimize(cg, world=4)
    cands = r["stats"]["candidates"]
    assert "dp4+tables_mp4" in cands and cands["dp4+tables_mp4"] <= cands["dp4"]
    forced = S.optimize(cg, world=4, algorithm="table_parallel")
    assert forced["stats"]["seed_strategy"] == "dp4+tables_mp4"
    with pytest.raises(ValueError):
        S.table_parallel_strategy(c.build_model("mlp", {}), 2)


def test_substitution_json_rules_join_the_search(tmp_path):
    """FFConfig.substitution_json_path (the reference's --substitution-json): a legacy rule collection is loaded and
    offered to the search next to the generated rules."""
    import json
    import os

    from flexflow_train_b200.api import FFConfig

    ref = os.path.join(os.environ.get("FF_REFERENCE_DIR") or
                       os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"),
                       "substitutions", "test_subst.json")
    if not os.path.exists(ref):
        pytest.skip("legacy rule files not available")
    cg = c.build_model("mlp", {})
    cfg = FFConfig(batch_size=64, search_budget=4, substitution_json_path=ref)
    pcg, stats = S.choose_strategy(cg, 2, cfg)
    assert stats["substitution_json"]["rules_in_file"] == 1 and stats["substitution_json"]["rules_loaded"] == 1
    assert "unity" in stats and len(pcg.nodes()) > 0
    json.dumps(stats["substitution_json"])


def test_parameter_and_attribute_parallel_flags_restrict_the_search():
    ms = c.MachineSpecification(1, 4)
    rules = c.get_substitution_set(ms)
    names = [r.name for r in rules]
    assert any(S.is_parameter_parallel_rule(n) for n in names) and any(S.is_attribute_parallel_rule(n) for n in names)
    assert S.is_attribute_parallel_rule("partition_RELU_combine_1_4") and not S.is_attribute_parallel_rule("partition_RELU_combine_0_4")
    assert not S.is_attribute_parallel_rule("partition_conv2d_combine_4_bias")
    assert S.is_attribute_parallel_rule("partition_linear_combine_1_2_bias") and S.is_parameter_parallel_rule("replicate_linear_combine_4")
    kept = S.filter_rules(rules, enable_parameter_parallel=False, enable_attribute_parallel=False)
    assert kept and not any(S.is_parameter_parallel_rule(r.name) or S.is_attribute_parallel_rule(r.name) for r in kept)
    assert len(S.filter_rules(rules)) == len(rules)
    cg = c.build_model("transformer_lm", {"num_features": 64, "sequence_length": 16, "batch_size": 8, "dim_feedforward": 128,
                                          "num_heads": 2, "num_decoder_layers": 1, "vocab_size": 64})
    full = S.optimize(cg, world=2)
    no_pp = S.optimize(cg, world=2, enable_parameter_parallel=False)
    assert "tp2" in full["stats"]["candidates"] and "tp2" not in no_pp["stats"]["candidates"]


def test_compile_on_cpu_exports_strategy_and_graph_files(tmp_path):
    """api.compile(device="cpu") trains on the host executor; the strategy JSON and the dot file of the chosen
    graph are written where FFConfig says."""
    import torch

    from flexflow_train_b200 import api
    from flexflow_train_b200.runtime.executor import OptimizerConfig

    cfg = api.FFConfig(batch_size=16, export_strategy_file=str(tmp_path / "strategy.json"),
                       export_strategy_computation_graph_file=str(tmp_path / "pcg.dot"))
    cm = api.compile("mlp", {"batch_size": 16}, config=cfg, optimizer=OptimizerConfig(kind="sgd", lr=0.1), device="cpu")
    g = cm.graph
    ins = {}
    for n in g.nodes():
        if n["type"] == "INPUT":
            ins[n["name"]] = torch.randn([int(v) for v in n["outputs"][0][1].sizes])
    out_sizes = [int(v) for v in g.shape(cm.executable.loss_value).sizes]
    labels = torch.randint(0, out_sizes[-1], (out_sizes[0],), dtype=torch.int32)
    losses = [cm.train_step(ins, labels) for _ in range(5)]
    assert losses[-1] < losses[0]
    assert (tmp_path / "pcg.dot").read_text().lstrip().startswith("digraph")
    assert c.Graph.from_v1((tmp_path / "strategy.json").read_text()).signature() == g.signature()


def test_hybrid_data_x_tensor_parallel_strategy_is_clean_and_scored():
    """dp2 x tp4 on 8 devices: the commute rules bring every data-parallel Combine next to the following Repartition,
    so only the input Repartition and the output Combine remain around the tensor-parallel collectives."""
    cfg = {"num_features": 128, "sequence_length": 32, "batch_size": 16, "dim_feedforward": 256, "num_heads": 8,
           "num_decoder_layers": 2, "vocab_size": 256}
    cg = c.build_model("transformer_lm", cfg)
    assert all(r.is_valid() for r in c.get_commute_rules())
    g = S.hybrid_strategy(cg, 2, 4)
    nodes = {n["id"]: n for n in g.nodes()}
    act_parallel = [n for n in nodes.values() if n["type"] in ("COMBINE", "REPARTITION")
                    and nodes[tuple(n["inputs"][0][1])[0]]["type"] != "WEIGHT"]
    assert sorted(n["type"] for n in act_parallel) == ["COMBINE", "REPARTITION"]
    lin = [n["outputs"][0][1] for n in nodes.values() if n["type"] == "LINEAR"]
    assert any(list(sh.degrees) == [2, 1, 4] for sh in lin) and any(sh.sum_degree == 4 and sh.degrees[0] == 2 for sh in lin)
    assert max(n["outputs"][0][1].total_degree for n in nodes.values()) == 8
    text = g.to_v1_string(parallel=True)
    assert c.Graph.from_v1(text).signature() == g.signature()
    # the mesh strategies are candidates of the search like the one-axis templates (the executor runs them)
    r = S.optimize(cg, world=8)
    cands = r["stats"]["candidates"]
    assert {"dp4xtp2", "dp2xtp4", "dp8", "tp8", "single_device"} <= set(cands) and all(v > 0 for v in cands.values())
    assert r["runtime_ms"] == min(cands.values())
    assert "dp4xtp2" not in S.optimize(cg, world=8, only_data_parallel=True)["stats"]["candidates"]


def test_every_strategy_template_computes_the_function_of_the_computation_graph():
    """Parallel operators are the identity on the logical tensor, so a strategy evaluated as a plain graph must give
    the loss and gradients of the computation graph it came from -- bit for bit.  This pins the wiring that the
    substitutions (including the commute and cancellation rules of the hybrid builder) leave behind."""
    import torch

    from flexflow_train_b200.runtime.torch_oracle import TorchOracle

    cfg = {"num_features": 64, "sequence_length": 16, "batch_size": 8, "dim_feedforward": 128, "num_heads": 4,
           "num_decoder_layers": 2, "vocab_size": 64, "dropout": 0.0}
    cg = c.build_model("transformer_lm", cfg)
    torch.manual_seed(0)
    ids = torch.randint(0, 64, (8, 16, 1), dtype=torch.int32)
    labels = torch.randint(0, 64, (8, 16), dtype=torch.int32)
    rows0, grads0 = TorchOracle(cg, seed=3).loss_and_grads({"input_ids": ids}, labels)
    strategies = {"dp4": S.data_parallel_strategy(cg, 4), "tp4": S.tensor_parallel_strategy(cg, 4),
                  "tp4_replicated": S.tensor_parallel_strategy(cg, 4, sequence_parallel=False),
                  "dp2xtp4": S.hybrid_strategy(cg, 2, 4), "dp4xtp2": S.hybrid_strategy(cg, 4, 2),
                  "searched8": S.optimize(cg, world=8, budget=4)["mapped_pcg"]}
    for name, g in strategies.items():
        rows, grads = TorchOracle(g, seed=3).loss_and_grads({"input_ids": ids}, labels)
        assert torch.equal(rows, rows0), name
        assert set(grads) == set(grads0), name
        for k in grads0:
            assert torch.equal(grads[k], grads0[k]), (name, k)
    dl = {"batch_size": 16, "embedding_dim": 8, "embedding_bag_size": 1, "embedding_size": [50, 30, 20, 10],
          "dense_arch_layer_sizes": [13, 16, 8], "over_arch_layer_sizes": [24, 16, 1], "arch_interaction_op": "DOT",
          "final_activation": "SIGMOID", "embedding_data_type": "FLOAT"}
    dcg = c.build_model("dlrm", dl)
    ins = {"dense": torch.randn(16, 13)}
    for i, n in enumerate(dl["embedding_size"]):
        ins[f"sparse{i}"] = torch.randint(0, n, (16, 1))
    y = torch.rand(16, 1)
    a = TorchOracle(dcg, seed=1, loss="mean_squared_error_avg_reduce").loss_and_grads(ins, y)
    b = TorchOracle(S.table_parallel_strategy(dcg, 4), seed=1, loss="mean_squared_error_avg_reduce").loss_and_grads(ins, y)
    assert torch.equal(a[0], b[0]) and all(torch.equal(a[1][k], b[1][k]) for k in a[1])


def test_cost_table_file_feeds_the_search_estimator(tmp_path):
    """A table of measured operator costs on disk is what the search's estimator answers from (the reference's
    LocalCostEstimator answers from measurements); shapes that were not measured keep the analytic estimate."""
    import json

    from flexflow_train_b200.api import FFConfig, _search_estimator
    from flexflow_train_b200.compiler.strategy import choose_strategy, machine_for
    from flexflow_train_b200.runtime.executor import ExecConfig
    cg = c.build_model("mlp", {"batch_size": 8})
    probe = c.CostEstimator(machine_for(2))
    lin = [n["id"] for n in cg.nodes() if n["type"] == "LINEAR"][0]
    key = probe.op_cost_key(cg, lin)
    analytic = probe.op_cost(cg, lin)
    path = tmp_path / "costs.json"
    path.write_text(json.dumps({key: {"fwd_ms": 123.0, "bwd_ms": 456.0, "memory_bytes": 10.0}}))
    cfg = FFConfig(cost_table_file=str(path))
    est, info = _search_estimator("mlp", {"batch_size": 8}, cg, 2, cfg, None, ExecConfig())
    assert info == {"source": str(path), "entries": 1}
    measured = est.op_cost(cg, lin)
    assert measured != analytic and abs(measured["fwd_ms"] - 123.0) < 1e-6 and abs(measured["bwd_ms"] - 456.0) < 1e-6
    strategy, stats = choose_strategy(cg, 2, cfg, estimator=est)
    assert strategy is not None and "candidates" in stats
    # no table and no measurement asked for: the search builds its own analytic estimator
    assert _search_estimator("mlp", None, cg, 2, FFConfig(), None, ExecConfig()) == (None, None)


def test_strided_machine_views_interleave_inside_a_node():
    """With strided=True the tasks may sit on every s-th device (the reference's MachineView stride); the contiguous views
    come first and are all the mapping search asks for on a uniform NVSwitch node."""
    ms = c.MachineSpecification(1, 8)
    views = c.allowed_machine_views([4], 0, 8, ms, strided=True)
    devs = [c.view_devices(v, [4], ms) for v in views]
    assert devs == [[0, 1, 2, 3], [4, 5, 6, 7], [0, 2, 4, 6], [1, 3, 5, 7]]
    assert [v["dimensions"][0]["stride"] for v in views] == [1, 1, 2, 2]
    two = [c.view_devices(v, [2, 2], ms) for v in c.allowed_machine_views([2, 2], 0, 8, ms, strided=True)]
    assert [0, 1, 2, 3] in two and [0, 2, 4, 6] in two and [1, 3, 5, 7] in two
    for d in two:
        assert len(set(d)) == 4 and all(0 <= x < 8 for x in d)
    # a strided view round-trips through the strategy file format like any other
    assert c.allowed_machine_views([4], 0, 8, ms) == views[:2]


def test_measured_collective_bandwidths_price_the_parallel_operators():
    """The cost of a collective comes from the bandwidth measured for its kind at (the nearest smaller measured) group size;
    kinds and sizes that were not measured keep the nominal NVLink figures."""
    ms = S.machine_for(8)
    base = c.CostEstimator(ms).params()
    assert base["measured_gbs"]["allreduce@8"] == 513.0 and base["measured_gbs"]["reducescatter@8"] == 172.0
    b = c.GraphBuilder(True)
    x = b.create_input([64, 4096], "FLOAT", False, "x")
    r = b.parallel_replicate(x, 8)
    y = b.parallel_partition(x, 0, 4)
    g = b.graph
    rep = [n["id"] for n in g.nodes() if n["type"] == "REPLICATE"][0]
    part = [n["id"] for n in g.nodes() if n["type"] == "REPARTITION"][0]
    slow = c.CostEstimator(ms, dict(base, measured_gbs={"allreduce@8": 51.3, "allgather@2": 77.0}))
    fast = c.CostEstimator(ms, dict(base, measured_gbs={}))
    lat = base["collective_latency_us"] / 1000.0
    t_meas, t_slow, t_nom = (e.op_cost(g, rep)["bwd_ms"] - lat for e in (c.CostEstimator(ms), slow, fast))
    assert abs(t_slow / t_meas - 10.0) < 1e-6                      # a tenth of the bandwidth, ten times the transfer time
    assert abs(t_nom / t_meas - 513.0 / base["allreduce_bus_gbs"]) < 1e-6
    # a 4-way all-gather: priced with the 2-way measurement when that is the nearest smaller one, nominal otherwise
    g4_slow, g4_nom = (e.op_cost(g, part)["bwd_ms"] - lat for e in (slow, fast))
    assert abs(g4_slow / g4_nom - base["nvlink_gbs"] / 77.0) < 1e-6


def test_cost_params_file_overrides_the_analytic_model(tmp_path):
    import json

    from flexflow_train_b200.api import FFConfig, _search_estimator
    from flexflow_train_b200.runtime.executor import ExecConfig
    path = tmp_path / "params.json"
    path.write_text(json.dumps({"measured_gbs": {"allreduce@4": 333.0}, "launch_us": 9.0}))
    cg = c.build_model("mlp", {"batch_size": 8})
    est, info = _search_estimator("mlp", None, cg, 4, FFConfig(cost_params_file=str(path)), None, ExecConfig())
    p = est.params()
    assert p["launch_us"] == 9.0 and p["measured_gbs"]["allreduce@4"] == 333.0 and p["measured_gbs"]["allreduce@8"] == 513.0
    assert info["source"] == "analytic" and info["cost_params"] == str(path)


# ------------------------------------------------------------------ generic event-driven task-graph execution
# cases and expected traces of the reference's test (lib/compiler/test/src/compiler/task_graph_simulator/
# simulate_task_graph_execution.cc)
def _trace(n, edges, cost, allowed):
    return sorted(c.simulate_task_graph_execution(n, edges, [float(x) for x in cost], allowed))


ALWAYS = lambda t, running, done: True            # noqa: E731
ONE_AT_A_TIME = lambda t, running, done: len(running) == 0   # noqa: E731


def test_task_graph_execution_linear():
    assert _trace(4, [(0, 1), (1, 2), (2, 3)], [1, 10, 100, 1000], ALWAYS) == [(0, 0, 1), (1, 1, 11), (2, 11, 111), (3, 111, 1111)]


def test_task_graph_execution_rhombus():
    edges, cost = [(0, 1), (0, 2), (1, 3), (2, 3)], [10, 15, 20, 25]
    assert _trace(4, edges, cost, ALWAYS) == [(0, 0, 10), (1, 10, 25), (2, 10, 30), (3, 30, 55)]
    assert _trace(4, edges, cost, ONE_AT_A_TIME) == [(0, 0, 10), (1, 10, 25), (2, 25, 45), (3, 45, 70)]


def test_task_graph_execution_diamond_with_crossing():
    edges = [(0, 1), (0, 2), (1, 3), (2, 3), (2, 4), (3, 5), (4, 5)]
    cost = [10, 15, 20, 25, 30, 35]
    assert _trace(6, edges, cost, ALWAYS) == [(0, 0, 10), (1, 10, 25), (2, 10, 30), (3, 30, 55), (4, 30, 60), (5, 60, 95)]
    assert _trace(6, edges, cost, ONE_AT_A_TIME) == [(0, 0, 10), (1, 10, 25), (2, 25, 45), (3, 45, 70), (4, 70, 100), (5, 100, 135)]


def test_task_graph_execution_all_to_all_with_two_slots():
    edges = [(0, 1), (0, 2), (0, 3), (1, 4), (2, 4), (3, 4)]
    at_most_two = lambda t, running, done: len(running) < 2   # noqa: E731
    assert _trace(5, edges, [10, 100, 100, 100, 20], at_most_two) == [(0, 0, 10), (1, 10, 110), (2, 10, 110), (3, 110, 210), (4, 210, 230)]


def test_task_graph_execution_constraint_sees_finished_tasks_and_stuck_graphs_are_errors():
    seen = []
    def allowed(t, running, done):
        seen.append((t, frozenset(running), frozenset(done)))
        return True
    _trace(3, [(0, 2), (1, 2)], [5, 7, 1], allowed)
    assert (2, frozenset(), frozenset({0, 1})) in seen          # task 2 is offered once both producers have finished
    with pytest.raises(Exception):
        _trace(2, [(0, 1), (1, 0)], [1, 1], ALWAYS)              # a cycle: nothing can ever start
    with pytest.raises(Exception):
        _trace(2, [], [1, 1], lambda t, running, done: t == 0)   # task 1 is refused for ever
    with pytest.raises(Exception):
        _trace(2, [(0, 5)], [1, 1], ALWAYS)


def test_pcg_simulation_of_a_branching_graph_is_deterministic_and_grows_with_backward():
    # the split_test model has parallel branches; on one device every task serialises: the simulated forward time of the
    # mapped graph equals the sum of its operators' forward costs, and backward adds to it
    g = c.build_model("split_test", {"batch_size": 8})
    ms = c.MachineSpecification(1, 1)
    est = c.CostEstimator(ms)
    m = c.evaluate_pcg(c.pcg_from_computation_graph(g), ms, est)["mapped_pcg"]
    f = c.simulate_task_graph(m, ms, est, False)
    fb = c.simulate_task_graph(m, ms, est, True)
    assert 0 < f < fb and f == c.simulate_task_graph(m, ms, est, False)
    total = sum(est.op_cost(m, n["id"])["fwd_ms"] for n in m.nodes()) if hasattr(est, "op_cost") else None
    if total is not None:
        assert abs(f - total) < 1e-6 * max(1.0, total)


# ------------------------------------------------------------------ machine views with the reference's stride semantics
# golden values of lib/compiler/test/src/compiler/machine_mapping/{machine_view,allowed_machine_views}.cc
def _view(node, dev, *dims):
    return {"start": {"node_idx": node, "device_idx": dev, "device_type": "GPU"},
            "dimensions": [{"stride": s, "projection": p} for s, p in dims]}


INTRA, INTER = "INTRA_NODE", "INTER_NODE"


@pytest.mark.parametrize("view,degrees,expected", [
    (_view(0, 1, (2, INTRA)), [3], {(0,): (0, 1), (1,): (0, 3), (2,): (0, 5)}),
    (_view(1, 2, (1, INTER), (2, INTRA)), [2, 2], {(0, 0): (1, 2), (0, 1): (1, 4), (1, 0): (2, 2), (1, 1): (2, 4)}),
    (_view(1, 0, (1, INTRA), (2, INTRA)), [2, 2], {(0, 0): (1, 0), (0, 1): (1, 4), (1, 0): (1, 1), (1, 1): (1, 5)}),
    (_view(0, 1, (1, INTER), (2, INTRA), (1, INTRA)), [2, 2, 2], {(0, 1, 0): (0, 3), (1, 0, 1): (1, 5), (1, 1, 1): (1, 7)}),
])
def test_reference_machine_coordinates(view, degrees, expected):
    for coord, where in expected.items():
        assert c.reference_machine_coordinate(view, degrees, list(coord)) == where
    with pytest.raises(Exception):
        c.reference_machine_coordinate(view, degrees, [d + 1 for d in degrees])     # outside the task space
    with pytest.raises(Exception):
        c.reference_machine_coordinate(view, degrees + [2], [0] * (len(degrees) + 1))  # rank mismatch


def _key(v):
    return (v["start"]["node_idx"], v["start"]["device_idx"], tuple((d["stride"], d["projection"]) for d in v["dimensions"]))


@pytest.mark.parametrize("degrees,nodes,gpus,expected", [
    ([3], 1, 5, [_view(0, 0, (1, INTRA)), _view(0, 1, (1, INTRA)), _view(0, 2, (1, INTRA)), _view(0, 0, (2, INTRA))]),
    ([2, 3], 3, 3, [_view(0, 0, (1, INTER), (1, INTRA)), _view(1, 0, (1, INTER), (1, INTRA)), _view(0, 0, (2, INTER), (1, INTRA)),
                    _view(0, 0, (1, INTRA), (1, INTER)), _view(0, 1, (1, INTRA), (1, INTER)), _view(0, 0, (2, INTRA), (1, INTER))]),
    ([], 2, 1, [_view(0, 0), _view(1, 0)]),
    ([2], 2, 2, [_view(0, 0, (1, INTRA)), _view(0, 0, (1, INTER)), _view(1, 0, (1, INTRA)), _view(0, 1, (1, INTER))]),
])
def test_reference_allowed_machine_views(degrees, nodes, gpus, expected):
    got = c.reference_allowed_machine_views(degrees, nodes, gpus)
    assert sorted(map(_key, got)) == sorted(map(_key, expected))


def test_reference_views_resolve_to_devices_through_absolute_strides():
    # every enumerated view, rewritten with absolute strides, resolves to distinct devices inside the machine, and task
    # by task to the device the reference's coordinate rule gives
    ms = c.MachineSpecification(2, 4)
    degrees = [2, 2]
    views = c.reference_allowed_machine_views(degrees, 2, 4)
    assert len(views) > 8
    for v in views:
        devs = c.view_devices(c.absolute_view_from_reference(v, degrees), degrees, ms)
        expect = []
        for i, j in itertools.product(range(2), range(2)):
            node, dev = c.reference_machine_coordinate(v, degrees, [i, j])
            assert 0 <= node < 2 and 0 <= dev < 4
            expect.append(node * 4 + dev)
        assert devs == expect and len(set(devs)) == 4


# ------------------------------------------------------------------ generic Metropolis search
def test_generic_mcmc_finds_the_minimum_of_a_parabola():
    # the reference's case (lib/compiler/test/src/compiler/mcmc/generic_mcmc_algorithm.cc): walk on [0, 1] with steps of
    # +-0.5, cost (x - 0.5)^2, start 0.1; a low temperature relative to the cost scale keeps what it finds
    def sampler(x, u):
        y = x + (u - 0.5)
        return y if 0.0 <= y <= 1.0 else None
    cost = lambda x: (x - 0.5) ** 2   # noqa: E731
    best, best_cost, accepted = c.run_mcmc(0.1, sampler, cost, temperature=0.01, num_iterations=400, seed=0)
    assert 0.47 < best < 0.53 and 0 <= best_cost < 0.001 and best_cost == cost(best) and 0 < accepted <= 400
    # the seed fixes the walk
    assert c.run_mcmc(0.1, sampler, cost, temperature=0.01, num_iterations=400, seed=0)[0] == best
    assert c.run_mcmc(0.1, sampler, cost, temperature=0.01, num_iterations=400, seed=1)[0] != best


def test_generic_mcmc_temperature_controls_acceptance_of_worse_states():
    sampler = lambda x, u: x + (1 if u < 0.5 else -1)   # noqa: E731
    cost = lambda x: float(abs(x))                      # noqa: E731
    cold = c.run_mcmc(0, sampler, cost, temperature=1e-6, num_iterations=300, seed=3)
    hot = c.run_mcmc(0, sampler, cost, temperature=1e6, num_iterations=300, seed=3)
    assert cold[0] == 0 and cold[2] == 0          # every proposal is worse than the start and a cold chain refuses them all
    assert hot[0] == 0 and hot[2] > 250           # a hot chain takes nearly everything and still reports the best state seen
    assert c.run_mcmc(5, lambda x, u: None, cost, 1.0, 10, 0) == (5, 5.0, 0)   # a sampler that proposes nothing


def test_mapping_search_over_the_reference_view_enumeration():
    # MachineSpecification.view_enumeration = 2: the DP chooses among every start, stride and projection that fits
    ms = c.MachineSpecification(1, 4)
    base = c.allowed_machine_views([2], 0, 4, ms)
    assert sorted(c.view_devices(v, [2], ms) for v in base) == [[0, 1], [2, 3]]
    ms.view_enumeration = 2
    every = c.allowed_machine_views([2], 0, 4, ms)
    assert sorted(c.view_devices(v, [2], ms) for v in every) == [[0, 1], [0, 2], [0, 3], [1, 2], [1, 3], [2, 3]]
    assert sorted(c.view_devices(v, [2], ms) for v in c.allowed_machine_views([2], 2, 2, ms)) == [[2, 3]]     # a resource sub-range
    two = c.MachineSpecification(2, 2)
    two.view_enumeration = 2
    devs = sorted(c.view_devices(v, [2], two) for v in c.allowed_machine_views([2], 0, 4, two))
    assert [0, 2] in devs and [1, 3] in devs and [0, 1] in devs         # across the nodes and inside one
    # on a uniform machine the richer view set finds the same optimum as the contiguous one
    g = c.build_model("mlp", {"batch_size": 16})
    plain = c.MachineSpecification(1, 4)
    pcg = S.optimize(g, world=4, algorithm="data_parallel")["pcg"]
    a = c.evaluate_pcg(pcg, plain, c.CostEstimator(plain))
    b = c.evaluate_pcg(pcg, ms, c.CostEstimator(ms))
    assert abs(a["runtime_ms"] - b["runtime_ms"]) < 1e-9 * max(1.0, a["runtime_ms"]) and b["mapped_pcg"].is_mapped()
