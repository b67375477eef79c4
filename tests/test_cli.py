"""Command-line tools: export-model-arch, protobuf-to-json, substitution-to-dot, sp-ization-benchmarking."""
import io
import json
from contextlib import redirect_stdout

import pytest

from flexflow_train_b200 import _ffcore as core
from flexflow_train_b200.bin import export_model_arch, protobuf_to_json, sp_ization_benchmarking, substitution_to_dot


def _run(mod, argv):
    buf = io.StringIO()
    with redirect_stdout(buf):
        assert mod.main(argv) == 0
    return buf.getvalue()


def test_export_model_arch_json_sp_and_dot():
    out = json.loads(_run(export_model_arch, ["--sp-decomposition", "split_test"]))
    assert set(out) == {"computation_graph", "sp_decomposition"}
    g = core.Graph.from_v1(json.dumps(out["computation_graph"]))
    assert len(g.nodes()) == len(core.build_model("split_test", {}).nodes())
    leaves = core.sp_nodes(core.sp_from_json(out["sp_decomposition"]))
    assert sorted(leaves) == sorted(n["id"] for n in g.nodes())
    assert _run(export_model_arch, ["--dot", "mlp"]).lstrip().startswith("digraph")
    pre = _run(export_model_arch, ["--preprocessed-dot", "mlp"])
    assert "WEIGHT" not in pre and "LINEAR" in pre
    small = json.loads(_run(export_model_arch, ["--config", '{"batch_size": 2}', "mlp"]))
    assert small["computation_graph"]


RULES = {"_t": "RuleCollection", "rule": [{
    "_t": "Rule", "name": "taso_rule_0",
    "srcOp": [{"_t": "Operator", "type": "OP_LINEAR", "input": [{"_t": "Tensor", "opId": -1, "tsId": 0}, {"_t": "Tensor", "opId": -2, "tsId": 0}],
               "para": [{"_t": "Parameter", "key": "PM_ACTI", "value": 0}]},
              {"_t": "Operator", "type": "OP_RELU", "input": [{"_t": "Tensor", "opId": 0, "tsId": 0}], "para": []}],
    "dstOp": [{"_t": "Operator", "type": "OP_LINEAR", "input": [{"_t": "Tensor", "opId": -1, "tsId": 0}, {"_t": "Tensor", "opId": -2, "tsId": 0}],
               "para": [{"_t": "Parameter", "key": "PM_ACTI", "value": 2}]}],
    "mappedOutput": [{"_t": "MapOutput", "srcOpId": 1, "dstOpId": 0, "srcTsId": 0, "dstTsId": 0}]}]}


def test_protobuf_to_json_roundtrip_and_negative_ids(tmp_path):
    pb = tmp_path / "rules.pb"
    pb.write_bytes(protobuf_to_json.encode_rule_collection(RULES))
    out = tmp_path / "rules.json"
    assert protobuf_to_json.main([str(pb), str(out)]) == 0
    got = json.loads(out.read_text())
    assert got == RULES  # negative opIds (external inputs) survive the 64-bit varint encoding
    sym = protobuf_to_json.decode_rule_collection(pb.read_bytes(), symbolic_values=True)
    assert sym["rule"][0]["dstOp"][0]["para"][0]["value"] == "AC_MODE_RELU"
    with pytest.raises(protobuf_to_json.WireError):
        protobuf_to_json.decode_rule_collection(pb.read_bytes()[:-3])
    # the converted file feeds the legacy rule loader
    stats = core.load_legacy_rules(json.dumps(got))
    assert stats is not None


def test_substitution_to_dot(tmp_path):
    f = tmp_path / "rules.json"
    f.write_text(json.dumps(RULES))
    dot = _run(substitution_to_dot, [str(f), "taso_rule_0"])
    assert dot.startswith("digraph") and "OP_RELU" in dot and "OP_LINEAR" in dot
    assert "pattern" in _run(substitution_to_dot, ["--builtin", "partition_linear"])
    with pytest.raises(SystemExit):
        substitution_to_dot.main([str(f), "taso_rule_7"])


def test_sp_ization_benchmarking_tables_and_invariants():
    text = _run(sp_ization_benchmarking, ["--graphs", "sample_dag,rhombus", "--repeat", "2"])
    assert "Technique | Work-Increase | Critical-Path-Increase" in text and "NO" not in text
    res = json.loads(_run(sp_ization_benchmarking, ["--graphs", "random,nasnet_cell,parallel_chains", "--repeat", "3", "--json"]))
    for title, techniques in res.items():
        for t, r in techniques.items():
            assert r["dependencies_preserved"], (title, t)
            assert r["relative_work_increase"] >= 1 - 1e-9 and r["relative_critical_path_increase"] >= 1 - 1e-9
        # synchronising techniques never duplicate work; duplicating ones never lengthen the critical path
        assert abs(techniques["stratum_sync"]["relative_work_increase"] - 1) < 1e-9
        assert abs(techniques["work_duplicating"]["relative_critical_path_increase"] - 1) < 1e-9
    # an SP graph needs no change at all (the non-coalescing duplicator still copies shared ancestors)
    sp = json.loads(_run(sp_ization_benchmarking, ["--graphs", "rhombus", "--repeat", "1", "--json"]))
    assert all(abs(r["relative_work_increase"] - 1) < 1e-9 and abs(r["relative_critical_path_increase"] - 1) < 1e-9
               for t, r in sp["rhombus, Constant(1)"].items() if t != "work_duplicating")


def test_run_model_parses_reference_flags():
    from flexflow_train_b200.bin import run_model

    with pytest.raises(SystemExit):  # --help exits after printing usage that lists the legacy flags
        buf = io.StringIO()
        with redirect_stdout(buf):
            run_model.main(["--help"])
    assert True


def test_run_model_trains_a_graph_file_on_the_host(tmp_path, capsys):
    """run-model <graph.json>: the reference's usage (a serialized graph, 5 iterations of SGD with momentum 0.9), here
    on the host executor so that it runs without a GPU."""
    from flexflow_train_b200 import _ffcore as core
    from flexflow_train_b200.bin import run_model

    path = tmp_path / "mlp.json"
    path.write_text(core.build_model("mlp", {"batch_size": 16}).to_v1_string())
    assert run_model.main([str(path), "--device", "cpu", "-p", "1"]) == 0
    out = capsys.readouterr().out
    losses = [float(l.rsplit("loss", 1)[1]) for l in out.splitlines() if "loss" in l and l.startswith("epoch 0 iter")]
    assert len(losses) == 5 and losses[-1] < losses[0], out
    assert "5 iterations" in out


def test_run_model_checkpoints_and_resumes_on_the_host(tmp_path, capsys):
    from flexflow_train_b200.bin import run_model
    from flexflow_train_b200.utils import checkpoint as ckpt

    cfg = '{"num_features": 32, "sequence_length": 16, "batch_size": 4, "dim_feedforward": 64, "num_heads": 2, ' \
          '"num_encoder_layers": 1, "num_decoder_layers": 1, "vocab_size": 32}'
    base = ["--model", "transformer", "--model-config", cfg, "-p", "1", "--checkpoint-dir", str(tmp_path), "--device", "cpu"]
    assert run_model.main(base + ["--iterations", "4", "--checkpoint-every", "2"]) == 0
    first = capsys.readouterr().out
    assert ckpt.latest(str(tmp_path)).endswith("step00000004")
    assert run_model.main(base + ["--iterations", "2", "--resume"]) == 0
    second = capsys.readouterr().out
    assert "resumed from" in second and "at step 4" in second
    last_before = float([l for l in first.splitlines() if "iter 3" in l][0].rsplit("loss", 1)[1])
    first_after = float([l for l in second.splitlines() if "iter 0" in l][0].rsplit("loss", 1)[1])
    assert first_after < last_before    # training went on from the restored weights, not from a fresh initialisation


def test_run_model_ignores_runtime_resource_flags_and_their_values(tmp_path, capsys):
    """`-ll:gpu 1 -ll:fsize 14000` (the reference's resource flags) must not leak their values into the positional
    graph-file argument, in either position relative to the other flags."""
    from flexflow_train_b200.bin import run_model

    assert run_model.split_runtime_flags(["-ll:gpu", "1", "--model", "mlp", "-lg:prof=2", "-ll:fsize", "14000", "-b", "8"]) == (
        ["--model", "mlp", "-b", "8"], ["-ll:gpu", "1", "-lg:prof=2", "-ll:fsize", "14000"])
    cfg = '{"batch_size": 8}'
    args = ["--model", "mlp", "--model-config", cfg, "--iterations", "3", "-p", "1", "--device", "cpu", "-ll:gpu", "1", "-ll:fsize", "14000"]
    assert run_model.main(args) == 0
    assert run_model.main(["-ll:gpu", "1"] + args[:-4]) == 0
    out = capsys.readouterr()
    assert out.out.count("iter 2: loss") == 2 and "were ignored" in out.err
    with pytest.raises(SystemExit):  # an unknown flag is still an error
        run_model.main(args + ["--no-such-flag"])


def test_search_model_emits_strategy_estimate_and_cpu_step(tmp_path, capsys):
    """CPU-only compile + Unity search from the unparallelised graph on a small Transformer for 4 simulated GPUs: writes the
    strategy, prints the estimated step time and trains one step on the host."""
    import json

    from flexflow_train_b200 import _ffcore as core
    from flexflow_train_b200.bin import search_model

    cfg = '{"num_encoder_layers": 1, "num_decoder_layers": 1, "num_features": 256, "sequence_length": 128, "batch_size": 64, ' \
          '"dim_feedforward": 1024, "vocab_size": 64}'
    out = tmp_path / "strategy.json"
    args = ["--model", "transformer", "--model-config", cfg, "--heads", "4", "--gpus", "4", "--budget", "3", "--time-limit", "60",
            "--seed", "0", "--out", str(out), "--cpu-step"]
    assert search_model.main(args) == 0
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    c = rec["search"]["candidates"]
    # the search started at the serial graph and found a plan at least as good as the hand-built data-parallel template
    assert rec["search"]["search_start"] == "serial" and rec["search"]["unity"]["evaluated"] > 10
    assert rec["estimated_step_ms"] <= min(c.values()) * 1.0001 and rec["search"]["unity"]["runtime_ms"] <= c["dp4"] * 1.0001
    assert rec["estimated_step_ms"] < c["single_device"]
    g = core.Graph.from_v1(out.read_text())
    assert g.is_mapped() and any(core.is_parallel_op(n["type"]) for n in g.nodes())
    assert rec["cpu_step"]["loss_after_one_update"] < rec["cpu_step"]["loss"]
    # the same seed gives the same answer
    assert search_model.main(args[:-1]) == 0
    again = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert again["estimated_step_ms"] == rec["estimated_step_ms"]


def test_bench_contract_pieces_that_need_no_gpu():
    """`bench.py --impl reference` prints the one-line unavailable record and exits 0; the clock sampler degrades to a
    record with no samples when neither NVML nor nvidia-smi can be read."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and "unavailable" in rec and len(rec["unavailable"]) > 20
    sys.path.insert(0, root)
    try:
        import bench
    finally:
        sys.path.pop(0)
    assert set(bench.MODEL_CONFIGS) == set(bench.TRAINING) == set(bench.L2_NOTE)
    s = bench.ClockSampler(0)
    s.start()
    out = s.stop()
    assert "sm_mhz" in out and "reasons" in out


def test_config_fields_flags_and_docs_come_from_one_table():
    """FFConfig, the tools' flags and the field documentation are generated from config_schema.FIELDS."""
    import argparse
    import dataclasses

    from flexflow_train_b200 import api, config_schema as cs
    assert api.FFConfig is cs.FFConfig
    names = [f.name for f in dataclasses.fields(cs.FFConfig)]
    assert names == [f.name for f in cs.FIELDS] and len(set(names)) == len(names)
    cfg = cs.FFConfig()
    for f in cs.FIELDS:
        assert getattr(cfg, f.name) == f.default
    p = argparse.ArgumentParser()
    cs.add_cli_arguments(p)
    flags = {a.dest for a in p._actions}
    assert {f.name for f in cs.FIELDS if f.flag} <= flags
    ns = p.parse_args(["--search-budget", "7", "--no-cuda-graph", "--export-strategy", "s.json", "-e", "3", "--measure-costs"])
    c = cs.config_from_args(ns, seed=5)
    assert (c.search_budget, c.use_cuda_graph, c.export_strategy_file, c.epochs, c.measure_costs, c.seed) == (7, False, "s.json", 3, True, 5)
    # the reference's opt-in switches: off on the command line unless given, on for library users
    assert c.enable_parameter_parallel is False and cs.FFConfig().enable_parameter_parallel is True
    table = cs.describe()
    assert all(f"`{f.name}`" in table for f in cs.FIELDS)
    with __import__("pytest").raises(SystemExit):
        p.parse_args(["--compute-dtype", "fp8"])


def test_documentation_pages_are_current():
    # the configuration page is generated from the schema; the index lists every page; tools named in the docs exist
    import importlib
    import os
    import re
    from flexflow_train_b200 import config_schema
    docs = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "docs")
    assert config_schema.describe() in open(os.path.join(docs, "configuration.md")).read()
    index = open(os.path.join(docs, "index.md")).read()
    pages = sorted(f for f in os.listdir(docs) if f.endswith(".md") and f != "index.md")
    assert pages and all(f"({p})" in index for p in pages)
    text = "\n".join(open(os.path.join(docs, p)).read() for p in pages)
    for mod in set(re.findall(r"python -m (flexflow_train_b200\.[a-z_.]+)", text)):
        if not mod.endswith("<tool>"):
            assert importlib.util.find_spec(mod.rstrip(".")) is not None, mod
    for path in set(re.findall(r"`((?:csrc|runtime|frontend|parallel|utils|ops|compiler|bin)/[A-Za-z0-9_/.]+\.(?:py|cc|cu|cuh|h))`", text)):
        assert os.path.exists(os.path.join(os.path.dirname(docs), "flexflow_train_b200", path)), path


def test_flexflow_python_launcher(tmp_path, capsys):
    from flexflow_train_b200.bin import flexflow_python as fp
    script = tmp_path / "train.py"
    script.write_text("import sys, json\nprint(json.dumps(sys.argv[1:]))\n")
    # one rank: the script runs in this process and sees only its own arguments
    assert fp.main([str(script), "-ll:gpu", "1", "-ll:fsize", "14000", "-ll:zsize=2048", "-b", "64", "--epochs", "2"]) == 0
    out = capsys.readouterr()
    assert json.loads(out.out.strip().splitlines()[-1]) == ["-b", "64", "--epochs", "2"]
    assert "-ll:fsize 14000" in out.err and "-ll:zsize=2048" in out.err and "-ll:gpu" not in out.err
    # several ranks: a torch.distributed.run command with one process per GPU and a loopback rendezvous
    ranks, opts, s, args, dropped = fp.plan([str(script), "-ll:gpu", "4", "--nodes", "2", "--node-rank", "1", "--master-addr", "10.0.0.1", "-b", "8"])
    assert (ranks, s, args, dropped) == (4, str(script), ["-b", "8"], [])
    cmd = fp.command(ranks, opts, s, args)
    assert cmd[1:4] == ["-m", "torch.distributed.run", "--nnodes"] and cmd[cmd.index("--nproc-per-node") + 1] == "4"
    assert cmd[cmd.index("--node-rank") + 1] == "1" and cmd[cmd.index("--master-addr") + 1] == "10.0.0.1" and cmd[-3:] == [str(script), "-b", "8"]
    assert fp.plan([str(script), "-ll:gpu=2"])[0] == 2
    with pytest.raises(SystemExit):
        fp.main([str(tmp_path / "missing.py"), "-ll:gpu", "1"])
    with pytest.raises(SystemExit):
        fp.plan([str(script), "-ll:gpu", "0"])
