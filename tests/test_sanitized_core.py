"""The C++ compiler core under UBSan: a copy built with -fsanitize=undefined -fno-sanitize-recover (any undefined
behaviour -- signed overflow, bad shifts, misaligned or null accesses, out-of-range enum loads -- aborts the process)
drives model building, shape inference, serialisation, graph algorithms, substitutions, both searches and the
lowering passes in a child process.  The reference builds all of its host code this way
(cmake/flexflow-utils.cmake:36-58)."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

DRIVER = textwrap.dedent('''
    import importlib.util, json, sys
    path = sys.argv[1]
    spec = importlib.util.spec_from_file_location("flexflow_train_b200._ffcore", path)
    core = importlib.util.module_from_spec(spec)
    sys.modules["flexflow_train_b200._ffcore"] = core   # the package and its modules pick this copy up
    spec.loader.exec_module(core)
    from flexflow_train_b200.compiler import strategy as S
    from flexflow_train_b200.runtime import lowering as L
    assert S.core is core

    small = {"transformer": {"num_features": 32, "sequence_length": 8, "batch_size": 4, "dim_feedforward": 64, "num_heads": 2,
                             "num_encoder_layers": 1, "num_decoder_layers": 1, "vocab_size": 32},
             "transformer_lm": {"num_features": 32, "sequence_length": 8, "batch_size": 4, "dim_feedforward": 64, "num_heads": 2,
                                "num_decoder_layers": 1, "vocab_size": 32},
             "bert": {"hidden_size": 32, "num_encoder_layers": 1, "num_heads": 2, "dim_feedforward": 64, "sequence_length": 8,
                      "batch_size": 4, "vocab_size": 64}}
    done = []
    for name in core.model_names():
        cg = core.build_model(name, small.get(name, {}))
        text = cg.to_v1_string()
        assert core.Graph.from_v1(text).signature() == cg.signature()
        cg.as_dot(); cg.topological_order()
        pcg = core.pcg_from_computation_graph(cg)
        core.get_graph_sp_decomposition(pcg)
        done.append(name)
    ms = core.MachineSpecification(1, 4)
    rules = core.get_substitution_set(ms)
    assert all(r.is_valid() for r in rules)
    for name in ("transformer_lm", "mlp", "dlrm", "split_test"):
        cg = core.build_model(name, small.get(name, {}))
        for algo, kw in (("unity", {"budget": 6}), ("mcmc", {"mcmc_iterations": 20}), ("data_parallel", {})):
            r = S.optimize(cg, world=4, algorithm=algo, **kw)
            assert r["runtime_ms"] > 0
            core.Graph.from_v1(r["mapped_pcg"].to_v1_string(parallel=True))
        low = L.lower(S.optimize(cg, world=2, algorithm="data_parallel")["mapped_pcg"], optimizer={"kind": "adam"})
        assert len(low) > 0
    U = core.utils
    assert U.positive_mul(6, 7) == 42 and U.orthotope_flatten([2, 3, 4], [1, 2, 3]) == 23
    try:
        U.positive_mul(2 ** 62, 4)
        raise SystemExit("overflow not reported")
    except OverflowError:
        pass
    assert U.lift_coord([2, 3, 4], [[0, 1], [2]], U.project_coord([2, 3, 4], [[0, 1], [2]], [1, 2, 3])) == [1, 2, 3]
    assert len(U.union_find_groups([(1, 2), (3, 4), (2, 3)])) == 1 and U.dedup_queue_order([2, 2, 1])[1] == [2, 1]
    print(json.dumps({"models": done, "rules": len(rules)}))
''')


def test_core_runs_clean_under_ubsan(tmp_path):
    sys.path.insert(0, ROOT)
    try:
        import build
    finally:
        sys.path.pop(0)
    try:
        so = build.build_core(sanitize=True)
    except Exception as e:  # no compiler or no libubsan on this machine
        pytest.skip(f"sanitized build not possible here: {e}")
    script = tmp_path / "drive.py"
    script.write_text(DRIVER)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""),
               UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1")
    r = subprocess.run([sys.executable, str(script), so], capture_output=True, text=True, env=env, timeout=900)
    assert "runtime error" not in r.stderr, r.stderr[-3000:]
    assert r.returncode == 0, (r.stdout[-1000:], r.stderr[-3000:])
    assert '"rules"' in r.stdout
