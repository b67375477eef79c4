"""CPU execution path (the autograd interpreter), initializers, metrics, checkpoint format, failure handling."""
import json
import os
import time

import pytest
import torch

from flexflow_train_b200 import _ffcore as core
from flexflow_train_b200.runtime.initializers import initialize
from flexflow_train_b200.runtime.torch_oracle import TorchOracle
from flexflow_train_b200.utils import checkpoint as ckpt
from flexflow_train_b200.utils import failure as F
from flexflow_train_b200.utils.metrics import PerfMetrics, StepLogger
from flexflow_train_b200.utils.profiling import ProfilingSettings, profiling_wrapper, roofline


# ---------------------------------------------------------------- oracle: one forward/backward step on CPU
def _split_test():
    return core.build_model("split_test", {"batch_size": 8})


def test_cpu_forward_backward_of_split_test_and_mlp():
    for name in ("split_test", "mlp"):
        g = core.build_model(name, {"batch_size": 8})
        orc = TorchOracle(g, seed=0)
        inp = [n for n in g.nodes() if n["type"] == "INPUT"][0]
        x = torch.randn([int(s) for s in inp["outputs"][0][1].sizes])
        pred = orc.forward({inp["name"] or f"input{inp['id']}": x})
        labels = torch.randint(0, pred.shape[-1], (pred.shape[0],))
        rows, grads = orc.loss_and_grads({inp["name"] or f"input{inp['id']}": x}, labels)
        assert rows.shape[0] == pred.shape[0] and torch.isfinite(rows).all()
        assert all(v is not None and torch.isfinite(v).all() for v in grads.values())
        assert any(float(v.abs().sum()) > 0 for v in grads.values())


def test_searched_strategy_computes_the_same_function_on_cpu():
    """A PCG found by the search evaluates to the same loss and gradients as the computation graph it came from
    (parallel operators are identities on the logical tensor)."""
    from flexflow_train_b200.compiler import strategy as S

    g = core.build_model("mlp", {"batch_size": 8})
    res = S.optimize(g, world=2, algorithm="unity", budget=8, seed=0)
    x = torch.randn(8, [int(s) for s in [n for n in g.nodes() if n["type"] == "INPUT"][0]["outputs"][0][1].sizes][1])
    labels = torch.randint(0, 10, (8,))
    a = TorchOracle(g, seed=0)
    b = TorchOracle(res["pcg"], seed=0)
    ra, ga = a.loss_and_grads({"input": x}, labels)
    rb, gb = b.loss_and_grads({"input": x}, labels)
    assert torch.allclose(ra, rb, atol=1e-5)
    for k in ga:
        assert torch.allclose(ga[k], gb[k], atol=1e-5), k


def test_transformer_oracle_gradients_match_finite_differences():
    g = core.build_model("transformer", {"num_encoder_layers": 1, "num_decoder_layers": 0, "num_features": 16, "num_heads": 2,
                                         "sequence_length": 4, "batch_size": 2, "dim_feedforward": 32, "vocab_size": 8,
                                         "dropout": 0.0})
    orc = TorchOracle(g, seed=1)
    ins = {}
    for n in g.nodes():
        if n["type"] == "INPUT":
            ins[n["name"] or f"input{n['id']}"] = torch.randn([int(s) for s in n["outputs"][0][1].sizes])
    pred = orc.forward(ins)
    labels = torch.randint(0, pred.shape[-1], (pred.reshape(-1, pred.shape[-1]).shape[0],))
    rows, grads = orc.loss_and_grads(ins, labels)
    name, p = next((k, v) for k, v in orc.params.items() if v.dim() == 2 and grads[k] is not None)
    with torch.no_grad():
        eps = 1e-3
        p[0, 0] += eps
        up = orc.loss(orc.forward(ins), labels).mean().item()
        p[0, 0] -= 2 * eps
        dn = orc.loss(orc.forward(ins), labels).mean().item()
        p[0, 0] += eps
    assert abs((up - dn) / (2 * eps) - grads[name][0, 0].item()) < 2e-3


# ---------------------------------------------------------------- initializers
@pytest.mark.parametrize("kind,value", [
    ("zero", {}), ("constant", {"value": 0.25}), ("uniform", {"seed": 3, "min_val": -1.0, "max_val": 2.0}),
    ("normal", {"seed": 3, "mean": 1.0, "stddev": 0.5}), ("truncated_normal", {"seed": 3, "mean": 0.0, "stddev": 1.0}),
    ("glorot_uniform", {"seed": 3}), ("glorot_normal", {"seed": 3}), ("kaiming_normal", {"seed": 3}),
])
def test_initializers(kind, value):
    t = initialize([64, 128], {"type": kind, "value": value}, base_seed=5, ordinal=2)
    again = initialize([64, 128], {"type": kind, "value": value}, base_seed=5, ordinal=2)
    assert torch.equal(t, again)  # deterministic
    if kind == "zero":
        assert float(t.abs().sum()) == 0
    elif kind == "constant":
        assert torch.all(t == 0.25)
    elif kind == "uniform":
        assert t.min() >= -1.0 and t.max() <= 2.0 and abs(float(t.mean()) - 0.5) < 0.1
    elif kind == "normal":
        assert abs(float(t.mean()) - 1.0) < 0.05 and abs(float(t.std()) - 0.5) < 0.05
    elif kind == "truncated_normal":
        assert t.min() >= -2.0 and t.max() <= 2.0
    elif kind == "glorot_uniform":
        a = (6.0 / (64 + 128)) ** 0.5
        assert t.abs().max() <= a + 1e-6 and float(t.std()) > 0.3 * a
    else:
        assert float(t.std()) > 0
    other = initialize([64, 128], {"type": kind, "value": value}, base_seed=5, ordinal=3)
    if kind not in ("zero", "constant"):
        assert not torch.equal(t, other)  # different weights get different streams


# ---------------------------------------------------------------- metrics
def test_perf_metrics_accuracy_and_losses():
    m = PerfMetrics()
    p = torch.tensor([[0.7, 0.2, 0.1], [0.1, 0.8, 0.1], [0.3, 0.3, 0.4], [0.6, 0.3, 0.1]])
    m.update(p, torch.tensor([0, 1, 1, 0]), ("accuracy", "sparse_categorical_crossentropy"))
    assert m.train_all == 4 and m.train_correct == 3 and m.accuracy == 0.75
    want = -(torch.log(torch.tensor([0.7, 0.8, 0.3, 0.6]))).sum().item()
    assert abs(m.sparse_cce_loss - want) < 1e-5
    m2 = PerfMetrics()
    t = torch.eye(3)[[0, 1, 1, 0]]
    m2.update(p, t, ("accuracy", "categorical_crossentropy", "mean_squared_error", "root_mean_squared_error", "mean_absolute_error"))
    assert m2.train_correct == 3 and abs(m2.cce_loss - want) < 1e-5
    d = p - t
    # the reference's formulas (lib/kernels/src/cuda/metrics_functions.cu:78-96): per-sample sums over the classes
    assert abs(m2.mse_loss - (d * d).sum(1).sum().item()) < 1e-6
    assert abs(m2.rmse_loss - (d * d).sum(1).sqrt().sum().item()) < 1e-6
    assert abs(m2.mae_loss - d.abs().sum(1).sum().item()) < 1e-6
    # sparse labels are scored against their one-hot targets
    m3 = PerfMetrics()
    m3.update(p, torch.tensor([0, 1, 1, 0]), ("mean_squared_error", "root_mean_squared_error", "mean_absolute_error"))
    assert abs(m3.mse_loss - m2.mse_loss) < 1e-6 and abs(m3.rmse_loss - m2.rmse_loss) < 1e-6 and abs(m3.mae_loss - m2.mae_loss) < 1e-6
    assert m2.summary()["samples"] == 4


def test_step_logger_writes_json_lines(tmp_path):
    fn = tmp_path / "log.jsonl"
    lg = StepLogger(str(fn))
    lg.log(1, 2.5, 100.0, lr=0.1)
    lg.log(2, 2.0, 110.0)
    recs = [json.loads(l) for l in open(fn)]
    assert [r["step"] for r in recs] == [1, 2] and recs[0]["lr"] == 0.1


def test_profiling_wrapper_on_cpu_and_roofline():
    calls = []
    ms = profiling_wrapper(lambda: calls.append(1), ProfilingSettings(warmup_iters=2, measure_iters=5), device="cpu")
    assert len(calls) == 7 and ms >= 0
    r = roofline(1.0, flops=1e12, hbm_bytes=1e9, peaks={"bf16_tflops": 1000.0, "bf16_tflops_sustained": 900.0, "hbm_gbs": 5000.0, "source": "test"})
    assert r["bound"] == "compute" and abs(r["fraction"] - 1.0) < 1e-9 and abs(r["tflops"] - 1000.0) < 1e-6


# ---------------------------------------------------------------- checkpoint format (CPU stand-in for the executable)
class _FakeExec:
    """The attributes the checkpoint module reads from an executable."""

    class _Cfg:
        class optimizer:
            kind = "adam"
        compute_dtype = "bf16"
        training = True

    def __init__(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.cfg = self._Cfg()
        self.step_count = 0
        self.nodes = {1: {"name": "w", "outputs": [(0, type("S", (), {"sizes": [4, 6]})(), None)]},
                      2: {"name": "b", "outputs": [(0, type("S", (), {"sizes": [6]})(), None)]}}
        self.param_nodes = [1, 2]
        self.param_offsets = {1: (0, 24), 2: (24, 6)}
        self.master = torch.randn(30, generator=g)
        self.shadow = self.master.to(torch.bfloat16)
        self.opt_m = torch.randn(30, generator=g)
        self.opt_v = torch.rand(30, generator=g)

    def local_weight_shape(self, nid):
        return [4, 6] if nid == 1 else [6]

    def shard_weight(self, nid, full):
        return full

    def state_dict(self):
        return {"master": self.master, "step": self.step_count, "opt_m": self.opt_m, "opt_v": self.opt_v}

    def load_state_dict(self, sd):
        self.master.copy_(sd["master"]); self.opt_m.copy_(sd["opt_m"]); self.opt_v.copy_(sd["opt_v"])
        self.shadow.copy_(self.master)
        self.step_count = int(sd["step"])


def test_checkpoint_roundtrip_latest_and_corruption(tmp_path):
    a = _FakeExec(0)
    a.step_count = 7
    p = ckpt.save(str(tmp_path), a)
    assert ckpt.latest(str(tmp_path)) == p
    b = _FakeExec(1)
    meta = ckpt.load(p, b)
    assert meta["step"] == 7 and b.step_count == 7
    assert torch.equal(a.master, b.master) and torch.equal(a.opt_v, b.opt_v)
    full = ckpt.gather_full_parameters(p)
    assert full["w"].shape == (4, 6) and torch.equal(full["b"], a.master[24:30])
    c = _FakeExec(2)
    ckpt.load_resharded(p, c)
    assert torch.equal(c.master, a.master)
    # an incomplete checkpoint (no metadata) is not picked up
    os.makedirs(tmp_path / "step00000009")
    assert ckpt.latest(str(tmp_path)) == p
    # several ranks without a barrier: refused, because the metadata could be written before the other ranks' files
    with pytest.raises(ckpt.CheckpointError):
        ckpt.save(str(tmp_path / "nobarrier"), a, world_size=2)
    # a rank file the metadata does not list (written after it) is refused on load
    import shutil
    shutil.copy(os.path.join(p, "rank0.pt"), os.path.join(p, "rank1.pt"))
    with pytest.raises(ckpt.CheckpointError, match="no recorded checksum"):
        ckpt.load(p, _FakeExec(4), rank=1)
    # a flipped byte is caught by the checksum
    F.corrupt_file(os.path.join(p, "rank0.pt"), offset=200)
    with pytest.raises(ckpt.CheckpointError):
        ckpt.load(p, _FakeExec(3))


# ---------------------------------------------------------------- failure detection (host side)
def test_heartbeat_monitor_finds_silent_rank():
    store = F.DictStore()
    mons = [F.HeartbeatMonitor(store, r, 3, timeout_s=0.2, grace_s=0.2) for r in range(3)]
    for m in mons:
        m.beat(0)
    assert mons[0].dead_ranks() == []
    mons[2].suppressed = True  # rank 2 goes silent
    time.sleep(0.3)
    mons[0].beat(1); mons[1].beat(1); mons[2].beat(1)
    assert mons[0].dead_ranks() == [2]
    with pytest.raises(F.RankFailure) as e:
        mons[1].check()
    assert e.value.ranks == [2]


def test_heartbeat_rank_that_never_joins():
    store = F.DictStore()
    m = F.HeartbeatMonitor(store, 0, 2, timeout_s=0.1, grace_s=0.15)
    m.beat()
    assert m.dead_ranks() == []  # within the grace period
    time.sleep(0.2)
    assert m.dead_ranks() == [1]


def test_recovery_restores_last_checkpoint_and_finishes(tmp_path):
    ex = _FakeExec(0)
    inj = F.FaultInjector(plan=[{"step": 3, "kind": "raise"}, {"step": 5, "kind": "raise"}])
    trace = []

    def step(i):
        inj.maybe_fail(i)
        ex.master += 1.0
        ex.step_count = i + 1
        trace.append(i)

    def save(step_no):
        ckpt.save(str(tmp_path), ex, step_no)

    def restore():
        p = ckpt.latest(str(tmp_path))
        if p is None:
            return 0
        return ckpt.load(p, ex)["step"]

    start = ex.master.clone()
    out = F.run_with_recovery(step, 8, save_fn=save, restore_fn=restore, checkpoint_every=2)
    assert out["restarts"] == 2
    assert torch.allclose(ex.master, start + 8.0)  # exactly 8 effective steps despite the replays
    assert trace[-1] == 7


def test_comm_timeout_is_recoverable_and_other_errors_are_not():
    n = {"calls": 0}

    def step(i):
        n["calls"] += 1
        if n["calls"] == 2:
            raise F.CommTimeoutError("peer flag wait ran out")
        if n["calls"] == 5:
            raise ValueError("bug")

    with pytest.raises(ValueError):
        F.run_with_recovery(step, 10, save_fn=lambda s: None, restore_fn=lambda: 0)
    assert n["calls"] == 5
