"""The GPU executor against the PyTorch oracle: same graph, same weights, same batch."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from flexflow_train_b200 import _ffcore as core  # noqa: E402
from flexflow_train_b200.runtime.executor import ExecConfig, Executable, OptimizerConfig  # noqa: E402
from flexflow_train_b200.runtime.torch_oracle import TorchOracle  # noqa: E402

SMALL_LM = {"num_features": 128, "sequence_length": 64, "batch_size": 4, "dim_feedforward": 256, "num_heads": 2,
            "num_decoder_layers": 2, "dropout": 0.0, "vocab_size": 256}


def rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).norm() / (b.float().cpu().norm() + 1e-12)).item()


@pytest.mark.parametrize("dtype,tol", [("fp32", 2e-2), ("bf16", 6e-2)])
def test_transformer_lm_matches_oracle(dtype, tol):
    g = core.build_model("transformer_lm", SMALL_LM)
    ex = Executable(g, ExecConfig(compute_dtype=dtype, seed=3))
    oracle = TorchOracle(g, seed=3)
    for (n1, p1), (n2, p2) in zip(ex.named_parameters(), oracle.params.items()):
        assert n1 == n2 and rel(p1, p2) < 1e-6
    torch.manual_seed(0)
    ids = torch.randint(0, 256, (4, 64, 1), dtype=torch.int32)
    labels = torch.randint(0, 256, (4, 64), dtype=torch.int32)
    ex.set_inputs({"input_ids": ids.cuda()}, labels.cuda())
    ex.forward()
    ex.compute_loss()
    ex.backward()
    rows_ref, grads_ref = oracle.loss_and_grads({"input_ids": ids}, labels)
    assert rel(ex.loss_rows, rows_ref) < tol
    worst = 0.0
    for name, g_ in ex.named_gradients():
        r = rel(g_, grads_ref[name])
        worst = max(worst, r)
        assert r < 5 * tol, (name, r)
    assert worst > 0


def test_mlp_loss_decreases():
    # mirrors the reference's end-to-end check (lib/local-execution/test/src/local-execution/computation_graph_instance.cc)
    g = core.build_model("mlp", {"batch_size": 64, "input_dim": 64, "hidden": [128, 128], "num_classes": 10})
    ex = Executable(g, ExecConfig(compute_dtype="bf16", optimizer=OptimizerConfig(kind="sgd", lr=0.05, momentum=0.9)))
    torch.manual_seed(1)
    x = torch.randn(64, 64, device="cuda")
    y = torch.randint(0, 10, (64,), device="cuda", dtype=torch.int32)
    losses = []
    for _ in range(20):
        ex.train_step({"input": x}, y)
        losses.append(ex.mean_loss())
    assert losses[-1] < 0.8 * losses[0] and losses[-1] < losses[len(losses) // 2], losses


def test_profile_step_leaves_weights_and_optimizer_state_alone():
    g = core.build_model("transformer_lm", SMALL_LM)
    ex = Executable(g, ExecConfig(compute_dtype="bf16", seed=5, use_cuda_graph=False, optimizer=OptimizerConfig(kind="adam", lr=1e-3)))
    ids = torch.randint(0, 256, (4, 64, 1), dtype=torch.int32, device="cuda")
    labels = torch.randint(0, 256, (4, 64), dtype=torch.int32, device="cuda")
    ex.train_step({"input_ids": ids}, labels)
    before = (ex.master.clone(), ex.opt_m.clone(), ex.opt_v.clone(), ex.step_count)
    prof = ex.profile_step()
    assert prof["total_ms"] > 0 and ("LINEAR", "fwd") in prof["by_type"] and ("update", "update") not in prof["by_type"]
    assert torch.equal(before[0], ex.master) and torch.equal(before[1], ex.opt_m) and torch.equal(before[2], ex.opt_v)
    assert ex.step_count == before[3]
    prof = ex.profile_step(update=True)
    assert ("update", "update") in prof["by_type"] and ex.step_count == before[3] + 1 and not torch.equal(before[0], ex.master)


def test_adam_cuda_graph_matches_eager():
    cfg = dict(SMALL_LM, dropout=0.1)
    ids = torch.randint(0, 256, (4, 64, 1), dtype=torch.int32, device="cuda")
    labels = torch.randint(0, 256, (4, 64), dtype=torch.int32, device="cuda")
    out = []
    for use_graph in (False, True):
        g = core.build_model("transformer_lm", cfg)
        ex = Executable(g, ExecConfig(compute_dtype="bf16", seed=5, use_cuda_graph=use_graph,
                                      optimizer=OptimizerConfig(kind="adam", lr=1e-3)))
        ls = []
        for _ in range(4):
            ex.train_step({"input_ids": ids}, labels)
            ls.append(ex.mean_loss())
        out.append(ls)
    assert out[0][-1] < out[0][0]
    for a, b in zip(*out):
        assert abs(a - b) < 2e-2 * abs(a), out


def _shape_ops_graph():
    b = core.GraphBuilder()
    x = b.create_input([8, 16], name="input")
    idx = b.create_input([8, 5], dtype="INT32", name="index")
    h = b.dense(x, 16, activation="TANH", name="fc0")
    p0, p1 = b.split(h, [10, 6], 1, name="split")
    a = b.reverse(p0, 1, name="rev")
    t = b.transpose(p1, [1, 0], name="tr")
    t = b.unary("SCALAR_MULTIPLY", t, 2.0, name="scale")
    t = b.transpose(t, [1, 0], name="tr_back")
    c = b.concat([a, t], 1, name="cat")
    r = b.reduce("REDUCE_MEAN", c, [1], True, name="rowmean")
    rb = b.broadcast(r, [8, 16], name="bcast")
    c = b.binary("EW_SUB", c, rb, name="center")
    top = b.top_k(c, 4, name="topk")[0]
    gat = b.gather(c, idx, 1, name="gather")
    f = b.concat([c, top, gat], 1, name="features")
    y = b.dense(f, 8, name="fc1")
    b.softmax(y, name="out_prob")
    return b.graph


def test_tensor_shape_operators_match_oracle():
    g = _shape_ops_graph()
    ex = Executable(g, ExecConfig(compute_dtype="fp32", seed=2))
    oracle = TorchOracle(g, seed=2)
    torch.manual_seed(0)
    x = torch.randn(8, 16)
    idx = torch.randint(0, 16, (8, 5), dtype=torch.int32)
    labels = torch.randint(0, 8, (8,), dtype=torch.int32)
    ex.set_inputs({"input": x.cuda(), "index": idx.cuda()}, labels.cuda())
    ex.forward()
    ex.compute_loss()
    ex.backward()
    rows_ref, grads_ref = oracle.loss_and_grads({"input": x, "index": idx}, labels)
    assert rel(ex.loss_rows, rows_ref) < 2e-2
    for name, g_ in ex.named_gradients():
        assert rel(g_, grads_ref[name]) < 5e-2, (name, rel(g_, grads_ref[name]))


def _reduce_broadcast_pool_graph():
    """max / min / prod reductions, mul / div with a row vector repeated over the batch, pooling with a fused ReLU."""
    b = core.GraphBuilder()
    x = b.create_input([8, 16], name="input")
    h = b.dense(x, 16, activation="TANH", name="fc0")
    cmax = b.reduce("REDUCE_MAX", h, [0], False, name="colmax")            # [16]
    cmin = b.unary("EXP", b.reduce("REDUCE_MIN", h, [0], False, name="colmin"), name="exp_colmin")
    m = b.binary("EW_MUL", h, cmax, name="scale_by_max")
    d = b.binary("EW_DIV", m, cmin, name="div_by_min")
    shifted = b.unary("SCALAR_ADD", h, 1.5, name="shift")
    p0, _ = b.split(shifted, [3, 13], 1, name="first3")
    pr = b.reduce("REDUCE_PROD", p0, [1], True, name="rowprod")               # [8, 1]
    img = b.reshape(d, [8, 1, 4, 4], name="as_image")
    pooled = b.pool2d(img, 2, 2, 2, 2, 0, 0, "MAX", "RELU", name="pool_relu")
    f = b.concat([d, pr, b.flat(pooled, 1, -1, name="flat")], 1, name="features")
    y = b.dense(f, 8, name="fc1")
    b.softmax(y, name="out_prob")
    return b.graph


def test_reductions_broadcast_products_and_activated_pooling_match_oracle():
    g = _reduce_broadcast_pool_graph()
    ex = Executable(g, ExecConfig(compute_dtype="fp32", seed=3))
    oracle = TorchOracle(g, seed=3)
    torch.manual_seed(1)
    x = torch.randn(8, 16)
    labels = torch.randint(0, 8, (8,), dtype=torch.int32)
    ex.set_inputs({"input": x.cuda()}, labels.cuda())
    ex.forward()
    ex.compute_loss()
    ex.backward()
    rows_ref, grads_ref = oracle.loss_and_grads({"input": x}, labels)
    assert rel(ex.loss_rows, rows_ref) < 2e-2
    for name, g_ in ex.named_gradients():
        assert rel(g_, grads_ref[name]) < 5e-2, (name, rel(g_, grads_ref[name]))


def test_dropout_fused_into_the_linear_epilogue_trains_like_the_separate_kernel():
    """Same salts and step seeds give the same masks, so the two executors follow the same trajectory."""
    cfg = dict(SMALL_LM, dropout=0.2)
    ids = torch.randint(0, 256, (4, 64, 1), dtype=torch.int32, device="cuda")
    labels = torch.randint(0, 256, (4, 64), dtype=torch.int32, device="cuda")
    out = []
    for fuse in (False, True):
        g = core.build_model("transformer_lm", cfg)
        ex = Executable(g, ExecConfig(compute_dtype="bf16", seed=5, fuse_dropout=fuse, optimizer=OptimizerConfig(kind="adam", lr=1e-3)))
        fused = sum(1 for op in ex.ops.values() if getattr(op, "fused_into", None) is not None)
        assert (fused > 0) == fuse
        ls = []
        for _ in range(4):
            ex.train_step({"input_ids": ids}, labels)
            ls.append(ex.mean_loss())
        out.append(ls)
    for a, b in zip(*out):
        assert abs(a - b) < 2e-2 * abs(a), out


def test_run_model_cli_trains_checkpoints_and_resumes(tmp_path, capsys):
    """The run-model tool end to end on one GPU: train, write checkpoints, resume from the newest one."""
    from flexflow_train_b200.bin import run_model
    from flexflow_train_b200.utils import checkpoint as ckpt

    cfg = '{"num_features": 64, "sequence_length": 32, "batch_size": 4, "dim_feedforward": 128, "num_heads": 2, ' \
          '"num_encoder_layers": 1, "num_decoder_layers": 1, "vocab_size": 64}'
    args = ["--model", "transformer", "--model-config", cfg, "--iterations", "4", "-p", "2", "--checkpoint-dir", str(tmp_path),
            "--checkpoint-every", "2", "--no-cuda-graph", "-ll:gpu", "1", "-ll:fsize", "14000"]
    assert run_model.main(args) == 0
    first = capsys.readouterr().out
    assert "iter 0: loss" in first and "samples/s" in first
    last = ckpt.latest(str(tmp_path))
    assert last is not None and last.endswith("step00000004")
    assert run_model.main(args + ["--resume"]) == 0
    second = capsys.readouterr().out
    assert "resumed from" in second and "at step 4" in second
    assert ckpt.latest(str(tmp_path)).endswith("step00000008")


def test_checkpoint_roundtrip_restores_training_state_on_gpu(tmp_path):
    from flexflow_train_b200.utils import checkpoint as ckpt

    ids = torch.randint(0, 256, (4, 64, 1), dtype=torch.int32, device="cuda")
    labels = torch.randint(0, 256, (4, 64), dtype=torch.int32, device="cuda")

    def make():
        return Executable(core.build_model("transformer_lm", SMALL_LM),
                          ExecConfig(compute_dtype="bf16", seed=9, optimizer=OptimizerConfig(kind="adam", lr=1e-3)))
    a = make()
    for _ in range(3):
        a.train_step({"input_ids": ids}, labels)
    path = ckpt.save(str(tmp_path), a)
    a.train_step({"input_ids": ids}, labels)
    want = a.mean_loss()
    b = make()
    meta = ckpt.load(path, b)
    assert meta["step"] == 3 and b.step_count == 3
    b.train_step({"input_ids": ids}, labels)
    assert abs(b.mean_loss() - want) < 1e-3 * abs(want)


@pytest.mark.parametrize("block_bytes", [0, 16384, 8192])
def test_blocked_attention_core_matches_oracle(block_bytes):
    """The L2-blocked attention core (blocks of batch elements, or of head groups of one batch element, with the
    probabilities recomputed in backward) computes the same loss and gradients as the whole-batch core."""
    g = core.build_model("transformer_lm", SMALL_LM)
    ex = Executable(g, ExecConfig(compute_dtype="bf16", seed=3, attention_block_bytes=block_bytes, fused_attention=False))
    att = [op for op in ex.ops.values() if op.type == "MULTIHEAD_ATTENTION"][0]
    assert (att.cb > 0) == (block_bytes > 0)
    if block_bytes == 8192:
        assert att.hb == 1 and att.cb == 1
    oracle = TorchOracle(g, seed=3)
    torch.manual_seed(0)
    ids = torch.randint(0, 256, (4, 64, 1), dtype=torch.int32)
    labels = torch.randint(0, 256, (4, 64), dtype=torch.int32)
    ex.set_inputs({"input_ids": ids.cuda()}, labels.cuda())
    ex.forward()
    ex.compute_loss()
    ex.backward()
    rows_ref, grads_ref = oracle.loss_and_grads({"input_ids": ids}, labels)
    assert rel(ex.loss_rows, rows_ref) < 6e-2
    for name, g_ in ex.named_gradients():
        assert rel(g_, grads_ref[name]) < 0.3, (name, rel(g_, grads_ref[name]))


def test_blocked_attention_with_dropout_is_consistent_between_forward_and_backward():
    """With dropout the blocked core regenerates each block's mask in backward; training must still converge and
    the CUDA-graph replay must follow the eager trajectory."""
    cfg = dict(SMALL_LM, dropout=0.1)
    ids = torch.randint(0, 256, (4, 64, 1), dtype=torch.int32, device="cuda")
    labels = torch.randint(0, 256, (4, 64), dtype=torch.int32, device="cuda")
    out = []
    for use_graph in (False, True):
        g = core.build_model("transformer_lm", cfg)
        ex = Executable(g, ExecConfig(compute_dtype="bf16", seed=5, use_cuda_graph=use_graph, attention_block_bytes=16384, fused_attention=False,
                                      optimizer=OptimizerConfig(kind="adam", lr=1e-3)))
        ls = []
        for _ in range(6):
            ex.train_step({"input_ids": ids}, labels)
            ls.append(ex.mean_loss())
        out.append(ls)
    assert out[0][-1] < out[0][0]
    for a, b in zip(*out):
        assert abs(a - b) < 2e-2 * abs(a), out


def test_dropout_backward_folded_into_linear_backward_gives_the_same_gradients():
    """Masks are a function of (salt, step seed, index), so an executor that folds the dropout's backward into the
    preceding Linear's bias/activation kernel and one that runs it as a separate kernel see identical masks."""
    cfg = dict(SMALL_LM, dropout=0.3)
    ids = torch.randint(0, 256, (4, 64, 1), dtype=torch.int32, device="cuda")
    labels = torch.randint(0, 256, (4, 64), dtype=torch.int32, device="cuda")
    grads = []
    for fold in (False, True):
        g = core.build_model("transformer_lm", cfg)
        ex = Executable(g, ExecConfig(compute_dtype="bf16", seed=5, fold_dropout_backward=fold))
        folded = sum(1 for op in ex.ops.values() if getattr(op, "bwd_folded", None) is not None)
        assert (folded > 0) == fold
        ex.set_inputs({"input_ids": ids}, labels)
        ex._pre_step()
        ex.forward()
        ex.compute_loss()
        ex.backward()
        grads.append({k: v.float().clone() for k, v in ex.named_gradients()})
    for k in grads[0]:
        assert rel(grads[1][k], grads[0][k]) < 2e-2, (k, rel(grads[1][k], grads[0][k]))


def test_sparse_embedding_update_matches_the_dense_update():
    """Plain SGD on an embedding table: rows updated from the output gradient inside the Embedding's backward give the
    same training as the dense table gradient + dense update, and the table then lives outside the parameter arenas."""
    from flexflow_train_b200 import _ffcore as core
    from flexflow_train_b200.runtime.executor import ExecConfig, Executable, OptimizerConfig

    cfg = {"batch_size": 64, "embedding_dim": 16, "embedding_bag_size": 1, "embedding_size": [500, 300],
           "dense_arch_layer_sizes": [13, 32, 16], "over_arch_layer_sizes": [48, 32, 1], "arch_interaction_op": "DOT",
           "final_activation": "SIGMOID", "embedding_data_type": "FLOAT"}
    cg = core.build_model("dlrm", cfg)
    opt = OptimizerConfig(kind="sgd", lr=0.05, momentum=0.0)
    mk = lambda sparse: Executable(cg, ExecConfig(compute_dtype="bf16", seed=2, optimizer=opt, loss="mean_squared_error_avg_reduce",
                                                  sparse_embedding_update=sparse))
    dense, sparse = mk(False), mk(True)
    assert not dense.sparse_tables and len(sparse.sparse_tables) == 2
    assert sparse.num_params < dense.num_params - 800 * 16 + 128
    torch.manual_seed(0)
    ins = {"dense": torch.randn(64, 13, device="cuda"), "sparse0": torch.randint(0, 500, (64, 1), device="cuda"),
           "sparse1": torch.randint(0, 300, (64, 1), device="cuda")}
    labels = torch.rand(64, 1, device="cuda")
    for _ in range(5):
        dense.train_step(ins, labels)
        sparse.train_step(ins, labels)
        assert abs(dense.mean_loss() - sparse.mean_loss()) < 3e-2 * abs(dense.mean_loss()) + 1e-4
    d = dict(dense.named_parameters())
    s = dict(sparse.named_parameters())
    for name in ("emb0.weight", "emb1.weight"):
        assert s[name].dtype == torch.float32
        # the dense path rounds the table gradient to bf16 before the update; the sparse path does not
        assert float((d[name] - s[name]).abs().max()) < 2e-3
    sd = sparse.state_dict()
    assert "table.emb0.weight" in sd
    # a momentum optimizer keeps the dense path
    mom = Executable(cg, ExecConfig(compute_dtype="bf16", seed=2, optimizer=OptimizerConfig(kind="sgd", lr=0.05, momentum=0.9),
                                    loss="mean_squared_error_avg_reduce"))
    assert not mom.sparse_tables


def test_checkpoint_carries_sparse_embedding_tables(tmp_path):
    """Sparsely updated tables live outside the parameter arena: a checkpoint stores them by name, a plain load
    restores them, and a load by name moves them between the sparse and the dense (arena) representation."""
    from flexflow_train_b200 import _ffcore as core
    from flexflow_train_b200.runtime.executor import ExecConfig, Executable, OptimizerConfig
    from flexflow_train_b200.utils import checkpoint as ckpt

    cfg = {"batch_size": 64, "embedding_dim": 16, "embedding_bag_size": 1, "embedding_size": [500, 300],
           "dense_arch_layer_sizes": [13, 32, 16], "over_arch_layer_sizes": [48, 32, 1], "arch_interaction_op": "DOT",
           "final_activation": "SIGMOID", "embedding_data_type": "FLOAT"}
    cg = core.build_model("dlrm", cfg)
    mk = lambda sparse, seed: Executable(cg, ExecConfig(compute_dtype="bf16", seed=seed, loss="mean_squared_error_avg_reduce",
                                                        optimizer=OptimizerConfig(kind="sgd", lr=0.05), sparse_embedding_update=sparse))
    torch.manual_seed(0)
    ins = {"dense": torch.randn(64, 13, device="cuda"), "sparse0": torch.randint(0, 500, (64, 1), device="cuda"),
           "sparse1": torch.randint(0, 300, (64, 1), device="cuda")}
    labels = torch.rand(64, 1, device="cuda")
    a = mk(True, 2)
    for _ in range(3):
        a.train_step(ins, labels)
    path = ckpt.save(str(tmp_path), a)
    b = mk(True, 9)  # other initial weights
    ckpt.load(path, b)
    pa, pb = dict(a.named_parameters()), dict(b.named_parameters())
    assert set(pa) == set(pb) and "emb0.weight" in pa
    for k in pa:
        assert torch.equal(pa[k], pb[k]), k
    a.train_step(ins, labels)
    b.train_step(ins, labels)
    assert abs(a.mean_loss() - b.mean_loss()) < 1e-6
    # by name into an executable that keeps the tables in the dense arenas, and back
    d = mk(False, 9)
    ckpt.load_resharded(path, d)
    pd = dict(d.named_parameters())
    full = ckpt.gather_full_parameters(path)
    for k in ("emb0.weight", "emb1.weight", "top0.weight"):
        assert torch.equal(pd[k].cpu(), full[k]), k
    path2 = ckpt.save(str(tmp_path / "dense"), d)
    e = mk(True, 11)
    ckpt.load_resharded(path2, e)
    assert torch.equal(dict(e.named_parameters())["emb1.weight"].cpu(), full["emb1.weight"])


def test_measured_costs_fill_the_search_estimator(tmp_path):
    """FFConfig.measure_costs: one profiled step per data-parallel shard size fills the estimator the search runs on, and
    the table is written to (then read from) the disk cache."""
    from flexflow_train_b200 import _ffcore as core
    from flexflow_train_b200.api import FFConfig, _search_estimator
    from flexflow_train_b200.runtime.executor import ExecConfig
    cfg_model = {"batch_size": 64}
    cg = core.build_model("mlp", cfg_model)
    path = tmp_path / "table.json"
    cfg = FFConfig(measure_costs=True, cost_table_file=str(path))
    est, info = _search_estimator("mlp", cfg_model, cg, 2, cfg, None, ExecConfig(compute_dtype="bf16"))
    assert info["source"] == "measured" and info["entries"] > 0 and est.num_measured() == info["entries"]
    lin = [n["id"] for n in cg.nodes() if n["type"] == "LINEAR"][0]
    cost = est.op_cost(cg, lin)
    assert cost["fwd_ms"] > 0 and cost["bwd_ms"] > 0
    # the half-batch graph of a 2-way data-parallel plan was measured too
    half = core.build_model("mlp", {"batch_size": 32})
    lin_h = [n["id"] for n in half.nodes() if n["type"] == "LINEAR"][0]
    measured_half = est.op_cost(half, lin_h)
    analytic_half = core.CostEstimator(__import__("flexflow_train_b200.compiler.strategy", fromlist=["machine_for"]).machine_for(2)).op_cost(half, lin_h)
    assert measured_half != analytic_half
    assert path.exists()
    est2, info2 = _search_estimator("mlp", cfg_model, cg, 2, FFConfig(cost_table_file=str(path)), None, ExecConfig())
    assert info2 == {"source": str(path), "entries": info["entries"]}
    assert est2.op_cost(cg, lin) == cost


def test_executor_buffers_come_from_the_tracked_allocator():
    """Arenas, activations and scratch are handed out by the executor's allocator, which counts them."""
    from flexflow_train_b200 import _ffcore as core
    from flexflow_train_b200.runtime.executor import ExecConfig, Executable
    cg = core.build_model("mlp", {"batch_size": 32})
    ex = Executable(cg, ExecConfig(compute_dtype="bf16"))
    rep = ex.memory_report()
    params = sum(n for _, n in ex.param_offsets.values())
    # fp32 master + bf16 shadow + bf16 gradients at least
    assert rep["current_bytes"] >= params * (4 + 2 + 2) and rep["peak_bytes"] >= rep["current_bytes"]
    assert ex.allocator.inner.num_live > 4
    small = Executable(core.build_model("mlp", {"batch_size": 8}), ExecConfig(compute_dtype="bf16"))
    assert small.memory_report()["current_bytes"] < rep["current_bytes"]
