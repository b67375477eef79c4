"""The SPMD executor on 2 GPUs: data-parallel and tensor-parallel strategies must train like one GPU does."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from test_comm_gpu import _run  # noqa: E402  (process-per-GPU harness)

CFG = {"num_features": 256, "sequence_length": 128, "batch_size": 8, "dim_feedforward": 512, "num_heads": 4,
       "num_decoder_layers": 2, "dropout": 0.0, "vocab_size": 512}


def _train(ctx, which):
    from flexflow_train_b200 import _ffcore as core
    from flexflow_train_b200.compiler import strategy as S
    from flexflow_train_b200.parallel.dist_executor import DistExecutable
    from flexflow_train_b200.runtime.executor import ExecConfig, Executable, OptimizerConfig

    cg = core.build_model("transformer_lm", CFG)
    W = ctx.world_size
    if which.startswith("dp"):
        pcg = S.data_parallel_strategy(cg, W)
    else:
        pcg = S.tensor_parallel_strategy(cg, W, sequence_parallel=which != "tp_replicated")
    opt = OptimizerConfig(kind="adam", lr=1e-3)
    single = Executable(cg, ExecConfig(compute_dtype="bf16", seed=4, optimizer=opt, device=f"cuda:{ctx.rank}"))
    multi = DistExecutable(pcg, ExecConfig(compute_dtype="bf16", seed=4, optimizer=opt, device=f"cuda:{ctx.rank}"), ctx,
                           fuse_collectives=which != "tp_nccl", fuse_optimizer=which != "dp_allreduce")
    torch.manual_seed(0)
    ids = torch.randint(0, 512, (8, 128, 1), dtype=torch.int32, device=ctx.device)
    labels = torch.randint(0, 512, (8, 128), dtype=torch.int32, device=ctx.device)
    a, b = [], []
    for _ in range(4):
        single.train_step({"input_ids": ids}, labels)
        a.append(single.mean_loss())
        multi.train_step({"input_ids": ids}, labels)
        b.append(multi.mean_loss())
    ctx.check_status()
    # the sharded update leaves each rank with the fp32 state of its own slices; consolidated, it must match the
    # bf16 weights every rank computes with
    sd = multi.state_dict()
    drift = float((sd["master"][:multi.rep_numel].to(torch.bfloat16).float() - multi.shadow[:multi.rep_numel].float()).abs().max())
    return {"single": a, "multi": b, "parallelism": multi.parallelism, "fused_in": len(multi.fused_in),
            "fused_out": len(multi.fused_out), "fused_update": bool(multi.fused_update), "drift": drift}


def w_dp(ctx):
    return _train(ctx, "dp")


def w_dp_allreduce(ctx):
    return _train(ctx, "dp_allreduce")


def w_tp(ctx):
    return _train(ctx, "tp")


def w_tp_nccl(ctx):
    return _train(ctx, "tp_nccl")


def w_tp_replicated(ctx):
    return _train(ctx, "tp_replicated")


@pytest.mark.parametrize("which", ["dp", "dp_allreduce", "tp", "tp_nccl", "tp_replicated"])
def test_two_rank_training_matches_single_gpu(which):
    """dp: data parallel, gradient reduce-scatter + sharded optimizer update + weight all-gather in one kernel per
    bucket.  dp_allreduce: gradient all-reduce kernel, every rank updates every weight.  tp: tensor + sequence parallel with the collectives
    fused into the GEMMs (all-gather -> GEMM, GEMM -> reduce-scatter).  tp_nccl: the same strategy on NCCL
    reduce-scatter / all-gather.  tp_replicated: the plain Megatron template with replicated activations."""
    res = _run("test_dist_executor_gpu:w_" + which)
    for r, out in res.items():
        assert which[:2] in out["parallelism"], out
        assert out["fused_update"] == (which != "dp_allreduce") and out["drift"] == 0.0, out
        if which == "tp":  # per layer: attention and the MLP each have one fused input and one fused output
            assert out["fused_in"] == 4 and out["fused_out"] == 4, out
        else:
            assert out["fused_in"] == 0 and out["fused_out"] == 0, out
        for x, y in zip(out["single"], out["multi"]):
            assert abs(x - y) < 3e-2 * abs(x), out
        assert out["multi"][-1] < out["multi"][0]


def w_mesh(ctx):
    """dp x tp on a two-axis device mesh (4 ranks: 2 x 2; 8 ranks: 4 x 2) against one GPU: same losses over four Adam
    steps, same first-step gradients of every weight shard, inputs fed as each data-parallel group's own rows."""
    from flexflow_train_b200 import _ffcore as core
    from flexflow_train_b200.compiler import strategy as S
    from flexflow_train_b200.parallel.dist_executor import DistExecutable
    from flexflow_train_b200.runtime.executor import ExecConfig, Executable, OptimizerConfig

    cfg = dict(CFG, sequence_length=64)
    cg = core.build_model("transformer_lm", cfg)
    W = ctx.world_size
    tp = 2
    dp = W // tp
    pcg = S.hybrid_strategy(cg, dp, tp)
    opt = OptimizerConfig(kind="adam", lr=1e-3)
    single = Executable(cg, ExecConfig(compute_dtype="bf16", seed=4, optimizer=opt, device=f"cuda:{ctx.rank}"))
    multi = DistExecutable(pcg, ExecConfig(compute_dtype="bf16", seed=4, optimizer=opt, device=f"cuda:{ctx.rank}"), ctx,
                           shard_inputs=True, fuse_optimizer=False)   # plain all-reduce: the summed gradients stay readable
    torch.manual_seed(0)
    ids = torch.randint(0, 512, (8, 64, 1), dtype=torch.int32, device=ctx.device)
    labels = torch.randint(0, 512, (8, 64), dtype=torch.int32, device=ctx.device)
    lb = 8 // dp
    i_dp = ctx.rank // tp
    my_ids, my_labels = ids[i_dp * lb:(i_dp + 1) * lb].contiguous(), labels[i_dp * lb:(i_dp + 1) * lb].contiguous()
    # first step by hand: gradients before any update
    single.set_inputs({"input_ids": ids}, labels)
    single.forward(); single.compute_loss(); single.backward()
    multi.set_inputs({"input_ids": my_ids}, my_labels)
    multi.forward(); multi.compute_loss(); multi.backward(); multi.sync_gradients()
    torch.cuda.synchronize()
    ref = dict(single.named_gradients())
    worst = 0.0
    report = []   # (relative error, weight, norm ratio) of the worst few, for the failure message
    for nid, (name, g) in zip(multi.param_nodes, multi.named_gradients()):
        full = ref[name].float()
        shard = multi.shard_weight(nid, full.view(list(multi.nodes[nid]["outputs"][0][1].sizes))).reshape(-1)
        # the bucket kernel leaves the data-parallel sum in the gradient arena when the update is not fused into it
        err = float((g.float().reshape(-1) - shard).norm() / (shard.norm() + 1e-9))
        worst = max(worst, err)
        report.append((round(err, 4), name, round(float(g.float().norm() / (shard.norm() + 1e-9)), 4)))
    report = sorted(report, reverse=True)[:6]
    a, b = [], []
    single2 = Executable(cg, ExecConfig(compute_dtype="bf16", seed=4, optimizer=opt, device=f"cuda:{ctx.rank}"))
    multi2 = DistExecutable(pcg, ExecConfig(compute_dtype="bf16", seed=4, optimizer=opt, device=f"cuda:{ctx.rank}", use_cuda_graph=True), ctx,
                            shard_inputs=True)
    for _ in range(4):
        single2.train_step({"input_ids": ids}, labels)
        a.append(single2.mean_loss())
        multi2.train_step({"input_ids": my_ids}, my_labels)
        b.append(multi2.mean_loss())
    # plain SGD is sensitive to the scale of the reduced gradients (Adam is not)
    sgd = OptimizerConfig(kind="sgd", lr=0.05)
    single3 = Executable(cg, ExecConfig(compute_dtype="bf16", seed=4, optimizer=sgd, device=f"cuda:{ctx.rank}"))
    multi3 = DistExecutable(pcg, ExecConfig(compute_dtype="bf16", seed=4, optimizer=sgd, device=f"cuda:{ctx.rank}"), ctx, shard_inputs=True)
    c, d = [], []
    for _ in range(3):
        single3.train_step({"input_ids": ids}, labels)
        c.append(single3.mean_loss())
        multi3.train_step({"input_ids": my_ids}, my_labels)
        d.append(multi3.mean_loss())
    ctx.check_status()
    return {"single": a, "multi": b, "single_sgd": c, "multi_sgd": d, "parallelism": multi2.parallelism, "worst_grad_err": worst, "nccl_ops": len(multi2.nccl_ops),
            "graph": bool(multi2.cfg.use_cuda_graph), "direct": sorted(multi2.direct_inputs), "worst_weights": report}


def test_mesh_dp_x_tp_matches_single_gpu():
    n = torch.cuda.device_count()
    world = 8 if n >= 8 else 4
    res = _run("test_dist_executor_gpu:w_mesh", world=world)
    for r, out in res.items():
        print(r, out)   # shown when an assertion below fails
        assert out["parallelism"] == f"dp{world // 2}xtp2" and out["direct"] == ["input_ids"], out
        assert out["nccl_ops"] == 0 and out["graph"], out   # the step is one captured graph: no library collective in it
        for x, y in zip(out["single"] + out["single_sgd"], out["multi"] + out["multi_sgd"]):
            assert abs(x - y) < 3e-2 * abs(x), out
        assert out["multi"][-1] < out["multi"][0]
        assert out["worst_grad_err"] < 5e-2, out


def _train_graph(ctx, build, loss, inputs_fn, steps=4):
    """Single-GPU vs data-parallel training of an arbitrary graph on the same global batch."""
    from flexflow_train_b200.compiler import strategy as S
    from flexflow_train_b200.parallel.dist_executor import DistExecutable
    from flexflow_train_b200.runtime.executor import ExecConfig, Executable, OptimizerConfig

    cg = build()
    pcg = S.data_parallel_strategy(cg, ctx.world_size)
    opt = OptimizerConfig(kind="sgd", lr=0.05, momentum=0.9)
    cfg = dict(compute_dtype="bf16", seed=2, optimizer=opt, device=f"cuda:{ctx.rank}", loss=loss)
    single = Executable(cg, ExecConfig(**cfg))
    multi = DistExecutable(pcg, ExecConfig(**cfg), ctx)
    torch.manual_seed(0)
    inputs, labels = inputs_fn(ctx.device)
    a, b = [], []
    for _ in range(steps):
        single.train_step(inputs, labels)
        a.append(single.mean_loss())
        multi.train_step(inputs, labels)
        b.append(multi.mean_loss())
    ctx.check_status()
    return {"single": a, "multi": b, "parallelism": multi.parallelism, "nccl_ops": len(multi.nccl_ops)}


def w_conv_dp(ctx):
    from flexflow_train_b200 import _ffcore as core

    def build():
        b = core.GraphBuilder()
        x = b.create_input([8, 3, 20, 20], name="input")
        t = b.conv2d(x, 16, 3, 3, 1, 1, 1, 1, activation="RELU", name="c1")
        t = b.pool2d(t, 2, 2, 2, 2, 0, 0, pool_type="MAX", name="p1")
        l = b.conv2d(t, 16, 1, 1, name="b1")
        r = b.conv2d(t, 8, 3, 3, 1, 1, 1, 1, activation="RELU", name="b2")
        t = b.concat([l, r], 1, name="cat")
        t = b.pool2d(t, 10, 10, 1, 1, 0, 0, pool_type="AVG", name="gap")
        b.softmax(b.dense(b.flat(t, name="flat"), 10, name="fc"), name="out_prob")
        return b.graph
    return _train_graph(ctx, build, "sparse_categorical_crossentropy",
                        lambda dev: ({"input": torch.randn(8, 3, 20, 20, device=dev)}, torch.randint(0, 10, (8,), dtype=torch.int32, device=dev)))


def w_dlrm_dp(ctx):
    from flexflow_train_b200 import _ffcore as core

    cfg = {"batch_size": 64, "embedding_dim": 16, "embedding_bag_size": 1, "embedding_size": [500, 300], "dense_arch_layer_sizes": [13, 32, 16],
           "over_arch_layer_sizes": [48, 32, 1], "arch_interaction_op": "CAT", "final_activation": "SIGMOID"}

    def data(dev):
        ins = {"dense": torch.randn(64, 13, device=dev), "sparse0": torch.randint(0, 500, (64, 1), device=dev),
               "sparse1": torch.randint(0, 300, (64, 1), device=dev)}
        return ins, torch.rand(64, 1, device=dev)
    return _train_graph(ctx, lambda: core.build_model("dlrm", cfg), "mean_squared_error_avg_reduce", data)


@pytest.mark.parametrize("which", ["conv_dp", "dlrm_dp"])
def test_data_parallel_convolution_stack_and_dlrm_match_single_gpu(which):
    """Batch norm is left out of the convolution stack on purpose: under data parallelism it normalises with the
    statistics of the local samples, which is not the single-GPU function."""
    res = _run("test_dist_executor_gpu:w_" + which)
    for r, out in res.items():
        assert "dp" in out["parallelism"], out
        for x, y in zip(out["single"], out["multi"]):
            assert abs(x - y) < 5e-2 * abs(x) + 1e-3, out
        assert out["multi"][-1] < out["multi"][0], out


def w_dlrm_tables(ctx):
    """Embedding tables model-parallel (one all-to-all kernel in each direction), MLPs data-parallel."""
    from flexflow_train_b200 import _ffcore as core
    from flexflow_train_b200.compiler import strategy as S
    from flexflow_train_b200.parallel.dist_executor import AllToAllEmbeddingOp, DistExecutable
    from flexflow_train_b200.runtime.executor import ExecConfig, Executable, OptimizerConfig

    cfg = {"batch_size": 64, "embedding_dim": 16, "embedding_bag_size": 1, "embedding_size": [500, 300, 200, 100],
           "dense_arch_layer_sizes": [13, 32, 16], "over_arch_layer_sizes": [48, 32, 1], "arch_interaction_op": "DOT",
           "final_activation": "SIGMOID", "embedding_data_type": "FLOAT"}
    cg = core.build_model("dlrm", cfg)
    pcg = S.table_parallel_strategy(cg, ctx.world_size)
    opt = OptimizerConfig(kind="sgd", lr=0.05, momentum=0.0)
    ecfg = dict(compute_dtype="bf16", seed=2, optimizer=opt, device=f"cuda:{ctx.rank}", loss="mean_squared_error_avg_reduce")
    single = Executable(cg, ExecConfig(**ecfg))
    multi = DistExecutable(pcg, ExecConfig(use_cuda_graph=True, **ecfg), ctx)
    torch.manual_seed(0)
    ins = {"dense": torch.randn(64, 13, device=ctx.device)}
    for i, n in enumerate(cfg["embedding_size"]):
        ins[f"sparse{i}"] = torch.randint(0, n, (64, 1), device=ctx.device)
    labels = torch.rand(64, 1, device=ctx.device)
    a, b = [], []
    for _ in range(6):
        single.train_step(ins, labels)
        a.append(single.mean_loss())
        multi.train_step(ins, labels)
        b.append(multi.mean_loss())
    ctx.check_status()
    names = {single.nodes[n]["name"]: t for n, t in single.sparse_tables.items()}
    owned = {multi.nodes[n]["name"]: t for n, t in multi.sparse_tables.items() if t is not None}
    diff = max(float((names[k] - t).abs().max()) for k, t in owned.items())
    moved = max(float((t - t.mean()).abs().max()) for t in owned.values())
    return {"single": a, "multi": b, "parallelism": multi.parallelism, "owned": sorted(owned), "table_diff": diff, "moved": moved,
            "a2a_ops": sum(isinstance(o, AllToAllEmbeddingOp) for o in multi.ops.values()), "graph": bool(multi.cfg.use_cuda_graph),
            "dense_params": int(multi.num_params)}


def test_model_parallel_embedding_tables_match_single_gpu():
    res = _run("test_dist_executor_gpu:w_dlrm_tables")
    for r, out in res.items():
        assert out["parallelism"] == "dp2+tables_mp2" and out["a2a_ops"] == 1 and out["graph"], out
        assert out["owned"] == [f"emb{r}.weight", f"emb{r + 2}.weight"], out   # table t lives on rank t % world
        assert out["dense_params"] < 20000, out                                # no table in the dense arenas
        for x, y in zip(out["single"], out["multi"]):
            assert abs(x - y) < 5e-2 * abs(x) + 1e-3, out
        assert out["table_diff"] < 2e-3, out
        assert out["multi"][-1] < out["multi"][0], out
