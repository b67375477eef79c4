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
