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
    pcg = S.data_parallel_strategy(cg, W) if which == "dp" else S.tensor_parallel_strategy(cg, W)
    opt = OptimizerConfig(kind="adam", lr=1e-3)
    single = Executable(cg, ExecConfig(compute_dtype="bf16", seed=4, optimizer=opt, device=f"cuda:{ctx.rank}"))
    multi = DistExecutable(pcg, ExecConfig(compute_dtype="bf16", seed=4, optimizer=opt, device=f"cuda:{ctx.rank}"), ctx)
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
    return {"single": a, "multi": b, "parallelism": multi.parallelism}


def w_dp(ctx):
    return _train(ctx, "dp")


def w_tp(ctx):
    return _train(ctx, "tp")


@pytest.mark.parametrize("which", ["dp", "tp"])
def test_two_rank_training_matches_single_gpu(which):
    res = _run("test_dist_executor_gpu:w_" + which)
    for r, out in res.items():
        assert which in out["parallelism"], out
        for x, y in zip(out["single"], out["multi"]):
            assert abs(x - y) < 3e-2 * abs(x), out
        assert out["multi"][-1] < out["multi"][0]
