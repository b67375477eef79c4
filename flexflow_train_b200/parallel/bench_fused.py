"""Roofline micro-benchmark of the fused compute+collective kernels, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m flexflow_train_b200.parallel.bench_fused [--rows 32768 --d-model 2048 --d-ff 8192]

For each fused path it prints one JSON line (rank 0): device time (CUDA events, max over ranks), the time of the
unfused library path on the same operands (cuBLAS GEMM + NCCL collective, run back to back), and the roofline
fraction = max(FLOPs / measured GEMM peak, bytes that must cross NVLink / measured peer bandwidth) / achieved.

  F1  GEMM -> reduce-scatter   x[rows, d_ff/W] . w[d_model, d_ff/W]^T, partial sums scattered and reduced to row shards
  F2  all-gather -> GEMM       allgather(x[rows/W, d_model]) . w[d_ff/W, d_model]^T
  F3  gradient all-reduce + scale over a bf16 arena
  F4  all-to-all + embedding gather (tables model-parallel, samples data-parallel), forward and sparse-SGD backward
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..utils.profiling import roofline
from .context import DistContext
from .fused_ops import AllGatherGemm, AllToAllEmbedding, GemmReduceScatter, GradAllReduce


def _timed(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--rows", type=int, default=32768)
    p.add_argument("--d-model", type=int, default=2048)
    p.add_argument("--d-ff", type=int, default=8192)
    p.add_argument("--grad-elements", type=int, default=256 * 1024 * 1024)
    p.add_argument("--tables", type=int, default=8)
    p.add_argument("--table-rows", type=int, default=1000000)
    p.add_argument("--emb-dim", type=int, default=64)
    p.add_argument("--batch", type=int, default=4096)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--only", default="f1,f2,f3,f4")
    p.add_argument("--write-cost-params", metavar="FILE",
                   help="merge the bandwidths measured here into FILE as the cost model's measured_gbs table (key kind@world): the "
                        "search reads it through FFConfig.cost_params_file")
    p.add_argument("--no-scatter-tma", action="store_true", help="F1: per-lane stores into the peers' stages instead of TMA stores")
    a = p.parse_args(argv)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = DistContext(rank, world, local)
    W, dev, bf = world, ctx.device, torch.bfloat16
    only = set(a.only.split(","))
    if a.no_scatter_tma:
        from ..ops import kernels as K
        K.lib().ffk_gemm_set_scatter_tma_store(0)
    es = 2

    measured = {}   # collective kind -> achieved GB/s at this world size, in the units of the cost model

    def emit(d):
        ctx.check_status()
        if rank == 0:
            print(json.dumps(d), flush=True)

    if "f1" in only:
        rows, n, k = a.rows, a.d_model, a.d_ff // W
        x = torch.randn(rows, k, device=dev).to(bf)
        w = torch.randn(n, k, device=dev).to(bf)
        out = torch.empty(rows // W, n, device=dev, dtype=bf)
        op = GemmReduceScatter(ctx, rows, n)
        ms = _timed(lambda: op(x, w, out), a.warmup, a.iters)
        full = torch.empty(rows, n, device=dev, dtype=bf)

        def lib():
            torch.matmul(x, w.t(), out=full)
            dist.reduce_scatter_tensor(out, full)
        ms_lib = _timed(lib, a.warmup, a.iters)
        r = roofline(ms, flops=2.0 * rows * n * k, nvlink_bytes=(W - 1) / W * rows * n * es, sustained=True)
        if r["nvlink_gbs"] > 0 and r["bound"] != "compute":   # a compute-bound run says nothing about the link
            measured["reducescatter"] = r["nvlink_gbs"]
        emit({"kernel": "F1 gemm->reduce_scatter", "world": W, "rows": rows, "n": n, "k_local": k, "library_ms": ms_lib,
              "speedup_vs_library": ms_lib / ms, **r})
        del op, full

    if "f2" in only:
        rows_local, k, n = a.rows // W, a.d_model, a.d_ff // W
        x = torch.randn(rows_local, k, device=dev).to(bf)
        w = torch.randn(n, k, device=dev).to(bf)
        out = torch.empty(a.rows, n, device=dev, dtype=bf)
        op = AllGatherGemm(ctx, rows_local, k)
        ms = _timed(lambda: op(x, w, out), a.warmup, a.iters)
        gathered = torch.empty(a.rows, k, device=dev, dtype=bf)

        def lib():
            dist.all_gather_into_tensor(gathered, x)
            torch.matmul(gathered, w.t(), out=out)
        ms_lib = _timed(lib, a.warmup, a.iters)
        r = roofline(ms, flops=2.0 * a.rows * n * k, nvlink_bytes=(W - 1) * rows_local * k * es, sustained=True)
        if r["nvlink_gbs"] > 0 and r["bound"] != "compute":
            measured["allgather"] = r["nvlink_gbs"]
        emit({"kernel": "F2 all_gather->gemm", "world": W, "rows": a.rows, "n_local": n, "k": k, "library_ms": ms_lib,
              "speedup_vs_library": ms_lib / ms, **r})
        del op, gathered

    if "f3" in only:
        n = a.grad_elements
        ar = GradAllReduce(ctx, n, bf)
        ar.tensor.normal_()
        ms = _timed(lambda: ar.run(scale=1.0 / W), a.warmup, a.iters)
        t = torch.randn(n, device=dev).to(bf)

        def lib():
            dist.all_reduce(t)
            t.mul_(1.0 / W)
        ms_lib = _timed(lib, a.warmup, a.iters)
        sent = 2.0 * (W - 1) / W * n * es
        r = roofline(ms, hbm_bytes=3.0 * n * es, nvlink_bytes=sent)
        if W > 1:
            measured["allreduce"] = sent / ms / 1e6
        emit({"kernel": "F3 grad all_reduce+scale", "world": W, "elements": n, "library_ms": ms_lib, "speedup_vs_library": ms_lib / ms,
              "bus_gbs": sent / ms / 1e6, **r})
        del ar, t

    if "f4" in only and a.tables % W == 0 and a.batch % W == 0:
        T, dim, lb = a.tables, a.emb_dim, a.batch // W
        local = [torch.randn(a.table_rows, dim, device=dev) * 0.01 for _ in range(T // W)]
        op = AllToAllEmbedding(ctx, local, T, dim, lb, out_dtype=bf)
        idx = torch.randint(0, a.table_rows, (a.batch, T), device=dev)
        ms_f = _timed(lambda: op.forward(idx), a.warmup, a.iters)
        op.dout_t.fill_(1e-3)
        ms_b = _timed(lambda: op.backward_sgd(idx, lr=0.01), a.warmup, a.iters)
        sent = (W - 1) / W * a.batch * (T // W) * dim * es
        rf = roofline(ms_f, hbm_bytes=a.batch * (T // W) * dim * (4 + es), nvlink_bytes=sent)
        rb = roofline(ms_b, hbm_bytes=a.batch * (T // W) * dim * (es + 8), nvlink_bytes=sent)
        emit({"kernel": "F4 all_to_all+embedding fwd", "world": W, "tables": T, "batch": a.batch, "dim": dim, **rf})
        emit({"kernel": "F4 all_to_all+embedding sparse-SGD bwd", "world": W, "tables": T, "batch": a.batch, "dim": dim, **rb})

    if a.write_cost_params and rank == 0 and W > 1:
        doc = {}
        if os.path.exists(a.write_cost_params):
            with open(a.write_cost_params) as f:
                doc = json.load(f)
        table = doc.setdefault("measured_gbs", {})
        for kind, gbs in measured.items():
            table[f"{kind}@{W}"] = round(gbs, 1)
        with open(a.write_cost_params, "w") as f:
            json.dump(doc, f, indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
