"""Peer-memory collectives and fused compute+collective kernels on 2+ GPUs, each against an NCCL / PyTorch
reference.  Every worker is one process per GPU; results come back through a queue."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fn_name, q):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flexflow_train_b200.parallel.context import DistContext

        ctx = DistContext(rank, world, rank)
        if ":" in fn_name:
            import importlib

            mod, f = fn_name.split(":")
            res = getattr(importlib.import_module(mod), f)(ctx)
        else:
            res = globals()[fn_name](ctx)
        torch.cuda.synchronize()
        ctx.check_status()
        q.put((rank, "ok", res))
    except Exception as e:  # report instead of hanging the parent
        import traceback

        q.put((rank, "error", traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def _run(fn_name, world=2):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    port = _free_port()
    procs = [ctxm.Process(target=_worker, args=(r, world, port, fn_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    for _ in range(world):
        results.append(q.get(timeout=300))
    for p in procs:
        p.join(timeout=60)
    for rank, status, payload in results:
        assert status == "ok", f"rank {rank}:\n{payload}"
    return {r: p for r, _, p in results}


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


# ------------------------------------------------------------------ worker bodies
def w_allreduce(ctx):
    import torch.distributed as dist
    from flexflow_train_b200.parallel.fused_ops import GradAllReduce

    n = 10_000_003
    ar = GradAllReduce(ctx, n, torch.bfloat16)
    out = []
    for it in range(3):  # repeated calls exercise the epoch protocol
        torch.manual_seed(100 * it + ctx.rank)
        g = torch.randn(n, device=ctx.device).to(torch.bfloat16)
        ar.tensor.copy_(g)
        ref = g.float().clone()
        dist.all_reduce(ref)
        ref *= 0.5
        ar.run(scale=0.5)
        torch.cuda.synchronize()
        out.append(_rel(ar.tensor, ref))
    return out


def w_allgather_gemm(ctx):
    import torch.distributed as dist
    from flexflow_train_b200.parallel.fused_ops import AllGatherGemm

    W = ctx.world_size
    rows_local, k, n = 512, 1024, 768
    op = AllGatherGemm(ctx, rows_local, k)
    errs = []
    for it in range(2):
        torch.manual_seed(7 + it * 10 + ctx.rank)
        x = torch.randn(rows_local, k, device=ctx.device, dtype=torch.bfloat16)
        w = torch.randn(n, k, device=ctx.device, dtype=torch.bfloat16)
        out = torch.empty(W * rows_local, n, device=ctx.device, dtype=torch.bfloat16)
        op(x, w, out)
        xs = [torch.empty_like(x) for _ in range(W)]
        dist.all_gather(xs, x)
        ref = torch.cat(xs).float() @ w.float().t()
        torch.cuda.synchronize()
        errs.append(_rel(out, ref))
    return errs


def w_gemm_reduce_scatter(ctx):
    import torch.distributed as dist
    from flexflow_train_b200.parallel.fused_ops import GemmReduceScatter

    W = ctx.world_size
    rows, k_local, n = 256 * W, 512, 1024
    op = GemmReduceScatter(ctx, rows, n)
    errs = []
    for it in range(2):
        torch.manual_seed(11 + it * 10 + ctx.rank)
        x = torch.randn(rows, k_local, device=ctx.device, dtype=torch.bfloat16)
        w = torch.randn(n, k_local, device=ctx.device, dtype=torch.bfloat16)
        res = torch.randn(rows // W, n, device=ctx.device, dtype=torch.bfloat16)
        out = torch.empty(rows // W, n, device=ctx.device, dtype=torch.bfloat16)
        op(x, w, out, residual=res)
        full = x.float() @ w.float().t()
        dist.all_reduce(full)
        ref = full[ctx.rank * (rows // W):(ctx.rank + 1) * (rows // W)] + res.float()
        torch.cuda.synchronize()
        errs.append(_rel(out, ref))
    return errs


def w_alltoall_embedding(ctx):
    import torch.distributed as dist
    from flexflow_train_b200.parallel.fused_ops import AllToAllEmbedding

    W = ctx.world_size
    num_tables, dim, entries, local_batch = 4 * W, 64, 1000, 32
    gb = local_batch * W
    torch.manual_seed(3)  # same seed everywhere: every rank can build every table for the reference
    all_tables = [torch.randn(entries, dim, device=ctx.device) for _ in range(num_tables)]
    idx = torch.randint(0, entries, (gb, num_tables), device=ctx.device)
    local = [all_tables[t].clone() for t in range(num_tables) if t % W == ctx.rank]
    op = AllToAllEmbedding(ctx, local, num_tables, dim, local_batch, out_dtype=torch.float32)
    out = op.forward(idx)
    ref = torch.stack([all_tables[t][idx[:, t]] for t in range(num_tables)], 1)  # [gb, T, dim]
    mine = ref[ctx.rank * local_batch:(ctx.rank + 1) * local_batch]
    torch.cuda.synchronize()
    e_fwd = _rel(out, mine)
    # backward: dout = 1 for my samples; table rows move by -lr * (number of hits over the global batch)
    op.dout_t.fill_(1.0)
    op.backward_sgd(idx, lr=0.5)
    torch.cuda.synchronize()
    errs = []
    for i, t in enumerate(t_ for t_ in range(num_tables) if t_ % W == ctx.rank):
        exp = all_tables[t].clone()
        exp.index_add_(0, idx[:, t], torch.full((gb, dim), -0.5, device=ctx.device))
        errs.append(_rel(local[i], exp))
    return [e_fwd, max(errs)]


# ------------------------------------------------------------------ tests
def w_peer_collectives(ctx):
    """Stand-alone all-gather and reduce-scatter over peer memory against NCCL, called repeatedly on the same buffers (the
    barriers around the copies are what makes reuse safe), on the whole job and on a sub-group view of it."""
    import torch.distributed as dist
    from flexflow_train_b200.parallel.fused_ops import PeerAllGather, PeerReduceScatter

    W, r = ctx.world_size, ctx.rank
    out = {}
    for dtype in (torch.bfloat16, torch.float32):
        n = 3 * 1024 + 8
        ag = PeerAllGather(ctx, n, dtype)
        rs = PeerReduceScatter(ctx, n, dtype)
        worst_ag = worst_rs = 0.0
        for it in range(4):
            torch.manual_seed(100 * it + r)
            shard = torch.randn(n, device="cuda").to(dtype)
            got = ag(shard).clone()
            ref = torch.empty(W, n, device="cuda", dtype=dtype)
            dist.all_gather_into_tensor(ref.view(-1), shard)
            worst_ag = max(worst_ag, float((got.float() - ref.float()).abs().max()))
            full = torch.randn(W * n, device="cuda").to(dtype)
            base = torch.randn(n, device="cuda").to(dtype)
            mine = base.clone()
            rs(full, mine, accumulate=(it % 2 == 1))
            ref_rs = torch.empty(n, device="cuda", dtype=torch.float32)
            dist.reduce_scatter_tensor(ref_rs, full.float())
            if it % 2 == 1:
                ref_rs += base.float()
            worst_rs = max(worst_rs, _rel(mine, ref_rs))
        out[str(dtype)] = (worst_ag, worst_rs)
    return out


def test_peer_all_gather_and_reduce_scatter_match_nccl():
    res = _run("w_peer_collectives")
    for rank, by_dtype in res.items():
        for dt, (e_ag, e_rs) in by_dtype.items():
            assert e_ag == 0.0, (rank, dt, e_ag)
            assert e_rs < (1e-2 if "bfloat16" in dt else 1e-5), (rank, dt, e_rs)


def test_grad_allreduce_scale_matches_nccl():
    res = _run("w_allreduce")
    for r, errs in res.items():
        assert max(errs) < 1e-2, (r, errs)


def test_allgather_gemm_matches_reference():
    res = _run("w_allgather_gemm")
    for r, errs in res.items():
        assert max(errs) < 1e-2, (r, errs)


def test_gemm_reduce_scatter_matches_reference():
    res = _run("w_gemm_reduce_scatter")
    for r, errs in res.items():
        assert max(errs) < 1e-2, (r, errs)


def test_alltoall_embedding_matches_reference():
    res = _run("w_alltoall_embedding")
    for r, errs in res.items():
        assert max(errs) < 1e-4, (r, errs)


def w_wait_expires(ctx):
    import time

    from flexflow_train_b200.ops import kernels as K
    from flexflow_train_b200.parallel import comm
    from flexflow_train_b200.utils.failure import CommTimeoutError

    n = 4096
    stage = torch.ones(1, n, device=ctx.device, dtype=torch.bfloat16)
    out = torch.zeros(n, device=ctx.device, dtype=torch.bfloat16)
    base, sync = ctx.alloc_flags(1), ctx.new_sync()
    torch.cuda.synchronize()
    t0 = time.time()
    comm.reduce_partials(ctx, stage, out, 1, base, sync)  # waits for a source flag that no peer will ever raise
    torch.cuda.synchronize()
    waited = time.time() - t0
    try:
        ctx.check_status()
        raised = False
    except CommTimeoutError:
        raised = True
    # the kernel returned by itself: the context is intact, later work runs, the status word is clear again
    a = torch.randn(256, 128, device=ctx.device, dtype=torch.bfloat16)
    b = torch.randn(192, 128, device=ctx.device, dtype=torch.bfloat16)
    err = float((K.matmul_nt(a, b).float() - a.float() @ b.float().t()).abs().max())
    ctx.check_status()
    return {"raised": raised, "waited": waited, "untouched": float(out.float().abs().max()) == 0.0, "gemm_err": err}


def test_device_side_wait_runs_out_and_reports_instead_of_hanging():
    """Failure detection on the device: a peer that never signals costs the bounded wait (about two seconds), after
    which the kernel records a timeout code that the host turns into CommTimeoutError; nothing hangs or faults."""
    out = _run("w_wait_expires", world=1)[0]
    assert out["raised"] and out["untouched"], out
    assert 1.0 < out["waited"] < 20.0, out
    assert out["gemm_err"] < 1.0, out
