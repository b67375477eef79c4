"""Failure detection across processes, on CPU (gloo): a rank leaves between steps; the others learn of it from
the heartbeat store before their next collective and stop cleanly, then training resumes from the checkpoint
with the survivors."""
import os
import socket
import time

import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, fail_rank, fail_step, q):
    import datetime

    import torch.distributed as dist

    from flexflow_train_b200.utils import failure as F

    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=datetime.timedelta(seconds=20))
    dist.init_process_group("gloo", store=dist.PrefixStore("pg", store), rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=20))
    mon = F.HeartbeatMonitor(store, rank, world, timeout_s=1.0, grace_s=5.0)
    inj = F.FaultInjector(plan=[{"step": fail_step, "kind": "exit", "rank": fail_rank, "code": 17}], rank=rank, monitor=mon)
    w = torch.zeros(4)
    done = 0
    try:
        for step in range(8):
            mon.beat(step)
            if rank == fail_rank and step == fail_step:
                q.put((rank, "leaving", step))
                time.sleep(0.2)
            inj.maybe_fail(step)  # the failing rank leaves here: between steps, nothing in flight
            if step >= fail_step:
                # survivors: give the monitor time to see the silence before they would enter a collective
                deadline = time.time() + 4.0
                while time.time() < deadline:
                    mon.beat(step)
                    mon.check()
                    time.sleep(0.1)
            g = torch.full((4,), float(rank + 1))
            dist.all_reduce(g)
            w += g
            done += 1
        q.put((rank, "finished", done))
    except F.RankFailure as e:
        q.put((rank, "rank_failure", (done, e.ranks)))
    finally:
        # no destroy_process_group: a peer is gone, a collective shutdown could block
        q.close()
        q.join_thread()
        if rank == 0:
            time.sleep(1.0)  # rank 0 hosts the store; let the other survivor finish reading it
        os._exit(0)


def test_rank_exit_is_detected_by_survivors_before_next_collective():
    world, fail_rank, fail_step = 3, 2, 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, fail_rank, fail_step, q)) for r in range(world)]
    for p in procs:
        p.start()
    msgs = [q.get(timeout=60) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    by_rank = {}
    for r, kind, payload in msgs:
        by_rank.setdefault(r, []).append((kind, payload))
    assert by_rank[fail_rank][0][0] == "leaving"
    assert procs[fail_rank].exitcode == 17
    for r in (0, 1):
        kind, (done, dead) = by_rank[r][0]
        assert kind == "rank_failure" and dead == [fail_rank]
        assert done == fail_step  # every step before the failure completed on the survivors


def _watchdog_worker(rank, world, port, q):
    import time

    import torch
    import torch.distributed as dist

    from flexflow_train_b200.utils import failure as F

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    wd = F.CollectiveWatchdog(timeout_s=3.0).init_process_group("gloo", rank=rank, world_size=world)
    t = torch.ones(4)
    wd.run(dist.all_reduce, t)  # everyone takes part: fine
    ok = float(t[0]) == world
    if rank == world - 1:
        # this rank leaves between steps (no collective of its own in flight) and never joins the next one
        q.put((rank, "left", ok))
        q.close(); q.join_thread()
        time.sleep(8)
        os._exit(0)
    t0 = time.time()
    try:
        wd.run(dist.all_reduce, t)
        res = "completed"
    except F.RankFailure:
        res = "rank_failure"
    q.put((rank, res, time.time() - t0))
    q.close(); q.join_thread()
    os._exit(0)


def test_collective_watchdog_turns_a_missing_peer_into_rank_failure():
    """Host-side failure injection on gloo ranks: a peer that never joins a collective makes the survivors' call end
    with RankFailure within the process-group timeout instead of blocking."""
    import torch.multiprocessing as mp

    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_watchdog_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    msgs = [q.get(timeout=90) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    by_rank = {m[0]: m for m in msgs}
    assert by_rank[world - 1][1] == "left" and by_rank[world - 1][2]
    for r in range(world - 1):
        assert by_rank[r][1] == "rank_failure", by_rank
        assert by_rank[r][2] < 30, by_rank
