"""flexflow-python: run a training script the way the legacy launcher did.

    python -m flexflow_train_b200.bin.flexflow_python train.py -ll:gpu 4 -ll:fsize 14000 -b 64 --epochs 2

The reference's ``flexflow_python`` (bindings/python/old/flexflow_python.py, flexflow/driver.py) starts the Legion runtime
with the resource flags of the command line and runs the script inside it.  Here a job is one process per GPU: the
launcher reads ``-ll:gpu N`` (GPUs on this node; default: the visible ones, or 1 without a GPU), drops the other runtime
flags with a note, and runs the script either in this process (one rank) or as N ranks under ``torch.distributed.run``
with the rendezvous on ``127.0.0.1`` (``--nodes`` / ``--node-rank`` / ``--master-addr`` for several machines).  What is left
of the command line reaches the script unchanged in ``sys.argv``.
"""
from __future__ import annotations

import argparse
import os
import runpy
import subprocess
import sys

from .run_model import split_runtime_flags


def _gpus_requested(ignored) -> int | None:
    for i, tok in enumerate(ignored):
        if tok.startswith("-ll:gpu"):
            if "=" in tok:
                return int(tok.split("=", 1)[1])
            if i + 1 < len(ignored):
                return int(ignored[i + 1])
    return None


def plan(argv):
    """(ranks on this node, launcher options, script, script arguments, runtime flags that were dropped)."""
    rest, ignored = split_runtime_flags(list(argv))
    p = argparse.ArgumentParser(prog="flexflow-python", description=__doc__.split("\n")[0], allow_abbrev=False)
    p.add_argument("--nodes", type=int, default=1, help="machines in the job")
    p.add_argument("--node-rank", type=int, default=0)
    p.add_argument("--master-addr", default="127.0.0.1")
    p.add_argument("--master-port", type=int, default=29500)
    p.add_argument("script", help="the training script")
    opts, script_args = p.parse_known_args(rest)
    ranks = _gpus_requested(ignored)
    if ranks is None:
        try:
            import torch
            ranks = max(torch.cuda.device_count(), 1)
        except ImportError:
            ranks = 1
    if ranks < 1:
        raise SystemExit("-ll:gpu wants a positive number of GPUs")
    dropped = [t for t in ignored if not t.startswith("-ll:gpu")]
    if _gpus_requested(ignored) is not None and "=" not in next(t for t in ignored if t.startswith("-ll:gpu")):
        dropped.remove(str(_gpus_requested(ignored)))
    return ranks, opts, opts.script, script_args, dropped


def command(ranks, opts, script, script_args):
    """The torch.distributed.run command line for a job of several ranks."""
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes", str(opts.nodes), "--node-rank", str(opts.node_rank),
            "--nproc-per-node", str(ranks), "--master-addr", opts.master_addr, "--master-port", str(opts.master_port), script] + list(script_args)


def main(argv=None) -> int:
    ranks, opts, script, script_args, dropped = plan(sys.argv[1:] if argv is None else argv)
    if dropped:
        print(f"flexflow-python: runtime flags without a counterpart are ignored: {' '.join(dropped)}", file=sys.stderr)
    if not os.path.exists(script):
        raise SystemExit(f"flexflow-python: no such script: {script}")
    if ranks == 1 and opts.nodes == 1:
        sys.argv = [script] + list(script_args)
        runpy.run_path(script, run_name="__main__")
        return 0
    return subprocess.call(command(ranks, opts, script, script_args))


if __name__ == "__main__":
    sys.exit(main())
