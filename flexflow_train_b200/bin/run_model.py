"""run-model: train a model-zoo model on synthetic data, on one GPU or (under torchrun) one rank per GPU.

    python -m flexflow_train_b200.bin.run_model --model transformer -b 64 -e 1 --iterations 20
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \\
        -m flexflow_train_b200.bin.run_model --model bert --search-budget 10 --export-strategy strategy.json

Counterpart of bin/run-model (src/run-model/run_model.cc) with the reference's command line flags
(README.md:58-81): ``-e`` epochs, ``-b`` batch size, ``-p`` print frequency, ``--search-budget``,
``--search-alpha``, ``--export-strategy``, ``--import-strategy``, ``--only-data-parallel``,
``--enable-parameter-parallel``, ``--enable-attribute-parallel``.  Legion/Realm resource flags (``-ll:gpu``,
``-ll:fsize``, ``-ll:zsize``, ``-ll:cpu``, ``-ll:util``, ``-ll:bgwork``) are accepted and ignored with a note:
there is one process per GPU and memory is managed by the executor.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

from .. import _ffcore as core
from .. import api
from .. import config_schema as schema
from ..runtime.executor import OptimizerConfig
from ..utils import checkpoint as ckpt
from ..utils.metrics import StepLogger

REGRESSION_MODELS = {"dlrm", "candle_uno"}


def synthetic_batch(graph, executable, loss: str, seed: int = 0, pinned: bool = True):
    """Random inputs and labels with the shapes and dtypes the graph's INPUT nodes declare."""
    gen = torch.Generator().manual_seed(seed)
    inputs = {}
    nodes = graph.nodes()
    for n in nodes:
        if n["type"] != "INPUT":
            continue
        sh = n["outputs"][0][1]
        sizes = [int(s) for s in sh.sizes]
        name = n["name"] or f"input{n['id']}"
        if sh.dtype in ("INT32", "INT64"):
            hi = 2
            for c in nodes:
                if c["type"] == "EMBEDDING" and any(tuple(v) == (n["id"], "OUTPUT") for _, v in c["inputs"]):
                    hi = int(c["attrs"]["num_entries"])
            t = torch.randint(0, max(hi, 2), sizes, generator=gen, dtype=torch.int32 if sh.dtype == "INT32" else torch.int64)
        else:
            t = torch.randn(sizes, generator=gen)
        inputs[name] = t.pin_memory() if pinned and torch.cuda.is_available() else t
    lv = executable.loss_value
    # the loss value is a node of the executable's own (possibly parallel) graph; `sizes` are its global sizes
    lsizes = [int(s) for s in executable.graph.shape(lv).sizes] if lv is not None else [1, 1]
    rows = 1
    for s in lsizes[:-1]:
        rows *= s
    if loss == "sparse_categorical_crossentropy":
        labels = torch.randint(0, lsizes[-1], (rows,), generator=gen, dtype=torch.int32)
    else:
        labels = torch.rand(rows, lsizes[-1], generator=gen)
    return inputs, (labels.pin_memory() if pinned and torch.cuda.is_available() else labels)


def split_runtime_flags(argv):
    """Separates the Legion/Realm resource flags (``-ll:gpu 1``, ``-lg:prof 2`` ...) and their values from the rest
    of the command line, so that a flag's value can never be taken for a positional argument."""
    rest, ignored = [], []
    i = 0
    while i < len(argv):
        tok = argv[i]
        if tok.startswith("-ll:") or tok.startswith("-lg:"):
            ignored.append(tok)
            if "=" not in tok and i + 1 < len(argv) and not argv[i + 1].startswith("-"):
                ignored.append(argv[i + 1])
                i += 1
        else:
            rest.append(tok)
        i += 1
    return rest, ignored


def main(argv=None) -> int:
    argv, ignored = split_runtime_flags(list(sys.argv[1:] if argv is None else argv))
    p = argparse.ArgumentParser(prog="run-model", description=__doc__.split("\n")[0])
    p.add_argument("graph_json", nargs="?", help="a v1 JSON file (computation graph, parallel or mapped parallel computation graph) to "
                   "train instead of a model-zoo model: as the reference's run-model, 5 iterations of SGD(0.001, momentum 0.9) "
                   "unless --iterations / --optimizer / --learning-rate say otherwise")
    p.add_argument("--device", choices=["cuda", "cpu"], default=None, help="cpu: host executor (fp32); default: the GPU")
    p.add_argument("--model", default="transformer", choices=sorted(core.model_names()))
    p.add_argument("--model-config", help="JSON object overriding fields of the model's default config")
    p.add_argument("-p", "--print-freq", type=int, default=10)
    p.add_argument("-d", "--dataset", default=None, help="ignored: data is synthetic")
    p.add_argument("--iterations", type=int, default=None, help="steps per epoch (default 20; 5 for a graph file)")
    p.add_argument("--optimizer", choices=["sgd", "adam"], default=None, help="default adam; sgd with momentum 0.9 for a graph file")
    # every FFConfig field that has a flag (epochs, batch size, the search and strategy options, dtype, seed ...) comes from
    # the one field table
    schema.add_cli_arguments(p, skip=("batch_size", "enable_profiling", "learning_rate"))
    p.add_argument("-b", "--batch-size", type=int, default=None, help="global batch size (default: the model's own)")
    p.add_argument("--learning-rate", type=float, default=1e-3)
    p.add_argument("--profiling", action="store_true", help="print a per-operator time table after training")
    p.add_argument("--checkpoint-dir")
    p.add_argument("--checkpoint-every", type=int, default=0)
    p.add_argument("--resume", action="store_true")
    p.add_argument("--log-file")
    a = p.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dist_ctx = None
    if world > 1:
        import torch.distributed as dist

        from ..parallel.context import DistContext

        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist_ctx = DistContext(rank, world, local)
    if ignored and rank == 0:
        print(f"note: runtime resource flags {ignored} are not needed here and were ignored", file=sys.stderr)

    device = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    if a.iterations is None:
        a.iterations = 5 if a.graph_json else 20
    momentum = 0.9 if (a.graph_json and a.optimizer in (None, "sgd")) else 0.0
    if a.optimizer is None:
        a.optimizer = "sgd" if a.graph_json else "adam"
    sync = torch.cuda.synchronize if device == "cuda" else (lambda: None)
    mcfg = json.loads(a.model_config) if a.model_config else {}
    if a.batch_size:
        mcfg["batch_size"] = a.batch_size
    loss = "mean_squared_error_avg_reduce" if a.model in REGRESSION_MODELS else "sparse_categorical_crossentropy"
    cfg = schema.config_from_args(a, batch_size=mcfg.get("batch_size", 64), enable_profiling=False, learning_rate=a.learning_rate,
                                  search_algorithm="data_parallel" if a.only_data_parallel else a.search_algorithm)
    model = a.model
    if a.graph_json:
        with open(a.graph_json) as f:
            model = core.Graph.from_v1(f.read())
        parallel = any(core.is_parallel_op(n["type"]) for n in model.nodes())
        if parallel and world > 1:
            cfg.import_strategy_file = a.graph_json  # the file is the strategy
        loss = "sparse_categorical_crossentropy"
    cm = api.compile(model, mcfg, config=cfg, optimizer=OptimizerConfig(kind=a.optimizer, lr=a.learning_rate, momentum=momentum),
                     loss=loss, dist=dist_ctx, device=device)
    ex = cm.executable
    if a.resume and a.checkpoint_dir:
        last = ckpt.latest(a.checkpoint_dir)
        if last:
            meta = ckpt.load(last, ex, rank=rank)
            if rank == 0:
                print(f"resumed from {last} at step {meta['step']}")
    inputs, labels = synthetic_batch(cm.graph, ex, loss, seed=1234)
    logger = StepLogger(a.log_file, rank)
    if a.graph_json:
        batch = next((int(n["outputs"][0][1].sizes[0]) for n in cm.graph.nodes() if n["type"] == "INPUT"), 0)
    else:
        batch = mcfg.get("batch_size", core.default_model_config(a.model).get("batch_size", 0))
    step = ex.step_count
    for epoch in range(a.epochs):
        sync()
        t0 = time.perf_counter()
        for it in range(a.iterations):
            want_loss = a.print_freq > 0 and (it % a.print_freq == 0 or it == a.iterations - 1)
            loss_v = cm.train_step(inputs, labels, return_loss=want_loss)
            step += 1
            if want_loss and rank == 0:
                print(f"epoch {epoch} iter {it}: loss {loss_v:.4f}")
                logger.log(step, loss_v)
            if a.checkpoint_dir and a.checkpoint_every and step % a.checkpoint_every == 0:
                ckpt.save(a.checkpoint_dir, ex, step, rank=rank, world_size=world, strategy=cm.strategy,
                          barrier=(torch.distributed.barrier if world > 1 else None))
        sync()
        dt = time.perf_counter() - t0
        if rank == 0:
            print(f"epoch {epoch}: {a.iterations} iterations in {dt:.3f} s, {a.iterations * batch / dt:.1f} samples/s "
                  f"(host wall clock, includes H2D copies and loss reads)")
    if a.profiling and world > 1 and rank == 0:
        print("note: --profiling times one rank's operators in isolation and is skipped with more than one rank", file=sys.stderr)
    if a.profiling and world == 1 and device == "cuda":
        prof = ex.profile_step()
        for (typ, phase), ms in sorted(prof["by_type"].items(), key=lambda kv: -kv[1])[:20]:
            print(f"  {typ:24s} {phase:4s} {ms:9.3f} ms")
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
