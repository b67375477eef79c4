"""search-model: compile a model-zoo model and search a parallelisation strategy for a simulated machine, on the CPU.

    python -m flexflow_train_b200.bin.search_model --model transformer --heads 16 --gpus 8 --seed 0 \\
        --algorithm unity --budget 8 --out strategy.json

The computation graph is built, turned into a parallel computation graph, and a strategy is searched for
``--nodes`` x ``--gpus`` simulated devices with the analytical cost model: the Unity search
(lib/compiler/src/compiler/unity_algorithm/unity_algorithm.cc:51-146) starting from the unparallelised graph, or the
MCMC search (lib/compiler/src/compiler/mcmc/mcmc_over_mapped_pcg.cc:18-66).  The chosen mapped parallel computation
graph is written in the v1 file format and its estimated step time is printed; ``--cpu-step`` then runs one forward /
backward / update step of the (unparallelised) model on the host with random-init weights and synthetic token ids, as a
check that the graph that was searched is a graph that trains.  Prints one JSON object.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch

from .. import _ffcore as core
from .. import api
from ..compiler.strategy import machine_for, optimize
from ..runtime.executor import OptimizerConfig
from .run_model import REGRESSION_MODELS, synthetic_batch


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="search-model", description=__doc__.split("\n")[0])
    p.add_argument("--model", default="transformer", choices=sorted(core.model_names()))
    p.add_argument("--model-config", help="JSON object overriding fields of the model's default config")
    p.add_argument("--heads", type=int, default=None, help="shorthand for num_heads in the model config")
    p.add_argument("--gpus", type=int, default=8, help="simulated GPUs per node")
    p.add_argument("--nodes", type=int, default=1)
    p.add_argument("--algorithm", choices=["unity", "mcmc", "data_parallel", "tensor_parallel"], default="unity")
    p.add_argument("--budget", type=int, default=8, help="Unity: iterations; MCMC: ignored (see --mcmc-iterations)")
    p.add_argument("--alpha", type=float, default=1.05)
    p.add_argument("--time-limit", type=float, default=120.0, help="seconds the Unity search may take")
    p.add_argument("--start", choices=["serial", "best_template"], default="serial")
    p.add_argument("--mcmc-iterations", type=int, default=200)
    p.add_argument("--mcmc-temperature", type=float, default=0.02, help="as a fraction of the starting cost")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--out", default=None, help="where to write the strategy (v1 JSON of the mapped parallel computation graph)")
    p.add_argument("--cpu-step", action="store_true", help="also run one training step of the model on the host")
    p.add_argument("--init-std", type=float, default=0.02)
    a = p.parse_args(argv)

    mcfg = json.loads(a.model_config) if a.model_config else {}
    if a.heads:
        mcfg["num_heads"] = a.heads
    cg = core.build_model(a.model, mcfg)
    world = a.gpus * a.nodes
    machine = machine_for(world) if a.nodes == 1 else core.MachineSpecification(a.nodes, a.gpus, 1, 25.0, 770.0)
    t0 = time.time()
    r = optimize(cg, machine, world=world, algorithm=a.algorithm, budget=a.budget, alpha=a.alpha, seed=a.seed,
                 time_limit_s=a.time_limit, start=a.start, mcmc_iterations=a.mcmc_iterations, mcmc_temperature=a.mcmc_temperature)
    out = {"model": a.model, "operators": len(cg), "devices": world, "algorithm": a.algorithm, "seed": a.seed,
           "estimated_step_ms": r["runtime_ms"], "estimated_memory_bytes_per_device": r["memory_bytes"],
           "strategy_operators": len(r["mapped_pcg"]), "search_seconds": round(time.time() - t0, 3), "search": r["stats"]}
    if a.out:
        with open(a.out, "w") as f:
            f.write(r["mapped_pcg"].to_v1_string(parallel=True, indent=1))
        out["strategy_file"] = a.out
    if a.cpu_step:
        loss = "mean_squared_error_avg_reduce" if a.model in REGRESSION_MODELS else "sparse_categorical_crossentropy"
        cm = api.compile(cg, None, config=api.FFConfig(seed=a.seed, compute_dtype="fp32"), optimizer=OptimizerConfig(kind="sgd", lr=0.01),
                         loss=loss, device="cpu")
        ex = cm.executable
        if a.init_std > 0:  # weight matrices and tables drawn N(0, init_std); norm scales and biases keep their defaults
            gen = torch.Generator().manual_seed(a.seed)
            with torch.no_grad():
                for name, t in ex.oracle.params.items():
                    if t.dim() >= 2:
                        t.normal_(0.0, a.init_std, generator=gen)
        inputs, labels = synthetic_batch(cm.graph, ex, loss, seed=a.seed, pinned=False)
        t1 = time.time()
        first = cm.train_step(inputs, labels)
        second = cm.train_step(inputs, labels)
        out["cpu_step"] = {"loss": first, "loss_after_one_update": second, "seconds_per_step": round((time.time() - t1) / 2, 3)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
