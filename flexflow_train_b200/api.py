"""Public entry points: ``compile`` a model into a trainable object and drive it.

This is the new-design flow of the reference (docs/plantuml/figures/pytorch-tracing.puml):
model -> ComputationGraph -> optimize (strategy search) -> CompiledModel -> forward/backward/update,
with the reference's ``FFConfig`` search flags (lib/task-spec/include/task-spec/ff_config.dtg.toml).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, Optional, Union

import torch

from . import _ffcore as core
from .runtime.executor import ExecConfig, Executable, OptimizerConfig


from .config_schema import FFConfig  # noqa: E402  (the dataclass is generated from the one field table)


class CompiledModel:
    """A computation graph bound to a strategy and an executor."""

    def __init__(self, graph, executable: Executable, strategy=None, search_stats: Optional[dict] = None):
        self.graph = graph
        self.executable = executable
        self.strategy = strategy
        self.search_stats = search_stats or {}
        self._pinned: Dict[str, torch.Tensor] = {}
        self._loss_host = torch.zeros(1, dtype=torch.float32).pin_memory() if torch.cuda.is_available() else torch.zeros(1)
        self.h2d_bytes_last_step = 0
        self.d2h_bytes_last_step = 0

    # ---- training
    def train_step(self, inputs: Dict[str, torch.Tensor], labels: Optional[torch.Tensor] = None, return_loss: bool = True):
        """One optimisation step on a batch given as host (ideally pinned) or device tensors.
        Returns the mean loss as a Python float when ``return_loss`` (one device->host read)."""
        ex = self.executable
        h2d = 0
        for t in list(inputs.values()) + ([labels] if labels is not None else []):
            if t is not None and not t.is_cuda:
                h2d += t.numel() * t.element_size()
        self.h2d_bytes_last_step = h2d
        ex.train_step(inputs, labels)
        if not return_loss:
            self.d2h_bytes_last_step = 0
            return None
        mean = ex.loss_rows.mean(dtype=torch.float32).reshape(1)
        self._loss_host.copy_(mean, non_blocking=False)
        self.d2h_bytes_last_step = 4
        return float(self._loss_host[0])

    def forward(self, inputs: Dict[str, torch.Tensor]):
        return self.executable.infer(inputs)

    def fit(self, data_loader, epochs: int = 1, log_every: int = 0):
        """Legacy ``FFModel.fit`` loop (bindings/python/old/flexflow/core/flexflow_cffi.py:2058-2100)."""
        history = []
        for _ in range(epochs):
            for step, (inputs, labels) in enumerate(data_loader):
                loss = self.train_step(inputs, labels)
                history.append(loss)
                if log_every and step % log_every == 0:
                    print(f"step {step}: loss {loss:.4f}")
        return history

    def state_dict(self):
        return self.executable.state_dict()

    def load_state_dict(self, sd):
        self.executable.load_state_dict(sd)

    def export_strategy(self, path: str):
        with open(path, "w") as f:
            f.write(self.graph.to_v1_string(parallel=True, indent=1))


def _as_graph(model, model_config):
    if isinstance(model, str):
        return core.build_model(model, model_config)
    return model


def _search_estimator(model, model_config, cg, world: int, config: "FFConfig", dist, exec_cfg):
    """The cost estimator the strategy search runs on: analytic, or filled with measured operator costs when the config
    asks for them (local_cost_estimator.cc:84-179 measures per query; here one profiled step per candidate shard size
    fills the table up front).  Returns (estimator or None, info for the search statistics)."""
    if not (config.measure_costs or config.cost_table_file or config.cost_params_file):
        return None, None
    import json
    import os

    from .compiler.strategy import machine_for
    from .runtime import cost_measure
    params = None
    if config.cost_params_file:
        # overrides of the analytic model's constants, merged over the defaults
        with open(config.cost_params_file) as f:
            overrides = json.load(f)
        params = core.CostEstimator(machine_for(world)).params()
        table = dict(params.get("measured_gbs", {}))
        table.update(overrides.pop("measured_gbs", {}))
        params.update(overrides)
        params["measured_gbs"] = table
    est = core.CostEstimator(machine_for(world), params)
    if not (config.measure_costs or config.cost_table_file):
        return est, {"source": "analytic", "cost_params": config.cost_params_file, "entries": 0}
    path = config.cost_table_file
    if path and os.path.exists(path):
        return est, {"source": path, "entries": cost_measure.load_table(est, path)}
    if not (config.measure_costs and torch.cuda.is_available() and exec_cfg.device != "cpu"):
        return est, {"source": "analytic", "entries": 0}
    table = None
    rank = dist.rank if dist is not None else 0
    if rank == 0:
        table = {}
        graphs = [(1, cg)]
        if isinstance(model, str):
            # the zoo rebuilds the same model at the per-device batch of every data-parallel degree of this machine
            base = dict(model_config or {})
            full = int(cg.shape(_first_input(cg)).sizes[0])
            for d in range(2, world + 1):
                if world % d == 0 and full % d == 0:
                    graphs.append((d, core.build_model(model, dict(base, batch_size=full // d))))
        for d, g in graphs:
            import dataclasses
            ex = Executable(g, dataclasses.replace(exec_cfg, use_cuda_graph=False))
            from .bin.run_model import synthetic_batch   # late: that module imports this one
            inputs, labels = synthetic_batch(g, ex, exec_cfg.loss, seed=config.seed, pinned=False)
            ex.set_inputs(inputs, labels)
            ex.profile_step()                    # warm-up: first-use allocations and kernel loading
            table.update(cost_measure.measure_into(est, ex, steps=2))
            del ex
            torch.cuda.empty_cache()
    if dist is not None and dist.world_size > 1:
        import torch.distributed as td
        box = [table]
        td.broadcast_object_list(box, src=0, group=dist.group)
        table = box[0]
        if rank != 0:
            for k, v in table.items():
                est.set_measured(k, v["fwd_ms"], v["bwd_ms"], v.get("memory_bytes", 0.0))
    if path and rank == 0:
        cost_measure.save_table(table, path)
    return est, {"source": "measured", "entries": len(table)}


def _first_input(g):
    for n in g.nodes():
        if n["type"] == "INPUT":
            return (n["id"], "OUTPUT")
    raise ValueError("the graph has no input")


def compile(model: Union[str, "core.Graph"], model_config: Optional[dict] = None, *, config: Optional[FFConfig] = None,
            optimizer: Optional[OptimizerConfig] = None, loss: Optional[str] = "sparse_categorical_crossentropy",
            dist=None, training: bool = True, device: str = "cuda") -> CompiledModel:
    """Build (or take) a computation graph, choose a parallelisation strategy and lower it to an executor.

    With one device the graph runs as is.  With a ``dist`` context the strategy comes from the
    search (``config.search_algorithm``) or from ``config.import_strategy_file``.
    """
    config = config or FFConfig()
    cg = _as_graph(model, model_config)
    exec_cfg = ExecConfig(compute_dtype=config.compute_dtype, loss=loss,
                          optimizer=optimizer or OptimizerConfig(kind="sgd", lr=config.learning_rate),
                          seed=config.seed, use_cuda_graph=config.use_cuda_graph, device=device, training=training,
                          profile_layers=config.enable_profiling)
    world = dist.world_size if dist is not None else 1
    strategy, stats = cg, {}
    if world > 1:
        from .compiler.strategy import choose_strategy
        estimator, cost_info = _search_estimator(model, model_config, cg, world, config, dist, exec_cfg)
        strategy, stats = choose_strategy(cg, world, config, estimator=estimator)
        if cost_info:
            stats["measured_costs"] = cost_info
        from .parallel.dist_executor import DistExecutable
        template = stats.pop("_template_strategy", None)
        try:
            ex = DistExecutable(strategy, exec_cfg, dist, fuse_collectives=config.fuse_collectives, shard_inputs=config.shard_inputs)
        except (NotImplementedError, ValueError, KeyError) as e:
            # a strategy the search composed from substitutions may use a placement the executor has no lowering for: every
            # rank sees the same exception at the same point (lowering is deterministic and happens before any collective),
            # so all of them fall back to the best hand-built template together
            if template is None:
                raise
            stats["strategy_fallback"] = f"{type(e).__name__}: {e}"
            strategy = template
            ex = DistExecutable(strategy, exec_cfg, dist, fuse_collectives=config.fuse_collectives, shard_inputs=config.shard_inputs)
    else:
        if config.import_strategy_file:
            with open(config.import_strategy_file) as f:
                strategy = core.Graph.from_v1(f.read())
        if device == "cpu":
            # reference-semantics execution on the host (fp32, torch autograd): for machines without a GPU and for
            # checking a model before it goes to one
            from .runtime.cpu_executor import CpuExecutable
            exec_cfg.compute_dtype = "fp32"
            ex = CpuExecutable(strategy, exec_cfg)
        else:
            ex = Executable(strategy, exec_cfg)
    cm = CompiledModel(cg, ex, strategy, stats)
    if config.export_strategy_file and (dist is None or dist.rank == 0):
        with open(config.export_strategy_file, "w") as f:
            f.write(strategy.to_v1_string(parallel=True, indent=1))
    if config.export_strategy_computation_graph_file and (dist is None or dist.rank == 0):
        # the chosen parallel computation graph as a dot file (the reference's --export-strategy-computation-graph-file)
        with open(config.export_strategy_computation_graph_file, "w") as f:
            f.write(strategy.as_dot())
    return cm
