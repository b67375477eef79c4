"""One table for the run configuration: the `FFConfig` dataclass, the command-line flags of the tools and the field
documentation are all generated from `FIELDS`, so a field is declared once (the role the reference gives its `.toml`
struct specifications and the dtgen generator, lib/runtime/include/runtime/config.h and the CLI flags of README.md:58-81)."""
from __future__ import annotations

import argparse
import dataclasses
from dataclasses import dataclass
from typing import Any, List, Optional, Sequence


@dataclass(frozen=True)
class Field:
    name: str
    type: Any
    default: Any
    help: str
    flag: Optional[str] = None        # command-line flag, None = not settable from the command line
    short: Optional[str] = None       # one-letter alias
    choices: Optional[Sequence[str]] = None
    negate: bool = False              # boolean given on the command line as the opposite switch (--no-cuda-graph)
    cli_default: Any = None           # default of the switch when it differs from the field's (opt-in switches)


FIELDS: List[Field] = [
    Field("epochs", int, 1, "passes over the data", "--epochs", "-e"),
    Field("batch_size", int, 64, "global batch size", "--batch-size", "-b"),
    Field("num_nodes", int, 1, "machines in the job"),
    Field("gpus_per_node", int, 0, "GPUs per machine; 0 = WORLD_SIZE / the visible devices"),
    Field("learning_rate", float, 0.01, "optimizer step size", "--learning-rate"),
    Field("weight_decay", float, 0.0001, "L2 penalty"),
    Field("workspace_size", int, 1 << 30, "scratch bytes an operator may ask for"),
    Field("enable_profiling", bool, False, "time every operator with CUDA events", "--profiling"),
    Field("search_budget", int, 0, "candidates the Unity search may expand on top of the scored templates; 0 = templates only", "--search-budget"),
    Field("search_alpha", float, 1.05, "Unity keeps candidates within this factor of the best cost", "--search-alpha"),
    Field("search_time_limit_s", float, 60.0, "wall-clock bound of the strategy search in seconds", "--search-time-limit"),
    Field("search_start", str, "best_template", "where the search starts: the cheapest template or the unparallelised graph", "--search-start",
          choices=("best_template", "serial")),
    Field("search_algorithm", str, "unity", "unity | mcmc | data_parallel | tensor_parallel | table_parallel | dp<a>xtp<b>", "--search-algorithm"),
    Field("only_data_parallel", bool, False, "restrict the search to data parallelism", "--only-data-parallel"),
    Field("enable_parameter_parallel", bool, True, "allow weight-sharding (tensor-parallel) rules", "--enable-parameter-parallel", cli_default=False),
    Field("enable_attribute_parallel", bool, True, "allow rules that shard non-sample activation dims", "--enable-attribute-parallel", cli_default=False),
    Field("score_hybrid_strategies", bool, False, "also report the estimates of data x tensor parallel meshes"),
    Field("substitution_json_path", Optional[str], None, "legacy rule collection to add to the generated rules", "--substitution-json"),
    Field("export_strategy_file", Optional[str], None, "write the chosen strategy (mapped PCG, v1 JSON) here", "--export-strategy"),
    Field("import_strategy_file", Optional[str], None, "run this strategy instead of searching", "--import-strategy"),
    Field("export_strategy_computation_graph_file", Optional[str], None, "write the chosen PCG as a dot drawing here"),
    Field("compute_dtype", str, "bf16", "dtype of activations and weight copies", "--compute-dtype", choices=("bf16", "fp32")),
    Field("use_cuda_graph", bool, True, "capture the training step into one CUDA graph", "--no-cuda-graph", negate=True),
    Field("fuse_collectives", bool, True, "collectives inside the neighbouring GEMMs / over peer memory (else NCCL)"),
    Field("shard_inputs", bool, True, "several ranks: an input cut over the sample dim may be fed as each rank's own piece"),
    Field("measure_costs", bool, False, "search on operator costs measured on this GPU (rank 0 measures, all ranks get the table)", "--measure-costs"),
    Field("cost_table_file", Optional[str], None, "measured operator costs: read when the file exists, written after measuring", "--cost-table"),
    Field("cost_params_file", Optional[str], None, "JSON overrides of the analytic cost model, e.g. the measured_gbs table that "
          "parallel.bench_fused --write-cost-params produces", "--cost-params"),
    Field("seed", int, 0, "seed of initializers, dropout and the search", "--seed"),
]

BY_NAME = {f.name: f for f in FIELDS}


def make_config_class():
    cls = dataclasses.make_dataclass(
        "FFConfig", [(f.name, f.type, dataclasses.field(default=f.default)) for f in FIELDS],
        namespace={"__doc__": "Run configuration; field names follow the reference's FFConfig / command-line flags.  Generated from "
                              "config_schema.FIELDS:\n\n" + "\n".join(f"    {f.name} ({getattr(f.type, '__name__', str(f.type))}, default {f.default!r}): {f.help}"
                                                                     for f in FIELDS)})
    cls.__module__ = __name__

    # the legacy FFConfig surface (bindings/python/old/flexflow/core/flexflow_cffi.py: parse_args, get_current_time,
    # begin_trace / end_trace, workers_per_node)
    def parse_args(self, argv=None):
        """Fills the fields that have a command-line flag from `argv` (default: sys.argv[1:]); unknown arguments and the
        Legion resource flags are left alone."""
        import sys
        parser = argparse.ArgumentParser(add_help=False, allow_abbrev=False)
        add_cli_arguments(parser)
        ns, _ = parser.parse_known_args(list(sys.argv[1:] if argv is None else argv))
        given = set()
        for tok in (sys.argv[1:] if argv is None else argv):
            for f in FIELDS:
                if tok in (f.flag, f.short) or (f.flag and tok.startswith(f.flag + "=")):
                    given.add(f.name)
        for name in given:
            setattr(self, name, getattr(ns, name))
        return self

    def get_current_time(self) -> float:
        """Microseconds on a monotonic clock, after the device has finished what was queued (the legacy call fenced the
        runtime the same way before reading the clock)."""
        import time
        try:
            import torch
            if torch.cuda.is_available():
                torch.cuda.synchronize()
        except ImportError:
            pass
        return time.perf_counter() * 1e6

    def begin_trace(self, trace_id: int) -> None:
        """Legion traces have no counterpart to switch on: a compiled model replays its step as one CUDA graph
        (`use_cuda_graph`).  Kept so that training scripts run unchanged."""

    def end_trace(self, trace_id: int) -> None:
        pass

    cls.parse_args = parse_args
    cls.get_current_time = get_current_time
    cls.begin_trace = begin_trace
    cls.end_trace = end_trace
    cls.workers_per_node = property(lambda self: self.gpus_per_node)
    return cls


FFConfig = make_config_class()


def add_cli_arguments(parser: argparse.ArgumentParser, skip: Sequence[str] = ()):
    """Adds one flag per field that has one; `skip` names fields the tool declares itself."""
    for f in FIELDS:
        if f.flag is None or f.name in skip:
            continue
        names = ([f.short] if f.short else []) + [f.flag]
        if f.type is bool:
            default = f.default if f.cli_default is None else f.cli_default
            if f.negate:
                parser.add_argument(*names, dest=f.name, action="store_false", default=True, help=f.help + " (this switch turns it off)")
            else:
                parser.add_argument(*names, dest=f.name, action="store_true", default=default, help=f.help)
        else:
            base = str if f.type == Optional[str] else f.type
            parser.add_argument(*names, dest=f.name, type=base, default=f.default, choices=f.choices, help=f"{f.help} (default {f.default!r})")


def config_from_args(ns: argparse.Namespace, **overrides):
    """An FFConfig from parsed arguments: every field with a flag is taken from `ns`, the rest keep their defaults."""
    kw = {f.name: getattr(ns, f.name) for f in FIELDS if f.flag is not None and hasattr(ns, f.name)}
    kw.update(overrides)
    return FFConfig(**kw)


def describe() -> str:
    """The fields as a Markdown table (used for the documentation of the tools)."""
    rows = ["| field | flag | default | meaning |", "|---|---|---|---|"]
    for f in FIELDS:
        rows.append(f"| `{f.name}` | {('`' + f.flag + '`') if f.flag else ''} | `{f.default!r}` | {f.help} |")
    return "\n".join(rows)
