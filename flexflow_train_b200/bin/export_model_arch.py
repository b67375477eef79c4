"""export-model-arch: export a model-zoo computation graph as JSON (v1 file format) or DOT, optionally with
the series-parallel decomposition of the graph.

    python -m flexflow_train_b200.bin.export_model_arch split_test
    python -m flexflow_train_b200.bin.export_model_arch --sp-decomposition split_test
    python -m flexflow_train_b200.bin.export_model_arch --dot --preprocessed-dot transformer

Counterpart of bin/export-model-arch (src/export-model-arch/export_model_arch.cc): same model names, the same
three switches, JSON with the keys ``computation_graph`` and, when asked, ``sp_decomposition``.
"""
from __future__ import annotations

import json
import sys

from .. import _ffcore as core


def export(model: str, sp_decomposition: bool = False, dot: bool = False, preprocessed_dot: bool = False, config=None) -> str:
    g = core.build_model(model, config or {})
    if dot or preprocessed_dot:
        if preprocessed_dot:
            # the preprocessed form drops weights and inputs: the operator skeleton the SP decomposition works on
            keep = {n["id"]: n for n in g.nodes() if n["type"] not in ("WEIGHT", "INPUT")}
            lines = ["digraph preprocessed {", "  node [shape=box, fontsize=10];"]
            for i, n in keep.items():
                lines.append(f'  n{i} [label="{n["name"] or n["type"]}\\n{n["type"]}"];')
            for i, n in keep.items():
                for _, (src, _slot) in n["inputs"]:
                    if src in keep:
                        lines.append(f"  n{src} -> n{i};")
            return "\n".join(lines + ["}"])
        return g.as_dot()
    out = {"computation_graph": g.to_v1()}
    if sp_decomposition:
        tree, exact = core.get_graph_sp_decomposition(g)
        if tree is None:
            raise SystemExit(f"the computation graph of {model} has no series-parallel decomposition")
        out["sp_decomposition"] = core.sp_to_json(core.sp_left_associative_binary(tree))
        if not exact:  # the graph itself is not series-parallel: the tree comes from SP-ization
            out["sp_decomposition_is_exact"] = False
    return json.dumps(out, indent=2)


def cli_spec():
    """The tool's command line as a declarative spec of the native core (flags are switches, positionals may carry a set of
    choices), the form the reference declares its tools in (lib/utils/include/utils/cli/cli_spec.h,
    bin/export-model-arch/src/export-model-arch/export_model_arch.cc main)."""
    d = core.dataflow
    spec = d.empty_cli_spec()
    keys = {
        "help": d.cli_add_help_flag(spec),
        "sp_decomposition": d.cli_add_flag(spec, "sp-decomposition", None, "also output a series-parallel decomposition of the graph"),
        "dot": d.cli_add_flag(spec, "dot", None, "output a DOT drawing instead of JSON"),
        "preprocessed_dot": d.cli_add_flag(spec, "preprocessed-dot", None, "DOT of the graph without inputs and weights"),
        "model": d.cli_add_positional_argument(spec, "model", sorted(core.model_names()), "name of the model to export"),
    }
    return spec, keys


def main(argv=None) -> int:
    d = core.dataflow
    argv = list(sys.argv[1:] if argv is None else argv)
    cfg = None
    if "--config" in argv:  # the one valued option: a JSON object overriding fields of the model's default config
        i = argv.index("--config")
        if i + 1 >= len(argv):
            sys.stderr.write("error: --config needs a JSON object\n")
            return 2
        cfg = json.loads(argv[i + 1])
        del argv[i:i + 2]
    spec, keys = cli_spec()
    try:
        r = d.cli_parse(spec, ["export-model-arch"] + argv)
    except ValueError as e:
        sys.stderr.write(f"error: {e}\n\n{d.cli_get_help_message('export-model-arch', spec)}")
        return 2
    if d.cli_get_flag(r, keys["help"]):
        sys.stdout.write(d.cli_get_help_message("export-model-arch", spec))
        return 0
    sys.stdout.write(export(d.cli_get_argument(r, keys["model"]), d.cli_get_flag(r, keys["sp_decomposition"]),
                            d.cli_get_flag(r, keys["dot"]), d.cli_get_flag(r, keys["preprocessed_dot"]), cfg) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
