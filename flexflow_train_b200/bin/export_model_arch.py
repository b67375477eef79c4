"""export-model-arch: export a model-zoo computation graph as JSON (v1 file format) or DOT, optionally with
the series-parallel decomposition of the graph.

    python -m flexflow_train_b200.bin.export_model_arch split_test
    python -m flexflow_train_b200.bin.export_model_arch --sp-decomposition split_test
    python -m flexflow_train_b200.bin.export_model_arch --dot --preprocessed-dot transformer

Counterpart of bin/export-model-arch (src/export-model-arch/export_model_arch.cc): same model names, the same
three switches, JSON with the keys ``computation_graph`` and, when asked, ``sp_decomposition``.
"""
from __future__ import annotations

import argparse
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


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="export-model-arch", description=__doc__.split("\n")[0])
    p.add_argument("model", choices=sorted(core.model_names()))
    p.add_argument("--sp-decomposition", action="store_true", help="also output a series-parallel decomposition of the graph")
    p.add_argument("--dot", action="store_true", help="output a DOT drawing instead of JSON")
    p.add_argument("--preprocessed-dot", action="store_true", help="DOT of the graph without inputs and weights")
    p.add_argument("--config", help="JSON object overriding fields of the model's default config")
    a = p.parse_args(argv)
    cfg = json.loads(a.config) if a.config else None
    sys.stdout.write(export(a.model, a.sp_decomposition, a.dot, a.preprocessed_dot, cfg) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
