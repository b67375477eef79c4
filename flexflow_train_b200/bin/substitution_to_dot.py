"""substitution-to-dot: draw one rule of a legacy substitution file (or of the built-in rule set) as DOT.

    python -m flexflow_train_b200.bin.substitution_to_dot rules.json taso_rule_12
    python -m flexflow_train_b200.bin.substitution_to_dot --builtin partition_linear_combine

Counterpart of bin/substitution-to-dot (src/substitution-to-dot.cc): pattern and replacement graphs as two
clusters with the output mapping drawn between them.
"""
from __future__ import annotations

import argparse
import json
import sys

from .. import _ffcore as core


def legacy_rule_dot(path: str, rule_name: str) -> str:
    with open(path) as f:
        coll = json.load(f)
    for i, r in enumerate(coll["rule"]):
        if r.get("name", f"taso_rule_{i}") == rule_name:
            return core.legacy_rule_as_dot(r)
    raise SystemExit(f"no rule named {rule_name} in {path} ({len(coll['rule'])} rules)")


def builtin_rule_dot(name: str, degree: int = 2) -> str:
    rules = core.get_substitution_set(core.MachineSpecification(1, degree))
    for r in rules:
        if r.name == name or r.name.startswith(name):
            return r.as_dot()
    raise SystemExit(f"no built-in rule named {name}; have e.g. {[r.name for r in rules[:8]]}")


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="substitution-to-dot", description=__doc__.split("\n")[0])
    p.add_argument("file_or_name", help="legacy JSON rule file, or a built-in rule name with --builtin")
    p.add_argument("rule", nargs="?", help="rule name inside the file (taso_rule_<n>)")
    p.add_argument("--builtin", action="store_true")
    p.add_argument("--degree", type=int, default=2)
    a = p.parse_args(argv)
    if a.builtin:
        sys.stdout.write(builtin_rule_dot(a.file_or_name, a.degree) + "\n")
    else:
        if not a.rule:
            p.error("a rule name is required with a rule file")
        sys.stdout.write(legacy_rule_dot(a.file_or_name, a.rule) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
