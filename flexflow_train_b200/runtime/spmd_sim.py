"""Shard-by-shard evaluation of a parallel computation graph on the host.

Every tensor of the PCG is held as its pieces, keyed by (shard coordinate, sum replica, discard-copy replica); every
operator runs once per point of its task space on the pieces that ``operator_tensor_coord`` names.  The four parallel
operators move, copy and add pieces -- Repartition cuts a piece, Combine concatenates pieces, Replicate copies one,
Reduction sums sum-replicas -- so a strategy is executed the way its degrees say, not as the identity it denotes.
``assemble`` puts the pieces of a value back together (concatenate shards, add sum replicas, check that copies agree),
which must give what the unsharded computation graph computes.

Covers the operators that have a shard mapping: Input, Weight, Linear (with fused activation when the output is not
a partial sum), element-wise unary and binary operators, Softmax and LayerNorm over unsharded dims, and the parallel
operators -- enough for MLP-shaped graphs under data, tensor, and hybrid parallel strategies.  Forward only; a tool for
checking strategies and the degree algebra, not an executor (lib/op-attrs' parallel shape inference has no such
numerical check in the reference).
"""
from __future__ import annotations

import itertools
from typing import Dict, List, Tuple

import torch

from .. import _ffcore as core

Key = Tuple[Tuple[int, ...], int, int]

_UNARY = {
    "RELU": torch.relu, "SIGMOID": torch.sigmoid, "TANH": torch.tanh, "GELU": torch.nn.functional.gelu, "EXP": torch.exp,
    "IDENTITY": lambda t: t, "NOOP": lambda t: t, "DROPOUT": lambda t: t, "CAST": lambda t: t, "ELU": torch.nn.functional.elu,
    "RSQRT": torch.rsqrt, "SIN": torch.sin, "COS": torch.cos,
}
_BINARY = {"EW_ADD": torch.add, "EW_SUB": torch.sub, "EW_MUL": torch.mul, "EW_DIV": torch.div, "EW_MAX": torch.maximum,
           "EW_MIN": torch.minimum}
_ACT = {None: lambda t: t, "RELU": torch.relu, "SIGMOID": torch.sigmoid, "TANH": torch.tanh, "GELU": torch.nn.functional.gelu}


def _key(c: dict) -> Key:
    return (tuple(c["shard"]), int(c["sum"]), int(c["discard_copy"]))


def _slice(full: torch.Tensor, degrees, shard) -> torch.Tensor:
    t = full
    for d, (deg, idx) in enumerate(zip(degrees, shard)):
        n = t.shape[d] // deg
        t = t.narrow(d, idx * n, n)
    return t


def _tasks(graph, nid):
    full = core.operator_full_task_degrees(graph, nid)
    return full, itertools.product(*[range(d) for d in full])


class ShardedEvaluation:
    def __init__(self, pcg, parameters: Dict[str, torch.Tensor], inputs: Dict[str, torch.Tensor], dtype=torch.float64):
        self.g = pcg
        self.nodes = {n["id"]: n for n in pcg.nodes()}
        self.pieces: Dict[Tuple[int, str], Dict[Key, torch.Tensor]] = {}
        self.dtype = dtype
        for nid in pcg.topological_order():
            self._run(nid, parameters, inputs)

    # ---- helpers
    def _in(self, nid, task, slot):
        n = self.nodes[nid]
        src = dict((s, tuple(v)) for s, v in n["inputs"])[slot]
        k = _key(core.operator_tensor_coord(self.g, nid, list(task), slot, False))
        return self.pieces[src][k]

    def _out_key(self, nid, task, slot="OUTPUT") -> Key:
        return _key(core.operator_tensor_coord(self.g, nid, list(task), slot, True))

    def _run(self, nid, parameters, inputs):
        n = self.nodes[nid]
        t = n["type"]
        out: Dict[Key, torch.Tensor] = {}
        sh = n["outputs"][0][1]
        full, tasks = _tasks(self.g, nid)
        if t in ("INPUT", "WEIGHT"):
            src = (inputs if t == "INPUT" else parameters)[n["name"]]
            src = src.to(self.dtype) if src.is_floating_point() else src
            for task in tasks:
                k = self._out_key(nid, task)
                out[k] = _slice(src, sh.degrees, k[0]).clone()
        elif t in _UNARY or t in ("SCALAR_MULTIPLY", "SCALAR_ADD", "SCALAR_SUB", "SCALAR_TRUE_DIV", "POW", "SOFTMAX", "LAYERNORM"):
            for task in tasks:
                out[self._out_key(nid, task)] = self._rowwise(n, nid, task)
        elif t in _BINARY:
            for task in tasks:
                out[self._out_key(nid, task)] = _BINARY[t](self._in(nid, task, "LHS_INPUT"), self._in(nid, task, "RHS_INPUT"))
        elif t == "LINEAR":
            has_bias = any(s == "BIAS" for s, _ in n["inputs"])
            act = n["attrs"].get("activation")
            if act and sh.sum_degree > 1:
                raise ValueError("an activation cannot be applied to partial sums")
            for task in tasks:
                y = self._in(nid, task, "INPUT") @ self._in(nid, task, "WEIGHT").t()
                if has_bias and task[-2] == 0:  # the task with sum component 0 adds the bias
                    y = y + self._in(nid, task, "BIAS")
                out[self._out_key(nid, task)] = _ACT[act](y)
        elif t == "REPARTITION":
            dim, k = int(n["attrs"]["repartition_dim"]) % len(sh.sizes), int(n["attrs"]["repartition_degree"])
            for task in tasks:
                src = self._in(nid, task, "INPUT")
                m = src.shape[dim] // k
                out[self._out_key(nid, task)] = src.narrow(dim, (task[dim] % k) * m, m).clone()
        elif t == "COMBINE":
            dim, k = int(n["attrs"]["combine_dim"]) % len(sh.sizes), int(n["attrs"]["combine_degree"])
            parts: Dict[Key, List] = {}
            for task in tasks:  # the task grid is the input's: k consecutive input pieces make one output piece
                parts.setdefault(self._out_key(nid, task), [None] * k)[task[dim] % k] = self._in(nid, task, "INPUT")
            out = {key: torch.cat(ps, dim) for key, ps in parts.items()}
        elif t == "REPLICATE":
            for task in tasks:
                out[self._out_key(nid, task)] = self._in(nid, task, "INPUT").clone()
        elif t == "REDUCTION":
            for task in tasks:  # the task grid is the input's: sum replicas that share an output replica are added
                key = self._out_key(nid, task)
                x = self._in(nid, task, "INPUT")
                out[key] = x.clone() if key not in out else out[key] + x
        else:
            raise NotImplementedError(f"no shard-wise evaluation for {t}")
        for slot, _, _ in n["outputs"][:1]:
            self.pieces[(nid, slot)] = out

    def _rowwise(self, n, nid, task):
        t, a = n["type"], n["attrs"]
        x = self._in(nid, task, "INPUT")
        if t in _UNARY:
            return _UNARY[t](x)
        if t == "SOFTMAX":
            return torch.softmax(x, int(a.get("dim", -1)))
        if t == "LAYERNORM":
            axes = [int(v) for v in a["axes"]]
            y = torch.nn.functional.layer_norm(x, [x.shape[d] for d in axes], eps=float(a.get("eps", 1e-5)))
            if any(s == "GAMMA" for s, _ in n["inputs"]):
                y = y * self._in(nid, task, "GAMMA") + self._in(nid, task, "BETA")
            return y
        s = float(a.get("scalar", 0.0))
        return {"SCALAR_MULTIPLY": x * s, "SCALAR_ADD": x + s, "SCALAR_SUB": x - s, "SCALAR_TRUE_DIV": x / s if s else x,
                "POW": x ** s}[t]

    # ---- results
    def assemble(self, value: Tuple[int, str]) -> torch.Tensor:
        """The logical tensor of `value` from its pieces; replicas must agree, sum replicas are added."""
        sh = self.g.shape(value)
        pcs = self.pieces[value]
        total = None
        for s in range(sh.sum_degree):
            ref = None
            for c in range(sh.discard_copy_degree):
                full = torch.empty([int(v) for v in sh.sizes], dtype=next(iter(pcs.values())).dtype)
                for shard in itertools.product(*[range(d) for d in sh.degrees]):
                    _slice(full, sh.degrees, shard).copy_(pcs[(tuple(shard), s, c)])
                if ref is None:
                    ref = full
                elif not torch.allclose(ref, full, atol=1e-12):
                    raise AssertionError(f"discard-copy replicas of {value} disagree")
            total = ref if total is None else total + ref
        return total
