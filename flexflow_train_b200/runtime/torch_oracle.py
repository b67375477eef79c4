"""Reference interpreter: evaluates a computation graph with plain PyTorch ops and autograd.

Runs on CPU (or any torch device) in fp32 and defines the numerics every hand-written kernel and the
GPU executor are tested against; it is also the CPU execution path (one forward/backward step of a
searched strategy without a GPU).  Parallel operators are evaluated on the whole logical tensor, where
they are identities -- the strategy does not change what is computed.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from .initializers import initialize

_DT = {"FLOAT": torch.float32, "DOUBLE": torch.float64, "HALF": torch.float32, "BFLOAT16": torch.float32,
       "INT32": torch.int32, "INT64": torch.int64, "BOOL": torch.bool}
_ACT = {None: lambda x: x, "RELU": torch.relu, "GELU": F.gelu, "SIGMOID": torch.sigmoid, "TANH": torch.tanh}


class TorchOracle:
    def __init__(self, graph, *, loss: Optional[str] = "sparse_categorical_crossentropy", seed: int = 0,
                 device: str = "cpu", training: bool = True, dropout: bool = False, causal_attention: bool = False):
        self.graph = graph
        self.loss_kind = loss
        self.device = torch.device(device)
        self.training = training
        self.use_dropout = dropout
        self.causal = causal_attention
        self.nodes = {n["id"]: n for n in graph.nodes()}
        self.order = list(graph.topological_order())
        self.params: Dict[str, torch.Tensor] = {}
        self.param_of_node: Dict[int, torch.Tensor] = {}
        i = 0
        for nid in self.order:
            n = self.nodes[nid]
            if n["type"] == "WEIGHT":
                sh = n["outputs"][0][1]
                t = initialize(list(sh.sizes), n["attrs"].get("initializer"), base_seed=seed, ordinal=i).to(self.device)
                t.requires_grad_(training)
                self.params[n["name"] or f"weight{nid}"] = t
                self.param_of_node[nid] = t
                i += 1
        sinks = [tuple(v) for v in graph.sink_values() if self.nodes[v[0]]["type"] not in ("WEIGHT", "INPUT")]
        named = [v for v in sinks if self.nodes[v[0]]["name"] == "out_prob"]
        self.loss_value = (named or sinks)[-1] if sinks else None
        self.values = {}

    # ------------------------------------------------------------------ forward
    def forward(self, inputs: Dict[str, torch.Tensor]):
        vals = {}
        for nid in self.order:
            n = self.nodes[nid]
            t, a = n["type"], n["attrs"]
            ins = {s: vals[tuple(v)] for s, v in n["inputs"]}
            outs = self._eval(nid, n, t, a, ins, inputs)
            if not isinstance(outs, dict):
                outs = {"OUTPUT": outs}
            for s, v in outs.items():
                vals[(nid, s)] = v
        self.values = vals
        return vals[self.loss_value] if self.loss_value else None

    def _eval(self, nid, n, t, a, ins, inputs):
        if t == "INPUT":
            name = n["name"] or f"input{nid}"
            sh = n["outputs"][0][1]
            x = inputs[name].to(self.device)
            if _DT[sh.dtype].is_floating_point:
                x = x.to(_DT[sh.dtype])
            return x.reshape(list(sh.sizes))
        if t == "WEIGHT":
            return self.param_of_node[nid]
        if t in ("NOOP", "IDENTITY", "REPARTITION", "COMBINE", "REPLICATE", "REDUCTION"):
            return ins["INPUT"]
        if t == "LINEAR":
            y = F.linear(ins["INPUT"], ins["WEIGHT"], ins.get("BIAS"))
            return _ACT[a.get("activation")](y)
        if t == "BATCHMATMUL":
            return ins["LHS_INPUT"] @ ins["RHS_INPUT"]
        if t == "MULTIHEAD_ATTENTION":
            return self._attention(a, ins)
        if t == "LAYERNORM":
            x = ins["INPUT"]
            axes = sorted(int(v) for v in a["axes"])
            shape = [x.shape[i] for i in axes]
            g = ins["GAMMA"].reshape(shape) if "GAMMA" in ins else None
            b = ins["BETA"].reshape(shape) if "BETA" in ins else None
            return F.layer_norm(x, shape, g, b, float(a.get("eps", 1e-5)))
        if t == "BATCHNORM":
            x = ins["INPUT"]
            y = F.batch_norm(x, None, None, ins.get("GAMMA"), ins.get("BETA"), True, 0.1, float(a.get("eps", 1e-5)))
            return torch.relu(y) if a.get("relu") else y
        if t == "CONV2D":
            y = F.conv2d(ins["INPUT"], ins["FILTER"], ins.get("BIAS"), (int(a["stride_h"]), int(a["stride_w"])),
                         (int(a["padding_h"]), int(a["padding_w"])), 1, int(a.get("groups", 1)))
            return _ACT[a.get("activation")](y)
        if t == "POOL2D":
            k, s, p = (int(a["kernel_h"]), int(a["kernel_w"])), (int(a["stride_h"]), int(a["stride_w"])), \
                      (int(a["padding_h"]), int(a["padding_w"]))
            if a.get("pool_type", "MAX") == "MAX":
                y = F.max_pool2d(ins["INPUT"], k, s, p)
            else:
                y = F.avg_pool2d(ins["INPUT"], k, s, p, count_include_pad=False)
            return _ACT[a.get("activation")](y)
        if t == "EMBEDDING":
            idx = ins["INPUT"].long()
            e = ins["WEIGHT"][idx]  # [..., bag, dim]
            e = e.sum(-2) if a.get("aggr") != "AVG" else e.mean(-2)
            return e
        if t == "DROPOUT":
            if self.use_dropout and self.training:
                return F.dropout(ins["INPUT"], float(a["rate"]), True)
            return ins["INPUT"]
        if t == "SOFTMAX":
            return torch.softmax(ins["INPUT"], int(a.get("dim", -1)))
        if t == "CAST":
            dt = _DT[a["dtype"]]
            return ins["INPUT"].to(dt)
        if t == "CONCAT":
            return torch.cat([ins[f"INPUT_{i}"] for i in range(int(a["num_inputs"]))], int(a["axis"]))
        if t == "SPLIT":
            parts = torch.split(ins["INPUT"], [int(s) for s in a["splits"]], int(a["axis"]))
            return {f"OUTPUT_{i}": p for i, p in enumerate(parts)}
        if t == "FLAT":
            return torch.flatten(ins["INPUT"], int(a.get("start_dim", 1)), int(a.get("end_dim", -1)))
        if t == "RESHAPE":
            return ins["INPUT"].reshape([int(s) for s in a["shape"]["dims"]["ff_ordered"]])
        if t == "TRANSPOSE":
            return ins["INPUT"].permute([int(p) for p in a["permutation"]])
        if t == "REVERSE":
            return torch.flip(ins["INPUT"], [int(a["axis"])])
        if t == "GATHER":
            return torch.gather(ins["INPUT"], int(a["dim"]), ins["INDEX"].long())
        if t == "TOPK":
            v, i = torch.topk(ins["INPUT"], int(a["k"]), -1, True, bool(a.get("sorted", True)))
            return {"OUTPUT": v, "INDEX": i.to(torch.int32)}
        if t == "BROADCAST":
            tgt = a["target_dims"]["ff_ordered"] if isinstance(a["target_dims"], dict) else a["target_dims"]
            return ins["INPUT"].expand([int(s) for s in tgt])
        if t in ("REDUCE_SUM", "REDUCE_MEAN", "MEAN", "REDUCE_MAX", "REDUCE_MIN", "REDUCE_PROD"):
            axes = [int(v) for v in a["axes"]]
            keep = bool(a.get("keepdims", False))
            x = ins["INPUT"]
            if t == "REDUCE_SUM":
                return x.sum(axes, keep)
            if t in ("REDUCE_MEAN", "MEAN"):
                return x.mean(axes, keep)
            if t == "REDUCE_MAX":
                return x.amax(axes, keep)
            if t == "REDUCE_MIN":
                return x.amin(axes, keep)
            for ax in sorted(axes, reverse=True):
                x = x.prod(ax, keep)
            return x
        unary = {"RELU": torch.relu, "SIGMOID": torch.sigmoid, "TANH": torch.tanh, "ELU": F.elu, "GELU": F.gelu,
                 "EXP": torch.exp, "RSQRT": torch.rsqrt, "SIN": torch.sin, "COS": torch.cos, "LOG": torch.log,
                 "SQRT": torch.sqrt}
        if t in unary:
            return unary[t](ins["INPUT"])
        s = a.get("scalar")
        if t == "SCALAR_MULTIPLY":
            return ins["INPUT"] * s
        if t == "SCALAR_ADD":
            return ins["INPUT"] + s
        if t == "SCALAR_SUB":
            return ins["INPUT"] - s
        if t == "SCALAR_TRUE_DIV":
            return ins["INPUT"] / s
        if t == "POW":
            return ins["INPUT"] ** s
        binary = {"EW_ADD": torch.add, "EW_SUB": torch.sub, "EW_MUL": torch.mul, "EW_DIV": torch.div,
                  "EW_MAX": torch.maximum, "EW_MIN": torch.minimum}
        if t in binary:
            return binary[t](ins["LHS_INPUT"], ins["RHS_INPUT"])
        raise NotImplementedError(f"oracle: operator {t}")

    def _attention(self, a, ins):
        q, k, v = ins["QUERY"], ins["KEY"], ins["VALUE"]
        H, kd, vd, E = int(a["num_heads"]), int(a["kdim"]), int(a["vdim"]), int(a["embed_dim"])
        dq, dk, dv = q.shape[-1], k.shape[-1], v.shape[-1]
        w = ins["WEIGHT"].reshape(-1)
        o = 0
        wq = w[o:o + H * kd * dq].view(H * kd, dq); o += H * kd * dq
        wk = w[o:o + H * kd * dk].view(H * kd, dk); o += H * kd * dk
        wv = w[o:o + H * vd * dv].view(H * vd, dv); o += H * vd * dv
        wo = w[o:o + E * H * vd].view(E, H * vd)
        B, Sq, Sk = q.shape[0], q.shape[1], k.shape[1]
        bi = ins.get("INPUT_BIAS")
        bq = bi[:H * kd] if bi is not None else None
        bk = bi[H * kd:2 * H * kd] if bi is not None else None
        bv = bi[2 * H * kd:] if bi is not None else None
        Q = F.linear(q, wq, bq).view(B, Sq, H, kd).transpose(1, 2)
        Kt = F.linear(k, wk, bk).view(B, Sk, H, kd).transpose(1, 2)
        Vt = F.linear(v, wv, bv).view(B, Sk, H, vd).transpose(1, 2)
        if getattr(self, "use_sdpa", False):  # library attention kernel (used by the PyTorch baseline arm of the bench)
            pdrop = float(a.get("dropout", 0)) if (self.use_dropout and self.training) else 0.0
            ctx = F.scaled_dot_product_attention(Q, Kt, Vt, dropout_p=pdrop, is_causal=self.causal)
            return F.linear(ctx.transpose(1, 2).reshape(B, Sq, H * vd), wo, ins.get("OUTPUT_BIAS"))
        s = (Q @ Kt.transpose(-1, -2)) / math.sqrt(kd)
        if self.causal:
            mask = torch.tril(torch.ones(Sq, Sk, dtype=torch.bool, device=s.device))
            s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, -1)
        if self.use_dropout and self.training and float(a.get("dropout", 0)) > 0:
            p = F.dropout(p, float(a["dropout"]), True)
        ctx = (p @ Vt).transpose(1, 2).reshape(B, Sq, H * vd)
        return F.linear(ctx, wo, ins.get("OUTPUT_BIAS"))

    # ------------------------------------------------------------------ loss / step
    def loss(self, pred, labels):
        kind = self.loss_kind
        cols = pred.shape[-1]
        p2 = pred.reshape(-1, cols)
        if kind == "sparse_categorical_crossentropy":
            lab = labels.reshape(-1).long().to(p2.device)
            return -torch.log(p2.gather(1, lab[:, None]).clamp_min(1e-30)).squeeze(1)
        t = labels.reshape(-1, cols).to(p2)
        if kind == "categorical_crossentropy":
            return -(t * torch.log(p2.clamp_min(1e-30))).sum(1)
        if kind in ("mean_squared_error_avg_reduce", "mean_squared_error_sum_reduce"):
            return ((p2 - t) ** 2).sum(1)
        if kind == "identity":
            return p2.sum(1)
        raise ValueError(kind)

    def loss_and_grads(self, inputs, labels):
        for p in self.params.values():
            p.grad = None
        pred = self.forward(inputs)
        rows = self.loss(pred, labels)
        rows.mean().backward()
        return rows.detach(), {k: p.grad for k, p in self.params.items()}
