"""PyTorch importer: ``torch.fx`` trace -> text IR -> ``FFModel`` layer calls.

Covers the node classes of the legacy importer (bindings/python/old/flexflow/torch/model.py:870-936 dispatch
table; text IR :2539-2604; HuggingFace tracing :2428-2446).  The import has two stages so that a model can be
exported on a machine with PyTorch and built elsewhere:

  1. ``PyTorchModel.to_ir()``    fx graph -> list of records ``{"name", "op", "inputs", "params"}``
     (``torch_to_file`` writes them one JSON object per line)
  2. ``emit_ir(records, ffmodel, input_tensors)``  records -> layer calls (``file_to_ff`` reads a file first)

``torch_to_ff`` does both.  After ``ffmodel.compile`` the PyTorch parameters can be copied into the executor
with ``copy_parameters`` so both frameworks start from the same weights.
"""
from __future__ import annotations

import json
import operator
from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .ffmodel import FFModel, Tensor
from .types import ActiMode, AggrMode, DataType, PoolType

_T5_NAMES = ("T5LayerNorm", "LlamaRMSNorm", "RMSNorm")


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def _lit(a):
    """An fx argument as a JSON-able literal: nodes become {"node": name}."""
    import torch.fx as fx

    if isinstance(a, fx.Node):
        return {"node": a.name}
    if isinstance(a, (list, tuple)):
        return [_lit(x) for x in a]
    if isinstance(a, slice):
        return {"slice": [a.start, a.stop, a.step]}
    if isinstance(a, torch.dtype):
        return {"dtype": str(a).replace("torch.", "")}
    if isinstance(a, torch.Size):
        return [int(x) for x in a]
    if a is Ellipsis:
        return {"ellipsis": True}
    if isinstance(a, (int, float, bool, str)) or a is None:
        return a
    if isinstance(a, torch.device):
        return str(a)
    raise NotImplementedError(f"fx argument of type {type(a).__name__}")


def _module_record(name, mod, ins):
    """Record for a call_module node."""
    p: dict = {}
    if isinstance(mod, nn.Linear):
        op, p = "LINEAR", {"out_dim": mod.out_features, "use_bias": mod.bias is not None}
    elif isinstance(mod, nn.Conv2d):
        if mod.padding_mode != "zeros" or _pair(mod.dilation) != (1, 1) or isinstance(mod.padding, str):
            raise NotImplementedError("Conv2d with dilation / non-zero padding mode / string padding")
        k, s, pd = _pair(mod.kernel_size), _pair(mod.stride), _pair(mod.padding)
        op, p = "CONV2D", {"out_channels": mod.out_channels, "kernel": k, "stride": s, "padding": pd, "groups": mod.groups,
                           "use_bias": mod.bias is not None}
    elif isinstance(mod, (nn.MaxPool2d, nn.AvgPool2d)):
        k = _pair(mod.kernel_size)
        s = _pair(mod.stride if mod.stride is not None else mod.kernel_size)
        op, p = "POOL2D", {"kernel": k, "stride": s, "padding": _pair(mod.padding), "pool_type": "MAX" if isinstance(mod, nn.MaxPool2d) else "AVG"}
    elif isinstance(mod, (nn.AdaptiveAvgPool2d, nn.AdaptiveMaxPool2d)):
        op, p = "ADAPTIVE_POOL2D", {"output": _pair(mod.output_size), "pool_type": "AVG" if isinstance(mod, nn.AdaptiveAvgPool2d) else "MAX"}
    elif isinstance(mod, nn.BatchNorm2d):
        op, p = "BATCHNORM", {"eps": mod.eps, "affine": mod.affine}
    elif isinstance(mod, nn.LayerNorm):
        op, p = "LAYERNORM", {"ndims": len(mod.normalized_shape), "eps": mod.eps, "affine": mod.elementwise_affine}
    elif type(mod).__name__ in _T5_NAMES:
        op, p = "T5_LAYERNORM", {"eps": float(getattr(mod, "variance_epsilon", getattr(mod, "eps", 1e-6)))}
    elif isinstance(mod, nn.Softmax):
        op, p = "SOFTMAX", {"dim": -1 if mod.dim is None else mod.dim}
    elif isinstance(mod, nn.Dropout):
        op, p = "DROPOUT", {"rate": mod.p}
    elif isinstance(mod, nn.Flatten):
        op, p = "FLAT", {"start_dim": mod.start_dim, "end_dim": mod.end_dim}
    elif isinstance(mod, nn.Embedding):
        op, p = "EMBEDDING", {"num_embeddings": mod.num_embeddings, "embedding_dim": mod.embedding_dim}
    elif isinstance(mod, nn.Identity):
        op = "IDENTITY"
    elif isinstance(mod, (nn.ReLU, nn.GELU, nn.Sigmoid, nn.Tanh, nn.ELU)):
        op = type(mod).__name__.upper()
    else:
        raise NotImplementedError(f"torch module {type(mod).__name__} ({name}) has no importer")
    return {"name": name, "op": op, "inputs": ins, "params": p}


# python-level callables / method names -> IR op of the importer
_FUNCTIONS = {
    operator.add: "ADD", torch.add: "ADD", operator.sub: "SUB", torch.sub: "SUB", operator.mul: "MUL", torch.mul: "MUL",
    operator.truediv: "TRUEDIV", torch.true_divide: "TRUEDIV", torch.div: "TRUEDIV", operator.floordiv: "FLOORDIV",
    torch.floor_divide: "FLOORDIV", torch.cat: "CAT", torch.split: "SPLIT", torch.flatten: "FLATTEN", F.relu: "RELU", torch.relu: "RELU",
    operator.getitem: "GETITEM", torch.matmul: "MATMUL", torch.bmm: "MATMUL", operator.matmul: "MATMUL", getattr: "GETATTR",
    torch.transpose: "TRANSPOSE", torch.reshape: "RESHAPE", torch.permute: "PERMUTE", F.softmax: "SOFTMAX", torch.softmax: "SOFTMAX",
    torch.pow: "POW", operator.pow: "POW", torch.mean: "MEAN", torch.rsqrt: "RSQRT", torch.unsqueeze: "UNSQUEEZE",
    F.dropout: "DROPOUT", torch.tanh: "TANH", F.gelu: "GELU", torch.sigmoid: "SIGMOID", F.sigmoid: "SIGMOID", torch.exp: "EXP",
    torch.sin: "SIN", torch.cos: "COS", F.elu: "ELU", F.layer_norm: "F_LAYERNORM", torch.sum: "SUM", torch.squeeze: "SQUEEZE",
    F.linear: "F_LINEAR", torch._C._nn.linear: "F_LINEAR",
}
_METHODS = {
    "add": "ADD", "sub": "SUB", "mul": "MUL", "div": "TRUEDIV", "true_divide": "TRUEDIV", "floor_divide": "FLOORDIV", "split": "SPLIT",
    "flatten": "FLATTEN", "relu": "RELU", "matmul": "MATMUL", "bmm": "MATMUL", "transpose": "TRANSPOSE", "expand": "EXPAND",
    "reshape": "RESHAPE", "permute": "PERMUTE", "softmax": "SOFTMAX", "view": "VIEW", "to": "TO", "pow": "POW", "mean": "MEAN",
    "rsqrt": "RSQRT", "unsqueeze": "UNSQUEEZE", "float": "FLOAT", "type_as": "TYPE_AS", "contiguous": "CONTIGUOUS", "tanh": "TANH",
    "gelu": "GELU", "sigmoid": "SIGMOID", "size": "SIZE", "exp": "EXP", "sum": "SUM", "squeeze": "SQUEEZE", "clone": "CONTIGUOUS",
    "detach": "CONTIGUOUS", "half": "FLOAT", "bfloat16": "FLOAT", "dropout": "DROPOUT",
}


class PyTorchModel:
    def __init__(self, model: nn.Module, is_hf_model: bool = False, input_names: Optional[List[str]] = None, batch_size: int = 1,
                 seq_length=None):
        self.model = model
        self.is_hf_model = is_hf_model
        self.input_names = input_names
        self.batch_size = batch_size
        self.seq_length = seq_length
        self._traced = None

    # ---- stage 1
    def trace(self):
        if self._traced is None:
            hf_trace = None
            if self.is_hf_model:
                try:  # the HuggingFace tracer (concrete shapes for control flow) was removed from recent releases
                    from transformers.utils.fx import symbolic_trace as hf_trace
                except ImportError:
                    hf_trace = None
            if hf_trace is not None:
                self._traced = hf_trace(self.model, input_names=self.input_names)
            else:
                import torch.fx

                self._traced = torch.fx.symbolic_trace(self.model)
        return self._traced

    def to_ir(self) -> List[dict]:
        traced = self.trace()
        mods = dict(traced.named_modules())
        out = []
        for node in traced.graph.nodes:
            args = [_lit(a) for a in node.args]
            kwargs = {k: _lit(v) for k, v in node.kwargs.items()}
            if node.op == "placeholder":
                out.append({"name": node.name, "op": "INPUT", "inputs": [], "params": {}})
            elif node.op == "output":
                out.append({"name": node.name, "op": "OUTPUT", "inputs": args, "params": {}})
            elif node.op == "get_attr":
                t = traced
                for part in node.target.split("."):
                    t = getattr(t, part)
                out.append({"name": node.name, "op": "ATTRIBUTE", "inputs": [],
                            "params": {"target": node.target, "shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", "")}})
            elif node.op == "call_module":
                rec = _module_record(node.name, mods[node.target], args)
                rec["params"]["module"] = node.target
                out.append(rec)
            elif node.op == "call_function":
                if node.target not in _FUNCTIONS:
                    raise NotImplementedError(f"torch function {getattr(node.target, '__name__', node.target)} has no importer")
                out.append({"name": node.name, "op": _FUNCTIONS[node.target], "inputs": args, "params": kwargs})
            elif node.op == "call_method":
                if node.target not in _METHODS:
                    raise NotImplementedError(f"tensor method {node.target} has no importer")
                out.append({"name": node.name, "op": _METHODS[node.target], "inputs": args, "params": kwargs})
        return out

    def torch_to_file(self, filename: str):
        with open(filename, "w") as f:
            for rec in self.to_ir():
                f.write(json.dumps(rec) + "\n")

    # ---- stage 2
    def torch_to_ff(self, ffmodel: FFModel, input_tensors: List[Tensor], verbose: bool = False):
        return emit_ir(self.to_ir(), ffmodel, input_tensors, verbose=verbose)

    @staticmethod
    def file_to_ff(filename: str, ffmodel: FFModel, input_tensors: List[Tensor], verbose: bool = False):
        with open(filename) as f:
            records = [json.loads(line) for line in f if line.strip()]
        return emit_ir(records, ffmodel, input_tensors, verbose=verbose)

    # ---- weights
    def copy_parameters(self, ffmodel: FFModel) -> int:
        """Copy this module's parameters into the compiled executor (matched through the layer names the import
        gave: fx node name + slot).  Returns the number of tensors copied."""
        sd = dict(self.model.named_parameters())
        sd.update(dict(self.model.named_buffers()))
        wanted = {}
        for rec in self.to_ir():
            mod = rec["params"].get("module")
            if mod is None:
                continue
            base = rec["name"]
            for slot, key in (("weight", "weight"), ("filter", "weight"), ("bias", "bias"), ("gamma", "weight"), ("beta", "bias")):
                if f"{mod}.{key}" in sd:
                    wanted[f"{base}.{slot}"] = sd[f"{mod}.{key}"]
        n = 0
        with torch.no_grad():
            for name, p in ffmodel.executable.named_parameters():
                if name in wanted and tuple(wanted[name].shape) == tuple(p.shape):
                    p.copy_(wanted[name].detach().to(p.dtype))
                    n += 1
        ex = ffmodel.executable
        if getattr(ex, "shadow", None) is not None:
            ex.shadow.copy_(ex.master)
        return n


# ------------------------------------------------------------------------------------------ stage 2: records -> layers
def _resolve(a, env):
    if isinstance(a, dict):
        if "node" in a:
            return env[a["node"]]
        if "slice" in a:
            return slice(*a["slice"])
        if "dtype" in a:
            return a
        if "ellipsis" in a:
            return Ellipsis
    if isinstance(a, list):
        return [_resolve(x, env) for x in a]
    return a


def _shape_args(args):
    """view/reshape/expand/permute accept either one sequence or the extents as separate arguments."""
    if len(args) == 1 and isinstance(args[0], (list, tuple)):
        return [int(v) for v in args[0]]
    return [int(v) for v in args]


def _infer_minus_one(shape, numel):
    shape = list(shape)
    if -1 in shape:
        known = 1
        for s in shape:
            if s != -1:
                known *= s
        shape[shape.index(-1)] = numel // known
    return shape


def _numel(t: Tensor):
    n = 1
    for d in t.dims:
        n *= d
    return n


def _binary(ff: FFModel, op: str, a, b, name):
    ta, tb = isinstance(a, Tensor), isinstance(b, Tensor)
    if ta and tb:
        return {"ADD": ff.add, "SUB": ff.subtract, "MUL": ff.multiply, "TRUEDIV": ff.divide}[op](a, b, name=name)
    if not ta and not tb:  # plain python arithmetic on sizes
        return {"ADD": operator.add, "SUB": operator.sub, "MUL": operator.mul, "TRUEDIV": operator.truediv,
                "FLOORDIV": operator.floordiv}[op](a, b)
    if op == "FLOORDIV":
        raise NotImplementedError("floor division of a tensor")
    if ta:
        return {"ADD": ff.scalar_add, "SUB": ff.scalar_sub, "MUL": ff.scalar_multiply, "TRUEDIV": ff.scalar_true_divide}[op](a, b, name=name)
    # scalar on the left
    if op == "ADD":
        return ff.scalar_add(b, a, name=name)
    if op == "MUL":
        return ff.scalar_multiply(b, a, name=name)
    if op == "SUB":
        return ff.scalar_add(ff.scalar_multiply(b, -1.0), a, name=name)
    return ff.scalar_multiply(ff.pow(b, -1.0), a, name=name)


def emit_ir(records: List[dict], ff: FFModel, input_tensors: List[Tensor], verbose: bool = False):
    env: Dict[str, object] = {}
    inputs = list(input_tensors)
    outputs = []
    for rec in records:
        name, op, p = rec["name"], rec["op"], rec.get("params", {})
        a = [_resolve(x, env) for x in rec.get("inputs", [])]
        kw = {k: _resolve(v, env) for k, v in p.items()}
        x = a[0] if a else None
        if verbose:
            print(f"{name}: {op}")
        if op == "INPUT":
            if not inputs:
                raise ValueError(f"no input tensor left for placeholder {name}")
            r = inputs.pop(0)
        elif op == "OUTPUT":
            flat = a[0] if isinstance(a[0], (list, tuple)) else [a[0]]
            outputs = [t for t in flat if isinstance(t, Tensor)]
            continue
        elif op == "ATTRIBUTE":
            dt = "FLOAT" if "float" in p["dtype"] or "bfloat" in p["dtype"] or "half" in p["dtype"] else ("INT64" if p["dtype"] == "int64" else "INT32")
            r = Tensor(ff, ff.builder.create_weight([int(s) for s in p["shape"]] or [1], dt, {"type": "zero", "value": {}}, dt == "FLOAT", name))
        elif op == "LINEAR":
            r = ff.dense(x, p["out_dim"], use_bias=p["use_bias"], name=name)
        elif op == "CONV2D":
            r = ff.conv2d(x, p["out_channels"], *p["kernel"], *p["stride"], *p["padding"], groups=p["groups"], use_bias=p["use_bias"], name=name)
        elif op == "POOL2D":
            r = ff.pool2d(x, *p["kernel"], *p["stride"], *p["padding"], pool_type=PoolType(p["pool_type"]), name=name)
        elif op == "ADAPTIVE_POOL2D":
            r = ff._t(ff.builder.adaptive_pool2d(x.value, p["output"][0], p["output"][1], p["pool_type"], name))
        elif op == "BATCHNORM":
            r = ff._t(ff.builder.batch_norm(x.value, bool(p.get("affine", True)), None, float(p.get("eps", 1e-5)), 0.1, name))
        elif op == "LAYERNORM":
            nd = int(p["ndims"])
            r = ff.layer_norm(x, list(range(-nd, 0)), p.get("affine", True), p.get("eps", 1e-5), name=name)
        elif op == "T5_LAYERNORM":
            # as in the legacy importer the RMS norm is mapped onto the LayerNorm operator over the last axis
            r = ff.layer_norm(x, [-1], True, p.get("eps", 1e-6), name=name)
        elif op == "F_LAYERNORM":
            shape = a[1] if len(a) > 1 else kw["normalized_shape"]
            r = ff.layer_norm(x, list(range(-len(shape), 0)), False, kw.get("eps", 1e-5) or 1e-5, name=name)
        elif op == "SOFTMAX":
            dim = a[1] if len(a) > 1 else kw.get("dim", -1)
            r = ff.softmax(x, -1 if dim is None else dim, name=name)
        elif op == "DROPOUT":
            rate = a[1] if len(a) > 1 else kw.get("p", kw.get("rate", 0.5))
            r = ff.dropout(x, rate, 0, name=name)
        elif op == "FLAT":
            r = ff._t(ff.builder.flat(x.value, int(p.get("start_dim", 1)), int(p.get("end_dim", -1)), name))
        elif op == "FLATTEN":
            s = a[1] if len(a) > 1 else kw.get("start_dim", 0)
            e = a[2] if len(a) > 2 else kw.get("end_dim", -1)
            r = ff._t(ff.builder.flat(x.value, int(s), int(e), name))
        elif op == "EMBEDDING":
            idx = x
            if idx.num_dims >= 1 and (idx.num_dims < 2 or idx.dims[-1] != 1):
                idx = ff.reshape(idx, list(idx.dims) + [1])  # one index per bag
            r = ff.embedding(idx, p["num_embeddings"], p["embedding_dim"], AggrMode.AGGR_MODE_SUM, name=name)
        elif op in ("IDENTITY", "TO", "FLOAT", "TYPE_AS", "CONTIGUOUS"):
            r = x
        elif op in ("RELU", "GELU", "SIGMOID", "TANH", "ELU", "EXP", "SIN", "COS", "RSQRT"):
            r = getattr(ff, op.lower())(x, name=name)
        elif op in ("ADD", "SUB", "MUL", "TRUEDIV", "FLOORDIV"):
            r = _binary(ff, op, a[0], a[1] if len(a) > 1 else kw.get("other"), name)
        elif op == "POW":
            r = ff.pow(x, a[1] if len(a) > 1 else kw["exponent"], name=name)
        elif op in ("MEAN", "SUM"):
            dims = a[1] if len(a) > 1 else kw.get("dim")
            if dims is None:
                dims = list(range(x.num_dims))
            dims = [dims] if isinstance(dims, int) else list(dims)
            keep = bool(a[2] if len(a) > 2 else kw.get("keepdim", False))
            r = (ff.mean if op == "MEAN" else ff.reduce_sum)(x, dims, keep, name=name)
        elif op == "CAT":
            dim = a[1] if len(a) > 1 else kw.get("dim", 0)
            r = ff.concat(list(a[0]), dim, name=name)
        elif op == "SPLIT":
            size = a[1] if len(a) > 1 else kw.get("split_size_or_sections")
            dim = a[2] if len(a) > 2 else kw.get("dim", 0)
            total = x.dims[dim]
            sizes = list(size) if isinstance(size, (list, tuple)) else [min(size, total - i) for i in range(0, total, size)]
            r = ff.split(x, sizes, dim, name=name)
        elif op == "GETITEM":
            if isinstance(x, (list, tuple)):
                r = x[a[1]]
            else:
                raise NotImplementedError("slicing a tensor with getitem")
        elif op == "GETATTR":
            attr = a[1]
            if attr == "shape":
                r = tuple(x.dims)
            elif attr in ("dtype", "device"):
                r = None
            else:
                raise NotImplementedError(f"getattr({attr})")
        elif op == "SIZE":
            r = tuple(x.dims) if len(a) == 1 else x.dims[a[1]]
        elif op == "F_LINEAR":
            # the functional form (what torch.compile's graphs contain): weight and bias are tensors of the graph, not
            # parameters owned by a layer, so this is a product with the transposed weight plus a broadcast bias
            w = a[1]
            b = a[2] if len(a) > 2 else kw.get("bias")
            rows = _numel(x) // x.dims[-1]
            x3 = ff.reshape(x, [1, rows, x.dims[-1]], name=name + ".x3")
            wt = ff.transpose(ff.reshape(w, [1, w.dims[0], w.dims[1]], name=name + ".w3"), [0, 2, 1], name=name + ".wt")
            y = ff.reshape(ff.batch_matmul(x3, wt, name=name + ".mm"), list(x.dims[:-1]) + [w.dims[0]], name=name + ".y")
            if isinstance(b, Tensor):
                y = ff.add(y, ff._t(ff.builder.broadcast(b.value, list(y.dims), name + ".bias")), name=name)
            r = y
        elif op == "MATMUL":
            r = ff.batch_matmul(a[0], a[1], name=name)
        elif op == "TRANSPOSE":
            perm = list(range(x.num_dims))
            d0, d1 = a[1] % x.num_dims, a[2] % x.num_dims
            perm[d0], perm[d1] = perm[d1], perm[d0]
            r = ff.transpose(x, perm, name=name)
        elif op == "PERMUTE":
            r = ff.transpose(x, [d % x.num_dims for d in _shape_args(a[1:])], name=name)
        elif op in ("RESHAPE", "VIEW"):
            r = ff.reshape(x, _infer_minus_one(_shape_args(a[1:]), _numel(x)), name=name)
        elif op == "EXPAND":
            tgt = _shape_args(a[1:])
            src = [1] * (len(tgt) - x.num_dims) + list(x.dims)
            tgt = [s if t == -1 else t for s, t in zip(src, tgt)]
            r = x if tuple(tgt) == tuple(x.dims) else ff._t(ff.builder.broadcast(x.value, tgt, name))
        elif op == "UNSQUEEZE":
            d = a[1] if len(a) > 1 else kw["dim"]
            dims = list(x.dims)
            d = d % (len(dims) + 1)
            r = ff.reshape(x, dims[:d] + [1] + dims[d:], name=name)
        elif op == "SQUEEZE":
            dims = list(x.dims)
            if len(a) > 1:
                d = a[1] % len(dims)
                dims = dims[:d] + dims[d + 1:] if dims[d] == 1 else dims
            else:
                dims = [s for s in dims if s != 1]
            r = ff.reshape(x, dims, name=name)
        else:
            raise NotImplementedError(f"importer op {op}")
        env[name] = r
    return outputs


# ------------------------------------------------------------------------------------------ one-call entry points
class CompiledModule:
    """An ``nn.Module`` compiled for this framework's executors: ``train_step`` / ``forward`` on tensors named after the
    module's ``forward`` arguments.  Returned by :func:`compile_module`; also what the ``torch.compile`` backend wraps."""

    def __init__(self, module: nn.Module, ffmodel: FFModel, importer: "PyTorchModel", input_names: List[str]):
        self.module, self.ffmodel, self.importer, self.input_names = module, ffmodel, importer, input_names
        self.compiled = ffmodel.compiled
        self.executable = ffmodel.executable
        self.graph = ffmodel.graph
        self.search_stats = getattr(self.compiled, "search_stats", {})

    def _named(self, args):
        if len(args) == 1 and isinstance(args[0], dict):
            return args[0]
        if len(args) != len(self.input_names):
            raise ValueError(f"the module takes {len(self.input_names)} inputs ({self.input_names}), got {len(args)}")
        return dict(zip(self.input_names, args))

    def train_step(self, *inputs, labels=None, return_loss: bool = True):
        return self.compiled.train_step(self._named(inputs), labels, return_loss=return_loss)

    def forward(self, *inputs):
        return self.executable.infer(self._named(inputs))

    __call__ = forward

    def sync_parameters_to_module(self):
        """Write the trained weights back into the ``nn.Module`` (fp32 master copies, matched by layer name)."""
        trained = dict(self.executable.named_parameters())
        n = 0
        with torch.no_grad():
            for rec in self.importer.to_ir():
                mod = rec["params"].get("module")
                if mod is None:
                    continue
                sub = self.module.get_submodule(mod)
                for slot, key in (("weight", "weight"), ("filter", "weight"), ("bias", "bias"), ("gamma", "weight"), ("beta", "bias")):
                    src = trained.get(f"{rec['name']}.{slot}")
                    dst = getattr(sub, key, None)
                    if src is not None and dst is not None and tuple(dst.shape) == tuple(src.shape):
                        dst.copy_(src.to(dst.dtype))
                        n += 1
        return n


def compile_module(module: nn.Module, example_inputs, *, optimizer=None, loss_type=None, metrics=None, config=None, algorithm: Optional[str] = None,
                   search_budget: Optional[int] = None, device: Optional[str] = None, dist=None, is_hf_model: bool = False,
                   copy_weights: bool = True) -> CompiledModule:
    """``nn.Module`` -> traced graph -> computation graph -> strategy search -> executor, in one call: the flow the
    reference draws for its PyTorch frontend (docs/plantuml/figures/pytorch-tracing.puml: ``model.compile(algorithm=...,
    optimizer=...)`` returning a compiled model with forward / backward / update).

    `example_inputs`: one tensor per ``forward`` argument (only shapes and dtypes are used).  `algorithm`: the search
    algorithm ("unity", "mcmc", "data_parallel", ...) when several ranks are present (`dist`); `search_budget` its budget.
    The module's current parameter values are copied into the executor unless ``copy_weights=False``."""
    from ..api import FFConfig as ApiConfig

    import inspect

    if isinstance(example_inputs, torch.Tensor):
        example_inputs = [example_inputs]
    example_inputs = list(example_inputs)
    names = [p for p in inspect.signature(module.forward).parameters][:len(example_inputs)]
    cfg = config or ApiConfig(batch_size=int(example_inputs[0].shape[0]))
    if algorithm is not None:
        cfg.search_algorithm = algorithm
    if search_budget is not None:
        cfg.search_budget = search_budget
    ff = FFModel(cfg)
    dt = {torch.float32: DataType.DT_FLOAT, torch.int32: DataType.DT_INT32, torch.int64: DataType.DT_INT64, torch.bfloat16: DataType.DT_FLOAT,
          torch.float16: DataType.DT_FLOAT}
    tensors = [ff.create_tensor(list(t.shape), dt.get(t.dtype, DataType.DT_FLOAT), create_grad=t.dtype.is_floating_point, name=n)
               for n, t in zip(names, example_inputs)]
    importer = PyTorchModel(module, is_hf_model=is_hf_model, input_names=names if is_hf_model else None)
    importer.torch_to_ff(ff, tensors)
    ff.compile(optimizer, loss_type, metrics, device=device, dist=dist)
    if copy_weights:
        importer.copy_parameters(ff)
    return CompiledModule(module, ff, importer, names)


def flexflow_backend(gm, example_inputs, **options):
    """``torch.compile(model, backend=flexflow_backend)``: the graph module dynamo hands over is imported and compiled for
    inference on this framework's executor; the returned callable has the calling convention dynamo expects (positional
    tensors in, tuple of tensors out).  Training through ``torch.compile`` is not offered -- autograd would have to call
    back into the executor per operator; use :func:`compile_module` and its ``train_step`` for that."""
    from .types import CompMode

    names = [n.name for n in gm.graph.nodes if n.op == "placeholder"]
    cfg_device = options.get("device")
    from ..api import FFConfig as ApiConfig

    ff = FFModel(ApiConfig(batch_size=int(example_inputs[0].shape[0]) if len(example_inputs) and example_inputs[0].dim() else 1))
    tensors = [ff.create_tensor(list(t.shape), DataType.DT_FLOAT if t.dtype.is_floating_point else DataType.DT_INT32,
                                create_grad=False, name=n) for n, t in zip(names, example_inputs)]
    importer = PyTorchModel(gm)
    importer._traced = gm
    importer.torch_to_ff(ff, tensors)
    ff.compile(None, None, None, comp_mode=CompMode.INFERENCE, device=cfg_device)
    importer.copy_parameters(ff)

    def run(*args):
        out = ff.executable.infer(dict(zip(names, args)))
        return (out,) if isinstance(out, torch.Tensor) else tuple(out)

    return run
