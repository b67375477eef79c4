"""Layer-by-layer model API with ``compile`` / ``fit`` / ``eval``.

The method names and arguments follow the legacy Python class (bindings/python/old/flexflow/core/flexflow_cffi.py:
948-2100) so model scripts port by changing the import.  Every layer call appends to a C++ ``GraphBuilder``;
``compile`` runs the strategy search and lowers to the GPU executor (or to the CPU interpreter when no GPU is
present or ``device="cpu"`` is asked for).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import _ffcore as core
from ..api import FFConfig
from ..runtime.executor import ExecConfig, OptimizerConfig
from ..utils.metrics import PerfMetrics
from .types import ActiMode, AggrMode, CompMode, DataType, LossType, MetricsType, PoolType, enum_value


# ------------------------------------------------------------------------------------------ small value classes
class Tensor:
    """Handle of a value in the graph under construction."""

    def __init__(self, model: "FFModel", value, name: Optional[str] = None):
        self.model = model
        self.value = tuple(value)
        self.name = name

    @property
    def dims(self):
        return tuple(int(s) for s in self.model.builder.graph.shape(self.value).sizes)

    @property
    def num_dims(self):
        return len(self.dims)

    @property
    def data_type(self):
        return DataType(self.model.builder.graph.shape(self.value).dtype)

    def __repr__(self):
        return f"Tensor(dims={self.dims}, dtype={self.data_type.name}, value={self.value})"

    # ---- data access of the legacy Tensor / Parameter classes (flexflow_cffi.py: get_weights, set_weights, get_gradients,
    # get_array, get_flat_array).  Valid once the model is compiled; arrays are numpy copies on the host.
    def _parameter_name(self, ffmodel) -> str:
        node = next(n for n in ffmodel.graph.nodes() if n["id"] == self.value[0])
        if node["type"] != "WEIGHT":
            raise TypeError(f"{self!r} is not a weight: only parameters can be read and written like this")
        return node["name"] or f"weight{node['id']}"

    def _lookup(self, ffmodel, pairs, what):
        if getattr(ffmodel, "executable", None) is None:
            raise RuntimeError(f"{what}: compile the model first")
        name = self._parameter_name(ffmodel)
        for k, t in pairs:
            if k == name:
                return t
        raise KeyError(f"{what}: no parameter named {name!r} on this device (a sharded strategy keeps shards: use the checkpoint API)")

    @staticmethod
    def _pairs(ffmodel, what, which):
        if getattr(ffmodel, "executable", None) is None:
            raise RuntimeError(f"{what}: compile the model first")
        return getattr(ffmodel.executable, which)()

    def get_weights(self, ffmodel):
        t = self._lookup(ffmodel, self._pairs(ffmodel, "get_weights", "named_parameters"), "get_weights")
        if tuple(t.shape) != self.dims:
            raise RuntimeError(f"get_weights: this rank holds a shard of shape {tuple(t.shape)} of a {self.dims} parameter")
        return t.detach().float().cpu().numpy().copy()

    def set_weights(self, ffmodel, np_array) -> bool:
        t = self._lookup(ffmodel, self._pairs(ffmodel, "set_weights", "named_parameters"), "set_weights")
        src = torch.as_tensor(np_array)
        if tuple(src.shape) != tuple(t.shape):
            raise ValueError(f"set_weights: array of shape {tuple(src.shape)} for a parameter of shape {tuple(t.shape)}")
        with torch.no_grad():
            t.copy_(src.to(device=t.device, dtype=t.dtype))
        ex = ffmodel.executable
        if getattr(ex, "shadow", None) is not None:      # the compute-dtype copy the kernels read
            ex.shadow.copy_(ex.master)
        return True

    def get_gradients(self, ffmodel, comm_type=None):
        t = self._lookup(ffmodel, self._pairs(ffmodel, "get_gradients", "named_gradients"), "get_gradients")
        if t is None:
            raise RuntimeError("get_gradients: no backward pass has run yet")
        return t.detach().float().cpu().numpy().copy()

    def get_array(self, ffmodel, data_type=None):
        return self.get_weights(ffmodel)

    def get_flat_array(self, ffmodel, data_type=None):
        return self.get_weights(ffmodel).reshape(-1)


class Initializer:
    def __init__(self, kind: str, **value):
        self.attrs = {"type": kind, "value": value}


class GlorotUniformInitializer(Initializer):
    def __init__(self, seed=0):
        super().__init__("glorot_uniform", seed=seed)


class ZeroInitializer(Initializer):
    def __init__(self):
        super().__init__("zero")


class UniformInitializer(Initializer):
    def __init__(self, seed, minv, maxv):
        super().__init__("uniform", seed=seed, min_val=minv, max_val=maxv)


class NormInitializer(Initializer):
    def __init__(self, seed, mean, stddev):
        super().__init__("normal", seed=seed, mean=mean, stddev=stddev)


def _init(i):
    return None if i is None else i.attrs


class SGDOptimizer:
    def __init__(self, ffmodel=None, lr=0.01, momentum=0.0, nesterov=False, weight_decay=0.0):
        self.config = OptimizerConfig(kind="sgd", lr=lr, momentum=momentum, nesterov=nesterov, weight_decay=weight_decay)

    def set_learning_rate(self, learning_rate):
        self.config.lr = learning_rate


class AdamOptimizer:
    def __init__(self, ffmodel=None, alpha=0.001, beta1=0.9, beta2=0.999, weight_decay=0.0, epsilon=1e-8):
        self.config = OptimizerConfig(kind="adam", lr=alpha, beta1=beta1, beta2=beta2, weight_decay=weight_decay, epsilon=epsilon)

    def set_learning_rate(self, learning_rate):
        self.config.lr = learning_rate


class SingleDataLoader:
    """Feeds one graph input (or the labels) from a full host array, batch by batch, through pinned memory."""

    def __init__(self, ffmodel: "FFModel", batch_tensor: Optional[Tensor], full_array, is_label=False):
        self.model = ffmodel
        self.batch_tensor = batch_tensor
        arr = torch.as_tensor(np.ascontiguousarray(full_array)) if not torch.is_tensor(full_array) else full_array
        self.full = arr.pin_memory() if torch.cuda.is_available() else arr
        self.num_samples = int(arr.shape[0])
        self.is_label = is_label
        self.pos = 0

    def reset(self):
        self.pos = 0

    def next_batch(self, ffmodel=None):
        bs = self.model.ffconfig.batch_size
        if self.pos + bs > self.num_samples:
            self.pos = 0
        out = self.full[self.pos:self.pos + bs]
        self.pos += bs
        return out


class Layer:
    def __init__(self, model, node_id):
        self.model, self.node_id = model, node_id

    @property
    def _node(self):
        return next(n for n in self.model.builder.graph.nodes() if n["id"] == self.node_id)

    @property
    def name(self):
        return self._node["name"]

    @property
    def op_type(self):
        return self._node["type"]

    def get_parameter_by_id(self, idx):
        ws = [tuple(v) for s, v in self._node["inputs"] if s not in ("INPUT", "LHS_INPUT", "RHS_INPUT", "QUERY", "KEY", "VALUE", "INDEX")]
        return Tensor(self.model, ws[idx])

    def get_weight_tensor(self):
        return self.get_parameter_by_id(0)

    def get_bias_tensor(self):
        return self.get_parameter_by_id(1)

    def get_output_tensor(self):
        return Tensor(self.model, (self.node_id, self._node["outputs"][0][0]))

    _ACTIVATION_SLOTS = ("INPUT", "LHS_INPUT", "RHS_INPUT", "QUERY", "KEY", "VALUE", "INDEX")

    def get_number_inputs(self) -> int:
        return sum(1 for s, _ in self._node["inputs"] if s in self._ACTIVATION_SLOTS)

    def get_number_parameters(self) -> int:
        return sum(1 for s, _ in self._node["inputs"] if s not in self._ACTIVATION_SLOTS)

    def get_number_outputs(self) -> int:
        return len(self._node["outputs"])

    def get_input_by_id(self, idx):
        ins = [tuple(v) for s, v in self._node["inputs"] if s in self._ACTIVATION_SLOTS]
        return Tensor(self.model, ins[idx])

    def get_input_tensor(self):
        return self.get_input_by_id(0)

    def get_output_by_id(self, idx):
        return Tensor(self.model, (self.node_id, self._node["outputs"][idx][0]))


# ------------------------------------------------------------------------------------------ the model
class FFModel:
    def __init__(self, ffconfig: Optional[FFConfig] = None):
        self.ffconfig = ffconfig or FFConfig()
        self.builder = core.GraphBuilder()
        self._inputs: List[Tensor] = []
        self._layers: List[Layer] = []
        self._loaders: Dict[str, SingleDataLoader] = {}
        self._label_loader: Optional[SingleDataLoader] = None
        self.compiled = None
        self.optimizer = None
        self.metrics: List[str] = []
        self.perf = PerfMetrics()
        self._label_tensor = None
        self._batch_inputs: Dict[str, torch.Tensor] = {}
        self._batch_labels = None

    # ---- bookkeeping
    def _t(self, value, name=None) -> Tensor:
        t = Tensor(self, value, name)
        self._layers.append(Layer(self, t.value[0]))
        return t

    @staticmethod
    def _n(name):
        return name or ""

    def get_layers(self):
        return {i: l for i, l in enumerate(self._layers)}

    def get_layer_by_id(self, layer_id):
        return self._layers[layer_id]

    def get_last_layer(self):
        return self._layers[-1]

    def get_layer_by_name(self, layer_name):
        for l in self._layers:
            if l.name == layer_name:
                return l
        return None

    def get_tensor_by_id(self, id):
        """The first output of the layer with that id (legacy `FFModel.get_tensor_by_id`)."""
        return self.get_layer_by_id(id).get_output_tensor()

    def print_layers(self, id=-1):
        for i, l in enumerate(self._layers):
            if id in (-1, i):
                print(f"layer {i}: {l.op_type} {l.name!r} -> {l.get_output_tensor().dims}")

    # ---- tensors
    def create_tensor(self, dims, data_type=DataType.DT_FLOAT, create_grad=True, name=None) -> Tensor:
        name = name or f"input{len(self._inputs)}"
        v = self.builder.create_input([int(d) for d in dims], enum_value(data_type), bool(create_grad), name)
        t = Tensor(self, v, name)
        self._inputs.append(t)
        return t

    def create_constant(self, dims, value, data_type=DataType.DT_FLOAT) -> Tensor:
        v = self.builder.create_weight([int(d) for d in dims], enum_value(data_type), {"type": "constant", "value": {"value": float(value)}},
                                       False, f"constant{len(self._layers)}")
        return Tensor(self, v)

    # ---- elementwise
    def _unary(self, op, x, scalar=None, name=None):
        return self._t(self.builder.unary(op, x.value, scalar, self._n(name)))

    def _binary(self, op, x, y, name=None):
        return self._t(self.builder.binary(op, x.value, y.value, self._n(name)))

    def exp(self, x, name=None): return self._unary("EXP", x, None, name)
    def sin(self, x, name=None): return self._unary("SIN", x, None, name)
    def cos(self, x, name=None): return self._unary("COS", x, None, name)
    def rsqrt(self, input, name=None): return self._unary("RSQRT", input, None, name)
    def pow(self, input, exponent, name=None): return self._unary("POW", input, float(exponent), name)
    def gelu(self, input, inplace=True, name=None): return self._unary("GELU", input, None, name)
    def relu(self, input, inplace=True, name=None): return self._unary("RELU", input, None, name)
    def sigmoid(self, input, name=None): return self._unary("SIGMOID", input, None, name)
    def tanh(self, input, name=None): return self._unary("TANH", input, None, name)
    def elu(self, input, inplace=True, name=None): return self._unary("ELU", input, None, name)
    def identity(self, input, name=None): return self._t(self.builder.noop(input.value, self._n(name)))
    def scalar_multiply(self, input, scalar, inplace=True, name=None): return self._unary("SCALAR_MULTIPLY", input, float(scalar), name)
    def scalar_add(self, input, scalar, inplace=True, name=None): return self._unary("SCALAR_ADD", input, float(scalar), name)
    def scalar_sub(self, input, scalar, inplace=True, name=None): return self._unary("SCALAR_SUB", input, float(scalar), name)
    def scalar_true_divide(self, input, scalar, inplace=True, name=None): return self._unary("SCALAR_TRUE_DIV", input, float(scalar), name)
    def add(self, x, y, inplace_a=False, name=None): return self._binary("EW_ADD", x, y, name)
    def subtract(self, x, y, inplace_a=False, name=None): return self._binary("EW_SUB", x, y, name)
    def multiply(self, x, y, inplace_a=False, name=None): return self._binary("EW_MUL", x, y, name)
    def divide(self, x, y, inplace_a=False, name=None): return self._binary("EW_DIV", x, y, name)
    def max(self, x, y, inplace_a=False, name=None): return self._binary("EW_MAX", x, y, name)
    def min(self, x, y, inplace_a=False, name=None): return self._binary("EW_MIN", x, y, name)

    # ---- reductions
    def reduce_sum(self, input, axes, keepdims=False, name=None):
        return self._t(self.builder.reduce("REDUCE_SUM", input.value, [int(a) for a in axes], bool(keepdims), self._n(name)))

    def mean(self, input, dims, keepdims=False, name=None):
        return self._t(self.builder.reduce("REDUCE_MEAN", input.value, [int(a) for a in dims], bool(keepdims), self._n(name)))

    # ---- layers with weights
    def conv2d(self, input, out_channels, kernel_h, kernel_w, stride_h, stride_w, padding_h, padding_w,
               activation=ActiMode.AC_MODE_NONE, groups=1, use_bias=True, shared_op=None, kernel_initializer=None,
               bias_initializer=None, name=None):
        return self._t(self.builder.conv2d(input.value, int(out_channels), int(kernel_h), int(kernel_w), int(stride_h), int(stride_w),
                                           int(padding_h), int(padding_w), enum_value(activation), int(groups), bool(use_bias),
                                           _init(kernel_initializer), _init(bias_initializer), self._n(name)))

    def embedding(self, input, num_embeddings, embedding_dim, aggr=AggrMode.AGGR_MODE_SUM, shared_op=None, kernel_initializer=None,
                  name=None):
        a = enum_value(aggr)
        return self._t(self.builder.embedding(input.value, int(num_embeddings), int(embedding_dim), "SUM" if a == "NONE" else a, "FLOAT",
                                              _init(kernel_initializer), self._n(name)))

    def pool2d(self, input, kernel_h, kernel_w, stride_h, stride_w, padding_h, padding_w, pool_type=PoolType.POOL_MAX,
               activation=ActiMode.AC_MODE_NONE, name=None):
        return self._t(self.builder.pool2d(input.value, int(kernel_h), int(kernel_w), int(stride_h), int(stride_w), int(padding_h),
                                           int(padding_w), enum_value(pool_type), enum_value(activation), self._n(name)))

    def batch_norm(self, input, relu=True, name=None):
        return self._t(self.builder.batch_norm(input.value, True, "RELU" if relu else None, 1e-5, 0.1, self._n(name)))

    def layer_norm(self, input, axes, elementwise_affine=True, eps=1e-5, name=None):
        return self._t(self.builder.layer_norm(input.value, [int(a) for a in axes], bool(elementwise_affine), float(eps), self._n(name)))

    def batch_matmul(self, A, B, a_seq_length_dim=None, b_seq_length_dim=None, name=None):
        return self._t(self.builder.batch_matmul(A.value, B.value, self._n(name)))

    def dense(self, input, out_dim, activation=ActiMode.AC_MODE_NONE, use_bias=True, datatype=DataType.DT_FLOAT, shared_op=None,
              kernel_initializer=None, bias_initializer=None, kernel_regularizer=None, name=None):
        return self._t(self.builder.dense(input.value, int(out_dim), enum_value(activation), bool(use_bias), _init(kernel_initializer),
                                          _init(bias_initializer), self._n(name)))

    def multihead_attention(self, query, key, value, embed_dim, num_heads, kdim=0, vdim=0, dropout=0.0, bias=True, add_bias_kv=False,
                            add_zero_attn=False, kernel_initializer=None, name=None):
        return self._t(self.builder.multihead_attention(query.value, key.value, value.value, int(embed_dim), int(num_heads),
                                                        int(kdim) or None, int(vdim) or None, float(dropout), bool(bias),
                                                        bool(add_bias_kv), bool(add_zero_attn), _init(kernel_initializer), self._n(name)))

    # ---- shape operators
    def concat(self, tensors, axis, name=None):
        return self._t(self.builder.concat([t.value for t in tensors], int(axis), self._n(name)))

    def split(self, input, sizes, axis, name=None):
        if isinstance(sizes, int):
            total = input.dims[axis]
            sizes = [total // sizes] * sizes
        outs = self.builder.split(input.value, [int(s) for s in sizes], int(axis), self._n(name))
        ts = [Tensor(self, v) for v in outs]
        self._layers.append(Layer(self, ts[0].value[0]))
        return ts

    def flat(self, input, name=None): return self._t(self.builder.flat(input.value, 1, -1, self._n(name)))
    def softmax(self, input, axis=-1, name=None): return self._t(self.builder.softmax(input.value, int(axis), self._n(name)))
    def reshape(self, input, shape, name=None): return self._t(self.builder.reshape(input.value, [int(s) for s in shape], self._n(name)))
    def gather(self, input, index, dim, name=None): return self._t(self.builder.gather(input.value, index.value, int(dim), self._n(name)))
    def transpose(self, input, perm, name=None): return self._t(self.builder.transpose(input.value, [int(p) for p in perm], self._n(name)))
    def reverse(self, input, axis, name=None): return self._t(self.builder.reverse(input.value, int(axis), self._n(name)))
    def dropout(self, input, rate, seed=0, name=None): return self._t(self.builder.dropout(input.value, float(rate), int(seed), self._n(name)))

    def cast(self, input, data_type, name=None): return self._t(self.builder.cast(input.value, enum_value(data_type), self._n(name)))

    # ---- training surface
    def set_optimizer(self, optimizer):
        self.optimizer = optimizer

    @property
    def graph(self):
        return self.builder.graph

    def compile(self, optimizer=None, loss_type=None, metrics=None, comp_mode=None, device: Optional[str] = None, dist=None):
        """Search a strategy and lower to an executor.  ``device`` defaults to the GPU when there is one."""
        from .. import api

        if optimizer is not None:
            self.optimizer = optimizer
        opt_cfg = self.optimizer.config if self.optimizer is not None else OptimizerConfig(kind="sgd", lr=self.ffconfig.learning_rate)
        self.loss = enum_value(loss_type) if loss_type is not None else LossType.LOSS_SPARSE_CATEGORICAL_CROSSENTROPY.value
        self.metrics = [enum_value(m) for m in (metrics or [])]
        training = enum_value(comp_mode) != CompMode.INFERENCE.value if comp_mode is not None else True
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        if device == "cpu":
            from ..runtime.cpu_executor import CpuExecutable

            cfg = ExecConfig(compute_dtype="fp32", loss=self.loss, optimizer=opt_cfg, seed=self.ffconfig.seed, device="cpu",
                             training=training)
            self.compiled = api.CompiledModel(self.graph, CpuExecutable(self.graph, cfg), self.graph, {})
        else:
            self.compiled = api.compile(self.graph, config=self.ffconfig, optimizer=opt_cfg, loss=self.loss, dist=dist,
                                        training=training, device=device)
        self.executable = self.compiled.executable
        return self.compiled

    @property
    def label_tensor(self):
        """Shape and type of the labels the compiled loss expects."""
        lv = self.executable.loss_value
        dims = list(self.graph.shape(lv).sizes)
        if self.loss == LossType.LOSS_SPARSE_CATEGORICAL_CROSSENTROPY.value:
            return {"dims": tuple(dims[:-1]) + (1,), "data_type": DataType.DT_INT32}
        return {"dims": tuple(dims), "data_type": DataType.DT_FLOAT}

    def create_data_loader(self, batch_tensor, full_array):
        is_label = not isinstance(batch_tensor, Tensor)
        dl = SingleDataLoader(self, None if is_label else batch_tensor, full_array, is_label=is_label)
        if is_label:
            self._label_loader = dl
        else:
            self._loaders[batch_tensor.name] = dl
        return dl

    def init_layers(self):
        """Weights are initialised when the executor is built; kept for script compatibility."""

    def reset_metrics(self):
        self.perf.reset()

    def get_perf_metrics(self):
        return self.perf

    def _next_batch(self, xs, y):
        self._batch_inputs = {dl.batch_tensor.name: dl.next_batch() for dl in xs}
        self._batch_labels = y.next_batch() if y is not None else None

    # piecewise step API of the legacy class
    def forward(self, seq_length=None):
        ex = self.executable
        ex.set_inputs(self._batch_inputs, self._batch_labels)
        if getattr(ex, "on_gpu", False):
            ex._pre_step()
        ex.forward()

    def zero_gradients(self):
        if hasattr(self.executable, "zero_gradients"):
            self.executable.zero_gradients()

    def backward(self, seq_length=None):
        ex = self.executable
        if getattr(ex, "on_gpu", False):
            ex.compute_loss()
            ex.backward()
            ex.sync_gradients()
        else:
            ex.backward()

    def update(self):
        self.executable.update()

    def _predictions(self):
        ex = self.executable
        if not getattr(ex, "on_gpu", False):
            return ex._pred.detach()
        from ..runtime.executor import SoftmaxOp

        op = ex.ops[ex.loss_value[0]]
        rows, cols = ex.loss_shape
        if isinstance(op, SoftmaxOp) and op.fused_loss:
            return torch.softmax(op.x().view(rows, cols).float(), -1)
        return ex.values[ex.loss_value].data.view(rows, cols).float()

    def compute_metrics(self):
        if not self.metrics or self._batch_labels is None:
            return self.perf
        pred = self._predictions()
        pred = pred.reshape(-1, pred.shape[-1]).cpu()
        lab = self._batch_labels.cpu()
        lab = lab.reshape(-1) if lab.numel() == pred.shape[0] else lab.reshape(pred.shape[0], -1)
        return self.perf.update(pred, lab, self.metrics)

    def _loaders_for(self, x, y, batch_size):
        if batch_size:
            self.ffconfig.batch_size = batch_size
        xs = x if isinstance(x, (list, tuple)) else [x]
        loaders = []
        for i, item in enumerate(xs):
            loaders.append(item if isinstance(item, SingleDataLoader) else self.create_data_loader(self._inputs[i], item))
        yl = y if (y is None or isinstance(y, SingleDataLoader)) else self.create_data_loader(None, y)
        return loaders, yl

    def fit(self, x=None, y=None, batch_size=None, epochs=1, verbose=False):
        """next_batch -> forward -> zero_gradients -> backward -> update, `epochs` passes over the loaders
        (bindings/python/old/flexflow/core/flexflow_cffi.py:2058-2100)."""
        xs, yl = self._loaders_for(x, y, batch_size)
        iters = xs[0].num_samples // self.ffconfig.batch_size
        history = []
        for epoch in range(epochs):
            for dl in xs + ([yl] if yl else []):
                dl.reset()
            self.reset_metrics()
            for _ in range(iters):
                self._next_batch(xs, yl)
                loss = self.compiled.train_step(self._batch_inputs, self._batch_labels)
                history.append(loss)
                self.compute_metrics()
            if verbose:
                print(f"epoch {epoch}: loss {history[-1]:.4f} {self.perf.summary()}")
        return history

    def eval(self, x=None, y=None, batch_size=None):
        xs, yl = self._loaders_for(x, y, batch_size)
        iters = xs[0].num_samples // self.ffconfig.batch_size
        for dl in xs + ([yl] if yl else []):
            dl.reset()
        self.reset_metrics()
        for _ in range(iters):
            self._next_batch(xs, yl)
            self.executable.infer(self._batch_inputs)
            self.compute_metrics()
        return self.perf

    def adaptive_pool2d(self, input, output_h, output_w, pool_type=PoolType.POOL_AVG, name=None):
        return self._t(self.builder.adaptive_pool2d(input.value, int(output_h), int(output_w), enum_value(pool_type), self._n(name)))
