"""ONNX importer: walks ``model.graph.node`` and calls the ``FFModel`` layer methods.

Operator handlers match the legacy importer (bindings/python/old/flexflow/onnx/model.py:74-290): Add, Sub, Mul,
Concat, Split, AveragePool, GlobalAveragePool, BatchNormalization, Conv, Dropout, Flatten, Gemm/Dense, MaxPool,
Relu, Pad, Softmax, Reshape, Cast, Unsqueeze, Constant, Range, plus MatMul, Transpose, Identity, Sigmoid, Tanh.
The Keras-exported variant (``ONNXModelKeras``) also folds the Transpose/Reshape pairs Keras emits around Dense.

The ``onnx`` package is optional: the importer only needs objects with the protobuf field names
(``graph.node[*].op_type/input/output/attribute``, ``graph.initializer[*].name/dims``), so a model can be passed as
a loaded ``ModelProto`` or as any stand-in with those attributes.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np

from .ffmodel import FFModel, Tensor
from .types import ActiMode, DataType, PoolType


def _attrs(node) -> dict:
    out = {}
    for a in getattr(node, "attribute", []):
        if getattr(a, "ints", None):
            out[a.name] = [int(v) for v in a.ints]
        elif getattr(a, "floats", None):
            out[a.name] = [float(v) for v in a.floats]
        elif getattr(a, "s", None):
            out[a.name] = a.s.decode() if isinstance(a.s, bytes) else a.s
        elif getattr(a, "t", None) is not None and getattr(a, "type", None) in (4, "TENSOR"):
            out[a.name] = _tensor_value(a.t)
        elif getattr(a, "f", None) not in (None, 0.0) or getattr(a, "type", None) in (1, "FLOAT"):
            out[a.name] = float(a.f)
        else:
            out[a.name] = int(getattr(a, "i", 0))
    return out


def _tensor_value(t):
    """Value of a TensorProto-like object as a numpy array."""
    if hasattr(t, "numpy_value"):
        return np.asarray(t.numpy_value)
    try:
        from onnx import numpy_helper

        return numpy_helper.to_array(t)
    except ImportError:
        for field, dt in (("float_data", np.float32), ("int64_data", np.int64), ("int32_data", np.int32)):
            v = getattr(t, field, None)
            if v:
                return np.asarray(list(v), dtype=dt).reshape([int(d) for d in t.dims])
        raise ValueError("cannot read tensor value without the onnx package")


class ONNXModel:
    def __init__(self, model):
        if isinstance(model, str):
            import onnx

            model = onnx.load(model)
        self.model = model
        self.inits: Dict[str, object] = {i.name: i for i in model.graph.initializer}
        self.symbols: Dict[str, object] = {}

    # ---- helpers
    def _const(self, name) -> Optional[np.ndarray]:
        if name in self.symbols and isinstance(self.symbols[name], np.ndarray):
            return self.symbols[name]
        if name in self.inits:
            return _tensor_value(self.inits[name])
        return None

    def _in(self, node, i) -> Tensor:
        return self.symbols[node.input[i]]

    # ---- handlers: each returns the value(s) bound to node.output
    def handleAdd(self, ff, node): return ff.add(self._in(node, 0), self._in(node, 1), name=node.name)
    def handleSub(self, ff, node): return ff.subtract(self._in(node, 0), self._in(node, 1), name=node.name)
    def handleMul(self, ff, node): return ff.multiply(self._in(node, 0), self._in(node, 1), name=node.name)
    def handleRelu(self, ff, node): return ff.relu(self._in(node, 0), name=node.name)
    def handleSigmoid(self, ff, node): return ff.sigmoid(self._in(node, 0), name=node.name)
    def handleTanh(self, ff, node): return ff.tanh(self._in(node, 0), name=node.name)
    def handleIdentity(self, ff, node): return self._in(node, 0)
    def handleCast(self, ff, node): return self._in(node, 0)
    def handleMatMul(self, ff, node): return ff.batch_matmul(self._in(node, 0), self._in(node, 1), name=node.name)

    def handleConcat(self, ff, node):
        return ff.concat([self.symbols[i] for i in node.input], _attrs(node)["axis"], name=node.name)

    def handleSplit(self, ff, node):
        a = _attrs(node)
        x = self._in(node, 0)
        sizes = a.get("split")
        if sizes is None and len(node.input) > 1:
            sizes = [int(v) for v in self._const(node.input[1])]
        if sizes is None:
            n = len(node.output)
            sizes = [x.dims[a.get("axis", 0)] // n] * n
        return ff.split(x, sizes, a.get("axis", 0), name=node.name)

    def _pool(self, ff, node, kind):
        a = _attrs(node)
        k = a["kernel_shape"]
        s = a.get("strides", [1, 1])
        p = a.get("pads", [0, 0, 0, 0])
        return ff.pool2d(self._in(node, 0), k[0], k[1], s[0], s[1], p[0], p[1], kind, name=node.name)

    def handleAveragePool(self, ff, node): return self._pool(ff, node, PoolType.POOL_AVG)
    def handleMaxPool(self, ff, node): return self._pool(ff, node, PoolType.POOL_MAX)

    def handleGlobalAveragePool(self, ff, node):
        x = self._in(node, 0)
        return ff.pool2d(x, x.dims[2], x.dims[3], 1, 1, 0, 0, PoolType.POOL_AVG, name=node.name)

    def handleBatchNormalization(self, ff, node):
        return ff.batch_norm(self._in(node, 0), relu=False, name=node.name)

    def handleConv(self, ff, node):
        a = _attrs(node)
        w = self.inits[node.input[1]]
        oc = int(w.dims[0])
        k = a.get("kernel_shape", [int(w.dims[2]), int(w.dims[3])])
        s = a.get("strides", [1, 1])
        p = a.get("pads", [0, 0, 0, 0])
        return ff.conv2d(self._in(node, 0), oc, k[0], k[1], s[0], s[1], p[0], p[1], ActiMode.AC_MODE_NONE, a.get("group", 1),
                         len(node.input) > 2, name=node.name)

    def handleDropout(self, ff, node):
        a = _attrs(node)
        return ff.dropout(self._in(node, 0), a.get("ratio", 0.5), 0, name=node.name)

    def handleFlatten(self, ff, node): return ff.flat(self._in(node, 0), name=node.name)

    def handleGemm(self, ff, node):
        w = self.inits[node.input[1]]
        a = _attrs(node)
        out_dim = int(w.dims[0]) if a.get("transB", 0) else int(w.dims[1])
        return ff.dense(self._in(node, 0), out_dim, use_bias=len(node.input) > 2, name=node.name)

    handleDense = handleGemm

    def handlePad(self, ff, node):
        pads = _attrs(node).get("pads")
        if pads is None and len(node.input) > 1:
            pads = [int(v) for v in self._const(node.input[1])]
        if pads and any(pads):
            raise NotImplementedError("Pad with non-zero padding (fold it into the following Conv/Pool)")
        return self._in(node, 0)

    def handleSoftmax(self, ff, node):
        return ff.softmax(self._in(node, 0), _attrs(node).get("axis", -1), name=node.name)

    def handleReshape(self, ff, node):
        x = self._in(node, 0)
        shape = [int(v) for v in self._const(node.input[1])]
        n = 1
        for d in x.dims:
            n *= d
        shape = [x.dims[i] if s == 0 else s for i, s in enumerate(shape)]
        if -1 in shape:
            known = 1
            for s in shape:
                known *= s if s != -1 else 1
            shape[shape.index(-1)] = n // known
        return ff.reshape(x, shape, name=node.name)

    def handleTranspose(self, ff, node):
        x = self._in(node, 0)
        perm = _attrs(node).get("perm", list(reversed(range(x.num_dims))))
        return ff.transpose(x, perm, name=node.name)

    def handleUnsqueeze(self, ff, node):
        x = self.symbols[node.input[0]]
        axes = _attrs(node).get("axes")
        if axes is None:
            axes = [int(v) for v in self._const(node.input[1])]
        if isinstance(x, np.ndarray):
            return np.expand_dims(x, tuple(axes))
        dims = list(x.dims)
        for ax in sorted(axes):
            dims.insert(ax % (len(dims) + 1), 1)
        return ff.reshape(x, dims, name=node.name)

    def handleConstant(self, ff, node):
        a = _attrs(node)
        v = a.get("value", a.get("value_float", a.get("value_int", a.get("value_ints", a.get("value_floats")))))
        return np.asarray(v)

    def handleRange(self, ff, node):
        start, limit, delta = (self._const(i) for i in node.input[:3])
        return np.arange(start.item(), limit.item(), delta.item())

    # ---- driver
    def apply(self, ffmodel: FFModel, input_dict: Dict[str, Tensor]) -> List[Tensor]:
        self.symbols = dict(input_dict)
        for node in self.model.graph.node:
            h = getattr(self, "handle" + node.op_type, None)
            if h is None:
                raise NotImplementedError(f"ONNX operator {node.op_type} has no importer")
            out = h(ffmodel, node)
            if isinstance(out, (list, tuple)):
                for name, v in zip(node.output, out):
                    self.symbols[name] = v
            else:
                self.symbols[node.output[0]] = out
        return [self.symbols[o.name] for o in self.model.graph.output if isinstance(self.symbols.get(o.name), Tensor)]


class ONNXModelKeras(ONNXModel):
    """Models exported from Keras carry Dense weights as [in, out] MatMul operands and wrap them in
    Transpose / Reshape nodes; those are folded into ``dense`` here."""

    def handleMatMul(self, ff, node):
        if node.input[1] in self.inits:
            w = self.inits[node.input[1]]
            return ff.dense(self._in(node, 0), int(w.dims[-1]), use_bias=False, name=node.name)
        return super().handleMatMul(ff, node)

    def handleTranspose(self, ff, node):
        if node.input[0] in self.inits:  # a transposed weight: keep the initializer, Dense handles the layout
            self.inits[node.output[0]] = self.inits[node.input[0]]
            return np.zeros(0)
        return super().handleTranspose(ff, node)

    def handleAdd(self, ff, node):
        # bias add after a folded Dense: the bias is an initializer
        for i in (0, 1):
            if node.input[i] in self.inits:
                x = self._in(node, 1 - i)
                b = self.inits[node.input[i]]
                bias = Tensor(ff, ff.builder.create_weight([int(d) for d in b.dims], "FLOAT", {"type": "zero", "value": {}}, True,
                                                           f"{node.name}.bias"))
                tgt = list(x.dims)
                bb = ff._t(ff.builder.broadcast(bias.value, tgt, f"{node.name}.bcast")) if tuple(bias.dims) != tuple(tgt) else bias
                return ff.add(x, bb, name=node.name)
        return super().handleAdd(ff, node)
