"""High-level Python API over the C interface of the compiler core (``csrc/core/ffi.h``).

A ``ComputationGraph`` owns a C builder handle; ``Tensor`` objects name values of it and build layers through
methods and arithmetic operators; the graph serialises to the v1 JSON, renders to dot and goes through the strategy
search -- all through ``ffc_*`` calls, so the same flow is available to any language that can call C.

Counterpart of the reference's cffi-based package (bindings/python/python/flexflow/pcg/{raw,high_level}.py over
lib/pcg/ffi/include/flexflow/pcg.h and lib/compiler/ffi/include/flexflow/compiler.h), whose C side is stubs; here the
C functions are implemented and loaded with ctypes from the core's shared object.
"""
from __future__ import annotations

import ctypes
import json
from ctypes import POINTER, byref, c_char_p, c_double, c_int, c_int64, c_uint, c_void_p
from typing import List, Optional, Sequence, Tuple, Union

from .. import _ffcore as core


class _Value(ctypes.Structure):
    _fields_ = [("node", c_int), ("slot", c_int)]


class FFIError(RuntimeError):
    pass


_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        l = ctypes.CDLL(core.__file__)
        l.ffc_last_error.restype = c_char_p
        l.ffc_builder_create.restype = c_void_p
        l.ffc_builder_destroy.argtypes = [c_void_p]
        l.ffc_builder_graph.restype = c_void_p
        l.ffc_builder_graph.argtypes = [c_void_p]
        l.ffc_builder_create_input.argtypes = [c_void_p, POINTER(c_int64), c_int, c_char_p, c_char_p, POINTER(_Value)]
        l.ffc_builder_create_weight.argtypes = [c_void_p, POINTER(c_int64), c_int, c_char_p, c_char_p, c_char_p, POINTER(_Value)]
        l.ffc_builder_dense.argtypes = [c_void_p, _Value, c_int64, c_char_p, c_int, c_char_p, POINTER(_Value)]
        l.ffc_builder_conv2d.argtypes = [c_void_p, _Value, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_char_p, c_int, c_int,
                                         c_char_p, POINTER(_Value)]
        l.ffc_builder_unary.argtypes = [c_void_p, c_char_p, _Value, c_int, c_double, c_char_p, POINTER(_Value)]
        l.ffc_builder_binary.argtypes = [c_void_p, c_char_p, _Value, _Value, c_char_p, POINTER(_Value)]
        l.ffc_builder_softmax.argtypes = [c_void_p, _Value, c_int, c_char_p, POINTER(_Value)]
        l.ffc_builder_value_shape.argtypes = [c_void_p, _Value, POINTER(c_int64), c_int, POINTER(c_int)]
        l.ffc_builder_add_layer.argtypes = [c_void_p, c_char_p, c_char_p, POINTER(_Value), POINTER(c_char_p), c_int, c_char_p,
                                            POINTER(_Value), c_int, POINTER(c_int)]
        l.ffc_model_build.restype = c_void_p
        l.ffc_model_build.argtypes = [c_char_p, c_char_p]
        l.ffc_graph_from_json.restype = c_void_p
        l.ffc_graph_from_json.argtypes = [c_char_p]
        l.ffc_graph_to_json.restype = c_void_p
        l.ffc_graph_to_json.argtypes = [c_void_p, c_int, c_int]
        l.ffc_graph_to_dot.restype = c_void_p
        l.ffc_graph_to_dot.argtypes = [c_void_p]
        l.ffc_graph_num_nodes.argtypes = [c_void_p]
        l.ffc_graph_destroy.argtypes = [c_void_p]
        l.ffc_string_free.argtypes = [c_void_p]
        l.ffc_graph_optimize.argtypes = [c_void_p, c_int, c_int, c_char_p, c_int, c_double, c_uint, POINTER(c_void_p), POINTER(c_double)]
        _LIB = l
    return _LIB


def _check(rc: int, what: str):
    if rc != 0:
        raise FFIError(f"{what}: {(_lib().ffc_last_error() or b'').decode()}")


def _b(s: Optional[str]):
    return None if s is None else s.encode()


def _take_string(p) -> str:
    if not p:
        raise FFIError((_lib().ffc_last_error() or b"").decode())
    s = ctypes.string_at(p).decode()
    _lib().ffc_string_free(p)
    return s


class Graph:
    """An immutable graph handle (computation graph or mapped parallel computation graph)."""

    def __init__(self, handle):
        if not handle:
            raise FFIError((_lib().ffc_last_error() or b"").decode())
        self._h = handle

    @classmethod
    def from_json(cls, text: str) -> "Graph":
        return cls(_lib().ffc_graph_from_json(text.encode()))

    @classmethod
    def from_model(cls, name: str, config: Optional[dict] = None) -> "Graph":
        return cls(_lib().ffc_model_build(name.encode(), json.dumps(config or {}).encode()))

    def to_json(self, parallel: bool = False, indent: int = -1) -> str:
        return _take_string(_lib().ffc_graph_to_json(self._h, int(parallel), indent))

    def to_dot(self) -> str:
        return _take_string(_lib().ffc_graph_to_dot(self._h))

    @property
    def num_nodes(self) -> int:
        return _lib().ffc_graph_num_nodes(self._h)

    def optimize(self, gpus_per_node: int, num_nodes: int = 1, algorithm: str = "unity", budget: int = 0, alpha: float = 1.05,
                 seed: int = 0) -> Tuple["Graph", float]:
        """Strategy search (flexflow_computation_graph_optimize): the mapped parallel graph and its estimated step time."""
        out, ms = c_void_p(), c_double()
        _check(_lib().ffc_graph_optimize(self._h, num_nodes, gpus_per_node, algorithm.encode(), budget, alpha, seed, byref(out),
                                         byref(ms)), "optimize")
        return Graph(out.value), ms.value

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _LIB is not None:
            _LIB.ffc_graph_destroy(h)


Number = Union[int, float]


class Tensor:
    """A value of a ComputationGraph under construction."""

    def __init__(self, graph: "ComputationGraph", value: _Value):
        self.graph = graph
        self._v = value

    @property
    def shape(self) -> List[int]:
        dims = (c_int64 * 8)()
        n = c_int()
        _check(_lib().ffc_builder_value_shape(self.graph._b, self._v, dims, 8, byref(n)), "value_shape")
        return [int(dims[i]) for i in range(n.value)]

    # ---- unary
    def _unary(self, op: str, scalar: Optional[Number] = None, name: str = "") -> "Tensor":
        out = _Value()
        _check(_lib().ffc_builder_unary(self.graph._b, op.encode(), self._v, int(scalar is not None), float(scalar or 0.0), _b(name),
                                        byref(out)), op)
        return Tensor(self.graph, out)

    def exp(self, name=""): return self._unary("EXP", name=name)
    def relu(self, name=""): return self._unary("RELU", name=name)
    def sigmoid(self, name=""): return self._unary("SIGMOID", name=name)
    def tanh(self, name=""): return self._unary("TANH", name=name)
    def gelu(self, name=""): return self._unary("GELU", name=name)
    def elu(self, name=""): return self._unary("ELU", name=name)
    def rsqrt(self, name=""): return self._unary("RSQRT", name=name)
    def sin(self, name=""): return self._unary("SIN", name=name)
    def cos(self, name=""): return self._unary("COS", name=name)
    def identity(self, name=""): return self._unary("IDENTITY", name=name)
    def pow(self, exponent: Number, name=""): return self._unary("POW", exponent, name)
    def scalar_multiply(self, s: Number, name=""): return self._unary("SCALAR_MULTIPLY", s, name)
    def scalar_add(self, s: Number, name=""): return self._unary("SCALAR_ADD", s, name)
    def scalar_sub(self, s: Number, name=""): return self._unary("SCALAR_SUB", s, name)
    def scalar_truediv(self, s: Number, name=""): return self._unary("SCALAR_TRUE_DIV", s, name)

    # ---- binary
    def _binary(self, op: str, other: "Tensor", name: str = "") -> "Tensor":
        if other.graph is not self.graph:
            raise ValueError("operands belong to different graphs")
        out = _Value()
        _check(_lib().ffc_builder_binary(self.graph._b, op.encode(), self._v, other._v, _b(name), byref(out)), op)
        return Tensor(self.graph, out)

    def add(self, o, name=""): return self._binary("EW_ADD", o, name)
    def subtract(self, o, name=""): return self._binary("EW_SUB", o, name)
    def multiply(self, o, name=""): return self._binary("EW_MUL", o, name)
    def divide(self, o, name=""): return self._binary("EW_DIV", o, name)
    def max(self, o, name=""): return self._binary("EW_MAX", o, name)
    def min(self, o, name=""): return self._binary("EW_MIN", o, name)

    def __add__(self, o): return self.add(o) if isinstance(o, Tensor) else self.scalar_add(o)
    def __radd__(self, o): return self.scalar_add(o)
    def __sub__(self, o): return self.subtract(o) if isinstance(o, Tensor) else self.scalar_sub(o)
    def __mul__(self, o): return self.multiply(o) if isinstance(o, Tensor) else self.scalar_multiply(o)
    def __rmul__(self, o): return self.scalar_multiply(o)
    def __truediv__(self, o): return self.divide(o) if isinstance(o, Tensor) else self.scalar_truediv(o)

    # ---- layers
    def dense(self, out_channels: int, activation: Optional[str] = None, use_bias: bool = True, name: str = "") -> "Tensor":
        out = _Value()
        _check(_lib().ffc_builder_dense(self.graph._b, self._v, out_channels, _b(activation), int(use_bias), _b(name), byref(out)), "dense")
        return Tensor(self.graph, out)

    def conv2d(self, out_channels: int, kernel: Tuple[int, int], stride=(1, 1), padding=(0, 0), activation: Optional[str] = None,
               groups: int = 1, use_bias: bool = True, name: str = "") -> "Tensor":
        out = _Value()
        _check(_lib().ffc_builder_conv2d(self.graph._b, self._v, out_channels, kernel[0], kernel[1], stride[0], stride[1], padding[0],
                                         padding[1], _b(activation), groups, int(use_bias), _b(name), byref(out)), "conv2d")
        return Tensor(self.graph, out)

    def softmax(self, dim: int = -1, name: str = "") -> "Tensor":
        out = _Value()
        _check(_lib().ffc_builder_softmax(self.graph._b, self._v, dim, _b(name), byref(out)), "softmax")
        return Tensor(self.graph, out)


class ComputationGraph:
    """Builds a computation graph layer by layer through the C builder."""

    def __init__(self):
        self._b = _lib().ffc_builder_create()
        if not self._b:
            raise FFIError("could not create a builder")

    def create_input(self, dims: Sequence[int], dtype: str = "FLOAT", name: str = "") -> Tensor:
        arr = (c_int64 * len(dims))(*dims)
        out = _Value()
        _check(_lib().ffc_builder_create_input(self._b, arr, len(dims), dtype.encode(), _b(name), byref(out)), "create_input")
        return Tensor(self, out)

    def create_weight(self, dims: Sequence[int], dtype: str = "FLOAT", initializer: Optional[dict] = None, name: str = "") -> Tensor:
        arr = (c_int64 * len(dims))(*dims)
        out = _Value()
        init = None if initializer is None else json.dumps(initializer).encode()
        _check(_lib().ffc_builder_create_weight(self._b, arr, len(dims), dtype.encode(), init, _b(name), byref(out)), "create_weight")
        return Tensor(self, out)

    def add_layer(self, op_type: str, attrs: dict, inputs: Sequence[Tuple[str, Tensor]], name: str = "") -> List[Tensor]:
        """Any operator by name: `inputs` are (slot name, tensor) pairs; missing weights get default initializers."""
        n = len(inputs)
        vals = (_Value * n)(*[t._v for _, t in inputs])
        slots = (c_char_p * n)(*[s.encode() for s, _ in inputs])
        outs = (_Value * 8)()
        count = c_int()
        _check(_lib().ffc_builder_add_layer(self._b, op_type.encode(), json.dumps(attrs).encode(), vals, slots, n, _b(name), outs, 8,
                                            byref(count)), op_type)
        return [Tensor(self, _Value(outs[i].node, outs[i].slot)) for i in range(count.value)]

    def graph(self) -> Graph:
        """A snapshot of what has been built."""
        return Graph(_lib().ffc_builder_graph(self._b))

    def to_json(self, indent: int = -1) -> str:
        return self.graph().to_json(indent=indent)

    def __del__(self):
        b, self._b = getattr(self, "_b", None), None
        if b and _LIB is not None:
            _LIB.ffc_builder_destroy(b)
