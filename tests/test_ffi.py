"""The C interface of the compiler core, driven through ctypes."""
import ctypes
import json
from ctypes import POINTER, byref, c_char_p, c_double, c_int, c_int64, c_uint, c_void_p

from flexflow_train_b200 import _ffcore as core


class Value(ctypes.Structure):
    _fields_ = [("node", c_int), ("slot", c_int)]


def _lib():
    l = ctypes.CDLL(core.__file__)
    l.ffc_last_error.restype = c_char_p
    l.ffc_builder_create.restype = c_void_p
    l.ffc_builder_graph.restype = c_void_p
    l.ffc_builder_graph.argtypes = [c_void_p]
    l.ffc_model_build.restype = c_void_p
    l.ffc_model_build.argtypes = [c_char_p, c_char_p]
    l.ffc_graph_from_json.restype = c_void_p
    l.ffc_graph_from_json.argtypes = [c_char_p]
    l.ffc_graph_to_json.restype = c_void_p
    l.ffc_graph_to_json.argtypes = [c_void_p, c_int, c_int]
    l.ffc_graph_num_nodes.argtypes = [c_void_p]
    l.ffc_graph_destroy.argtypes = [c_void_p]
    l.ffc_string_free.argtypes = [c_void_p]
    l.ffc_builder_destroy.argtypes = [c_void_p]
    l.ffc_builder_create_input.argtypes = [c_void_p, POINTER(c_int64), c_int, c_char_p, c_char_p, POINTER(Value)]
    l.ffc_builder_dense.argtypes = [c_void_p, Value, c_int64, c_char_p, c_int, c_char_p, POINTER(Value)]
    l.ffc_builder_binary.argtypes = [c_void_p, c_char_p, Value, Value, c_char_p, POINTER(Value)]
    l.ffc_builder_softmax.argtypes = [c_void_p, Value, c_int, c_char_p, POINTER(Value)]
    l.ffc_builder_value_shape.argtypes = [c_void_p, Value, POINTER(c_int64), c_int, POINTER(c_int)]
    l.ffc_builder_add_layer.argtypes = [c_void_p, c_char_p, c_char_p, POINTER(Value), POINTER(c_char_p), c_int, c_char_p, POINTER(Value),
                                        c_int, POINTER(c_int)]
    l.ffc_graph_optimize.argtypes = [c_void_p, c_int, c_int, c_char_p, c_int, c_double, c_uint, POINTER(c_void_p), POINTER(c_double)]
    return l


def _json(l, g, parallel=0):
    p = l.ffc_graph_to_json(g, parallel, -1)
    s = ctypes.string_at(p).decode()
    l.ffc_string_free(p)
    return s


def test_build_serialise_and_optimize_through_the_c_api():
    l = _lib()
    b = l.ffc_builder_create()
    x, h, y, z, out = Value(), Value(), Value(), Value(), Value()
    dims = (c_int64 * 2)(16, 32)
    assert l.ffc_builder_create_input(b, dims, 2, b"FLOAT", b"x", byref(x)) == 0
    assert l.ffc_builder_dense(b, x, 64, b"RELU", 1, b"fc1", byref(h)) == 0
    assert l.ffc_builder_dense(b, h, 64, None, 1, b"fc2", byref(y)) == 0
    assert l.ffc_builder_binary(b, b"EW_ADD", h, y, b"res", byref(z)) == 0
    outs, n_out = (Value * 2)(), c_int()
    slots = (c_char_p * 1)(b"INPUT")
    assert l.ffc_builder_add_layer(b, b"DROPOUT", b'{"rate": 0.1, "seed": 0}', byref(z), slots, 1, b"drop", outs, 2, byref(n_out)) == 0
    assert n_out.value == 1
    assert l.ffc_builder_softmax(b, outs[0], -1, b"prob", byref(out)) == 0
    shape, nd = (c_int64 * 4)(), c_int()
    assert l.ffc_builder_value_shape(b, out, shape, 4, byref(nd)) == 0 and list(shape[:nd.value]) == [16, 64]
    # errors are reported, not thrown across the boundary
    assert l.ffc_builder_binary(b, b"EW_ADD", x, y, b"bad", byref(z)) != 0
    assert b"shape" in l.ffc_last_error().lower() or len(l.ffc_last_error()) > 0
    g = l.ffc_builder_graph(b)
    text = _json(l, g)
    g2 = l.ffc_graph_from_json(text.encode())
    assert l.ffc_graph_num_nodes(g2) == l.ffc_graph_num_nodes(g)
    assert core.Graph.from_v1(text).signature() == core.Graph.from_v1(_json(l, g2)).signature()
    # optimize for 4 GPUs: a mapped PCG with parallel operators comes back
    mapped, ms = c_void_p(), c_double()
    assert l.ffc_graph_optimize(g, 1, 4, b"unity", 2, 1.05, 0, byref(mapped), byref(ms)) == 0, l.ffc_last_error()
    pcg = core.Graph.from_v1(_json(l, mapped, 1))
    assert pcg.is_mapped() and ms.value > 0
    for h_ in (g, g2, mapped):
        l.ffc_graph_destroy(h_)
    l.ffc_builder_destroy(b)
    m = l.ffc_model_build(b"mlp", b'{"batch_size": 8}')
    assert l.ffc_graph_num_nodes(m) == len(core.build_model("mlp", {"batch_size": 8}).nodes())
    l.ffc_graph_destroy(m)
    assert l.ffc_model_build(b"no_such_model", None) is None and l.ffc_last_error()
