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


def _typed(l):
    V, P, I, L, D = Value, POINTER(Value), c_int, c_int64, c_double
    sigs = {
        "ffc_builder_pool2d": [c_void_p, V, I, I, I, I, I, I, c_char_p, c_char_p, c_char_p, P],
        "ffc_builder_conv2d": [c_void_p, V, L, I, I, I, I, I, I, c_char_p, I, I, c_char_p, P],
        "ffc_builder_batch_norm": [c_void_p, V, I, c_char_p, D, D, c_char_p, P],
        "ffc_builder_layer_norm": [c_void_p, V, POINTER(I), I, I, D, c_char_p, P],
        "ffc_builder_embedding": [c_void_p, V, L, L, c_char_p, c_char_p, c_char_p, P],
        "ffc_builder_multihead_attention": [c_void_p, V, V, V, L, L, L, L, D, I, I, I, c_char_p, P],
        "ffc_builder_batch_matmul": [c_void_p, V, V, c_char_p, P],
        "ffc_builder_dropout": [c_void_p, V, D, ctypes.c_uint64, c_char_p, P],
        "ffc_builder_cast": [c_void_p, V, c_char_p, c_char_p, P],
        "ffc_builder_concat": [c_void_p, P, I, I, c_char_p, P],
        "ffc_builder_split": [c_void_p, V, POINTER(L), I, I, c_char_p, P],
        "ffc_builder_flat": [c_void_p, V, c_char_p, P],
        "ffc_builder_transpose": [c_void_p, V, POINTER(I), I, c_char_p, P],
        "ffc_builder_reshape": [c_void_p, V, POINTER(L), I, c_char_p, P],
        "ffc_builder_reverse": [c_void_p, V, I, c_char_p, P],
        "ffc_builder_gather": [c_void_p, V, V, I, c_char_p, P],
        "ffc_builder_top_k": [c_void_p, V, I, I, c_char_p, P, P],
        "ffc_builder_reduce": [c_void_p, c_char_p, V, POINTER(I), I, I, c_char_p, P],
        "ffc_builder_broadcast": [c_void_p, V, POINTER(L), I, c_char_p, P],
        "ffc_builder_parallel_partition": [c_void_p, V, I, I, c_char_p, P],
        "ffc_builder_parallel_combine": [c_void_p, V, I, I, c_char_p, P],
        "ffc_builder_parallel_replicate": [c_void_p, V, I, c_char_p, P],
        "ffc_builder_parallel_reduce": [c_void_p, V, I, c_char_p, P],
        "ffc_builder_value_degrees": [c_void_p, V, POINTER(I), I, POINTER(I), POINTER(I), POINTER(I)],
        "ffc_graph_estimate": [c_void_p, I, I, POINTER(D)],
    }
    for name, args in sigs.items():
        getattr(l, name).argtypes = args
    l.ffc_builder_create_parallel.restype = c_void_p
    l.ffc_graph_sp_decomposition.restype = c_void_p
    l.ffc_graph_sp_decomposition.argtypes = [c_void_p]
    return l


def _shape(l, b, v):
    dims, nd = (c_int64 * 8)(), c_int()
    assert l.ffc_builder_value_shape(b, v, dims, 8, byref(nd)) == 0, l.ffc_last_error()
    return list(dims[:nd.value])


def test_typed_layer_functions_build_a_convolution_stack_and_a_transformer_block():
    l = _typed(_lib())
    b = l.ffc_builder_create()
    x, t = Value(), Value()
    assert l.ffc_builder_create_input(b, (c_int64 * 4)(8, 3, 32, 32), 4, b"FLOAT", b"image", byref(x)) == 0
    assert l.ffc_builder_conv2d(b, x, 16, 3, 3, 1, 1, 1, 1, b"RELU", 1, 1, b"conv", byref(t)) == 0 and _shape(l, b, t) == [8, 16, 32, 32]
    assert l.ffc_builder_batch_norm(b, t, 1, b"RELU", 1e-5, 0.1, b"bn", byref(t)) == 0
    assert l.ffc_builder_pool2d(b, t, 2, 2, 2, 2, 0, 0, b"MAX", None, b"pool", byref(t)) == 0 and _shape(l, b, t) == [8, 16, 16, 16]
    assert l.ffc_builder_flat(b, t, b"flat", byref(t)) == 0 and _shape(l, b, t) == [8, 4096]
    halves = (Value * 2)()
    assert l.ffc_builder_split(b, t, (c_int64 * 2)(1024, 3072), 2, 1, b"split", halves) == 0 and _shape(l, b, halves[1]) == [8, 3072]
    assert l.ffc_builder_concat(b, halves, 2, 1, b"cat", byref(t)) == 0 and _shape(l, b, t) == [8, 4096]
    assert l.ffc_builder_reshape(b, t, (c_int64 * 3)(8, 64, 64), 3, b"seq", byref(t)) == 0
    q = Value()
    assert l.ffc_builder_layer_norm(b, t, (c_int * 1)(-1), 1, 1, 1e-5, b"ln", byref(q)) == 0
    a = Value()
    assert l.ffc_builder_multihead_attention(b, q, q, q, 64, 4, 0, 0, 0.1, 1, 0, 0, b"attn", byref(a)) == 0 and _shape(l, b, a) == [8, 64, 64]
    assert l.ffc_builder_dropout(b, a, 0.1, 7, b"drop", byref(a)) == 0
    tr = Value()
    assert l.ffc_builder_transpose(b, a, (c_int * 3)(0, 2, 1), 3, b"tr", byref(tr)) == 0
    mm = Value()
    assert l.ffc_builder_batch_matmul(b, a, tr, b"bmm", byref(mm)) == 0 and _shape(l, b, mm) == [8, 64, 64]
    red = Value()
    assert l.ffc_builder_reduce(b, b"REDUCE_MEAN", mm, (c_int * 1)(2), 1, 0, b"mean", byref(red)) == 0 and _shape(l, b, red) == [8, 64]
    vals, idx = Value(), Value()
    assert l.ffc_builder_top_k(b, red, 5, 1, b"topk", byref(vals), byref(idx)) == 0 and _shape(l, b, idx) == [8, 5]
    rv = Value()
    assert l.ffc_builder_reverse(b, red, 1, b"rev", byref(rv)) == 0 and _shape(l, b, rv) == [8, 64]
    c64 = Value()
    assert l.ffc_builder_cast(b, rv, b"DOUBLE", b"cast", byref(c64)) == 0
    ids, emb = Value(), Value()
    assert l.ffc_builder_create_input(b, (c_int64 * 2)(8, 10), 2, b"INT32", b"ids", byref(ids)) == 0
    assert l.ffc_builder_embedding(b, ids, 100, 32, b"SUM", b"FLOAT", b"emb", byref(emb)) == 0 and _shape(l, b, emb) == [8, 32]
    g = l.ffc_builder_graph(b)
    types = [n["type"] for n in core.Graph.from_v1(_json(l, g)).nodes()]
    for want in ("CONV2D", "BATCHNORM", "POOL2D", "FLAT", "SPLIT", "CONCAT", "LAYERNORM", "MULTIHEAD_ATTENTION", "BATCHMATMUL", "TOPK", "EMBEDDING"):
        assert want in types, want
    p = l.ffc_graph_sp_decomposition(g)
    assert p, l.ffc_last_error()
    tree = json.loads(ctypes.string_at(p).decode())
    l.ffc_string_free(p)
    assert tree["type"] in ("series", "parallel")
    l.ffc_graph_destroy(g)
    l.ffc_builder_destroy(b)


def test_parallel_builder_through_the_c_api():
    l = _typed(_lib())
    b = l.ffc_builder_create_parallel()
    x, p, h, y = Value(), Value(), Value(), Value()
    assert l.ffc_builder_create_input(b, (c_int64 * 2)(16, 32), 2, b"FLOAT", b"x", byref(x)) == 0
    assert l.ffc_builder_parallel_partition(b, x, 0, 4, b"part", byref(p)) == 0
    assert l.ffc_builder_dense(b, p, 64, None, 1, b"fc", byref(h)) == 0
    deg, nd, sd, cd = (c_int * 4)(), c_int(), c_int(), c_int()
    assert l.ffc_builder_value_degrees(b, h, deg, 4, byref(nd), byref(sd), byref(cd)) == 0
    assert list(deg[:nd.value]) == [4, 1] and sd.value == 1 and cd.value == 1
    assert l.ffc_builder_parallel_combine(b, h, 0, 4, b"comb", byref(y)) == 0
    assert l.ffc_builder_value_degrees(b, y, deg, 4, byref(nd), byref(sd), byref(cd)) == 0 and list(deg[:nd.value]) == [1, 1]
    # a Reduction needs partial sums to reduce
    assert l.ffc_builder_parallel_reduce(b, y, 2, b"bad", byref(y)) != 0 and l.ffc_last_error()
    g = l.ffc_builder_graph(b)
    pcg = core.Graph.from_v1(_json(l, g, 1))
    types = [n["type"] for n in pcg.nodes()]
    assert "REPARTITION" in types and "COMBINE" in types and "REPLICATE" in types   # the weights were replicated for the 4 shards
    ms = c_double()
    assert l.ffc_graph_estimate(g, 1, 4, byref(ms)) == 0 and ms.value > 0, l.ffc_last_error()
    # on a machine without enough devices there is no mapping
    assert l.ffc_graph_estimate(g, 1, 2, byref(ms)) != 0
    l.ffc_graph_destroy(g)
    l.ffc_builder_destroy(b)
    # the unparallel builder refuses parallel operators
    b2 = l.ffc_builder_create()
    assert l.ffc_builder_create_input(b2, (c_int64 * 2)(16, 32), 2, b"FLOAT", b"x", byref(x)) == 0
    assert l.ffc_builder_parallel_replicate(b2, x, 2, b"r", byref(y)) != 0
    l.ffc_builder_destroy(b2)


def test_graph_inspection_and_files_through_the_c_api(tmp_path):
    l = _lib()
    I, L = c_int, c_int64
    l.ffc_graph_save_file.argtypes = [c_void_p, c_char_p, I, I]
    l.ffc_graph_load_file.restype = c_void_p
    l.ffc_graph_load_file.argtypes = [c_char_p]
    l.ffc_graph_node_ids.argtypes = [c_void_p, POINTER(I), I, POINTER(I)]
    for f in ("ffc_graph_node_op_type", "ffc_graph_node_name", "ffc_graph_node_attrs_json", "ffc_graph_node_view_json"):
        getattr(l, f).restype = c_void_p
        getattr(l, f).argtypes = [c_void_p, I]
    l.ffc_graph_value_shape.argtypes = [c_void_p, Value, POINTER(L), I, POINTER(I)]
    l.ffc_graph_value_dtype.restype = c_char_p
    l.ffc_graph_value_dtype.argtypes = [c_void_p, Value]
    l.ffc_graph_value_create_grad.argtypes = [c_void_p, Value, POINTER(I)]
    l.ffc_datatype_size.argtypes = [c_char_p]
    l.ffc_builder_value_dtype.restype = c_char_p
    l.ffc_builder_value_dtype.argtypes = [c_void_p, Value]

    def text(p):
        assert p, l.ffc_last_error()
        s = ctypes.string_at(p).decode()
        l.ffc_string_free(p)
        return s

    assert [l.ffc_datatype_size(n) for n in (b"BOOL", b"INT32", b"INT64", b"HALF", b"BFLOAT16", b"FLOAT", b"DOUBLE")] == [1, 4, 8, 2, 2, 4, 8]
    assert l.ffc_datatype_size(b"QUADRUPLE") == -1 and l.ffc_last_error()

    ref = core.build_model("mlp", {"batch_size": 8})
    g = l.ffc_model_build(b"mlp", b'{"batch_size": 8}')
    n = c_int()
    assert l.ffc_graph_node_ids(g, None, 0, byref(n)) == 0 and n.value == len(ref.nodes())
    ids = (I * n.value)()
    assert l.ffc_graph_node_ids(g, ids, n.value, byref(n)) == 0 and list(ids) == list(ref.topological_order())
    by_id = {nd["id"]: nd for nd in ref.nodes()}
    slot_out = l.ffc_slot_from_name(b"OUTPUT")
    for nid in ids:
        nd = by_id[nid]
        assert text(l.ffc_graph_node_op_type(g, nid)) == nd["type"] and text(l.ffc_graph_node_name(g, nid)) == nd["name"]
        assert json.loads(text(l.ffc_graph_node_attrs_json(g, nid))) == nd["attrs"]
        dims, nd_ = (L * 8)(), c_int()
        v = Value(nid, slot_out)
        assert l.ffc_graph_value_shape(g, v, dims, 8, byref(nd_)) == 0
        sh = ref.shape((nid, "OUTPUT"))
        assert list(dims[:nd_.value]) == list(sh.sizes) and l.ffc_graph_value_dtype(g, v).decode() == sh.dtype
        cg = c_int(-1)
        assert l.ffc_graph_value_create_grad(g, v, byref(cg)) == 0 and cg.value in (0, 1)
    assert l.ffc_graph_node_op_type(g, 10 ** 6) is None and l.ffc_last_error()
    assert l.ffc_graph_node_view_json(g, ids[0]) is None and b"view" in l.ffc_last_error()

    # a mapped graph: every node has a view; the file round trip keeps it
    mapped, ms = c_void_p(), c_double()
    l.ffc_graph_optimize.argtypes = [c_void_p, c_int, c_int, c_char_p, c_int, c_double, c_uint, POINTER(c_void_p), POINTER(c_double)]
    assert l.ffc_graph_optimize(g, 1, 2, b"data_parallel", 0, 1.05, 0, byref(mapped), byref(ms)) == 0, l.ffc_last_error()
    path = str(tmp_path / "strategy.json").encode()
    assert l.ffc_graph_save_file(mapped, path, 1, 1) == 0, l.ffc_last_error()
    back = l.ffc_graph_load_file(path)
    assert back and l.ffc_graph_num_nodes(back) == l.ffc_graph_num_nodes(mapped)
    assert l.ffc_graph_node_ids(back, None, 0, byref(n)) == 0
    ids2 = (I * n.value)()
    l.ffc_graph_node_ids(back, ids2, n.value, byref(n))
    views = [json.loads(text(l.ffc_graph_node_view_json(back, i))) for i in ids2]
    assert all("start" in v and "dimensions" in v for v in views)
    assert any(len(v["dimensions"]) == 1 for v in views)        # the batch-parallel operators run over a 1-d view of 2 devices
    assert l.ffc_graph_load_file(str(tmp_path / "missing.json").encode()) is None and b"cannot open" in l.ffc_last_error()
    assert l.ffc_graph_save_file(mapped, str(tmp_path / "no_dir" / "x.json").encode(), 1, 1) != 0
    for h in (g, mapped, back):
        l.ffc_graph_destroy(h)
    b = l.ffc_builder_create()
    x = Value()
    assert l.ffc_builder_create_input(b, (c_int64 * 2)(4, 4), 2, b"INT32", b"ids", byref(x)) == 0
    assert l.ffc_builder_value_dtype(b, x) == b"INT32"
    l.ffc_builder_destroy(b)
