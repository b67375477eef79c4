"""Parallel shape inference against hand-computed golden cases: for each operator the four ways an input can be
parallel (sample dim, contracted / channel dim, replicated input, partial sums) and what they do to the output, the
weights and the bias.  The cases and sizes follow lib/op-attrs/test/src/op-attrs/ops/{conv_2d,linear,attention,embedding,
batch_norm,layer_norm,pool_2d,concat,softmax,element_binary,flat,cast,dropout}.cc."""
import pytest

from flexflow_train_b200 import _ffcore as c

PTS = c.ParallelTensorShape


def infer(op, attrs, inputs):
    r = c.infer_shapes(op, attrs, inputs)
    return dict(r["outputs"]), dict(r["weights"])


def par(sizes, degrees=None, sum_degree=1, copy_degree=1, dtype="FLOAT"):
    return PTS(list(sizes), dtype, list(degrees or [1] * len(sizes)), sum_degree, copy_degree)


def sig(s):
    return (list(s.sizes), list(s.degrees), s.sum_degree, s.discard_copy_degree)


CONV = {"out_channels": 4, "kernel_h": 3, "kernel_w": 2, "stride_h": 2, "stride_w": 2, "padding_h": 1, "padding_w": 1, "groups": 1,
        "use_bias": True}
CONV_IN, CONV_OUT, CONV_K = [8, 4, 11, 15], [8, 4, 6, 8], [4, 4, 3, 2]


@pytest.mark.parametrize("name,inp,out,kernel,bias", [
    #                 input (degrees, sum, copy)      output                    kernel                      bias
    ("unparallel",    ([1, 1, 1, 1], 1, 1), ([1, 1, 1, 1], 1, 1), ([1, 1, 1, 1], 1, 1), ([1], 1, 1)),
    ("data",          ([2, 1, 1, 1], 1, 1), ([2, 1, 1, 1], 1, 1), ([1, 1, 1, 1], 1, 2), ([1], 1, 2)),
    ("input channel", ([1, 2, 1, 1], 1, 1), ([1, 1, 1, 1], 2, 1), ([1, 2, 1, 1], 1, 1), ([1], 2, 1)),
    ("output channel", ([1, 1, 1, 1], 1, 2), ([1, 2, 1, 1], 1, 1), ([2, 1, 1, 1], 1, 1), ([2], 1, 1)),
    ("partial sums",  ([1, 1, 1, 1], 2, 1), ([1, 1, 1, 1], 2, 1), ([1, 1, 1, 1], 1, 2), ([1], 2, 1)),
])
def test_conv2d_parallel_shapes(name, inp, out, kernel, bias):
    o, w = infer("CONV2D", CONV, [("INPUT", par(CONV_IN, *inp))])
    assert sig(o["OUTPUT"]) == (CONV_OUT, *out), name
    assert sig(w["FILTER"]) == (CONV_K, *kernel), name
    assert sig(w["BIAS"]) == ([4], *bias), name


def test_conv2d_without_bias_has_no_bias_slot():
    o, w = infer("CONV2D", dict(CONV, use_bias=False), [("INPUT", par(CONV_IN))])
    assert set(w) == {"FILTER"} and o["OUTPUT"].sizes == CONV_OUT


LIN = {"out_channels": 16, "use_bias": True}


@pytest.mark.parametrize("name,inp,out,proj,bias", [
    # input [batch 12, extra 16, in 8]; projection [out 16, in 8]
    ("data + extra dim + partial sums", ([4, 2, 1], 2, 1), ([4, 2, 1], 2, 1), ([1, 1], 1, 16), ([1], 2, 8)),
    ("contracted dim",                  ([1, 1, 2], 3, 1), ([1, 1, 1], 6, 1), ([1, 2], 1, 3),  ([1], 6, 1)),
    ("output channels",                 ([1, 1, 1], 2, 4), ([1, 1, 4], 2, 1), ([4, 1], 1, 2),  ([4], 2, 1)),
])
def test_linear_parallel_shapes(name, inp, out, proj, bias):
    o, w = infer("LINEAR", LIN, [("INPUT", par([12, 16, 8], *inp))])
    assert sig(o["OUTPUT"]) == ([12, 16, 16], *out), name
    assert sig(w["WEIGHT"]) == ([16, 8], *proj), name
    assert sig(w["BIAS"]) == ([16], *bias), name


def test_attention_parallel_shapes():
    attrs = {"embed_dim": 32, "num_heads": 10, "kdim": 32, "vdim": 32, "dropout": 0.0, "bias": True, "add_bias_kv": False, "add_zero_attn": False}
    q = [40, 48, 32]  # batch, sequence, feature
    # data parallelism: batch cut 4 ways, weights replicated 4 ways
    o, w = infer("MULTIHEAD_ATTENTION", attrs, [(s, par(q, [4, 1, 1])) for s in ("QUERY", "KEY", "VALUE")])
    assert sig(o["OUTPUT"]) == ([40, 48, 32], [4, 1, 1], 1, 1)
    assert w["WEIGHT"].discard_copy_degree == 4 and w["WEIGHT"].sum_degree == 1
    # head parallelism: replicated inputs -> heads cut, partial sums out of the output projection
    o, w = infer("MULTIHEAD_ATTENTION", attrs, [(s, par(q, [1, 1, 1], 1, 2)) for s in ("QUERY", "KEY", "VALUE")])
    assert o["OUTPUT"].sum_degree == 2 and o["OUTPUT"].degrees == [1, 1, 1] and o["OUTPUT"].discard_copy_degree == 1
    assert max(w["WEIGHT"].degrees) == 2 and w["WEIGHT"].discard_copy_degree == 1
    # both at once
    o, w = infer("MULTIHEAD_ATTENTION", attrs, [(s, par(q, [4, 1, 1], 1, 2)) for s in ("QUERY", "KEY", "VALUE")])
    assert sig(o["OUTPUT"]) == ([40, 48, 32], [4, 1, 1], 2, 1)
    assert w["WEIGHT"].discard_copy_degree == 4 and max(w["WEIGHT"].degrees) == 2


def test_embedding_parallel_shapes():
    attrs = {"num_entries": 32, "out_channels": 128, "aggr": None, "data_type": "FLOAT"}
    ids = [12, 10]   # batch x features: the features dim becomes the output channels
    o, w = infer("EMBEDDING", attrs, [("INPUT", par(ids, dtype="INT32"))])
    assert o["OUTPUT"].sizes == [12, 128] and o["OUTPUT"].dtype == "FLOAT" and w["WEIGHT"].sizes == [32, 128]
    # data parallel: ids cut 4 ways -> output cut the same way, table replicated
    o, w = infer("EMBEDDING", attrs, [("INPUT", par(ids, [4, 1], dtype="INT32"))])
    assert sig(o["OUTPUT"]) == ([12, 128], [4, 1], 1, 1) and sig(w["WEIGHT"]) == ([32, 128], [1, 1], 1, 4)
    # replicated ids -> output channels cut, table cut along its channels
    o, w = infer("EMBEDDING", attrs, [("INPUT", par(ids, [1, 1], 1, 4, dtype="INT32"))])
    assert sig(o["OUTPUT"]) == ([12, 128], [1, 4], 1, 1) and sig(w["WEIGHT"]) == ([32, 128], [1, 4], 1, 1)
    # features cut -> every shard holds a partial sum of the output
    o, w = infer("EMBEDDING", attrs, [("INPUT", par(ids, [1, 2], dtype="INT32"))])
    assert sig(o["OUTPUT"]) == ([12, 128], [1, 1], 2, 1) and sig(w["WEIGHT"]) == ([32, 128], [1, 1], 1, 2)


def test_batch_norm_shapes_and_what_may_be_parallel():
    x = [12, 14, 16, 18]
    o, w = infer("BATCHNORM", {"relu": True, "affine": True, "eps": 1e-5, "momentum": 0.1}, [("INPUT", par(x))])
    assert o["OUTPUT"].sizes == x and w["GAMMA"].sizes == [14] and w["BETA"].sizes == [14]
    o, w = infer("BATCHNORM", {"relu": False, "affine": False, "eps": 1e-5, "momentum": 0.1}, [("INPUT", par(x))])
    assert not w
    # channel parallelism is the only kind that keeps the statistics local
    o, w = infer("BATCHNORM", {"relu": True, "affine": True, "eps": 1e-5, "momentum": 0.1}, [("INPUT", par(x, [1, 2, 1, 1]))])
    assert sig(o["OUTPUT"]) == (x, [1, 2, 1, 1], 1, 1) and sig(w["GAMMA"]) == ([14], [2], 1, 1)
    for bad in (par(x, [1, 1, 1, 1], 2, 1), par(x, [1, 1, 1, 1], 1, 2)):
        with pytest.raises(c.CoreError):
            infer("BATCHNORM", {"relu": True, "affine": True, "eps": 1e-5, "momentum": 0.1}, [("INPUT", bad)])


def test_layer_norm_shapes_and_what_may_be_parallel():
    x = [12, 14, 16, 18]
    attrs = {"axes": [1, 3], "elementwise_affine": True, "eps": 1e-5}
    o, w = infer("LAYERNORM", attrs, [("INPUT", par(x))])
    # gamma and beta have the extents of the normalised dims (what the kernels and PyTorch use; the reference's rule takes
    # the *other* dims, which would tie the weight to the batch size)
    assert o["OUTPUT"].sizes == x and w["GAMMA"].sizes == [14, 18] and w["BETA"].sizes == [14, 18]
    assert not infer("LAYERNORM", dict(attrs, elementwise_affine=False), [("INPUT", par(x))])[1]
    # dims that are not normalised over may be cut; every shard then needs the whole weight
    o, w = infer("LAYERNORM", attrs, [("INPUT", par(x, [2, 1, 3, 1]))])
    assert sig(o["OUTPUT"]) == (x, [2, 1, 3, 1], 1, 1) and sig(w["GAMMA"]) == ([14, 18], [1, 1], 1, 6)
    # a normalised dim must not be cut; partial sums and replicas are refused
    for bad in (par(x, [1, 2, 1, 1]), par(x, [1, 1, 1, 1], 2, 1), par(x, [1, 1, 1, 1], 1, 2)):
        with pytest.raises(c.CoreError):
            infer("LAYERNORM", attrs, [("INPUT", bad)])


def test_pool2d_shapes():
    attrs = {"kernel_h": 3, "kernel_w": 2, "stride_h": 2, "stride_w": 2, "padding_h": 1, "padding_w": 1, "pool_type": "MAX", "activation": None}
    o, _ = infer("POOL2D", attrs, [("INPUT", par([11, 13, 12, 6]))])
    assert o["OUTPUT"].sizes == [11, 13, 6, 4]
    o, _ = infer("POOL2D", attrs, [("INPUT", par([11, 13, 12, 6], [1, 1, 1, 1], 1, 1))])
    # samples and channels may be cut, replicas pass through, partial sums may not be pooled with max
    o, _ = infer("POOL2D", attrs, [("INPUT", par([12, 14, 12, 6], [4, 2, 1, 1], 1, 3))])
    assert sig(o["OUTPUT"]) == ([12, 14, 6, 4], [4, 2, 1, 1], 1, 3)


def test_concat_shapes():
    a, b, d = [12, 8, 20], [12, 3, 20], [12, 5, 20]
    o, _ = infer("CONCAT", {"axis": 1, "num_inputs": 3}, [("INPUT_0", par(a)), ("INPUT_1", par(b)), ("INPUT_2", par(d))])
    assert o["OUTPUT"].sizes == [12, 16, 20]
    with pytest.raises(c.CoreError):   # the other dims must agree
        infer("CONCAT", {"axis": 1, "num_inputs": 2}, [("INPUT_0", par(a)), ("INPUT_1", par([11, 3, 20]))])
    # every input cut the same way along a non-concat dim
    o, _ = infer("CONCAT", {"axis": 1, "num_inputs": 2}, [("INPUT_0", par(a, [2, 1, 1])), ("INPUT_1", par(b, [2, 1, 1]))])
    assert sig(o["OUTPUT"]) == ([12, 11, 20], [2, 1, 1], 1, 1)
    with pytest.raises(c.CoreError):   # cut along the concat dim
        infer("CONCAT", {"axis": 1, "num_inputs": 2}, [("INPUT_0", par([12, 8, 20], [1, 2, 1])), ("INPUT_1", par([12, 4, 20], [1, 2, 1]))])


def test_softmax_refuses_a_cut_softmax_dim_and_partial_sums():
    x = [12, 14, 16]
    o, _ = infer("SOFTMAX", {"dim": 2}, [("INPUT", par(x, [2, 1, 1]))])
    assert sig(o["OUTPUT"]) == (x, [2, 1, 1], 1, 1)
    for bad in (par(x, [1, 1, 2]), par(x, [1, 1, 1], 2, 1)):
        with pytest.raises(c.CoreError):
            infer("SOFTMAX", {"dim": 2}, [("INPUT", bad)])


def test_element_binary_needs_matching_operands():
    x = [12, 14, 16]
    o, _ = infer("EW_ADD", {}, [("LHS_INPUT", par(x, [2, 1, 1])), ("RHS_INPUT", par(x, [2, 1, 1]))])
    assert sig(o["OUTPUT"]) == (x, [2, 1, 1], 1, 1)
    with pytest.raises(c.CoreError):
        infer("EW_ADD", {}, [("LHS_INPUT", par(x, [2, 1, 1])), ("RHS_INPUT", par(x, [1, 2, 1]))])
    with pytest.raises(c.CoreError):
        infer("EW_ADD", {}, [("LHS_INPUT", par(x)), ("RHS_INPUT", par([12, 14, 15]))])


def test_flat_cast_dropout_shapes():
    o, _ = infer("FLAT", {}, [("INPUT", par([2, 4, 2, 3]))])
    assert o["OUTPUT"].sizes == [2, 24]
    o, _ = infer("FLAT", {}, [("INPUT", par([4, 8, 2, 3], [2, 1, 1, 1]))])
    assert sig(o["OUTPUT"]) == ([4, 48], [2, 1], 1, 1)
    o, _ = infer("CAST", {"dtype": "DOUBLE"}, [("INPUT", par([12, 4], [2, 1], 3, 1))])
    assert o["OUTPUT"].dtype == "DOUBLE" and sig(o["OUTPUT"]) == ([12, 4], [2, 1], 3, 1)
    o, _ = infer("DROPOUT", {"rate": 0.5, "seed": 1}, [("INPUT", par([12, 4], [2, 2]))])
    assert sig(o["OUTPUT"]) == ([12, 4], [2, 2], 1, 1)
    with pytest.raises(c.CoreError):   # a mask over partial sums would not commute with the reduction
        infer("DROPOUT", {"rate": 0.5, "seed": 1}, [("INPUT", par([12, 4], [1, 1], 2, 1))])


# ------------------------------------------------------------------ plain tensor dims (lib/op-attrs/test/src/op-attrs/tensor_dims.cc)
def test_tensor_dims_has_dim():
    assert all(c.tensor_dims_has_dim([6, 9, 8], i) for i in (0, 1, 2))
    assert not c.tensor_dims_has_dim([6, 9, 8], 3) and not c.tensor_dims_has_dim([], 0)


@pytest.mark.parametrize("curr,ok", [
    ([1, 1, 4, 3], True),          # dims match
    ([4, 3], True),                # rank promotion only
    ([1, 1, 1, 3], True),          # dim expansion only
    ([1, 3], True),                # both
    ([1, 1, 2, 3], False),         # 2 does not expand to 4
    ([1, 1, 10, 4, 3], False),     # the goal has fewer dims
])
def test_tensor_dims_is_broadcastable_to(curr, ok):
    assert c.tensor_dims_is_broadcastable_to(curr, [1, 1, 4, 3]) is ok


def test_get_broadcast_target_dims():
    d1, d2 = [1, 10, 4, 3], [10, 4, 1]
    assert c.get_broadcast_target_dims([d1, d2, [1, 1, 4, 3]]) == d1
    assert c.get_broadcast_target_dims([d1, d2, [1, 1, 1, 4]]) is None
    d3, possible = [1, 1, 1, 4, 3], [1, 1, 10, 4, 3]
    assert all(c.tensor_dims_is_broadcastable_to(d, possible) for d in (d1, d2, d3))
    assert c.get_broadcast_target_dims([d1, d2, d3]) is None          # a target outside the inputs does not count
    assert c.get_broadcast_target_dims([]) is None
    assert c.get_broadcast_target_dims([d1] * 5) == d1


def test_tensor_dims_coord_set_and_drop_dims():
    assert c.get_tensor_dims_coord_set([3, 1, 2]) == [[0, 0, 0], [0, 0, 1], [1, 0, 0], [1, 0, 1], [2, 0, 0], [2, 0, 1]]
    assert c.get_tensor_dims_coord_set([]) == [[]]
    dims = [3, 5, 1, 2]
    assert c.tensor_dims_drop_dims(dims, lambda i: i in (0, 2)) == [5, 2]
    assert c.tensor_dims_drop_dims(dims, lambda i: False) == dims
    assert c.tensor_dims_drop_dims(dims, lambda i: True) == []
