"""Frontends on the CPU execution path: layer API, torch.fx importer (+ text IR), ONNX importer, Keras classes."""
from types import SimpleNamespace as NS

import numpy as np
import pytest
import torch
import torch.nn as nn

from flexflow_train_b200.api import FFConfig
from flexflow_train_b200.frontend import (ActiMode, AdamOptimizer, DataType, FFModel, LossType, MetricsType, PoolType, SGDOptimizer)
from flexflow_train_b200.frontend import keras
from flexflow_train_b200.frontend.onnx_model import ONNXModel
from flexflow_train_b200.frontend.torch_fx import PyTorchModel


def _toy_data(n=128, d=20, classes=4, seed=0):
    rng = np.random.RandomState(seed)
    x = rng.randn(n, d).astype(np.float32)
    y = (x @ rng.randn(d, classes)).argmax(1).astype(np.int32).reshape(-1, 1)
    return x, y


def test_ffmodel_layer_api_fit_and_eval():
    m = FFModel(FFConfig(batch_size=32))
    x = m.create_tensor([32, 20], DataType.DT_FLOAT, name="x")
    t = m.dense(x, 32, ActiMode.AC_MODE_RELU, name="fc1")
    t = m.dropout(t, 0.0, 0)
    t = m.softmax(m.dense(t, 4, name="fc2"))
    m.compile(AdamOptimizer(m, alpha=0.01), LossType.LOSS_SPARSE_CATEGORICAL_CROSSENTROPY,
              [MetricsType.METRICS_ACCURACY, MetricsType.METRICS_SPARSE_CATEGORICAL_CROSSENTROPY], device="cpu")
    X, Y = _toy_data()
    hist = m.fit(X, Y, epochs=15)
    assert hist[-1] < 0.5 * hist[0]
    assert m.eval(X, Y).accuracy > 0.9
    assert m.get_layer_by_name("fc1").get_weight_tensor().dims == (32, 20)
    assert m.label_tensor["dims"] == (32, 1)
    assert len(m.get_layers()) == 4


def test_ffmodel_piecewise_step_matches_fit_step():
    def build():
        m = FFModel(FFConfig(batch_size=16, seed=3))
        x = m.create_tensor([16, 20], name="x")
        m.softmax(m.dense(m.dense(x, 8, ActiMode.AC_MODE_TANH), 4))
        m.compile(SGDOptimizer(m, lr=0.1, momentum=0.9), LossType.LOSS_SPARSE_CATEGORICAL_CROSSENTROPY, device="cpu")
        return m
    X, Y = _toy_data(16)
    a, b = build(), build()
    a.fit(X, Y, epochs=2)
    dlx, dly = b.create_data_loader(b._inputs[0], X), b.create_data_loader(None, Y)
    for _ in range(2):
        dlx.reset(); dly.reset()
        b._next_batch([dlx], dly)
        b.forward(); b.zero_gradients(); b.backward(); b.update()
    for (_, p), (_, q) in zip(a.executable.named_parameters(), b.executable.named_parameters()):
        assert torch.allclose(p, q, atol=1e-6)


def test_all_layer_methods_build_a_valid_graph():
    m = FFModel(FFConfig(batch_size=4))
    x = m.create_tensor([4, 3, 16, 16], name="img")
    t = m.conv2d(x, 8, 3, 3, 1, 1, 1, 1, ActiMode.AC_MODE_RELU)
    t = m.batch_norm(t, relu=True)
    t = m.pool2d(t, 2, 2, 2, 2, 0, 0, PoolType.POOL_MAX)
    t = m.flat(t)
    a, b = m.split(t, [256, 256], 1)
    t = m.concat([m.add(a, b), m.subtract(a, b), m.multiply(a, b), m.max(a, b), m.min(a, b)], 1)
    t = m.dense(t, 32)
    for f in (m.exp, m.sin, m.cos, m.rsqrt, m.gelu, m.relu, m.sigmoid, m.tanh, m.elu, m.identity):
        t = f(t)
    t = m.scalar_true_divide(m.scalar_sub(m.scalar_add(m.scalar_multiply(m.pow(t, 2.0), 0.5), 1.0), 0.25), 2.0)
    t = m.layer_norm(t, [-1])
    t = m.reverse(m.transpose(m.reshape(t, [4, 4, 8]), [0, 2, 1]), 1)
    t = m.batch_matmul(t, m.transpose(t, [0, 2, 1]))
    t = m.reduce_sum(t, [2])
    t = m.mean(m.reshape(t, [4, 2, 4]), [1])
    q = m.create_tensor([4, 6, 16], name="seq")
    att = m.multihead_attention(q, q, q, 16, 4)
    ids = m.create_tensor([4, 6, 1], DataType.DT_INT32, name="ids")
    emb = m.embedding(ids, 50, 16)
    s = m.reduce_sum(m.add(att, emb), [1])
    idx = m.create_tensor([4, 3], DataType.DT_INT32, name="gidx")
    g = m.gather(s, idx, 1)
    out = m.softmax(m.dense(m.concat([t, g], 1), 5))
    assert out.dims == (4, 5)
    types = {n["type"] for n in m.graph.nodes()}
    for need in ("CONV2D", "BATCHNORM", "POOL2D", "SPLIT", "CONCAT", "BATCHMATMUL", "MULTIHEAD_ATTENTION", "EMBEDDING", "GATHER",
                 "REVERSE", "TRANSPOSE", "REDUCE_SUM", "LAYERNORM"):
        assert need in types, need


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.c1 = nn.Conv2d(3, 8, 3, padding=1)
        self.bn = nn.BatchNorm2d(8)
        self.pool = nn.MaxPool2d(2)
        self.gap = nn.AdaptiveAvgPool2d((2, 2))
        self.fc1 = nn.Linear(8 * 2 * 2, 32)
        self.ln = nn.LayerNorm(32)
        self.act = nn.GELU()
        self.fc2 = nn.Linear(32, 5)
        self.drop = nn.Dropout(0.0)

    def forward(self, x):
        t = torch.relu(self.bn(self.c1(x)))
        t = self.gap(self.pool(t))
        t = torch.flatten(t, 1)
        a, b = torch.split(self.fc1(t), 16, 1)
        t = torch.cat([a * 2.0, (b + a) / 2], 1)
        t = self.act(self.ln(t)).view(t.size(0), -1)
        t = t.unsqueeze(1).transpose(1, 2).reshape(t.shape[0], 32).contiguous().float()
        return torch.softmax(self.fc2(self.drop(t)), -1)


def test_torch_fx_import_matches_pytorch_and_text_ir_roundtrips(tmp_path):
    torch.manual_seed(0)
    net = _Net()
    m = FFModel(FFConfig(batch_size=4))
    x = m.create_tensor([4, 3, 8, 8], name="x")
    pm = PyTorchModel(net)
    outs = pm.torch_to_ff(m, [x])
    assert len(outs) == 1 and outs[0].dims == (4, 5)
    m.compile(SGDOptimizer(lr=0.01), LossType.LOSS_SPARSE_CATEGORICAL_CROSSENTROPY, device="cpu")
    assert pm.copy_parameters(m) == len(list(net.parameters()))
    xin = torch.randn(4, 3, 8, 8)
    net.train()  # batch statistics, as the executor computes them
    assert torch.allclose(net(xin), m.executable.infer({"x": xin}), atol=1e-5)
    fn = tmp_path / "net.ir"
    pm.torch_to_file(str(fn))
    m2 = FFModel(FFConfig(batch_size=4))
    PyTorchModel.file_to_ff(str(fn), m2, [m2.create_tensor([4, 3, 8, 8], name="x")])
    assert m.graph.to_v1_string() == m2.graph.to_v1_string()


def test_torch_fx_unsupported_module_is_reported():
    class Bad(nn.Module):
        def __init__(self):
            super().__init__()
            self.l = nn.LSTM(4, 4)

        def forward(self, x):
            return self.l(x)
    with pytest.raises(NotImplementedError):
        PyTorchModel(Bad()).to_ir()


def _onnx_attr(name, **kw):
    return NS(name=name, ints=kw.get("ints"), floats=None, s=kw.get("s"), t=None, f=kw.get("f"), i=kw.get("i", 0), type=kw.get("type"))


def test_onnx_importer_on_a_protobuf_shaped_graph():
    init = lambda name, dims: NS(name=name, dims=dims, numpy_value=np.zeros(dims, np.float32))  # noqa: E731
    shape_init = NS(name="shape", dims=[2], numpy_value=np.array([0, -1], np.int64))
    nodes = [
        NS(op_type="Conv", name="conv", input=["x", "w", "b"], output=["c"], attribute=[_onnx_attr("kernel_shape", ints=[3, 3]),
                                                                                       _onnx_attr("pads", ints=[1, 1, 1, 1]),
                                                                                       _onnx_attr("strides", ints=[1, 1])]),
        NS(op_type="BatchNormalization", name="bn", input=["c"], output=["n"], attribute=[]),
        NS(op_type="Relu", name="relu", input=["n"], output=["r"], attribute=[]),
        NS(op_type="MaxPool", name="mp", input=["r"], output=["p"], attribute=[_onnx_attr("kernel_shape", ints=[2, 2]),
                                                                               _onnx_attr("strides", ints=[2, 2])]),
        NS(op_type="GlobalAveragePool", name="gap", input=["p"], output=["g"], attribute=[]),
        NS(op_type="Reshape", name="rs", input=["g", "shape"], output=["f"], attribute=[]),
        NS(op_type="Gemm", name="fc", input=["f", "fw", "fb"], output=["l"], attribute=[_onnx_attr("transB", i=1, type=2)]),
        NS(op_type="Dropout", name="do", input=["l"], output=["d"], attribute=[_onnx_attr("ratio", f=0.25, type=1)]),
        NS(op_type="Softmax", name="sm", input=["d"], output=["y"], attribute=[_onnx_attr("axis", i=1, type=2)]),
    ]
    graph = NS(node=nodes, initializer=[init("w", [8, 3, 3, 3]), init("b", [8]), init("fw", [10, 8]), init("fb", [10]), shape_init],
               output=[NS(name="y")])
    m = FFModel(FFConfig(batch_size=2))
    x = m.create_tensor([2, 3, 8, 8], name="x")
    outs = ONNXModel(NS(graph=graph)).apply(m, {"x": x})
    assert outs[0].dims == (2, 10)
    kinds = [n["type"] for n in m.graph.nodes() if n["type"] not in ("WEIGHT", "INPUT")]
    assert kinds == ["CONV2D", "BATCHNORM", "RELU", "POOL2D", "POOL2D", "RESHAPE", "LINEAR", "DROPOUT", "SOFTMAX"]
    with pytest.raises(NotImplementedError):
        ONNXModel(NS(graph=NS(node=[NS(op_type="LSTM", name="l", input=["x"], output=["y"], attribute=[])], initializer=[], output=[]))) \
            .apply(m, {"x": x})


def test_keras_sequential_and_functional_models_train():
    from flexflow_train_b200.frontend.keras.callbacks import EpochVerifyMetrics, LearningRateScheduler
    from flexflow_train_b200.frontend.keras.layers import Dense, concatenate

    X, Y = _toy_data()
    m = keras.Sequential([Dense(32, activation="relu", input_shape=(20,)), Dense(4, activation="softmax")])
    m.compile(optimizer=keras.optimizers.Adam(0.01), loss="sparse_categorical_crossentropy", metrics=["accuracy"], batch_size=32,
              device="cpu")
    h = m.fit(X, Y, epochs=30, callbacks=[EpochVerifyMetrics(95), LearningRateScheduler(lambda e: 0.01)])
    assert h.history["accuracy"][-1] >= 0.95 and len(h.epoch) < 30  # stopped early
    a, b = keras.Input((20,), name="a"), keras.Input((20,), name="b")
    out = Dense(4, activation="softmax")(concatenate([Dense(16, activation="relu")(a), Dense(16, activation="tanh")(b)]))
    fm = keras.Model([a, b], out)
    fm.compile("sgd", "sparse_categorical_crossentropy", ["accuracy"], batch_size=32, device="cpu")
    hist = fm.fit([X, X], Y, epochs=3).history["loss"]
    assert hist[-1] < hist[0]
    assert fm.predict([X, X]).shape == (128, 4)
    assert fm.evaluate([X, X], Y)["samples"] == 128


class _SmallMlp(nn.Module):
    def __init__(self):
        super().__init__()
        self.f1 = nn.Linear(16, 32)
        self.f2 = nn.Linear(32, 5)

    def forward(self, x):
        return torch.softmax(self.f2(torch.relu(self.f1(x))), -1)


def test_compile_module_is_a_one_call_path_from_nn_module_to_a_trainable_model():
    """nn.Module -> trace -> computation graph -> (search) -> executor in one call, as the reference's PyTorch frontend is
    drawn (docs/plantuml/figures/pytorch-tracing.puml): same outputs as the module, the loss goes down, and the trained
    weights can be written back into the module."""
    from flexflow_train_b200.frontend.torch_fx import compile_module

    torch.manual_seed(0)
    net = _SmallMlp()
    x, y = torch.randn(8, 16), torch.randint(0, 5, (8,), dtype=torch.int32)
    cm = compile_module(net, [x], optimizer=SGDOptimizer(lr=0.1), loss_type=LossType.LOSS_SPARSE_CATEGORICAL_CROSSENTROPY, device="cpu")
    assert cm.input_names == ["x"] and torch.allclose(cm(x), net(x), atol=1e-5)
    losses = [cm.train_step(x, labels=y) for _ in range(6)]
    assert losses[-1] < losses[0]
    before = net.f1.weight.detach().clone()
    assert cm.sync_parameters_to_module() == 4 and not torch.equal(before, net.f1.weight)
    assert torch.allclose(cm(x), net(x), atol=1e-5)


def test_torch_compile_backend_runs_the_dynamo_graph_on_the_executor():
    from flexflow_train_b200.frontend.torch_fx import flexflow_backend

    torch.manual_seed(1)
    net = _SmallMlp()
    x = torch.randn(8, 16)
    compiled = torch.compile(net, backend=lambda gm, example_inputs: flexflow_backend(gm, example_inputs, device="cpu"))
    with torch.no_grad():
        assert torch.allclose(compiled(x), net(x), atol=1e-5)


def test_legacy_weight_access_layer_queries_and_config_helpers():
    # the data-access surface of the legacy Tensor / Layer / FFConfig / PerfMetrics classes
    # (bindings/python/old/flexflow/core/flexflow_cffi.py)
    import numpy as np
    from flexflow_train_b200.frontend import ActiMode, DataType, FFConfig, FFModel, LossType, SGDOptimizer
    cfg = FFConfig(batch_size=4)
    cfg.parse_args(["-b", "8", "--epochs", "3", "-ll:gpu", "1", "--unknown-flag"])
    assert cfg.batch_size == 8 and cfg.epochs == 3 and cfg.learning_rate == FFConfig().learning_rate
    assert cfg.workers_per_node == cfg.gpus_per_node
    t0 = cfg.get_current_time()
    cfg.begin_trace(111)
    cfg.end_trace(111)
    assert cfg.get_current_time() >= t0

    ff = FFModel(cfg)
    x = ff.create_tensor([8, 6], DataType.DT_FLOAT, name="x")
    h = ff.dense(x, 5, ActiMode.AC_MODE_RELU, name="fc1")
    ff.softmax(ff.dense(h, 3, name="fc2"))
    fc1 = ff.get_layer_by_name("fc1")
    assert (fc1.get_number_inputs(), fc1.get_number_parameters(), fc1.get_number_outputs()) == (1, 2, 1)
    assert fc1.get_input_tensor().dims == (8, 6) and fc1.get_input_by_id(0).value == x.value
    assert fc1.get_output_by_id(0).dims == (8, 5) and ff.get_tensor_by_id(0).dims == ff.get_layer_by_id(0).get_output_tensor().dims
    w = fc1.get_weight_tensor()
    with pytest.raises(RuntimeError):
        w.get_weights(ff)                                   # not compiled yet
    ff.compile(optimizer=SGDOptimizer(ff, 0.1), loss_type=LossType.LOSS_SPARSE_CATEGORICAL_CROSSENTROPY, device="cpu")
    before = w.get_weights(ff)
    assert before.shape == (5, 6) and before.dtype == np.float32
    new = np.arange(30, dtype=np.float32).reshape(5, 6) / 30.0
    assert w.set_weights(ff, new) and np.array_equal(w.get_weights(ff), new)
    assert np.array_equal(w.get_flat_array(ff), new.reshape(-1)) and np.array_equal(w.get_array(ff), new)
    with pytest.raises(ValueError):
        w.set_weights(ff, np.zeros((6, 5), dtype=np.float32))
    with pytest.raises(TypeError):
        h.get_weights(ff)                                   # an activation, not a parameter
    # a step with the new weights: the gradient of fc1's weight exists and the weight moves by -lr * gradient
    xs = np.random.RandomState(0).rand(8, 6).astype(np.float32)
    ys = np.random.RandomState(1).randint(0, 3, size=(8, 1)).astype(np.int32)
    ff.fit(x=xs, y=ys, epochs=1)
    g = w.get_gradients(ff)
    assert g.shape == (5, 6) and np.abs(g).sum() > 0
    assert np.allclose(w.get_weights(ff), new - 0.1 * g, atol=1e-6)
    assert ff.get_perf_metrics().get_accuracy() == 100.0 * ff.get_perf_metrics().accuracy


def test_keras_utils_preprocessing_and_datasets(tmp_path):
    import numpy as np
    from flexflow_train_b200.frontend import keras
    K = keras
    assert K.utils.to_categorical([0, 2, 1]).tolist() == [[1, 0, 0], [0, 0, 1], [0, 1, 0]]
    assert K.utils.to_categorical([[1], [0]], num_classes=3).shape == (2, 3)
    assert K.utils.to_categorical(np.array([[0, 1], [1, 0]])).shape == (2, 2, 2)
    with pytest.raises(ValueError):
        K.utils.to_categorical([3], num_classes=3)
    n = K.utils.normalize(np.array([[3.0, 4.0], [0.0, 0.0]]))
    assert np.allclose(n, [[0.6, 0.8], [0.0, 0.0]])
    pad = K.preprocessing.sequence.pad_sequences
    assert pad([[1, 2, 3], [4], []], maxlen=2).tolist() == [[2, 3], [0, 4], [0, 0]]
    assert pad([[1, 2, 3], [4]], padding="post", truncating="post", maxlen=2).tolist() == [[1, 2], [4, 0]]
    assert pad([[1], [2, 3]]).shape == (2, 2)
    tok = K.preprocessing.text.Tokenizer(num_words=3, oov_token="<unk>")
    tok.fit_on_texts(["The cat sat.", "the cat ran!"])
    assert tok.word_index["<unk>"] == 1 and tok.word_index["the"] == 2 and tok.word_index["cat"] == 3
    assert tok.texts_to_sequences(["the dog sat"]) == [[2, 1, 1]]            # only indices below num_words are kept
    # data sets read local files and name the file they miss
    with pytest.raises(FileNotFoundError, match="mnist.npz"):
        K.datasets.mnist.load_data(str(tmp_path / "mnist.npz"))
    np.savez(tmp_path / "mnist.npz", x_train=np.zeros((5, 28, 28), np.uint8), y_train=np.arange(5), x_test=np.zeros((2, 28, 28), np.uint8), y_test=np.arange(2))
    (xtr, ytr), (xte, yte) = K.datasets.mnist.load_data(str(tmp_path / "mnist.npz"))
    assert xtr.shape == (5, 28, 28) and yte.tolist() == [0, 1]
    x = np.empty(4, dtype=object)
    x[:] = [[1, 2], [3], [4, 5, 6], [7]]
    np.savez(tmp_path / "reuters.npz", x=x, y=np.array([0, 1, 2, 3]))
    (a, la), (b, lb) = K.datasets.reuters.load_data(str(tmp_path / "reuters.npz"), test_split=0.25, num_words=8)
    assert len(a) == 3 and len(b) == 1 and all(s[0] == 1 for s in list(a) + list(b))
    assert all(w in (1, 2) or 3 <= w < 8 for s in list(a) + list(b) for w in s)
    with pytest.raises(FileNotFoundError):
        K.datasets.cifar10.load_data(str(tmp_path / "nowhere"))


def test_keras_initializers_regularizers_and_backend_functions():
    import numpy as np
    from flexflow_train_b200.frontend import keras
    from flexflow_train_b200.frontend.types import RegularizerMode
    L, B = keras.layers, keras.backend
    assert keras.regularizers.L2(0.5)._lambda == 0.5 and keras.regularizers.L1().type == RegularizerMode.REG_MODE_L1
    assert isinstance(keras.initializers.get("zeros"), keras.initializers.Zeros)
    with pytest.raises(ValueError):
        keras.initializers.get("no_such")
    inp = keras.Input(shape=(6,))
    h = L.Dense(5, activation="relu", kernel_initializer=keras.initializers.Zeros(), bias_initializer="zeros",
                kernel_regularizer=keras.regularizers.L2(0.01), name="zeroed")(inp)
    h = B.exp(h)                                     # exp(relu(0)) = 1 everywhere
    h = B.pow(h, 2.0)
    s = B.sum(h, axis=1, keepdims=True)              # 5 ones per sample
    out = L.Dense(3, activation="softmax", name="head")(L.Concatenate(axis=1)([h, s]))
    model = keras.Model(inp, out)
    model.compile(optimizer=keras.optimizers.SGD(0.0), loss="sparse_categorical_crossentropy", metrics=["accuracy"], device="cpu")
    xs = np.random.RandomState(0).rand(8, 6).astype(np.float32)
    ys = np.zeros((8, 1), dtype=np.int32)
    model.fit(xs, ys, batch_size=8, epochs=1)        # the graph is built at the first fit; learning rate 0 leaves the weights
    ff = model.ffmodel
    w = ff.get_layer_by_name("zeroed").get_weight_tensor()
    assert not w.get_weights(ff).any()
    types = [n["type"] for n in ff.graph.nodes()]
    assert "EXP" in types and "POW" in types and "REDUCE_SUM" in types
