"""Frontends driving the GPU executor: layer API, Keras classes and the torch.fx importer compile to the kernel
library and train there (the CPU-path versions of these tests are in test_frontend.py)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from flexflow_train_b200.api import FFConfig  # noqa: E402
from flexflow_train_b200.frontend import ActiMode, AdamOptimizer, DataType, FFModel, LossType, MetricsType, SGDOptimizer  # noqa: E402
from flexflow_train_b200.frontend import keras  # noqa: E402
from flexflow_train_b200.frontend.torch_fx import PyTorchModel  # noqa: E402
from flexflow_train_b200.ops import kernels as K  # noqa: E402


def _toy_data(n=256, d=32, classes=4, seed=0):
    rng = np.random.RandomState(seed)
    x = rng.randn(n, d).astype(np.float32)
    y = (x @ rng.randn(d, classes)).argmax(1).astype(np.int32).reshape(-1, 1)
    return x, y


def test_ffmodel_fit_and_eval_on_gpu():
    before = K.launch_count()
    m = FFModel(FFConfig(batch_size=64))
    x = m.create_tensor([64, 32], DataType.DT_FLOAT, name="x")
    t = m.dense(x, 64, ActiMode.AC_MODE_RELU, name="fc1")
    t = m.dropout(t, 0.0, 0)
    t = m.softmax(m.dense(t, 4, name="fc2"))
    m.compile(AdamOptimizer(m, alpha=0.01), LossType.LOSS_SPARSE_CATEGORICAL_CROSSENTROPY,
              [MetricsType.METRICS_ACCURACY, MetricsType.METRICS_SPARSE_CATEGORICAL_CROSSENTROPY], device="cuda")
    X, Y = _toy_data()
    hist = m.fit(X, Y, epochs=20)
    assert hist[-1] < 0.5 * hist[0]
    assert m.eval(X, Y).accuracy > 0.85
    assert K.launch_count() > before  # the kernel library did the work


def test_keras_models_train_on_gpu():
    from flexflow_train_b200.frontend.keras.layers import Dense, concatenate

    X, Y = _toy_data()
    m = keras.Sequential([Dense(64, activation="relu", input_shape=(32,)), Dense(4, activation="softmax")])
    m.compile(optimizer=keras.optimizers.Adam(0.01), loss="sparse_categorical_crossentropy", metrics=["accuracy"], batch_size=64,
              device="cuda")
    h = m.fit(X, Y, epochs=20)
    assert h.history["loss"][-1] < 0.5 * h.history["loss"][0]
    a, b = keras.Input((32,), name="a"), keras.Input((32,), name="b")
    out = Dense(4, activation="softmax")(concatenate([Dense(16, activation="relu")(a), Dense(16, activation="tanh")(b)]))
    fm = keras.Model([a, b], out)
    fm.compile("sgd", "sparse_categorical_crossentropy", ["accuracy"], batch_size=64, device="cuda")
    hist = fm.fit([X, X], Y, epochs=3).history["loss"]
    assert hist[-1] < hist[0]
    assert fm.predict([X, X]).shape == (256, 4)


class _Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.c1 = torch.nn.Conv2d(3, 8, 3, padding=1)
        self.pool = torch.nn.MaxPool2d(2)
        self.fc1 = torch.nn.Linear(8 * 4 * 4, 32)
        self.ln = torch.nn.LayerNorm(32)
        self.fc2 = torch.nn.Linear(32, 5)

    def forward(self, x):
        t = self.pool(torch.relu(self.c1(x)))
        t = torch.flatten(t, 1)
        t = torch.nn.functional.gelu(self.ln(self.fc1(t)))
        return torch.softmax(self.fc2(t), -1)


def test_torch_fx_import_runs_on_gpu_and_matches_pytorch():
    torch.manual_seed(0)
    net = _Net()
    m = FFModel(FFConfig(batch_size=8))
    x = m.create_tensor([8, 3, 8, 8], name="x")
    pm = PyTorchModel(net)
    pm.torch_to_ff(m, [x])
    m.compile(SGDOptimizer(lr=0.05), LossType.LOSS_SPARSE_CATEGORICAL_CROSSENTROPY, device="cuda")
    assert pm.copy_parameters(m) == len(list(net.parameters()))
    xin = torch.randn(8, 3, 8, 8)
    got = m.executable.infer({"x": xin.cuda()}).float().cpu()
    assert (got - net(xin)).abs().max() < 3e-2  # bf16 compute
    labels = torch.randint(0, 5, (8,), dtype=torch.int32)
    losses = []
    for _ in range(8):
        m.executable.train_step({"x": xin.cuda()}, labels.cuda())
        losses.append(m.executable.mean_loss())
    assert losses[-1] < losses[0]


def test_legacy_weight_access_on_gpu():
    # Tensor.get_weights / set_weights / get_gradients of the legacy API against the GPU executor: a written weight is what
    # the kernels compute with (the bf16 copy follows the fp32 master), and the gradient comes back after a step
    m = FFModel(FFConfig(batch_size=64, use_cuda_graph=False))
    x = m.create_tensor([64, 32], DataType.DT_FLOAT, name="x")
    m.softmax(m.dense(x, 4, use_bias=False, name="fc"))
    m.compile(SGDOptimizer(m, 0.0), LossType.LOSS_SPARSE_CATEGORICAL_CROSSENTROPY)
    w = m.get_layer_by_name("fc").get_weight_tensor()
    assert w.get_weights(m).shape == (4, 32)
    new = np.zeros((4, 32), dtype=np.float32)
    new[2, :] = 0.5                                           # class 2 wins for inputs with a positive sum
    assert w.set_weights(m, new) and np.array_equal(w.get_weights(m), new)
    xs = np.abs(np.random.RandomState(0).randn(64, 32)).astype(np.float32)
    ys = np.full((64, 1), 2, dtype=np.int32)
    m.fit(x=xs, y=ys, epochs=1)
    pred = m._predictions().argmax(-1).cpu().numpy()
    assert (pred == 2).all()
    g = w.get_gradients(m)
    assert g.shape == (4, 32) and np.isfinite(g).all() and np.abs(g).sum() > 0
    assert np.array_equal(w.get_weights(m), new)              # learning rate 0: the step left the weight alone
