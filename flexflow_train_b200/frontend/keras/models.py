"""Keras-style ``Sequential`` and functional ``Model`` on top of ``FFModel``
(bindings/python/old/flexflow/keras/models/{base_model,sequential,model}.py)."""
from __future__ import annotations

from typing import List, Optional

import numpy as np

from ...api import FFConfig
from ..ffmodel import FFModel
from ..types import DataType
from . import losses as _losses
from . import metrics as _metrics
from . import optimizers as _optimizers
from .callbacks import History
from .layers import Input, InputLayer, KTensor, Layer

_DT = {"float32": DataType.DT_FLOAT, "float64": DataType.DT_DOUBLE, "int32": DataType.DT_INT32, "int64": DataType.DT_INT64,
       "float16": DataType.DT_HALF}


class BaseModel:
    def __init__(self, name=None):
        self.name = name or type(self).__name__.lower()
        self.ffmodel: Optional[FFModel] = None
        self.optimizer = None
        self.stop_training = False
        self._inputs: List[KTensor] = []
        self._outputs: List[KTensor] = []

    # ---- graph replay
    def _materialise(self, batch_size):
        ff = FFModel(FFConfig(batch_size=batch_size))
        for i, kt in enumerate(self._inputs):
            kt.ff = ff.create_tensor([batch_size] + list(kt.shape), _DT[kt.dtype], name=kt.layer.name if kt.layer.name else f"input{i}")
        done = {id(k): k.ff for k in self._inputs}

        def visit(kt: KTensor):
            if id(kt) in done:
                return done[id(kt)]
            xs = [visit(p) for p in kt.inputs]
            out = kt.layer.build(ff, xs)
            done[id(kt)] = out[kt.index] if isinstance(out, (list, tuple)) else out
            return done[id(kt)]

        self._ff_outputs = [visit(o) for o in self._outputs]
        self.ffmodel = ff
        return ff

    def compile(self, optimizer="sgd", loss="sparse_categorical_crossentropy", metrics=None, batch_size=64, device=None, **kw):
        self.optimizer = _optimizers.get(optimizer)
        self._loss = _losses.get(loss)
        self._metrics = [_metrics.get(m) for m in (metrics or [])]
        self._batch_size = batch_size
        self._device = device
        self._compiled_for = None

    def _ensure(self, batch_size):
        if self._compiled_for != batch_size:
            ff = self._materialise(batch_size)
            ff.compile(self.optimizer, self._loss, self._metrics, device=self._device)
            self._compiled_for = batch_size

    def fit(self, x, y, batch_size=None, epochs=1, callbacks=None, verbose=False):
        bs = batch_size or self._batch_size
        self._ensure(bs)
        ff = self.ffmodel
        xs = list(x) if isinstance(x, (list, tuple)) else [x]
        cbs = [History()] + list(callbacks or [])
        for c in cbs:
            c.set_model(self)
            c.on_train_begin()
        logs = {}
        self.stop_training = False
        for epoch in range(epochs):
            for c in cbs:
                c.on_epoch_begin(epoch)
            hist = ff.fit([np.asarray(a) for a in xs], np.asarray(y), batch_size=bs, epochs=1)
            logs = dict(ff.get_perf_metrics().summary(), loss=float(np.mean(hist)))
            if verbose:
                print(f"epoch {epoch}: {logs}")
            for c in cbs:
                c.on_epoch_end(epoch, logs)
            if self.stop_training:
                break
        for c in cbs:
            c.on_train_end(logs)
        return cbs[0]

    def evaluate(self, x, y, batch_size=None):
        bs = batch_size or self._batch_size
        self._ensure(bs)
        xs = list(x) if isinstance(x, (list, tuple)) else [x]
        return self.ffmodel.eval([np.asarray(a) for a in xs], np.asarray(y), batch_size=bs).summary()

    def predict(self, x, batch_size=None):
        import torch

        xs = list(x) if isinstance(x, (list, tuple)) else [x]
        bs = batch_size or self._batch_size
        self._ensure(bs)
        outs = []
        n = len(xs[0])
        for i in range(0, n - bs + 1, bs):
            feed = {kt.ff.name: torch.as_tensor(np.asarray(a[i:i + bs])) for kt, a in zip(self._inputs, xs)}
            outs.append(self.ffmodel.executable.infer(feed).detach().float().cpu())
        return torch.cat(outs).numpy()

    def summary(self):
        if self.ffmodel is None:
            self._materialise(self._batch_size if hasattr(self, "_batch_size") else 1)
        self.ffmodel.print_layers()

    @property
    def layers(self):
        seen, out = set(), []

        def visit(kt):
            for p in kt.inputs:
                visit(p)
            if id(kt.layer) not in seen:
                seen.add(id(kt.layer))
                out.append(kt.layer)
        for o in self._outputs:
            visit(o)
        return out


class Model(BaseModel):
    """Functional model: ``Model(inputs=[...], outputs=[...])``."""

    def __init__(self, inputs, outputs, name=None):
        super().__init__(name)
        self._inputs = list(inputs) if isinstance(inputs, (list, tuple)) else [inputs]
        self._outputs = list(outputs) if isinstance(outputs, (list, tuple)) else [outputs]


class Sequential(BaseModel):
    def __init__(self, layers=None, name=None):
        super().__init__(name)
        self._stack: List[Layer] = []
        for l in layers or []:
            self.add(l)

    def add(self, layer):
        if isinstance(layer, KTensor):  # an Input(...)
            self._inputs, self._outputs = [layer], [layer]
            return
        if isinstance(layer, InputLayer):
            t = KTensor(layer, [], shape=layer.shape, dtype=layer.dtype)
            self._inputs, self._outputs = [t], [t]
            return
        if not self._inputs:
            if layer.input_shape is None:
                raise ValueError("the first layer of a Sequential model needs input_shape=...")
            t = Input(layer.input_shape)
            self._inputs, self._outputs = [t], [t]
        self._stack.append(layer)
        self._outputs = [layer(self._outputs[0])]

    def pop(self):
        self._stack.pop()
        self._outputs = [self._outputs[0].inputs[0]]
