"""CPU execution path: the autograd interpreter plus the reference's optimizer update rules.

The reference keeps a CPU-only executor for tests and cost measurement (lib/local-execution with
``DeviceType::CPU``, exercised by lib/local-execution/test/src/local-execution/computation_graph_instance.cc).
Here the same role is played by ``CpuExecutable``: it has the surface of the GPU ``Executable`` (``train_step``,
``infer``, ``loss_rows``, ``named_parameters``, ``state_dict`` ...) and evaluates the graph with plain PyTorch
ops in fp32, so a model built through any frontend can be stepped, checkpointed and compared without a GPU.

Update rules (lib/kernels/src/cuda/optimizer_kernels.cu:11-31, 177-203):
  SGD:  g' = g + wd*w;  v = momentum*v + g';  g'' = nesterov ? g' + momentum*v : v;  w -= lr*g''
  Adam: g' = g + wd*w;  m = b1*m + (1-b1)*g';  v = b2*v + (1-b2)*g'^2;  w -= alpha_t * m / (sqrt(v) + eps)
        with alpha_t = lr * sqrt(1 - b2^t) / (1 - b1^t)
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .executor import ExecConfig
from .torch_oracle import TorchOracle


class CpuExecutable:
    on_gpu = False

    def __init__(self, graph, cfg: Optional[ExecConfig] = None):
        self.graph = graph
        self.cfg = cfg or ExecConfig(device="cpu")
        self.oracle = TorchOracle(graph, loss=self.cfg.loss, seed=self.cfg.seed, device="cpu", training=self.cfg.training,
                                  dropout=False, causal_attention=self.cfg.causal_attention)
        self.nodes = self.oracle.nodes
        self.step_count = 0
        self.loss_rows = None
        self.loss_value = self.oracle.loss_value
        self._inputs: Dict[str, torch.Tensor] = {}
        self._labels = None
        self._m = {k: torch.zeros_like(p) for k, p in self.oracle.params.items()}
        self._v = {k: torch.zeros_like(p) for k, p in self.oracle.params.items()}
        self.launches_per_step = 0

    # ---- step pieces (the legacy API drives them one by one)
    def set_inputs(self, inputs: Dict[str, torch.Tensor], labels: Optional[torch.Tensor] = None):
        self._inputs.update({k: v.detach().cpu() for k, v in inputs.items()})
        if labels is not None:
            self._labels = labels.detach().cpu()

    def forward(self):
        self._pred = self.oracle.forward(self._inputs)
        return self._pred

    def compute_loss(self):
        self.loss_rows = self.oracle.loss(self._pred, self._labels)
        return self.loss_rows

    def zero_gradients(self):
        for p in self.oracle.params.values():
            p.grad = None

    def backward(self):
        self.zero_gradients()
        self.compute_loss().mean().backward()
        self.loss_rows = self.loss_rows.detach()

    def update(self):
        o = self.cfg.optimizer
        self.step_count += 1
        t = self.step_count
        with torch.no_grad():
            for k, p in self.oracle.params.items():
                if p.grad is None:
                    continue
                g = p.grad + o.weight_decay * p
                if o.kind == "adam":
                    m, v = self._m[k], self._v[k]
                    m.mul_(o.beta1).add_(g, alpha=1 - o.beta1)
                    v.mul_(o.beta2).addcmul_(g, g, value=1 - o.beta2)
                    alpha_t = o.lr * math.sqrt(1 - o.beta2 ** t) / (1 - o.beta1 ** t)
                    p.sub_(alpha_t * m / (v.sqrt() + o.epsilon))
                else:
                    if o.momentum > 0:
                        v = self._v[k]
                        v.mul_(o.momentum).add_(g)
                        g = g + o.momentum * v if o.nesterov else v
                    p.sub_(o.lr * g)

    def train_step(self, inputs: Optional[Dict[str, torch.Tensor]] = None, labels: Optional[torch.Tensor] = None):
        if inputs is not None or labels is not None:
            self.set_inputs(inputs or {}, labels)
        self.forward()
        self.backward()
        self.update()
        return self.loss_rows

    def infer(self, inputs: Dict[str, torch.Tensor]):
        self.set_inputs(inputs)
        with torch.no_grad():
            return self.forward()

    def mean_loss(self) -> float:
        return float(self.loss_rows.mean().item())

    # ---- parameter access
    def named_parameters(self):
        return ((k, p.detach()) for k, p in self.oracle.params.items())

    def named_gradients(self):
        return ((k, p.grad) for k, p in self.oracle.params.items())

    def state_dict(self):
        return {"params": {k: p.detach().clone() for k, p in self.oracle.params.items()},
                "m": {k: v.clone() for k, v in self._m.items()}, "v": {k: v.clone() for k, v in self._v.items()},
                "step": self.step_count}

    def load_state_dict(self, sd):
        with torch.no_grad():
            for k, p in self.oracle.params.items():
                p.copy_(sd["params"][k])
                self._m[k].copy_(sd["m"][k])
                self._v[k].copy_(sd["v"][k])
        self.step_count = int(sd["step"])
