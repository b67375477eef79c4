"""Training metrics and step logging.

``PerfMetrics`` has the fields of the reference's struct (lib/kernels/include/kernels/perf_metrics.dtg.toml):
train_all, train_correct, cce, sparse_cce, mse, rmse, mae, start/current time; ``update`` computes them for a
batch from predictions and labels (the reference's metrics kernels, lib/kernels/src/cuda/metrics_functions.cu:48-98,
accumulate the same sums with atomics).  Batches on the GPU go through ``ffk_metrics_update`` (csrc/kernels/metrics.cu):
one launch per batch into a device accumulator that is read when a number is asked for.  ``StepLogger`` writes one
JSON line per step.
"""
from __future__ import annotations

import json
import math
import time
from dataclasses import asdict, dataclass, field
from typing import Iterable, Optional

import torch

METRICS = ("accuracy", "categorical_crossentropy", "sparse_categorical_crossentropy", "mean_squared_error",
           "root_mean_squared_error", "mean_absolute_error")


@dataclass
class PerfMetrics:
    train_all: int = 0
    train_correct: int = 0
    cce_loss: float = 0.0
    sparse_cce_loss: float = 0.0
    mse_loss: float = 0.0
    rmse_loss: float = 0.0
    mae_loss: float = 0.0
    start_time: float = field(default_factory=time.time)
    current_time: float = field(default_factory=time.time)

    def reset(self):
        acc = self.__dict__.get("_dev")
        if acc is not None:
            acc.zero_()
            self.__dict__["_dirty"] = False
        self.__init__()

    # ---- device path: batches whose predictions live on the GPU are added by one kernel launch into a device
    # accumulator (no host synchronisation per step); the fields above are refreshed from it when they are read
    def _update_on_device(self, pred, label, metrics) -> bool:
        from ..ops import kernels as K
        if not (pred.is_cuda and K.available() and pred.dtype in (torch.float32, torch.bfloat16)):
            return False
        p = pred.detach().reshape(-1, pred.shape[-1]).contiguous()
        n = p.shape[0]
        sparse = label.dim() == 1 or label.numel() == n
        lab = label.detach().to(p.device)
        if sparse:
            lab = lab.reshape(-1)
            if lab.dtype not in (torch.int32, torch.int64):
                lab = lab.long()
        else:
            lab = lab.reshape(n, -1).to(p.dtype)
        acc = self.__dict__.get("_dev")
        if acc is None or acc.device != p.device:
            self.pull()
            acc = torch.zeros(8, dtype=torch.float64, device=p.device)
            self.__dict__["_dev"] = acc
        K.metrics_update(p, lab.contiguous(), acc, [m for m in metrics if m in K.METRIC_FLAGS])
        self.__dict__["_dirty"] = True
        return True

    def pull(self):
        """Fold the device accumulator into the host fields (one device-to-host read)."""
        acc = self.__dict__.get("_dev")
        if acc is None or not self.__dict__.get("_dirty"):
            return self
        v = acc.cpu().tolist()
        acc.zero_()
        self.__dict__["_dirty"] = False
        self.train_all += int(round(v[0]))
        self.train_correct += int(round(v[1]))
        self.cce_loss += v[2]
        self.sparse_cce_loss += v[3]
        self.mse_loss += v[4]
        self.rmse_loss += v[5]
        self.mae_loss += v[6]
        return self

    def update(self, pred: torch.Tensor, label: torch.Tensor, metrics: Iterable[str] = ("accuracy",)):
        """pred: [N, C] probabilities or values; label: [N] class ids (sparse) or [N, C] targets."""
        metrics = tuple(metrics)
        if self._update_on_device(pred, label, metrics):
            self.current_time = time.time()
            return self
        p = pred.detach().float().reshape(-1, pred.shape[-1])
        n = p.shape[0]
        sparse = label.dim() == 1 or label.numel() == n
        self.train_all += n
        if "accuracy" in metrics:
            tgt = label.reshape(-1).long() if sparse else label.reshape(n, -1).argmax(1)
            self.train_correct += int((p.argmax(1).to(tgt.device) == tgt).sum().item())
        # the reference's definitions: probabilities clamped at 1e-8 before the logarithm, squared / absolute errors
        # summed over a sample's classes, sparse labels compared as one-hot targets
        if sparse and "sparse_categorical_crossentropy" in metrics:
            tgt = label.reshape(-1).long().to(p.device)
            self.sparse_cce_loss += float(-torch.log(p.gather(1, tgt[:, None]).clamp_min(1e-8)).sum().item())
        if sparse:
            t = torch.nn.functional.one_hot(label.reshape(-1).long().to(p.device), p.shape[1]).float()
        else:
            t = label.reshape(n, -1).float().to(p.device)
            if "categorical_crossentropy" in metrics:
                self.cce_loss += float(-(t * torch.log(p.clamp_min(1e-8))).sum().item())
        d = p - t
        if "mean_squared_error" in metrics:
            self.mse_loss += float((d * d).sum(1).sum().item())
        if "root_mean_squared_error" in metrics:
            self.rmse_loss += float((d * d).sum(1).sqrt().sum().item())
        if "mean_absolute_error" in metrics:
            self.mae_loss += float(d.abs().sum(1).sum().item())
        self.current_time = time.time()
        return self

    @property
    def accuracy(self) -> float:
        self.pull()
        return self.train_correct / max(self.train_all, 1)

    def get_accuracy(self) -> float:
        """Accuracy in percent, as the legacy ``PerfMetrics.get_accuracy`` reports it
        (bindings/python/old/flexflow/core/flexflow_cffi.py)."""
        return 100.0 * self.accuracy

    def throughput(self) -> float:
        self.pull()
        return self.train_all / max(self.current_time - self.start_time, 1e-9)

    def summary(self) -> dict:
        self.pull()
        n = max(self.train_all, 1)
        return {"samples": self.train_all, "accuracy": self.accuracy, "cce": self.cce_loss / n,
                "sparse_cce": self.sparse_cce_loss / n, "mse": self.mse_loss / n, "rmse": self.rmse_loss / n,
                "mae": self.mae_loss / n, "samples_per_s": self.throughput()}


class StepLogger:
    """One JSON object per line: step, loss, samples/s (device-timed by the caller), free-form extras."""

    def __init__(self, path: Optional[str] = None, rank: int = 0):
        self.path, self.rank = path, rank
        self.records = []

    def log(self, step: int, loss: float, samples_per_s: Optional[float] = None, **extra):
        rec = {"step": step, "loss": float(loss), "samples_per_s": samples_per_s, "time": time.time(), "rank": self.rank}
        rec.update(extra)
        self.records.append(rec)
        if self.path and self.rank == 0:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")
        return rec
