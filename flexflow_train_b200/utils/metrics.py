"""Training metrics and step logging.

``PerfMetrics`` has the fields of the reference's struct (lib/kernels/include/kernels/perf_metrics.dtg.toml):
train_all, train_correct, cce, sparse_cce, mse, rmse, mae, start/current time; ``update`` computes them for a
batch from predictions and labels (the reference's metrics kernels, lib/kernels/src/cuda/metrics_functions.cu:48-98,
accumulate the same sums with atomics).  ``StepLogger`` writes one JSON line per step.
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
        self.__init__()

    def update(self, pred: torch.Tensor, label: torch.Tensor, metrics: Iterable[str] = ("accuracy",)):
        """pred: [N, C] probabilities or values; label: [N] class ids (sparse) or [N, C] targets."""
        p = pred.detach().float().reshape(-1, pred.shape[-1])
        n = p.shape[0]
        sparse = label.dim() == 1 or label.numel() == n
        self.train_all += n
        if "accuracy" in metrics:
            tgt = label.reshape(-1).long() if sparse else label.reshape(n, -1).argmax(1)
            self.train_correct += int((p.argmax(1).to(tgt.device) == tgt).sum().item())
        if sparse and "sparse_categorical_crossentropy" in metrics:
            tgt = label.reshape(-1).long().to(p.device)
            self.sparse_cce_loss += float(-torch.log(p.gather(1, tgt[:, None]).clamp_min(1e-30)).sum().item())
        if not sparse:
            t = label.reshape(n, -1).float().to(p.device)
            if "categorical_crossentropy" in metrics:
                self.cce_loss += float(-(t * torch.log(p.clamp_min(1e-30))).sum().item())
            d = p - t
            if "mean_squared_error" in metrics:
                self.mse_loss += float((d * d).mean(1).sum().item())
            if "root_mean_squared_error" in metrics:
                self.rmse_loss += float((d * d).mean(1).sqrt().sum().item())
            if "mean_absolute_error" in metrics:
                self.mae_loss += float(d.abs().mean(1).sum().item())
        self.current_time = time.time()
        return self

    @property
    def accuracy(self) -> float:
        return self.train_correct / max(self.train_all, 1)

    def throughput(self) -> float:
        return self.train_all / max(self.current_time - self.start_time, 1e-9)

    def summary(self) -> dict:
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
