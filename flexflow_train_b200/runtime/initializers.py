"""Weight initializers (all eight ``InitializerAttrs`` kinds of the reference,
lib/op-attrs/include/op-attrs/initializer_attrs.dtg.toml), seeded and shard-consistent.

A weight is always initialised as the *whole* logical tensor from a generator
seeded by ``(global seed, initializer seed, weight ordinal)`` and then sliced to
the local shard, so every rank that holds a copy (or a piece) of the weight sees
the same values regardless of the parallelisation strategy.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch


def _fans(shape: Sequence[int]):
    if len(shape) < 2:
        n = shape[0] if shape else 1
        return n, n
    receptive = 1
    for s in shape[2:]:
        receptive *= s
    return shape[1] * receptive, shape[0] * receptive


def initialize(shape: Sequence[int], init: dict | None, *, base_seed: int = 0, ordinal: int = 0,
               device="cpu") -> torch.Tensor:
    """Return a float32 tensor of ``shape`` filled according to ``init`` ({"type", "value"})."""
    shape = tuple(int(s) for s in shape)
    kind = (init or {}).get("type", "zero")
    v = (init or {}).get("value", {}) or {}
    gen = torch.Generator(device=device)
    gen.manual_seed((int(base_seed) * 1000003 + int(v.get("seed", 0)) * 7919 + ordinal * 104729 + 17) % (2 ** 63))
    out = torch.empty(shape, dtype=torch.float32, device=device)
    if kind == "zero":
        out.zero_()
    elif kind == "constant":
        c = v.get("value", 0.0)
        if isinstance(c, dict):
            c = c.get("value", 0.0)
        out.fill_(float(c))
    elif kind == "uniform":
        out.uniform_(float(v.get("min_val", 0.0)), float(v.get("max_val", 1.0)), generator=gen)
    elif kind in ("normal", "norm"):
        out.normal_(float(v.get("mean", 0.0)), float(v.get("stddev", 1.0)), generator=gen)
    elif kind == "truncated_normal":
        mean, std = float(v.get("mean", 0.0)), float(v.get("stddev", 1.0))
        lo, hi = float(v.get("min_cutoff", mean - 2 * std)), float(v.get("max_cutoff", mean + 2 * std))
        out.normal_(mean, std, generator=gen)
        for _ in range(8):  # resample the tails
            bad = (out < lo) | (out > hi)
            if not bool(bad.any()):
                break
            fresh = torch.empty_like(out).normal_(mean, std, generator=gen)
            out = torch.where(bad, fresh, out)
        out.clamp_(lo, hi)
    elif kind == "glorot_uniform":
        fan_in, fan_out = _fans(shape)
        a = math.sqrt(6.0 / (fan_in + fan_out))
        out.uniform_(-a, a, generator=gen)
    elif kind == "glorot_normal":
        fan_in, fan_out = _fans(shape)
        out.normal_(0.0, math.sqrt(2.0 / (fan_in + fan_out)), generator=gen)
    elif kind == "kaiming_normal":
        fan_in, fan_out = _fans(shape)
        fan = fan_out if str(v.get("mode", "fan_in")).lower() == "fan_out" else fan_in
        a = float(v.get("a", 0.0))
        nl = str(v.get("nonlinearity", "leaky_relu")).lower()
        gain = math.sqrt(2.0) if nl == "relu" else (math.sqrt(2.0 / (1 + a * a)) if nl == "leaky_relu" else 1.0)
        out.normal_(0.0, gain / math.sqrt(max(fan, 1)), generator=gen)
    else:
        raise ValueError(f"unknown initializer kind {kind!r}")
    return out


INITIALIZER_KINDS = ("glorot_uniform", "glorot_normal", "kaiming_normal", "zero", "uniform", "normal",
                     "truncated_normal", "constant")
