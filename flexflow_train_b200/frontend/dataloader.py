"""Data loader: whole data sets stay in page-locked host memory, batches are assembled on the GPU.

For every batch one kernel per array (`ops.kernels.load_rows`) gathers the batch's samples -- by index, so a shuffled epoch
costs no host-side gather -- straight out of host memory into a device buffer of a small ring, on a side stream, while the
previous step is still computing; `next_batch()` hands out buffers whose copies have finished.  The reference's loaders
(bindings/python/old/flexflow_dataloader.{h,cc,cu}: SingleDataLoader with the full data set in zero-copy memory and a
load task per batch) work the same way; without a GPU the loader falls back to host slicing.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from ..ops import kernels as K

Array = Union[np.ndarray, torch.Tensor]


class DataLoader:
    """Batches of several aligned arrays (inputs by name, optionally labels).

    `arrays`: name -> [num_samples, ...] array.  `drop_last` batches only (the executors are compiled for one batch size).
    `shuffle` draws a new permutation per epoch from `seed`; `prefetch` is the depth of the device-buffer ring."""

    def __init__(self, arrays: Dict[str, Array], batch_size: int, *, shuffle: bool = False, seed: int = 0, prefetch: int = 2,
                 device: Optional[str] = None):
        if not arrays:
            raise ValueError("no arrays to load")
        self.names = list(arrays)
        self.batch_size = int(batch_size)
        tens = {k: (v if torch.is_tensor(v) else torch.as_tensor(np.ascontiguousarray(v))).contiguous() for k, v in arrays.items()}
        ns = {int(t.shape[0]) for t in tens.values()}
        if len(ns) != 1:
            raise ValueError(f"arrays disagree on the number of samples: {sorted(ns)}")
        self.num_samples = ns.pop()
        if self.batch_size <= 0 or self.batch_size > self.num_samples:
            raise ValueError("batch size must be between 1 and the number of samples")
        self.num_batches = self.num_samples // self.batch_size
        self.shuffle, self.seed, self.epoch = shuffle, seed, 0
        self.on_gpu = torch.cuda.is_available() and (device is None or str(device).startswith("cuda"))
        self.device = torch.device(device or ("cuda" if self.on_gpu else "cpu"))
        if self.on_gpu:
            K.lib()
            self.data = {k: t.pin_memory() for k, t in tens.items()}
            self.stream = torch.cuda.Stream(device=self.device)
            depth = max(1, int(prefetch))
            self.ring = [{k: torch.empty((self.batch_size,) + tuple(t.shape[1:]), dtype=t.dtype, device=self.device) for k, t in tens.items()}
                         for _ in range(depth + 1)]
            self.ready = [torch.cuda.Event() for _ in self.ring]
            self.consumed = [None] * len(self.ring)   # event after which a buffer may be overwritten
        else:
            self.data = tens
        self.reset()

    def __len__(self) -> int:
        return self.num_batches

    def _order(self) -> torch.Tensor:
        if not self.shuffle:
            return torch.arange(self.num_samples, dtype=torch.int64)
        g = torch.Generator().manual_seed(self.seed + self.epoch)
        return torch.randperm(self.num_samples, generator=g)

    def reset(self):
        """Start a new epoch (a new permutation when shuffling)."""
        self.order = self._order()
        self.order_dev = self.order.to(self.device) if self.on_gpu else None
        self.epoch += 1
        self.issued = 0      # batches whose copies were launched
        self.taken = 0       # batches handed out
        if self.on_gpu:
            # work queued so far may still read batches of the previous epoch: no buffer is overwritten before it has run
            e = torch.cuda.Event()
            e.record()
            self.consumed = [e] * len(self.ring)
            for _ in range(len(self.ring) - 1):
                self._issue()

    def _issue(self):
        if self.issued >= self.num_batches:
            return
        slot = self.issued % len(self.ring)
        with torch.cuda.stream(self.stream):
            if self.consumed[slot] is not None:          # whoever read this buffer last has finished
                self.stream.wait_event(self.consumed[slot])
            idx = self.order_dev[self.issued * self.batch_size:(self.issued + 1) * self.batch_size]
            for k in self.names:
                if self.shuffle:
                    K.load_rows(self.data[k], self.ring[slot][k], indices=idx)
                else:
                    K.load_rows(self.data[k], self.ring[slot][k], first=self.issued * self.batch_size)
            self.ready[slot].record(self.stream)
        self.issued += 1

    def next_batch(self) -> Dict[str, torch.Tensor]:
        """The next batch (device tensors valid on the current stream until the ring comes round again)."""
        if self.taken >= self.num_batches:
            self.reset()
        if not self.on_gpu:
            rows = self.order[self.taken * self.batch_size:(self.taken + 1) * self.batch_size]
            self.taken += 1
            return {k: self.data[k][rows] for k in self.names}
        slot = self.taken % len(self.ring)
        torch.cuda.current_stream().wait_event(self.ready[slot])
        batch = self.ring[slot]
        # the buffer handed out one ring-turn ago is free once the work queued so far has run
        prev = (self.taken - 1) % len(self.ring)
        if self.taken > 0:
            e = torch.cuda.Event()
            e.record()
            self.consumed[prev] = e
        self.taken += 1
        self._issue()
        return batch

    def __iter__(self):
        self.reset()
        for _ in range(self.num_batches):
            yield self.next_batch()

    def sample_indices(self, batch: int) -> torch.Tensor:
        """Which samples batch `batch` of the current epoch holds (host tensor)."""
        return self.order[batch * self.batch_size:(batch + 1) * self.batch_size]
