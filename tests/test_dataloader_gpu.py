"""The device-side data loader: batches gathered by index out of page-locked host memory, prefetched on a side stream."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from flexflow_train_b200.frontend.dataloader import DataLoader  # noqa: E402
from flexflow_train_b200.ops import kernels as K  # noqa: E402


def test_load_rows_by_index_and_by_range():
    torch.manual_seed(0)
    for shape, dtype in (((1000, 3, 7), torch.float32), ((513, 24), torch.bfloat16), ((300, 5), torch.int32), ((64, 1), torch.int64)):
        data = (torch.randn(shape) * 100).to(dtype).pin_memory()
        idx = torch.randint(0, shape[0], (37,), dtype=torch.int64, device="cuda")
        out = torch.empty((37,) + shape[1:], dtype=dtype, device="cuda")
        K.load_rows(data, out, indices=idx)
        assert torch.equal(out.cpu(), data[idx.cpu()])
        K.load_rows(data, out, first=11)
        assert torch.equal(out.cpu(), data[11:48])
    with pytest.raises(K.KernelError):
        K.load_rows(torch.zeros(10, 4), torch.empty(2, 4, device="cuda"))   # pageable host memory


@pytest.mark.parametrize("shuffle", [False, True])
def test_loader_covers_every_sample_once_per_epoch(shuffle):
    n, bs = 1000, 64
    x = np.arange(n * 6, dtype=np.float32).reshape(n, 2, 3)
    y = np.arange(n, dtype=np.int32)
    dl = DataLoader({"x": x, "labels": y}, bs, shuffle=shuffle, seed=3, prefetch=3)
    assert len(dl) == n // bs
    for epoch in range(2):
        seen = []
        for b, batch in enumerate(dl):
            want = dl.sample_indices(b)
            assert torch.equal(batch["labels"].cpu().long(), want)
            assert torch.equal(batch["x"].cpu(), torch.from_numpy(x)[want])
            seen.append(batch["labels"].cpu())
        seen = torch.cat(seen)
        assert seen.numel() == (n // bs) * bs and seen.unique().numel() == seen.numel()
        if not shuffle:
            assert torch.equal(seen.long(), torch.arange(seen.numel()))
    if shuffle:   # a new permutation each epoch
        first = dl.sample_indices(0).clone()
        dl.reset()
        assert not torch.equal(first, dl.sample_indices(0))


def test_batches_stay_valid_while_later_ones_are_prefetched():
    """A batch is consumed by work queued on the current stream after the loader already launched the copies of the next
    batches: the ring must not let a copy overwrite a buffer that queued work still reads."""
    n, bs = 4096, 256
    x = torch.arange(n * 512, dtype=torch.float32).reshape(n, 512)
    dl = DataLoader({"x": x}, bs, prefetch=1)
    sums = []
    for batch in dl:
        t = batch["x"]
        for _ in range(20):          # keep the stream busy so that the consumer runs late
            t = t * 1.0
        sums.append(t.sum(dtype=torch.float64))
    got = torch.stack(sums).cpu()
    want = x.reshape(n // bs, bs * 512).sum(dim=1, dtype=torch.float64)
    assert torch.equal(got, want)
