"""The allocation-free LayerNorm backward (``ffk_layernorm_bwd_noalloc``), called the way its users call it:
straight through the exported C symbol of ``libffk.so`` with raw device pointers.

Its users are programs that cannot hand the library a workspace -- plug-ins inside an application that owns the
device heap, serving loops that must not hit the implicit synchronisation of ``cudaMalloc``/``cudaFree``, C code
with no tensor framework -- so the scratch lives inside the library.  The check: two calls in a row (the second
sees the first one's leftovers in the shared scratch) must each agree with the regular entry point, which takes
its scratch from the caller.  The file name sorts last so that a run that stops at the first failure has already
run everything else.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "flexflow_train_b200", "libffk.so")


def _entry():
    lib = ctypes.CDLL(LIB)
    fn = lib.ffk_layernorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return fn


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _autograd_reference(x, dy, gamma):
    """fp32 PyTorch autograd result of layer_norm over the last dim for the same inputs."""
    xf = x.float().clone().requires_grad_(True)
    gf = gamma.float().clone().requires_grad_(True) if gamma is not None else None
    bf = torch.zeros(x.shape[1], device=x.device, requires_grad=True)
    y = torch.nn.functional.layer_norm(xf, (x.shape[1],), gf, bf, 1e-5)
    y.backward(dy.float())
    return xf.grad, (gf.grad if gf is not None else None), bf.grad


def _case(fn, rows, cols, dtype, seed, with_gamma=True, with_param_grads=True):
    from flexflow_train_b200.ops import kernels as K

    torch.manual_seed(seed)
    dev = "cuda"
    x = torch.randn(rows, cols, device=dev, dtype=dtype)
    dy = torch.randn(rows, cols, device=dev, dtype=dtype)
    gamma = torch.randn(cols, device=dev, dtype=dtype) if with_gamma else None
    xf = x.float()
    mean = xf.mean(1).contiguous()
    rstd = torch.rsqrt(xf.var(1, unbiased=False) + 1e-5).contiguous()
    # regular entry point: scratch supplied by the caller
    dx_ref = torch.empty_like(x)
    dg_ref, db_ref = torch.empty(cols, device=dev, dtype=dtype), torch.empty(cols, device=dev, dtype=dtype)
    scratch = torch.empty(K.layernorm_bwd_scratch(rows, cols), device=dev)
    K.layernorm_bwd(dy, x, gamma, mean, rstd, dx_ref, dg_ref, db_ref, scratch)
    # allocation-free entry point: inputs and outputs only
    dx = torch.empty_like(x)
    dg, db = (torch.empty_like(dg_ref), torch.empty_like(db_ref)) if with_param_grads else (None, None)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(dy.data_ptr(), x.data_ptr(), gamma.data_ptr() if with_gamma else None, mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
            dg.data_ptr() if with_param_grads else None, db.data_ptr() if with_param_grads else None, rows, cols,
            1 if dtype == torch.bfloat16 else 0, stream)
    assert rc == 0
    torch.cuda.synchronize()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert _rel(dx, dx_ref) < tol
    # and against fp32 PyTorch autograd of the same layer norm
    ax, ag, ab = _autograd_reference(x, dy, gamma)
    assert _rel(dx, ax) < tol
    if with_param_grads:
        assert _rel(dg, dg_ref) < tol and _rel(db, db_ref) < tol
        assert _rel(db, ab) < tol
        if with_gamma:
            assert _rel(dg, ag) < tol


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    fn = _entry()
    # second call: different shape and data, so stale partial sums of the first would show up
    _case(fn, 300, 2048, torch.bfloat16, seed=1)
    _case(fn, 77, 1000, torch.float32, seed=2)
    _case(fn, 300, 2048, torch.bfloat16, seed=3)


def test_noalloc_few_rows_and_optional_pointers():
    fn = _entry()
    _case(fn, 5, 384, torch.float32, seed=4)                           # fewer rows than blocks
    _case(fn, 1, 64, torch.bfloat16, seed=5)
    _case(fn, 40, 512, torch.float32, seed=6, with_gamma=False)        # no scale
    _case(fn, 130, 768, torch.bfloat16, seed=7, with_param_grads=False)  # dx only
    _case(fn, 5, 384, torch.float32, seed=8)                           # after the above, leftovers in the scratch


def test_noalloc_rejects_oversize():
    fn = _entry()
    x = torch.zeros(8, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), None, x.data_ptr(), x.data_ptr(), x.data_ptr(), None, None, 4, 16385, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -2
    rc = fn(x.data_ptr(), x.data_ptr(), None, x.data_ptr(), x.data_ptr(), x.data_ptr(), None, None, 0, 16, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -2
