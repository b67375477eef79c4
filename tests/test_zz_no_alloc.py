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


def _case(fn, rows, cols, dtype, seed):
    from flexflow_train_b200.ops import kernels as K

    torch.manual_seed(seed)
    dev = "cuda"
    x = torch.randn(rows, cols, device=dev, dtype=dtype)
    dy = torch.randn(rows, cols, device=dev, dtype=dtype)
    gamma = torch.randn(cols, device=dev, dtype=dtype)
    xf = x.float()
    mean = xf.mean(1).contiguous()
    rstd = torch.rsqrt(xf.var(1, unbiased=False) + 1e-5).contiguous()
    # regular entry point: scratch supplied by the caller
    dx_ref, dg_ref, db_ref = torch.empty_like(x), torch.empty_like(gamma), torch.empty_like(gamma)
    scratch = torch.empty(K.layernorm_bwd_scratch(rows, cols), device=dev)
    K.layernorm_bwd(dy, x, gamma, mean, rstd, dx_ref, dg_ref, db_ref, scratch)
    # allocation-free entry point: inputs and outputs only
    dx, dg, db = torch.empty_like(x), torch.empty_like(gamma), torch.empty_like(gamma)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dg.data_ptr(),
            db.data_ptr(), rows, cols, 1 if dtype == torch.bfloat16 else 0, stream)
    assert rc == 0
    torch.cuda.synchronize()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert _rel(dx, dx_ref) < tol
    assert _rel(dg, dg_ref) < tol
    assert _rel(db, db_ref) < tol


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    fn = _entry()
    # second call: different shape and data, so stale partial sums of the first would show up
    _case(fn, 300, 2048, torch.bfloat16, seed=1)
    _case(fn, 77, 1000, torch.float32, seed=2)
    _case(fn, 300, 2048, torch.bfloat16, seed=3)


def test_noalloc_rejects_oversize():
    fn = _entry()
    x = torch.zeros(8, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), None, x.data_ptr(), x.data_ptr(), x.data_ptr(), None, None, 4, 16385, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -2
    rc = fn(x.data_ptr(), x.data_ptr(), None, x.data_ptr(), x.data_ptr(), x.data_ptr(), None, None, 0, 16, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -2
