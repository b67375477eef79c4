"""Numerics of the hand-written sm_100a kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from flexflow_train_b200.ops import kernels as k  # noqa: E402

DEV = "cuda"


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("M,N,K,bn", [(256, 256, 128, 128), (300, 200, 136, 0), (128, 512, 1024, 256), (64, 64, 64, 64)])
def test_gemm_nt_bf16(M, N, K, bn):
    torch.manual_seed(1)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    out = k.matmul_nt(a, b, bn=bn)
    ref = a.float() @ b.float().t()
    assert k.gemm_last_error() == 0
    assert rel(out, ref) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (384, 520, 264)])
def test_gemm_nn_tn_bf16(M, N, K):
    torch.manual_seed(2)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    assert rel(k.matmul_nn(a, b), a.float() @ b.float()) < 1e-2
    at = torch.randn(K, M, device=DEV, dtype=torch.bfloat16)
    assert rel(k.matmul_tn(at, b), at.float().t() @ b.float()) < 1e-2
    assert k.gemm_last_error() == 0


def test_gemm_tf32():
    torch.manual_seed(3)
    a = torch.randn(256, 160, device=DEV)
    b = torch.randn(192, 160, device=DEV)
    assert rel(k.matmul_nt(a, b), a @ b.t()) < 3e-3
    b2 = torch.randn(160, 192, device=DEV)
    assert rel(k.matmul_nn(a, b2), a @ b2) < 3e-3
    a2 = torch.randn(160, 256, device=DEV)
    assert rel(k.matmul_tn(a2, b2), a2.t() @ b2) < 3e-3
    assert k.gemm_last_error() == 0


def test_gemm_epilogue_and_accumulate():
    torch.manual_seed(4)
    M, N, K = 512, 768, 256
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    add = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    pre = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    out = k.matmul_nt(a, b, bias=bias, act="gelu", addend=add, pre_act_out=pre, alpha=0.5)
    refpre = 0.5 * (a.float() @ b.float().t()) + bias.float()
    ref = torch.nn.functional.gelu(refpre) + add.float()
    assert rel(pre, refpre) < 1e-2
    assert rel(out, ref) < 1e-2
    acc = torch.ones(M, N, device=DEV, dtype=torch.float32)
    k.matmul_nt(a, b, out=acc, accumulate=True)
    assert rel(acc, 1.0 + a.float() @ b.float().t()) < 1e-2


def test_gemm_batched_strided():
    torch.manual_seed(5)
    B, S, H, D = 2, 256, 4, 64
    q = torch.randn(B, S, H, D, device=DEV, dtype=torch.bfloat16)
    kk = torch.randn(B, S, H, D, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(B, H, S, S, device=DEV, dtype=torch.bfloat16)
    k.gemm_raw(M=S, N=S, K=D, A=q.data_ptr(), lda=H * D, a_sh=D, a_sb=S * H * D, B=kk.data_ptr(), ldb=H * D,
               b_sh=D, b_sb=S * H * D, C=out.data_ptr(), ldc=S, c_sh=S * S, c_sb=H * S * S, nh=H, nb=B)
    ref = torch.einsum("bshd,bthd->bhst", q.float(), kk.float())
    assert rel(out, ref) < 1e-2
    # P @ V with V taken as an MN-major operand: o[b,s,h,:] = sum_t p[b,h,s,t] v[b,t,h,:]
    p = torch.softmax(ref, -1).to(torch.bfloat16)
    v = torch.randn(B, S, H, D, device=DEV, dtype=torch.bfloat16)
    o = torch.empty(B, S, H, D, device=DEV, dtype=torch.bfloat16)
    k.gemm_raw(M=S, N=D, K=S, A=p.data_ptr(), lda=S, a_sh=S * S, a_sb=H * S * S, B=v.data_ptr(), ldb=H * D,
               b_mn=True, b_sh=D, b_sb=S * H * D, C=o.data_ptr(), ldc=H * D, c_sh=D, c_sb=S * H * D, nh=H, nb=B)
    assert rel(o, torch.einsum("bhst,bthd->bshd", p.float(), v.float())) < 1e-2
    assert k.gemm_last_error() == 0


@pytest.mark.parametrize("M,N,K", [(4096, 512, 13), (100, 1, 256), (37, 145, 4099), (9, 9, 64), (70, 33, 31)])
def test_gemm_general_shape_kernel_all_layouts(M, N, K):
    """Operands whose row pitch is not a multiple of 16 bytes cannot be described to TMA and take the CUDA-core
    kernel: every layout, tiles cut by all three extents, the epilogue, batches and a long reduction dim."""
    torch.manual_seed(6)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    tol = 2e-2
    assert rel(k.matmul_nt(a, b), ref) < tol
    assert rel(k.matmul_nt(a, b, bias=bias, act="relu"), torch.relu(ref + bias.float())) < tol
    bt = b.t().contiguous()  # [K, N]
    assert rel(k.matmul_nn(a, bt), ref) < tol
    at = a.t().contiguous()  # [K, M]
    assert rel(k.matmul_tn(at, bt), ref) < tol
    acc = torch.ones(M, N, device=DEV, dtype=torch.float32)
    k.matmul_tn(at, bt, out=acc, accumulate=True)
    assert rel(acc, 1.0 + ref) < tol
    if M * N <= 4096:  # a batch of small problems, strided
        nb = 5
        x = torch.randn(nb, M, K, device=DEV, dtype=torch.bfloat16)
        w = torch.randn(nb, N, K, device=DEV, dtype=torch.bfloat16)
        out = torch.empty(nb, M, N, device=DEV, dtype=torch.bfloat16)
        k.gemm_raw(M=M, N=N, K=K, A=x.data_ptr(), lda=K, a_sb=M * K, B=w.data_ptr(), ldb=K, b_sb=N * K, C=out.data_ptr(), ldc=N,
                   c_sb=M * N, nb=nb)
        assert rel(out, torch.einsum("bmk,bnk->bmn", x.float(), w.float())) < tol
    assert k.gemm_last_error() == 0


@pytest.mark.parametrize("M,N,K", [(9, 9, 64), (64, 9, 9), (9, 64, 9), (32, 32, 35), (1, 7, 130)])
def test_gemm_batches_of_small_problems(M, N, K):
    """One warp per problem: K-major and MN-major operands, aligned or not, with the epilogue."""
    torch.manual_seed(7)
    nb = 300
    x = torch.randn(nb, M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(nb, N, K, device=DEV, dtype=torch.bfloat16)
    ref = torch.einsum("bmk,bnk->bmn", x.float(), w.float())
    out = torch.empty(nb, M, N, device=DEV, dtype=torch.bfloat16)
    k.gemm_raw(M=M, N=N, K=K, A=x.data_ptr(), lda=K, a_sb=M * K, B=w.data_ptr(), ldb=K, b_sb=N * K, C=out.data_ptr(), ldc=N, c_sb=M * N, nb=nb)
    assert rel(out, ref) < 1e-2
    xt = x.transpose(1, 2).contiguous()  # [nb, K, M]
    wt = w.transpose(1, 2).contiguous()  # [nb, K, N]
    acc = torch.ones(nb, M, N, device=DEV, dtype=torch.float32)
    k.gemm_raw(M=M, N=N, K=K, A=xt.data_ptr(), lda=M, a_mn=True, a_sb=M * K, B=wt.data_ptr(), ldb=N, b_mn=True, b_sb=N * K,
               C=acc.data_ptr(), ldc=N, c_sb=M * N, nb=nb, out_fp32=True, accumulate=True, alpha=0.5)
    assert rel(acc, 1.0 + 0.5 * ref) < 1e-2
    assert k.gemm_last_error() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unary_binary(dtype):
    torch.manual_seed(6)
    x = torch.randn(1000, 37, device=DEV, dtype=dtype)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    refs = {"relu": torch.relu, "sigmoid": torch.sigmoid, "tanh": torch.tanh, "gelu": torch.nn.functional.gelu,
            "exp": torch.exp, "sin": torch.sin, "cos": torch.cos, "elu": torch.nn.functional.elu}
    for name, fn in refs.items():
        y = k.unary_fwd(name, x)
        assert rel(y, fn(x.float())) < tol, name
        xr = x.float().clone().requires_grad_(True)
        yr = fn(xr)
        dy = torch.randn_like(x)
        yr.backward(dy.float())
        dx = k.unary_bwd(name, x, y, dy)
        assert rel(dx, xr.grad) < 3 * tol, name
    y = k.unary_fwd("scalar_multiply", x, scalar=2.5)
    assert rel(y, x.float() * 2.5) < tol
    xp = x.abs() + 0.5
    assert rel(k.unary_fwd("rsqrt", xp), torch.rsqrt(xp.float())) < tol
    assert rel(k.unary_fwd("pow", xp, scalar=2.0), xp.float() ** 2) < tol
    b = torch.randn_like(x)
    for name, fn in {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "max": torch.maximum,
                     "min": torch.minimum}.items():
        assert rel(k.binary_fwd(name, x, b), fn(x.float(), b.float())) < tol, name
    row = torch.randn(37, device=DEV, dtype=dtype)
    assert rel(k.binary_fwd("add", x, row), x.float() + row.float()) < tol
    da, db = torch.empty_like(x), torch.empty_like(x)
    dy = torch.randn_like(x)
    k.binary_bwd("mul", x, b, dy, da, db)
    assert rel(da, dy.float() * b.float()) < tol and rel(db, dy.float() * x.float()) < tol


def test_dropout_cast_axpby():
    x = torch.ones(1 << 20, device=DEV, dtype=torch.bfloat16)
    y = k.dropout(x, 0.25, seed=123)
    keep = (y != 0).float().mean().item()
    assert abs(keep - 0.75) < 0.01
    assert torch.allclose(y[y != 0].float(), torch.tensor(1 / 0.75, device=DEV), atol=1e-2)
    y2 = k.dropout(x, 0.25, seed=123)
    assert torch.equal(y, y2)
    f = torch.randn(1001, device=DEV)
    h = torch.empty(1001, device=DEV, dtype=torch.bfloat16)
    k.cast(f, h)
    assert torch.equal(h, f.to(torch.bfloat16))
    i = torch.empty(1001, device=DEV, dtype=torch.int32)
    k.cast(f * 10, i)
    assert torch.equal(i, (f * 10).to(torch.int32))
    yy = torch.ones(1001, device=DEV)
    k.axpby(f, yy, 2.0, 3.0)
    assert torch.allclose(yy, 2 * f + 3, atol=1e-5)


@pytest.mark.parametrize("dtype,rows,cols", [(torch.bfloat16, 512, 2048), (torch.float32, 33, 100), (torch.bfloat16, 64, 768)])
def test_layernorm(dtype, rows, cols):
    torch.manual_seed(7)
    x = torch.randn(rows, cols, device=DEV, dtype=dtype)
    r = torch.randn(rows, cols, device=DEV, dtype=dtype)
    g = torch.randn(cols, device=DEV, dtype=dtype)
    b = torch.randn(cols, device=DEV, dtype=dtype)
    mean = torch.empty(rows, device=DEV)
    rstd = torch.empty(rows, device=DEV)
    xsum = torch.empty_like(x)
    y = k.layernorm_fwd(x, g, b, 1e-5, residual=r, xsum=xsum, mean=mean, rstd=rstd)
    xs = xsum.float().clone().requires_grad_(True)
    gr = g.float().clone().requires_grad_(True)
    br = b.float().clone().requires_grad_(True)
    ref = torch.nn.functional.layer_norm(xs, (cols,), gr, br, 1e-5)
    tol = 1e-4 if dtype == torch.float32 else 1e-2
    assert rel(xsum, x.float() + r.float()) < tol
    assert rel(y, ref) < tol
    dy = torch.randn_like(x)
    ref.backward(dy.float())
    dx = torch.empty_like(x)
    dg = torch.empty_like(g)
    db = torch.empty_like(b)
    scratch = torch.empty(k.layernorm_bwd_scratch(rows, cols), device=DEV)
    k.layernorm_bwd(dy, xsum, g, mean, rstd, dx, dg, db, scratch)
    assert rel(dx, xs.grad) < 2 * tol
    assert rel(dg, gr.grad) < 2 * tol
    assert rel(db, br.grad) < 2 * tol


def test_softmax_and_ce():
    torch.manual_seed(8)
    x = torch.randn(64, 16, 300, device=DEV, dtype=torch.bfloat16)
    y = k.softmax_fwd(x, scale=0.5)
    ref = torch.softmax(x.float() * 0.5, -1)
    assert rel(y, ref) < 1e-2
    dy = torch.randn_like(x)
    xr = x.float().clone().requires_grad_(True)
    torch.softmax(xr * 0.5, -1).backward(dy.float())
    assert rel(k.softmax_bwd(dy, y, scale=0.5), xr.grad) < 2e-2
    # causal
    s = torch.randn(2 * 128, 128, device=DEV)
    yc = k.softmax_fwd(s, causal_q=128)
    mask = torch.tril(torch.ones(128, 128, device=DEV)).repeat(2, 1).bool()
    assert rel(yc, torch.softmax(s.masked_fill(~mask, -1e30), -1)) < 1e-5
    logits = torch.randn(257, 1000, device=DEV)
    labels = torch.randint(0, 1000, (257,), device=DEV)
    loss = torch.empty(257, device=DEV)
    dl = torch.empty_like(logits)
    probs = torch.empty_like(logits)
    k.softmax_ce(logits, labels, loss, dl, probs, grad_scale=1 / 257)
    lr = logits.clone().requires_grad_(True)
    lref = torch.nn.functional.cross_entropy(lr, labels, reduction="none")
    lref.mean().backward()
    assert rel(loss, lref) < 1e-5
    assert rel(dl, lr.grad) < 1e-4
    assert rel(probs, torch.softmax(logits, -1)) < 1e-5
    d2 = torch.empty_like(logits)
    k.loss_bwd("sparse_categorical_crossentropy", probs, labels, d2, 1 / 257)
    assert rel(d2, lr.grad) < 1e-4
    lrow = torch.empty(257, device=DEV)
    k.loss_fwd("sparse_categorical_crossentropy", probs, labels, lrow)
    assert rel(lrow, lref) < 1e-4


def test_bias_act_bwd():
    torch.manual_seed(9)
    rows, cols = 1000, 520
    pre = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16)
    dy = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16)
    dz = torch.empty_like(dy)
    dbias = torch.empty(cols, device=DEV, dtype=torch.bfloat16)
    scratch = torch.empty(k.bias_act_bwd_scratch(rows, cols), device=DEV)
    k.bias_act_bwd(dy, pre, dz, dbias, scratch, "gelu")
    pr = pre.float().clone().requires_grad_(True)
    torch.nn.functional.gelu(pr).backward(dy.float())
    assert rel(dz, pr.grad) < 1e-2
    assert rel(dbias, pr.grad.sum(0)) < 1e-2


def test_optimizers():
    torch.manual_seed(10)
    n = 100003
    w = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV).to(torch.bfloat16)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    shadow = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    wr = w.clone()
    opt_m, opt_v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    lr, b1, b2, eps = 1e-3, 0.9, 0.999, 1e-8
    for t in range(1, 4):
        alpha_t = lr * math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
        k.adam_update(w, m, v, g, shadow, alpha_t, b1, b2, eps)
        gf = g.float()
        opt_m = b1 * opt_m + (1 - b1) * gf
        opt_v = b2 * opt_v + (1 - b2) * gf * gf
        wr = wr - alpha_t * opt_m / (opt_v.sqrt() + eps)
    assert torch.allclose(w, wr, atol=1e-5)
    assert torch.equal(shadow, w.to(torch.bfloat16))
    w2 = torch.randn(n, device=DEV)
    w2r = w2.clone()
    mom = torch.zeros(n, device=DEV)
    momr = torch.zeros(n, device=DEV)
    gf = torch.randn(n, device=DEV)
    for _ in range(3):
        k.sgd_update(w2, mom, gf, None, 0.1, momentum=0.9, nesterov=True, weight_decay=0.01)
        gt = gf + 0.01 * w2r
        momr = momr * 0.9 + gt
        w2r = w2r - 0.1 * (gt + 0.9 * momr)
    assert torch.allclose(w2, w2r, atol=1e-5)


def test_embedding():
    torch.manual_seed(11)
    table = torch.randn(1000, 64, device=DEV)
    idx = torch.randint(0, 1000, (128, 3), device=DEV)
    out = torch.empty(128, 64, device=DEV, dtype=torch.bfloat16)
    k.embedding_fwd(idx, table, out.view(128, 64), aggr="sum") if False else None
    out2 = torch.empty(128, 3, 64, device=DEV)
    k.embedding_fwd(idx, table, out2)
    assert torch.allclose(out2, table[idx])
    dt = torch.zeros_like(table)
    dout = torch.randn(128, 3, 64, device=DEV)
    k.embedding_bwd(idx, dout, dt)
    ref = torch.zeros_like(table).index_add_(0, idx.reshape(-1), dout.reshape(-1, 64))
    assert torch.allclose(dt, ref, atol=1e-4)


def test_dropout_fused_into_gemm_epilogue_and_its_backward_use_the_standalone_mask(K=k):
    """matmul_nt(..., dropout=) must draw exactly the mask of the stand-alone dropout kernel for the same
    (salt, step seed), and bias_act_bwd(..., dropout=) must take the gradient back through that mask."""
    torch.manual_seed(0)
    m, n, k, p, salt = 512, 384, 256, 0.25, 0x1234567
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = torch.randn(n, k, device="cuda").to(torch.bfloat16)
    bias = torch.randn(n, device="cuda").to(torch.bfloat16)
    seed = torch.tensor([987654321], dtype=torch.int64, device="cuda")
    pre = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    fused = K.matmul_nt(x, w, bias=bias, act="gelu", pre_act_out=pre, dropout=(p, salt, seed))
    plain = K.matmul_nt(x, w, bias=bias, act="gelu")
    ref = torch.empty_like(plain)
    K.dropout(plain, p, salt, out=ref, seed_tensor=seed)
    assert torch.equal(fused == 0, ref == 0)                      # the same elements are dropped
    live = plain != 0                                             # GELU is exactly 0 for very negative inputs
    frac = float((fused[live] == 0).float().mean())
    assert abs(frac - p) < 0.02
    assert ((fused.float() - ref.float()).abs() <= 0.02 * ref.float().abs() + 1e-3).all()
    # backward: dz = gelu'(pre) * dropout_mask(dy) / (1 - p); bias gradient = column sums
    dy = torch.randn(m, n, device="cuda").to(torch.bfloat16)
    scratch = torch.empty(K.bias_act_bwd_scratch(m, n), device="cuda")
    dz, db = torch.empty_like(dy), torch.empty(n, device="cuda", dtype=torch.bfloat16)
    K.bias_act_bwd(dy, pre, dz, db, scratch, "gelu", dropout=(p, salt, seed))
    dmask = torch.empty_like(dy)
    K.dropout(dy, p, salt, out=dmask, seed_tensor=seed)
    dz2, db2 = torch.empty_like(dy), torch.empty_like(db)
    K.bias_act_bwd(dmask, pre, dz2, db2, scratch, "gelu")
    assert torch.equal(dz == 0, dz2 == 0)
    assert rel(dz, dz2) < 1e-2 and rel(db, db2) < 2e-2
    # a different step seed draws a different mask
    seed2 = seed + 1
    other = K.matmul_nt(x, w, bias=bias, act="gelu", dropout=(p, salt, seed2))
    assert not torch.equal(other == 0, fused == 0)
    assert K.gemm_last_error() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_metrics_kernel_matches_the_host_computation(dtype):
    """Accuracy and the five losses accumulated on the device over two batches equal the torch computation on the host."""
    from flexflow_train_b200.utils.metrics import METRICS, PerfMetrics

    torch.manual_seed(8)
    dev_m, host_m = PerfMetrics(), PerfMetrics()
    for n, c in ((300, 10), (77, 1000)):
        p = torch.softmax(torch.randn(n, c), -1).to(dtype)
        sparse = torch.randint(0, c, (n,), dtype=torch.int32)
        dense = torch.softmax(torch.randn(n, c), -1).to(dtype)
        for lab in (sparse, dense):
            dev_m.update(p.cuda(), lab.cuda(), METRICS)
            host_m.update(p, lab if lab.dtype == torch.int32 else lab.float(), METRICS)
    a, b = dev_m.summary(), host_m.summary()
    assert a["samples"] == b["samples"] == 2 * (300 + 77)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    for key in ("accuracy", "cce", "sparse_cce", "mse", "rmse", "mae"):
        assert abs(a[key] - b[key]) <= tol * abs(b[key]) + 1e-7, (key, a[key], b[key])
    dev_m.reset()
    assert dev_m.summary()["samples"] == 0
