"""Convolution-stack kernels and operators against PyTorch fp32 references."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from flexflow_train_b200 import _ffcore as core  # noqa: E402
from flexflow_train_b200.ops import kernels as K  # noqa: E402
from flexflow_train_b200.runtime.executor import ExecConfig, Executable  # noqa: E402
from flexflow_train_b200.runtime.torch_oracle import TorchOracle  # noqa: E402


def rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).norm() / (b.float().cpu().norm() + 1e-12)).item()


@pytest.mark.parametrize("c,k,s,p,nhwc", [(16, 3, 1, 1, True), (8, 3, 2, 0, True), (3, 3, 2, 0, False), (24, 5, 1, 2, True),
                                          (16, 1, 2, 0, True)])
def test_im2col_col2im_match_unfold(c, k, s, p, nhwc):
    n, h, w = 3, 13, 11
    torch.manual_seed(0)
    x = torch.randn(n, c, h, w, device="cuda").to(torch.bfloat16)
    xin = x.permute(0, 2, 3, 1).contiguous() if nhwc else x
    strides = K.nhwc_strides(n, c, h, w) if nhwc else K.nchw_strides(n, c, h, w)
    g = K.ConvGeometry(n, c, h, w, k, k, s, s, p, p, strides)
    col = torch.full((g.rows, g.kp), 7.0, device="cuda", dtype=torch.bfloat16)
    K.im2col(xin, col, g)
    ref = F.unfold(x.float(), k, padding=p, stride=s)  # [n, c*k*k, L] with (c, kh, kw) order
    ref = ref.view(n, c, k * k, -1).permute(0, 3, 2, 1).reshape(g.rows, k * k * c)
    assert torch.equal(col[:, :g.k].float(), ref)
    assert float(col[:, g.k:].abs().sum()) == 0
    # col2im is the adjoint of im2col
    dcol = torch.randn(g.rows, g.kp, device="cuda").to(torch.bfloat16)
    dx = torch.empty_like(xin)
    K.col2im(dcol, dx, g)
    d = dcol[:, :g.k].float().view(n, -1, k * k, c).permute(0, 3, 2, 1).reshape(n, c * k * k, -1)
    ref_dx = F.fold(d, (h, w), k, padding=p, stride=s)
    got = dx.float().permute(0, 3, 1, 2) if nhwc else dx.float()
    assert rel(got, ref_dx) < 1e-2
    base = torch.randn_like(dx)
    acc = base.clone()
    K.col2im(dcol, acc, g, accumulate=True)
    got = acc.float().permute(0, 3, 1, 2) if nhwc else acc.float()
    b = base.float().permute(0, 3, 1, 2) if nhwc else base.float()
    assert rel(got, ref_dx + b) < 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode,k,s,p", [("max", 3, 2, 0), ("max", 3, 1, 1), ("avg", 3, 1, 1), ("avg", 8, 1, 0)])
def test_pool2d_matches_torch(dtype, mode, k, s, p):
    n, c, h, w = 2, 12, 17, 17
    torch.manual_seed(1)
    x = torch.randn(n, c, h, w, device="cuda").to(dtype)
    xcl = x.permute(0, 2, 3, 1).contiguous()
    g = K.ConvGeometry(n, c, h, w, k, k, s, s, p, p, K.nhwc_strides(n, c, h, w), kp=0)
    y = torch.empty(n, g.oh, g.ow, c, device="cuda", dtype=dtype)
    arg = torch.empty(y.numel(), device="cuda", dtype=torch.uint8) if mode == "max" else None
    K.pool2d_fwd(xcl, y, arg, g, mode)
    xr = x.float().requires_grad_(True)
    yr = F.max_pool2d(xr, k, s, p) if mode == "max" else F.avg_pool2d(xr, k, s, p, count_include_pad=False)
    assert rel(y.permute(0, 3, 1, 2), yr) < (1e-6 if dtype == torch.float32 else 5e-3)
    dy = torch.randn_like(y)
    dx = torch.empty_like(xcl)
    K.pool2d_bwd(dy.view(-1), arg, dx, g, mode)
    yr.backward(dy.float().permute(0, 3, 1, 2))
    assert rel(dx.permute(0, 3, 1, 2), xr.grad) < (1e-5 if dtype == torch.float32 else 1e-2)
    # strided (NCHW) input and gradient
    g2 = K.ConvGeometry(n, c, h, w, k, k, s, s, p, p, K.nchw_strides(n, c, h, w), kp=0)
    y2 = torch.empty_like(y)
    K.pool2d_fwd(x, y2, arg, g2, mode)
    assert torch.equal(y2, y)
    dx2 = torch.empty_like(x)
    K.pool2d_bwd(dy.view(-1), arg, dx2, g2, mode)
    assert rel(dx2, xr.grad) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("relu", [False, True])
@pytest.mark.parametrize("rows,cols", [(4 * 35 * 35, 64), (777, 48), (130, 7)])
def test_batchnorm_matches_torch(dtype, tol, relu, rows, cols):
    torch.manual_seed(2)
    x = (torch.randn(rows, cols, device="cuda") * 2 + 0.5).to(dtype)
    gamma = (torch.rand(cols, device="cuda") + 0.5).to(dtype)
    beta = torch.randn(cols, device="cuda").to(dtype)
    y = torch.empty_like(x)
    mean = torch.empty(cols, device="cuda")
    rstd = torch.empty(cols, device="cuda")
    scratch = torch.empty(K.batchnorm_scratch(rows, cols), device="cuda")
    K.batchnorm_fwd(x, y, gamma, beta, mean, rstd, scratch, rows, cols, 1e-5, relu=relu)
    xr = x.float().requires_grad_(True)
    gr = gamma.float().requires_grad_(True)
    br = beta.float().requires_grad_(True)
    yr = F.batch_norm(xr, None, None, gr, br, True, 0.1, 1e-5)
    if relu:
        yr = torch.relu(yr)
    assert rel(y, yr) < tol
    assert rel(mean, xr.detach().mean(0)) < 1e-4
    dy = torch.randn_like(y)
    # the reference sees the same ReLU mask as the kernel (taken from the kernel's own output)
    if relu:
        yr2 = F.batch_norm(xr, None, None, gr, br, True, 0.1, 1e-5) * (y.float() > 0)
    else:
        yr2 = yr
    yr2.backward(dy.float())
    dx = torch.empty_like(x)
    dgamma = torch.empty_like(gamma)
    dbeta = torch.empty_like(beta)
    K.batchnorm_bwd(dy, x, y if relu else None, gamma, mean, rstd, dx, dgamma, dbeta, scratch, rows, cols)
    assert rel(dx, xr.grad) < 3 * tol
    assert rel(dgamma, gr.grad) < 3 * tol and rel(dbeta, br.grad) < 3 * tol


def _conv_net():
    b = core.GraphBuilder()
    x = b.create_input([4, 3, 19, 19], name="input")
    t = b.conv2d(x, 16, 3, 3, 2, 2, 0, 0, activation="RELU", name="conv1")   # NCHW input, K = 27 padded to 32
    t = b.batch_norm(t, activation="RELU", name="bn1")
    l = b.conv2d(t, 24, 1, 1, name="branch1x1")                               # pointwise: the activation is the operand
    r = b.conv2d(t, 8, 3, 3, 1, 1, 1, 1, activation="RELU", name="branch3x3")
    p = b.pool2d(t, 3, 3, 1, 1, 1, 1, pool_type="AVG", name="branch_pool")
    t = b.concat([l, r, p], 1, name="mix")
    t = b.pool2d(t, 3, 3, 2, 2, 0, 0, pool_type="MAX", name="pool")
    t = b.conv2d(t, 32, 1, 1, 2, 2, name="strided1x1")
    t = b.flat(t, name="flat")
    t = b.dense(t, 10, name="fc")
    b.softmax(t, name="out_prob")
    return b.graph


def test_conv_stack_matches_oracle():
    g = _conv_net()
    ex = Executable(g, ExecConfig(compute_dtype="bf16", seed=3))
    oracle = TorchOracle(g, seed=3)
    torch.manual_seed(0)
    x = torch.randn(4, 3, 19, 19)
    labels = torch.randint(0, 10, (4,), dtype=torch.int32)
    ex.set_inputs({"input": x.cuda()}, labels.cuda())
    ex.forward()
    ex.compute_loss()
    ex.backward()
    rows_ref, grads_ref = oracle.loss_and_grads({"input": x}, labels)
    assert rel(ex.loss_rows, rows_ref) < 5e-2
    for name, g_ in ex.named_gradients():
        # bf16 activations through batch norm: gradients of zero-mean inputs cancel heavily, so their
        # relative error is many times the per-element rounding error
        assert rel(g_, grads_ref[name]) < 0.4, (name, rel(g_, grads_ref[name]))
    assert K.gemm_last_error() == 0


@pytest.mark.parametrize("k,s,p,cin,cout", [(3, 1, 1, 16, 24), (1, 1, 0, 16, 32), (5, 2, 2, 8, 16), (3, 2, 0, 3, 8), (1, 2, 0, 16, 8)])
def test_single_convolution_matches_oracle(k, s, p, cin, cout):
    """One convolution between two layers without normalisation: output and all gradients to bf16 accuracy, for
    the packed (KxK), pointwise (activation used in place) and strided paths, including the split-K weight
    gradient (few output tiles, thousands of rows)."""
    b = core.GraphBuilder()
    x = b.create_input([8, cin, 20, 20], name="input")
    t = b.conv2d(x, cin, 1, 1, name="pre") if cin % 8 == 0 else x      # makes the tested conv's input channels-last
    t = b.conv2d(t, cout, k, k, s, s, p, p, activation="RELU", name="conv")
    t = b.pool2d(t, 2, 2, 2, 2, 0, 0, pool_type="AVG", name="pool")
    t = b.dense(b.flat(t, name="flat"), 10, name="fc")
    b.softmax(t, name="out_prob")
    g = b.graph
    ex = Executable(g, ExecConfig(compute_dtype="bf16", seed=5))
    oracle = TorchOracle(g, seed=5)
    torch.manual_seed(1)
    xin = torch.randn(8, cin, 20, 20) + 0.5
    labels = torch.randint(0, 10, (8,), dtype=torch.int32)
    ex.set_inputs({"input": xin.cuda()}, labels.cuda())
    ex.forward()
    ex.compute_loss()
    ex.backward()
    rows_ref, grads_ref = oracle.loss_and_grads({"input": xin}, labels)
    assert rel(ex.loss_rows, rows_ref) < 3e-2
    for name, g_ in ex.named_gradients():
        # a bias gradient is a sum of thousands of bf16-rounded activation gradients of both signs: its relative
        # error is several times that of the weight gradients
        tol = 0.25 if name.endswith(".bias") else 8e-2
        assert rel(g_, grads_ref[name]) < tol, (name, rel(g_, grads_ref[name]))
    assert K.gemm_last_error() == 0


@pytest.mark.parametrize("groups,cin,cout,k", [(2, 16, 24, 3), (4, 16, 16, 1), (16, 16, 16, 3)])
def test_grouped_convolution_matches_oracle(groups, cin, cout, k):
    """Grouped (down to depthwise) convolution: per group one im2col + GEMM on channel slices of the same buffers."""
    b = core.GraphBuilder()
    x = b.create_input([4, cin, 12, 12], name="input")
    t = b.conv2d(x, cin, 1, 1, name="pre")
    t = b.conv2d(t, cout, k, k, 1, 1, k // 2, k // 2, activation="RELU", groups=groups, name="gconv")
    t = b.pool2d(t, 2, 2, 2, 2, 0, 0, pool_type="AVG", name="pool")
    t = b.dense(b.flat(t, name="flat"), 10, name="fc")
    b.softmax(t, name="out_prob")
    g = b.graph
    ex = Executable(g, ExecConfig(compute_dtype="bf16", seed=5))
    oracle = TorchOracle(g, seed=5)
    torch.manual_seed(1)
    xin = torch.randn(4, cin, 12, 12) + 0.5
    labels = torch.randint(0, 10, (4,), dtype=torch.int32)
    ex.set_inputs({"input": xin.cuda()}, labels.cuda())
    ex.forward()
    ex.compute_loss()
    ex.backward()
    rows_ref, grads_ref = oracle.loss_and_grads({"input": xin}, labels)
    assert rel(ex.loss_rows, rows_ref) < 3e-2
    for name, g_ in ex.named_gradients():
        assert rel(g_, grads_ref[name]) < 8e-2, (name, rel(g_, grads_ref[name]))
    assert K.gemm_last_error() == 0


def test_split_k_weight_gradient_gemm_matches_fp32():
    torch.manual_seed(3)
    rows, oc, kp = 40000, 96, 288
    dy = torch.randn(rows, oc, device="cuda").to(torch.bfloat16)
    col = torch.randn(rows, kp, device="cuda").to(torch.bfloat16)
    out = torch.full((oc, kp), 7.0, device="cuda")
    K.matmul_tn(dy, col, out=out)                       # few tiles, long K: takes the split-K path
    ref = dy.float().t() @ col.float()
    assert rel(out, ref) < 2e-3
    K.matmul_tn(dy, col, out=out, accumulate=True)
    assert rel(out, 2 * ref) < 2e-3
    assert K.gemm_last_error() == 0


def test_inception_v3_trains_one_step():
    g = core.build_model("inception_v3", {"batch_size": 2, "num_classes": 100})
    ex = Executable(g, ExecConfig(compute_dtype="bf16", seed=1))
    torch.manual_seed(0)
    inp = [n for n in g.nodes() if n["type"] == "INPUT"][0]
    x = torch.randn([int(s) for s in inp["outputs"][0][1].sizes], device="cuda")
    labels = torch.randint(0, 100, (2,), dtype=torch.int32, device="cuda")
    losses = []
    for _ in range(3):
        ex.train_step({inp["name"] or f"input{inp['id']}": x}, labels)
        losses.append(ex.mean_loss())
    assert all(l == l and l < 1e4 for l in losses), losses
    assert K.gemm_last_error() == 0
