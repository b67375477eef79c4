"""Implicit-GEMM convolution (tcgen05, shifted TMA boxes, no im2col matrix): forward, data gradient and weight gradient
against torch.nn.functional.conv2d in fp32 on the same bf16-rounded operands."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from flexflow_train_b200.ops import kernels as K  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


CASES = [
    # n, c, h, w, oc, kh, kw, ph, pw
    (4, 64, 17, 17, 96, 3, 3, 1, 1),      # box = one image row band, 64-channel chunks
    (3, 48, 35, 35, 64, 5, 5, 2, 2),      # C not a multiple of 64: zero channels meet the next tap's filter columns
    (16, 128, 8, 8, 320, 3, 3, 1, 1),     # two images per tile, N tile 256 with a ragged edge
    (2, 192, 17, 17, 160, 1, 7, 0, 3),    # 1 x 7
    (2, 160, 17, 17, 192, 7, 1, 3, 0),    # 7 x 1
    (2, 32, 20, 23, 32, 3, 3, 0, 0),      # no padding: output smaller than input, short channel chunk
    (1, 8, 9, 150, 8, 3, 3, 1, 1),        # rows wider than a tile
    (5, 80, 12, 12, 200, 1, 1, 0, 0),     # pointwise
]


def _setup(case):
    n, c, h, w, oc, kh, kw, ph, pw = case
    torch.manual_seed(sum(case))
    x = torch.randn(n, c, h, w, device="cuda").to(torch.bfloat16)
    wt = (torch.randn(oc, c, kh, kw, device="cuda") / (c * kh * kw) ** 0.5).to(torch.bfloat16)
    g = K.ConvGeometry(n, c, h, w, kh, kw, 1, 1, ph, pw, K.nhwc_strides(n, c, h, w))
    assert K.conv_implicit_supported(g, oc)
    wp = torch.empty(oc, g.kp, device="cuda", dtype=torch.bfloat16)
    K.filter_pack(wt, wp, oc, c, kh, kw, g.kp)
    return x, wt, g, wp


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("act", [None, "relu"])
def test_forward_matches_conv2d(case, act):
    n, c, h, w, oc, kh, kw, ph, pw = case
    x, wt, g, wp = _setup(case)
    bias = torch.randn(oc, device="cuda").to(torch.bfloat16)
    xcl = x.permute(0, 2, 3, 1).contiguous()
    y = torch.full((n, g.oh, g.ow, oc), 9.0, device="cuda", dtype=torch.bfloat16)
    pre = torch.empty_like(y) if act else None
    K.conv_fprop(xcl, wp, y, g, oc, bias=bias, act=act, pre_act_out=pre)
    assert K.conv_last_error() == 0
    ref = F.conv2d(x.float(), wt.float(), bias.float(), padding=(ph, pw))
    if act:
        assert rel(pre.permute(0, 3, 1, 2), ref) < 1e-2
        ref = ref.relu()
    assert rel(y.permute(0, 3, 1, 2), ref) < 1e-2


@pytest.mark.parametrize("case", CASES)
def test_gradients_match_autograd(case):
    n, c, h, w, oc, kh, kw, ph, pw = case
    x, wt, g, wp = _setup(case)
    xr, wr = x.float().requires_grad_(True), wt.float().requires_grad_(True)
    yr = F.conv2d(xr, wr, None, padding=(ph, pw))
    dy = torch.randn_like(yr).to(torch.bfloat16)
    yr.backward(dy.float())
    dycl = dy.permute(0, 2, 3, 1).contiguous()
    xcl = x.permute(0, 2, 3, 1).contiguous()
    # data gradient, then accumulated onto an existing gradient
    dx = torch.full((n, h, w, c), 5.0, device="cuda", dtype=torch.bfloat16)
    K.conv_dgrad(dycl, wp, dx, g, oc)
    assert rel(dx.permute(0, 3, 1, 2), xr.grad) < 1e-2
    base = torch.randn_like(dx)
    acc = base.clone()
    K.conv_dgrad(dycl, wp, acc, g, oc, accumulate=True)
    assert rel(acc.permute(0, 3, 1, 2), xr.grad + base.float().permute(0, 3, 1, 2)) < 1e-2
    # weight gradient in the packed layout [OC, (r, s, c)]
    dwp = torch.full((oc, g.kp), 3.0, device="cuda", dtype=torch.float32)
    K.conv_wgrad(xcl, dycl, dwp, g, oc)
    ref_w = wr.grad.permute(0, 2, 3, 1).reshape(oc, kh * kw * c)
    assert rel(dwp, ref_w) < 1e-2
    K.conv_wgrad(xcl, dycl, dwp, g, oc, accumulate=True)
    assert rel(dwp, 2 * ref_w) < 1e-2
    assert K.conv_last_error() == 0
