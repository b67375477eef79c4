"""The fused tcgen05 attention kernels against an fp32 PyTorch computation of the same attention (autograd for the
gradients), with the dropout mask restated on the host from the kernels' counter-based generator."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from flexflow_train_b200.ops import kernels as K  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.fixture(params=[1, 2, 3], ids=["one_tile", "two_tiles_smem_p", "two_tiles_tmem_p"])
def fwd_variant(request):
    """Every forward test runs on the three forward kernels (one query tile per CTA; two tiles per CTA with the
    probabilities handed to the second product through shared or through tensor memory)."""
    K.attention_set_forward_variant(request.param)
    yield request.param
    K.attention_set_forward_variant(1)


def _reference(q, k, v, B, H, S_q, S_k, D, scale, causal, keep, p):
    """q/k/v: [B*S, H*D] fp32 leaves.  Returns the [B*Sq, H*D] context."""
    qh = q.view(B, S_q, H, D).permute(0, 2, 1, 3)
    kh = k.view(B, S_k, H, D).permute(0, 2, 1, 3)
    vh = v.view(B, S_k, H, D).permute(0, 2, 1, 3)
    s = torch.matmul(qh, kh.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(torch.ones(S_q, S_k, dtype=torch.bool, device=s.device).triu(1), float("-inf"))
    pr = torch.softmax(s, -1)
    if keep is not None:
        pr = pr * keep.to(pr.dtype) / (1.0 - p)
    return torch.matmul(pr, vh).permute(0, 2, 1, 3).reshape(B * S_q, H * D)


def _packed_qkv(B, S, H, D, seed):
    torch.manual_seed(seed)
    qkv = (torch.randn(B * S, 3 * H * D, device="cuda") * 0.8).to(torch.bfloat16)
    return qkv, qkv[:, :H * D], qkv[:, H * D:2 * H * D], qkv[:, 2 * H * D:]


@pytest.mark.parametrize("S", [128, 1000, 1024])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal,p", [(False, 0.0), (True, 0.0), (False, 0.1)])
def test_attention_forward_matches_fp32_reference(S, D, causal, p, fwd_variant):
    B, H = 2, 3
    qkv, q, k, v = _packed_qkv(B, S, H, D, seed=S + D)
    out = torch.zeros(B * S, H * D, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(B, H, S, device="cuda")
    scale = 1.0 / math.sqrt(D)
    seed_t = torch.tensor([991], dtype=torch.int64, device="cuda")
    K.attention_fwd(q, k, v, out, lse, B=B, H=H, Sq=S, Sk=S, D=D, scale=scale, causal=causal, dropout=(p, 4242, seed_t) if p else None)
    assert K.attention_last_error() == 0
    keep = K.attention_keep_mask(B, H, S, S, p, 4242, seed=991, device="cuda") if p else None
    ref = _reference(q.float(), k.float(), v.float(), B, H, S, S, D, scale, causal, keep, p)
    assert rel(out, ref) < 1e-2
    # log-sum-exp (base 2) of the scaled scores
    s = torch.matmul(q.float().view(B, S, H, D).permute(0, 2, 1, 3), k.float().view(B, S, H, D).permute(0, 2, 3, 1)) * scale
    if causal:
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device="cuda").triu(1), float("-inf"))
    assert (lse - torch.logsumexp(s, -1) * math.log2(math.e)).abs().max() < 2e-2


def test_attention_forward_cross_lengths(fwd_variant):
    """Different query and key lengths (neither a multiple of the tile sizes), separate q / k / v matrices."""
    B, H, D, Sq, Sk = 2, 2, 128, 200, 333
    torch.manual_seed(5)
    q = torch.randn(B * Sq, H * D, device="cuda").to(torch.bfloat16)
    k = torch.randn(B * Sk, H * D, device="cuda").to(torch.bfloat16)
    v = torch.randn(B * Sk, H * D, device="cuda").to(torch.bfloat16)
    out = torch.zeros(B * Sq, H * D, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(B, H, Sq, device="cuda")
    scale = 1.0 / math.sqrt(D)
    K.attention_fwd(q, k, v, out, lse, B=B, H=H, Sq=Sq, Sk=Sk, D=D, scale=scale)
    assert K.attention_last_error() == 0
    ref = _reference(q.float(), k.float(), v.float(), B, H, Sq, Sk, D, scale, False, None, 0.0)
    assert rel(out, ref) < 1e-2


@pytest.mark.parametrize("S", [128, 1000, 1024])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal,p", [(False, 0.0), (True, 0.0), (False, 0.1), (True, 0.2)])
def test_attention_backward_matches_fp32_autograd(S, D, causal, p):
    B, H = 2, 2
    qkv, q, k, v = _packed_qkv(B, S, H, D, seed=S + 7)
    out = torch.zeros(B * S, H * D, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(B, H, S, device="cuda")
    scale = 1.0 / math.sqrt(D)
    seed_t = torch.tensor([17], dtype=torch.int64, device="cuda")
    drop = (p, 99, seed_t) if p else None
    K.attention_fwd(q, k, v, out, lse, B=B, H=H, Sq=S, Sk=S, D=D, scale=scale, causal=causal, dropout=drop)
    dout = (torch.randn(B * S, H * D, device="cuda") * 0.5).to(torch.bfloat16)
    dqkv = torch.zeros_like(qkv)
    dq, dk, dv = dqkv[:, :H * D], dqkv[:, H * D:2 * H * D], dqkv[:, 2 * H * D:]
    delta = torch.empty(B * H * S, device="cuda")
    acc = torch.empty(K.attention_bwd_scratch_floats(B, H, S, D), device="cuda")
    K.attention_bwd(q, k, v, out, lse, dout, dq, dk, dv, delta, acc, B=B, H=H, Sq=S, Sk=S, D=D, scale=scale, causal=causal, dropout=drop)
    assert K.attention_last_error() == 0
    keep = K.attention_keep_mask(B, H, S, S, p, 99, seed=17, device="cuda") if p else None
    qf, kf, vf = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    ref = _reference(qf, kf, vf, B, H, S, S, D, scale, causal, keep, p)
    ref.backward(dout.float())
    assert rel(dv, vf.grad) < 1.5e-2
    assert rel(dk, kf.grad) < 1.5e-2
    assert rel(dq, qf.grad) < 1.5e-2


@pytest.mark.parametrize("D", [64, 128])
def test_attention_backward_cross_lengths(D):
    """Query and key lengths that differ and are not multiples of the block sizes; separate q / k / v / gradient matrices."""
    B, H, Sq, Sk = 2, 3, 200, 333
    torch.manual_seed(11)
    q, k, v = (torch.randn(B * n, H * D, device="cuda").mul(0.7).to(torch.bfloat16) for n in (Sq, Sk, Sk))
    out = torch.zeros(B * Sq, H * D, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(B, H, Sq, device="cuda")
    scale = 1.0 / math.sqrt(D)
    K.attention_fwd(q, k, v, out, lse, B=B, H=H, Sq=Sq, Sk=Sk, D=D, scale=scale)
    dout = (torch.randn(B * Sq, H * D, device="cuda") * 0.5).to(torch.bfloat16)
    dq, dk, dv = torch.full_like(q, 3.0), torch.full_like(k, 3.0), torch.full_like(v, 3.0)
    delta = torch.empty(B * H * Sq, device="cuda")
    acc = torch.empty(K.attention_bwd_scratch_floats(B, H, Sq, D), device="cuda")
    K.attention_bwd(q, k, v, out, lse, dout, dq, dk, dv, delta, acc, B=B, H=H, Sq=Sq, Sk=Sk, D=D, scale=scale)
    assert K.attention_last_error() == 0
    qf, kf, vf = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    ref = _reference(qf, kf, vf, B, H, Sq, Sk, D, scale, False, None, 0.0)
    ref.backward(dout.float())
    assert rel(dv, vf.grad) < 1.5e-2 and rel(dk, kf.grad) < 1.5e-2 and rel(dq, qf.grad) < 1.5e-2


def test_attention_mask_changes_with_the_step_seed():
    B, H, D, S = 1, 2, 128, 256
    qkv, q, k, v = _packed_qkv(B, S, H, D, seed=3)
    lse = torch.empty(B, H, S, device="cuda")
    outs = []
    for seed in (1, 2, 1):
        out = torch.zeros(B * S, H * D, device="cuda", dtype=torch.bfloat16)
        K.attention_fwd(q, k, v, out, lse, B=B, H=H, Sq=S, Sk=S, D=D, scale=0.1, dropout=(0.3, 5, torch.tensor([seed], dtype=torch.int64, device="cuda")))
        outs.append(out)
    assert torch.equal(outs[0], outs[2]) and not torch.equal(outs[0], outs[1])
