"""Micro-benchmarks of single kernels with roofline fractions.

    python -m flexflow_train_b200.ops.bench_kernels --op gemm --m 8192 --n 8192 --k 8192
    python -m flexflow_train_b200.ops.bench_kernels --op layernorm --rows 32768 --cols 2048

Each run does warm-up launches, then times `--iters` launches with CUDA events on the launching stream; inputs are
sized past L2 or L2 is flushed between launches (``--flush``).  Prints one JSON line per op with achieved
throughput against the measured peaks.  Small `--iters` with `--warmup 1` gives a short launch list for a profiler.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..utils.profiling import roofline
from . import kernels as K


def _time(fn, warmup, iters, flush):
    buf = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if buf is not None:
            buf.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def bench_gemm_batched(a):
    """nb problems out[b] = x[b] @ w[b]^T, the shape of the attention score GEMM (short K, output-bound)."""
    nb, m, n, k = a.batched, a.m, a.n, a.k
    x = torch.randn(nb, m, k, device="cuda").to(torch.bfloat16)
    w = torch.randn(nb, n, k, device="cuda").to(torch.bfloat16)
    out = torch.empty(nb, m, n, device="cuda", dtype=torch.bfloat16)

    def run():
        K.gemm_raw(M=m, N=n, K=k, A=x.data_ptr(), lda=k, a_sb=m * k, B=w.data_ptr(), ldb=k, b_sb=n * k, C=out.data_ptr(), ldc=n, c_sb=m * n, nb=nb)
    ms = _time(run, a.warmup, a.iters, a.flush)
    r = roofline(ms, flops=2.0 * nb * m * n * k, hbm_bytes=2.0 * nb * (m * k + n * k + m * n))
    ref = _time(lambda: torch.bmm(x, w.transpose(1, 2), out=out), a.warmup, a.iters, a.flush) if a.compare else None
    return {"op": "gemm_nt_bf16_batched", "batch": nb, "m": m, "n": n, "k": k, **r, "torch_bmm_ms": ref, "gemm_error": K.gemm_last_error()}


def bench_gemm_layouts(a):
    """The three GEMMs of a Linear layer with `m` tokens, `k` inputs, `n` outputs: forward (NT), data gradient
    (NN: dY[m,n] . W[n,k]) and weight gradient (TN: dY[m,n]^T . X[m,k])."""
    m, n, k = a.m, a.n, a.k
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = torch.randn(n, k, device="cuda").to(torch.bfloat16)
    dy = torch.randn(m, n, device="cuda").to(torch.bfloat16)
    y, dx, dw = torch.empty(m, n, device="cuda", dtype=torch.bfloat16), torch.empty_like(x), torch.empty_like(w)
    out = {"op": "linear_gemms_bf16", "tokens": m, "in": k, "out": n}
    flops = 2.0 * m * n * k
    for name, fn, ref in (("fwd_nt", lambda: K.matmul_nt(x, w, out=y), lambda: torch.matmul(x, w.t(), out=y)),
                          ("dgrad_nn", lambda: K.matmul_nn(dy, w, out=dx), lambda: torch.matmul(dy, w, out=dx)),
                          ("wgrad_tn", lambda: K.matmul_tn(dy, x, out=dw), lambda: torch.matmul(dy.t(), x, out=dw))):
        ms = _time(fn, a.warmup, a.iters, a.flush)
        out[name] = {"ms": ms, "tflops": flops / ms / 1e9, "torch_ms": _time(ref, a.warmup, a.iters, a.flush) if a.compare else None}
    out["gemm_error"] = K.gemm_last_error()
    return out


def bench_gemm(a):
    if a.batched:
        return bench_gemm_batched(a)
    if a.layouts:
        return bench_gemm_layouts(a)
    m, n, k = a.m, a.n, a.k
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = torch.randn(n, k, device="cuda").to(torch.bfloat16)
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(n, device="cuda").to(torch.bfloat16) if a.bias else None
    ms = _time(lambda: K.matmul_nt(x, w, out=out, bias=bias, act="relu" if a.relu else None), a.warmup, a.iters, a.flush)
    r = roofline(ms, flops=2.0 * m * n * k, hbm_bytes=2.0 * (m * k + n * k + m * n))
    ref = None
    if a.compare:
        ref = _time(lambda: torch.matmul(x, w.t(), out=out), a.warmup, a.iters, a.flush)
    return {"op": "gemm_nt_bf16", "m": m, "n": n, "k": k, "bias": a.bias, "relu": a.relu, **r, "torch_matmul_ms": ref,
            "gemm_error": K.gemm_last_error()}


def bench_layernorm(a):
    rows, cols = a.rows, a.cols
    x = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    g = torch.ones(cols, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(cols, device="cuda", dtype=torch.bfloat16)
    y = torch.empty_like(x)
    mean = torch.empty(rows, device="cuda")
    rstd = torch.empty(rows, device="cuda")
    ms = _time(lambda: K.layernorm_fwd(x, g, b, 1e-5, out=y, mean=mean, rstd=rstd), a.warmup, a.iters, a.flush)
    return {"op": "layernorm_fwd_bf16", "rows": rows, "cols": cols, **roofline(ms, hbm_bytes=4.0 * rows * cols)}


def bench_layernorm_bwd(a):
    rows, cols = a.rows, a.cols
    x = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    dy = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    g = torch.ones(cols, device="cuda", dtype=torch.bfloat16)
    mean = x.float().mean(1)
    rstd = torch.rsqrt(x.float().var(1, unbiased=False) + 1e-5)
    dx = torch.empty_like(x)
    dg, db = torch.empty_like(g), torch.empty_like(g)
    scratch = torch.empty(K.layernorm_bwd_scratch(rows, cols), device="cuda")
    ms = _time(lambda: K.layernorm_bwd(dy, x, g, mean, rstd, dx, dg, db, scratch), a.warmup, a.iters, a.flush)
    # reads dy and x, writes dx
    return {"op": "layernorm_bwd_bf16", "rows": rows, "cols": cols, **roofline(ms, hbm_bytes=6.0 * rows * cols)}


def bench_softmax(a):
    rows, cols = a.rows, a.cols
    x = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    y = torch.empty_like(x)
    ms = _time(lambda: K.softmax_fwd(x, out=y), a.warmup, a.iters, a.flush)
    return {"op": "softmax_fwd_bf16", "rows": rows, "cols": cols, **roofline(ms, hbm_bytes=4.0 * rows * cols)}


def bench_batchnorm(a):
    rows, cols = a.rows, a.cols
    x = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    g = torch.ones(cols, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(cols, device="cuda", dtype=torch.bfloat16)
    y = torch.empty_like(x)
    mean = torch.empty(cols, device="cuda")
    rstd = torch.empty(cols, device="cuda")
    scratch = torch.empty(K.batchnorm_scratch(rows, cols), device="cuda")
    ms = _time(lambda: K.batchnorm_fwd(x, y, g, b, mean, rstd, scratch, rows, cols, 1e-5, relu=True), a.warmup, a.iters, a.flush)
    # two reads of x (statistics, then normalise) and one write
    return {"op": "batchnorm_fwd_bf16", "rows": rows, "cols": cols, **roofline(ms, hbm_bytes=6.0 * rows * cols)}


def bench_im2col(a):
    n, c, h, w = a.batch, a.channels, a.size, a.size
    x = torch.randn(n, h, w, c, device="cuda").to(torch.bfloat16)
    g = K.ConvGeometry(n, c, h, w, 3, 3, 1, 1, 1, 1, K.nhwc_strides(n, c, h, w))
    col = torch.empty(g.rows, g.kp, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: K.im2col(x, col, g), a.warmup, a.iters, a.flush)
    return {"op": "im2col_3x3_bf16", "n": n, "c": c, "hw": h, **roofline(ms, hbm_bytes=2.0 * (x.numel() + col.numel()))}


def bench_conv(a):
    """Implicit-GEMM convolution (forward, data gradient, weight gradient) on channels-last bf16 data: --batch, --channels
    (input), --n (output channels), --size (height = width), --k (square filter, stride 1, "same" padding).  --compare also
    times torch's convolution (cuDNN, channels-last) forward and its two gradients."""
    n, c, h, w, oc, kk = a.batch, a.channels, a.size, a.size, a.n, a.k
    pad = kk // 2
    x = torch.randn(n, h, w, c, device="cuda").to(torch.bfloat16)
    wt = (torch.randn(oc, c, kk, kk, device="cuda") / (c * kk * kk) ** 0.5).to(torch.bfloat16)
    g = K.ConvGeometry(n, c, h, w, kk, kk, 1, 1, pad, pad, K.nhwc_strides(n, c, h, w))
    wp = torch.empty(oc, g.kp, device="cuda", dtype=torch.bfloat16)
    K.filter_pack(wt, wp, oc, c, kk, kk, g.kp)
    y = torch.empty(n, g.oh, g.ow, oc, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn_like(y)
    dx = torch.empty_like(x)
    dwp = torch.empty(oc, g.kp, device="cuda", dtype=torch.float32)
    flops = 2.0 * n * g.oh * g.ow * oc * c * kk * kk
    act_bytes = 2.0 * (x.numel() + y.numel())
    res = {"op": "conv2d_implicit_bf16", "n": n, "c": c, "hw": h, "oc": oc, "k": kk}
    res["fprop"] = roofline(_time(lambda: K.conv_fprop(x, wp, y, g, oc), a.warmup, a.iters, a.flush), flops=flops, hbm_bytes=act_bytes)
    res["dgrad"] = roofline(_time(lambda: K.conv_dgrad(dy, wp, dx, g, oc), a.warmup, a.iters, a.flush), flops=flops, hbm_bytes=act_bytes)
    res["wgrad"] = roofline(_time(lambda: K.conv_wgrad(x, dy, dwp, g, oc), a.warmup, a.iters, a.flush), flops=flops, hbm_bytes=act_bytes)
    if a.compare:
        import torch.nn.functional as F
        xt = x.permute(0, 3, 1, 2).requires_grad_(True)          # NCHW view of channels-last storage
        wl = wt.contiguous(memory_format=torch.channels_last).requires_grad_(True)
        fwd = lambda: F.conv2d(xt, wl, None, padding=pad)         # noqa: E731
        res["torch_fprop_ms"] = _time(fwd, a.warmup, a.iters, a.flush)
        yt = fwd()
        dyt = dy.permute(0, 3, 1, 2)
        res["torch_dgrad_ms"] = _time(lambda: torch.autograd.grad(yt, xt, dyt, retain_graph=True), a.warmup, a.iters, a.flush)
        res["torch_wgrad_ms"] = _time(lambda: torch.autograd.grad(yt, wl, dyt, retain_graph=True), a.warmup, a.iters, a.flush)
    res["conv_error"] = K.conv_last_error()
    return res


def bench_attention(a):
    """Fused attention forward and backward on a packed QKV buffer: --batch, --heads, --seq, --head-dim, --dropout, --causal.
    FLOPs counted: 4 B H Sq Sk D forward, 10 B H Sq Sk D backward (halved when causal).  --compare also times the
    library attention (torch scaled_dot_product_attention, forward and its autograd backward) on the same data."""
    import math
    B, H, S, D = a.batch, a.heads, a.seq, a.head_dim
    qkv = (torch.randn(B * S, 3 * H * D, device="cuda") * 0.5).to(torch.bfloat16)
    q, k, v = qkv[:, :H * D], qkv[:, H * D:2 * H * D], qkv[:, 2 * H * D:]
    out = torch.empty(B * S, H * D, device="cuda", dtype=torch.bfloat16)
    dout = torch.randn_like(out)
    dqkv = torch.empty_like(qkv)
    dq, dk, dv = dqkv[:, :H * D], dqkv[:, H * D:2 * H * D], dqkv[:, 2 * H * D:]
    lse = torch.empty(B, H, S, device="cuda")
    delta = torch.empty(B * H * S, device="cuda")
    seed = torch.tensor([1], dtype=torch.int64, device="cuda")
    drop = (a.dropout, 7, seed) if a.dropout > 0 else None
    scale = 1.0 / math.sqrt(D)
    kw = dict(B=B, H=H, Sq=S, Sk=S, D=D, scale=scale, causal=a.causal, dropout=drop)
    f = (0.5 if a.causal else 1.0) * B * H * S * S * D
    res = {"op": "attention_bf16", "batch": B, "heads": H, "seq": S, "head_dim": D, "dropout": a.dropout, "causal": a.causal}
    ms = _time(lambda: K.attention_fwd(q, k, v, out, lse, **kw), a.warmup, a.iters, a.flush)
    res["fwd"] = roofline(ms, flops=4.0 * f, hbm_bytes=2.0 * 4 * B * S * H * D)
    if K.attention_supported(D, backward=True):
        acc = torch.empty(K.attention_bwd_scratch_floats(B, H, S, D), device="cuda")
        ms = _time(lambda: K.attention_bwd(q, k, v, out, lse, dout, dq, dk, dv, delta, acc, **kw), a.warmup, a.iters, a.flush)
        res["bwd"] = roofline(ms, flops=10.0 * f, hbm_bytes=2.0 * 8 * B * S * H * D)
    if a.compare:
        import torch.nn.functional as F
        q4, k4, v4 = (t.reshape(B, S, H, D).transpose(1, 2).contiguous().requires_grad_(True) for t in (q, k, v))
        do4 = dout.reshape(B, S, H, D).transpose(1, 2).contiguous()
        fwd = lambda: F.scaled_dot_product_attention(q4, k4, v4, dropout_p=a.dropout, is_causal=a.causal)  # noqa: E731
        res["torch_sdpa_fwd_ms"] = _time(fwd, a.warmup, a.iters, a.flush)
        o4 = fwd()
        res["torch_sdpa_bwd_ms"] = _time(lambda: torch.autograd.grad(o4, (q4, k4, v4), do4, retain_graph=True), a.warmup, a.iters, a.flush)
    res["attention_error"] = K.attention_last_error()
    return res


OPS = {"attention": bench_attention, "gemm": bench_gemm, "layernorm": bench_layernorm, "layernorm_bwd": bench_layernorm_bwd, "softmax": bench_softmax, "batchnorm": bench_batchnorm,
       "im2col": bench_im2col, "conv": bench_conv}


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--op", choices=sorted(OPS), required=True)
    p.add_argument("--m", type=int, default=8192)
    p.add_argument("--n", type=int, default=8192)
    p.add_argument("--k", type=int, default=8192)
    p.add_argument("--rows", type=int, default=32768)
    p.add_argument("--cols", type=int, default=2048)
    p.add_argument("--batch", type=int, default=32)
    p.add_argument("--channels", type=int, default=192)
    p.add_argument("--size", type=int, default=35)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--seq", type=int, default=1024)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--dropout", type=float, default=0.0)
    p.add_argument("--causal", action="store_true")
    p.add_argument("--bias", action="store_true")
    p.add_argument("--relu", action="store_true")
    p.add_argument("--compare", action="store_true", help="also time torch.matmul (cuBLAS) on the same operands")
    p.add_argument("--flush", action="store_true", help="write a buffer larger than L2 between timed launches")
    p.add_argument("--no-tma-store", action="store_true", help="GEMM epilogue through per-lane global stores instead of TMA stores")
    p.add_argument("--tma-store", action="store_true", help="GEMM epilogue through TMA stores")
    p.add_argument("--layouts", action="store_true", help="gemm: time the forward / data-gradient / weight-gradient GEMMs of a Linear")
    p.add_argument("--batched", type=int, default=0, help="gemm: run as a batch of this many [m, n, k] problems (attention-shaped)")
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--iters", type=int, default=10)
    a = p.parse_args(argv)
    if a.no_tma_store:
        K.lib().ffk_gemm_set_tma_store(0)
    if a.tma_store:
        K.lib().ffk_gemm_set_tma_store(1)
    print(json.dumps(OPS[a.op](a)))


if __name__ == "__main__":
    main()
