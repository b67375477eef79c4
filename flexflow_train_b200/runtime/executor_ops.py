"""Operator implementations for convolution stacks (Conv2D, Pool2D, BatchNorm) and the tensor-shape operators
(Concat, Split, Transpose, Reverse, Gather, TopK, Reduce*, Broadcast).

Convolution stacks keep their 4-D activations channels-last in memory (the logical shape stays NCHW): a 1x1
convolution is then the GEMM [N*H*W, C] x [OC, C]^T on the activation as it lies, a KxK convolution needs one
im2col pass into a K-major bf16 matrix, and pooling / batch-norm / channel concatenation are coalesced over
channels.  The executable tracks which values are channels-last; operators here declare ``layout_aware``.

Reference operators: lib/kernels/src/cuda/ops/{conv_2d,pool_2d,batch_norm,concat,split,transpose,reverse,gather,
topk,reduce}_kernels.cu and the task wrappers in lib/task-spec/src/task-spec/ops/impl/.
"""
from __future__ import annotations

from typing import List

import torch

from ..ops import kernels as K
from .executor import _ACT, OpImpl, register


def _sizes(op: OpImpl, slot="INPUT") -> List[int]:
    return [int(v) for v in op.ex.graph.shape(op.inputs[slot]).piece_sizes]


def _scratch_view(ex, slot: int, shape, dtype):
    n = 1
    for s in shape:
        n *= s
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    return ex._big[slot][:nbytes].view(dtype).view(list(shape))


def _elt(dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


# ------------------------------------------------------------------------------------------ Conv2D
@register("CONV2D")
class Conv2dOp(OpImpl):
    layout_aware = True

    def setup(self):
        a = self.attrs
        self.groups = int(a.get("groups", 1) or 1)
        x = self.x()
        if x.dtype != torch.bfloat16:
            raise NotImplementedError("Conv2D runs on the bf16 tensor-core path; use compute_dtype='bf16'")
        if self.groups != 1:
            return self._setup_grouped()
        n, c, h, w = _sizes(self)
        oc, _, kh, kw = _sizes(self, "FILTER")
        self.in_nhwc = self.ex.is_nhwc(self.inputs["INPUT"])
        strides = K.nhwc_strides(n, c, h, w) if self.in_nhwc else K.nchw_strides(n, c, h, w)
        self.g = g = K.ConvGeometry(n, c, h, w, kh, kw, int(a["stride_h"]), int(a["stride_w"]), int(a["padding_h"]),
                                    int(a["padding_w"]), strides)
        self.oc = oc
        self.act = _ACT[a.get("activation")]
        y = torch.empty(n, g.oh, g.ow, oc, dtype=x.dtype, device=x.device)
        self.out().data = y
        self.ex.mark_nhwc((self.nid, "OUTPUT"))
        self.y2d = y.view(g.rows, oc)
        pointwise = kh == 1 and kw == 1 and c % 8 == 0
        # the activation itself is the GEMM operand of a 1x1 stride-1 convolution over channels-last data
        self.direct = pointwise and g.sh == 1 and g.sw == 1 and g.ph == 0 and g.pw == 0 and (self.in_nhwc or h * w == 1)
        self.packed = not pointwise  # a 1x1 filter [OC, C, 1, 1] already is the K-major matrix [OC, C]
        # stride-1 convolutions over channels-last data run as an implicit GEMM: the kernel loads shifted boxes of the
        # activation itself, so there is no im2col / col2im matrix to write, keep or read back
        self.implicit = (not self.direct and self.in_nhwc and self.ex.cfg.implicit_conv and K.conv_implicit_supported(g, oc))
        w_ = self.x("FILTER")
        self.wp = torch.empty(oc, g.kp, dtype=torch.bfloat16, device=x.device) if self.packed else w_.view(oc, g.kp)
        self.bias = self.x("BIAS") if "BIAS" in self.inputs else None
        self.pre = torch.empty_like(self.y2d) if (self.act == "gelu" and self.ex.cfg.training) else None
        if not self.direct and not self.implicit:
            self.ex.need_big_scratch(g.rows * g.kp * 2, 2)  # slot 0: col, slot 1: dcol
        # slot 2: filter gradient in GEMM layout, fp32 (the weight-gradient GEMM has few output tiles and a very long
        # reduction over N*OH*OW rows; with an fp32 output the kernel splits that reduction over the SMs)
        self.ex.need_big_scratch(oc * g.kp * 4, 3)
        self.ex.need_scratch(4 * K.bias_act_bwd_scratch(g.rows, oc))
        self._col = self._dcol = self._dwp = None
        self._kept = None
        col_bytes = g.rows * g.kp * 2
        claimed = getattr(self.ex, "_im2col_kept_bytes", 0)
        if not self.direct and not self.implicit and self.ex.cfg.training and self.buf("FILTER").requires_grad and \
                claimed + col_bytes <= self.ex.cfg.keep_im2col_bytes:
            free = torch.cuda.mem_get_info(x.device)[0] if x.is_cuda else 0
            if col_bytes * 4 < free:  # never take more than a quarter of what is left
                self._kept = torch.empty(g.rows, g.kp, dtype=torch.bfloat16, device=x.device)
                self.ex._im2col_kept_bytes = claimed + col_bytes

    # ---- grouped convolution: one im2col + GEMM per group on strided views of the same buffers.  Group j reads
    # input channels [j*cg, (j+1)*cg) (a channel offset into the activation, same strides), filter rows
    # [j*ocg, (j+1)*ocg) and writes output columns [j*ocg, (j+1)*ocg) of the [rows, oc] result (ldc = oc).
    def _setup_grouped(self):
        a, x, G = self.attrs, self.x(), self.groups
        n, c, h, w = _sizes(self)
        oc, cg, kh, kw = _sizes(self, "FILTER")
        if c % G or oc % G or cg != c // G:
            raise ValueError(f"Conv2D groups={G} does not divide channels {c} -> {oc} (filter has {cg} input channels)")
        self.in_nhwc = self.ex.is_nhwc(self.inputs["INPUT"])
        strides = K.nhwc_strides(n, c, h, w) if self.in_nhwc else K.nchw_strides(n, c, h, w)
        self.cstride = strides[1]
        self.g = g = K.ConvGeometry(n, cg, h, w, kh, kw, int(a["stride_h"]), int(a["stride_w"]), int(a["padding_h"]),
                                    int(a["padding_w"]), strides)
        self.oc, self.ocg, self.cg = oc, oc // G, cg
        self.act = _ACT[a.get("activation")]
        y = torch.empty(n, g.oh, g.ow, oc, dtype=x.dtype, device=x.device)
        self.out().data = y
        self.ex.mark_nhwc((self.nid, "OUTPUT"))
        self.y2d = y.view(g.rows, oc)
        self.direct, self.packed = False, True
        self.wp = torch.empty(G, self.ocg, g.kp, dtype=torch.bfloat16, device=x.device)
        self.bias = self.x("BIAS") if "BIAS" in self.inputs else None
        self.pre = torch.empty_like(self.y2d) if (self.act == "gelu" and self.ex.cfg.training) else None
        self.ex.need_big_scratch(g.rows * g.kp * 2, 2)
        self.ex.need_big_scratch(self.ocg * g.kp * 4, 3)
        self.ex.need_scratch(4 * K.bias_act_bwd_scratch(g.rows, oc))
        self._col = self._dcol = self._dwp = None

    def _group_input(self, t, j):
        return t.view(-1)[j * self.cg * self.cstride:]

    def _forward_grouped(self):
        g, G, ocg = self.g, self.groups, self.ocg
        w_ = self.x("FILTER").view(G, ocg, -1)
        if self._col is None:
            self._col = _scratch_view(self.ex, 0, (g.rows, g.kp), torch.bfloat16)
        for j in range(G):
            K.filter_pack(w_[j], self.wp[j], ocg, g.c, g.kh, g.kw, g.kp)
            K.im2col(self._group_input(self.x(), j), self._col, g)
            K.gemm_raw(M=g.rows, N=ocg, K=g.kp, A=self._col.data_ptr(), lda=g.kp, B=self.wp[j].data_ptr(), ldb=g.kp,
                       C=self.y2d.data_ptr() + j * ocg * 2, ldc=self.oc,
                       C2=None if self.pre is None else self.pre.data_ptr() + j * ocg * 2,
                       bias=None if self.bias is None else self.bias.data_ptr() + j * ocg * 2, act=K.ACT_CODES[self.act])

    def _backward_grouped(self, dy):
        g, G, ocg = self.g, self.groups, self.ocg
        wb, xb = self.buf("FILTER"), self.buf("INPUT")
        if self._dwp is None:
            self._dwp = _scratch_view(self.ex, 2, (ocg, g.kp), torch.float32)
            self._dcol = _scratch_view(self.ex, 1, (g.rows, g.kp), torch.bfloat16)
        for j in range(G):
            dyj = dy.data_ptr() + j * ocg * 2
            if wb.requires_grad:
                K.im2col(self._group_input(self.x(), j), self._col, g)
                # dW_j[ocg, kp] = dY_j^T . col  (both operands read along their rows: MN-major)
                K.gemm_raw(M=ocg, N=g.kp, K=g.rows, A=dyj, lda=self.oc, a_mn=True, B=self._col.data_ptr(), ldb=g.kp, b_mn=True,
                           C=self._dwp.data_ptr(), ldc=g.kp, out_fp32=True)
                K.filter_unpack(self._dwp, wb.grad.view(G, ocg, -1)[j], ocg, g.c, g.kh, g.kw, g.kp, accumulate=self.acc["FILTER"])
            if xb.requires_grad:
                K.gemm_raw(M=g.rows, N=g.kp, K=ocg, A=dyj, lda=self.oc, B=self.wp[j].data_ptr(), ldb=g.kp, b_mn=True,
                           C=self._dcol.data_ptr(), ldc=g.kp)
                K.col2im(self._dcol, self._group_input(xb.grad, j), g, accumulate=self.acc["INPUT"])

    def _operand(self):
        if self.direct:
            return self.x().view(self.g.rows, self.g.kp)
        if self._kept is not None:  # this convolution's own matrix, still valid in backward
            K.im2col(self.x(), self._kept, self.g)
            return self._kept
        if self._col is None:
            self._col = _scratch_view(self.ex, 0, (self.g.rows, self.g.kp), torch.bfloat16)
        K.im2col(self.x(), self._col, self.g)
        return self._col

    def forward(self):
        if self.groups != 1:
            return self._forward_grouped()
        if self.packed:
            g = self.g
            K.filter_pack(self.x("FILTER"), self.wp, self.oc, g.c, g.kh, g.kw, g.kp)
        if self.implicit:
            K.conv_fprop(self.x(), self.wp, self.out().data, self.g, self.oc, bias=self.bias, act=self.act, pre_act_out=self.pre)
            return
        K.matmul_nt(self._operand(), self.wp, out=self.y2d, bias=self.bias, act=self.act, pre_act_out=self.pre)

    def backward(self):
        g = self.g
        dy = self.out().grad.view(g.rows, self.oc)
        if self.act is not None or self.bias is not None:
            saved = self.pre if self.act == "gelu" else (self.y2d if self.act else None)
            bb = self.buf("BIAS") if self.bias is not None else None
            K.bias_act_bwd(dy, saved, dy if self.act else None, bb.grad if bb is not None else None, self.ex.scratch_f32(), self.act,
                           accumulate=self.acc.get("BIAS", False))
        if self.groups != 1:
            return self._backward_grouped(dy)
        wb = self.buf("FILTER")
        if self.implicit:
            if wb.requires_grad:
                if self._dwp is None:
                    self._dwp = _scratch_view(self.ex, 2, (self.oc, g.kp), torch.float32)
                K.conv_wgrad(self.x(), dy, self._dwp, g, self.oc)
                K.filter_unpack(self._dwp, wb.grad, self.oc, g.c, g.kh, g.kw, g.kp, accumulate=self.acc["FILTER"])
            xb = self.buf("INPUT")
            if xb.requires_grad:
                K.conv_dgrad(dy, self.wp, xb.grad, g, self.oc, accumulate=self.acc["INPUT"])
            return
        if wb.requires_grad:
            # the forward pass's matrix when it was kept, else recomputed (it is KH*KW times the activation)
            col = self._kept if self._kept is not None else self._operand()
            if self._dwp is None:
                self._dwp = _scratch_view(self.ex, 2, (self.oc, g.kp), torch.float32)
            K.matmul_tn(dy, col, out=self._dwp)
            K.filter_unpack(self._dwp, wb.grad, self.oc, g.c, g.kh, g.kw, g.kp, accumulate=self.acc["FILTER"])
        xb = self.buf("INPUT")
        if xb.requires_grad:
            if self.direct:
                K.matmul_nn(dy, self.wp, out=xb.grad.view(g.rows, g.kp), accumulate=self.acc["INPUT"])
            else:
                if self._dcol is None:
                    self._dcol = _scratch_view(self.ex, 1, (g.rows, g.kp), torch.bfloat16)
                K.matmul_nn(dy, self.wp, out=self._dcol)
                K.col2im(self._dcol, xb.grad, g, accumulate=self.acc["INPUT"])


# ------------------------------------------------------------------------------------------ Pool2D
@register("POOL2D")
class Pool2dOp(OpImpl):
    layout_aware = True

    def setup(self):
        a = self.attrs
        self.act = {"RELU": "relu", "SIGMOID": "sigmoid", "TANH": "tanh", "GELU": "gelu"}[a["activation"]] if a.get("activation") else None
        x = self.x()
        n, c, h, w = _sizes(self)
        self.in_nhwc = self.ex.is_nhwc(self.inputs["INPUT"])
        strides = K.nhwc_strides(n, c, h, w) if self.in_nhwc else K.nchw_strides(n, c, h, w)
        self.g = g = K.ConvGeometry(n, c, h, w, int(a["kernel_h"]), int(a["kernel_w"]), int(a["stride_h"]), int(a["stride_w"]),
                                    int(a["padding_h"]), int(a["padding_w"]), strides, kp=0)
        on, oc, oh, ow = [int(v) for v in dict(self.outputs)["OUTPUT"].piece_sizes]
        if (oh, ow) != (g.oh, g.ow):
            raise ValueError(f"Pool2D output extent {(oh, ow)} does not match its window geometry {(g.oh, g.ow)}")
        self.mode = "max" if a.get("pool_type", "MAX") == "MAX" else "avg"
        self.out().data = torch.empty(n, g.oh, g.ow, c, dtype=x.dtype, device=x.device)
        self.ex.mark_nhwc((self.nid, "OUTPUT"))
        self.arg = torch.empty(n * g.oh * g.ow * c, dtype=torch.uint8, device=x.device) \
            if (self.mode == "max" and self.ex.cfg.training) else None
        # fused activation (Pool2DAttrs.activation): the pooled values are kept for its backward
        self.pooled = torch.empty_like(self.out().data) if (self.act and self.ex.cfg.training) else None
        self.dpool = torch.empty_like(self.out().data) if self.pooled is not None else None

    def forward(self):
        y = self.out().data
        if self.act is None:
            K.pool2d_fwd(self.x(), y, self.arg, self.g, self.mode)
            return
        t = self.pooled if self.pooled is not None else y
        K.pool2d_fwd(self.x(), t, self.arg, self.g, self.mode)
        K.unary_fwd(self.act, t, out=y)

    def backward(self):
        b = self.buf("INPUT")
        if not b.requires_grad:
            return
        dy = self.out().grad.view(-1)
        if self.act is not None:
            K.unary_bwd(self.act, self.pooled.view(-1), self.out().data.view(-1), dy, dx=self.dpool.view(-1))
            dy = self.dpool.view(-1)
        K.pool2d_bwd(dy, self.arg, b.grad, self.g, self.mode, accumulate=self.acc["INPUT"])


# ------------------------------------------------------------------------------------------ BatchNorm
@register("BATCHNORM")
class BatchNormOp(OpImpl):
    """Training-mode batch normalisation (batch statistics) with the optional fused ReLU of the reference's
    BatchNormAttrs.  Under data parallelism the statistics are those of the local shard of the batch."""
    layout_aware = True

    def setup(self):
        x = self.x()
        n, c, h, w = _sizes(self)
        self.shape = (n, c, h, w)
        self.rows, self.cols = n * h * w, c
        self.in_nhwc = self.ex.is_nhwc(self.inputs["INPUT"]) or h * w == 1 or c == 1
        self.relu = bool(self.attrs.get("relu"))
        self.eps = float(self.attrs.get("eps", 1e-5))
        self.gamma = self.x("GAMMA") if "GAMMA" in self.inputs else None
        self.beta = self.x("BETA") if "BETA" in self.inputs else None
        self.out().data = torch.empty(n, h, w, c, dtype=x.dtype, device=x.device)
        self.ex.mark_nhwc((self.nid, "OUTPUT"))
        self.mean = torch.empty(c, dtype=torch.float32, device=x.device)
        self.rstd = torch.empty(c, dtype=torch.float32, device=x.device)
        self.xcl = None if self.in_nhwc else torch.empty(n, h, w, c, dtype=x.dtype, device=x.device)
        self.ex.need_scratch(4 * K.batchnorm_scratch(self.rows, self.cols))

    def _x(self):
        if self.in_nhwc:
            return self.x()
        n, c, h, w = self.shape
        K.permute(self.x().view(n, c, h, w), (0, 2, 3, 1), out=self.xcl)
        return self.xcl

    def forward(self):
        K.batchnorm_fwd(self._x(), self.out().data, self.gamma, self.beta, self.mean, self.rstd, self.ex.scratch_f32(), self.rows,
                        self.cols, self.eps, relu=self.relu)

    def backward(self):
        xb = self.buf("INPUT")
        gb = self.buf("GAMMA") if self.gamma is not None else None
        bb = self.buf("BETA") if self.beta is not None else None
        dy = self.out().grad.view(-1)
        x = self.x() if self.in_nhwc else self.xcl
        dx = None
        if xb.requires_grad:
            dx = xb.grad if self.in_nhwc else torch.empty_like(self.xcl)
        K.batchnorm_bwd(dy, x, self.out().data if self.relu else None, self.gamma, self.mean, self.rstd, dx,
                        gb.grad if gb is not None and gb.requires_grad else None,
                        bb.grad if bb is not None and bb.requires_grad else None, self.ex.scratch_f32(), self.rows, self.cols,
                        accumulate_dx=self.acc.get("INPUT", False) and self.in_nhwc,
                        accumulate_gamma=self.acc.get("GAMMA", False), accumulate_beta=self.acc.get("BETA", False))
        if dx is not None and not self.in_nhwc:
            n, c, h, w = self.shape
            K.permute(dx.view(n, h, w, c), (0, 3, 1, 2), out=xb.grad.view(n, c, h, w), accumulate=self.acc["INPUT"])


# ------------------------------------------------------------------------------------------ Concat / Split
def _phys_axis(shape4_nhwc: bool, axis: int, ndim: int):
    """Axis and extents in memory order for a logical axis of a tensor that may be stored channels-last."""
    if not shape4_nhwc:
        return axis
    return {0: 0, 1: 3, 2: 1, 3: 2}[axis]


def _phys_sizes(sizes, nhwc):
    if nhwc:
        n, c, h, w = sizes
        return [n, h, w, c]
    return list(sizes)


@register("CONCAT")
class ConcatOp(OpImpl):
    layout_aware = True

    def setup(self):
        k = int(self.attrs.get("num_inputs", len(self.inputs)))
        self.slots = [f"INPUT_{i}" for i in range(k)]
        flags = [self.ex.is_nhwc(self.inputs[s]) for s in self.slots]
        if any(flags) and not all(flags):
            raise NotImplementedError("Concat of channels-last and plain inputs")
        self.nhwc = all(flags) and len(_sizes(self, self.slots[0])) == 4
        out_sizes = [int(v) for v in dict(self.outputs)["OUTPUT"].piece_sizes]
        axis = int(self.attrs["axis"]) % len(out_sizes)
        pa = _phys_axis(self.nhwc, axis, len(out_sizes))
        po = _phys_sizes(out_sizes, self.nhwc)
        y = self.alloc_out(shape=po)
        if self.nhwc:
            self.ex.mark_nhwc((self.nid, "OUTPUT"))
        self.outer = 1
        for s in po[:pa]:
            self.outer *= s
        inner = 1
        for s in po[pa + 1:]:
            inner *= s
        self.dst_ld = po[pa] * inner
        self.blocks, off = [], 0
        for s in self.slots:
            ext = _phys_sizes(_sizes(self, s), self.nhwc)[pa] * inner
            self.blocks.append((s, off, ext))
            off += ext

    def forward(self):
        y = self.out().data
        for s, off, ext in self.blocks:
            K.block_copy(self.x(s), 0, ext, y, off, self.dst_ld, self.outer, ext)

    def backward(self):
        dy = self.out().grad
        for s, off, ext in self.blocks:
            b = self.buf(s)
            if b.requires_grad:
                K.block_copy(dy, off, self.dst_ld, b.grad, 0, ext, self.outer, ext, accumulate=self.acc[s])


@register("SPLIT")
class SplitOp(OpImpl):
    def setup(self):
        sizes = _sizes(self)
        axis = int(self.attrs["axis"]) % len(sizes)
        self.outer = 1
        for s in sizes[:axis]:
            self.outer *= s
        inner = 1
        for s in sizes[axis + 1:]:
            inner *= s
        self.src_ld = sizes[axis] * inner
        self.blocks, off = [], 0
        for slot, sh in self.outputs:
            ext = int(sh.piece_sizes[axis]) * inner
            self.alloc_out(slot)
            self.blocks.append((slot, off, ext))
            off += ext

    def forward(self):
        x = self.x()
        for slot, off, ext in self.blocks:
            K.block_copy(x, off, self.src_ld, self.out(slot).data, 0, ext, self.outer, ext)

    def backward(self):
        b = self.buf("INPUT")
        if not b.requires_grad:
            return
        acc = self.acc["INPUT"]
        live = {slot: self.out(slot).grad is not None and self.grad_written.get(slot, False) for slot, _, _ in self.blocks}
        if not acc and not all(live.values()):
            b.grad.zero_()  # parts nobody consumed contribute zero
        for slot, off, ext in self.blocks:
            g = self.out(slot).grad
            if live[slot]:
                K.block_copy(g, 0, ext, b.grad, off, self.src_ld, self.outer, ext, accumulate=acc)


# ------------------------------------------------------------------------------------------ Transpose / Reverse
@register("TRANSPOSE")
class TransposeOp(OpImpl):
    def setup(self):
        self.perm = [int(p) for p in self.attrs["permutation"]]
        self.inv = [self.perm.index(i) for i in range(len(self.perm))]
        self.alloc_out()

    def forward(self):
        K.permute(self.x(), self.perm, out=self.out().data)

    def backward(self):
        b = self.buf("INPUT")
        if b.requires_grad:
            K.permute(self.out().grad.view_as(self.out().data), self.inv, out=b.grad.view_as(self.x()), accumulate=self.acc["INPUT"])


@register("REVERSE")
class ReverseOp(OpImpl):
    def setup(self):
        self.axis = int(self.attrs["axis"]) % self.x().dim()
        self.alloc_out()

    def forward(self):
        K.reverse(self.x(), self.out().data, self.axis)

    def backward(self):
        b = self.buf("INPUT")
        if not b.requires_grad:
            return
        dy = self.out().grad.view_as(self.x())
        if self.acc["INPUT"]:
            t = torch.empty_like(dy)
            K.reverse(dy, t, self.axis)
            self.ex.write_grad(b, t, True)
        else:
            K.reverse(dy, b.grad.view_as(dy), self.axis)


# ------------------------------------------------------------------------------------------ Gather / TopK
@register("GATHER")
class GatherOp(OpImpl):
    def setup(self):
        self.dim = int(self.attrs["dim"]) % self.x().dim()
        self.alloc_out()

    def forward(self):
        K.gather(self.x(), self.x("INDEX"), self.out().data, self.dim)

    def backward(self):
        b = self.buf("INPUT")
        if not b.requires_grad:
            return
        if not self.acc["INPUT"]:
            b.grad.zero_()
        K.gather_bwd(self.out().grad.view_as(self.out().data), self.x("INDEX"), b.grad.view_as(self.x()), self.dim)


@register("TOPK")
class TopKOp(OpImpl):
    def setup(self):
        self.k = int(self.attrs["k"])
        self.alloc_out("OUTPUT")
        self.alloc_out("INDEX", dtype=torch.int32)

    def forward(self):
        K.topk(self.x(), self.k, vals=self.out("OUTPUT").data, idxs=self.out("INDEX").data)

    def backward(self):
        b = self.buf("INPUT")
        if b.requires_grad and self.out("OUTPUT").grad is not None:
            K.topk_bwd(self.out("OUTPUT").grad.view_as(self.out("OUTPUT").data), self.out("INDEX").data, b.grad.view_as(self.x()),
                       accumulate=self.acc["INPUT"])


# ------------------------------------------------------------------------------------------ Reduce / Broadcast
_REDUCE = {"REDUCE_SUM": "sum", "REDUCE_MEAN": "mean", "MEAN": "mean", "REDUCE_MAX": "max", "REDUCE_MIN": "min",
           "REDUCE_PROD": "prod"}


def _contiguous_run(axes, what):
    axes = sorted(axes)
    if axes != list(range(axes[0], axes[0] + len(axes))):
        raise NotImplementedError(f"{what} over non-adjacent axes {axes}")
    return axes


@register(*_REDUCE.keys())
class ReduceOp(OpImpl):
    def setup(self):
        self.op = _REDUCE[self.type]
        sizes = _sizes(self)
        axes = _contiguous_run([int(a) % len(sizes) for a in self.attrs["axes"]], "reduction")
        self.outer = self.red = self.inner = 1
        for i, s in enumerate(sizes):
            if i < axes[0]:
                self.outer *= s
            elif i > axes[-1]:
                self.inner *= s
            else:
                self.red *= s
        self.alloc_out()

    def forward(self):
        K.reduce(self.x(), self.out().data, self.outer, self.red, self.inner, self.op)

    def backward(self):
        b = self.buf("INPUT")
        if not b.requires_grad:
            return
        if self.op not in ("sum", "mean"):
            K.reduce_select_bwd(self.x().view(-1), self.out().data.view(-1), self.out().grad.view(-1), b.grad.view(-1), self.outer,
                                self.red, self.inner, self.op, accumulate=self.acc["INPUT"])
            return
        K.reduce_bwd(self.out().grad.view(-1), b.grad.view(-1), self.outer, self.red, self.inner,
                     1.0 if self.op == "sum" else 1.0 / self.red, accumulate=self.acc["INPUT"])


@register("BROADCAST")
class BroadcastOp(OpImpl):
    def setup(self):
        tgt = [int(v) for v in dict(self.outputs)["OUTPUT"].piece_sizes]
        src = _sizes(self)
        pad = [1] * (len(tgt) - len(src)) + src
        self.src_view = pad
        self.tgt = tgt
        self.bcast_axes = [i for i, (a, b) in enumerate(zip(pad, tgt)) if a == 1 and b > 1]
        self.alloc_out()

    def forward(self):
        x = self.x().view(self.src_view).expand(self.tgt)
        K.permute(x, list(range(len(self.tgt))), out=self.out().data)

    def backward(self):
        b = self.buf("INPUT")
        if not b.requires_grad:
            return
        dy = self.out().grad.view(self.tgt)
        if not self.bcast_axes:
            self.ex.write_grad(b, dy, self.acc["INPUT"])
            return
        axes = _contiguous_run(self.bcast_axes, "broadcast gradient")
        outer = red = inner = 1
        for i, s in enumerate(self.tgt):
            if i < axes[0]:
                outer *= s
            elif i > axes[-1]:
                inner *= s
            else:
                red *= s
        if self.acc["INPUT"]:
            t = torch.empty(outer * inner, dtype=dy.dtype, device=dy.device)
            K.reduce(dy, t, outer, red, inner, "sum")
            self.ex.write_grad(b, t, True)
        else:
            K.reduce(dy, b.grad.view(-1), outer, red, inner, "sum")
