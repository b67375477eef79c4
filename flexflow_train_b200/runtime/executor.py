"""GPU executor: runs a (parallel) computation graph with the sm_100a kernel library.

Counterpart of the reference's local executor
(lib/local-execution/src/local-execution/computation_graph_instance.cc:61-155) and, with a
``DistContext``, of its distributed executor (lib/realm-execution/src/realm-execution/pcg_instance.cc):
the graph is lowered once into a static plan -- per operator a forward and a backward closure over
pre-allocated tensors -- and a training step replays the plan (optionally as one CUDA graph).

Differences from the reference that matter for speed:
  * every rank runs the same program on its own shard (SPMD) instead of one controller that
    serialises task arguments to JSON for each launch;
  * parameters, gradients and optimizer state live in flat arenas, so the optimizer is one launch;
  * gradients are written, not accumulated, by their first producer, so no buffer is zeroed per step
    (the reference accumulates with beta = 1 everywhere and zeroes all gradients each iteration);
  * pointwise neighbours are fused into the producing kernel (bias/activation in the GEMM epilogue,
    residual add in LayerNorm, softmax in the cross-entropy loss).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch

from .. import _ffcore as core
from ..ops import kernels as K
from .initializers import initialize

Value = Tuple[int, str]

_TORCH_DT = {"FLOAT": torch.float32, "DOUBLE": torch.float64, "HALF": torch.float16, "BFLOAT16": torch.bfloat16,
             "INT32": torch.int32, "INT64": torch.int64, "BOOL": torch.bool}


@dataclass
class OptimizerConfig:
    """SGDOptimizerAttrs / AdamOptimizerAttrs of the reference (lib/pcg/src/pcg/optimizer_attrs.cc:7-45)."""
    kind: str = "adam"  # "adam" | "sgd"
    lr: float = 1e-3
    momentum: float = 0.0
    nesterov: bool = False
    weight_decay: float = 0.0
    beta1: float = 0.9
    beta2: float = 0.999
    epsilon: float = 1e-8


@dataclass
class ExecConfig:
    compute_dtype: str = "bf16"          # "bf16" (fp32 master weights) or "fp32" (tf32 tensor cores)
    loss: Optional[str] = "sparse_categorical_crossentropy"
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    seed: int = 0
    use_cuda_graph: bool = False
    device: str = "cuda"
    training: bool = True
    causal_attention: bool = False
    profile_layers: bool = False
    # Apply a Dropout that follows a Linear inside that GEMM's epilogue.  Off by default: measured on the large
    # Transformer it costs more in the epilogue (which is on the GEMM's critical path) than the separate
    # bandwidth-bound dropout kernel it removes (343.8 vs 335.2 ms per step; 291.5 vs 287.4 ms with the cheaper mask generator).
    fuse_dropout: bool = False
    fold_dropout_backward: bool = True  # Linear -> Dropout: mask the gradient inside the Linear's bias/activation backward
    keep_dropped_probs: bool = True  # attention: keep dropout(P) for backward when device memory allows
    # Attention core (scores, softmax, dropout, context) in one tcgen05 kernel per direction, without a score tensor in
    # global memory, where the head dimension is covered (ops/kernels.py: attention_supported); otherwise the
    # batched-GEMM + softmax path below runs.
    fused_attention: bool = True
    # Attention core in blocks: scores, probabilities and their gradients of a few batch elements (or head groups)
    # at a time live in small reused buffers and backward recomputes the probabilities of a block, so no
    # B x H x S x S tensor is ever stored (saves 2 such tensors per layer; 48 GB on the large Transformer).
    # Value: target bytes of one block's score tensor; 0 = off (whole-batch kernels, probabilities saved), which
    # is faster when the memory is there: 329.9 vs 371.8 ms per step on the large Transformer with 32 MB blocks --
    # many small kernels with partial last waves cost more than the HBM round trips they avoid.
    attention_block_bytes: int = 0
    # Embedding tables trained by plain SGD (no momentum, no weight decay) are kept as fp32 tables outside the
    # parameter arenas and updated row by row from the output gradient inside the Embedding's backward, so a
    # step touches batch x dim elements of a table instead of the whole table three times (gradient clear,
    # dense scatter target, dense update).
    sparse_embedding_update: bool = True
    # K x K convolutions: keep the forward pass's im2col matrix for the weight-gradient GEMM instead of recomputing
    # it in backward (it is KH*KW times the activation, so this trades memory for one im2col pass per convolution
    # and step).  Value: total bytes that may be kept, claimed by the convolutions in graph order; 0 = recompute.
    keep_im2col_bytes: int = 48 << 30
    # stride-1 convolutions over channels-last data as an implicit GEMM (shifted TMA boxes of the activation, no im2col
    # matrix); off = every K x K convolution goes through im2col + GEMM
    implicit_conv: bool = True


class _Buf:
    """A tensor slot of the plan: data plus (optionally) gradient."""
    __slots__ = ("data", "grad", "requires_grad", "shape")

    def __init__(self, data=None, requires_grad=False):
        self.data = data
        self.grad = None
        self.requires_grad = requires_grad


class _GradPool:
    """Reuses gradient buffers whose lifetimes do not overlap (plan-time, so addresses stay static)."""

    def __init__(self, device):
        self.free: Dict[Tuple[int, torch.dtype], List[torch.Tensor]] = {}
        self.device = device
        self.total_bytes = 0

    def take(self, numel, dtype):
        key = (numel, dtype)
        lst = self.free.get(key)
        if lst:
            return lst.pop()
        self.total_bytes += numel * torch.empty((), dtype=dtype).element_size()
        return torch.empty(numel, dtype=dtype, device=self.device)

    def give(self, t):
        self.free.setdefault((t.numel(), t.dtype), []).append(t)


class OpImpl:
    """Base class of operator implementations.  ``setup`` allocates outputs; ``forward`` /
    ``backward`` launch kernels only."""

    def __init__(self, ex: "Executable", nid: int, node: dict):
        self.ex = ex
        self.nid = nid
        self.node = node
        self.attrs = node["attrs"]
        self.type = node["type"]
        self.inputs: Dict[str, Value] = {s: tuple(v) for s, v in node["inputs"]}
        self.outputs = [(s, sh) for s, sh, _ in node["outputs"]]
        self.acc: Dict[str, bool] = {}  # per input slot: accumulate into its grad?

    # helpers
    def buf(self, slot) -> _Buf:
        return self.ex.values[self.inputs[slot]]

    def x(self, slot="INPUT"):
        return self.buf(slot).data

    def out(self, slot="OUTPUT") -> _Buf:
        return self.ex.values[(self.nid, slot)]

    def alloc_out(self, slot="OUTPUT", dtype=None, shape=None):
        sh = dict(self.outputs)[slot]
        shape = list(sh.piece_sizes) if shape is None else shape
        dt = self.ex.torch_dtype(sh.dtype) if dtype is None else dtype
        t = self.ex.allocator.allocate(shape, dt)
        self.out(slot).data = t
        return t

    def setup(self):
        raise NotImplementedError

    def forward(self):
        raise NotImplementedError

    def backward(self):
        pass

    def grad_inputs(self) -> List[str]:
        """input slots that receive a gradient from this op"""
        return [s for s, v in self.inputs.items() if self.ex.values[v].requires_grad]

    def extra_grad_targets(self):
        """(pseudo slot, value) pairs whose gradient this operator's backward writes although the value is not
        one of its inputs; the accumulate flag arrives in ``self.acc[pseudo slot]``."""
        fi = getattr(self, "fuse_in", None)
        return [("FUSE_IN", fi.combine.inputs["INPUT"])] if fi is not None else []

    def extra_grad_sources(self):
        """Values whose gradient this operator's backward reads although they are not its outputs."""
        fo = getattr(self, "fuse_out", None)
        out = [(fo.repartition.nid, "OUTPUT")] if fo is not None else []
        d = getattr(self, "bwd_dropout", None)
        if d is not None:
            out.append((d.nid, "OUTPUT"))
        return out


_REGISTRY: Dict[str, type] = {}


def register(*types):
    def deco(cls):
        for t in types:
            _REGISTRY[t] = cls
        return cls
    return deco


# ------------------------------------------------------------------------------------------ leaf ops
@register("INPUT")
class InputOp(OpImpl):
    def setup(self):
        self.alloc_out()

    def forward(self):
        pass


@register("WEIGHT")
class WeightOp(OpImpl):
    def setup(self):
        pass  # bound to the parameter arena by the executable

    def forward(self):
        pass


@register("NOOP", "IDENTITY")
class NoopOp(OpImpl):
    def setup(self):
        self.out().data = self.x()

    def forward(self):
        pass

    def backward(self):
        g = self.out().grad
        b = self.buf("INPUT")
        if b.requires_grad:
            self.ex.write_grad(b, g, self.acc["INPUT"])


class SkippedOp(OpImpl):
    """An operator whose result nobody on this rank needs (e.g. the Combine that would gather the model output
    although the loss is taken on the local shard)."""

    def setup(self):
        pass

    def forward(self):
        pass


# ------------------------------------------------------------------------------------------ Linear
_ACT = {None: None, "RELU": "relu", "GELU": "gelu", "SIGMOID": "sigmoid", "TANH": "tanh"}


@register("LINEAR")
class LinearOp(OpImpl):
    """y = act(x W^T + b).  Under tensor parallelism the distributed executable may attach ``fuse_in`` (the
    input arrives as row shards: all-gather fused into this GEMM) or ``fuse_out`` (the output is a partial sum
    that is wanted as row shards: reduce-scatter fused into this GEMM); see parallel/dist_executor.py."""
    fuse_in = None
    fuse_out = None
    fused_dropout = None  # a Dropout that directly follows: applied by this GEMM's epilogue, undone in its backward
    bwd_dropout = None    # a Dropout that directly follows and runs as its own kernel in forward; its backward (masking
                          # the incoming gradient) is folded into this operator's bias/activation backward pass

    def _drop(self):
        d = self.fused_dropout
        return None if d is None else (d.p, d.salt, self.ex.seed_tensor)

    def setup(self):
        self.act = _ACT[self.attrs.get("activation")]
        if self.fuse_out is None:
            y = self.alloc_out()
            self.y2d = y.view(-1, y.shape[-1])
        else:
            self.y2d = None  # the reduced shards land in the Repartition's output
        x = self.x()
        self.x2d = x.view(-1, x.shape[-1])
        self.w = self.x("WEIGHT")
        self.bias = self.x("BIAS") if ("BIAS" in self.inputs and self.ex.use_bias(self, "BIAS")) else None
        # a bias this rank holds but does not add (row-parallel shard): its gradient is still the column sum of dY
        self.bias_grad = self.bias is not None or ("BIAS" in self.inputs and self.ex.bias_grad_without_use(self, "BIAS"))
        rows, cols = self.x2d.shape[0], self.w.shape[0]
        self.pre = torch.empty(rows, cols, dtype=x.dtype, device=x.device) if (self.act == "gelu" and self.ex.cfg.training) else None
        self.ex.need_scratch(4 * K.bias_act_bwd_scratch(rows, cols) if K.available() and self.ex.on_gpu else 0)
        # A small layer under a large batch: the weight gradient has a handful of output tiles and a reduction over
        # thousands of rows.  Computed into an fp32 scratch, the GEMM splits that reduction over all SMs (one CTA
        # streaming 4096 rows takes ~25 us; 148 CTAs sharing them a few); a cast then adds it into the bf16 gradient.
        if self.ex.cfg.training and self.ex.wgrad_splits(rows, cols, self.w.shape[1], x.dtype):
            self.ex.need_scratch(4 * cols * self.w.shape[1])

    def forward(self):
        if self.fuse_in is not None:
            self.fuse_in.gemm(self.w, self.y2d, bias=self.bias, act=self.act, pre_act_out=self.pre, dropout=self._drop())
        elif self.fuse_out is not None:
            self.fuse_out.gemm(self.x2d, self.w, bias=self.bias)
        else:
            K.matmul_nt(self.x2d, self.w, out=self.y2d, bias=self.bias, act=self.act, pre_act_out=self.pre, dropout=self._drop())

    def backward(self):
        xb = self.buf("INPUT")
        if self.fuse_out is not None:
            # gathers the row shards of dY from all ranks and, in the same kernel, computes dX = dY W
            dy = self.fuse_out.gather_grad_gemm(self.w, xb.grad.view_as(self.x2d) if xb.requires_grad else None,
                                                accumulate=self.acc.get("INPUT", False))
        else:
            dy = self.out().grad.view_as(self.y2d)
        if self.bwd_dropout is not None:
            d = self.bwd_dropout
            src = d.out().grad.view_as(self.y2d)  # gradient w.r.t. the dropped output; masked and passed on in one pass
            saved = self.pre if self.act == "gelu" else (self.y2d if self.act else None)
            bb = self.buf("BIAS") if self.bias_grad else None
            K.bias_act_bwd(src, saved, dy, bb.grad if bb is not None else None, self.ex.scratch_f32(), self.act,
                           accumulate=self.acc.get("BIAS", False), dropout=(d.p, d.salt, self.ex.seed_tensor))
        elif self.act is not None or self.bias_grad or self.fused_dropout is not None:
            saved = self.pre if self.act == "gelu" else (self.y2d if self.act else None)
            bb = self.buf("BIAS") if self.bias_grad else None
            rewrite = self.act is not None or self.fused_dropout is not None
            K.bias_act_bwd(dy, saved, dy if rewrite else None, bb.grad if bb is not None else None,
                           self.ex.scratch_f32(), self.act, accumulate=self.acc.get("BIAS", False), dropout=self._drop())
        wb = self.buf("WEIGHT")
        if wb.requires_grad:
            self.ex.wgrad_gemm(dy, self.x2d, wb.grad, self.acc["WEIGHT"])
        if self.fuse_out is not None:
            return
        if self.fuse_in is not None:
            # dX partial sums -> reduce-scatter into the row shard's gradient
            self.fuse_in.grad_gemm(dy, self.w, self.acc.get("FUSE_IN", False))
        elif xb.requires_grad:
            K.matmul_nn(dy, self.w, out=xb.grad.view_as(self.x2d), accumulate=self.acc["INPUT"])


@register("BATCHMATMUL")
class BatchMatmulOp(OpImpl):
    """out[b, n, p] = lhs[b, n, m] @ rhs[b, m, p] (declared but unimplemented in the reference)."""

    def setup(self):
        self.a, self.b = self.x("LHS_INPUT"), self.x("RHS_INPUT")
        self.c = self.alloc_out()
        *batch, self.n, self.m = self.a.shape
        self.p = self.b.shape[-1]
        self.nb = 1
        for s in batch:
            self.nb *= s

    def _gemm(self, A, a_mn, lda, a_sb, B, b_mn, ldb, b_sb, C, ldc, c_sb, M, N, Kd, acc):
        if A.dtype == torch.float32:  # MN-major operands need 16-bit storage: run the product in bf16
            A16, B16 = torch.empty_like(A, dtype=torch.bfloat16), torch.empty_like(B, dtype=torch.bfloat16)
            K.cast(A, A16)
            K.cast(B, B16)
            A, B = A16, B16
        K.gemm_raw(M=M, N=N, K=Kd, A=A.data_ptr(), lda=lda, a_mn=a_mn, a_sb=a_sb, B=B.data_ptr(), ldb=ldb, b_mn=b_mn,
                   b_sb=b_sb, C=C.data_ptr(), ldc=ldc, c_sb=c_sb, nb=self.nb, es=A.element_size(),
                   out_fp32=C.dtype == torch.float32, accumulate=acc)

    def forward(self):
        n, m, p = self.n, self.m, self.p
        self._gemm(self.a, False, m, n * m, self.b, True, p, m * p, self.c, p, n * p, n, p, m, False)

    def backward(self):
        n, m, p = self.n, self.m, self.p
        dc = self.out().grad
        ab, bb = self.buf("LHS_INPUT"), self.buf("RHS_INPUT")
        if ab.requires_grad:  # dA[n, m] = dC[n, p] . B[m, p]^T
            self._gemm(dc, False, p, n * p, self.b, False, p, m * p, ab.grad, m, n * m, n, m, p, self.acc["LHS_INPUT"])
        if bb.requires_grad:  # dB[m, p] = A[n, m]^T . dC[n, p]
            self._gemm(self.a, True, m, n * m, dc, True, p, n * p, bb.grad, p, m * p, m, p, n, self.acc["RHS_INPUT"])


# ------------------------------------------------------------------------------------------ attention
@register("MULTIHEAD_ATTENTION")
class AttentionOp(OpImpl):
    """Multi-head attention with packed projections.

    The WEIGHT tensor has the reference's element count
    ((q_in*kdim + k_in*kdim + v_in*vdim + vdim*embed) * heads, lib/op-attrs/src/op-attrs/ops/attention.cc:97-112)
    and is laid out here as four row-major blocks Wq [H*kdim, q_in], Wk [H*kdim, k_in], Wv [H*vdim, v_in],
    Wo [embed, H*vdim], so that self-attention runs one fused QKV GEMM.  Scores are scaled by 1/sqrt(kdim).
    """
    fuse_in = None   # see LinearOp: all-gather fused into the QKV projection
    fuse_out = None  # reduce-scatter fused into the output projection

    def setup(self):
        a = self.attrs
        ex = self.ex
        self.H = int(a["num_heads"]) // ex.head_shards(self)
        self.kd, self.vd, self.embed = int(a["kdim"]), int(a["vdim"]), int(a["embed_dim"])
        self.p_drop = float(a.get("dropout", 0.0)) if ex.cfg.training else 0.0
        q, k, v = self.x("QUERY"), self.x("KEY"), self.x("VALUE")
        self.B, self.Sq, self.dq = q.shape
        self.Sk, self.dk, self.dv = k.shape[1], k.shape[2], v.shape[2]
        self.self_attn = self.inputs["QUERY"] == self.inputs["KEY"] == self.inputs["VALUE"]
        if not self.self_attn:
            self.fuse_in = None
        H, kd, vd = self.H, self.kd, self.vd
        w = self.x("WEIGHT").view(-1)
        o0 = 0
        self.wq = w[o0:o0 + H * kd * self.dq].view(H * kd, self.dq); o0 += H * kd * self.dq
        self.wk = w[o0:o0 + H * kd * self.dk].view(H * kd, self.dk); o0 += H * kd * self.dk
        self.wv = w[o0:o0 + H * vd * self.dv].view(H * vd, self.dv); o0 += H * vd * self.dv
        self.wo = w[o0:o0 + self.embed * H * vd].view(self.embed, H * vd)
        dt = q.dtype
        dev = ex.device
        self.ldqkv = H * (2 * kd + vd)
        if self.self_attn:
            self.wqkv = w[:self.ldqkv * self.dq].view(self.ldqkv, self.dq)
            self.qkv = torch.empty(self.B * self.Sq, self.ldqkv, dtype=dt, device=dev)
            self.qv = self.qkv[:, :H * kd]
            self.kv = self.qkv[:, H * kd:2 * H * kd]
            self.vv = self.qkv[:, 2 * H * kd:]
            self.ldq = self.ldk = self.ldv = self.ldqkv
        else:
            self.qv = torch.empty(self.B * self.Sq, H * kd, dtype=dt, device=dev)
            self.kv = torch.empty(self.B * self.Sk, H * kd, dtype=dt, device=dev)
            self.vv = torch.empty(self.B * self.Sk, H * vd, dtype=dt, device=dev)
            self.ldq, self.ldk, self.ldv = H * kd, H * kd, H * vd
        # The batched core (scores, probabilities, context) always runs on bf16 tensor cores; with fp32
        # activations the projections stay fp32/tf32 and q, k, v, ctx are cast at the boundary.
        self.core16 = dt != torch.bfloat16
        cdt = torch.bfloat16
        if self.core16:
            if self.self_attn:
                self.c_qkv = torch.empty_like(self.qkv, dtype=cdt)
                self.c_q, self.c_k, self.c_v = self.c_qkv[:, :H * kd], self.c_qkv[:, H * kd:2 * H * kd], self.c_qkv[:, 2 * H * kd:]
            else:
                self.c_q, self.c_k, self.c_v = (torch.empty_like(t, dtype=cdt) for t in (self.qv, self.kv, self.vv))
            self.c_ctx = torch.empty(self.B * self.Sq, H * vd, dtype=cdt, device=dev)
        else:
            self.c_q, self.c_k, self.c_v = self.qv, self.kv, self.vv
        self.fused = bool(ex.on_gpu and ex.cfg.fused_attention and kd == vd and K.attention_supported(kd, backward=ex.cfg.training)
                          and (not ex.cfg.causal_attention or self.Sq == self.Sk))
        per_batch = H * self.Sq * self.Sk * 2
        blk = int(ex.cfg.attention_block_bytes)
        self.cb = 0   # batch elements per block (0 = unblocked)
        self.hb = H   # heads per block
        if self.fused:
            self.lse = torch.empty(self.B, H, self.Sq, dtype=torch.float32, device=dev)
            if ex.cfg.training:   # delta [B, H, Sq] followed by the fp32 dK / dV accumulators
                ex.need_scratch(4 * (self.B * H * self.Sq + 4 + K.attention_bwd_scratch_floats(self.B, H, self.Sq, kd)))
        elif ex.on_gpu and blk > 0 and self.B * per_batch > 2 * blk:
            if per_batch <= blk:
                self.cb = max(1, min(self.B, blk // per_batch))
            else:  # one batch element at a time, a group of heads per block
                self.cb = 1
                self.hb = max(1, min(H, (H * blk) // per_batch))
                while H % self.hb:
                    self.hb -= 1
        self.probs = torch.empty(self.B if not (self.cb or self.fused) else 0, H, self.Sq, self.Sk, dtype=cdt, device=dev)
        self.ctx = torch.empty(self.B * self.Sq, H * vd, dtype=dt, device=dev)
        if not self.core16:
            self.c_ctx = self.ctx
        if self.fuse_out is None:
            self.alloc_out()
        self.bias_in = self.x("INPUT_BIAS") if "INPUT_BIAS" in self.inputs else None
        self.bias_out = self.x("OUTPUT_BIAS") if ("OUTPUT_BIAS" in self.inputs and ex.use_bias(self, "OUTPUT_BIAS")) else None
        self.bias_out_grad = self.bias_out is not None or ("OUTPUT_BIAS" in self.inputs and ex.bias_grad_without_use(self, "OUTPUT_BIAS"))
        self.alpha = 1.0 / math.sqrt(kd)
        nbytes = self.probs.numel() * self.probs.element_size()
        if self.cb:
            self.kept_p = None
            # scores/probabilities, dropped probabilities, d(scores) of one block
            ex.need_big_scratch(self.cb * self.hb * self.Sq * self.Sk * 2, 3)
        # The dropped probabilities feed the P.V GEMM and, in backward, the dV GEMM.  Keeping them costs one
        # score-sized tensor per layer and saves regenerating them (a read and a write of that tensor); it is
        # done while plenty of device memory is free, otherwise they are rebuilt in a shared scratch buffer.
        self.kept_p = None
        if not self.cb and not self.fused and self.p_drop > 0 and ex.cfg.training and ex.on_gpu and ex.cfg.keep_dropped_probs:
            free, _total = torch.cuda.mem_get_info(ex.device)
            if free > 8 * nbytes + (40 << 30):
                self.kept_p = torch.empty_like(self.probs)
        if not self.cb and not self.fused:
            ex.need_big_scratch(nbytes, 2 if (self.p_drop > 0 and self.kept_p is None) else 1)
        ex.need_scratch(4 * K.bias_act_bwd_scratch(self.B * self.Sq, max(self.ldqkv, self.embed)) if ex.on_gpu else 0)
        if ex.cfg.training and ex.wgrad_splits(self.B * self.Sq, self.embed, self.H * self.vd, torch.bfloat16):
            ex.need_scratch(4 * self.embed * self.H * self.vd)
        self.salt = ex.next_salt()
        self.es = 2
        if self.ex.cfg.training:
            if self.self_attn:
                self.dqkv = torch.empty_like(self.qkv)
                self.dq_, self.dk_, self.dv_ = (self.dqkv[:, :H * kd], self.dqkv[:, H * kd:2 * H * kd], self.dqkv[:, 2 * H * kd:])
            else:
                self.dq_, self.dk_, self.dv_ = torch.empty_like(self.qv), torch.empty_like(self.kv), torch.empty_like(self.vv)
            self.dctx = torch.empty_like(self.ctx)
            if self.core16:
                if self.self_attn:
                    self.c_dqkv = torch.empty_like(self.c_qkv)
                    self.c_dq, self.c_dk, self.c_dv = (self.c_dqkv[:, :H * kd], self.c_dqkv[:, H * kd:2 * H * kd], self.c_dqkv[:, 2 * H * kd:])
                else:
                    self.c_dq, self.c_dk, self.c_dv = (torch.empty_like(t) for t in (self.c_q, self.c_k, self.c_v))
                self.c_dctx = torch.empty_like(self.c_ctx)
            else:
                self.c_dq, self.c_dk, self.c_dv, self.c_dctx = self.dq_, self.dk_, self.dv_, self.dctx

    # batched GEMM over (head, batch) on strided [tokens, H*d] views
    def _bg(self, M, N, Kd, A, lda, a_sh, a_sb, a_mn, Bm, ldb, b_sh, b_sb, b_mn, C, ldc, c_sh, c_sb, alpha=1.0, nb=None, nh=None):
        K.gemm_raw(M=M, N=N, K=Kd, A=A.data_ptr(), lda=lda, a_sh=a_sh, a_sb=a_sb, a_mn=a_mn, B=Bm.data_ptr(), ldb=ldb,
                   b_sh=b_sh, b_sb=b_sb, b_mn=b_mn, C=C.data_ptr(), ldc=ldc, c_sh=c_sh, c_sb=c_sb, nh=self.H if nh is None else nh,
                   nb=self.B if nb is None else nb, alpha=alpha, es=self.es, out_fp32=C.dtype == torch.float32)

    # ---- L2-blocked core: batch elements [b0, b0 + n) x heads [h0, h0 + hb) at a time in reused block buffers
    def _blocks(self):
        ci = 0
        for b0 in range(0, self.B, self.cb):
            for h0 in range(0, self.H, self.hb):
                yield ci, b0, min(self.cb, self.B - b0), h0
                ci += 1

    def _block_buffers(self, n):
        shape = (n, self.hb, self.Sq, self.Sk)
        nbytes = n * self.hb * self.Sq * self.Sk * 2
        return [self.ex._big[i][:nbytes].view(torch.bfloat16).view(shape) for i in range(3)]

    def _rows(self, t, b0, n, S, h0, d):
        """Rows of batch elements [b0, b0+n) and the columns of heads [h0, h0+hb) of a [tokens, H*d] view."""
        return t[b0 * S:(b0 + n) * S, h0 * d:(h0 + self.hb) * d]

    def _block_probs(self, ci, b0, n, h0, S, Pd):
        """S <- softmax(alpha * q k^T) for the block; Pd <- dropout(S) when dropout is on.  Returns the operand of P.V"""
        hb, kd, Sq, Sk = self.hb, self.kd, self.Sq, self.Sk
        q, k = self._rows(self.c_q, b0, n, Sq, h0, kd), self._rows(self.c_k, b0, n, Sk, h0, kd)
        self._bg(Sq, Sk, kd, q, self.ldq, kd, Sq * self.ldq, False, k, self.ldk, kd, Sk * self.ldk, False, S, Sk, Sq * Sk, hb * Sq * Sk,
                 alpha=self.alpha, nb=n, nh=hb)
        causal_q = Sq if self.ex.cfg.causal_attention else 0
        salt = self.salt + 0x51ED27 * (ci + 1)  # every block draws its own mask, the same in forward and backward
        if self.p_drop > 0 and K.softmax_dropout_supported(S):
            K.softmax_dropout_fwd(S, S, Pd, self.p_drop, salt, self.ex.seed_tensor, causal_q=causal_q)
            return Pd, salt
        K.softmax_fwd(S, out=S, causal_q=causal_q)
        if self.p_drop > 0:
            K.dropout(S, self.p_drop, salt, out=Pd, seed_tensor=self.ex.seed_tensor)
            return Pd, salt
        return S, salt

    def _forward_core_blocked(self):
        hb, vd, Sq, Sk, Hvd = self.hb, self.vd, self.Sq, self.Sk, self.H * self.vd
        for ci, b0, n, h0 in self._blocks():
            S, Pd, _ = self._block_buffers(n)
            p, _salt = self._block_probs(ci, b0, n, h0, S, Pd)
            v = self._rows(self.c_v, b0, n, Sk, h0, vd)
            self._bg(Sq, vd, Sk, p, Sk, Sq * Sk, hb * Sq * Sk, False, v, self.ldv, vd, Sk * self.ldv, True,
                     self._rows(self.c_ctx, b0, n, Sq, h0, vd), Hvd, vd, Sq * Hvd, nb=n, nh=hb)

    def _backward_core_blocked(self):
        hb, kd, vd, Sq, Sk, Hvd = self.hb, self.kd, self.vd, self.Sq, self.Sk, self.H * self.vd
        for ci, b0, n, h0 in self._blocks():
            S, Pd, dP = self._block_buffers(n)
            p, salt = self._block_probs(ci, b0, n, h0, S, Pd)  # recomputed: nothing of size B*H*S*S is ever stored
            q, k = self._rows(self.c_q, b0, n, Sq, h0, kd), self._rows(self.c_k, b0, n, Sk, h0, kd)
            v, dctx = self._rows(self.c_v, b0, n, Sk, h0, vd), self._rows(self.c_dctx, b0, n, Sq, h0, vd)
            self._bg(Sq, Sk, vd, dctx, Hvd, vd, Sq * Hvd, False, v, self.ldv, vd, Sk * self.ldv, False, dP, Sk, Sq * Sk, hb * Sq * Sk,
                     nb=n, nh=hb)
            self._bg(Sk, vd, Sq, p, Sk, Sq * Sk, hb * Sq * Sk, True, dctx, Hvd, vd, Sq * Hvd, True,
                     self._rows(self.c_dv, b0, n, Sk, h0, vd), self.ldv, vd, Sk * self.ldv, nb=n, nh=hb)
            if K.softmax_dropout_supported(S):
                K.softmax_dropout_bwd(dP, S, dP, self.p_drop, salt, self.ex.seed_tensor, scale=self.alpha)
            else:
                if self.p_drop > 0:
                    K.dropout(dP, self.p_drop, salt, out=dP, seed_tensor=self.ex.seed_tensor)
                K.softmax_bwd(dP, S, dx=dP, scale=self.alpha)
            self._bg(Sq, kd, Sk, dP, Sk, Sq * Sk, hb * Sq * Sk, False, k, self.ldk, kd, Sk * self.ldk, True,
                     self._rows(self.c_dq, b0, n, Sq, h0, kd), self.ldq, kd, Sq * self.ldq, nb=n, nh=hb)
            self._bg(Sk, kd, Sq, dP, Sk, Sq * Sk, hb * Sq * Sk, True, q, self.ldq, kd, Sq * self.ldq, True,
                     self._rows(self.c_dk, b0, n, Sk, h0, kd), self.ldk, kd, Sk * self.ldk, nb=n, nh=hb)

    def forward(self):
        H, kd, vd, Sq, Sk = self.H, self.kd, self.vd, self.Sq, self.Sk
        q2 = self.x("QUERY").view(-1, self.dq)
        if self.fuse_in is not None:
            self.fuse_in.gemm(self.wqkv, self.qkv, bias=self.bias_in)
        elif self.self_attn:
            K.matmul_nt(q2, self.wqkv, out=self.qkv, bias=self.bias_in)
        else:
            K.matmul_nt(q2, self.wq, out=self.qv)
            K.matmul_nt(self.x("KEY").view(-1, self.dk), self.wk, out=self.kv)
            K.matmul_nt(self.x("VALUE").view(-1, self.dv), self.wv, out=self.vv)
        if self.core16:
            if self.self_attn:
                K.cast(self.qkv, self.c_qkv)
            else:
                K.cast(self.qv, self.c_q); K.cast(self.kv, self.c_k); K.cast(self.vv, self.c_v)
        if self.fused:
            K.attention_fwd(self.c_q, self.c_k, self.c_v, self.c_ctx, self.lse, B=self.B, H=H, Sq=Sq, Sk=Sk, D=kd, scale=self.alpha,
                            causal=self.ex.cfg.causal_attention, dropout=self._fused_dropout())
            return self._forward_out()
        if self.cb:
            self._forward_core_blocked()
            return self._forward_out()
        # scores[b,h,sq,sk] = alpha * q . k^T
        self._bg(Sq, Sk, kd, self.c_q, self.ldq, kd, Sq * self.ldq, False, self.c_k, self.ldk, kd, Sk * self.ldk, False,
                 self.probs, Sk, Sq * Sk, H * Sq * Sk, alpha=self.alpha)
        causal_q = Sq if self.ex.cfg.causal_attention else 0
        p = self.probs
        if self.p_drop > 0 and K.softmax_dropout_supported(self.probs):
            # probabilities and their dropped copy in one pass
            p = self.kept_p if self.kept_p is not None else self.ex.big_scratch(1, self.probs)
            K.softmax_dropout_fwd(self.probs, self.probs, p, self.p_drop, self.salt, self.ex.seed_tensor, causal_q=causal_q)
        else:
            K.softmax_fwd(self.probs, out=self.probs, causal_q=causal_q)
            if self.p_drop > 0:
                p = self.kept_p if self.kept_p is not None else self.ex.big_scratch(1, self.probs)
                K.dropout(self.probs, self.p_drop, self.salt, out=p, seed_tensor=self.ex.seed_tensor)
        # ctx[b,sq,h,:] = p . v
        self._bg(Sq, vd, Sk, p, Sk, Sq * Sk, H * Sq * Sk, False, self.c_v, self.ldv, vd, Sk * self.ldv, True,
                 self.c_ctx, H * vd, vd, Sq * H * vd)
        self._forward_out()

    def _fused_dropout(self):
        return (self.p_drop, self.salt, self.ex.seed_tensor) if self.p_drop > 0 else None

    def _forward_out(self):
        if self.core16:
            K.cast(self.c_ctx, self.ctx)
        if self.fuse_out is not None:
            self.fuse_out.gemm(self.ctx, self.wo, bias=self.bias_out)
        else:
            K.matmul_nt(self.ctx, self.wo, out=self.out().data.view(-1, self.embed), bias=self.bias_out)

    def backward(self):
        H, kd, vd, Sq, Sk = self.H, self.kd, self.vd, self.Sq, self.Sk
        ex = self.ex
        if self.fuse_out is not None:
            dy = self.fuse_out.gather_grad_gemm(self.wo, self.dctx)
        else:
            dy = self.out().grad.view(-1, self.embed)
        wbuf = self.buf("WEIGHT")
        wg = wbuf.grad.view(-1)
        accw = self.acc["WEIGHT"]
        n_q, n_k, n_v = H * kd * self.dq, H * kd * self.dk, H * vd * self.dv
        g_wo = wg[n_q + n_k + n_v:].view(self.embed, H * vd)
        if self.bias_out_grad:
            K.bias_act_bwd(dy, None, None, self.buf("OUTPUT_BIAS").grad, ex.scratch_f32(), None,
                           accumulate=self.acc.get("OUTPUT_BIAS", False))
        self.ex.wgrad_gemm(dy, self.ctx, g_wo, accw)
        if self.fuse_out is None:
            K.matmul_nn(dy, self.wo, out=self.dctx)
        if self.core16:
            K.cast(self.dctx, self.c_dctx)
        if self.fused:
            n_stat = self.B * H * Sq
            n_stat += (-n_stat) % 4   # keeps the accumulators 16-byte aligned
            scratch = ex.scratch_f32()
            K.attention_bwd(self.c_q, self.c_k, self.c_v, self.c_ctx, self.lse, self.c_dctx, self.c_dq, self.c_dk, self.c_dv,
                            scratch[:n_stat], scratch[n_stat:], B=self.B, H=H, Sq=Sq, Sk=Sk, D=kd, scale=self.alpha,
                            causal=ex.cfg.causal_attention, dropout=self._fused_dropout())
            return self._backward_projections(wg, accw, n_q, n_k, n_v)
        if self.cb:
            self._backward_core_blocked()
            return self._backward_projections(wg, accw, n_q, n_k, n_v)
        p = self.probs
        if self.p_drop > 0 and self.kept_p is not None:
            p = self.kept_p
        elif self.p_drop > 0:  # regenerate the dropped probabilities (mask is a function of the step seed)
            p = ex.big_scratch(1, self.probs)
            K.dropout(self.probs, self.p_drop, self.salt, out=p, seed_tensor=ex.seed_tensor)
        dP = ex.big_scratch(0, self.probs)
        # dP[b,h,sq,sk] = dctx[b,sq,h,:] . v[b,sk,h,:]^T
        self._bg(Sq, Sk, vd, self.c_dctx, H * vd, vd, Sq * H * vd, False, self.c_v, self.ldv, vd, Sk * self.ldv, False,
                 dP, Sk, Sq * Sk, H * Sq * Sk)
        # dV[b,sk,h,:] = p^T . dctx
        self._bg(Sk, vd, Sq, p, Sk, Sq * Sk, H * Sq * Sk, True, self.c_dctx, H * vd, vd, Sq * H * vd, True,
                 self.c_dv, self.ldv, vd, Sk * self.ldv)
        if K.softmax_dropout_supported(self.probs):
            K.softmax_dropout_bwd(dP, self.probs, dP, self.p_drop, self.salt, ex.seed_tensor, scale=self.alpha)
        else:
            if self.p_drop > 0:
                K.dropout(dP, self.p_drop, self.salt, out=dP, seed_tensor=ex.seed_tensor)
            K.softmax_bwd(dP, self.probs, dx=dP, scale=self.alpha)
        # dQ = dS . K ; dK = dS^T . Q
        self._bg(Sq, kd, Sk, dP, Sk, Sq * Sk, H * Sq * Sk, False, self.c_k, self.ldk, kd, Sk * self.ldk, True,
                 self.c_dq, self.ldq, kd, Sq * self.ldq)
        self._bg(Sk, kd, Sq, dP, Sk, Sq * Sk, H * Sq * Sk, True, self.c_q, self.ldq, kd, Sq * self.ldq, True,
                 self.c_dk, self.ldk, kd, Sk * self.ldk)
        self._backward_projections(wg, accw, n_q, n_k, n_v)

    def _backward_projections(self, wg, accw, n_q, n_k, n_v):
        H, kd, vd = self.H, self.kd, self.vd
        ex = self.ex
        if self.core16:
            if self.self_attn:
                K.cast(self.c_dqkv, self.dqkv)
            else:
                K.cast(self.c_dq, self.dq_); K.cast(self.c_dk, self.dk_); K.cast(self.c_dv, self.dv_)
        qb, kb, vb = self.buf("QUERY"), self.buf("KEY"), self.buf("VALUE")
        q2 = self.x("QUERY").view(-1, self.dq)
        if self.self_attn:
            if self.bias_in is not None:
                K.bias_act_bwd(self.dqkv, None, None, self.buf("INPUT_BIAS").grad, ex.scratch_f32(), None,
                               accumulate=self.acc.get("INPUT_BIAS", False))
            K.matmul_tn(self.dqkv, q2, out=wg[:n_q + n_k + n_v].view(self.ldqkv, self.dq), accumulate=accw)
            if self.fuse_in is not None:
                self.fuse_in.grad_gemm(self.dqkv, self.wqkv, self.acc.get("FUSE_IN", False))
            elif qb.requires_grad:
                K.matmul_nn(self.dqkv, self.wqkv, out=qb.grad.view(-1, self.dq), accumulate=self.acc["QUERY"])
        else:
            k2, v2 = self.x("KEY").view(-1, self.dk), self.x("VALUE").view(-1, self.dv)
            K.matmul_tn(self.dq_, q2, out=wg[:n_q].view(H * kd, self.dq), accumulate=accw)
            K.matmul_tn(self.dk_, k2, out=wg[n_q:n_q + n_k].view(H * kd, self.dk), accumulate=accw)
            K.matmul_tn(self.dv_, v2, out=wg[n_q + n_k:n_q + n_k + n_v].view(H * vd, self.dv), accumulate=accw)
            if qb.requires_grad:
                K.matmul_nn(self.dq_, self.wq, out=qb.grad.view(-1, self.dq), accumulate=self.acc["QUERY"])
            if kb.requires_grad:
                K.matmul_nn(self.dk_, self.wk, out=kb.grad.view(-1, self.dk), accumulate=self.acc["KEY"])
            if vb.requires_grad:
                same = self.inputs["KEY"] == self.inputs["VALUE"]
                K.matmul_nn(self.dv_, self.wv, out=vb.grad.view(-1, self.dv), accumulate=self.acc["VALUE"] or same)


# ------------------------------------------------------------------------------------------ normalisation
@register("LAYERNORM")
class LayerNormOp(OpImpl):
    """LayerNorm over the trailing dims; absorbs a preceding residual add when it is the add's only consumer."""
    fused_add: Optional[OpImpl] = None

    def setup(self):
        x = self.x()
        axes = sorted(int(a) for a in self.attrs["axes"])
        nd = x.dim()
        if axes != list(range(nd - len(axes), nd)):
            raise NotImplementedError("layer_norm over non-trailing dims")
        self.cols = 1
        for a in axes:
            self.cols *= x.shape[a]
        self.rows = x.numel() // self.cols
        self.eps = float(self.attrs.get("eps", 1e-5))
        self.gamma = self.x("GAMMA").view(-1) if "GAMMA" in self.inputs else None
        self.beta = self.x("BETA").view(-1) if "BETA" in self.inputs else None
        y = self.alloc_out()
        self.y2d = y.view(self.rows, self.cols)
        self.mean = torch.empty(self.rows, dtype=torch.float32, device=self.ex.device)
        self.rstd = torch.empty_like(self.mean)
        self.ex.need_scratch(4 * K.layernorm_bwd_scratch(self.rows, self.cols) if self.ex.on_gpu else 0)

    def forward(self):
        if self.fused_add is not None:
            add = self.fused_add
            a, b = add.x("LHS_INPUT").view(self.rows, self.cols), add.x("RHS_INPUT").view(self.rows, self.cols)
            K.layernorm_fwd(a, self.gamma, self.beta, self.eps, residual=b, xsum=self.x().view(self.rows, self.cols),
                            out=self.y2d, mean=self.mean, rstd=self.rstd)
        else:
            K.layernorm_fwd(self.x().view(self.rows, self.cols), self.gamma, self.beta, self.eps, out=self.y2d,
                            mean=self.mean, rstd=self.rstd)

    def backward(self):
        dy = self.out().grad.view(self.rows, self.cols)
        x2d = self.x().view(self.rows, self.cols)
        gb = self.buf("GAMMA") if self.gamma is not None else None
        bb = self.buf("BETA") if self.beta is not None else None
        dg = gb.grad.view(-1) if gb is not None and gb.requires_grad else None
        db = bb.grad.view(-1) if bb is not None and bb.requires_grad else None
        accp = self.acc.get("GAMMA", False)
        if self.fused_add is not None:
            add = self.fused_add
            lb, rb = add.buf("LHS_INPUT"), add.buf("RHS_INPUT")
            targets = [(b.grad.view(self.rows, self.cols), add.acc[s]) for s, b in (("LHS_INPUT", lb), ("RHS_INPUT", rb))
                       if b.requires_grad]
            if not targets:
                targets = [(torch.empty_like(x2d), False)]
            dx, a1 = targets[0]
            dx2, a2 = targets[1] if len(targets) > 1 else (None, False)
            if dx2 is not None and dx2.data_ptr() == dx.data_ptr():  # x + x: one buffer receives both
                dx2, a2 = None, False
            K.layernorm_bwd(dy, x2d, self.gamma, self.mean, self.rstd, dx, dg, db, self.ex.scratch_f32(),
                            accumulate_dx=a1, accumulate_params=accp, dx2=dx2, accumulate_dx2=a2)
        else:
            xb = self.buf("INPUT")
            dx = xb.grad.view(self.rows, self.cols) if xb.requires_grad else torch.empty_like(x2d)
            K.layernorm_bwd(dy, x2d, self.gamma, self.mean, self.rstd, dx, dg, db, self.ex.scratch_f32(),
                            accumulate_dx=self.acc.get("INPUT", False) and xb.requires_grad, accumulate_params=accp)


# ------------------------------------------------------------------------------------------ pointwise
_UNARY = {"RELU": "relu", "SIGMOID": "sigmoid", "TANH": "tanh", "ELU": "elu", "GELU": "gelu", "EXP": "exp",
          "RSQRT": "rsqrt", "SIN": "sin", "COS": "cos", "SCALAR_MULTIPLY": "scalar_multiply", "SCALAR_ADD": "scalar_add",
          "SCALAR_SUB": "scalar_sub", "SCALAR_TRUE_DIV": "scalar_truediv", "POW": "pow", "LOG": "log", "SQRT": "sqrt"}


@register(*_UNARY.keys())
class UnaryOp(OpImpl):
    def setup(self):
        self.op = _UNARY[self.type]
        self.scalar = float(self.attrs.get("scalar") or 0.0)
        self.alloc_out()

    def forward(self):
        K.unary_fwd(self.op, self.x(), out=self.out().data, scalar=self.scalar)

    def backward(self):
        b = self.buf("INPUT")
        if b.requires_grad:
            K.unary_bwd(self.op, self.x(), self.out().data, self.out().grad.view_as(self.x()), dx=b.grad.view_as(self.x()),
                        scalar=self.scalar, accumulate=self.acc["INPUT"])


_BINARY = {"EW_ADD": "add", "EW_SUB": "sub", "EW_MUL": "mul", "EW_DIV": "div", "EW_MAX": "max", "EW_MIN": "min"}


@register(*_BINARY.keys())
class BinaryOp(OpImpl):
    fused_into_ln = False
    _bfull = _da = _dbfull = None

    def setup(self):
        self.op = _BINARY[self.type]
        self.alloc_out()

    def forward(self):
        if self.fused_into_ln:
            return  # the consuming LayerNorm writes this sum
        K.binary_fwd(self.op, self.x("LHS_INPUT"), self.x("RHS_INPUT"), out=self.out().data)

    def backward(self):
        if self.fused_into_ln:
            return
        lb, rb = self.buf("LHS_INPUT"), self.buf("RHS_INPUT")
        dy = self.out().grad
        a, b = lb.data, rb.data
        if a.shape != b.shape and self.op in ("add", "sub"):
            if lb.requires_grad:
                self.ex.write_grad(lb, dy, self.acc["LHS_INPUT"])
            if rb.requires_grad:
                red = dy.float().reshape(-1, b.numel()).sum(0).to(dy.dtype)
                if self.op == "sub":
                    red = -red
                self.ex.write_grad(rb, red.view_as(b), self.acc["RHS_INPUT"])
            return
        if a.shape != b.shape:
            # mul / div / max / min with the right operand repeated along the leading dims: the element-wise
            # gradients are taken against the materialised repeat, then summed over the repeats
            reps = a.numel() // b.numel()
            if self._bfull is None:
                self._bfull = torch.empty_like(a)
                self._da = torch.empty_like(a)
                self._dbfull = torch.empty_like(a)
            K.permute(b.reshape(1, -1).expand(reps, b.numel()), (0, 1), out=self._bfull.view(reps, -1))
            K.binary_bwd(self.op, a, self._bfull, dy.view_as(a), self._da, self._dbfull)
            if lb.requires_grad:
                self.ex.write_grad(lb, self._da, self.acc["LHS_INPUT"])
            if rb.requires_grad:
                red = torch.empty_like(b) if self.acc["RHS_INPUT"] else rb.grad.view_as(b)
                K.reduce(self._dbfull.view(-1), red.view(-1), 1, reps, b.numel(), "sum")
                if self.acc["RHS_INPUT"]:
                    self.ex.write_grad(rb, red, True)
            return
        if self.op == "add":
            if lb.requires_grad:
                self.ex.write_grad(lb, dy, self.acc["LHS_INPUT"])
            if rb.requires_grad:
                self.ex.write_grad(rb, dy, self.acc["RHS_INPUT"])
            return
        da = lb.grad.view_as(a) if lb.requires_grad else None
        db = rb.grad.view_as(b) if rb.requires_grad else None
        acc = self.acc.get("LHS_INPUT", False) or self.acc.get("RHS_INPUT", False)
        if acc and da is not None and db is not None and self.acc["LHS_INPUT"] != self.acc["RHS_INPUT"]:
            ta = torch.empty_like(a)
            tb = torch.empty_like(b)
            K.binary_bwd(self.op, a, b, dy, ta, tb)
            self.ex.write_grad(lb, ta, self.acc["LHS_INPUT"])
            self.ex.write_grad(rb, tb, self.acc["RHS_INPUT"])
        else:
            K.binary_bwd(self.op, a, b, dy, da, db, accumulate=acc)


@register("DROPOUT")
class DropoutOp(OpImpl):
    fused_into = None  # the Linear whose GEMM epilogue applies this dropout (then this operator is an alias)
    bwd_folded = None  # the Linear whose backward also undoes this dropout (forward stays a kernel of its own)

    def setup(self):
        self.p = float(self.attrs["rate"]) if self.ex.cfg.training else 0.0
        self.salt = self.ex.next_salt() + int(self.attrs.get("seed", 0))
        if self.fused_into is not None:
            if self.p > 0:
                self.out().data = self.x()
                self.ex.alias(self.nid, self.inputs["INPUT"])
                return
            self.fused_into.fused_dropout = None
            self.fused_into = None
        if self.bwd_folded is not None and not self.p > 0:
            self.bwd_folded.bwd_dropout = None
            self.bwd_folded = None
        if self.p > 0:
            self.alloc_out()
        else:
            self.out().data = self.x()

    def forward(self):
        if self.p > 0 and self.fused_into is None:
            K.dropout(self.x(), self.p, self.salt, out=self.out().data, seed_tensor=self.ex.seed_tensor)

    def backward(self):
        b = self.buf("INPUT")
        if not b.requires_grad or self.fused_into is not None or self.bwd_folded is not None:
            return
        dy = self.out().grad
        if self.p > 0:
            if self.acc["INPUT"]:
                K.dropout(dy, self.p, self.salt, residual=b.grad.view_as(dy), out=b.grad.view_as(dy),
                          seed_tensor=self.ex.seed_tensor)
            else:
                K.dropout(dy, self.p, self.salt, out=b.grad.view_as(dy), seed_tensor=self.ex.seed_tensor)
        else:
            self.ex.write_grad(b, dy, self.acc["INPUT"])


@register("CAST")
class CastOp(OpImpl):
    def setup(self):
        src = self.x()
        want = self.ex.torch_dtype(self.attrs["dtype"])
        if want == src.dtype:
            self.out().data = src
            self.alias = True
        else:
            self.alloc_out(dtype=want)
            self.alias = False

    def forward(self):
        if not self.alias:
            K.cast(self.x(), self.out().data)

    def backward(self):
        b = self.buf("INPUT")
        if not b.requires_grad:
            return
        if self.alias:
            self.ex.write_grad(b, self.out().grad, self.acc["INPUT"])
        else:
            K.cast(self.out().grad.view_as(self.x()), b.grad.view_as(self.x()), accumulate=self.acc["INPUT"])


@register("EMBEDDING")
class EmbeddingOp(OpImpl):
    def setup(self):
        self.aggr = "avg" if self.attrs.get("aggr") == "AVG" else "sum"
        self.alloc_out()
        self.table = self.x("WEIGHT")
        self.sparse = self.inputs["WEIGHT"][0] in self.ex.sparse_tables

    def forward(self):
        K.embedding_fwd(self.x(), self.table, self.out().data, aggr=self.aggr)

    def backward(self):
        wb = self.buf("WEIGHT")
        if self.sparse:
            # table[idx] -= lr * d(out): the update itself, no table-sized gradient exists
            K.embedding_sgd(self.x(), self.out().grad.view_as(self.out().data), self.table, self.ex.cfg.optimizer.lr, aggr=self.aggr)
        elif wb.requires_grad:
            if not self.acc["WEIGHT"]:
                wb.grad.zero_()
            K.embedding_bwd(self.x(), self.out().grad.view_as(self.out().data), wb.grad, aggr=self.aggr)


class EmbeddingStackOp(OpImpl):
    """Takes the place of a Concat(axis 1) whose inputs are all single-index lookups into sparsely updated tables
    (through their Reshapes): one kernel gathers from all tables straight into the stacked [batch, tables, dim]
    tensor, one kernel applies all tables' sparse SGD updates from the stack's gradient.  The lookups, Reshapes
    and the Concat's copies disappear (recommendation models: 4 launches and 2 copies per table per step)."""
    members = None  # [(weight node, index value)] in stack order

    def setup(self):
        ex = self.ex
        tables = [ex.sparse_tables[w] for w, _ in self.members]
        self.table_ptrs = torch.tensor([t.data_ptr() for t in tables], dtype=torch.int64, device=ex.device)
        self.entries = torch.tensor([t.shape[0] for t in tables], dtype=torch.int64, device=ex.device)
        y = self.alloc_out()
        idx0 = ex.values[self.members[0][1]].data
        self.idx = torch.empty(y.shape[0], len(tables), dtype=idx0.dtype, device=ex.device)
        for v in self.inputs.values():
            ex.values[v].requires_grad = False  # the per-table outputs are never materialised

    def forward(self):
        torch.cat([self.ex.values[v].data.view(-1, 1) for _, v in self.members], dim=1, out=self.idx)
        K.embedding_stack_fwd(self.table_ptrs, self.entries, self.idx, self.out().data)

    def backward(self):
        K.embedding_stack_sgd(self.table_ptrs, self.entries, self.idx, self.out().grad.view_as(self.out().data), self.ex.cfg.optimizer.lr)


@register("SOFTMAX")
class SoftmaxOp(OpImpl):
    fused_loss = False  # set when this softmax feeds the loss: probabilities are then not materialised

    def setup(self):
        x = self.x()
        d = int(self.attrs.get("dim", -1)) % x.dim()
        if d != x.dim() - 1:
            raise NotImplementedError("softmax over a non-trailing dim")
        if self.fused_loss:
            self.out().data = None
        else:
            self.alloc_out()

    def forward(self):
        if not self.fused_loss:
            K.softmax_fwd(self.x(), out=self.out().data)

    def probabilities(self):
        if self.fused_loss:
            return K.softmax_fwd(self.x())
        return self.out().data

    def backward(self):
        if self.fused_loss:
            return  # the loss wrote d(logits) directly
        b = self.buf("INPUT")
        if b.requires_grad:
            if self.acc["INPUT"]:
                t = K.softmax_bwd(self.out().grad.view_as(self.x()), self.out().data)
                self.ex.write_grad(b, t, True)
            else:
                K.softmax_bwd(self.out().grad.view_as(self.x()), self.out().data, dx=b.grad.view_as(self.x()))


# ------------------------------------------------------------------------------------------ shape ops
@register("FLAT", "RESHAPE")
class ReshapeOp(OpImpl):
    """A view of the input.  A channels-last 4-D input (output of a convolution stack) with more than one spatial
    position is first brought back to the logical NCHW order, since the flattened feature order is part of the
    model's meaning (it indexes the rows of the following Linear's weight)."""
    layout_aware = True

    def setup(self):
        sh = dict(self.outputs)["OUTPUT"]
        self.permute = None
        src = self.inputs["INPUT"]
        if self.ex.is_nhwc(src):
            n, c, h, w = [int(v) for v in self.ex.graph.shape(src).piece_sizes]
            if h * w > 1 and c > 1:
                self.permute = (n, c, h, w)
                self.alloc_out()
                return
        self.out().data = self.x().view(list(sh.piece_sizes))

    def forward(self):
        if self.permute:
            n, c, h, w = self.permute
            K.permute(self.x().view(n, h, w, c), (0, 3, 1, 2), out=self.out().data.view(n, c, h, w))

    def backward(self):
        b = self.buf("INPUT")
        if not b.requires_grad:
            return
        if self.permute:
            n, c, h, w = self.permute
            K.permute(self.out().grad.view(n, c, h, w), (0, 2, 3, 1), out=b.grad.view(n, h, w, c), accumulate=self.acc["INPUT"])
        else:
            self.ex.write_grad(b, self.out().grad, self.acc["INPUT"])


_LAYOUT_TRANSPARENT = set(_UNARY) | set(_BINARY) | {"DROPOUT", "CAST", "NOOP", "IDENTITY"}


# ------------------------------------------------------------------------------------------ the executable
class Executable:
    """A computation graph lowered onto one device (one rank's shard of a parallel graph)."""

    def __init__(self, graph, cfg: Optional[ExecConfig] = None, dist=None):
        self.graph = graph
        self.cfg = cfg or ExecConfig()
        self.dist = dist
        self.device = torch.device(self.cfg.device)
        self.on_gpu = self.device.type == "cuda"
        if self.on_gpu:
            K.lib()  # fail loudly if the kernel library is missing
        # every long-lived device buffer of the plan (parameter / gradient / optimizer arenas, activations, scratch) comes
        # from the handle's allocator, which counts bytes (the reference's per-device Allocator behind a tracking wrapper,
        # lib/kernels/include/kernels/allocation.h, lib/local-execution/.../tracked_allocator.h); symmetric peer-memory
        # arenas of the multi-GPU executor are the exception: they come from the peer-memory context.  The handle also
        # owns the one workspace the operators' scratch needs are folded into.
        from .device_handle import create_local_handle_for_device, create_multi_gpu_handle
        if dist is not None and self.on_gpu:
            self.handle = create_multi_gpu_handle(dist)
        else:
            self.handle = create_local_handle_for_device(self.device)
        self.allocator = self.handle.allocator
        self.values: Dict[Value, _Buf] = {}
        self.layout: Dict[Value, str] = {}
        self.ops: Dict[int, OpImpl] = {}
        self.order: List[int] = list(graph.topological_order())
        self._big_scratch_bytes = 0
        self._big_scratch_slots = 0
        self._salt = 0
        self.step_count = 0
        self.seed_tensor = torch.zeros(1, dtype=torch.int64, device=self.device) if self.on_gpu else None
        self.alpha_tensor = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.layer_ms: Dict[int, float] = {}
        self._graph = None
        self._build()

    # ---- dtype policy: FLOAT tensors run in the compute dtype
    def torch_dtype(self, name: str):
        if name == "FLOAT" and self.cfg.compute_dtype == "bf16":
            return torch.bfloat16
        if name == "HALF" and self.cfg.compute_dtype == "bf16":
            return torch.bfloat16
        return _TORCH_DT[name]

    def head_shards(self, op) -> int:
        """How many ways the heads of an attention operator are sharded on this rank (1 on a single device)."""
        return getattr(self, "_head_shards", {}).get(op.nid, 1)

    def use_bias(self, op, slot: str) -> bool:
        """False when `slot` is the bias of an operator that produces partial sums and this rank is not the one
        that contributes it (a row-parallel Linear adds its bias once, not once per shard)."""
        return True

    def bias_grad_without_use(self, op, slot: str) -> bool:
        """True when this rank keeps a copy of a bias it does not add in forward (see use_bias) and still has to compute
        that bias's gradient itself, because the gradient reduction does not reach the rank that adds it."""
        return False

    # ---- physical layout: 4-D activations produced by convolution-stack operators are kept channels-last
    def is_nhwc(self, v: Value) -> bool:
        return self.layout.get(self.canon(v)) == "NHWC"

    def mark_nhwc(self, v: Value):
        self.layout[v] = "NHWC"

    def _propagate_layout(self, op: OpImpl):
        ins = [v for _, v in op.inputs.items() if len(self.graph.shape(v).piece_sizes) == 4]
        flags = [self.is_nhwc(v) for v in ins]
        if not any(flags) or getattr(op, "layout_aware", False):
            return
        if op.type in _LAYOUT_TRANSPARENT and all(flags):
            for s, _ in op.outputs:
                self.mark_nhwc((op.nid, s))
            return
        raise NotImplementedError(f"operator {op.type} ({op.node['name']}) got a channels-last input it cannot consume")

    def next_salt(self) -> int:
        self._salt += 1
        return self._salt * 0x1000003

    def need_scratch(self, nbytes: int):
        self.handle.reserve_workspace(nbytes)

    @property
    def _scratch(self) -> torch.Tensor:
        return self.handle.workspace

    def need_big_scratch(self, nbytes: int, slots: int):
        self._big_scratch_bytes = max(self._big_scratch_bytes, int(nbytes))
        self._big_scratch_slots = max(self._big_scratch_slots, slots)

    def scratch_f32(self):
        return self._scratch

    def big_scratch(self, slot: int, like: torch.Tensor):
        n = like.numel() * like.element_size()
        return self._big[slot][:n].view(like.dtype).view(like.shape)

    # A small layer under a large batch: its weight gradient has a handful of output tiles and a reduction over
    # thousands of rows, so a direct GEMM keeps a few CTAs streaming all rows while the other SMs idle.  Computed into
    # an fp32 scratch instead, the GEMM splits the reduction over all SMs; a cast then adds it into the bf16 gradient.
    @staticmethod
    def wgrad_splits(rows: int, n_out: int, k_in: int, dtype) -> bool:
        tiles = ((n_out + 127) // 128) * ((k_in + 127) // 128)
        return dtype == torch.bfloat16 and tiles * 2 <= 148 and rows >= 1024

    def wgrad_gemm(self, dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor, accumulate: bool):
        """out[n_out, k_in] (+)= dy[rows, n_out]^T . x[rows, k_in]"""
        if self.wgrad_splits(dy.shape[0], out.shape[0], out.shape[1], out.dtype) and self._scratch.numel() >= out.numel():
            part = self._scratch[:out.numel()].view(out.shape)
            K.matmul_tn(dy, x, out=part)
            K.cast(part, out, accumulate=accumulate)
        else:
            K.matmul_tn(dy, x, out=out, accumulate=accumulate)

    def write_grad(self, buf: _Buf, g: torch.Tensor, accumulate: bool):
        tgt = buf.grad.view(-1)
        src = g.reshape(-1)
        if tgt.data_ptr() == src.data_ptr():
            return
        if accumulate:
            K.axpby(src, tgt, 1.0, 1.0)
        else:
            tgt.copy_(src)

    # ---- plan construction
    def _build(self):
        g = self.graph
        nodes = {n["id"]: n for n in g.nodes()}
        self.nodes = nodes
        # 1. which values need gradients
        req: Dict[Value, bool] = {}
        for nid in self.order:
            n = nodes[nid]
            if n["type"] == "WEIGHT":
                r = self.cfg.training
            elif n["type"] == "INPUT":
                r = False
            else:
                r = any(req[tuple(v)] for _, v in n["inputs"])
            for s, sh, _ in n["outputs"]:
                req[(nid, s)] = r and sh.dtype in ("FLOAT", "HALF", "DOUBLE", "BFLOAT16")
                self.values[(nid, s)] = _Buf(None, req[(nid, s)])
        # 2. parameters: flat arenas
        self._build_params()
        # 3. operator objects + fusion decisions
        for nid in self.order:
            n = nodes[nid]
            cls = _REGISTRY.get(n["type"])
            if cls is None:
                raise NotImplementedError(f"no kernel implementation registered for operator {n['type']}")
            self.ops[nid] = cls(self, nid, n)
        self._fuse()
        for nid in self.order:
            op = self.ops[nid]
            op.setup()
            self._propagate_layout(op)
        # 4. loss
        self._build_loss()
        # 5. gradient buffers + accumulate flags
        if self.cfg.training:
            self._plan_gradients()
        self.handle.materialize_workspace()
        self._big = [self.allocator.allocate([max(self._big_scratch_bytes, 1)], torch.uint8) for _ in range(max(self._big_scratch_slots, 1))]

    def sparse_weight_nodes(self) -> List[int]:
        """Weights that are the table of exactly one Embedding and can take the sparse SGD update."""
        o = self.cfg.optimizer
        if not (self.cfg.training and self.cfg.sparse_embedding_update and o.kind == "sgd" and o.momentum == 0
                and o.weight_decay == 0):
            return []
        out = []
        for nid in self.order:
            if self.nodes[nid]["type"] != "WEIGHT":
                continue
            cons = self.graph.consumers((nid, "OUTPUT"))
            if len(cons) == 1 and cons[0][1] == "WEIGHT" and self.nodes[cons[0][0]]["type"] == "EMBEDDING" \
                    and self.sparse_embedding_allowed(cons[0][0]):
                out.append(nid)
        return out

    def sparse_embedding_allowed(self, embedding_nid: int) -> bool:
        return True

    def owns_sparse_table(self, nid: int) -> bool:
        """Does this rank hold the sparsely updated table `nid`?  (Model-parallel tables live on one rank each.)"""
        return True

    def _build_params(self):
        nodes, dev = self.nodes, self.device
        sparse = set(self.sparse_weight_nodes())
        self.sparse_tables: Dict[int, Optional[torch.Tensor]] = {}
        self.param_nodes = self.order_params([nid for nid in self.order if nodes[nid]["type"] == "WEIGHT" and nid not in sparse])
        ordinal = {nid: i for i, nid in enumerate(nid for nid in self.order if nodes[nid]["type"] == "WEIGHT")}
        offs, total = {}, 0
        for nid in self.param_nodes:
            sh = nodes[nid]["outputs"][0][1]
            n = 1
            for s in self.local_weight_shape(nid):
                n *= s
            offs[nid] = (total, n)
            total += (n + 63) // 64 * 64  # keep every parameter 256-byte aligned in the arena
        self.param_offsets = offs
        self.num_params = total
        mixed = self.cfg.compute_dtype == "bf16"
        self.master = self.allocator.allocate([max(total, 1)], torch.float32).zero_()
        self.shadow = self.alloc_shadow_arena(max(total, 1)) if mixed else None
        if self.cfg.training:
            self.grads = self.alloc_grad_arena(max(total, 1), torch.bfloat16 if mixed else torch.float32)
            self.opt_m = self.allocator.allocate([max(total, 1)], torch.float32).zero_() \
                if (self.cfg.optimizer.kind == "adam" or self.cfg.optimizer.momentum > 0) else None
            self.opt_v = self.allocator.allocate([max(total, 1)], torch.float32).zero_() if self.cfg.optimizer.kind == "adam" else None
        for i, nid in enumerate(self.param_nodes):
            o, n = offs[nid]
            shape = self.local_weight_shape(nid)
            full = initialize(list(nodes[nid]["outputs"][0][1].sizes), nodes[nid]["attrs"].get("initializer"),
                              base_seed=self.cfg.seed, ordinal=ordinal[nid])
            self.master[o:o + n].copy_(self.shard_weight(nid, full).reshape(-1))
            b = self.values[(nid, "OUTPUT")]
            b.data = (self.shadow if mixed else self.master)[o:o + n].view(shape)
            if self.cfg.training:
                b.grad = self.grads[o:o + n].view(shape)
        if mixed:
            self.shadow.copy_(self.master)
        for nid in sorted(sparse):
            t = None
            if self.owns_sparse_table(nid):
                full = initialize(list(nodes[nid]["outputs"][0][1].sizes), nodes[nid]["attrs"].get("initializer"),
                                  base_seed=self.cfg.seed, ordinal=ordinal[nid])
                t = full.to(device=dev, dtype=torch.float32).contiguous()
            self.sparse_tables[nid] = t
            b = self.values[(nid, "OUTPUT")]
            b.data, b.requires_grad = t, False

    # value aliasing: an operator that forwards its input unchanged shares data *and* gradient buffers with it
    def alias(self, nid: int, src: Value, slot: str = "OUTPUT"):
        if not hasattr(self, "alias_of"):
            self.alias_of = {}
        self.alias_of[(nid, slot)] = src

    def canon(self, v: Value) -> Value:
        a = getattr(self, "alias_of", None)
        if a:
            while v in a:
                v = a[v]
        return v

    # hooks the distributed executable overrides
    def order_params(self, param_nodes):
        return param_nodes

    def alloc_grad_arena(self, numel, dtype):
        return self.allocator.allocate([numel], dtype).zero_()

    def memory_report(self) -> dict:
        """Bytes the plan's buffers hold, as counted by the executor's allocator."""
        a = self.allocator
        return {"current_bytes": a.current_bytes, "peak_bytes": a.peak_bytes, "total_allocated_bytes": a.total_allocated_bytes}

    def alloc_shadow_arena(self, numel):
        """The bf16 copy of the weights that the kernels read (the fp32 master arena is only touched by the update)."""
        return self.allocator.allocate([numel], torch.bfloat16).zero_()

    def resolve_loss_value(self, v: Value) -> Value:
        """The value the loss is computed on; the distributed executable steps back over a trailing Combine."""
        return v

    def local_label_rows(self, labels: torch.Tensor, rows: int) -> torch.Tensor:
        return labels

    # single-device: a weight's local shape is its full shape
    def local_weight_shape(self, nid):
        return list(self.nodes[nid]["outputs"][0][1].sizes)

    def shard_weight(self, nid, full):
        return full

    def embedding_stack_members(self, concat_nid: int):
        """If node `concat_nid` is a Concat(axis 1) of [batch, 1, dim] Reshapes of single-index lookups into sparsely
        updated tables this rank holds: ([(weight node, index value)], [nodes made redundant]); else None."""
        g, nodes = self.graph, self.nodes
        c = nodes[concat_nid]
        sh = c["outputs"][0][1]
        if c["type"] != "CONCAT" or len(sh.sizes) != 3 or int(c["attrs"]["axis"]) % 3 != 1 or sh.total_degree != 1:
            return None
        members, redundant = [], []
        for _, v in sorted(c["inputs"], key=lambda sv: int(sv[0].split("_")[-1])):
            v = tuple(v)
            p = nodes[v[0]]
            if p["type"] in ("RESHAPE", "FLAT") and len(g.consumers(v)) == 1:
                redundant.append(p["id"])
                v = tuple(p["inputs"][0][1])
                p = nodes[v[0]]
            if p["type"] != "EMBEDDING" or len(g.consumers(v)) != 1:
                return None
            ins = {s: tuple(x) for s, x in p["inputs"]}
            w, i = ins["WEIGHT"], ins["INPUT"]
            ish = g.shape(i)
            bag = 1
            for d in ish.sizes[1:]:
                bag *= d
            if self.sparse_tables.get(w[0]) is None or bag != 1 or ish.sizes[0] != sh.sizes[0] or ish.total_degree != 1 \
                    or g.shape(w).sizes[1] != sh.sizes[2]:
                return None
            redundant.append(p["id"])
            members.append((w[0], i))
        if len(members) != sh.sizes[1] or len({g.shape(i).dtype for _, i in members}) != 1:
            return None
        return members, redundant

    def _fuse(self):
        g = self.graph
        for nid in self.order:
            found = self.embedding_stack_members(nid) if self.sparse_tables else None
            if found is not None:
                members, redundant = found
                for r in redundant:
                    self.ops[r] = SkippedOp(self, r, self.nodes[r])
                op = EmbeddingStackOp(self, nid, self.nodes[nid])
                op.members = members
                self.ops[nid] = op
        for nid in self.order:
            op = self.ops[nid]
            if isinstance(op, LayerNormOp):
                src = op.inputs["INPUT"]
                prod = self.ops[src[0]]
                if (isinstance(prod, BinaryOp) and prod.type == "EW_ADD" and len(g.consumers(src)) == 1
                        and self._same_shape(prod.inputs["LHS_INPUT"], prod.inputs["RHS_INPUT"])):
                    op.fused_add = prod
                    prod.fused_into_ln = True
            # Linear -> Dropout: the GEMM epilogue applies the mask (bf16, 16-byte rows; not for a row-parallel GEMM
            # whose output is still a partial sum)
            if (isinstance(op, DropoutOp) and not self.cfg.fuse_dropout and self.cfg.fold_dropout_backward and self.on_gpu and self.cfg.training
                    and self.cfg.compute_dtype == "bf16" and float(op.attrs.get("rate", 0)) > 0):
                # backward half only: Linear -> Dropout with the dropout's gradient masking folded into the Linear's
                # bias/activation backward kernel
                src = op.inputs["INPUT"]
                prod = self.ops[src[0]]
                cols = int(g.shape(src).piece_sizes[-1])
                if (isinstance(prod, LinearOp) and prod.bwd_dropout is None and len(g.consumers(src)) == 1 and cols % 8 == 0
                        and g.shape(src).sum_degree == 1 and g.shape(src).dtype in ("FLOAT", "HALF", "BFLOAT16")):
                    prod.bwd_dropout = op
                    op.bwd_folded = prod
            if (isinstance(op, DropoutOp) and self.cfg.fuse_dropout and self.on_gpu and self.cfg.training
                    and self.cfg.compute_dtype == "bf16" and float(op.attrs.get("rate", 0)) > 0):
                src = op.inputs["INPUT"]
                prod = self.ops[src[0]]
                cols = int(g.shape(src).piece_sizes[-1])
                k_in = int(g.shape(prod.inputs["INPUT"]).piece_sizes[-1]) if isinstance(prod, LinearOp) else 1
                if (isinstance(prod, LinearOp) and prod.fused_dropout is None and len(g.consumers(src)) == 1 and cols % 8 == 0
                        and k_in % 8 == 0 and g.shape(src).sum_degree == 1 and g.shape(src).dtype in ("FLOAT", "HALF", "BFLOAT16")):
                    prod.fused_dropout = op
                    op.fused_into = prod
        # a trailing softmax that only feeds the loss is fused into it
        self.loss_value: Optional[Value] = None
        if self.cfg.loss:
            sinks = [self.resolve_loss_value(tuple(v)) for v in g.sink_values()
                     if self.nodes[v[0]]["type"] not in ("WEIGHT", "INPUT")]
            named = [v for v in sinks if self.nodes[v[0]]["name"] == "out_prob"]
            self.loss_value = (named or sinks)[-1] if sinks else None
            for nid in getattr(self, "_skip_nodes", ()):  # trailing parallel ops behind the loss input
                self.ops[nid] = SkippedOp(self, nid, self.nodes[nid])
            if self.loss_value is not None:
                op = self.ops[self.loss_value[0]]
                if isinstance(op, SoftmaxOp) and self.cfg.loss == "sparse_categorical_crossentropy":
                    op.fused_loss = True

    def _same_shape(self, a: Value, b: Value) -> bool:
        return list(self.graph.shape(a).piece_sizes) == list(self.graph.shape(b).piece_sizes)

    def _build_loss(self):
        self.loss_rows = None
        self.labels = None
        if self.loss_value is None:
            return
        op = self.ops[self.loss_value[0]]
        sh = self.graph.shape(self.loss_value)
        sizes = list(sh.piece_sizes)
        cols = sizes[-1]
        rows = 1
        for s in sizes[:-1]:
            rows *= s
        self.loss_shape = (rows, cols)
        self.loss_rows = torch.zeros(rows, dtype=torch.float32, device=self.device)
        if self.cfg.loss == "sparse_categorical_crossentropy":
            self.labels = torch.zeros(rows, dtype=torch.int32, device=self.device)
        else:
            self.labels = torch.zeros(rows, cols, dtype=self.torch_dtype(sh.dtype), device=self.device)
        self.loss_scale = 1.0 / self.global_loss_rows(rows, sh)

    def global_loss_rows(self, local_rows: int, shape) -> int:
        return local_rows

    def _plan_gradients(self):
        pool = _GradPool(self.device)
        written: Dict[Value, bool] = {}
        # the loss seeds the gradient of its input
        seeds: List[Value] = []
        if self.loss_value is not None:
            op = self.ops[self.loss_value[0]]
            tgt = op.inputs["INPUT"] if (isinstance(op, SoftmaxOp) and op.fused_loss) else self.loss_value
            seeds.append(tgt)
        live: Dict[Value, torch.Tensor] = {}
        canon = self.canon
        hold_until: Dict[Value, int] = {}
        held_by: Dict[int, List[Value]] = {}
        for nid, op in self.ops.items():
            for v in op.extra_grad_sources():
                hold_until[canon(v)] = nid
                held_by.setdefault(nid, []).append(canon(v))

        def ensure(v: Value):
            """Give v a gradient buffer; aliases share the buffer of the value they alias."""
            c = canon(v)
            b = self.values[c]
            if b.grad is None and b.requires_grad:
                ref = b.data if b.data is not None else None
                sizes = list(self.graph.shape(c).piece_sizes)
                n = 1
                for s in sizes:
                    n *= s
                dt = ref.dtype if ref is not None else self.torch_dtype(self.graph.shape(c).dtype)
                flat = pool.take(n, dt)
                b.grad = flat.view(sizes)
                live[c] = flat
            if c != v and b.grad is not None:
                self.values[v].grad = b.grad.view(list(self.graph.shape(v).piece_sizes))

        for v in seeds:
            ensure(v)
            written[canon(v)] = True
        for nid in reversed(self.order):
            op = self.ops[nid]
            if op.type in ("WEIGHT", "INPUT"):
                continue
            # an op whose outputs received no gradient has nothing to propagate
            outs = [(nid, s) for s, _ in op.outputs]
            op.has_grad = any(written.get(canon(o), False) for o in outs)
            # per output: does any consumer write its gradient?  (an unused output of a multi-output operator has a
            # gradient buffer that nobody fills)
            op.grad_written = {o[1]: written.get(canon(o), False) for o in outs}
            if isinstance(op, BinaryOp) and op.fused_into_ln:
                op.has_grad = False
            if isinstance(op, SkippedOp):
                op.has_grad = False
            if op.has_grad or (isinstance(op, SoftmaxOp) and op.fused_loss):
                for o in outs:
                    if self.values[o].requires_grad:
                        ensure(o)
                # an operator with a fused collective writes the gradient of a value it does not consume itself
                targets = list(op.inputs.items()) + list(op.extra_grad_targets())
                if isinstance(op, LayerNormOp) and op.fused_add is not None:
                    # the LayerNorm writes straight into the add's operands
                    add = op.fused_add
                    for s, v in add.inputs.items():
                        if self.values[v].requires_grad:
                            ensure(v)
                            add.acc[s] = written.get(canon(v), False)
                            written[canon(v)] = True
                    targets = [(s, v) for s, v in targets if s != "INPUT"]
                if isinstance(op, SoftmaxOp) and op.fused_loss:
                    targets = []
                seen_here = set()
                for s, v in targets:
                    if not self.values[v].requires_grad:
                        continue
                    ensure(v)
                    op.acc[s] = written.get(canon(v), False) or (canon(v) in seen_here)
                    seen_here.add(canon(v))
                for c in seen_here:
                    written[c] = True
            # outputs of this node are dead once its backward ran (aliases are released with their source), unless
            # an earlier operator reads them in its own backward (fused collectives): then they live until that one
            for o in outs:
                if o in live and o not in hold_until:
                    pool.give(live.pop(o))
            for o in held_by.get(nid, ()):
                if o in live:
                    pool.give(live.pop(o))
        self.grad_pool_bytes = pool.total_bytes

    # ---- execution
    def set_inputs(self, inputs: Dict[str, torch.Tensor], labels: Optional[torch.Tensor] = None):
        for nid in self.order:
            n = self.nodes[nid]
            if n["type"] != "INPUT":
                continue
            name = n["name"] or f"input{nid}"
            if name in inputs:
                dst = self.values[(nid, "OUTPUT")].data
                src = inputs[name]
                dst.copy_(src.reshape(dst.shape), non_blocking=True)
        if labels is not None and self.labels is not None:
            labels = self.local_label_rows(labels, self.labels.shape[0])
            self.labels.copy_(labels.reshape(self.labels.shape), non_blocking=True)

    def forward(self):
        if self.cfg.profile_layers:
            return self._forward_profiled()
        for nid in self.order:
            self.ops[nid].forward()

    def _forward_profiled(self):
        for nid in self.order:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            self.ops[nid].forward()
            e1.record()
            e1.synchronize()
            self.layer_ms[nid] = e0.elapsed_time(e1)

    def compute_loss(self):
        """Loss forward (per-row values) and, in training, the gradient of the loss input."""
        if self.loss_value is None:
            return None
        op = self.ops[self.loss_value[0]]
        rows, cols = self.loss_shape
        kind = self.cfg.loss
        if isinstance(op, SoftmaxOp) and op.fused_loss:
            logits = op.x().view(rows, cols)
            dl = self.values[op.inputs["INPUT"]].grad.view(rows, cols) if self.cfg.training else None
            K.softmax_ce(logits, self.labels, self.loss_rows, dlogits=dl, grad_scale=self.loss_scale)
        else:
            pred = self.values[self.loss_value].data.view(rows, cols)
            K.loss_fwd(kind, pred, self.labels, self.loss_rows)
            if self.cfg.training:
                K.loss_bwd(kind, pred, self.labels, self.values[self.loss_value].grad.view(rows, cols), self.loss_scale)
        return self.loss_rows

    def backward(self):
        for nid in reversed(self.order):
            op = self.ops[nid]
            if getattr(op, "has_grad", False):
                op.backward()

    def step_plan(self):
        """The training step as the list of (task, node) this executor runs, in its stream order: FWD of every operator,
        LOSS on the loss value, BWD of the operators that have a backward in reverse order, UPD of every parameter.
        `runtime.lowering.check_plan` compares this with the lowered step (pass expansion, loss and update insertion)
        and its reader / writer dependencies."""
        plan = [("FWD", nid) for nid in self.order]
        if self.loss_value is not None:
            plan.append(("LOSS", self.loss_value[0]))
        if self.cfg.training:
            plan += [("BWD", nid) for nid in reversed(self.order) if getattr(self.ops[nid], "has_grad", False)]
            plan += [("UPD", nid) for nid in self.param_nodes]
            plan += [("UPD", nid) for nid, t in self.sparse_tables.items() if t is not None and nid not in self.param_nodes]
        return plan

    def profile_step(self, update: bool = False):
        """Run one eager forward + backward with CUDA events around every operator's forward and backward.

        Returns ``{"by_type": {(op type, phase): ms}, "by_node": {(node id, phase): ms}, "total_ms": ms}``.
        This is the per-layer timing the reference collects through its ``profile(...)`` wrapper
        (lib/task-spec/include/task-spec/profiling.h:11-24) and the source of measured operator costs.

        Profiling is an observation: weights, optimizer state and the step counter are left as they were unless
        `update=True` asks for the optimizer step to be run (and timed) as well.  Activations and gradient
        buffers are overwritten, as by any step.  A multi-rank executable refuses: its gradient reduction and
        fused collectives need every rank inside the same step."""
        if self.dist is not None and self.dist.world_size > 1:
            raise RuntimeError("profile_step() runs one rank's operators in isolation; with more than one rank the "
                               "collectives inside the step would wait for peers that are not in it")
        self._pre_step()
        recs = []

        def timed(key, fn):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            recs.append((key, e0, e1))

        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for nid in self.order:
            timed((nid, "fwd"), self.ops[nid].forward)
        timed((-1, "loss"), self.compute_loss)
        for nid in reversed(self.order):
            op = self.ops[nid]
            if getattr(op, "has_grad", False):
                timed((nid, "bwd"), op.backward)
        if update:
            timed((-2, "sync_gradients"), self.sync_gradients)
            timed((-3, "update"), self.update)
        t1.record()
        torch.cuda.synchronize()
        by_type, by_node = {}, {}
        for (nid, phase), e0, e1 in recs:
            ms = e0.elapsed_time(e1)
            typ = self.nodes[nid]["type"] if nid >= 0 else phase
            by_type[(typ, phase)] = by_type.get((typ, phase), 0.0) + ms
            by_node[(nid, phase)] = ms
        return {"by_type": by_type, "by_node": by_node, "total_ms": t0.elapsed_time(t1)}

    def sync_gradients(self):
        """Hook for the distributed executable (gradient all-reduce of replicated weights)."""

    def zero_gradients(self):
        """Nothing to clear: the plan marks, per gradient buffer, which operator writes it first (a plain store)
        and which accumulate, so no buffer is read before it has been written in the same step."""

    def update(self, start: int = 0):
        """Optimizer step over the parameter arena from element `start` (the distributed executable updates the
        replicated prefix inside its gradient all-reduce and passes the end of that prefix here)."""
        o = self.cfg.optimizer
        self.step_count += 1
        if start >= self.master.numel():
            return
        sl = slice(start, None)
        shadow = self.shadow[sl] if self.shadow is not None else None
        if o.kind == "adam":
            K.adam_update(self.master[sl], self.opt_m[sl], self.opt_v[sl], self.grads[sl], shadow, 0.0, o.beta1, o.beta2, o.epsilon,
                          o.weight_decay, 1.0, alpha_tensor=self.alpha_tensor)
        else:
            K.sgd_update(self.master[sl], self.opt_m[sl] if self.opt_m is not None else None, self.grads[sl], shadow, o.lr, o.momentum,
                         o.nesterov, o.weight_decay)

    def _pre_step(self):
        """Per-step scalars that a captured graph reads from device memory."""
        o = self.cfg.optimizer
        t = self.step_count + 1
        if o.kind == "adam":
            alpha_t = o.lr * math.sqrt(1.0 - o.beta2 ** t) / (1.0 - o.beta1 ** t)
            self.alpha_tensor.fill_(alpha_t)
        if self.seed_tensor is not None:
            self.seed_tensor.fill_((self.cfg.seed * 7919 + t * 104729) & 0x7FFFFFFFFFFFFFFF)

    def _step_body(self):
        self.forward()
        self.compute_loss()
        self.backward()
        self.sync_gradients()
        self.update()

    def train_step(self, inputs: Optional[Dict[str, torch.Tensor]] = None, labels: Optional[torch.Tensor] = None):
        """One optimisation step; returns the per-row loss tensor (device)."""
        if inputs is not None or labels is not None:
            self.set_inputs(inputs or {}, labels)
        self._pre_step()
        if self.cfg.use_cuda_graph and self.on_gpu:
            if not getattr(self, "_warmed", False):
                # the first step runs eagerly (lazy library initialisation must not happen during capture);
                # the graph is captured at the second call, which then replays it
                self._warmed = True
                self._step_body()
                return self.loss_rows
            if self._graph is None:
                torch.cuda.synchronize()
                self._graph = torch.cuda.CUDAGraph()
                cap_stream = torch.cuda.Stream()
                cap_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(cap_stream):
                    count = self.step_count
                    l0 = K.launch_count()
                    with torch.cuda.graph(self._graph, stream=cap_stream):
                        self._step_body()
                    self.launches_per_step = K.launch_count() - l0
                    self.step_count = count
                torch.cuda.current_stream().wait_stream(cap_stream)
            self._graph.replay()
            self.step_count += 1
        else:
            self._step_body()
        return self.loss_rows

    def infer(self, inputs: Dict[str, torch.Tensor]):
        self.set_inputs(inputs)
        self.forward()
        op = self.ops[self.loss_value[0]] if self.loss_value is not None else None
        if isinstance(op, SoftmaxOp):
            return op.probabilities()
        return self.values[self.loss_value].data if self.loss_value else None

    def mean_loss(self) -> float:
        return float(self.loss_rows.mean().item())

    # ---- parameter access (checkpointing, tests)
    def named_parameters(self):
        for nid in self.param_nodes:
            o, n = self.param_offsets[nid]
            name = self.nodes[nid]["name"] or f"weight{nid}"
            yield name, self.master[o:o + n].view(self.local_weight_shape(nid))
        for nid, t in self.sparse_tables.items():
            if t is not None:
                yield self.nodes[nid]["name"] or f"weight{nid}", t

    def named_gradients(self):
        for nid in self.param_nodes:
            o, n = self.param_offsets[nid]
            name = self.nodes[nid]["name"] or f"weight{nid}"
            yield name, self.grads[o:o + n].view(self.local_weight_shape(nid))

    def state_dict(self):
        sd = {"master": self.master, "step": self.step_count}
        for nid, t in self.sparse_tables.items():
            if t is not None:
                sd[f"table.{self.nodes[nid]['name'] or nid}"] = t
        if self.cfg.training:
            if self.opt_m is not None:
                sd["opt_m"] = self.opt_m
            if self.opt_v is not None:
                sd["opt_v"] = self.opt_v
        return sd

    def load_state_dict(self, sd):
        self.master.copy_(sd["master"])
        if self.shadow is not None:
            self.shadow.copy_(self.master)
        self.step_count = int(sd.get("step", 0))
        for nid, t in self.sparse_tables.items():
            key = f"table.{self.nodes[nid]['name'] or nid}"
            if t is not None and key in sd:
                t.copy_(sd[key])
        if self.cfg.training:
            if "opt_m" in sd and self.opt_m is not None:
                self.opt_m.copy_(sd["opt_m"])
            if "opt_v" in sd and self.opt_v is not None:
                self.opt_v.copy_(sd["opt_v"])


from . import executor_ops  # noqa: E402,F401  (registers the convolution-stack and tensor-shape operators)
