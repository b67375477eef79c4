"""SPMD executor for a parallel computation graph: every rank runs the same plan on its own shards.

This replaces the reference's single-controller Realm executor (lib/realm-execution/src/realm-execution/
pcg_instance.cc:80-273), which spawns one JSON-serialised task per shard and cannot execute the parallel
operators at all.  Here

* a tensor whose parallel shape has degree `world` on one dim is held as the rank-th piece; a tensor of total
  degree 1 is replicated (operators on it run redundantly, as in Megatron-style tensor parallelism);
* the four parallel operators become: Repartition = take the local slice (backward: all-gather), Combine =
  all-gather (backward: slice), Replicate = nothing (backward: all-reduce), Reduction = all-reduce (backward:
  nothing);
* a Weight followed only by parallel operators is materialised directly as its local shard; if that chain
  contains a Replicate the weight's gradient is summed over ranks by the fused all-reduce+scale kernel over
  NVLink peer memory, bucketed and launched on a side stream while backward is still running.

Supported strategies: one mesh axis (every parallel degree equals the world size), which covers pure data
parallelism, pure tensor parallelism and per-operator mixtures of the two.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..runtime import executor as E
from ..runtime.executor import ExecConfig, Executable, OpImpl, Value, register
from . import comm
from .context import DistContext
from .fused_ops import GradAllReduce

PARALLEL = ("REPARTITION", "COMBINE", "REPLICATE", "REDUCTION")


def _degree(attrs) -> int:
    for k in ("repartition_degree", "combine_degree", "replicate_degree", "reduction_degree"):
        if k in attrs:
            return int(attrs[k])
    return 1


class _ParallelOp(OpImpl):
    """Common part: on one device, or inside a weight chain, a parallel operator is an alias of its input."""

    def is_alias(self) -> bool:
        ex = self.ex
        return ex.dist is None or ex.dist.world_size == 1 or self.nid in getattr(ex, "weight_chain_nodes", ())

    def alias_setup(self):
        self.out().data = self.x()
        self.ex.alias(self.nid, self.inputs["INPUT"])

    def check_degree(self):
        d = _degree(self.attrs)
        if d != self.ex.dist.world_size:
            raise NotImplementedError(f"{self.type} of degree {d} on {self.ex.dist.world_size} ranks: only one mesh axis is supported")


@register("REPARTITION")
class RepartitionOp(_ParallelOp):
    def setup(self):
        if self.is_alias():
            return self.alias_setup()
        self.check_degree()
        x = self.x()
        self.dim = int(self.attrs["repartition_dim"]) % x.dim()
        self.piece = x.shape[self.dim] // self.ex.dist.world_size
        self.alloc_out()

    def forward(self):
        if self.is_alias():
            return
        r = self.ex.dist.rank
        self.out().data.copy_(self.x().narrow(self.dim, r * self.piece, self.piece))

    def backward(self):
        if self.is_alias():
            return
        b = self.buf("INPUT")
        if b.requires_grad:
            g = comm.nccl_all_gather_dim(self.out().grad.view_as(self.out().data), self.dim, self.ex.dist.world_size, self.ex.dist.group)
            self.ex.write_grad(b, g, self.acc["INPUT"])


@register("COMBINE")
class CombineOp(_ParallelOp):
    def setup(self):
        if self.is_alias():
            return self.alias_setup()
        self.check_degree()
        self.dim = int(self.attrs["combine_dim"]) % self.x().dim()
        self.alloc_out()

    def forward(self):
        if self.is_alias():
            return
        comm.nccl_all_gather_dim(self.x(), self.dim, self.ex.dist.world_size, self.ex.dist.group, out=self.out().data)

    def backward(self):
        if self.is_alias():
            return
        b = self.buf("INPUT")
        if b.requires_grad:
            piece = self.x().shape[self.dim]
            g = self.out().grad.view_as(self.out().data).narrow(self.dim, self.ex.dist.rank * piece, piece)
            self.ex.write_grad(b, g.contiguous(), self.acc["INPUT"])


@register("REPLICATE")
class ReplicateOp(_ParallelOp):
    def setup(self):
        if self.is_alias():
            return self.alias_setup()
        self.check_degree()
        self.out().data = self.x()  # already present on every rank

    def forward(self):
        pass

    def backward(self):
        if self.is_alias():
            return
        b = self.buf("INPUT")
        if b.requires_grad:
            g = self.out().grad
            dist.all_reduce(g, group=self.ex.dist.group)  # the replicas' gradients add up
            self.ex.write_grad(b, g, self.acc["INPUT"])


@register("REDUCTION")
class ReductionOp(_ParallelOp):
    def setup(self):
        if self.is_alias():
            return self.alias_setup()
        self.check_degree()
        # the partial sum is reduced in place and every rank keeps the full result
        self.out().data = self.x()
        self.ex.alias(self.nid, self.inputs["INPUT"])

    def forward(self):
        if self.ex.dist is None or self.ex.dist.world_size == 1 or self.nid in getattr(self.ex, "weight_chain_nodes", ()):
            return
        dist.all_reduce(self.x(), group=self.ex.dist.group)


class DistExecutable(Executable):
    def __init__(self, pcg, cfg: Optional[ExecConfig], ctx: DistContext, bucket_mb: int = 128, overlap: bool = True):
        self.ctx = ctx
        self.bucket_bytes = bucket_mb << 20
        self.overlap = overlap
        self._pre_analyse(pcg, ctx)
        super().__init__(pcg, cfg, dist=ctx)
        self._plan_buckets()
        self.parallelism = self._describe()

    # ------------------------------------------------------------------ static analysis of the strategy
    def _pre_analyse(self, g, ctx):
        nodes = {n["id"]: n for n in g.nodes()}
        W = ctx.world_size
        self.weight_chain_nodes = set()
        self.weight_final: Dict[int, Tuple[int, str]] = {}      # weight node -> last value of its parallel-op chain
        self.weight_replicated: Dict[int, bool] = {}
        self.weight_consumer: Dict[int, Tuple[int, str]] = {}   # weight node -> (consumer node, slot)
        for nid, n in nodes.items():
            if n["type"] != "WEIGHT":
                continue
            v = (nid, "OUTPUT")
            replicated = False
            while True:
                cons = g.consumers(v)
                if len(cons) == 1 and nodes[cons[0][0]]["type"] in PARALLEL:
                    c = cons[0][0]
                    self.weight_chain_nodes.add(c)
                    if nodes[c]["type"] == "REPLICATE":
                        replicated = True
                    v = (c, nodes[c]["outputs"][0][0])
                else:
                    if cons:
                        self.weight_consumer[nid] = (cons[0][0], cons[0][1])
                    break
            self.weight_final[nid] = v
            self.weight_replicated[nid] = replicated
        self._nodes_pre = nodes
        self._g_pre = g

    def _final_shape(self, nid):
        return self._g_pre.shape(self.weight_final[nid])

    def local_weight_shape(self, nid):
        return list(self._final_shape(nid).piece_sizes)

    def shard_weight(self, nid, full):
        sh = self._final_shape(nid)
        r = self.ctx.rank
        cons = self.weight_consumer.get(nid)
        if cons is not None and self._nodes_pre[cons[0]]["type"] == "MULTIHEAD_ATTENTION" and any(d > 1 for d in sh.degrees):
            return self._shard_attention_weight(nid, full, cons)
        t = full
        for d, deg in enumerate(sh.degrees):
            if deg > 1:
                piece = t.shape[d] // deg
                t = t.narrow(d, (r % deg) * piece, piece)
        return t.contiguous()

    def _shard_attention_weight(self, nid, full, cons):
        """Head-parallel attention: slice the packed projection blocks (see AttentionOp) by heads."""
        a = self._nodes_pre[cons[0]]["attrs"]
        node = self._nodes_pre[cons[0]]
        H, kd, vd, E_ = int(a["num_heads"]), int(a["kdim"]), int(a["vdim"]), int(a["embed_dim"])
        W, r = self.ctx.world_size, self.ctx.rank
        Hl = H // W
        ins = {s: tuple(v) for s, v in node["inputs"]}
        dq = self._g_pre.shape(ins["QUERY"]).sizes[-1]
        dk = self._g_pre.shape(ins["KEY"]).sizes[-1]
        dv = self._g_pre.shape(ins["VALUE"]).sizes[-1]
        flat = full.reshape(-1)
        if cons[1] == "WEIGHT":
            o = 0
            wq = flat[o:o + H * kd * dq].view(H, kd * dq); o += H * kd * dq
            wk = flat[o:o + H * kd * dk].view(H, kd * dk); o += H * kd * dk
            wv = flat[o:o + H * vd * dv].view(H, vd * dv); o += H * vd * dv
            wo = flat[o:o + E_ * H * vd].view(E_, H, vd)
            parts = [wq[r * Hl:(r + 1) * Hl].reshape(-1), wk[r * Hl:(r + 1) * Hl].reshape(-1), wv[r * Hl:(r + 1) * Hl].reshape(-1),
                     wo[:, r * Hl:(r + 1) * Hl].reshape(-1)]
            return torch.cat(parts)
        if cons[1] == "INPUT_BIAS":
            bq, bk, bv = flat[:H * kd].view(H, kd), flat[H * kd:2 * H * kd].view(H, kd), flat[2 * H * kd:].view(H, vd)
            return torch.cat([bq[r * Hl:(r + 1) * Hl].reshape(-1), bk[r * Hl:(r + 1) * Hl].reshape(-1), bv[r * Hl:(r + 1) * Hl].reshape(-1)])
        return full

    def order_params(self, param_nodes):
        # gradients that must be summed over ranks first: they form one contiguous range of the arena
        rep = [n for n in param_nodes if self.weight_replicated[n]]
        rest = [n for n in param_nodes if not self.weight_replicated[n]]
        self._num_rep_params = len(rep)
        return rep + rest

    def alloc_grad_arena(self, numel, dtype):
        self.grad_ar = GradAllReduce(self.ctx, numel, dtype)
        return self.grad_ar.tensor

    def head_shards(self, op) -> int:
        w = op.inputs.get("WEIGHT")
        if w is None:
            return 1
        return max(self.graph.shape(w).degrees + [1])

    def use_bias(self, op, slot: str) -> bool:
        v = op.inputs.get(slot)
        if v is None:
            return False
        out_sum = self.graph.shape((op.nid, op.outputs[0][0])).sum_degree
        return out_sum == 1 or self.ctx.rank == 0

    # ------------------------------------------------------------------ loss on the local shard
    def resolve_loss_value(self, v: Value) -> Value:
        skip = getattr(self, "_skip_nodes", set())
        while self.nodes[v[0]]["type"] in ("COMBINE",) and v[0] not in self.weight_chain_nodes:
            skip.add(v[0])
            v = tuple(self.nodes[v[0]]["inputs"][0][1])
        self._skip_nodes = skip
        return v

    def global_loss_rows(self, local_rows: int, shape) -> int:
        n = local_rows
        for d in shape.degrees[:-1]:
            n *= d
        return n

    def local_label_rows(self, labels, rows):
        flat = labels.reshape(-1) if self.cfg.loss == "sparse_categorical_crossentropy" else labels.reshape(-1, labels.shape[-1])
        if flat.shape[0] == rows:
            return flat
        r = self.ctx.rank
        return flat[r * rows:(r + 1) * rows]

    # ------------------------------------------------------------------ gradient synchronisation (F3)
    def _plan_buckets(self):
        if not self.cfg.training:
            return
        offs = self.param_offsets
        rep = self.param_nodes[:self._num_rep_params]
        self.rep_numel = 0
        if rep:
            last = rep[-1]
            self.rep_numel = (offs[last][0] + offs[last][1] + 7) // 8 * 8
        es = self.grads.element_size()
        per_bucket = max(self.bucket_bytes // es, 1)
        # buckets are arena ranges; a bucket may be launched once every parameter in it has its gradient,
        # i.e. after the backward of the operator that produces the bucket's last-finished gradient
        self.buckets: List[Tuple[int, int]] = []
        start = 0
        while start < self.rep_numel:
            end = min(self.rep_numel, start + per_bucket)
            end = (end + 7) // 8 * 8 if end < self.rep_numel else self.rep_numel
            self.buckets.append((start, end))
            start = end
        done_after: Dict[int, int] = {}  # param node -> position in backward order of the op writing its gradient
        bwd_order = [nid for nid in reversed(self.order) if getattr(self.ops[nid], "has_grad", False)]
        pos = {nid: i for i, nid in enumerate(bwd_order)}
        for p in rep:
            cons = self.weight_consumer.get(p)
            done_after[p] = pos.get(cons[0], len(bwd_order) - 1) if cons else len(bwd_order) - 1
        self._launch_after: Dict[int, List[int]] = {}
        for bi, (s, e) in enumerate(self.buckets):
            members = [p for p in rep if offs[p][0] < e and offs[p][0] + offs[p][1] > s]
            when = max([done_after[p] for p in members], default=len(bwd_order) - 1)
            nid = bwd_order[when] if bwd_order else -1
            self._launch_after.setdefault(nid, []).append(bi)
        self.side = torch.cuda.Stream() if self.overlap else None
        self._pending = False

    def backward(self):
        if not getattr(self, "buckets", None):
            return super().backward()
        main = torch.cuda.current_stream()
        for nid in reversed(self.order):
            op = self.ops[nid]
            if getattr(op, "has_grad", False):
                op.backward()
                for bi in self._launch_after.get(nid, ()):
                    self._launch_bucket(bi, main)
        for bi in self._launch_after.get(-1, ()):
            self._launch_bucket(bi, main)

    def _launch_bucket(self, bi, main):
        s, e = self.buckets[bi]
        if self.side is not None:
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                self.grad_ar.run(scale=1.0, offset=s, n=e - s)
            self._pending = True
        else:
            self.grad_ar.run(scale=1.0, offset=s, n=e - s)

    def sync_gradients(self):
        if self.side is not None and self._pending:
            torch.cuda.current_stream().wait_stream(self.side)
            self._pending = False

    def _describe(self) -> str:
        W = self.ctx.world_size
        kinds = set()
        for n in self.nodes.values():
            if n["type"] in ("LINEAR", "MULTIHEAD_ATTENTION", "CONV2D", "EMBEDDING"):
                sh = n["outputs"][0][1]
                if sh.sum_degree > 1 or (sh.degrees and sh.degrees[-1] > 1):
                    kinds.add("tp")
                elif sh.degrees and sh.degrees[0] > 1:
                    kinds.add("dp")
        if not kinds:
            return f"replicated{W}"
        return "+".join(f"{k}{W}" for k in sorted(kinds))

    def mean_loss(self) -> float:
        """Mean loss over the global batch (sums the local rows over ranks when the loss is batch-sharded)."""
        s = self.loss_rows.sum().reshape(1).to(torch.float64)
        sharded = self.global_loss_rows(1, self.graph.shape(self.loss_value)) > 1
        if sharded:
            dist.all_reduce(s, group=self.ctx.group)
        return float(s.item() * self.loss_scale)
