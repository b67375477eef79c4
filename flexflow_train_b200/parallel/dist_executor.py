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
parallelism, pure tensor parallelism, per-operator mixtures of the two, and model-parallel embedding tables
under a data-parallel model (``AllToAllEmbeddingOp``); and two mesh axes, data parallel of degree dp around tensor
parallel of degree tp (``compiler.strategy.hybrid_strategy``): rank r = i_dp * tp + i_tp, sample-dimension operators
work inside the group of ranks that share i_tp, Replicate / Reduction and weight shards inside the group that shares
i_dp, and the gradients of every weight are summed over the data-parallel group by the fused bucket kernel.
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
from .fused_ops import PeerAllGather, PeerReduceScatter, AllGatherGemm, AllToAllEmbedding, GemmReduceScatter, GradAllReduce

PARALLEL = ("REPARTITION", "COMBINE", "REPLICATE", "REDUCTION")


def _degree(attrs) -> int:
    for k in ("repartition_degree", "combine_degree", "replicate_degree", "reduction_degree"):
        if k in attrs:
            return int(attrs[k])
    return 1


class _ParallelOp(OpImpl):
    """Common part: on one device, or inside a weight chain, a parallel operator is an alias of its input.

    ``absorbed`` marks an operator whose collective is executed inside a neighbouring GEMM (see ``FuseIn`` /
    ``FuseOut``): it only owns buffers.  ``pair`` links Reduction->Repartition and Combine->Replicate couples
    that are not fused into a GEMM: together they are one reduce-scatter / all-gather instead of an all-reduce
    followed by a slice."""
    absorbed = False
    pair = None

    def communicates(self) -> bool:
        """Does this operator call NCCL in forward or backward?"""
        if self.is_alias() or self.absorbed or isinstance(self, E.SkippedOp):
            return False
        if self.type in ("REPLICATE", "REDUCTION") and self.pair is None and self.ex.peer_allreduce:
            return False  # summed in place by the peer-memory all-reduce kernel
        if self.type == "REPARTITION":
            if self.pair is None:  # forward is a local slice; backward all-gathers
                return self.buf("INPUT").requires_grad and self.peer_ag is None
            return self.peer_rs is None or (self.pair.buf("INPUT").requires_grad and self.peer_ag is None)
        if self.type == "COMBINE":
            return self.peer_ag is None
        if self.type == "REPLICATE" and self.pair is not None:
            return self.pair.buf("INPUT").requires_grad and self.peer_rs is None
        return True

    def is_alias(self) -> bool:
        ex = self.ex
        return ex.dist is None or ex.dist.world_size == 1 or self.nid in getattr(ex, "weight_chain_nodes", ())

    # ---- stand-alone collectives over peer memory (NCCL when the executable was built without them or the piece does not
    # fit the kernels' 16-byte vectors).  The buffers are symmetric allocations, so they are made in setup(), where every
    # rank passes in the same order.
    peer_ag = None
    peer_rs = None

    def _peer_fits(self, numel: int, dtype) -> bool:
        if not getattr(self.ex, "peer_collectives", False) or dtype not in (torch.bfloat16, torch.float32):
            return False
        es = 2 if dtype == torch.bfloat16 else 4
        return numel % 8 == 0 and (numel * es) % 16 == 0

    def make_peer_all_gather(self, shard: torch.Tensor):
        if self._peer_fits(shard.numel(), shard.dtype):
            self.peer_ag = PeerAllGather(self.gctx, shard.numel(), shard.dtype)

    def make_peer_reduce_scatter(self, piece: torch.Tensor):
        if self._peer_fits(piece.numel(), piece.dtype):
            self.peer_rs = PeerReduceScatter(self.gctx, piece.numel(), piece.dtype)

    def all_gather_dim(self, t: torch.Tensor, dim: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """All ranks' `t` concatenated along `dim` (materialised contiguously, into `out` when given)."""
        W = self.gctx.world_size
        if self.peer_ag is None:
            return comm.nccl_all_gather_dim(t, dim, W, self.gctx.group, out=out)
        parts = self.peer_ag(t.contiguous().view(-1)).view((W,) + tuple(t.shape))
        if dim == 0:
            res = parts.view((W * t.shape[0],) + tuple(t.shape[1:]))
        else:
            perm = list(range(1, dim + 1)) + [0] + list(range(dim + 1, t.dim() + 1))
            res = K.permute(parts, perm).view(tuple(t.shape[:dim]) + (W * t.shape[dim],) + tuple(t.shape[dim + 1:]))
        if out is not None:
            out.copy_(res)
            return out
        # the staging buffer is overwritten by this operator's next call: hand out a copy unless the caller consumes it now
        return res

    def reduce_scatter(self, out_flat: torch.Tensor, full_flat: torch.Tensor, accumulate: bool = False):
        """out (+)= this rank's piece of the sum of `full` over the group."""
        if self.peer_rs is not None:
            self.peer_rs(full_flat, out_flat, accumulate=accumulate)
        elif accumulate:
            t = torch.empty_like(out_flat)
            dist.reduce_scatter_tensor(t, full_flat, group=self.gctx.group)
            out_flat.add_(t)
        else:
            dist.reduce_scatter_tensor(out_flat, full_flat, group=self.gctx.group)

    def uses_library_collectives(self, needs_gather: bool, needs_scatter: bool) -> bool:
        return (needs_gather and self.peer_ag is None) or (needs_scatter and self.peer_rs is None)

    def alias_setup(self):
        self.out().data = self.x()
        self.ex.alias(self.nid, self.inputs["INPUT"])

    @property
    def gctx(self):
        """The ranks this operator's collective spans: the whole job on a one-axis plan; on a dp x tp mesh the
        data-parallel group for Repartition / Combine of the sample dimension and the tensor-parallel group for
        everything else."""
        ex = self.ex
        mesh = getattr(ex, "mesh", None)
        if mesh is None:
            return ex.dist
        if self.type in ("REPARTITION", "COMBINE"):
            dim = int(self.attrs["repartition_dim" if self.type == "REPARTITION" else "combine_dim"])
            if dim == 0:
                return ex.ctx_dp
        return ex.ctx_tp

    def check_degree(self):
        d = _degree(self.attrs)
        if d != self.gctx.world_size:
            raise NotImplementedError(f"{self.type} of degree {d} on a group of {self.gctx.world_size} ranks "
                                      f"({self.ex.dist.world_size} in the job): the strategy does not fit the device mesh")


@register("REPARTITION")
class RepartitionOp(_ParallelOp):
    def setup(self):
        if self.is_alias():
            return self.alias_setup()
        self.check_degree()
        y = self.alloc_out()
        self.dim = int(self.attrs["repartition_dim"]) % y.dim()
        self.piece = y.shape[self.dim]
        # A graph input that is only read through this Repartition can be fed shard by shard: with
        # `DistExecutable.shard_inputs` the caller hands each rank its own piece, which is copied straight into this
        # operator's output and the whole-tensor copy disappears from the step (host-to-device traffic per rank then
        # shrinks with the number of ranks).
        src = self.ex.nodes[self.inputs["INPUT"][0]]
        self.direct = bool(getattr(self.ex, "shard_inputs", False) and src["type"] == "INPUT" and not src["outputs"][0][2]
                           and len(self.ex.graph.consumers(self.inputs["INPUT"])) == 1)
        if self.direct:
            self.ex.direct_inputs[src["name"] or f"input{src['id']}"] = self
        if not self.absorbed:
            if self.pair is not None:
                self.make_peer_reduce_scatter(y)
            if self.ex.cfg.training and (self.pair.buf("INPUT") if self.pair is not None else self.buf("INPUT")).requires_grad:
                self.make_peer_all_gather(y)

    def forward(self):
        if self.is_alias() or self.absorbed or getattr(self, "direct", False):
            return
        if self.pair is not None:  # Reduction -> Repartition(0): one reduce-scatter of the partial sums
            self.reduce_scatter(self.out().data.view(-1), self.pair.x().view(-1))
            return
        r = self.gctx.rank
        self.out().data.copy_(self.x().narrow(self.dim, r * self.piece, self.piece))

    def backward(self):
        if self.is_alias() or self.absorbed:
            return
        if self.pair is not None:
            b = self.pair.buf("INPUT")
            if b.requires_grad:
                g = self.all_gather_dim(self.out().grad.view_as(self.out().data), 0)
                self.ex.write_grad(b, g, self.pair.acc["INPUT"])
            return
        b = self.buf("INPUT")
        if b.requires_grad:
            g = self.all_gather_dim(self.out().grad.view_as(self.out().data), self.dim)
            self.ex.write_grad(b, g, self.acc["INPUT"])


@register("COMBINE")
class CombineOp(_ParallelOp):
    def setup(self):
        if self.is_alias():
            return self.alias_setup()
        self.check_degree()
        self.dim = int(self.attrs["combine_dim"]) % self.x().dim()
        if self.absorbed:
            self.out().data = self.fuse.bind_gathered(self)  # the staging buffer of the fused all-gather
            return
        self.alloc_out()
        self.make_peer_all_gather(self.x())

    def forward(self):
        if self.is_alias() or self.absorbed:
            return
        self.all_gather_dim(self.x(), self.dim, out=self.out().data)

    def backward(self):
        if self.is_alias() or self.absorbed or self.pair is not None:
            return  # (paired: the Replicate reduce-scattered straight into this operator's input gradient)
        b = self.buf("INPUT")
        if b.requires_grad:
            piece = self.x().shape[self.dim]
            g = self.out().grad.view_as(self.out().data).narrow(self.dim, self.gctx.rank * piece, piece)
            self.ex.write_grad(b, g.contiguous(), self.acc["INPUT"])


@register("REPLICATE")
class ReplicateOp(_ParallelOp):
    def setup(self):
        if self.is_alias():
            return self.alias_setup()
        self.check_degree()
        self.out().data = self.x()  # already present on every rank
        if self.pair is not None and not self.absorbed and self.ex.cfg.training and self.pair.buf("INPUT").requires_grad:
            self.make_peer_reduce_scatter(self.pair.x())

    def forward(self):
        pass

    def backward(self):
        if self.is_alias() or self.absorbed:
            return
        if self.pair is not None:  # Combine(0) -> Replicate: sum over ranks and keep the own rows = reduce-scatter
            cb = self.pair.buf("INPUT")
            if cb.requires_grad:
                self.reduce_scatter(cb.grad.view(-1), self.out().grad.view(-1), accumulate=self.pair.acc["INPUT"])
            return
        b = self.buf("INPUT")
        if b.requires_grad:
            g = self.out().grad
            self.ex.all_reduce_activation(g, self.gctx)  # the replicas' gradients add up
            self.ex.write_grad(b, g, self.acc["INPUT"])


@register("REDUCTION")
class ReductionOp(_ParallelOp):
    def setup(self):
        if self.is_alias():
            return self.alias_setup()
        self.check_degree()
        if self.absorbed or self.pair is not None:
            self.out().data = None  # nobody reads the unreduced full tensor: the Repartition holds the result
            return
        # the partial sum is reduced in place and every rank keeps the full result
        self.out().data = self.x()
        self.ex.alias(self.nid, self.inputs["INPUT"])

    def forward(self):
        if self.ex.dist is None or self.ex.dist.world_size == 1 or self.nid in getattr(self.ex, "weight_chain_nodes", ()):
            return
        if self.absorbed or self.pair is not None:
            return
        self.ex.all_reduce_activation(self.x(), self.gctx)


class AllToAllEmbeddingOp(_ParallelOp):
    """The Repartition(0) behind a stack of whole-table Embeddings (tables model-parallel, samples data-parallel).

    Takes the place of the lookups, their Reshapes, the Concat and the Repartition: every rank gathers, for the
    whole batch, the rows of the tables it owns and writes them straight into the sample owners' buffers over
    NVLink (forward); backward pulls the rows of d(stack) from the sample owners and applies the sparse SGD
    update to the local tables.  No table and no table-sized gradient ever leaves its rank."""
    group = None

    def communicates(self) -> bool:
        return False  # peer-memory kernels with device-side barriers, no NCCL call

    def setup(self):
        ex, grp = self.ex, self.group
        W, r = ex.ctx.world_size, ex.ctx.rank
        sh = dict(self.outputs)["OUTPUT"]
        lb, T, dim = [int(v) for v in sh.piece_sizes]
        local = [ex.sparse_tables[m["weight"]] for t, m in enumerate(grp["members"]) if t % W == r]
        dt = ex.torch_dtype(sh.dtype)
        self.f4 = AllToAllEmbedding(ex.ctx, local, T, dim, lb, out_dtype=dt)
        b = self.out()
        b.data, b.grad = self.f4.out_t, self.f4.dout_t
        self.index_values = [m["index"] for m in grp["members"]]
        idx0 = ex.values[self.index_values[0]].data
        self.idx = torch.empty(lb * W, T, dtype=idx0.dtype, device=ex.device)
        ex.values[self.inputs["INPUT"]].requires_grad = False  # the stack itself is never materialised

    def forward(self):
        torch.cat([self.ex.values[v].data.view(-1, 1) for v in self.index_values], dim=1, out=self.idx)
        self.f4.forward(self.idx)

    def backward(self):
        self.f4.backward_sgd(self.idx, self.ex.cfg.optimizer.lr)


class FuseIn:
    """Combine(dim 0) -> Replicate -> GEMM: the operand arrives as row shards.

    Forward runs the all-gather inside the GEMM (peers push their shard into this rank's staging buffer; the TMA
    producer waits per row block).  The staging buffer *is* the Combine's output, so the weight-gradient GEMM of
    backward reads the gathered operand from it.  Backward of the pair is a reduce-scatter of the data
    gradient's partial sums, run inside the data-gradient GEMM whose epilogue scatters tiles to their owners."""

    def __init__(self, ex: "DistExecutable", combine: CombineOp, replicate: ReplicateOp):
        self.ex, self.combine, self.replicate = ex, combine, replicate
        self.ag: Optional[AllGatherGemm] = None

    def bind_gathered(self, combine: CombineOp) -> torch.Tensor:
        x = combine.x()
        self.rows_local, self.k = x.numel() // x.shape[-1], x.shape[-1]
        self.ag = AllGatherGemm(self.ex.ctx, self.rows_local, self.k, x.dtype)
        self.rs = self.ex.shared_reduce_scatter(self.rows_local * self.ex.ctx.world_size, self.k, x.dtype)
        full = [int(v) for v in dict(combine.outputs)["OUTPUT"].piece_sizes]
        return self.ag.gathered_t.view(full)

    def gemm(self, w, out, bias=None, act=None, pre_act_out=None, dropout=None):
        self.ag(self.combine.x().view(self.rows_local, self.k), w, out, bias=bias, act=act, pre_act_out=pre_act_out, dropout=dropout)

    def grad_gemm(self, dy, w, accumulate: bool):
        """d(shard) (+)= reduce_scatter(dy @ w) with w [N_local, K] used as the [k, n] operand."""
        b = self.combine.buf("INPUT")
        if not b.requires_grad:
            return
        g = b.grad.view(self.rows_local, self.k)
        self.rs(dy, w, g, residual=g if accumulate else None, w_kn=True)


class FuseOut:
    """GEMM -> Reduction -> Repartition(dim 0): the partial sums are wanted as row shards.

    Forward: the GEMM epilogue writes each output tile into the owning rank's stage and a flag-gated kernel sums
    the staged partials into the Repartition's output.  Backward: the shard gradients are all-gathered inside the
    data-gradient GEMM; the gathered dY stays in the staging buffer for the weight and bias gradients."""

    def __init__(self, ex: "DistExecutable", reduction: ReductionOp, repartition: RepartitionOp, rows: int, n: int, dtype):
        self.ex, self.reduction, self.repartition = ex, reduction, repartition
        W = ex.ctx.world_size
        self.rows, self.n = rows, n
        self.rs = ex.shared_reduce_scatter(rows, n, dtype)
        self.ag = ex.shared_grad_gather(rows // W, n, dtype)

    def gemm(self, x, w, bias=None):
        out = self.repartition.out().data
        self.rs(x, w, out.view(self.rows // self.ex.ctx.world_size, self.n), bias=bias)

    def gather_grad_gemm(self, w, dx, accumulate=False):
        dy_shard = self.repartition.out().grad.view(self.rows // self.ex.ctx.world_size, self.n)
        if dx is None:
            dx = self.ex.discard_buffer(self.rows, w.shape[1], dy_shard.dtype)
        self.ag(dy_shard, w, dx, w_kn=True, accumulate=accumulate)
        return self.ag.gathered_t


class DistExecutable(Executable):
    def __init__(self, pcg, cfg: Optional[ExecConfig], ctx: DistContext, bucket_mb: int = 128, overlap: bool = True,
                 fuse_collectives: bool = True, fuse_optimizer: bool = True, shard_inputs: bool = False):
        self.ctx = ctx
        self.shard_inputs = shard_inputs
        self.direct_inputs: Dict[str, "RepartitionOp"] = {}
        self.fuse_collectives = fuse_collectives
        self.fuse_optimizer = fuse_optimizer
        self._rs_shared: Dict[tuple, GemmReduceScatter] = {}
        self._ag_shared: Dict[tuple, AllGatherGemm] = {}
        self._discard: Dict[tuple, torch.Tensor] = {}
        self.fused_in: List[int] = []
        self.fused_out: List[int] = []
        self.bucket_bytes = bucket_mb << 20
        self.overlap = overlap
        self._ar_stage: Dict[tuple, object] = {}
        # activations are summed over ranks (Replicate backward, Reduction forward) by the peer-memory all-reduce kernel
        # through a symmetric staging buffer, so that a plan with such operators is still one CUDA graph
        self.peer_allreduce = fuse_collectives
        # the same for the stand-alone all-gathers and reduce-scatters of Combine / Repartition / Replicate
        self.peer_collectives = fuse_collectives
        self._pre_analyse(pcg, ctx)
        super().__init__(pcg, cfg, dist=ctx)
        # NCCL collectives are issued eagerly: a plan that still contains one (a parallel operator that is neither
        # an alias nor absorbed into a GEMM and that communicates) is not captured into a CUDA graph
        self.nccl_ops = [nid for nid, op in self.ops.items() if isinstance(op, _ParallelOp) and op.communicates()]
        if self.nccl_ops and self.cfg.use_cuda_graph:
            self.cfg.use_cuda_graph = False
        self._plan_buckets()
        self.parallelism = self._describe()

    # ------------------------------------------------------------------ fused collectives
    def shared_reduce_scatter(self, rows, n, dtype) -> GemmReduceScatter:
        """Stages are scratch within one call (a barrier opens every call), so operators of one shape share them."""
        key = (rows, n, dtype)
        if key not in self._rs_shared:
            self._rs_shared[key] = GemmReduceScatter(self.ctx, rows, n, dtype)
        return self._rs_shared[key]

    def shared_grad_gather(self, rows_local, k, dtype) -> AllGatherGemm:
        key = (rows_local, k, dtype)
        if key not in self._ag_shared:
            self._ag_shared[key] = AllGatherGemm(self.ctx, rows_local, k, dtype)
        return self._ag_shared[key]

    def discard_buffer(self, rows, cols, dtype):
        key = (rows, cols, dtype)
        if key not in self._discard:
            self._discard[key] = torch.empty(rows, cols, dtype=dtype, device=self.device)
        return self._discard[key]

    # ------------------------------------------------------------------ model-parallel embedding tables
    def _find_table_groups(self) -> List[dict]:
        """Repartition(0, world) <- Concat(axis 1) <- Reshape <- Embedding(whole table, whole batch, bag of one)."""
        g, nodes, W = self.graph, self.nodes, self.ctx.world_size
        groups = []
        for nid in self.order:
            n = nodes[nid]
            if n["type"] != "REPARTITION" or nid in self.weight_chain_nodes or _degree(n["attrs"]) != W \
                    or int(n["attrs"]["repartition_dim"]) != 0:
                continue
            src = tuple(n["inputs"][0][1])
            c = nodes[src[0]]
            csh = g.shape(src)
            if c["type"] != "CONCAT" or len(g.consumers(src)) != 1 or len(csh.sizes) != 3 or csh.total_degree != 1 \
                    or int(c["attrs"]["axis"]) % 3 != 1 or csh.sizes[0] % W != 0:
                continue
            members, skipped, ok = [], [c["id"]], True
            for _, v in sorted(c["inputs"], key=lambda sv: int(sv[0].split("_")[-1])):
                v = tuple(v)
                p = nodes[v[0]]
                if p["type"] in ("RESHAPE", "FLAT") and len(g.consumers(v)) == 1:
                    skipped.append(p["id"])
                    v = tuple(p["inputs"][0][1])
                    p = nodes[v[0]]
                ins = {s: tuple(x) for s, x in p["inputs"]}
                if p["type"] != "EMBEDDING" or len(g.consumers(v)) != 1 or nodes[ins["WEIGHT"][0]]["type"] != "WEIGHT" \
                        or nodes[ins["INPUT"][0]]["type"] != "INPUT":
                    ok = False
                    break
                ish, wsh = g.shape(ins["INPUT"]), g.shape(ins["WEIGHT"])
                bag = 1
                for d in ish.sizes[1:]:
                    bag *= d
                if bag != 1 or ish.total_degree != 1 or wsh.total_degree != 1 or ish.sizes[0] != csh.sizes[0] \
                        or wsh.sizes[1] != csh.sizes[2] or len(g.consumers(ins["WEIGHT"])) != 1:
                    ok = False
                    break
                skipped.append(p["id"])
                members.append({"embedding": p["id"], "weight": ins["WEIGHT"][0], "index": ins["INPUT"]})
            idx_types = {g.shape(m["index"]).dtype for m in members}
            if ok and len(members) == csh.sizes[1] and len(members) % W == 0 and len(idx_types) == 1:
                groups.append({"repartition": nid, "members": members, "skipped": skipped})
        return groups

    def sparse_weight_nodes(self):
        self.table_groups: List[dict] = []
        self._table_index: Dict[int, int] = {}
        self._group_embeddings = set()
        if self.ctx.world_size > 1 and self.fuse_collectives:
            self.table_groups = self._find_table_groups()
            for grp in self.table_groups:
                for t, m in enumerate(grp["members"]):
                    self._table_index[m["weight"]] = t
                    self._group_embeddings.add(m["embedding"])
        out = super().sparse_weight_nodes()
        if not all(m["weight"] in out for grp in self.table_groups for m in grp["members"]):
            self.table_groups = []  # the optimizer is not plain SGD: tables stay in the dense arenas
            self._table_index = {}
        return out

    def sparse_embedding_allowed(self, embedding_nid: int) -> bool:
        """A model-parallel table can take sparse updates; so can one whose lookup runs unsharded on every rank
        (all ranks then apply the same update from the same whole batch).  A table under a Replicate cannot: its
        ranks see different samples and their row updates would have to be exchanged."""
        if embedding_nid in self._group_embeddings:
            return True
        n = self.nodes[embedding_nid]
        ins = {s: tuple(v) for s, v in n["inputs"]}
        whole = all(self.graph.shape(v).total_degree == 1 for v in ins.values()) and n["outputs"][0][1].total_degree == 1
        return whole and self.nodes[ins["WEIGHT"][0]]["type"] == "WEIGHT"

    def owns_sparse_table(self, nid: int) -> bool:
        t = self._table_index.get(nid)
        return True if t is None else t % self.ctx.world_size == self.ctx.rank

    def _fuse(self):
        super()._fuse()
        W = self.ctx.world_size
        if W == 1:
            return
        for grp in getattr(self, "table_groups", ()):
            for nid in grp["skipped"]:
                self.ops[nid] = E.SkippedOp(self, nid, self.nodes[nid])
            op = AllToAllEmbeddingOp(self, grp["repartition"], self.nodes[grp["repartition"]])
            op.group = grp
            self.ops[grp["repartition"]] = op
        g = self.graph
        bf16 = self.cfg.compute_dtype == "bf16"

        def sole_consumer(v, kind):
            cons = g.consumers(v)
            if len({c[0] for c in cons}) != 1:
                return None
            op = self.ops[cons[0][0]]
            return op if op.type == kind and op.nid not in self.weight_chain_nodes else None

        for nid in self.order:
            op = self.ops[nid]
            # ---- Reduction -> Repartition(0)
            if isinstance(op, ReductionOp) and nid not in self.weight_chain_nodes and _degree(op.attrs) == W:
                rep = sole_consumer((nid, "OUTPUT"), "REPARTITION")
                if rep is None or int(rep.attrs["repartition_dim"]) != 0 or _degree(rep.attrs) != W:
                    continue
                prod = self.ops[op.inputs["INPUT"][0]]
                sizes = [int(v) for v in g.shape(op.inputs["INPUT"]).piece_sizes]
                rows, n = 1, sizes[-1]
                for v in sizes[:-1]:
                    rows *= v
                fusable = (self.fuse_collectives and bf16 and isinstance(prod, (E.LinearOp, E.AttentionOp)) and
                           (isinstance(prod, E.AttentionOp) or prod.fuse_in is None) and
                           len(g.consumers(op.inputs["INPUT"])) == 1 and rows % (128 * W) == 0 and n % 8 == 0 and
                           not prod.attrs.get("activation") and sizes[0] % W == 0)
                if fusable:
                    prod.fuse_out = FuseOut(self, op, rep, rows, n, torch.bfloat16)
                    op.absorbed = rep.absorbed = True
                    self.fused_out.append(prod.nid)
                elif sizes[0] % W == 0:
                    op.pair, rep.pair = rep, op
            # ---- Combine(0) -> Replicate
            if isinstance(op, CombineOp) and nid not in self.weight_chain_nodes and _degree(op.attrs) == W \
                    and int(op.attrs["combine_dim"]) % len(g.shape((nid, "OUTPUT")).sizes) == 0:
                rpl = sole_consumer((nid, "OUTPUT"), "REPLICATE")
                if rpl is None or _degree(rpl.attrs) != W:
                    continue
                cons = g.consumers((rpl.nid, "OUTPUT"))
                users = {c[0] for c in cons}
                sizes = [int(v) for v in g.shape(op.inputs["INPUT"]).piece_sizes]
                rows_local, k = 1, sizes[-1]
                for v in sizes[:-1]:
                    rows_local *= v
                user = self.ops[next(iter(users))] if len(users) == 1 else None
                slots_ok = user is not None and (
                    (isinstance(user, E.LinearOp) and [c[1] for c in cons] == ["INPUT"]) or
                    (isinstance(user, E.AttentionOp) and sorted(c[1] for c in cons) == ["KEY", "QUERY", "VALUE"]))
                if self.fuse_collectives and bf16 and slots_ok and rows_local % 128 == 0 and k % 8 == 0:
                    fi = FuseIn(self, op, rpl)
                    op.fuse = fi
                    user.fuse_in = fi
                    op.absorbed = rpl.absorbed = True
                    self.fused_in.append(user.nid)
                else:
                    op.pair, rpl.pair = rpl, op

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
        self._infer_mesh(g, nodes, ctx)

    def _infer_mesh(self, g, nodes, ctx):
        """One axis when every parallel operator spans the whole job.  Otherwise dp x tp: dp is the degree the sample
        dimension of the inputs is cut into, tp the degree of the Replicate / Reduction operators on activations and of
        the weight shards; rank r sits at (r // tp, r % tp)."""
        W = ctx.world_size
        self.mesh = None
        self.ctx_dp = self.ctx_tp = ctx
        self.tp_size, self.tp_idx, self.dp_size, self.dp_idx = W, ctx.rank, W, ctx.rank
        degrees = {_degree(n["attrs"]) for n in nodes.values() if n["type"] in PARALLEL}
        if W == 1 or not degrees or degrees <= {W, 1}:
            return
        dp = tp = None
        for nid, n in nodes.items():
            if n["type"] not in PARALLEL or nid in self.weight_chain_nodes:
                continue
            d = _degree(n["attrs"])
            dim0 = (n["type"] == "REPARTITION" and int(n["attrs"]["repartition_dim"]) == 0) or \
                   (n["type"] == "COMBINE" and int(n["attrs"]["combine_dim"]) == 0)
            if dim0:
                dp = d if dp is None else dp
                if d != dp:
                    raise NotImplementedError(f"sample-dimension operators of degrees {dp} and {d} in one strategy")
            else:
                tp = d if tp is None else tp
                if d != tp:
                    raise NotImplementedError(f"tensor-parallel operators of degrees {tp} and {d} in one strategy")
        dp = dp or (W // tp if tp else W)
        tp = tp or W // dp
        if dp * tp != W:
            raise NotImplementedError(f"strategy of degrees {sorted(degrees)} does not form a dp x tp mesh over {W} ranks")
        self.mesh = (dp, tp)
        self.dp_size, self.tp_size = dp, tp
        self.dp_idx, self.tp_idx = ctx.rank // tp, ctx.rank % tp
        self.ctx_dp, self.ctx_tp = ctx.make_mesh_groups(dp, tp)

    def all_reduce_activation(self, t: torch.Tensor, gctx):
        """Sum `t` over the ranks of `gctx`, in place."""
        if gctx.world_size == 1:
            return
        n = t.numel()
        if not (self.peer_allreduce and t.dtype in (torch.bfloat16, torch.float32) and t.is_contiguous() and n % 8 == 0):
            dist.all_reduce(t, group=gctx.group)
            return
        key = (id(gctx), t.dtype)
        ar = self._ar_stage.get(key)
        if ar is None or ar.numel < n:
            # grown at set-up time only (operators run once eagerly before a step is captured)
            ar = GradAllReduce(gctx, max(n, ar.numel if ar is not None else 0), t.dtype)
            self._ar_stage[key] = ar
        stage = ar.tensor[:n]
        stage.copy_(t.view(-1))
        ar.run(scale=1.0, offset=0, n=n)
        t.view(-1).copy_(stage)

    def _final_shape(self, nid):
        return self._g_pre.shape(self.weight_final[nid])

    def local_weight_shape(self, nid):
        return list(self._final_shape(nid).piece_sizes)

    def shard_weight(self, nid, full):
        sh = self._final_shape(nid)
        r = self.tp_idx if self.mesh is not None else self.ctx.rank
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
        W, r = (self.tp_size, self.tp_idx) if self.mesh is not None else (self.ctx.world_size, self.ctx.rank)
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
        # gradients are summed over the ranks that hold the same weight shard: the data-parallel group
        self.grad_ar = GradAllReduce(self.ctx_dp, numel, dtype)
        return self.grad_ar.tensor

    def alloc_shadow_arena(self, numel):
        # peers write the updated weights of the slices they own straight into this arena
        self.shadow_buf = self.ctx_dp.symmetric(numel * 2)
        t = self.shadow_buf.view(torch.bfloat16, numel=numel)
        t.zero_()
        return t

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
        return out_sum == 1 or (self.tp_idx if self.mesh is not None else self.ctx.rank) == 0

    def bias_grad_without_use(self, op, slot: str) -> bool:
        # On one axis the gradient reduction spans all ranks, so the zero gradients of the ranks that do not add the bias
        # and the full gradient of the one that does sum to the right value.  On a mesh, gradients are summed over the
        # data-parallel group only: the tensor-parallel peers never see each other's bias gradient, and each computes it.
        return self.mesh is not None and op.inputs.get(slot) is not None and not self.use_bias(op, slot)

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

    def set_inputs(self, inputs, labels=None):
        """As the single-device executor, plus: with `shard_inputs`, an input that is consumed through a sample-dimension
        Repartition may be given as this rank's piece only (or still as the whole tensor, of which the piece is taken)."""
        rest = dict(inputs)
        for name, op in self.direct_inputs.items():
            if name not in rest:
                continue
            src = rest.pop(name)
            dst = op.out().data
            if src.numel() != dst.numel():  # the whole tensor: keep this rank's piece
                full = list(dst.shape)
                full[op.dim] *= op.gctx.world_size
                src = src.reshape(full).narrow(op.dim, op.gctx.rank * op.piece, op.piece)
            dst.copy_(src.reshape(dst.shape) if src.numel() == dst.numel() and src.shape != dst.shape else src, non_blocking=True)
        super().set_inputs(rest, labels)

    def local_label_rows(self, labels, rows):
        flat = labels.reshape(-1) if self.cfg.loss == "sparse_categorical_crossentropy" else labels.reshape(-1, labels.shape[-1])
        if flat.shape[0] == rows:
            return flat
        r = self.dp_idx if self.mesh is not None else self.ctx.rank
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
        # sharded update inside the all-reduce: bf16 mixed precision, every bucket a multiple of 8 elements
        o = self.cfg.optimizer
        self.fused_update = bool(self.fuse_optimizer and self.buckets and self.shadow is not None and o.kind in ("adam", "sgd")
                                 and all((e - s) % 8 == 0 and s % 8 == 0 for s, e in self.buckets))

    # ------------------------------------------------------------------ step timeline (CUDA events, eager steps only)
    def enable_timeline(self):
        """Record CUDA events at the phase boundaries of the following eager steps and around every gradient bucket kernel;
        `timeline()` turns them into milliseconds.  Use with ``use_cuda_graph=False``."""
        self._tl = {"marks": [], "buckets": []}

    def _mark(self, name):
        tl = getattr(self, "_tl", None)
        if tl is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            tl["marks"].append((name, e))

    def timeline(self) -> dict:
        """Milliseconds, relative to the start of the last recorded step: phase boundaries on the main stream and
        (start, end, elements) of every bucket kernel on the side stream."""
        tl = getattr(self, "_tl", None)
        if not tl or not tl["marks"]:
            return {}
        torch.cuda.synchronize()
        starts = [i for i, (n, _) in enumerate(tl["marks"]) if n == "step_start"]
        marks = tl["marks"][starts[-1]:]
        t0 = marks[0][1]
        out = {"marks": [(n, t0.elapsed_time(e)) for n, e in marks]}
        out["buckets"] = [(t0.elapsed_time(a), t0.elapsed_time(b), n) for a, b, n in tl["buckets"] if t0.elapsed_time(a) >= 0]
        return out

    def forward(self):
        self._mark("step_start")
        super().forward()
        self._mark("forward_end")

    def compute_loss(self):
        r = super().compute_loss()
        self._mark("loss_end")
        return r

    def backward(self):
        if not getattr(self, "buckets", None):
            r = super().backward()
            self._mark("backward_end")
            return r
        main = torch.cuda.current_stream()
        for nid in reversed(self.order):
            op = self.ops[nid]
            if getattr(op, "has_grad", False):
                op.backward()
                for bi in self._launch_after.get(nid, ()):
                    self._launch_bucket(bi, main)
        for bi in self._launch_after.get(-1, ()):
            self._launch_bucket(bi, main)
        self._mark("backward_end")

    def _reduce_bucket(self, s, e):
        if self.fused_update:
            self.grad_ar.run_update(self.shadow_buf, self.master, self.opt_m, self.opt_v, self.cfg.optimizer,
                                    self.alpha_tensor.data_ptr(), scale=1.0, offset=s, n=e - s)
        else:
            self.grad_ar.run(scale=1.0, offset=s, n=e - s)

    def _launch_bucket(self, bi, main):
        s, e = self.buckets[bi]
        if self.side is not None:
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                tl = getattr(self, "_tl", None)
                if tl is not None:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                self._reduce_bucket(s, e)
                if tl is not None:
                    b.record()
                    tl["buckets"].append((a, b, e - s))
            self._pending = True
        else:
            self._reduce_bucket(s, e)

    def update(self, start: int = 0):
        # replicated parameters were updated (sharded over ranks) by the bucket kernels
        super().update(self.rep_numel if getattr(self, "fused_update", False) else start)
        self._mark("update_end")

    def consolidate_state(self):
        """With the sharded update every rank holds current fp32 master weights and moments only for the slices it
        owns; this gathers them so that every rank (and a checkpoint) has the whole state again."""
        if not getattr(self, "fused_update", False):
            return
        for t in (self.master, self.opt_m, self.opt_v):
            if t is None:
                continue
            keep = torch.zeros_like(t[:self.rep_numel])
            for s, e in self.buckets:
                a, b = self.grad_ar.owned_ranges(s, e - s)
                keep[a:b] = t[a:b]
            dist.all_reduce(keep, group=self.ctx_dp.group)
            t[:self.rep_numel].copy_(keep)

    def state_dict(self):
        self.consolidate_state()
        return super().state_dict()

    def named_parameters(self):
        """fp32 master weights by name.  A collective when the update is sharded (every rank must call it): the
        slices other ranks own are gathered first."""
        self.consolidate_state()
        return super().named_parameters()

    def sync_gradients(self):
        if self.side is not None and self._pending:
            torch.cuda.current_stream().wait_stream(self.side)
            self._pending = False
        self._mark("gradients_synced")

    def _describe(self) -> str:
        W = self.ctx.world_size
        if self.mesh is not None:
            return f"dp{self.mesh[0]}xtp{self.mesh[1]}"
        kinds = set()
        for n in self.nodes.values():
            if n["type"] in ("LINEAR", "MULTIHEAD_ATTENTION", "CONV2D", "EMBEDDING"):
                sh = n["outputs"][0][1]
                if sh.sum_degree > 1 or (sh.degrees and sh.degrees[-1] > 1):
                    kinds.add("tp")
                elif sh.degrees and sh.degrees[0] > 1:
                    kinds.add("dp")
        if getattr(self, "table_groups", None):
            kinds.add("tables_mp")
        if not kinds:
            return f"replicated{W}"
        return "+".join(f"{k}{W}" for k in sorted(kinds))

    def mean_loss(self) -> float:
        """Mean loss over the global batch (sums the local rows over ranks when the loss is batch-sharded)."""
        s = self.loss_rows.sum().reshape(1).to(torch.float64)
        sharded = self.global_loss_rows(1, self.graph.shape(self.loss_value)) > 1
        if sharded:  # on a mesh the rows are split over the data-parallel group only
            dist.all_reduce(s, group=self.ctx_dp.group)
        return float(s.item() * self.loss_scale)
