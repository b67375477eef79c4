"""Fused compute + collective operators over NVLink peer memory.

The PCG patterns they implement (none of which the reference can execute -- its parallel operators have no
device implementation, lib/op-attrs/src/op-attrs/computation_graph_op_attrs.cc:24-33):

  F1  row-parallel Linear -> Reduction          GemmReduceScatter  (tcgen05 GEMM whose epilogue writes each
                                                 output tile straight into the owning rank's stage, then a
                                                 flag-gated reduction of the staged partial sums)
  F2  Combine -> column-parallel Linear          AllGatherGemm      (peers push their row shards into a local
                                                 staging buffer; the GEMM starts on the local shard and its TMA
                                                 producer waits per row block for the pushed data)
  F3  Replicate backward on weights              GradAllReduce      (two-shot all-reduce fused with the scale,
                                                 in place on the gradient arena, launched on a side stream)
  F4  Repartition around model-parallel tables   AllToAllEmbedding  (gather from local tables directly into the
                                                 sample owners' buffers; backward pulls and applies sparse SGD)

TMA never reads peer memory here: remote data is first written into this GPU's own memory by the peer.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from ..ops import kernels as K
from . import comm
from .context import DistContext


class GradAllReduce:
    """F3.  The gradient arena lives in symmetric memory; ``run`` sums it over ranks and scales it in place."""

    def __init__(self, ctx: DistContext, numel: int, dtype=torch.bfloat16, blocks: int = 48):
        self.ctx = ctx
        self.dtype = dtype
        es = torch.empty((), dtype=dtype).element_size()
        self.buf = ctx.symmetric(numel * es)
        self.tensor = self.buf.view(dtype, numel=numel)
        self.numel = numel
        self.flag_base = ctx.alloc_flags(ctx.world_size)
        self.sync = ctx.new_sync()
        self.blocks = blocks

    def run(self, scale: float = 1.0, offset: int = 0, n: Optional[int] = None):
        n = self.numel - offset if n is None else n
        comm.grad_allreduce_scale(self.ctx, self.buf, offset, n, scale, self.dtype, self.flag_base, self.sync, self.blocks)


    def run_update(self, shadow, master, m, v, opt, alpha_ptr, scale: float = 1.0, offset: int = 0, n: Optional[int] = None):
        """Sharded-update form: reduce-scatter the gradients, update the owned slice of the fp32 state, all-gather
        the new bf16 weights into every rank's `shadow` (a SymmetricBuffer).  The gradient arena is left partly
        reduced (each rank holds nothing useful in it afterwards)."""
        n = self.numel - offset if n is None else n
        comm.grad_allreduce_update(self.ctx, self.buf, shadow, master, m, v, offset, n, scale, opt, alpha_ptr, self.flag_base, self.sync,
                                   self.blocks)

    def owned_ranges(self, offset: int, n: int):
        """[start, end) element range of [offset, offset+n) whose optimizer state this rank owns under run_update."""
        nvec = n // 8
        per = (nvec + self.ctx.world_size - 1) // self.ctx.world_size
        v0, v1 = per * self.ctx.rank, min(nvec, per * (self.ctx.rank + 1))
        return offset + v0 * 8, offset + max(v1, v0) * 8


class PeerAllGather:
    """All-gather of equal shards over peer memory (the stand-alone Combine, and Repartition's backward): every rank
    copies its shard into slot `rank` of every peer's staging buffer with plain stores over NVLink.  The result
    ``gathered`` ([world, shard elements]) lives in the staging buffer until the next call.  Two flag barriers frame the
    copy: the first keeps a fast rank from overwriting a buffer a peer is still reading from the previous call, the second
    tells every rank that all shards have landed.  No library call, so a plan built from these stays one CUDA graph."""

    def __init__(self, ctx: DistContext, shard_numel: int, dtype=torch.bfloat16):
        es = torch.empty((), dtype=dtype).element_size()
        if (shard_numel * es) % 16 != 0:
            raise ValueError("a shard must be a multiple of 16 bytes")
        self.ctx, self.n, self.dtype = ctx, shard_numel, dtype
        self.shard_bytes = shard_numel * es
        self.stage = ctx.symmetric(ctx.world_size * self.shard_bytes)
        self.gathered = self.stage.view(dtype, shape=(ctx.world_size, shard_numel), numel=ctx.world_size * shard_numel)
        self.flag_base = ctx.alloc_flags(ctx.world_size)
        self.bar_pre, self.bar_post = ctx.alloc_flags(ctx.world_size), ctx.alloc_flags(ctx.world_size)
        self.sync_push, self.sync_pre, self.sync_post = ctx.new_sync(), ctx.new_sync(), ctx.new_sync()

    def __call__(self, shard: torch.Tensor) -> torch.Tensor:
        ctx = self.ctx
        if shard.numel() != self.n or shard.dtype != self.dtype or not shard.is_contiguous():
            raise ValueError("shard does not match the buffer this all-gather was built for")
        comm.barrier(ctx, self.bar_pre, self.sync_pre)
        comm.push_rows(ctx, shard, self.stage, ctx.rank * self.shard_bytes, self.flag_base, self.sync_push)
        comm.barrier(ctx, self.bar_post, self.sync_post)
        return self.gathered


class PeerReduceScatter:
    """Reduce-scatter over peer memory (Reduction -> Repartition without a GEMM to fuse into, and the backward of
    Combine -> Replicate): piece p of this rank's partial sums goes into slot `rank` of peer p's staging buffer; every
    rank then sums the `world` slots it received (the kernel waits for the senders' flags itself)."""

    def __init__(self, ctx: DistContext, piece_numel: int, dtype=torch.bfloat16):
        es = torch.empty((), dtype=dtype).element_size()
        if (piece_numel * es) % 16 != 0 or piece_numel % 8 != 0:
            raise ValueError("a piece must be a multiple of 8 elements and of 16 bytes")
        self.ctx, self.n, self.dtype = ctx, piece_numel, dtype
        self.piece_bytes = piece_numel * es
        self.stage = ctx.symmetric(ctx.world_size * self.piece_bytes)
        self.stage_t = self.stage.view(dtype, numel=ctx.world_size * piece_numel)
        self.flag_base = ctx.alloc_flags(ctx.world_size)
        self.bar_base = ctx.alloc_flags(ctx.world_size)
        self.sync_send, self.sync_red, self.sync_bar = ctx.new_sync(), ctx.new_sync(), ctx.new_sync()

    def __call__(self, full: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
        """out[piece] (+)= sum over ranks of their full[rank * piece : (rank + 1) * piece]."""
        ctx = self.ctx
        if full.numel() != ctx.world_size * self.n or out.numel() != self.n or full.dtype != self.dtype or out.dtype != self.dtype:
            raise ValueError("operands do not match the buffer this reduce-scatter was built for")
        comm.barrier(ctx, self.bar_base, self.sync_bar)   # peers may still be summing the previous call's pieces
        comm.scatter_pieces(ctx, full, self.stage, self.piece_bytes, self.flag_base, self.sync_send)
        comm.reduce_partials(ctx, self.stage_t, out, ctx.world_size, self.flag_base, self.sync_red, residual=out if accumulate else None)
        return out


class GemmReduceScatter:
    """F1.  y_shard[rows/world, N] = sum_over_ranks( x_r[rows, K_r] @ w_r[N, K_r]^T )  (+ residual shard)."""

    def __init__(self, ctx: DistContext, rows: int, n: int, dtype=torch.bfloat16):
        w = ctx.world_size
        if rows % (128 * w) != 0:
            raise ValueError("rows must be a multiple of 128 * world_size for the scatter epilogue")
        self.ctx, self.rows, self.n, self.dtype = ctx, rows, n, dtype
        self.rows_per = rows // w
        es = torch.empty((), dtype=dtype).element_size()
        self.stage = ctx.symmetric(w * self.rows_per * n * es)       # [src][rows_per][n] on every rank
        self.stage_t = self.stage.view(dtype, numel=w * self.rows_per * n)
        self.flag_base = ctx.alloc_flags(w)
        self.bar_base = ctx.alloc_flags(w)
        self.sync_sig, self.sync_red, self.sync_bar = ctx.new_sync(), ctx.new_sync(), ctx.new_sync()

    def __call__(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, residual: Optional[torch.Tensor] = None, bias=None,
                 w_kn: bool = False):
        """`w` is [N, K] (K-major, a Linear weight) or, with ``w_kn``, [K, N] (the same weight used transposed, as
        in a data-gradient GEMM).  `bias` (length N) is added by the GEMM epilogue of the calling rank only --
        pass it on one rank.  `residual` [rows/world, N] is added to the reduced shard."""
        ctx = self.ctx
        rows, k = x.shape
        # peers may still be reducing the previous call's partials out of their stages
        comm.barrier(ctx, self.bar_base, self.sync_bar)
        K.gemm_raw(M=rows, N=self.n, K=k, A=x.data_ptr(), lda=k, B=w.data_ptr(), ldb=self.n if w_kn else k, b_mn=w_kn,
                   C=self.stage.local_ptr, ldc=self.n, bias=None if bias is None else bias.data_ptr(),
                   scatter=self.stage.peer_ptrs, scatter_rows=self.rows_per, scatter_src=ctx.rank)
        comm.signal(ctx, self.stage, self.flag_base, self.sync_sig)
        comm.reduce_partials(ctx, self.stage_t, out, ctx.world_size, self.flag_base, self.sync_red, residual=residual)
        return out


class AllGatherGemm:
    """F2.  y[world*rows_local, N] = allgather(x_local)[world*rows_local, K] @ w[N, K]^T (+bias, activation)."""

    def __init__(self, ctx: DistContext, rows_local: int, k: int, dtype=torch.bfloat16, overlap: bool = True):
        if rows_local % 128 != 0:
            raise ValueError("rows_local must be a multiple of 128")
        w = ctx.world_size
        self.ctx, self.rows_local, self.k, self.dtype = ctx, rows_local, k, dtype
        es = torch.empty((), dtype=dtype).element_size()
        self.shard_bytes = rows_local * k * es
        self.gathered = ctx.symmetric(w * self.shard_bytes)
        self.gathered_t = self.gathered.view(dtype, shape=(w * rows_local, k), numel=w * rows_local * k)
        self.flag_base = ctx.alloc_flags(w)
        self.bar_base = ctx.alloc_flags(w)
        self.sync_push, self.sync_gate, self.sync_bar = ctx.new_sync(), ctx.new_sync(), ctx.new_sync()

    def __call__(self, x_local: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias=None, act=None, pre_act_out=None,
                 w_kn: bool = False, accumulate: bool = False, dropout=None):
        """`w` is [N, K] or, with ``w_kn``, [K, N].  After the call ``gathered_t`` holds the gathered operand
        (all ranks' row shards in rank order), which backward passes reuse."""
        ctx = self.ctx
        W = ctx.world_size
        n = w.shape[1] if w_kn else w.shape[0]
        # nobody may overwrite a staging buffer that a peer's previous GEMM might still be reading
        comm.barrier(ctx, self.bar_base, self.sync_bar)
        es = x_local.element_size()
        if self.k * es % 16 != 0:
            raise ValueError("row size must be a multiple of 16 bytes")
        flag_ptrs = [p + (self.flag_base + ctx.rank) * 8 for p in ctx.flags.peer_ptrs]
        # one kernel: two warps of every CTA push the local shard to the peers while the rest start on the local rows
        K.gemm_raw(M=W * self.rows_local, N=n, K=self.k, A=self.gathered.local_ptr, lda=self.k, B=w.data_ptr(),
                   ldb=n if w_kn else self.k, b_mn=w_kn, C=out.data_ptr(), ldc=n, accumulate=accumulate,
                   out_fp32=out.dtype == torch.float32, bias=None if bias is None else bias.data_ptr(),
                   act=K.ACT_CODES[act] if not isinstance(act, int) else act,
                   C2=None if pre_act_out is None else pre_act_out.data_ptr(),
                   gate_flags=ctx.flags.local_ptr + self.flag_base * 8, gate_sync=self.sync_gate.data_ptr(),
                   gate_rows=self.rows_local, mb_rotate=ctx.rank * (self.rows_local // 128), dropout=dropout,
                   push=dict(src=x_local.data_ptr(), nbytes=self.shard_bytes, dst_offset=ctx.rank * self.shard_bytes,
                             dst=self.gathered.peer_ptrs, flag=flag_ptrs, sync=self.sync_push.data_ptr(), world=W, rank=ctx.rank))
        return out


class AllToAllEmbedding:
    """F4.  Tables are model-parallel (table t lives on rank t % world), samples are data-parallel.

    forward(idx_global [global_batch, num_tables]) fills out_local [local_batch, num_tables, dim] on every rank:
    each rank gathers, for *all* samples, the rows of its own tables and writes them into the owners' buffers.
    backward pulls d(out) rows from the owners and applies the sparse SGD update to the local tables."""

    def __init__(self, ctx: DistContext, tables: List[torch.Tensor], num_tables: int, dim: int, local_batch: int, out_dtype=torch.bfloat16):
        self.ctx, self.num_tables, self.dim, self.local_batch = ctx, num_tables, dim, local_batch
        self.tables = tables  # local fp32 tables, in local order (global table id = i * world + rank)
        dev = ctx.device
        self.table_ptrs = torch.tensor([t.data_ptr() for t in tables], dtype=torch.int64, device=dev)
        self.entries = torch.tensor([t.shape[0] for t in tables], dtype=torch.int64, device=dev)
        es = torch.empty((), dtype=out_dtype).element_size()
        self.out_dtype = out_dtype
        nbytes = local_batch * num_tables * dim * es
        self.out = ctx.symmetric(nbytes)
        self.dout = ctx.symmetric(nbytes)
        self.out_t = self.out.view(out_dtype, shape=(local_batch, num_tables, dim), numel=local_batch * num_tables * dim)
        self.dout_t = self.dout.view(out_dtype, shape=(local_batch, num_tables, dim), numel=local_batch * num_tables * dim)
        self.bar_base = ctx.alloc_flags(ctx.world_size)
        self.sync_bar = ctx.new_sync()

    def forward(self, idx_global: torch.Tensor) -> torch.Tensor:
        ctx = self.ctx
        gb = idx_global.shape[0]
        lib = comm._lib()
        comm.barrier(ctx, self.bar_base, self.sync_bar)   # previous consumers of `out` are done everywhere
        comm._chk(lib.ffk_alltoall_embedding_fwd(self.table_ptrs.data_ptr(), self.entries.data_ptr(), idx_global.data_ptr(),
                                                 self.out.ptr_array, gb, self.local_batch, self.num_tables, self.dim, ctx.rank,
                                                 ctx.world_size, K.DT_BF16 if self.out_dtype == torch.bfloat16 else K.DT_F32,
                                                 K._DT[idx_global.dtype], comm._stream()), "ffk_alltoall_embedding_fwd")
        comm.barrier(ctx, self.bar_base, self.sync_bar)   # all rows have landed
        return self.out_t

    def backward_sgd(self, idx_global: torch.Tensor, lr: float):
        """dout_t must hold d(loss)/d(out) of the local samples before the call."""
        ctx = self.ctx
        gb = idx_global.shape[0]
        lib = comm._lib()
        comm.barrier(ctx, self.bar_base, self.sync_bar)   # every rank's dout is complete
        comm._chk(lib.ffk_alltoall_embedding_bwd(self.table_ptrs.data_ptr(), None, self.entries.data_ptr(), idx_global.data_ptr(),
                                                 self.dout.ptr_array, gb, self.local_batch, self.num_tables, self.dim, ctx.rank,
                                                 ctx.world_size, lr, K.DT_BF16 if self.out_dtype == torch.bfloat16 else K.DT_F32,
                                                 K._DT[idx_global.dtype], comm._stream()), "ffk_alltoall_embedding_bwd")
        comm.barrier(ctx, self.bar_base, self.sync_bar)   # peers finished reading my dout
