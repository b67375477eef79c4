"""Python bindings of the NVLink peer-memory collectives (csrc/kernels/comm_kernels.cu) and the NCCL baseline.

The fused operators built from these live in ``fused_ops.py``; the distributed executor uses both.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K
from .context import DistContext, SymmetricBuffer

_declared = [False]


def _lib():
    l = K.lib()
    if not _declared[0]:
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        PP = ctypes.POINTER(c_void_p)
        sig = {
            "ffk_comm_barrier": [PP, I, I, I, P, P, P],
            "ffk_grad_allreduce_scale": [PP, PP, I, L, L, F, I, I, P, P, I, I, P],
            "ffk_grad_allreduce_update": [PP, PP, P, P, P, PP, I, L, L, F, I, I, P, P, I, F, P, F, F, F, F, F, I, I, P],
            "ffk_push_rows": [P, PP, L, L, PP, I, I, I, P, I, I, P],
            "ffk_scatter_pieces": [P, PP, L, PP, I, I, I, P, I, P],
            "ffk_reduce_partials": [P, P, P, L, I, P, I, P, P, I, I, P],
            "ffk_alltoall_embedding_fwd": [P, P, P, PP, I, I, I, I, I, I, I, I, P],
            "ffk_alltoall_embedding_bwd": [P, P, P, P, PP, I, I, I, I, I, I, F, I, I, P],
        }
        for name, args in sig.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = c_int
        _declared[0] = True
    return l


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _chk(rc, what):
    K._LAUNCHES[0] += 1
    if rc != 0:
        raise K.KernelError(f"{what} failed with code {rc}")


def barrier(ctx: DistContext, flag_base: int, sync: torch.Tensor):
    """Device-side barrier over all ranks (no host synchronisation)."""
    _chk(_lib().ffk_comm_barrier(ctx.flags.ptr_array, flag_base, ctx.rank, ctx.world_size, sync.data_ptr(),
                                 ctx.status.data_ptr(), _stream()), "ffk_comm_barrier")


def grad_allreduce_scale(ctx: DistContext, buf: SymmetricBuffer, offset_elems: int, n: int, scale: float, dtype,
                         flag_base: int, sync: torch.Tensor, blocks: int = 32):
    """In-place sum over ranks of buf[offset : offset+n] times scale (two-shot over peer memory)."""
    dt = K.DT_BF16 if dtype == torch.bfloat16 else K.DT_F32
    _chk(_lib().ffk_grad_allreduce_scale(buf.ptr_array, ctx.flags.ptr_array, flag_base, offset_elems, n, scale, ctx.rank,
                                         ctx.world_size, sync.data_ptr(), ctx.status.data_ptr(), dt, blocks, _stream()),
         "ffk_grad_allreduce_scale")


def grad_allreduce_update(ctx: DistContext, grads: SymmetricBuffer, shadow: SymmetricBuffer, master, m, v, offset_elems: int, n: int,
                          scale: float, opt, alpha_ptr, flag_base: int, sync: torch.Tensor, blocks: int = 32):
    """Reduce-scatter grads[offset : offset+n], apply the optimizer to the owned slice of master/m/v and write the new
    bf16 weights into every rank's `shadow`.  `opt` is an OptimizerConfig; offset and n are multiples of 8."""
    kind = 0 if opt.kind == "adam" else 1
    mp = m.data_ptr() if m is not None else None
    vp = v.data_ptr() if v is not None else None
    _chk(_lib().ffk_grad_allreduce_update(grads.ptr_array, shadow.ptr_array, master.data_ptr(), mp, vp, ctx.flags.ptr_array, flag_base,
                                          offset_elems, n, scale, ctx.rank, ctx.world_size, sync.data_ptr(), ctx.status.data_ptr(), kind,
                                          opt.lr, alpha_ptr, opt.beta1, opt.beta2, opt.epsilon, opt.weight_decay, opt.momentum,
                                          int(opt.nesterov), blocks, _stream()), "ffk_grad_allreduce_update")


def push_rows(ctx: DistContext, src: torch.Tensor, dst: SymmetricBuffer, dst_byte_offset: int, flag_base: int,
              sync: torch.Tensor, skip_self: bool = False, blocks: int = 32, nbytes: Optional[int] = None):
    """Copy src into every peer's `dst` at dst_byte_offset and raise flag[flag_base + rank] there."""
    nb = src.numel() * src.element_size() if nbytes is None else nbytes
    _chk(_lib().ffk_push_rows(src.data_ptr(), dst.ptr_array, dst_byte_offset, nb, ctx.flags.ptr_array, flag_base, ctx.rank,
                              ctx.world_size, sync.data_ptr(), int(skip_self), blocks, _stream()), "ffk_push_rows")


def scatter_pieces(ctx: DistContext, src: torch.Tensor, dst: SymmetricBuffer, piece_bytes: int, flag_base: int, sync: torch.Tensor,
                   blocks: int = 32):
    """Piece p of `src` (world pieces of piece_bytes) goes into slot `rank` of peer p's `dst` ([world][piece]); then
    flag[flag_base + rank] is raised on every peer."""
    _chk(_lib().ffk_scatter_pieces(src.data_ptr(), dst.ptr_array, piece_bytes, ctx.flags.ptr_array, flag_base, ctx.rank, ctx.world_size,
                                   sync.data_ptr(), blocks, _stream()), "ffk_scatter_pieces")


def signal(ctx: DistContext, dst: SymmetricBuffer, flag_base: int, sync: torch.Tensor):
    """Raise flag[flag_base + rank] on every peer without moving data (orders after prior work on the stream)."""
    _chk(_lib().ffk_push_rows(dst.local_ptr, dst.ptr_array, 0, 0, ctx.flags.ptr_array, flag_base, ctx.rank, ctx.world_size,
                              sync.data_ptr(), 0, 1, _stream()), "ffk_push_rows(signal)")


def reduce_partials(ctx: DistContext, stage: torch.Tensor, out: torch.Tensor, nsrc: int, flag_base: int, sync: torch.Tensor,
                    residual: Optional[torch.Tensor] = None):
    """out = sum over the nsrc staged partial copies (+ residual), after all nsrc source flags arrived."""
    n = out.numel()
    _chk(_lib().ffk_reduce_partials(stage.data_ptr(), None if residual is None else residual.data_ptr(), out.data_ptr(), n, nsrc,
                                    ctx.flags.local_ptr, flag_base, sync.data_ptr(), ctx.status.data_ptr(),
                                    K.DT_BF16 if out.dtype == torch.bfloat16 else K.DT_F32, 0, _stream()), "ffk_reduce_partials")


# --------------------------------------------------------------------------- NCCL baseline collectives
def nccl_all_reduce(t: torch.Tensor, group=None):
    dist.all_reduce(t, group=group)
    return t


def nccl_all_gather_dim(t: torch.Tensor, dim: int, world: int, group=None, out: Optional[torch.Tensor] = None):
    """All-gather along `dim` (materialised contiguously)."""
    parts = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(parts.view(-1), t.contiguous().view(-1), group=group)
    if dim == 0:
        res = parts.view((world * t.shape[0],) + tuple(t.shape[1:]))
    else:
        # [w, d0, .., dk, ..] -> [d0, .., w, dk, ..] -> merge
        perm = list(range(1, dim + 1)) + [0] + list(range(dim + 1, t.dim() + 1))
        res = K.permute(parts, perm).view(tuple(t.shape[:dim]) + (world * t.shape[dim],) + tuple(t.shape[dim + 1:]))
    if out is not None:
        out.copy_(res)
        return out
    return res
