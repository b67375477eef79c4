"""ctypes bindings of the sm_100a kernel library (``libffk.so``).

Every function here takes torch CUDA tensors, checks what the kernel cannot
check for itself (dtype, contiguity, device) and launches on the current torch
stream.  Nothing falls back to a torch op: if the shared object is missing the
import of the library raises, so a GPU run can never silently use another path.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_LIB_PATH = os.path.join(_PKG_DIR, "libffk.so")
_lib = None

# dtype codes of the C API
DT_F32, DT_BF16, DT_I32, DT_I64, DT_F16, DT_BOOL, DT_F64 = range(7)
_DT = {
    torch.float32: DT_F32, torch.bfloat16: DT_BF16, torch.int32: DT_I32, torch.int64: DT_I64,
    torch.float16: DT_F16, torch.bool: DT_BOOL, torch.float64: DT_F64,
}
ACT_NONE, ACT_RELU, ACT_GELU, ACT_SIGMOID, ACT_TANH = range(5)
ACT_CODES = {None: 0, "none": 0, "relu": 1, "gelu": 2, "sigmoid": 3, "tanh": 4}

UNARY_OPS = {
    "identity": 0, "relu": 1, "sigmoid": 2, "tanh": 3, "elu": 4, "gelu": 5, "exp": 6, "rsqrt": 7, "sin": 8,
    "cos": 9, "scalar_multiply": 10, "scalar_add": 11, "scalar_sub": 12, "scalar_truediv": 13, "pow": 14,
    "log": 15, "sqrt": 16, "neg": 17,
}
BINARY_OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4, "min": 5}
LOSS_KINDS = {"sparse_categorical_crossentropy": 0, "categorical_crossentropy": 1,
              "mean_squared_error_avg_reduce": 2, "identity": 3, "mean_squared_error_sum_reduce": 4}


class KernelError(RuntimeError):
    pass


class GemmDesc(ctypes.Structure):
    _fields_ = [
        ("M", c_int), ("N", c_int), ("K", c_int), ("nh", c_int), ("nb", c_int), ("es", c_int),
        ("a_mn", c_int), ("b_mn", c_int),
        ("A", c_void_p), ("lda", c_longlong), ("a_sh", c_longlong), ("a_sb", c_longlong),
        ("B", c_void_p), ("ldb", c_longlong), ("b_sh", c_longlong), ("b_sb", c_longlong),
        ("C", c_void_p), ("ldc", c_longlong), ("c_sh", c_longlong), ("c_sb", c_longlong),
        ("C2", c_void_p), ("bias", c_void_p), ("addend", c_void_p),
        ("ld_add", c_longlong), ("add_sh", c_longlong), ("add_sb", c_longlong),
        ("alpha", c_float), ("act", c_int), ("out_fp32", c_int), ("accumulate", c_int),
        ("bn", c_int), ("max_ctas", c_int),
        # fused collectives (see gemm_sm100.cu): scatter epilogue and gated A operand
        ("scatter", c_void_p * 8), ("scatter_rows", c_int), ("scatter_src", c_int),
        ("gate_flags", c_void_p), ("gate_sync", c_void_p), ("gate_rows", c_int), ("mb_rotate", c_int),
        # in-kernel push of this rank's shard to the peers' staging buffers (all-gather -> GEMM)
        ("push_src", c_void_p), ("push_bytes", c_longlong), ("push_dst_offset", c_longlong), ("push_dst", c_void_p * 8),
        ("push_flag", c_void_p * 8), ("push_sync", c_void_p), ("push_world", c_int), ("push_rank", c_int),
        # dropout applied by the epilogue after the activation
        ("drop_p", c_float), ("drop_salt", c_ulonglong), ("drop_seed_ptr", c_void_p),
    ]


class AttnDesc(ctypes.Structure):
    _fields_ = [
        ("B", c_int), ("H", c_int), ("Sq", c_int), ("Sk", c_int), ("D", c_int), ("scale", c_float), ("causal", c_int),
        ("drop_p", c_float), ("drop_salt", c_ulonglong), ("drop_seed_ptr", c_void_p),
        ("Q", c_void_p), ("ldq", c_longlong), ("K", c_void_p), ("ldk", c_longlong), ("V", c_void_p), ("ldv", c_longlong),
        ("O", c_void_p), ("ldo", c_longlong), ("lse", c_void_p),
        ("dO", c_void_p), ("lddo", c_longlong), ("delta", c_void_p),
        ("dQ", c_void_p), ("lddq", c_longlong), ("dK", c_void_p), ("lddk", c_longlong), ("dV", c_void_p), ("lddv", c_longlong),
        ("acc", c_void_p),
    ]


class ConvDesc(ctypes.Structure):
    _fields_ = [
        ("N", c_int), ("H", c_int), ("W", c_int), ("C", c_int), ("OC", c_int), ("KH", c_int), ("KW", c_int),
        ("pad_h", c_int), ("pad_w", c_int), ("OH", c_int), ("OW", c_int),
        ("x", c_void_p), ("wp", c_void_p), ("ldw", c_longlong), ("y", c_void_p), ("pre", c_void_p), ("bias", c_void_p), ("act", c_int),
        ("dy", c_void_p), ("dx", c_void_p), ("accumulate", c_int), ("dwp", c_void_p),
    ]


def available() -> bool:
    return os.path.exists(_LIB_PATH)


def lib():
    """The loaded kernel library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise KernelError(
                f"{_LIB_PATH} is missing: run `python build.py` (nvcc, sm_100a) before using the GPU path")
        _lib = ctypes.CDLL(_LIB_PATH)
        _declare(_lib)
        # epilogue through TMA stores: FFK_TMA_STORE=1/0 overrides the library default
        if os.environ.get("FFK_CTA_PAIRS") in ("0", "1"):
            _lib.ffk_gemm_set_cta_pairs(int(os.environ["FFK_CTA_PAIRS"]))
        if os.environ.get("FFK_TMA_STORE") in ("0", "1"):
            _lib.ffk_gemm_set_tma_store(int(os.environ["FFK_TMA_STORE"]))
    return _lib


def _declare(l):
    P, I, L, F, S = c_void_p, c_int, c_longlong, c_float, c_void_p
    sig = {
        "ffk_gemm": [ctypes.POINTER(GemmDesc), S],
        "ffk_gemm_last_error": [],
        "ffk_attention_fwd": [ctypes.POINTER(AttnDesc), S],
        "ffk_attention_bwd": [ctypes.POINTER(AttnDesc), S],
        "ffk_attention_last_error": [],
        "ffk_attention_supported": [I, I],
        "ffk_conv_fprop": [ctypes.POINTER(ConvDesc), S],
        "ffk_conv_dgrad": [ctypes.POINTER(ConvDesc), S],
        "ffk_conv_wgrad": [ctypes.POINTER(ConvDesc), S],
        "ffk_conv_implicit_supported": [I, I, I, I],
        "ffk_conv_last_error": [],
        "ffk_unary_fwd": [I, P, P, L, F, I, S],
        "ffk_unary_bwd": [I, P, P, P, P, L, F, I, I, S],
        "ffk_binary_fwd": [I, P, P, P, L, L, I, S],
        "ffk_binary_bwd": [I, P, P, P, P, P, L, I, I, S],
        "ffk_dropout": [P, P, P, L, F, c_ulonglong, P, I, S],
        "ffk_axpby": [P, P, L, F, F, I, S],
        "ffk_fill": [P, L, F, I, S],
        "ffk_cast": [P, I, P, I, L, I, S],
        "ffk_bias_act_bwd": [P, P, P, P, P, I, I, I, I, I, S],
        "ffk_layernorm_fwd": [P, P, P, P, P, P, P, P, I, I, F, I, S],
        "ffk_layernorm_bwd": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, S],
        "ffk_softmax_fwd": [P, P, I, I, F, I, I, S],
        "ffk_softmax_bwd": [P, P, P, I, I, F, I, S],
        "ffk_softmax_ce": [P, P, P, P, P, I, I, F, I, I, S],
        "ffk_loss_bwd": [I, P, P, P, L, I, F, I, I, S],
        "ffk_loss_fwd": [I, P, P, P, I, I, I, I, S],
        "ffk_adam_update": [P, P, P, P, P, L, F, F, F, F, F, F, P, I, S],
        "ffk_sgd_update": [P, P, P, P, L, F, F, I, F, F, I, S],
        "ffk_embedding_fwd": [P, P, P, L, I, I, L, I, I, I, I, S],
        "ffk_embedding_bwd": [P, P, P, L, I, I, L, I, I, I, I, S],
        "ffk_embedding_sgd": [P, P, P, L, I, I, L, F, I, I, S],
    }
    for name, args in sig.items():
        if hasattr(l, name):
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = c_int
    if hasattr(l, "ffk_attention_bwd_scratch_floats"):
        l.ffk_attention_bwd_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
        l.ffk_attention_bwd_scratch_floats.restype = c_longlong
    for name in ("ffk_bias_act_bwd_scratch", "ffk_layernorm_bwd_scratch"):
        if hasattr(l, name):
            fn = getattr(l, name)
            fn.argtypes = [c_int, c_int]
            fn.restype = c_longlong


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_LAUNCHES = [0]


def launch_count() -> int:
    """Number of kernel-library calls issued so far by this process (each is at least one launch)."""
    return _LAUNCHES[0]


def _check(code: int, what: str):
    _LAUNCHES[0] += 1
    if code != 0:
        raise KernelError(f"{what} failed with code {code}")


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}")


def _cuda_contig(*ts):
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError("kernel called with a CPU tensor")
        if not t.is_contiguous():
            raise KernelError("kernel called with a non-contiguous tensor")


# --------------------------------------------------------------------------- GEMM
_REPACK_SCRATCH = {}          # operand slot -> uint8 scratch (grows to the largest operand repacked so far)
_REPACK_RETIRED = []          # outgrown scratches stay allocated: a captured CUDA graph may still address them
_REPACK_MIN_FLOPS = 2.0e6     # below this the general-shape kernel is a single cheap launch anyway


def _tma_addressable(ptr, ld, sh, sb, nh, nb, es) -> bool:
    """TMA wants a 16-byte aligned base and pitches that are multiples of 16 bytes."""
    if ptr % 16 or (ld * es) % 16:
        return False
    return not ((nh > 1 and (sh * es) % 16) or (nb > 1 and (sb * es) % 16))


def _repack_operand(slot, ptr, ld, rows, cols, nh, sh, nb, sb, es):
    """Copy an operand whose rows TMA cannot address into a scratch with the pitch rounded up to 16 bytes.
    Returns (ptr, ld, sh, sb) of the copy, or None when the operand's batches are not evenly spaced rows.

    The scratch is per operand slot and reused by later calls on the same stream; the copy is one small strided
    kernel, after which odd feature counts (13 dense features, a 145-wide concatenation, a 9 x 9 interaction)
    run on the tensor cores instead of the general-shape kernel."""
    batches = max(nh, 1) * max(nb, 1)
    if batches > 1:
        if nh > 1 and nb > 1:
            if sh != rows * ld or sb != nh * sh:
                return None
        elif (nh > 1 and sh != rows * ld) or (nb > 1 and sb != rows * ld):
            return None
    pad = 16 // es
    ld2 = (cols + pad - 1) // pad * pad
    total_rows = batches * rows
    need = total_rows * ld2 * es
    dev = torch.cuda.current_device()
    buf = _REPACK_SCRATCH.get((slot, dev))
    if buf is None or buf.numel() < need:
        if buf is not None:
            _REPACK_RETIRED.append(buf)
        buf = torch.empty(max(need, 1 << 20, 2 * (buf.numel() if buf is not None else 0)), dtype=torch.uint8, device=f"cuda:{dev}")
        _REPACK_SCRATCH[(slot, dev)] = buf
    _check(_tlib().ffk_block_copy(ptr, ld, buf.data_ptr(), ld2, total_rows, cols, es, 0, 0, _stream()), "ffk_block_copy(repack)")
    return buf.data_ptr(), ld2, rows * ld2, (nh if nh > 1 else 1) * rows * ld2


def gemm_raw(*, M, N, K, A, lda, B, ldb, C, ldc, a_mn=False, b_mn=False, es=2, nh=1, nb=1,
             a_sh=0, a_sb=0, b_sh=0, b_sb=0, c_sh=0, c_sb=0, C2=None, bias=None, addend=None,
             ld_add=0, add_sh=0, add_sb=0, alpha=1.0, act=0, out_fp32=False, accumulate=False,
             bn=0, max_ctas=0, scatter=None, scatter_rows=0, scatter_src=0, gate_flags=None, gate_sync=None,
             gate_rows=0, mb_rotate=0, push=None, dropout=None):
    """D = epilogue(alpha * A[M,K] . B[N,K]^T) on raw pointers; see gemm_sm100.cu.

    scatter / scatter_rows / scatter_src: write each output tile into the owning rank's staging buffer
    (GEMM -> reduce-scatter).  gate_flags / gate_sync / gate_rows / mb_rotate: wait for pushed row blocks of A
    (all-gather -> GEMM)."""
    plain = not scatter and gate_flags is None and push is None and dropout is None
    # (batches of small problems have a kernel of their own that reads any layout: same condition as in ffk_gemm)
    small_batched = max(nh, 1) * max(nb, 1) >= 32 and M * N <= 1024 and (M + N) * (K + 1) <= 2304
    if plain and not small_batched and 2.0 * M * N * K * max(nh, 1) * max(nb, 1) >= _REPACK_MIN_FLOPS:
        if not _tma_addressable(A, lda, a_sh, a_sb, nh, nb, es):
            r = _repack_operand("A", A, lda, K if a_mn else M, M if a_mn else K, nh, a_sh, nb, a_sb, es)
            if r is not None:
                A, lda, a_sh, a_sb = r
        if not _tma_addressable(B, ldb, b_sh, b_sb, nh, nb, es):
            r = _repack_operand("B", B, ldb, K if b_mn else N, N if b_mn else K, nh, b_sh, nb, b_sb, es)
            if r is not None:
                B, ldb, b_sh, b_sb = r
    sc = (c_void_p * 8)(*([int(p) for p in scatter] + [None] * (8 - len(scatter)))) if scatter else (c_void_p * 8)()
    d = GemmDesc(M, N, K, nh, nb, es, int(a_mn), int(b_mn), A, lda, a_sh, a_sb, B, ldb, b_sh, b_sb,
                 C, ldc, c_sh, c_sb, C2, bias, addend, ld_add, add_sh, add_sb, alpha, act, int(out_fp32),
                 int(accumulate), bn, max_ctas, sc, scatter_rows, scatter_src, gate_flags, gate_sync, gate_rows,
                 mb_rotate)
    if dropout is not None:  # (p, salt, seed tensor or None)
        d.drop_p, d.drop_salt = float(dropout[0]), int(dropout[1]) & (2**64 - 1)
        d.drop_seed_ptr = None if dropout[2] is None else dropout[2].data_ptr()
    if push is not None:  # dict(src, nbytes, dst_offset, dst=[peer ptrs], flag=[peer flag ptrs], sync, world, rank)
        d.push_src, d.push_bytes, d.push_dst_offset = push["src"], push["nbytes"], push["dst_offset"]
        d.push_dst = (c_void_p * 8)(*([int(x) for x in push["dst"]] + [None] * (8 - len(push["dst"]))))
        d.push_flag = (c_void_p * 8)(*([int(x) for x in push["flag"]] + [None] * (8 - len(push["flag"]))))
        d.push_sync, d.push_world, d.push_rank = push["sync"], push["world"], push["rank"]
    _check(lib().ffk_gemm(ctypes.byref(d), _stream()), "ffk_gemm")


def gemm_last_error() -> int:
    return lib().ffk_gemm_last_error()


# --------------------------------------------------------------------------- fused attention
def attention_supported(head_dim: int, backward: bool = True) -> bool:
    """True when the fused attention kernels cover this head dimension (forward: 64 and 128; backward: 128)."""
    return bool(lib().ffk_attention_supported(int(head_dim), int(backward)))


def attention_bwd_scratch_floats(B, H, Sq, D) -> int:
    """fp32 elements of scratch `attention_bwd` needs (the dQ accumulator)."""
    return int(lib().ffk_attention_bwd_scratch_floats(B, H, Sq, D))


def attention_set_forward_variant(v: int):
    """Which forward kernel `attention_fwd` launches: 1 = one 128-query tile per CTA (default), 2 / 3 = two tiles per CTA
    sharing the K / V tiles, probabilities passed to the second product through shared (2) or tensor (3) memory."""
    lib().ffk_attention_set_fwd_variant(int(v))


def attention_last_error() -> int:
    return lib().ffk_attention_last_error()


def _attn_view(t, D, H):
    """A [B*S, >= H*D] bf16 matrix view (last dim contiguous) -> (pointer, leading dimension)."""
    if t.dtype != torch.bfloat16 or not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.shape[1] < H * D:
        raise KernelError("attention operands are 2-D bf16 CUDA matrices [batch*seq, heads*head_dim] with unit column stride")
    return t.data_ptr(), t.stride(0)


def _attn_desc(B, H, Sq, Sk, D, scale, causal, dropout):
    d = AttnDesc()
    d.B, d.H, d.Sq, d.Sk, d.D, d.scale, d.causal = B, H, Sq, Sk, D, float(scale), int(bool(causal))
    if dropout is not None and dropout[0] > 0:
        p, salt, seed = dropout
        d.drop_p, d.drop_salt, d.drop_seed_ptr = float(p), int(salt) & 0xFFFFFFFFFFFFFFFF, _p(seed)
    return d


def attention_fwd(q, k, v, out, lse, *, B, H, Sq, Sk, D, scale, causal=False, dropout=None):
    """out[b, q, h, :] = dropout(softmax(scale * q k^T)) v for every (batch, head); q / k / v / out are [B*S, ld] bf16
    matrices with head h in columns [h*D, (h+1)*D) (views into a packed QKV buffer are fine).  lse [B, H, Sq] fp32
    receives the row log-sum-exp (base 2, of the scaled scores) that `attention_bwd` needs.
    dropout = (p, salt, seed tensor or None)."""
    d = _attn_desc(B, H, Sq, Sk, D, scale, causal, dropout)
    d.Q, d.ldq = _attn_view(q, D, H)
    d.K, d.ldk = _attn_view(k, D, H)
    d.V, d.ldv = _attn_view(v, D, H)
    d.O, d.ldo = _attn_view(out, D, H)
    if lse.dtype != torch.float32 or lse.numel() < B * H * Sq or not lse.is_contiguous():
        raise KernelError("lse must be a contiguous fp32 tensor of B*H*Sq elements")
    d.lse = lse.data_ptr()
    _check(lib().ffk_attention_fwd(ctypes.byref(d), _stream()), "ffk_attention_fwd")
    return out


def attention_bwd(q, k, v, out, lse, dout, dq, dk, dv, delta, acc, *, B, H, Sq, Sk, D, scale, causal=False, dropout=None):
    """Gradients of `attention_fwd` with respect to q, k, v (same layouts).  delta: fp32 scratch of B*H*Sq elements;
    acc: fp32 scratch of attention_bwd_scratch_floats(B, H, Sq, D) elements."""
    d = _attn_desc(B, H, Sq, Sk, D, scale, causal, dropout)
    d.Q, d.ldq = _attn_view(q, D, H)
    d.K, d.ldk = _attn_view(k, D, H)
    d.V, d.ldv = _attn_view(v, D, H)
    d.O, d.ldo = _attn_view(out, D, H)
    d.dO, d.lddo = _attn_view(dout, D, H)
    d.dQ, d.lddq = _attn_view(dq, D, H)
    d.dK, d.lddk = _attn_view(dk, D, H)
    d.dV, d.lddv = _attn_view(dv, D, H)
    if delta.dtype != torch.float32 or delta.numel() < B * H * Sq or acc.dtype != torch.float32 or acc.numel() < B * H * Sq * D:
        raise KernelError("attention_bwd scratch too small")
    d.lse, d.delta, d.acc = lse.data_ptr(), delta.data_ptr(), acc.data_ptr()
    _check(lib().ffk_attention_bwd(ctypes.byref(d), _stream()), "ffk_attention_bwd")


def attention_keep_mask(B, H, Sq, Sk, p, salt, seed=None, device="cpu"):
    """The dropout keep mask [B, H, Sq, Sk] (bool) the fused attention kernels draw: a host restatement of their
    counter-based generator (csrc/kernels/attention_sm100.cu: attn_row_mix / attn_group_word), for tests and debugging."""
    M64, M32 = (1 << 64) - 1, (1 << 32) - 1
    sd = int(salt) & M64
    if seed is not None:
        sd = (sd * 0x9E3779B97F4A7C15 + int(seed)) & M64
    s0, s1 = sd & M32, sd >> 32
    groups = (Sk + 3) // 4
    rows = torch.arange(B * H * Sq, dtype=torch.int64, device=device)[:, None]
    g = torch.arange(groups, dtype=torch.int64, device=device)[None, :]
    row_mix = (s0 + (rows & M32) * 0x9E3779B9) & M32
    a = (g * 0xB5297A4D + row_mix) & M32
    m = a * 0xCC9E2D51                       # below 2^64: the int64 product wraps, the two 32-bit halves are still right
    word = ((m & M32) ^ ((m >> 32) & M32) ^ s1) & M32
    t = torch.tensor(float(p), dtype=torch.float32).item() * 4294967296.0   # the kernel scales the fp32 value of p (exact: a power of two)
    thr = 0xFFFFFF00 if t >= 4294967040.0 else int(t)
    fields = torch.stack([(word * c) & M32 for c in (0x9E3779B1, 0x85EBCA6B, 0xC2B2AE35, 0x27D4EB2F)], dim=-1)  # [rows, groups, 4]
    keep = (fields >= thr).reshape(B * H * Sq, groups * 4)[:, :Sk]
    return keep.reshape(B, H, Sq, Sk)


def _es(t):
    if t.dtype == torch.bfloat16:
        return 2
    if t.dtype == torch.float32:
        return 4
    raise KernelError(f"gemm operands must be bf16 or fp32, got {t.dtype}")


def matmul_nt(a, b, out=None, *, bias=None, act=None, addend=None, pre_act_out=None, alpha=1.0,
              accumulate=False, out_dtype=None, bn=0, dropout=None):
    """out[M,N] = a[M,K] @ b[N,K]^T (+bias, activation, dropout, +addend).  Linear forward.
    dropout = (p, salt, seed_tensor): applied by the epilogue after the activation."""
    M, K = a.shape
    N = b.shape[0]
    out = _gemm_out(out, M, N, a, out_dtype)
    _cuda_contig(a, b, out, bias, addend, pre_act_out)
    gemm_raw(M=M, N=N, K=K, A=a.data_ptr(), lda=K, B=b.data_ptr(), ldb=K, C=out.data_ptr(), ldc=N,
             es=_es(a), C2=_p(pre_act_out), bias=_p(bias), addend=_p(addend), ld_add=N, alpha=alpha,
             act=ACT_CODES[act] if not isinstance(act, int) else act, out_fp32=out.dtype == torch.float32,
             accumulate=accumulate, bn=bn, dropout=dropout)
    return out


def matmul_nn(a, b, out=None, *, alpha=1.0, accumulate=False, out_dtype=None, bn=0):
    """out[M,N] = a[M,K] @ b[K,N].  Linear dgrad (a = dY, b = W[out,in])."""
    M, K = a.shape
    N = b.shape[1]
    out = _gemm_out(out, M, N, a, out_dtype)
    _cuda_contig(a, b, out)
    if a.dtype == torch.float32:
        # fp32 storage runs on the tf32 path, whose operands must be K-major: transpose b once
        return matmul_nt(a, transpose2d(b), out=out, alpha=alpha, accumulate=accumulate, bn=bn)
    gemm_raw(M=M, N=N, K=K, A=a.data_ptr(), lda=K, B=b.data_ptr(), ldb=N, b_mn=True, C=out.data_ptr(), ldc=N,
             es=_es(a), alpha=alpha, out_fp32=out.dtype == torch.float32, accumulate=accumulate, bn=bn)
    return out


def matmul_tn(a, b, out=None, *, alpha=1.0, accumulate=False, out_dtype=None, bn=0):
    """out[M,N] = a[K,M]^T @ b[K,N].  Linear wgrad (a = dY[tokens,out], b = X[tokens,in])."""
    K, M = a.shape
    N = b.shape[1]
    out = _gemm_out(out, M, N, a, out_dtype)
    _cuda_contig(a, b, out)
    if a.dtype == torch.float32:
        return matmul_nt(transpose2d(a), transpose2d(b), out=out, alpha=alpha, accumulate=accumulate, bn=bn)
    gemm_raw(M=M, N=N, K=K, A=a.data_ptr(), lda=M, a_mn=True, B=b.data_ptr(), ldb=N, b_mn=True,
             C=out.data_ptr(), ldc=N, es=_es(a), alpha=alpha, out_fp32=out.dtype == torch.float32,
             accumulate=accumulate, bn=bn)
    return out


def _gemm_out(out, M, N, like, out_dtype):
    if out is None:
        out = torch.empty((M, N), device=like.device, dtype=out_dtype or like.dtype)
    return out


# --------------------------------------------------------------------------- elementwise
def unary_fwd(op: str, x, out=None, scalar: float = 0.0):
    out = torch.empty_like(x) if out is None else out
    _cuda_contig(x, out)
    _check(lib().ffk_unary_fwd(UNARY_OPS[op], x.data_ptr(), out.data_ptr(), x.numel(), scalar, _dt(x), _stream()),
           "ffk_unary_fwd")
    return out


def unary_bwd(op: str, x, y, dy, dx=None, scalar: float = 0.0, accumulate=False):
    dx = torch.empty_like(x) if dx is None else dx
    _cuda_contig(x, y, dy, dx)
    _check(lib().ffk_unary_bwd(UNARY_OPS[op], x.data_ptr(), y.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel(),
                               scalar, _dt(x), int(accumulate), _stream()), "ffk_unary_bwd")
    return dx


def binary_fwd(op: str, a, b, out=None):
    out = torch.empty_like(a) if out is None else out
    _cuda_contig(a, b, out)
    if a.dtype != b.dtype:
        raise KernelError("binary op operands must share a dtype")
    if a.numel() % b.numel() != 0:
        raise KernelError("second operand must broadcast over trailing dims")
    _check(lib().ffk_binary_fwd(BINARY_OPS[op], a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), b.numel(),
                                _dt(a), _stream()), "ffk_binary_fwd")
    return out


def binary_bwd(op: str, a, b, dy, da=None, db=None, accumulate=False):
    _cuda_contig(a, b, dy, da, db)
    _check(lib().ffk_binary_bwd(BINARY_OPS[op], a.data_ptr(), b.data_ptr(), dy.data_ptr(), _p(da), _p(db),
                                dy.numel(), _dt(dy), int(accumulate), _stream()), "ffk_binary_bwd")


def dropout(x, p: float, seed: int, residual=None, out=None, seed_tensor=None):
    """out = dropout(x) [+ residual]; the mask is a function of (seed, *seed_tensor, element index)."""
    out = torch.empty_like(x) if out is None else out
    _cuda_contig(x, residual, out, seed_tensor)
    _check(lib().ffk_dropout(x.data_ptr(), _p(residual), out.data_ptr(), x.numel(), p, seed & (2**64 - 1),
                             _p(seed_tensor), _dt(x), _stream()), "ffk_dropout")
    return out


def axpby(x, y, a: float = 1.0, b: float = 1.0):
    """y = a*x + b*y in place."""
    _cuda_contig(x, y)
    _check(lib().ffk_axpby(x.data_ptr(), y.data_ptr(), x.numel(), a, b, _dt(x), _stream()), "ffk_axpby")
    return y


def fill(y, v: float):
    _cuda_contig(y)
    _check(lib().ffk_fill(y.data_ptr(), y.numel(), v, _dt(y), _stream()), "ffk_fill")
    return y


def cast(src, dst, accumulate=False):
    _cuda_contig(src, dst)
    _check(lib().ffk_cast(src.data_ptr(), _dt(src), dst.data_ptr(), _dt(dst), src.numel(), int(accumulate),
                          _stream()), "ffk_cast")
    return dst


def bias_act_bwd_scratch(rows, cols) -> int:
    return lib().ffk_bias_act_bwd_scratch(rows, cols)


def bias_act_bwd(dy, saved, dz, dbias, scratch, act, accumulate=False, dropout=None):
    """dz = dy * act'(saved); dbias (+)= column sums of dz.  dropout = (p, salt, seed_tensor): dy first goes back
    through the dropout that the forward GEMM epilogue applied after the activation."""
    rows, cols = dy.shape
    _cuda_contig(dy, saved, dz, dbias, scratch)
    if dropout is not None and dropout[0] > 0:
        l = lib()
        if not getattr(l, "_bad_declared", False):
            l.ffk_bias_act_dropout_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                   c_float, c_ulonglong, c_void_p, c_void_p]
            l.ffk_bias_act_dropout_bwd.restype = c_int
            l._bad_declared = True
        _check(l.ffk_bias_act_dropout_bwd(dy.data_ptr(), _p(saved), _p(dz), _p(dbias), _p(scratch), rows, cols,
                                          ACT_CODES[act] if not isinstance(act, int) else act, _dt(dy), int(accumulate), float(dropout[0]),
                                          int(dropout[1]) & (2**64 - 1), _p(dropout[2]), _stream()), "ffk_bias_act_dropout_bwd")
        return
    _check(lib().ffk_bias_act_bwd(dy.data_ptr(), _p(saved), _p(dz), _p(dbias), _p(scratch), rows, cols,
                                  ACT_CODES[act] if not isinstance(act, int) else act, _dt(dy), int(accumulate),
                                  _stream()), "ffk_bias_act_bwd")


# --------------------------------------------------------------------------- row-wise
def layernorm_fwd(a, gamma, beta, eps, residual=None, xsum=None, out=None, mean=None, rstd=None):
    rows, cols = a.shape
    out = torch.empty_like(a) if out is None else out
    _cuda_contig(a, residual, gamma, beta, xsum, out, mean, rstd)
    _check(lib().ffk_layernorm_fwd(a.data_ptr(), _p(residual), _p(gamma), _p(beta), _p(xsum), out.data_ptr(),
                                   _p(mean), _p(rstd), rows, cols, eps, _dt(a), _stream()), "ffk_layernorm_fwd")
    return out


def layernorm_bwd_scratch(rows, cols) -> int:
    return lib().ffk_layernorm_bwd_scratch(rows, cols)


def layernorm_bwd(dy, x, gamma, mean, rstd, dx, dgamma, dbeta, scratch, accumulate_dx=False,
                  accumulate_params=False, dx2=None, accumulate_dx2=False):
    rows, cols = dy.shape
    _cuda_contig(dy, x, gamma, mean, rstd, dx, dx2, dgamma, dbeta, scratch)
    _check(lib().ffk_layernorm_bwd(dy.data_ptr(), x.data_ptr(), _p(gamma), mean.data_ptr(), rstd.data_ptr(),
                                   dx.data_ptr(), _p(dx2), _p(dgamma), _p(dbeta), _p(scratch), rows, cols, _dt(dy),
                                   int(accumulate_dx), int(accumulate_dx2), int(accumulate_params), _stream()),
           "ffk_layernorm_bwd")


def softmax_fwd(x, out=None, scale=1.0, causal_q=0):
    cols = x.shape[-1]
    rows = x.numel() // cols
    out = torch.empty_like(x) if out is None else out
    _cuda_contig(x, out)
    _check(lib().ffk_softmax_fwd(x.data_ptr(), out.data_ptr(), rows, cols, scale, causal_q, _dt(x), _stream()),
           "ffk_softmax_fwd")
    return out


def softmax_bwd(dy, y, dx=None, scale=1.0):
    cols = y.shape[-1]
    rows = y.numel() // cols
    dx = torch.empty_like(y) if dx is None else dx
    _cuda_contig(dy, y, dx)
    _check(lib().ffk_softmax_bwd(dy.data_ptr(), y.data_ptr(), dx.data_ptr(), rows, cols, scale, _dt(y), _stream()),
           "ffk_softmax_bwd")
    return dx


def softmax_ce(logits, labels, loss, dlogits=None, probs=None, grad_scale=1.0):
    rows, cols = logits.shape
    _cuda_contig(logits, labels, loss, dlogits, probs)
    _check(lib().ffk_softmax_ce(logits.data_ptr(), labels.data_ptr(), _p(probs), _p(dlogits), _p(loss), rows, cols,
                                grad_scale, _dt(logits), _dt(labels), _stream()), "ffk_softmax_ce")


def loss_bwd(kind: str, pred, target, dpred, scale):
    cols = pred.shape[-1]
    rows = pred.numel() // cols
    _cuda_contig(pred, target, dpred)
    ldt = _dt(target) if target is not None and target.dtype in (torch.int32, torch.int64) else DT_I32
    _check(lib().ffk_loss_bwd(LOSS_KINDS[kind], pred.data_ptr(), _p(target), dpred.data_ptr(), rows, cols, scale,
                              _dt(pred), ldt, _stream()), "ffk_loss_bwd")


def loss_fwd(kind: str, pred, target, loss_rows):
    cols = pred.shape[-1]
    rows = pred.numel() // cols
    _cuda_contig(pred, target, loss_rows)
    ldt = _dt(target) if target is not None and target.dtype in (torch.int32, torch.int64) else DT_I32
    _check(lib().ffk_loss_fwd(LOSS_KINDS[kind], pred.data_ptr(), _p(target), loss_rows.data_ptr(), rows, cols,
                              _dt(pred), ldt, _stream()), "ffk_loss_fwd")


# --------------------------------------------------------------------------- optimizers / embedding
def adam_update(w, m, v, g, shadow, alpha_t, beta1, beta2, eps, weight_decay=0.0, grad_scale=1.0, alpha_tensor=None):
    """One Adam step over an arena; alpha_tensor (1-element fp32 device tensor) overrides alpha_t when given."""
    _cuda_contig(w, m, v, g, shadow, alpha_tensor)
    _check(lib().ffk_adam_update(w.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), _p(shadow), w.numel(),
                                 alpha_t, beta1, beta2, eps, weight_decay, grad_scale, _p(alpha_tensor), _dt(g),
                                 _stream()), "ffk_adam_update")


def sgd_update(w, mom, g, shadow, lr, momentum=0.0, nesterov=False, weight_decay=0.0, grad_scale=1.0):
    _cuda_contig(w, mom, g, shadow)
    _check(lib().ffk_sgd_update(w.data_ptr(), _p(mom), g.data_ptr(), _p(shadow), w.numel(), lr, momentum,
                                int(nesterov), weight_decay, grad_scale, _dt(g), _stream()), "ffk_sgd_update")


def embedding_fwd(idx, table, out, aggr="sum"):
    bag = idx.shape[-1] if out.dim() == idx.dim() else 1
    tokens = idx.numel() // bag
    _cuda_contig(idx, table, out)
    _check(lib().ffk_embedding_fwd(idx.data_ptr(), table.data_ptr(), out.data_ptr(), tokens, bag, table.shape[1],
                                   table.shape[0], int(aggr == "avg"), _dt(table), _dt(idx), _dt(out), _stream()),
           "ffk_embedding_fwd")
    return out


def embedding_bwd(idx, dout, dtable, aggr="sum"):
    bag = idx.shape[-1] if dout.dim() == idx.dim() else 1
    tokens = idx.numel() // bag
    _cuda_contig(idx, dout, dtable)
    _check(lib().ffk_embedding_bwd(idx.data_ptr(), dout.data_ptr(), dtable.data_ptr(), tokens, bag,
                                   dtable.shape[1], dtable.shape[0], int(aggr == "avg"), _dt(dtable), _dt(idx),
                                   _dt(dout), _stream()), "ffk_embedding_bwd")
    return dtable


def embedding_sgd(idx, dout, table, lr, aggr="sum"):
    """Sparse plain-SGD step of an fp32 table from the gradient of the gathered rows: table[idx] -= lr * dout."""
    bag = idx.shape[-1] if dout.dim() == idx.dim() else 1
    tokens = idx.numel() // bag
    _cuda_contig(idx, dout, table)
    if table.dtype != torch.float32:
        raise KernelError("embedding_sgd needs an fp32 table")
    _check(lib().ffk_embedding_sgd(idx.data_ptr(), dout.data_ptr(), table.data_ptr(), tokens, bag, table.shape[1], table.shape[0],
                                   lr / bag if aggr == "avg" else lr, _dt(idx), _dt(dout), _stream()), "ffk_embedding_sgd")
    return table


METRIC_FLAGS = {"accuracy": 1, "categorical_crossentropy": 2, "sparse_categorical_crossentropy": 4, "mean_squared_error": 8,
                "root_mean_squared_error": 16, "mean_absolute_error": 32}
_metrics_declared = [False]


def metrics_update(pred, label, acc, metrics=("accuracy",)):
    """Add one batch to the device accumulator `acc` (8 float64: samples, correct, cce, sparse cce, mse, rmse, mae, -)
    in one launch and without a host synchronisation.  pred: [n, c] fp32/bf16; label: [n] int32/int64 class ids, or
    [n, c] targets of pred's dtype."""
    l = lib()
    if not _metrics_declared[0]:
        l.ffk_metrics_update.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
        l.ffk_metrics_update.restype = c_int
        _metrics_declared[0] = True
    _cuda_contig(pred, label, acc)
    n, c = pred.shape
    if acc.dtype != torch.float64 or acc.numel() < 8:
        raise KernelError("metrics accumulator must be 8 float64 values")
    flags = 0
    for m in metrics:
        flags |= METRIC_FLAGS[m]
    sparse = label.dtype in (torch.int32, torch.int64)
    if not sparse and (label.dtype != pred.dtype or label.numel() != pred.numel()):
        raise KernelError("dense metric targets must have the predictions' dtype and shape")
    if sparse and label.numel() != n:
        raise KernelError("sparse metric labels must be one class id per row")
    _check(l.ffk_metrics_update(pred.data_ptr(), label.data_ptr() if sparse else None, None if sparse else label.data_ptr(), n, c,
                                _dt(pred), _dt(label) if sparse else 0, flags, acc.data_ptr(), _stream()), "ffk_metrics_update")
    return acc


_stack_declared = [False]


def _stack_lib():
    l = lib()
    if not _stack_declared[0]:
        P, I, F = c_void_p, c_int, c_float
        PP = ctypes.POINTER(c_void_p)
        l.ffk_alltoall_embedding_fwd.argtypes = [P, P, P, PP, I, I, I, I, I, I, I, I, P]
        l.ffk_alltoall_embedding_bwd.argtypes = [P, P, P, P, PP, I, I, I, I, I, I, F, I, I, P]
        l.ffk_alltoall_embedding_fwd.restype = l.ffk_alltoall_embedding_bwd.restype = c_int
        _stack_declared[0] = True
    return l


def embedding_stack_fwd(table_ptrs, entries, idx, out):
    """out[b, t, :] = table_t[idx[b, t], :] for T fp32 tables of equal width in one launch (`table_ptrs`, `entries`:
    int64 device tensors of the tables' addresses and row counts).  The single-device form of the all-to-all
    embedding gather."""
    _cuda_contig(table_ptrs, entries, idx, out)
    b, t, dim = out.shape
    peers = (c_void_p * 1)(out.data_ptr())
    _check(_stack_lib().ffk_alltoall_embedding_fwd(table_ptrs.data_ptr(), entries.data_ptr(), idx.data_ptr(), peers, b, b, t, dim, 0, 1,
                                                   _dt(out), _dt(idx), _stream()), "ffk_alltoall_embedding_fwd")
    return out


def embedding_stack_sgd(table_ptrs, entries, idx, dout, lr):
    """table_t[idx[b, t], :] -= lr * dout[b, t, :] for all T tables in one launch."""
    _cuda_contig(table_ptrs, entries, idx, dout)
    b, t, dim = dout.shape
    peers = (c_void_p * 1)(dout.data_ptr())
    _check(_stack_lib().ffk_alltoall_embedding_bwd(table_ptrs.data_ptr(), None, entries.data_ptr(), idx.data_ptr(), peers, b, b, t, dim, 0, 1,
                                                   lr, _dt(dout), _dt(idx), _stream()), "ffk_alltoall_embedding_bwd")


# --------------------------------------------------------------------------- data movement
def _decl_tensor_ops(l):
    P, I, L, F, S = c_void_p, c_int, c_longlong, c_float, c_void_p
    LP = ctypes.POINTER(c_longlong)
    sig = {
        "ffk_permute": [P, P, I, LP, LP, I, I, S],
        "ffk_transpose2d": [P, P, I, I, I, I, S],
        "ffk_block_copy": [P, L, P, L, L, L, I, I, I, S],
        "ffk_reduce": [P, P, L, L, L, I, I, S],
        "ffk_reduce_bwd": [P, P, L, L, L, F, I, I, S],
        "ffk_reduce_select_bwd": [P, P, P, P, L, L, L, I, I, I, S],
        "ffk_gather": [P, P, P, L, L, L, L, I, I, S],
        "ffk_gather_bwd": [P, P, P, L, L, L, L, I, I, S],
        "ffk_topk": [P, P, P, I, I, I, I, S],
        "ffk_topk_bwd": [P, P, P, I, I, I, I, I, S],
        "ffk_reverse": [P, P, L, L, L, I, S],
        "ffk_load_rows": [P, P, P, L, L, L, L, S],
    }
    for name, args in sig.items():
        fn = getattr(l, name)
        fn.argtypes = args
        fn.restype = c_int


_tensor_ops_declared = [False]


def _tlib():
    l = lib()
    if not _tensor_ops_declared[0]:
        _decl_tensor_ops(l)
        _tensor_ops_declared[0] = True
    return l


def permute(src, perm, out=None, accumulate=False):
    """out = src.permute(perm), materialised contiguously (accumulate: out += ...).  `src` may be any strided
    view (an expanded tensor broadcasts)."""
    _cuda_contig(out)
    if not src.is_cuda:
        raise KernelError("kernel called with a CPU tensor")
    sizes = [src.shape[p] for p in perm]
    strides = [src.stride(p) for p in perm]
    out = torch.empty(sizes, dtype=src.dtype, device=src.device) if out is None else out
    n = len(sizes)
    arr = (c_longlong * n)
    acc = 0
    if accumulate:
        acc = 1 if src.dtype == torch.float32 else 2
    _check(_tlib().ffk_permute(src.data_ptr(), out.data_ptr(), n, arr(*sizes), arr(*strides), src.element_size(), acc,
                               _stream()), "ffk_permute")
    return out


def transpose2d(src, out=None):
    """[..., r, c] -> [..., c, r] through shared-memory tiles."""
    _cuda_contig(src, out)
    r, c = src.shape[-2], src.shape[-1]
    batch = src.numel() // (r * c)
    out = torch.empty(*src.shape[:-2], c, r, dtype=src.dtype, device=src.device) if out is None else out
    _check(_tlib().ffk_transpose2d(src.data_ptr(), out.data_ptr(), batch, r, c, src.element_size(), _stream()),
           "ffk_transpose2d")
    return out


def block_copy(src, src_off, src_ld, dst, dst_off, dst_ld, outer, block, accumulate=False):
    """dst[o*dst_ld + dst_off + b] (+)= src[o*src_ld + src_off + b] for o < outer, b < block (flat element offsets)."""
    _cuda_contig(src, dst)
    es = src.element_size()
    _check(_tlib().ffk_block_copy(src.data_ptr() + src_off * es, src_ld, dst.data_ptr() + dst_off * es, dst_ld, outer, block, es,
                                  _DT.get(src.dtype, 0), int(accumulate), _stream()), "ffk_block_copy")


REDUCE_OPS = {"sum": 0, "mean": 1, "max": 2, "min": 3, "prod": 4}


def reduce(x, out, outer, red, inner, op="sum"):
    _cuda_contig(x, out)
    _check(_tlib().ffk_reduce(x.data_ptr(), out.data_ptr(), outer, red, inner, REDUCE_OPS[op], _dt(x), _stream()), "ffk_reduce")
    return out


def reduce_bwd(dy, dx, outer, red, inner, scale=1.0, accumulate=False):
    _cuda_contig(dy, dx)
    _check(_tlib().ffk_reduce_bwd(dy.data_ptr(), dx.data_ptr(), outer, red, inner, scale, _dt(dy), int(accumulate), _stream()),
           "ffk_reduce_bwd")


def reduce_select_bwd(x, y, dy, dx, outer, red, inner, op, accumulate=False):
    """Backward of a max / min / prod reduction over the middle dim of x[outer, red, inner] (y, dy: [outer, inner])."""
    _cuda_contig(x, y, dy, dx)
    _check(_tlib().ffk_reduce_select_bwd(x.data_ptr(), y.data_ptr(), dy.data_ptr(), dx.data_ptr(), outer, red, inner, REDUCE_OPS[op],
                                         _dt(x), int(accumulate), _stream()), "ffk_reduce_select_bwd")


def load_rows(dataset, out, indices=None, first=0):
    """out[i] = dataset[indices[i]] (or dataset[first + i] without indices).  `dataset` is a contiguous [num_samples, ...]
    tensor in page-locked host memory (read by the GPU in place) or on the device; `indices` an int64 device tensor."""
    if not (dataset.is_contiguous() and out.is_contiguous() and out.is_cuda):
        raise KernelError("load_rows: contiguous data set and a contiguous device batch expected")
    if not (dataset.is_cuda or dataset.is_pinned()):
        raise KernelError("load_rows: the data set must be in page-locked host memory (tensor.pin_memory()) or on the device")
    n = out.shape[0]
    row_bytes = (dataset.numel() // max(dataset.shape[0], 1)) * dataset.element_size()
    if out.numel() * out.element_size() != n * row_bytes or out.dtype != dataset.dtype:
        raise KernelError("load_rows: batch rows do not match the data set's rows")
    if indices is not None:
        if indices.dtype != torch.int64 or not indices.is_cuda or indices.numel() < n:
            raise KernelError("load_rows: indices must be an int64 device tensor with one entry per batch row")
    _check(_tlib().ffk_load_rows(dataset.data_ptr(), None if indices is None else indices.data_ptr(), out.data_ptr(), n, row_bytes, int(first),
                                 dataset.shape[0], _stream()), "ffk_load_rows")
    return out


def gather(x, idx, out, dim):
    _cuda_contig(x, idx, out)
    outer = 1
    for s in x.shape[:dim]:
        outer *= s
    inner = 1
    for s in x.shape[dim + 1:]:
        inner *= s
    if list(idx.shape[:dim]) != list(x.shape[:dim]) or list(idx.shape[dim + 1:]) != list(x.shape[dim + 1:]):
        raise KernelError("gather: index must match the input outside the gather dim")
    _check(_tlib().ffk_gather(x.data_ptr(), idx.data_ptr(), out.data_ptr(), outer, x.shape[dim], idx.shape[dim], inner,
                              x.element_size(), _dt(idx), _stream()), "ffk_gather")
    return out


def gather_bwd(dy, idx, dx, dim):
    _cuda_contig(dy, idx, dx)
    outer = 1
    for s in dx.shape[:dim]:
        outer *= s
    inner = 1
    for s in dx.shape[dim + 1:]:
        inner *= s
    _check(_tlib().ffk_gather_bwd(dy.data_ptr(), idx.data_ptr(), dx.data_ptr(), outer, dx.shape[dim], idx.shape[dim], inner,
                                  _dt(dy), _dt(idx), _stream()), "ffk_gather_bwd")


def topk(x, k, vals=None, idxs=None):
    _cuda_contig(x, vals, idxs)
    cols = x.shape[-1]
    rows = x.numel() // cols
    vals = torch.empty(*x.shape[:-1], k, dtype=x.dtype, device=x.device) if vals is None else vals
    idxs = torch.empty(*x.shape[:-1], k, dtype=torch.int32, device=x.device) if idxs is None else idxs
    _check(_tlib().ffk_topk(x.data_ptr(), vals.data_ptr(), idxs.data_ptr(), rows, cols, k, _dt(x), _stream()), "ffk_topk")
    return vals, idxs


def topk_bwd(dvals, idxs, dx, accumulate=False):
    _cuda_contig(dvals, idxs, dx)
    cols, k = dx.shape[-1], idxs.shape[-1]
    rows = dx.numel() // cols
    _check(_tlib().ffk_topk_bwd(dvals.data_ptr(), idxs.data_ptr(), dx.data_ptr(), rows, cols, k, _dt(dx), int(accumulate),
                                _stream()), "ffk_topk_bwd")


def reverse(x, out, axis):
    _cuda_contig(x, out)
    outer = 1
    for s in x.shape[:axis]:
        outer *= s
    inner = 1
    for s in x.shape[axis + 1:]:
        inner *= s
    _check(_tlib().ffk_reverse(x.data_ptr(), out.data_ptr(), outer, x.shape[axis], inner, x.element_size(), _stream()),
           "ffk_reverse")
    return out


# --------------------------------------------------------------------------- fused softmax + dropout (attention probabilities)
def softmax_dropout_supported(t) -> bool:
    cols = t.shape[-1]
    return t.dtype == torch.bfloat16 and cols % 256 == 0 and cols // 256 in (1, 2, 4, 8, 16)


def _decl_softmax_dropout(l):
    P, I, F, S = c_void_p, c_int, c_float, c_void_p
    l.ffk_softmax_dropout_fwd.argtypes = [P, P, P, I, I, F, I, F, c_ulonglong, P, I, S]
    l.ffk_softmax_dropout_fwd.restype = c_int
    l.ffk_softmax_dropout_bwd.argtypes = [P, P, P, I, I, F, F, c_ulonglong, P, I, S]
    l.ffk_softmax_dropout_bwd.restype = c_int


_sd_declared = [False]


def _sdlib():
    l = lib()
    if not _sd_declared[0]:
        _decl_softmax_dropout(l)
        _sd_declared[0] = True
    return l


def softmax_dropout_fwd(x, y, y_dropped, p, salt, seed_tensor=None, scale=1.0, causal_q=0):
    """y = softmax(scale*x) and, in the same pass, y_dropped = dropout(y, p) (y_dropped may be None)."""
    _cuda_contig(x, y, y_dropped, seed_tensor)
    cols = x.shape[-1]
    rows = x.numel() // cols
    _check(_sdlib().ffk_softmax_dropout_fwd(x.data_ptr(), y.data_ptr(), _p(y_dropped), rows, cols, scale, causal_q, p,
                                            salt & (2**64 - 1), _p(seed_tensor), _dt(x), _stream()), "ffk_softmax_dropout_fwd")


def softmax_dropout_bwd(dy, y, dx, p, salt, seed_tensor=None, scale=1.0):
    """dx = softmax backward of the gradient that first goes back through the same dropout mask."""
    _cuda_contig(dy, y, dx, seed_tensor)
    cols = y.shape[-1]
    rows = y.numel() // cols
    _check(_sdlib().ffk_softmax_dropout_bwd(dy.data_ptr(), y.data_ptr(), dx.data_ptr(), rows, cols, scale, p,
                                            salt & (2**64 - 1), _p(seed_tensor), _dt(y), _stream()), "ffk_softmax_dropout_bwd")


# --------------------------------------------------------------------------- convolution support, pooling, batch norm
def _decl_conv(l):
    P, I, L, F, S = c_void_p, c_int, c_longlong, c_float, c_void_p
    IP, LP = ctypes.POINTER(c_int), ctypes.POINTER(c_longlong)
    sig = {
        "ffk_im2col": ([P, P, IP, LP, I, S], c_int),
        "ffk_col2im": ([P, P, IP, LP, I, I, S], c_int),
        "ffk_filter_pack": ([P, P, I, I, I, I, I, I, S], c_int),
        "ffk_filter_unpack": ([P, P, I, I, I, I, I, I, I, S], c_int),
        "ffk_pool2d_fwd": ([P, P, P, IP, LP, I, I, S], c_int),
        "ffk_pool2d_bwd": ([P, P, P, IP, LP, I, I, I, S], c_int),
        "ffk_batchnorm_scratch": ([L, I], c_longlong),
        "ffk_batchnorm_fwd": ([P, P, P, P, P, P, P, L, I, F, I, I, S], c_int),
        "ffk_batchnorm_bwd": ([P, P, P, P, P, P, P, P, P, P, L, I, I, I, I, I, S], c_int),
    }
    for name, (args, res) in sig.items():
        fn = getattr(l, name)
        fn.argtypes = args
        fn.restype = res


_conv_declared = [False]


def _clib():
    l = lib()
    if not _conv_declared[0]:
        _decl_conv(l)
        _conv_declared[0] = True
    return l


class ConvGeometry:
    """Window geometry shared by im2col/col2im and pooling: logical NCHW extents, the activation's element strides
    in (n, c, h, w) order, and the padded GEMM depth Kp."""

    def __init__(self, n, c, h, w, kh, kw, sh, sw, ph, pw, strides, kp=None):
        self.n, self.c, self.h, self.w = n, c, h, w
        self.kh, self.kw, self.sh, self.sw, self.ph, self.pw = kh, kw, sh, sw, ph, pw
        self.oh = (h + 2 * ph - kh) // sh + 1
        self.ow = (w + 2 * pw - kw) // sw + 1
        k = kh * kw * c
        self.k = k
        self.kp = (k + 7) // 8 * 8 if kp is None else kp
        self.rows = n * self.oh * self.ow
        self._geom = (c_int * 13)(n, c, h, w, kh, kw, sh, sw, ph, pw, self.oh, self.ow, self.kp)
        self._strides = (c_longlong * 4)(*strides)


def nhwc_strides(n, c, h, w):
    return (h * w * c, 1, w * c, c)


def nchw_strides(n, c, h, w):
    return (c * h * w, h * w, w, 1)


def im2col(x, col, geom: ConvGeometry):
    _cuda_contig(x, col)
    _check(_clib().ffk_im2col(x.data_ptr(), col.data_ptr(), geom._geom, geom._strides, _dt(x), _stream()), "ffk_im2col")


def col2im(dcol, dx, geom: ConvGeometry, accumulate=False):
    _cuda_contig(dcol, dx)
    _check(_clib().ffk_col2im(dcol.data_ptr(), dx.data_ptr(), geom._geom, geom._strides, _dt(dx), int(accumulate), _stream()),
           "ffk_col2im")


def conv_implicit_supported(geom: "ConvGeometry", oc: int) -> bool:
    """Whether the implicit-GEMM kernel (no im2col matrix) takes this convolution: stride 1, channel counts that are
    multiples of 8, channels-last bf16 data."""
    if geom.sh != 1 or geom.sw != 1 or geom.kp != geom.kh * geom.kw * geom.c:
        return False
    return bool(_clib().ffk_conv_implicit_supported(geom.c, oc, geom.kh, geom.kw))


def _conv_desc(geom: "ConvGeometry", oc: int, wp) -> ConvDesc:
    d = ConvDesc()
    d.N, d.H, d.W, d.C, d.OC, d.KH, d.KW = geom.n, geom.h, geom.w, geom.c, oc, geom.kh, geom.kw
    d.pad_h, d.pad_w, d.OH, d.OW = geom.ph, geom.pw, geom.oh, geom.ow
    d.wp, d.ldw = wp.data_ptr(), wp.stride(0)
    return d


def conv_fprop(x, wp, y, geom: "ConvGeometry", oc: int, bias=None, act=None, pre_act_out=None):
    """y[N, OH, OW, OC] = act(conv(x[N, H, W, C], filter) + bias) over channels-last bf16 data; `wp` is the packed filter
    [OC, KH*KW*C]."""
    _cuda_contig(x, wp, y)
    d = _conv_desc(geom, oc, wp)
    d.x, d.y = x.data_ptr(), y.data_ptr()
    d.bias = bias.data_ptr() if bias is not None else None
    d.pre = pre_act_out.data_ptr() if pre_act_out is not None else None
    d.act = ACT_CODES[act]
    _check(_clib().ffk_conv_fprop(ctypes.byref(d), _stream()), "ffk_conv_fprop")


def conv_dgrad(dy, wp, dx, geom: "ConvGeometry", oc: int, accumulate=False):
    """dx[N, H, W, C] (+)= the data gradient of the convolution from dy[N, OH, OW, OC]."""
    _cuda_contig(dy, wp, dx)
    d = _conv_desc(geom, oc, wp)
    d.dy, d.dx, d.accumulate = dy.data_ptr(), dx.data_ptr(), int(accumulate)
    _check(_clib().ffk_conv_dgrad(ctypes.byref(d), _stream()), "ffk_conv_dgrad")


def conv_wgrad(x, dy, dwp, geom: "ConvGeometry", oc: int, accumulate=False):
    """dwp[OC, KH*KW*C] (fp32, packed layout) (+)= the filter gradient."""
    _cuda_contig(x, dy, dwp)
    d = _conv_desc(geom, oc, dwp)
    d.x, d.dy, d.dwp, d.accumulate = x.data_ptr(), dy.data_ptr(), dwp.data_ptr(), int(accumulate)
    _check(_clib().ffk_conv_wgrad(ctypes.byref(d), _stream()), "ffk_conv_wgrad")


def conv_last_error() -> int:
    return int(_clib().ffk_conv_last_error())


def filter_pack(w, wp, oc, c, kh, kw, kp):
    _cuda_contig(w, wp)
    _check(_clib().ffk_filter_pack(w.data_ptr(), wp.data_ptr(), oc, c, kh, kw, kp, _dt(w), _stream()), "ffk_filter_pack")


def filter_unpack(dwp, dw, oc, c, kh, kw, kp, accumulate=False):
    _cuda_contig(dwp, dw)
    if dwp.dtype != torch.float32:
        raise KernelError("filter_unpack: packed gradient must be fp32")
    _check(_clib().ffk_filter_unpack(dwp.data_ptr(), dw.data_ptr(), oc, c, kh, kw, kp, _dt(dw), int(accumulate), _stream()),
           "ffk_filter_unpack")


def pool2d_fwd(x, y, arg, geom: ConvGeometry, mode: str):
    _cuda_contig(x, y, arg)
    _check(_clib().ffk_pool2d_fwd(x.data_ptr(), y.data_ptr(), _p(arg), geom._geom, geom._strides, 0 if mode == "max" else 1, _dt(x),
                                  _stream()), "ffk_pool2d_fwd")


def pool2d_bwd(dy, arg, dx, geom: ConvGeometry, mode: str, accumulate=False):
    _cuda_contig(dy, arg, dx)
    _check(_clib().ffk_pool2d_bwd(dy.data_ptr(), _p(arg), dx.data_ptr(), geom._geom, geom._strides, 0 if mode == "max" else 1,
                                  _dt(dy), int(accumulate), _stream()), "ffk_pool2d_bwd")


def batchnorm_scratch(rows, cols) -> int:
    """fp32 elements of scratch that batchnorm_fwd / batchnorm_bwd need for [rows, cols]."""
    return int(_clib().ffk_batchnorm_scratch(rows, cols))


def batchnorm_fwd(x, y, gamma, beta, mean, rstd, scratch, rows, cols, eps, relu=False):
    _cuda_contig(x, y, gamma, beta, mean, rstd, scratch)
    _check(_clib().ffk_batchnorm_fwd(x.data_ptr(), y.data_ptr(), _p(gamma), _p(beta), mean.data_ptr(), rstd.data_ptr(),
                                     scratch.data_ptr(), rows, cols, eps, int(relu), _dt(x), _stream()), "ffk_batchnorm_fwd")


def batchnorm_bwd(dy, x, relu_y, gamma, mean, rstd, dx, dgamma, dbeta, scratch, rows, cols, accumulate_dx=False,
                  accumulate_gamma=False, accumulate_beta=False):
    _cuda_contig(dy, x, relu_y, gamma, mean, rstd, dx, dgamma, dbeta, scratch)
    _check(_clib().ffk_batchnorm_bwd(dy.data_ptr(), x.data_ptr(), _p(relu_y), _p(gamma), mean.data_ptr(), rstd.data_ptr(), _p(dx),
                                     _p(dgamma), _p(dbeta), scratch.data_ptr(), rows, cols, _dt(dy), int(accumulate_dx),
                                     int(accumulate_gamma), int(accumulate_beta), _stream()), "ffk_batchnorm_bwd")
