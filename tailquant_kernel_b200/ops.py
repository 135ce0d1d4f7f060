"""Operator layer: the reference's extension entry points, backed by libtailquant.so.

Names, argument order, in-place convention ("caller allocates, kernel writes on the current
CUDA stream") and error behaviour (RuntimeError with a message) follow the reference's
pybind functions:

  fused_topr_pack / threshold_topr_pack ........ tools/fused_topr_pack_ext_v55.py:112-155,
                                                 tools/fused_threshold_topr_pack_ext_v57.py:236-273
  scale_sparse_epilogue_quad / _oct ............. tools/fused_sparse_epilogue_ext_v58.py:123-174
  sparse_correction_add_{bf16,fp16}_oct ......... tools/sparse_correction_add_ext_v1.py:175-224
  sparse_{i32,u16}_c{4,8,16}_b{128,256}, idx_i32_to_u16  tools/split_sparse_idx16_ext_v1.py:138-163
  matmul(A_pack, B_pack) -> int32 ............... call site tools/bench_hadamard_three_schemes_quarot_dense_sharedqkv_inplace_fusedtopr_v43.py:235-239

plus the entry points that only exist here (bf16 tail, fused rotation, fused dequant):
split_prologue, prepare_weight, tail_gather, split_gemm_fused, matmul_splitk, dequant_finish.

PyTorch is used for device memory and streams only.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import TQ_BF16, TQ_FP16, TQ_HAD_BLOCK128, TQ_HAD_KRON12, TQ_HAD_NONE, TQ_HAD_WHT

EPS = 1e-8
TAIL_REC_CAP = 12  # TQ_TAIL_REC_CAP of include/tailquant.h


# --------------------------------------------------------------------------- helpers
def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_cuda(t: torch.Tensor, name: str, dtype=None) -> None:
    _check(torch.is_tensor(t) and t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.is_contiguous(), f"{name} must be contiguous")
    if dtype is not None:
        _check(t.dtype == dtype, f"{name} must be {dtype}")


def _f16_code(dtype) -> int:
    if dtype == torch.bfloat16:
        return TQ_BF16
    if dtype == torch.float16:
        return TQ_FP16
    raise RuntimeError("expected a bf16 or fp16 tensor")


def ceil_ratio_count(k: int, ratio: float) -> int:
    """R for a ratio: min(K-1, max(1, ceil(K*ratio))), 0 for ratio <= 0
    (tools/bench_v61_dense_sparse_matrix_breakdown_v1.py:81-84)."""
    if ratio <= 0.0:
        return 0
    return min(k - 1, max(1, int(math.ceil(k * ratio))))


def split_select_params(K: int, R: int, activation_percentile: float = 100.0):
    """(R, descending_rank, select_k) (tools/bench_qwen3_l18_split_opts_v57.py:83-93)."""
    pct = min(max(float(activation_percentile), 0.0), 100.0)
    body_len = K - R
    body_kth = min(K, max(1, int(math.ceil(body_len * pct / 100.0))))
    descending_rank = K - body_kth + 1
    return R, descending_rank, max(R, descending_rank)


def default_had_kind(K: int) -> int:
    """Rotation used for an input dimension: full transform for powers of two, 12 (x) 2^n when
    K = 12*2^n, else block-diagonal 128 (the reference falls back to a block transform for
    dimensions its Hadamard helper does not know: tools/romeorot_blockhad_utils_v1.py:34-64)."""
    if K & (K - 1) == 0:
        return TQ_HAD_WHT
    if K % 12 == 0 and (K // 12) & (K // 12 - 1) == 0:
        return TQ_HAD_KRON12
    if K % 2048 == 0:
        return TQ_HAD_BLOCK128
    raise RuntimeError(f"no rotation is built for K={K}")


# --------------------------------------------------------------------------- prologue
@dataclass
class PrologueOut:
    a_pack: Optional[torch.Tensor]       # [M, K/2] u8
    body_scale: torch.Tensor             # [M] f32
    top_scale: torch.Tensor              # [M] f32
    tail_idx: Optional[torch.Tensor]     # [M, ld] int16 storage of u16 indices (first R valid)
    tail_val: Optional[torch.Tensor]     # [M, ld] bf16
    R: int
    idx32: Optional[torch.Tensor] = None  # [M, R] i32   (T4)
    top_q: Optional[torch.Tensor] = None  # [M, R] i8    (T4)
    x_rot: Optional[torch.Tensor] = None  # [M, K] bf16
    a_q8: Optional[torch.Tensor] = None   # [M, K] i8, operand order of split_gemm_mma
    tail_ptr: Optional[torch.Tensor] = None  # [M, K/128 + 1] int16 storage of u16 run boundaries
    tail_rec: Optional[torch.Tensor] = None  # [2 ceil(M/256), K/64, 128, TAIL_REC_CAP] int32: tile position | bf16 << 16
    tail_cnt: Optional[torch.Tensor] = None  # [2 ceil(M/256), K/64, 128] int16: entries per (row, 64-wide half slice)
    tail_dense: Optional[torch.Tensor] = None  # [M, K] bf16: the rotated row, zero outside the tail (R > 0)


def split_prologue(x: torch.Tensor, had_kind: int, R: int, descending_rank: Optional[int] = None,
                   eps: float = EPS, t16: bool = True, t4: bool = False, want_x_rot: bool = False,
                   want_q8: bool = False, want_pack: bool = True, out: Optional[PrologueOut] = None,
                   rms_weight: Optional[torch.Tensor] = None, rms_eps: float = 1e-6,
                   want_dense: bool = False) -> PrologueOut:
    """Rotation + per-token INT4 + top-R tail split of x [M,K] bf16 in one kernel.  With `rms_weight` ([K] bf16)
    an RMSNorm is applied to x first, inside the same kernel (no T4 outputs then)."""
    _check_cuda(x, "x", torch.bfloat16)
    _check(x.dim() == 2, "x must be [M, K]")
    M, K = x.shape
    if descending_rank is None:
        descending_rank = R + 1
    if out is None:
        dev = x.device
        ld = (R + 7) // 8 * 8
        out = PrologueOut(
            a_pack=torch.empty((M, K // 2), dtype=torch.uint8, device=dev) if want_pack else None,
            body_scale=torch.empty(M, dtype=torch.float32, device=dev),
            top_scale=torch.empty(M, dtype=torch.float32, device=dev),
            tail_idx=torch.zeros((M, ld), dtype=torch.int16, device=dev) if (t16 and R) else None,
            tail_val=torch.zeros((M, ld), dtype=torch.bfloat16, device=dev) if (t16 and R) else None,
            R=R,
            a_q8=torch.empty((M, K), dtype=torch.int8, device=dev) if want_q8 else None,
            tail_ptr=torch.empty((M, K // 128 + 1), dtype=torch.int16, device=dev) if (want_q8 and R) else None,
            tail_rec=torch.empty((2 * ((M + 255) // 256), K // 64, 128, TAIL_REC_CAP), dtype=torch.int32, device=dev)
            if (want_q8 and R) else None,
            tail_cnt=torch.zeros((2 * ((M + 255) // 256), K // 64, 128), dtype=torch.int16, device=dev)
            if (want_q8 and R) else None,
            idx32=torch.empty((M, R), dtype=torch.int32, device=dev) if (t4 and R) else None,
            top_q=torch.empty((M, R), dtype=torch.int8, device=dev) if (t4 and R) else None,
            x_rot=torch.empty((M, K), dtype=torch.bfloat16, device=dev) if want_x_rot else None,
            tail_dense=torch.empty((M, K), dtype=torch.bfloat16, device=dev) if (want_dense and R) else None,
        )
    ld = out.tail_idx.shape[1] if out.tail_idx is not None else 0
    pld = out.tail_ptr.shape[1] if out.tail_ptr is not None else 0
    if rms_weight is not None:
        _check_cuda(rms_weight, "rms_weight", torch.bfloat16)
        _check(rms_weight.numel() == K, "rms_weight must have K elements")
        _check(out.idx32 is None and out.top_q is None, "the fused RMSNorm prologue has no T4 outputs")
        rc = _lib.load().tq_split_prologue_rmsnorm(
            _ptr(x), _ptr(rms_weight), float(rms_eps), M, K, had_kind, R, descending_rank, eps, _ptr(out.a_pack),
            _ptr(out.a_q8), _ptr(out.body_scale), _ptr(out.top_scale), _ptr(out.tail_idx), _ptr(out.tail_val), ld,
            _ptr(out.tail_ptr), pld, _ptr(out.tail_rec), _ptr(out.tail_cnt), _ptr(out.tail_dense), _ptr(out.x_rot),
            _stream())
        _lib.check(rc, f"split_prologue_rmsnorm(M={M}, K={K}, had_kind={had_kind}, R={R})")
        return out
    rc = _lib.load().tq_split_prologue(
        _ptr(x), M, K, had_kind, R, descending_rank, eps, _ptr(out.a_pack), _ptr(out.a_q8), _ptr(out.body_scale),
        _ptr(out.top_scale), _ptr(out.tail_idx), _ptr(out.tail_val), ld, _ptr(out.tail_ptr), pld, _ptr(out.tail_rec),
        _ptr(out.tail_cnt), _ptr(out.tail_dense), _ptr(out.idx32), _ptr(out.top_q), _ptr(out.x_rot), _stream())
    _lib.check(rc, f"split_prologue(M={M}, K={K}, had_kind={had_kind}, R={R})")
    return out


def _topr_pack(name, A, R, descending_rank, A_pack, body_scale, top_scale, top_q, idx, eps):
    _check_cuda(A, "A")
    _check(A.dim() == 2, "A must be [M, K]")
    _check(A.dtype in (torch.bfloat16, torch.float16), "A must be bf16 or fp16")
    M, K = A.shape
    R, descending_rank = int(R), int(descending_rank)
    _check_cuda(A_pack, "A_pack", torch.uint8)
    _check(A_pack.numel() >= (M * K + 1) // 2, "A_pack is too small")
    _check_cuda(body_scale, "body_scale", torch.float32)
    _check_cuda(top_scale, "top_scale", torch.float32)
    _check(body_scale.numel() >= M and top_scale.numel() >= M, "scale tensors must hold M values")
    if R > 0:
        _check_cuda(top_q, "top_q", torch.int8)
        _check_cuda(idx, "idx", torch.int32)
        _check(top_q.numel() >= M * R and idx.numel() >= M * R, "top_q / idx must be [M, R]")
    rc = _lib.load().tq_topr_pack(_ptr(A), _f16_code(A.dtype), M, K, R, descending_rank, _ptr(A_pack),
                                  _ptr(body_scale), _ptr(top_scale), _ptr(top_q) if R else None,
                                  _ptr(idx) if R else None, float(eps), _stream())
    _lib.check(rc, f"{name}(M={M}, K={K}, R={R}, descending_rank={descending_rank})")


def fused_topr_pack(A, R, descending_rank, A_pack, body_scale, top_scale, top_q, idx, eps) -> None:
    """tools/fused_topr_pack_ext_v55.py:112-121 (same argument order; idx ascending)."""
    _topr_pack("fused_topr_pack", A, R, descending_rank, A_pack, body_scale, top_scale, top_q, idx, eps)


def threshold_topr_pack(A, R, descending_rank, A_pack, body_scale, top_scale, top_q, idx, eps) -> None:
    """tools/fused_threshold_topr_pack_ext_v57.py:236-245 (same argument order)."""
    _topr_pack("threshold_topr_pack", A, R, descending_rank, A_pack, body_scale, top_scale, top_q, idx, eps)


# --------------------------------------------------------------------------- weights
@dataclass
class PreparedWeight:
    N: int
    K: int
    had_kind: int
    b_col: torch.Tensor               # [N, K/2] u8
    w_scale: torch.Tensor             # [N] f32
    w_t: Optional[torch.Tensor]       # [K, N] bf16   (T16 tail)
    b_row: Optional[torch.Tensor]     # [K, N/2] u8   (T4 tail)
    w_rot: Optional[torch.Tensor]     # [N, K] bf16
    bias: Optional[torch.Tensor] = None  # [N] f32


def prepare_weight(W: torch.Tensor, had_kind: Optional[int] = None, eps: float = EPS, t16: bool = True,
                   t4: bool = False, keep_w_rot: bool = False, bias: Optional[torch.Tensor] = None) -> PreparedWeight:
    """Offline: rotate the input dim, RTN INT4 per output channel, tail layouts. W is [N,K]."""
    _check(torch.is_tensor(W) and W.is_cuda and W.dim() == 2, "W must be a CUDA [N, K] tensor")
    Wb = W.detach().to(torch.bfloat16).contiguous()
    N, K = Wb.shape
    if had_kind is None:
        had_kind = default_had_kind(K)
    dev = Wb.device
    b_col = torch.empty((N, K // 2), dtype=torch.uint8, device=dev)
    w_scale = torch.empty(N, dtype=torch.float32, device=dev)
    need_rot = bool(t16 or keep_w_rot)
    w_rot = torch.empty((N, K), dtype=torch.bfloat16, device=dev) if need_rot else None
    w_t = torch.empty((K, N), dtype=torch.bfloat16, device=dev) if t16 else None
    b_row = torch.empty((K, N // 2), dtype=torch.uint8, device=dev) if t4 else None
    rc = _lib.load().tq_prepare_weight(_ptr(Wb), N, K, had_kind, eps, _ptr(b_col), _ptr(w_scale), _ptr(w_rot),
                                       _ptr(b_row), _ptr(w_t), _stream())
    _lib.check(rc, f"prepare_weight(N={N}, K={K}, had_kind={had_kind})")
    b32 = None if bias is None else bias.detach().to(device=dev, dtype=torch.float32).contiguous()
    return PreparedWeight(N, K, had_kind, b_col, w_scale, w_t, b_row, w_rot if keep_w_rot else None, b32)


# --------------------------------------------------------------------------- GEMM
def _gemm_dims(A_pack, B_pack, M, N, K):
    _check_cuda(A_pack, "A_pack", torch.uint8)
    _check_cuda(B_pack, "B_pack", torch.uint8)
    if M is None:
        _check(A_pack.dim() == 2 and B_pack.dim() == 2, "A_pack / B_pack must be [M, K/2] / [N, K/2]")
        M, N, K = A_pack.shape[0], B_pack.shape[0], A_pack.shape[1] * 2
        _check(B_pack.shape[1] * 2 == K, "A_pack and B_pack disagree on K")
    _check(A_pack.numel() >= M * K // 2 and B_pack.numel() >= N * K // 2, "packed operand too small")
    return int(M), int(N), int(K)


def matmul(A_pack: torch.Tensor, B_pack: torch.Tensor, M: Optional[int] = None, N: Optional[int] = None,
           K: Optional[int] = None) -> torch.Tensor:
    """INT4 x INT4 -> int32 [M,N]; accepts matmul(A, B) and matmul(A, B, M, N, K)
    (tools/bench_v61_dense_sparse_matrix_breakdown_v1.py:184-187). The only entry point that
    allocates its result, like the reference's."""
    M, N, K = _gemm_dims(A_pack, B_pack, M, N, K)
    C = torch.empty((M, N), dtype=torch.int32, device=A_pack.device)
    rc = _lib.load().tq_int4_matmul(_ptr(A_pack), _ptr(B_pack), _ptr(C), M, N, K, 1, _stream())
    _lib.check(rc, f"matmul(M={M}, N={N}, K={K})")
    return C


def matmul_splitk(A_pack, B_pack, C: torch.Tensor, split_k: int, M=None, N=None, K=None) -> torch.Tensor:
    """Small-M path: the reduction is split over `split_k` CTAs per tile and accumulated with
    int32 atomics into C, which is zeroed here first."""
    M, N, K = _gemm_dims(A_pack, B_pack, M, N, K)
    _check_cuda(C, "C", torch.int32)
    _check(C.numel() >= M * N, "C too small")
    C.zero_()
    rc = _lib.load().tq_int4_matmul(_ptr(A_pack), _ptr(B_pack), _ptr(C), M, N, K, int(split_k), _stream())
    _lib.check(rc, f"matmul_splitk(M={M}, N={N}, K={K}, split_k={split_k})")
    return C


def split_gemm_fused(A_pack, body_scale, B_pack, w_scale, out, tail=None, bias=None, M=None, N=None, K=None):
    """out[m,n] = bf16((float(acc)*body_scale[m])*w_scale[n] + tail[m,n] + bias[n])."""
    M, N, K = _gemm_dims(A_pack, B_pack, M, N, K)
    _check_cuda(body_scale, "body_scale", torch.float32)
    _check_cuda(w_scale, "w_scale", torch.float32)
    _check_cuda(out, "out", torch.bfloat16)
    _check(out.numel() >= M * N, "out too small")
    if tail is not None:
        _check_cuda(tail, "tail", torch.float32)
        _check(tail.numel() >= M * N, "tail too small")
    if bias is not None:
        _check_cuda(bias, "bias", torch.float32)
    rc = _lib.load().tq_split_gemm_fused(_ptr(A_pack), _ptr(body_scale), _ptr(B_pack), _ptr(w_scale), _ptr(tail),
                                         _ptr(bias), _ptr(out), M, N, K, _stream())
    _lib.check(rc, f"split_gemm_fused(M={M}, N={N}, K={K})")
    return out


def split_gemm_mma(a_q8, body_scale, B_pack, w_scale, out, w_rot=None, pro: Optional[PrologueOut] = None,
                   R: int = 0, bias=None, dbg_acc=None, dbg_tail=None, act: str = "none"):
    """One kernel: dense INT4 x INT4 part on tcgen05 kind::i8 plus the tail as a bf16 tensor-core product
    over the zero-filled tail matrix, fused dequant + bias, bf16 out.  act="swiglu": the weight rows are
    interleaved (gate_i, up_i) pairs and out is [M, N/2] = bf16(bf16(silu(gate)) * up)."""
    _check(act in ("none", "swiglu"), "act must be 'none' or 'swiglu'")
    _check_cuda(a_q8, "a_q8", torch.int8)
    _check_cuda(B_pack, "B_pack", torch.uint8)
    _check_cuda(body_scale, "body_scale", torch.float32)
    _check_cuda(w_scale, "w_scale", torch.float32)
    _check_cuda(out, "out", torch.bfloat16)
    M, K = a_q8.shape
    N = B_pack.shape[0]
    _check(B_pack.shape[1] * 2 == K, "a_q8 and B_pack disagree on K")
    _check(out.numel() >= (M * N // 2 if act == "swiglu" else M * N), "out too small")
    _check(act == "none" or (dbg_acc is None and dbg_tail is None), "no debug outputs with a fused activation")
    ld = 0
    if R:
        _check_cuda(w_rot, "w_rot", torch.bfloat16)
        _check(tuple(w_rot.shape) == (N, K), "w_rot must be [N, K]")
        _check(pro is not None, "the prologue outputs are needed when R > 0")
        tail_idx, tail_val, tail_ptr, tail_rec, tail_cnt = pro.tail_idx, pro.tail_val, pro.tail_ptr, pro.tail_rec, pro.tail_cnt
        _check_cuda(tail_idx, "tail_idx", torch.int16)
        _check_cuda(tail_val, "tail_val", torch.bfloat16)
        _check_cuda(tail_ptr, "tail_ptr", torch.int16)
        _check_cuda(tail_rec, "tail_rec", torch.int32)
        _check_cuda(tail_cnt, "tail_cnt", torch.int16)
        _check(tail_ptr.shape[0] == M and tail_ptr.shape[1] >= K // 128 + 1, "tail_ptr must be [M, K/128 + 1]")
        _check(tuple(tail_rec.shape) == (2 * ((M + 255) // 256), K // 64, 128, TAIL_REC_CAP), "tail_rec has the wrong shape")
        _check(tuple(tail_cnt.shape) == (2 * ((M + 255) // 256), K // 64, 128), "tail_cnt has the wrong shape")
        ld = tail_idx.shape[1]
        if pro.tail_dense is not None:
            _check_cuda(pro.tail_dense, "tail_dense", torch.bfloat16)
            _check(tuple(pro.tail_dense.shape) == (M, K), "tail_dense must be [M, K]")
    if bias is not None:
        _check_cuda(bias, "bias", torch.float32)
    common = (_ptr(a_q8), _ptr(body_scale), _ptr(B_pack), _ptr(w_scale),
              _ptr(w_rot) if R else None, _ptr(tail_idx) if R else None,
              _ptr(tail_val) if R else None, ld, _ptr(tail_ptr) if R else None,
              tail_ptr.shape[1] if R else 0, _ptr(tail_rec) if R else None,
              _ptr(tail_cnt) if R else None, _ptr(pro.tail_dense) if R else None, int(R), _ptr(bias), _ptr(out))
    if act == "swiglu":
        rc = _lib.load().tq_split_gemm_mma_swiglu(*common, M, N, K, _stream())
    else:
        rc = _lib.load().tq_split_gemm_mma(*common, _ptr(dbg_acc), _ptr(dbg_tail), M, N, K, _stream())
    _lib.check(rc, f"split_gemm_mma(M={M}, N={N}, K={K}, R={R}, act={act})")
    return out


def set_gemm_pair_mode(mode: int) -> None:
    """-1: split_gemm_mma picks its kernel by problem size; 0: one CTA per tile; 1: CTA pairs (256 x 256 tiles)."""
    _lib.check(_lib.load().tq_set_gemm_pair_mode(int(mode)), "set_gemm_pair_mode")


def set_gemv_channel_tiles(tiles: int) -> None:
    """8-channel tiles per warp of the decode GEMV for calls with more than 16 rows: -1 (default: 4), 1, 2 or 4.
    `gemv_plan` follows it, so buffers of partial sums sized before a change no longer fit."""
    _lib.check(_lib.load().tq_set_gemv_channel_tiles(int(tiles)), "set_gemv_channel_tiles")


def set_prologue_mode(mode: int) -> None:
    """-1: the prologue kernel specialised for K = 4096 / 12288 / 14336 where it applies; 0: the general kernel only
    (both give the same bits; a switch for comparisons)."""
    _lib.check(_lib.load().tq_set_prologue_mode(int(mode)), "set_prologue_mode")


def dequant_finish(C, body_scale, w_scale, out, tail=None, bias=None):
    _check_cuda(C, "C", torch.int32)
    M, N = C.shape
    _check_cuda(out, "out", torch.bfloat16)
    rc = _lib.load().tq_dequant_finish(_ptr(C), _ptr(body_scale), _ptr(w_scale), _ptr(tail), _ptr(bias), _ptr(out),
                                       M, N, _stream())
    _lib.check(rc, "dequant_finish")
    return out


def gemv_splitk(A, B_pack, C: torch.Tensor, split_k: int = 0) -> torch.Tensor:
    """Decode path (M <= 64): exact INT4 x INT4 -> int32 with the weights streamed once; C is zeroed by the
    call; split_k < 1 lets the library choose.  A is the packed uint8 [M,K/2] or the prologue's int8 [M,K]."""
    _check_cuda(A, "A")
    _check_cuda(B_pack, "B_pack", torch.uint8)
    _check(A.dtype in (torch.uint8, torch.int8) and A.dim() == 2, "A must be uint8 [M,K/2] or int8 [M,K]")
    a8 = A.dtype == torch.int8
    M, N, K = A.shape[0], B_pack.shape[0], B_pack.shape[1] * 2
    _check(A.shape[1] == (K if a8 else K // 2), "A and B_pack disagree on K")
    _check_cuda(C, "C", torch.int32)
    _check(C.numel() >= M * N, "C too small")
    rc = _lib.load().tq_int4_gemv_splitk(None if a8 else _ptr(A), _ptr(A) if a8 else None, _ptr(B_pack), _ptr(C), M, N,
                                         K, int(split_k), _stream())
    _lib.check(rc, f"gemv_splitk(M={M}, N={N}, K={K}, split_k={split_k})")
    return C


def gemv_plan(M: int, N: int, K: int, a_is_int8: bool = False) -> int:
    """Number of K ranges the library uses for the decode GEMV of this shape (= leading size of the partials)."""
    n = _lib.load().tq_int4_gemv_plan(int(M), int(N), int(K), 1 if a_is_int8 else 0)
    if n < 1:
        _lib.check(n, f"gemv_plan(M={M}, N={N}, K={K})")
    return int(n)


def gemv_partials(A, B_pack, partials: torch.Tensor) -> torch.Tensor:
    """Decode GEMV with the K ranges kept apart: partials [splits, M, N] int32 (splits = gemv_plan(...)),
    written by plain stores in one launch; `dequant_finish_partials` adds them up."""
    _check_cuda(A, "A")
    _check_cuda(B_pack, "B_pack", torch.uint8)
    _check(A.dtype in (torch.uint8, torch.int8) and A.dim() == 2, "A must be uint8 [M,K/2] or int8 [M,K]")
    a8 = A.dtype == torch.int8
    M, N, K = A.shape[0], B_pack.shape[0], B_pack.shape[1] * 2
    _check(A.shape[1] == (K if a8 else K // 2), "A and B_pack disagree on K")
    _check_cuda(partials, "partials", torch.int32)
    _check(partials.dim() == 3 and tuple(partials.shape[1:]) == (M, N), "partials must be [splits, M, N]")
    rc = _lib.load().tq_int4_gemv_partials(None if a8 else _ptr(A), _ptr(A) if a8 else None, _ptr(B_pack),
                                           _ptr(partials), M, N, K, int(partials.shape[0]), _stream())
    _lib.check(rc, f"gemv_partials(M={M}, N={N}, K={K}, splits={partials.shape[0]})")
    return partials


def dequant_finish_partials(partials, body_scale, w_scale, out, tail=None, bias=None, act: str = "none"):
    """out = bf16((float(sum_s partials[s]) * body_scale[m]) * w_scale[n] + tail + bias); act="swiglu" as in
    split_gemm_mma (out [M, N/2])."""
    _check(act in ("none", "swiglu"), "act must be 'none' or 'swiglu'")
    _check_cuda(partials, "partials", torch.int32)
    _check(partials.dim() == 3, "partials must be [splits, M, N]")
    S, M, N = partials.shape
    _check_cuda(out, "out", torch.bfloat16)
    _check(out.numel() >= (M * N // 2 if act == "swiglu" else M * N), "out too small")
    rc = _lib.load().tq_dequant_finish_partials(_ptr(partials), int(S), _ptr(body_scale), _ptr(w_scale), _ptr(tail),
                                                _ptr(bias), _ptr(out), M, N, 1 if act == "swiglu" else 0, _stream())
    _lib.check(rc, f"dequant_finish_partials(S={S}, M={M}, N={N})")
    return out


def tail_gather_small(tail_idx, tail_val, w_t, tail_out, R: int):
    """Tail sums for few rows (decode): gathers only the needed weight rows; eight interleaved fp32 chains per
    output combined pairwise in a fixed order."""
    _check_cuda(tail_idx, "tail_idx", torch.int16)
    _check_cuda(tail_val, "tail_val", torch.bfloat16)
    _check_cuda(w_t, "w_t", torch.bfloat16)
    _check_cuda(tail_out, "tail_out", torch.float32)
    M, ld = tail_idx.shape
    K, N = w_t.shape
    _check(tail_out.numel() >= M * N, "tail_out too small")
    rc = _lib.load().tq_tail_gather_small(_ptr(tail_idx), _ptr(tail_val), _ptr(w_t), _ptr(tail_out), M, N, K, int(R),
                                          ld, _stream())
    _lib.check(rc, f"tail_gather_small(M={M}, N={N}, K={K}, R={R})")
    return tail_out


NOALLOC_MAX_ELEMS = 1 << 20  # TQ_NOALLOC_MAX_ELEMS of include/tailquant.h


def linear_splitk_noalloc(A_pack, body_scale, B_pack, w_scale, out, split_k: int, tail=None, bias=None):
    """Split-K linear whose int32 accumulators live in a fixed array inside libtailquant.so, for hosts that
    cannot allocate device memory when they run it (M * N <= NOALLOC_MAX_ELEMS).  Same result as
    matmul_splitk + dequant_finish.  Calls on one device share the array: do not let two of them overlap on
    the GPU, and make the first call on a device during start-up."""
    M, N, K = _gemm_dims(A_pack, B_pack, None, None, None)
    _check_cuda(body_scale, "body_scale", torch.float32)
    _check_cuda(w_scale, "w_scale", torch.float32)
    _check_cuda(out, "out", torch.bfloat16)
    _check(out.numel() >= M * N, "out too small")
    rc = _lib.load().tq_int4_linear_splitk_noalloc(_ptr(A_pack), _ptr(body_scale), _ptr(B_pack), _ptr(w_scale),
                                                   _ptr(tail), _ptr(bias), _ptr(out), M, N, K, int(split_k),
                                                   _stream())
    _lib.check(rc, f"linear_splitk_noalloc(M={M}, N={N}, K={K}, split_k={split_k})")
    return out


def tail_gather(tail_idx, tail_val, w_t, tail_out, R: int):
    """tail_out[m,n] = sum_r tail_val[m,r] * w_t[tail_idx[m,r], n] (fp32 fma chain, ascending r)."""
    _check_cuda(tail_idx, "tail_idx", torch.int16)
    _check_cuda(tail_val, "tail_val", torch.bfloat16)
    _check_cuda(w_t, "w_t", torch.bfloat16)
    _check_cuda(tail_out, "tail_out", torch.float32)
    M, ld = tail_idx.shape
    K, N = w_t.shape
    _check(tail_val.shape == tail_idx.shape, "tail_idx / tail_val shapes differ")
    _check(tail_out.numel() >= M * N, "tail_out too small")
    rc = _lib.load().tq_tail_gather(_ptr(tail_idx), _ptr(tail_val), _ptr(w_t), _ptr(tail_out), M, N, K, int(R), ld,
                                    _stream())
    _lib.check(rc, f"tail_gather(M={M}, N={N}, K={K}, R={R})")
    return tail_out


# --------------------------------------------------------------------------- T4 (reference) tail
def _t4_common(top_q, idx, B_row_pack, top_scale, w_scale, out):
    _check_cuda(top_q, "top_q", torch.int8)
    _check_cuda(B_row_pack, "B_row_pack", torch.uint8)
    _check_cuda(top_scale, "top_scale", torch.float32)
    _check_cuda(out, "out")
    _check(top_q.dim() == 2 and out.dim() == 2, "top_q must be [M, R] and out [M, N]")
    M, R = top_q.shape
    N = out.shape[1]
    _check(out.shape[0] == M, "out and top_q disagree on M")
    _check(idx.numel() == M * R, "idx must be [M, R]")
    _check(w_scale.numel() >= N and top_scale.numel() >= M, "scale tensors too small")
    _check((B_row_pack.numel() * 2) % N == 0, "B_row_pack must be [K, N/2]")
    K = B_row_pack.numel() * 2 // N
    return M, N, K, R


def _scale_sparse_epilogue(name, C, body_scale, top_q, idx, B_row_pack, top_scale, w_scale, out, K):
    _check_cuda(C, "C", torch.int32)
    _check_cuda(idx, "idx", torch.int32)
    _check_cuda(body_scale, "body_scale", torch.float32)
    _check_cuda(w_scale, "w_scale", torch.float32)
    M, N, K2, R = _t4_common(top_q, idx, B_row_pack, top_scale, w_scale, out)
    _check(int(K) == K2, "K does not match B_row_pack")
    _check(C.numel() == M * N, "C must be [M, N]")
    rc = _lib.load().tq_scale_sparse_epilogue(_ptr(C), _ptr(body_scale), _ptr(top_q), _ptr(idx), _ptr(B_row_pack),
                                              _ptr(top_scale), _ptr(w_scale), _ptr(out), _f16_code(out.dtype), M, N,
                                              K2, R, _stream())
    _lib.check(rc, name)


def scale_sparse_epilogue_quad(C, body_scale, top_q, idx, B_row_pack, top_scale, w_scale, out, K) -> None:
    """tools/fused_sparse_epilogue_ext_v58.py:123-145 (the column-per-thread count is a tuning
    detail of the reference; both names run the same kernel here)."""
    _scale_sparse_epilogue("scale_sparse_epilogue_quad", C, body_scale, top_q, idx, B_row_pack, top_scale, w_scale,
                           out, K)


def scale_sparse_epilogue_oct(C, body_scale, top_q, idx, B_row_pack, top_scale, w_scale, out, K) -> None:
    """tools/fused_sparse_epilogue_ext_v58.py:147-169."""
    _scale_sparse_epilogue("scale_sparse_epilogue_oct", C, body_scale, top_q, idx, B_row_pack, top_scale, w_scale,
                           out, K)


def _sparse_correction_add(name, out, top_q, idx, B_row_pack, top_scale, w_scale, out_dtype, ws_dtype):
    _check_cuda(idx, "idx", torch.int32)
    _check_cuda(out, "out", out_dtype)
    _check_cuda(w_scale, "w_scale", ws_dtype)
    M, N, K, R = _t4_common(top_q, idx, B_row_pack, top_scale, w_scale, out)
    rc = _lib.load().tq_sparse_correction_add(_ptr(out), _f16_code(out.dtype), _ptr(top_q), _ptr(idx),
                                              _ptr(B_row_pack), _ptr(top_scale), _ptr(w_scale),
                                              1 if ws_dtype == torch.bfloat16 else 0, M, N, K, R, _stream())
    _lib.check(rc, name)


def sparse_correction_add_bf16_oct(out, top_q, idx, B_row_pack, top_scale, w_scale) -> None:
    """tools/sparse_correction_add_ext_v1.py:175-187."""
    _sparse_correction_add("sparse_correction_add_bf16_oct", out, top_q, idx, B_row_pack, top_scale, w_scale,
                           torch.bfloat16, torch.float32)


def sparse_correction_add_bf16_wscale_bf16_oct(out, top_q, idx, B_row_pack, top_scale, w_scale) -> None:
    """tools/sparse_correction_add_ext_v1.py:189-201."""
    _sparse_correction_add("sparse_correction_add_bf16_wscale_bf16_oct", out, top_q, idx, B_row_pack, top_scale,
                           w_scale, torch.bfloat16, torch.bfloat16)


def sparse_correction_add_fp16_oct(out, top_q, idx, B_row_pack, top_scale, w_scale) -> None:
    """tools/sparse_correction_add_ext_v1.py:203-215."""
    _sparse_correction_add("sparse_correction_add_fp16_oct", out, top_q, idx, B_row_pack, top_scale, w_scale,
                           torch.float16, torch.float32)


def sparse_top_write(top_q, idx, B_row_pack, top_scale, w_scale, out) -> None:
    """Write-only sparse term with int32 or uint16 (int16 storage) indices: the eight
    sparse_{i32,u16}_c{4,8,16}_b{128,256} variants of tools/split_sparse_idx16_ext_v1.py:144-151
    differ only in launch shape and all map here."""
    _check(idx.dtype in (torch.int32, torch.int16, torch.uint16), "idx must be int32 or 16-bit")
    _check_cuda(idx, "idx")
    _check_cuda(w_scale, "w_scale", torch.float32)
    M, N, K, R = _t4_common(top_q, idx, B_row_pack, top_scale, w_scale, out)
    rc = _lib.load().tq_sparse_top_write(_ptr(out), _f16_code(out.dtype), _ptr(top_q), _ptr(idx),
                                         0 if idx.dtype == torch.int32 else 1, _ptr(B_row_pack), _ptr(top_scale),
                                         _ptr(w_scale), M, N, K, R, _stream())
    _lib.check(rc, "sparse_top_write")


def idx_i32_to_u16(idx: torch.Tensor, out: torch.Tensor) -> None:
    """tools/split_sparse_idx16_ext_v1.py:31-48,138-142."""
    _check_cuda(idx, "idx", torch.int32)
    _check_cuda(out, "out")
    _check(out.element_size() == 2 and out.numel() >= idx.numel(), "out must hold idx.numel() 16-bit values")
    rc = _lib.load().tq_idx_i32_to_u16(_ptr(idx), _ptr(out), idx.numel(), _stream())
    _lib.check(rc, "idx_i32_to_u16")


def gemm_status() -> int:
    """Device status word of the pipelined kernels (0 = every bounded wait completed)."""
    import ctypes
    v = ctypes.c_uint(0)
    _lib.load().tq_gemm_status(ctypes.byref(v))
    return int(v.value)


# --------------------------------------------------------------------------- loader shims
class _Ext:
    """Stands in for the module object the reference's `load_*_ext(verbose=False)` return."""

    def __init__(self, **fns):
        self.__dict__.update(fns)


def load_fused_topr_pack_ext_v55(verbose: bool = False):
    _lib.load()
    return _Ext(fused_topr_pack=fused_topr_pack)


def load_fused_threshold_topr_pack_ext_v57(verbose: bool = False):
    _lib.load()
    return _Ext(threshold_topr_pack=threshold_topr_pack)


def load_fused_sparse_epilogue_ext_v58(verbose: bool = False):
    _lib.load()
    return _Ext(scale_sparse_epilogue_quad=scale_sparse_epilogue_quad,
                scale_sparse_epilogue_oct=scale_sparse_epilogue_oct)


def load_sparse_correction_add_ext_v1(verbose: bool = False):
    _lib.load()
    return _Ext(sparse_correction_add_bf16_oct=sparse_correction_add_bf16_oct,
                sparse_correction_add_bf16_wscale_bf16_oct=sparse_correction_add_bf16_wscale_bf16_oct,
                sparse_correction_add_fp16_oct=sparse_correction_add_fp16_oct)


def load_split_sparse_idx16_ext_v1(verbose: bool = False):
    _lib.load()
    fns = {"idx_i32_to_u16": idx_i32_to_u16}
    for it in ("i32", "u16"):
        for c in (4, 8, 16):
            for b in (128, 256):
                fns[f"sparse_{it}_c{c}_b{b}"] = sparse_top_write
    return _Ext(**fns)


def load_quarot_sm120_extension_v1(verbose: bool = False):
    """Name kept from tools/load_quarot_sm120_extension_v1.py; the GEMM behind it is the
    tcgen05 kernel of this package."""
    _lib.load()
    return _Ext(matmul=matmul)
