"""CPU oracle for the split W4A4 + tail linear.  TEST INFRASTRUCTURE ONLY.

This file restates, in numpy, the arithmetic of the reference's split linear so that the
CUDA path can be checked against it.  Nothing in the shipped package may import it: only
the tests, the smoke entry and the benchmark's CPU-baseline leg do.

Parity status: "parity unpinned" for the pieces whose reference implementation lives in
packages that are not part of the reference repository (the CUTLASS INT4 GEMM, the
activation pack kernel, the Hadamard utilities).  The pieces that ARE stated in the
reference repository are pinned by golden vectors generated from the reference's own
Python functions (tests/golden/make_golden.py):

  * select parameters ........ tools/bench_qwen3_l18_split_opts_v57.py:83-93
  * R from a ratio ........... tools/bench_v61_dense_sparse_matrix_breakdown_v1.py:81-84
  * thresholds + tail indices  tools/bench_topr_select_algos_v38.py:24-37
  * body / tail fake quant ... tools/compare_single_matrix_fake_vs_kernel_quant_l2_v1.py:81-97
  * nibble order ............. tools/compare_single_matrix_fake_vs_kernel_quant_l2_v1.py:47-55
  * RTN weight scale ......... tools/bench_multimodel_all_layers_policy_fastqf_v29.py:245-247
  * RTN weight codes ......... tools/bench_real_split_fullstack_rtn_ppl_v1.py:79-85
  * fused dequant + sparse ... tools/fused_sparse_epilogue_ext_v58.py:59-86
  * select order (ties) ...... tools/fused_threshold_topr_pack_ext_v57.py:141-181

Every float step is written so that one and only one IEEE-754 evaluation order is legal:
fp32 butterflies in ascending stride order, one fp32 multiply by the normalisation, one
round-to-nearest-even to bf16, true fp32 division for the quantiser, int32 accumulation,
`(acc * s_x) * s_w` for the dequant and a left-to-right fp32 fused multiply-add chain over
the tail in ascending index order.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

HAD_NONE = 0      # no rotation (input is already rotated)
HAD_WHT = 1       # K = 2^n            : normalised Walsh-Hadamard over the whole row
HAD_KRON12 = 2    # K = 12 * 2^n       : (H12 (x) H_{2^n}) / sqrt(K)
HAD_BLOCK128 = 3  # K = 128 * b        : block-diagonal H_128 / sqrt(128)

EPS = 1e-8


# ----------------------------------------------------------------------------- bf16
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16, returned as uint16 bit patterns."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounding = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    out = ((u + rounding) >> np.uint32(16)).astype(np.uint16)
    nan = (u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# ----------------------------------------------------------------------------- scalars
def ceil_ratio_count(k: int, ratio: float) -> int:
    """R for a ratio (tools/bench_v61_dense_sparse_matrix_breakdown_v1.py:81-84)."""
    if ratio <= 0.0:
        return 0
    return min(k - 1, max(1, int(math.ceil(k * ratio))))


def split_select_params(K: int, R: int, activation_percentile: float = 100.0) -> Tuple[int, int, int]:
    """(R, descending_rank, select_k) (tools/bench_qwen3_l18_split_opts_v57.py:83-93)."""
    pct = min(max(float(activation_percentile), 0.0), 100.0)
    body_len = K - R
    body_kth = min(K, max(1, int(math.ceil(body_len * pct / 100.0))))
    descending_rank = K - body_kth + 1
    return R, descending_rank, max(R, descending_rank)


# ----------------------------------------------------------------------------- Hadamard
def hadamard12() -> np.ndarray:
    """12x12 Hadamard matrix, Paley construction I over GF(11): H = I + S with
    S = [[0, 1^T], [-1, Q]], Q[i][j] = Legendre(i - j mod 11).  H @ H.T = 12 I.
    The reference takes its 12x12 factor from an external package that is not part of the
    repository (call site tools/bench_qwen3_l18_split_opts_v58.py:164); any Hadamard
    matrix gives a valid rotation as long as weights and activations share it."""
    q = 11
    residues = {(i * i) % q for i in range(1, q)}

    def chi(a: int) -> int:
        a %= q
        return 0 if a == 0 else (1 if a in residues else -1)

    H = np.zeros((12, 12), dtype=np.int32)
    H[0, :] = 1
    H[1:, 0] = -1
    for i in range(q):
        for j in range(q):
            H[1 + i, 1 + j] = chi(i - j) + (1 if i == j else 0)
    return H


def had_layout(kind: int, K: int) -> Tuple[int, bool]:
    """(segment length L of the power-of-two transform, whether the 12-point mix follows)."""
    if kind == HAD_NONE:
        return 1, False
    if kind == HAD_WHT:
        if K & (K - 1):
            raise ValueError("HAD_WHT needs a power-of-two K")
        return K, False
    if kind == HAD_KRON12:
        if K % 12 or (K // 12) & (K // 12 - 1):
            raise ValueError("HAD_KRON12 needs K = 12 * 2^n")
        return K // 12, True
    if kind == HAD_BLOCK128:
        if K % 128:
            raise ValueError("HAD_BLOCK128 needs K % 128 == 0")
        return 128, False
    raise ValueError(f"unknown hadamard kind {kind}")


def had_scale(kind: int, K: int) -> np.float32:
    if kind == HAD_NONE:
        return np.float32(1.0)
    n = 128 if kind == HAD_BLOCK128 else K
    return np.float32(1.0 / math.sqrt(float(n)))


def rotate_f32(x_f32: np.ndarray, kind: int) -> np.ndarray:
    """Un-normalised rotation in fp32 with the canonical operation order.
    Semantics of the rotation: x <- x.H on the last dim, power-of-two by butterflies,
    12*2^n by the 12x12 factor applied across 2^n-long segments after their own transform,
    else per-block (tools/romeorot_blockhad_utils_v1.py:57-64)."""
    x = np.array(x_f32, dtype=np.float32, copy=True)
    M, K = x.shape
    L, mix = had_layout(kind, K)
    if kind == HAD_NONE:
        return x
    v = x.reshape(M, K // L, L)
    s = 1
    while s < L:  # ascending strides; pair (i, i+s): lo' = lo + hi, hi' = lo - hi
        w = v.reshape(M, K // L, L // (2 * s), 2, s)
        lo = w[:, :, :, 0, :].copy()
        hi = w[:, :, :, 1, :].copy()
        w[:, :, :, 0, :] = lo + hi
        w[:, :, :, 1, :] = lo - hi
        s *= 2
    if mix:
        H = hadamard12()
        seg = v.reshape(M, 12, L)
        out = np.empty_like(seg)
        for a2 in range(12):
            acc = seg[:, 0, :] if H[a2, 0] > 0 else -seg[:, 0, :]
            acc = acc.astype(np.float32, copy=True)
            for a in range(1, 12):
                acc = acc + seg[:, a, :] if H[a2, a] > 0 else acc - seg[:, a, :]
            out[:, a2, :] = acc
        v = out
    return np.ascontiguousarray(v.reshape(M, K), dtype=np.float32)


def rotate_bf16(x_bits: np.ndarray, kind: int) -> np.ndarray:
    """bf16 bits in, bf16 bits out: rotation, one fp32 multiply by 1/sqrt(n), one rounding."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    if kind == HAD_NONE:
        return x_bits.copy()
    y = rotate_f32(bf16_bits_to_f32(x_bits), kind)
    y = y * had_scale(kind, x_bits.shape[1])
    return f32_to_bf16_bits(y)


# ----------------------------------------------------------------------------- select
@dataclass
class Selection:
    idx: np.ndarray        # [M, R] int32, ascending per row
    body_key: np.ndarray   # [M] uint16 : |x| bits at sorted position descending_rank-1
    top_key: np.ndarray    # [M] uint16 : row maximum of |x| bits
    tail_mask: np.ndarray  # [M, K] bool


def select_tail(x_bits: np.ndarray, R: int, descending_rank: Optional[int] = None) -> Selection:
    """Order = (|x| descending, index ascending); the first R form the tail.  This is the
    order of the reference's radix-threshold kernel (all keys above the threshold in index
    order, then ties in index order: tools/fused_threshold_topr_pack_ext_v57.py:141-181)."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    M, K = x_bits.shape
    if descending_rank is None:
        descending_rank = R + 1
    if not (0 <= R < K) or not (1 <= descending_rank <= K):
        raise ValueError("bad R / descending_rank")
    keys = (x_bits & np.uint16(0x7FFF)).astype(np.int32)
    order = np.argsort(-keys, axis=1, kind="stable")
    sorted_keys = np.take_along_axis(keys, order, axis=1)
    idx = np.sort(order[:, :R], axis=1).astype(np.int32)
    mask = np.zeros((M, K), dtype=bool)
    if R:
        np.put_along_axis(mask, idx, True, axis=1)
    return Selection(
        idx=idx,
        body_key=sorted_keys[:, descending_rank - 1].astype(np.uint16),
        top_key=sorted_keys[:, 0].astype(np.uint16),
        tail_mask=mask,
    )


# ----------------------------------------------------------------------------- quantise
def f16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b, dtype=np.uint16).view(np.float16).astype(np.float32)


def act_scale(key_bits: np.ndarray, eps: float = EPS, fmt: str = "bf16") -> np.ndarray:
    """max(threshold, eps) / 7 in fp32 (tools/fused_topr_pack_ext_v55.py:76-79)."""
    t = bf16_bits_to_f32(key_bits) if fmt == "bf16" else f16_bits_to_f32(key_bits)
    return (np.maximum(t, np.float32(eps)) / np.float32(7.0)).astype(np.float32)


def quant_s4(x_f32: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """clamp(rint(x / scale), -8, 7), rint = round-half-to-even, true fp32 division
    (tools/fused_topr_pack_ext_v55.py:21-26)."""
    t = (x_f32.astype(np.float32) / scale.astype(np.float32).reshape(-1, 1)).astype(np.float32)
    return np.clip(np.rint(t), -8, 7).astype(np.int8)


def pack_s4(q: np.ndarray) -> np.ndarray:
    """Element 2i -> low nibble, 2i+1 -> high nibble
    (tools/fused_topr_pack_ext_v55.py:107-108)."""
    u = (q.astype(np.int16) & 0xF).astype(np.uint8)
    return (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)


def unpack_s4(p: np.ndarray) -> np.ndarray:
    """Inverse of pack_s4 (tools/compare_single_matrix_fake_vs_kernel_quant_l2_v1.py:47-55)."""
    lo = (p & 0xF).astype(np.int8)
    hi = (p >> 4).astype(np.int8)
    out = np.empty((p.shape[0], p.shape[1] * 2), dtype=np.int8)
    out[:, 0::2] = lo
    out[:, 1::2] = hi
    return np.where(out >= 8, out - 16, out).astype(np.int8)


@dataclass
class Prologue:
    x_rot: np.ndarray       # [M, K] uint16 bf16 bits after rotation
    codes: np.ndarray       # [M, K] int8, tail positions zero
    a_pack: np.ndarray      # [M, K/2] uint8
    body_scale: np.ndarray  # [M] f32
    top_scale: np.ndarray   # [M] f32 (row max / 7)
    idx: np.ndarray         # [M, R] int32 ascending
    tail_val: np.ndarray    # [M, R] uint16 bf16 bits        (tail mode T16)
    top_q: np.ndarray       # [M, R] int8                    (tail mode T4)


def prologue(x_bits: np.ndarray, kind: int, R: int, descending_rank: Optional[int] = None,
             eps: float = EPS, fmt: str = "bf16") -> Prologue:
    """fmt = "fp16": the rows are IEEE half bits (the reference kernels' input type,
    tools/fused_threshold_topr_pack_ext_v57.py:32-35: the same 15-bit magnitude keys); no rotation then."""
    if fmt not in ("bf16", "fp16") or (fmt == "fp16" and kind != HAD_NONE):
        raise ValueError("fp16 rows are taken as they are (kind = HAD_NONE)")
    xr = rotate_bf16(x_bits, kind)
    M, K = xr.shape
    sel = select_tail(xr, R, descending_rank)
    xf = bf16_bits_to_f32(xr) if fmt == "bf16" else f16_bits_to_f32(xr)
    bscale = act_scale(sel.body_key, eps, fmt)
    tscale = act_scale(sel.top_key, eps, fmt)
    codes = quant_s4(xf, bscale)
    codes[sel.tail_mask] = 0
    if R:
        tail_val = np.take_along_axis(xr, sel.idx.astype(np.int64), axis=1)
        top_q = np.take_along_axis(quant_s4(xf, tscale), sel.idx.astype(np.int64), axis=1)
    else:
        tail_val = np.zeros((M, 0), np.uint16)
        top_q = np.zeros((M, 0), np.int8)
    return Prologue(xr, codes, pack_s4(codes), bscale, tscale, sel.idx, tail_val, top_q)


# ----------------------------------------------------------------------------- weights
@dataclass
class PreparedWeight:
    w_rot: np.ndarray    # [N, K] uint16 bf16 bits of the rotated weight
    codes: np.ndarray    # [N, K] int8
    b_col: np.ndarray    # [N, K/2] uint8, K-contiguous per output channel
    b_row: np.ndarray    # [K, N/2] uint8, low nibble = even n
    w_scale: np.ndarray  # [N] f32
    _codes_f64_t: Optional[np.ndarray] = None  # [K, N] float64 copy of the codes (cache for int_gemm)
    _w_t_f32: Optional[np.ndarray] = None      # [K, N] float32 rotated weight (cache for tail_t16)

    def codes_f64_t(self) -> np.ndarray:
        if self._codes_f64_t is None:
            self._codes_f64_t = np.ascontiguousarray(self.codes.T).astype(np.float64)
        return self._codes_f64_t

    def w_t_f32(self) -> np.ndarray:
        if self._w_t_f32 is None:
            self._w_t_f32 = np.ascontiguousarray(bf16_bits_to_f32(self.w_rot).T)
        return self._w_t_f32


def prepare_weight(w_bits: np.ndarray, kind: int, eps: float = EPS) -> PreparedWeight:
    """Rotate the input dim with the same transform as the activations, store back as
    16-bit (tools/bench_real_split_fullstack_rtn_ppl_v1.py:92-110), then RTN per output
    channel: scale = max(amax/7, eps) (tools/bench_multimodel_all_layers_policy_fastqf_v29.py:245-247),
    q = clamp(round(w/scale), -8, 7) (tools/bench_real_split_fullstack_rtn_ppl_v1.py:79-85)."""
    wr = rotate_bf16(w_bits, kind)
    wf = bf16_bits_to_f32(wr)
    amax = np.abs(wf).max(axis=1).astype(np.float32)
    scale = np.maximum((amax / np.float32(7.0)).astype(np.float32), np.float32(eps)).astype(np.float32)
    codes = quant_s4(wf, scale)
    return PreparedWeight(wr, codes, pack_s4(codes), pack_s4(np.ascontiguousarray(codes.T)), scale)


# ----------------------------------------------------------------------------- GEMM + tail
def int_gemm(qa: np.ndarray, qw) -> np.ndarray:
    """Exact int32 Qx . Qw^T (float64 BLAS is exact here: |sum| <= 64 K << 2^53).
    `qw` is an [N,K] int8 array or a PreparedWeight (whose float64 copy is cached)."""
    wt = qw.codes_f64_t() if isinstance(qw, PreparedWeight) else qw.astype(np.float64).T
    acc = qa.astype(np.float64) @ wt
    return np.rint(acc).astype(np.int32)


def dequant(acc: np.ndarray, s_x: np.ndarray, s_w: np.ndarray) -> np.ndarray:
    """(float(acc) * s_x[m]) * s_w[n] in fp32, in that order."""
    d = acc.astype(np.float32) * s_x.astype(np.float32).reshape(-1, 1)
    return (d * s_w.astype(np.float32).reshape(1, -1)).astype(np.float32)


def tail_t16(idx: np.ndarray, tail_val_bits: np.ndarray, w_rot_bits) -> np.ndarray:
    """sum_r x_tail[m,r] * W_rot[n, idx[m,r]] as a left-to-right fp32 fma chain in ascending
    index order.  bf16 x bf16 is exact in fp32, so fma(x, w, acc) == fl(acc + x*w).
    `w_rot_bits` is an [N,K] bf16-bit array or a PreparedWeight."""
    M, R = idx.shape
    if isinstance(w_rot_bits, PreparedWeight):
        wt = w_rot_bits.w_t_f32()
    else:
        wt = np.ascontiguousarray(bf16_bits_to_f32(w_rot_bits).T)  # [K, N]
    N = wt.shape[1]
    xv = bf16_bits_to_f32(tail_val_bits)
    acc = np.zeros((M, N), dtype=np.float32)
    for r in range(R):
        acc = acc + xv[:, r:r + 1] * wt[idx[:, r]]
    return acc


def tail_t16_chains(idx: np.ndarray, tail_val_bits: np.ndarray, w_rot_bits, chains: int = 8) -> np.ndarray:
    """The tail sum in the order of the small-M kernel: entry r goes to chain r mod `chains`, each chain is a
    left-to-right fp32 fma chain, and the chains are combined pairwise: ((c0+c1)+(c2+c3))+((c4+c5)+(c6+c7))."""
    M, R = idx.shape
    wt = w_rot_bits.w_t_f32() if isinstance(w_rot_bits, PreparedWeight) else \
        np.ascontiguousarray(bf16_bits_to_f32(w_rot_bits).T)
    N = wt.shape[1]
    xv = bf16_bits_to_f32(tail_val_bits)
    parts = [np.zeros((M, N), dtype=np.float32) for _ in range(chains)]
    for r in range(R):
        c = r % chains
        parts[c] = parts[c] + xv[:, r:r + 1] * wt[idx[:, r]]
    while len(parts) > 1:
        parts = [(parts[i] + parts[i + 1]).astype(np.float32) for i in range(0, len(parts), 2)]
    return parts[0]


def split_linear_t16(x_bits: np.ndarray, w: PreparedWeight, kind: int, R: int,
                     bias: Optional[np.ndarray] = None, descending_rank: Optional[int] = None,
                     tail_chains: int = 1):
    """Full path, tail mode T16.  Returns (bf16 bits [M,N], fp32 pre-rounding, Prologue, int32 acc).
    tail_chains = 1: one fma chain per output (prefill gather kernel); 8: the small-M kernel's order."""
    p = prologue(x_bits, kind, R, descending_rank)
    acc = int_gemm(p.codes, w)
    y = dequant(acc, p.body_scale, w.w_scale)
    if R:
        t = tail_t16(p.idx, p.tail_val, w) if tail_chains == 1 else tail_t16_chains(p.idx, p.tail_val, w, tail_chains)
        y = (y + t).astype(np.float32)
    if bias is not None:
        y = (y + bias.astype(np.float32).reshape(1, -1)).astype(np.float32)
    return f32_to_bf16_bits(y), y, p, acc


def rmsnorm_sum_layout(K: int) -> Tuple[int, int]:
    """(threads, chunk) of the sum of squares inside the fused prologue: the widths that have the specialised
    kernel (one thread per 64 contiguous elements) and the general kernel (256 threads, 16-element chunks)."""
    return (K // 64, 64) if K in (4096, 12288, 14336) else (256, 16)


def rmsnorm_bf16(x_bits: np.ndarray, gamma_bits: np.ndarray, eps: float = 1e-6, threads: Optional[int] = None,
                 chunk: Optional[int] = None) -> np.ndarray:
    """RMSNorm of bf16 rows as a bf16 framework rounds it (x * rsqrt(mean(x^2) + eps) in fp32 -> bf16, times the
    bf16 weight -> bf16; e.g. transformers' Qwen3RMSNorm), with the fp32 sum of squares taken in the order of the
    fused prologue kernel: thread t adds the squares of elements [chunk w, chunk w + chunk) for w = t, t + threads,
    ... one after the other, a butterfly (xor 16, 8, 4, 2, 1) adds the 32 threads of a warp, and the warp sums are
    added in order.  (threads, chunk) default to `rmsnorm_sum_layout(K)`."""
    M, K = x_bits.shape
    if threads is None or chunk is None:
        threads, chunk = rmsnorm_sum_layout(K)
    x = bf16_bits_to_f32(x_bits)
    chunks = K // chunk
    sq = (x * x).astype(np.float32).reshape(M, chunks, chunk)       # exact: squares of bf16 values fit fp32
    part = np.zeros((M, threads), np.float32)
    for w0 in range(0, chunks, threads):
        n = min(threads, chunks - w0)
        for e in range(chunk):
            part[:, :n] = (part[:, :n] + sq[:, w0:w0 + n, e]).astype(np.float32)
    lanes = part.reshape(M, threads // 32, 32)
    idx = np.arange(32)
    for o in (16, 8, 4, 2, 1):
        lanes = (lanes + lanes[:, :, idx ^ o]).astype(np.float32)
    warp = lanes[:, :, 0]
    tot = warp[:, 0].copy()
    for w in range(1, threads // 32):
        tot = (tot + warp[:, w]).astype(np.float32)
    mean = (tot / np.float32(K)).astype(np.float32)
    inv = (np.float32(1.0) / np.sqrt((mean + np.float32(eps)).astype(np.float32)).astype(np.float32)).astype(np.float32)
    xn = bf16_bits_to_f32(f32_to_bf16_bits((x * inv[:, None]).astype(np.float32)))
    return f32_to_bf16_bits((xn * bf16_bits_to_f32(gamma_bits)[None, :]).astype(np.float32))


def swiglu_bf16(y_bits: np.ndarray) -> np.ndarray:
    """SwiGLU over interleaved (gate, up) columns of a bf16 matrix [M, 2I] -> bf16 bits [M, I], evaluated the way
    a bf16 framework does on the two linears' outputs (the reference computes act(gate) * up in PyTorch,
    tools/bench_prefill_bf16_romeoquarotdense_split_total_v61_sharedprepare.py:214): silu(g) = g / (1 + exp(-g))
    in fp32, rounded to bf16, times up, rounded to bf16."""
    g = bf16_bits_to_f32(y_bits[:, 0::2])
    u = bf16_bits_to_f32(y_bits[:, 1::2])
    with np.errstate(over="ignore"):
        e = np.exp(-g, dtype=np.float32)
    s = bf16_bits_to_f32(f32_to_bf16_bits((g / (np.float32(1.0) + e)).astype(np.float32)))
    return f32_to_bf16_bits((s * u).astype(np.float32))


def sparse_int_t4(top_q: np.ndarray, idx: np.ndarray, w_codes: np.ndarray) -> np.ndarray:
    """sum_r top_q[m,r] * qw[n, idx[m,r]] in int32 (tools/fused_sparse_epilogue_ext_v58.py:59-74)."""
    M, R = idx.shape
    wt = np.ascontiguousarray(w_codes.T).astype(np.int32)  # [K, N]
    acc = np.zeros((M, w_codes.shape[0]), dtype=np.int32)
    for r in range(R):
        acc += top_q[:, r:r + 1].astype(np.int32) * wt[idx[:, r]]
    return acc


def epilogue_t4(acc: np.ndarray, body_scale: np.ndarray, sparse_acc: np.ndarray, top_scale: np.ndarray,
                w_scale: np.ndarray) -> np.ndarray:
    """fp32 value before the 16-bit rounding (tools/fused_sparse_epilogue_ext_v58.py:76-86):
    dense = float(C)*bs*ws ; sparse = float(acc)*ts*ws ; dense + sparse."""
    ws = w_scale.astype(np.float32).reshape(1, -1)
    dense = (acc.astype(np.float32) * body_scale.astype(np.float32).reshape(-1, 1)).astype(np.float32) * ws
    sparse = (sparse_acc.astype(np.float32) * top_scale.astype(np.float32).reshape(-1, 1)).astype(np.float32) * ws
    return (dense.astype(np.float32) + sparse.astype(np.float32)).astype(np.float32)


# ----------------------------------------------------------------------------- synthetic data
def make_activations(M: int, K: int, seed: int = 0, n_outlier: int = 16, outlier_scale: float = 50.0) -> np.ndarray:
    """N(0,1) with `n_outlier` fixed random channels scaled; bf16 bits."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K), dtype=np.float32)
    if n_outlier:
        ch = rng.permutation(K)[:n_outlier]
        x[:, ch] *= np.float32(outlier_scale)
    return f32_to_bf16_bits(x)


def make_weights(N: int, K: int, seed: int = 1, std: float = 0.02) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return f32_to_bf16_bits(rng.standard_normal((N, K), dtype=np.float32) * np.float32(std))
