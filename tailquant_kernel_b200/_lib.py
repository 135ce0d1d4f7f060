"""ctypes binding of libtailquant.so (the C ABI declared in include/tailquant.h).

There is no fallback: if the library is missing or a call fails, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# TAILQUANT_LIB may point at another build of the same C ABI (e.g. an instrumented one)
LIB_PATH = os.environ.get("TAILQUANT_LIB") or os.path.join(HERE, "libtailquant.so")

TQ_HAD_NONE, TQ_HAD_WHT, TQ_HAD_KRON12, TQ_HAD_BLOCK128 = 0, 1, 2, 3
TQ_BF16, TQ_FP16 = 0, 1

_P, _I, _F, _LL = C.c_void_p, C.c_int, C.c_float, C.c_longlong

# name -> argument types; must list every function declared in include/tailquant.h
SIGNATURES = {
    "tq_version": [],
    "tq_error_string": [_I],
    "tq_last_cuda_error": [],
    "tq_split_prologue": [_P, _I, _I, _I, _I, _I, _F, _P, _P, _P, _P, _P, _P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P],
    # x, gamma, rms_eps, M, K, had, R, rank, eps, a_pack, a_q8, body, top, idx16, val, ld, ptr, pld, rec, cnt, dense, x_rot, stream
    "tq_split_prologue_rmsnorm": [_P, _P, _F, _I, _I, _I, _I, _I, _F, _P, _P, _P, _P, _P, _P, _I, _P, _I, _P, _P, _P, _P, _P],
    "tq_set_gemv_channel_tiles": [_I],
    "tq_split_gemm_mma": [_P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _P],
    "tq_split_gemm_mma_swiglu": [_P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _P],
    "tq_topr_pack": [_P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _F, _P],
    "tq_prepare_weight": [_P, _I, _I, _I, _F, _P, _P, _P, _P, _P, _P],
    "tq_int4_matmul": [_P, _P, _P, _I, _I, _I, _I, _P],
    "tq_split_gemm_fused": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "tq_dequant_finish": [_P, _P, _P, _P, _P, _P, _I, _I, _P],
    "tq_tail_gather": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "tq_scale_sparse_epilogue": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "tq_sparse_correction_add": [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "tq_sparse_top_write": [_P, _I, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _P],
    "tq_idx_i32_to_u16": [_P, _P, _LL, _P],
    "tq_int4_linear_splitk_noalloc": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    "tq_int4_gemv_splitk": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
    "tq_int4_gemv_plan": [_I, _I, _I, _I],
    "tq_int4_gemv_partials": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
    "tq_dequant_finish_partials": [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "tq_tail_gather_small": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "tq_set_gemm_pair_mode": [_I],
    "tq_set_prologue_mode": [_I],
    "tq_gemm_status": [_P],
}
_CHAR_P_RETURNS = {"tq_error_string", "tq_last_cuda_error"}

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m tailquant_kernel_b200.build` "
            "(there is no CPU or PyTorch fallback for this path)")
    lib = C.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.argtypes = argtypes
        fn.restype = C.c_char_p if name in _CHAR_P_RETURNS else C.c_int
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    lib = load()
    msg = lib.tq_error_string(rc).decode()
    if rc == -4:
        msg += ": " + lib.tq_last_cuda_error().decode()
    raise RuntimeError(f"{what}: {msg} (code {rc})")
