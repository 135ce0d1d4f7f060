"""The no-allocation split-K linear (tq_int4_linear_splitk_noalloc), called through the C ABI, against the
existing entry points tq_int4_matmul(split_k) + tq_dequant_finish on the same inputs.

The entry point exists for hosts that cannot allocate device memory when they run a small-M linear (a serving
process whose pool owns the whole device, a C host loop that must not call cudaMalloc/cudaFree per token): its
int32 accumulators sit in a fixed array inside the library.  Because that array is shared by all calls and keeps
the last call's contents, the test makes two calls in a row with different shapes and data and requires both to
match bit for bit (integer accumulation and the same float operations: no tolerance is needed).

This file sorts last so that a run that stops at the first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _case(M, N, K, split_k, seed, with_tail, with_bias):
    from tailquant_kernel_b200 import _lib, ops
    rng = np.random.default_rng(seed)
    qa = rng.integers(-8, 8, size=(M, K)).astype(np.int8)
    qw = rng.integers(-8, 8, size=(N, K)).astype(np.int8)
    g = lambda a: torch.from_numpy(a).cuda()
    A, B = g(O.pack_s4(qa)), g(O.pack_s4(qw))
    sx = g(rng.uniform(0.001, 0.02, M).astype(np.float32))
    sw = g(rng.uniform(0.001, 0.02, N).astype(np.float32))
    tail = g(rng.standard_normal((M, N), dtype=np.float32)) if with_tail else None
    bias = g(rng.standard_normal(N, dtype=np.float32)) if with_bias else None

    # existing entry points, caller-supplied accumulator buffer
    C = torch.empty((M, N), dtype=torch.int32, device="cuda")
    want = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    ops.matmul_splitk(A, B, C, split_k)
    ops.dequant_finish(C, sx, sw, want, tail=tail, bias=bias)

    # new entry point, straight through ctypes
    lib = _lib.load()
    got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ptr = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    rc = lib.tq_int4_linear_splitk_noalloc(ptr(A), ptr(sx), ptr(B), ptr(sw), ptr(tail), ptr(bias), ptr(got), M, N, K,
                                           split_k, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.tq_error_string(rc)
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)), "differs from matmul_splitk + dequant_finish"
    # and against the CPU oracle's integer product
    assert np.array_equal(C.cpu().numpy(), O.int_gemm(qa, qw))


def test_no_alloc_splitk_linear_two_calls_in_a_row():
    _case(M=64, N=4096, K=1024, split_k=4, seed=1, with_tail=True, with_bias=True)   # fills 256 Ki accumulators
    _case(M=8, N=520, K=512, split_k=3, seed=2, with_tail=False, with_bias=False)    # reuses the start of the array
    _case(M=33, N=1032, K=4096, split_k=8, seed=3, with_tail=True, with_bias=False)


def test_no_alloc_rejects_sizes_beyond_its_array():
    from tailquant_kernel_b200 import _lib, ops
    lib = _lib.load()
    x = torch.zeros(64, dtype=torch.uint8, device="cuda")
    p = ctypes.c_void_p(x.data_ptr())
    rc = lib.tq_int4_linear_splitk_noalloc(p, p, p, p, None, None, p, 1025, 1024, 128, 1, None)
    assert rc == -6 and b"maximum" in lib.tq_error_string(rc)
    assert ops.NOALLOC_MAX_ELEMS == 1 << 20
