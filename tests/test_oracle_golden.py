"""The numpy oracle against vectors produced by the reference's own Python functions
(tests/golden/make_golden.py) and against its own algebraic properties."""
import json
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def vec():
    return np.load(os.path.join(GOLD, "reference_vectors.npz"))


def test_scalars_match_reference():
    for row in json.load(open(os.path.join(GOLD, "scalars.json"))):
        R = O.ceil_ratio_count(row["K"], row["ratio"])
        assert R == row["R"], row
        _, dr, sk = O.split_select_params(row["K"], R, row["pct"])
        assert (dr, sk) == (row["descending_rank"], row["select_k"]), row


def test_nibble_order(vec):
    packed = vec["nibble_packed"].reshape(1, -1)
    assert np.array_equal(O.unpack_s4(packed).reshape(-1), vec["nibble_decoded"].reshape(-1))
    assert np.array_equal(O.pack_s4(O.unpack_s4(packed)), packed)


def test_select_and_fake_quant(vec):
    for ci in range(int(vec["n_cases"][0])):
        xb = vec[f"c{ci}_x_bits"]
        M, K, R = (int(v) for v in vec[f"c{ci}_meta"])
        pct = float(vec[f"c{ci}_pct"][0])
        _, dr, _ = O.split_select_params(K, R, pct)
        sel = O.select_tail(xb, R, dr)
        assert np.array_equal(sel.idx, vec[f"c{ci}_idx"]), ci
        assert np.array_equal(O.bf16_bits_to_f32(sel.body_key), vec[f"c{ci}_body_thr"]), ci
        assert np.array_equal(O.bf16_bits_to_f32(sel.top_key), vec[f"c{ci}_tail_thr"]), ci
        p = O.prologue(xb, O.HAD_NONE, R, dr)
        recon = p.codes.astype(np.float32) * p.body_scale.reshape(-1, 1)
        tq = p.top_q.astype(np.float32) * p.top_scale.reshape(-1, 1)
        np.put_along_axis(recon, p.idx.astype(np.int64), tq, axis=1)
        gold = vec[f"c{ci}_recon"]
        x = O.bf16_bits_to_f32(xb)
        thr = vec[f"c{ci}_body_thr"].reshape(-1, 1)
        # the fake path clamps to +-thr before rounding, the kernels only clamp the code;
        # they can differ only for body entries below -thr (code -8 instead of -7)
        inside = ~((x < -thr) & ~sel.tail_mask)
        assert np.array_equal(recon[inside], gold[inside]), ci
        if pct == 100.0:
            assert inside.all()
        diff = ~inside
        assert np.all(np.isin(p.codes[diff], (-8, -7)))


def test_rtn_weights(vec):
    w = O.prepare_weight(vec["rtn_w_bits"], O.HAD_NONE)
    assert np.array_equal(w.w_scale, vec["rtn_scale"])
    assert np.array_equal(w.codes.astype(np.float32) * w.w_scale.reshape(-1, 1), vec["rtn_wq"])
    assert np.array_equal(O.unpack_s4(w.b_col), w.codes)
    assert np.array_equal(O.unpack_s4(w.b_row), w.codes.T)


def test_tie_rule_lowest_index_first():
    # tools/fused_threshold_topr_pack_ext_v57.py:141-181: all keys above the threshold in
    # index order, then equal keys in index order until R entries are taken.
    x = np.array([[1.0, -2.0, 2.0, 0.5, 2.0, -2.0, 3.0, 0.25]], dtype=np.float32)
    xb = O.f32_to_bf16_bits(x)
    sel = O.select_tail(xb, 3)
    assert sel.idx.tolist() == [[1, 2, 6]]
    assert O.bf16_bits_to_f32(sel.body_key).tolist() == [2.0]
    sel = O.select_tail(xb, 5)
    assert sel.idx.tolist() == [[1, 2, 4, 5, 6]]
    assert O.bf16_bits_to_f32(sel.body_key).tolist() == [1.0]


@pytest.mark.parametrize("kind,K", [(O.HAD_WHT, 64), (O.HAD_WHT, 4096), (O.HAD_KRON12, 12 * 64),
                                    (O.HAD_KRON12, 12288), (O.HAD_BLOCK128, 14336), (O.HAD_BLOCK128, 256)])
def test_rotation_is_orthogonal(kind, K):
    rng = np.random.default_rng(0)
    x = O.round_bf16(rng.standard_normal((3, K), dtype=np.float32))
    y = O.rotate_f32(x, kind) * O.had_scale(kind, K)
    # norm preserved, and an explicit matrix gives the same numbers up to fp32 rounding
    assert np.allclose((y.astype(np.float64) ** 2).sum(1), (x.astype(np.float64) ** 2).sum(1), rtol=1e-5)
    if K <= 4096:
        eye = np.eye(K, dtype=np.float32)
        Q = O.rotate_f32(eye, kind).astype(np.float64) * float(O.had_scale(kind, K))
        assert np.allclose(Q @ Q.T, np.eye(K), atol=1e-5)
        assert np.allclose(x.astype(np.float64) @ Q, y, atol=1e-4)


def test_hadamard12():
    H = O.hadamard12()
    assert np.array_equal(H @ H.T, 12 * np.eye(12, dtype=np.int32))
    assert set(np.unique(H)) == {-1, 1}


def test_bf16_rounding():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.140625, 1e-40, 65504.0, 3.3895314e38], dtype=np.float32)
    import torch
    ref = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.f32_to_bf16_bits(x), ref)
    rng = np.random.default_rng(1)
    r = rng.standard_normal(100000, dtype=np.float32) * 100
    ref = torch.from_numpy(r).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.f32_to_bf16_bits(r), ref)


def test_split_linear_close_to_float_linear():
    M, K, N, R = 32, 256, 48, 13
    xb = O.make_activations(M, K, seed=0, n_outlier=4)
    wb = O.make_weights(N, K, seed=1)
    w = O.prepare_weight(wb, O.HAD_WHT)
    yb, y32, p, acc = O.split_linear_t16(xb, w, O.HAD_WHT, R)
    ref = O.bf16_bits_to_f32(xb).astype(np.float64) @ O.bf16_bits_to_f32(wb).astype(np.float64).T
    rel = np.linalg.norm(y32 - ref) / np.linalg.norm(ref)
    assert rel < 0.2  # W4A4: a sanity bound, not a parity bound
    # the tail must reduce the error compared with R = 0
    y0 = O.split_linear_t16(xb, w, O.HAD_WHT, 0)[1]
    assert np.linalg.norm(y32 - ref) < np.linalg.norm(y0 - ref)
    # T4 mode (reference-compatible) is self-consistent
    sp = O.sparse_int_t4(p.top_q, p.idx, w.codes)
    y4 = O.epilogue_t4(acc, p.body_scale, sp, p.top_scale, w.w_scale)
    assert np.linalg.norm(y4 - ref) / np.linalg.norm(ref) < 0.25
