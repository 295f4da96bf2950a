"""The two CPU restatements (numpy, C) agree bit for bit, on random data and on the edge cases."""
import numpy as np
import pytest

from oracle import quant_linear as ql
from util import randn_fp16, np16, bits, edge_case_matrix

SHAPES = [(1, 4, 4), (2, 4, 8), (3, 12, 12), (1, 33, 40), (2, 17, 128), (1, 64, 500)]


@pytest.mark.parametrize("shape", SHAPES)
def test_scales_and_codes(c_oracle, shape):
    x = np16(randn_fp16(shape, seed=sum(shape)))
    s_r, s_c = ql.gemm_calc_scale(x), ql.gemm_calc_scale_transpose(x)
    assert (bits(s_r) == bits(c_oracle.gemm_calc_scale(x))).all()
    assert (bits(s_c) == bits(c_oracle.gemm_calc_scale_transpose(x))).all()
    assert (ql.gemm_round(x, s_r) == c_oracle.gemm_round(x, s_r)).all()
    assert (ql.gemm_round_transpose(x, s_c) == c_oracle.gemm_round_transpose(x, s_c)).all()
    assert np.abs(ql.gemm_round(x, s_r).astype(np.int32)).max() == 127


def test_edge_cases_agree(c_oracle):
    x = np16(edge_case_matrix())
    s_r, s_c = ql.gemm_calc_scale(x), ql.gemm_calc_scale_transpose(x)
    assert (bits(s_r) == bits(c_oracle.gemm_calc_scale(x))).all()
    assert (bits(s_c) == bits(c_oracle.gemm_calc_scale_transpose(x))).all()
    assert (ql.gemm_round(x, s_r) == c_oracle.gemm_round(x, s_r)).all()
    assert (ql.gemm_round_transpose(x, s_c) == c_oracle.gemm_round_transpose(x, s_c)).all()
    # scale semantics: NaN elements are dropped from the max, inf is kept, zero row gives scale 0
    assert s_r[0, 0] == 0 and np.isfinite(s_r[0, 3]) and np.isinf(s_r[0, 4])
    # ties round to even with scale exactly 1
    assert s_r[0, 7] == np.float16(1.0)
    q = ql.gemm_round(x, s_r)[0, 7, 1:40]
    assert (q % 2 == 0).all()


@pytest.mark.parametrize("aT,bT", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("bA,bB", [(1, 1), (2, 2), (1, 3), (3, 1)])
def test_gemm_int8_layouts(c_oracle, aT, bT, bA, bB):
    m, k, n = 12, 20, 8
    rng = np.random.default_rng(m + k + n + bA * 7 + bB)
    A = rng.integers(-127, 128, (bA, m, k) if aT else (bA, k, m), dtype=np.int8)
    B = rng.integers(-127, 128, (bB, k, n) if bT else (bB, n, k), dtype=np.int8)
    got = ql.gemm_int8(m, k, n, aT, bT, A, B)
    want = c_oracle.gemm_int8(m, k, n, aT, bT, A, B)
    assert (got == want).all()
    # first principles
    a = (A.transpose(0, 2, 1) if aT else A).astype(np.int64)     # (bA, k, m)
    b = (B.transpose(0, 2, 1) if bT else B).astype(np.int64)     # (bB, n, k)
    assert (np.matmul(b, a) == got).all()


def test_dequant_and_bmm(c_oracle):
    A = np16(randn_fp16((2, 12, 20), 3))
    B = np16(randn_fp16((1, 20, 8), 4, std=0.02))
    r = ql.bmm_int8(A, False, B, False)
    acc = c_oracle.gemm_int8(8, 20, 12, False, False, r["quant_B"], r["quant_A"])
    assert (acc == r["acc"]).all()
    out = c_oracle.gemm_scale(acc, r["scale_A"], r["scale_B"], False, True)
    assert (bits(out) == bits(r["out"])).all()
    assert (bits(c_oracle.gemm_scale_x(acc, r["scale_A"])) == bits(ql.gemm_scale_x(acc, r["scale_A"]))).all()
    sB2 = np.repeat(r["scale_B"], 2, axis=0)
    assert (bits(c_oracle.gemm_scale_y(acc, sB2)) == bits(ql.gemm_scale_y(acc, sB2))).all()
    # the reference's own (looser) test formula agrees within its tolerance (tests/test_gemm.py:98)
    import torch
    from oracle import test_formula
    ans = test_formula.real_bmm(torch.from_numpy(A), False, torch.from_numpy(B), False, True).numpy()
    assert np.isclose(r["out"].astype(np.float32), ans.astype(np.float32), rtol=0.5, atol=0.5).all()


def test_backward_helpers(c_oracle):
    g = np16(randn_fp16((2, 10, 16), 5))
    sy = np.abs(np16(randn_fp16((2, 16), 6, std=0.01))) + np.float16(1e-3)
    sx = np.abs(np16(randn_fp16((1, 10), 8, std=0.01))) + np.float16(1e-3)
    q1, s1 = ql.gemm_backward_round_scale(g, sy, False)
    q1c, s1c = c_oracle.gemm_backward_round_scale(g, sy, False)
    assert (q1 == q1c).all() and (bits(s1) == bits(s1c)).all()
    q2, s2 = ql.gemm_backward_scale_round(g, sx, True)
    q2c, s2c = c_oracle.gemm_backward_scale_round(g, sx, True)
    assert (q2 == q2c).all() and (bits(s2) == bits(s2c)).all()


def test_gemv(c_oracle):
    mat = np16(randn_fp16((3, 10, 24), 9, std=0.02))
    vec = np16(randn_fp16((3, 24), 10))
    assert np.allclose(ql.gemv_fp16(mat, vec), c_oracle.gemv_fp16(mat, vec), rtol=1e-12, atol=1e-12)
    mt = np.ascontiguousarray(mat.transpose(0, 2, 1))
    assert np.allclose(ql.gemv_fp16_transpose(mt, vec), c_oracle.gemv_fp16_transpose(mt, vec), rtol=1e-12, atol=1e-12)
    assert np.allclose(ql.gemv_broadcast_mat_fp16(mat[0], vec), c_oracle.gemv_broadcast_mat_fp16(mat[0], vec), rtol=1e-12, atol=1e-12)
    rng = np.random.default_rng(0)
    qm = rng.integers(-127, 128, (10, 24), dtype=np.int8)
    qv = rng.integers(-127, 128, (3, 24), dtype=np.int8)
    sm = np.abs(np16(randn_fp16((10,), 11, std=0.01)))
    sv = np.abs(np16(randn_fp16((3,), 12, std=0.01)))
    assert (bits(ql.gemv_broadcast_mat_int8(sm, qm, sv, qv)) == bits(c_oracle.gemv_broadcast_mat_int8(sm, qm, sv, qv))).all()


def test_test_formula_differs_from_kernel_formula_as_documented():
    """The reference's unit-test formula keeps the scale in fp32; a fraction of a percent of the codes differ by one."""
    x = np16(randn_fp16((1, 64, 2560), 0))
    q_kernel = ql.gemm_round(x, ql.gemm_calc_scale(x)).astype(np.int32)
    xf = x.astype(np.float32)
    q_test = np.rint(xf / (np.abs(xf).max(-1, keepdims=True) / np.float32(127))).astype(np.int32)
    diff = np.abs(q_kernel - q_test)
    assert diff.max() <= 1 and 0 < (diff != 0).mean() < 0.02
