"""Pins both CPU restatements to the reference's own device code: tests/golden/reference_sm100.npz holds what
the reference's unmodified cuda/gemm.cu and cuda/gemv.cu kernels (compiled for sm_100) and its cublasLt call
sequence wrote on a B200 for seeded inputs (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

from oracle import quant_linear as ql

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_sm100.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN)


def f16(a):
    return a.view(np.float16)


@pytest.mark.parametrize("key", ["a", "w", "s", "e"])
def test_scales_and_codes(gold, c_oracle, key):
    x = f16(gold[key + "_x"])
    for impl in (ql, c_oracle):
        sr = impl.gemm_calc_scale(x)
        sc = impl.gemm_calc_scale_transpose(x)
        assert (sr.view(np.uint16) == gold[key + "_scale_rows"]).all()
        assert (sc.view(np.uint16) == gold[key + "_scale_cols"]).all()
        assert (impl.gemm_round(x, sr) == gold[key + "_codes_rows"]).all()
        assert (impl.gemm_round_transpose(x, sc) == gold[key + "_codes_cols"]).all()


def test_out_of_range_casts(gold, c_oracle):
    """Quotients beyond [-128, 127], infinite and NaN: the cast the reference's compiled code performs."""
    x, s = f16(gold["c_x"]), f16(gold["c_s"])
    for impl in (ql, c_oracle):
        assert (impl.gemm_round(x, s) == gold["c_codes"]).all()
    assert (np.abs(gold["c_codes"].astype(np.int32)) > 127).any() or (gold["c_codes"] == -128).any()


def test_dequant(gold, c_oracle):
    acc, sx, sy = gold["d_acc"], f16(gold["d_sx"]), f16(gold["d_sy"])
    for impl in (ql, c_oracle):
        assert (impl.gemm_scale(acc, sx, sy, False, False).view(np.uint16) == gold["d_out_ff"]).all()
        assert (impl.gemm_scale(acc, np.ascontiguousarray(sx[:1]), sy, True, False).view(np.uint16) == gold["d_out_tf"]).all()
        assert (impl.gemm_scale(acc, sx, np.ascontiguousarray(sy[:1]), False, True).view(np.uint16) == gold["d_out_ft"]).all()
        big = impl.gemm_scale(gold["d_big_acc"], f16(gold["d_big_sx"]), f16(gold["d_big_sy"]), False, False)
        assert (big.view(np.uint16) == gold["d_big_out"]).all()


def test_backward_helpers(gold, c_oracle):
    g, sy, sx = f16(gold["b_grad"]), f16(gold["b_sy"]), f16(gold["b_sx"])
    for impl in (ql, c_oracle):
        q, s = impl.gemm_backward_round_scale(g, sy, False)
        assert (q == gold["b_q_rows"]).all() and (s.view(np.uint16) == gold["b_s_rows"]).all()
        q, s = impl.gemm_backward_scale_round(g, sx, True)
        assert (q == gold["b_q_cols"]).all() and (s.view(np.uint16) == gold["b_s_cols"]).all()


def test_gemv_within_the_references_own_tolerance(gold, c_oracle):
    """The reference's GEMV kernels accumulate in fp16 pairs (cuda/gemv.cu:92-97); its tests accept 5e-2
    (tests/test_gemv.py:103).  The oracle is the exact sum; the reference's outputs must lie within that bound."""
    mat, vec = f16(gold["v_mat"]), f16(gold["v_vec"])
    want = ql.gemv_fp16(mat, vec)
    assert np.isclose(f16(gold["v_out_rows"]).astype(np.float64), want, rtol=5e-2, atol=5e-2).all()
    mt = np.ascontiguousarray(mat.transpose(0, 2, 1))
    assert np.isclose(f16(gold["v_out_transpose"]).astype(np.float64), ql.gemv_fp16_transpose(mt, vec), rtol=5e-2, atol=5e-2).all()
    assert np.isclose(f16(gold["v_out_shared"]).astype(np.float64), ql.gemv_broadcast_mat_fp16(mat[0], vec), rtol=5e-2, atol=5e-2).all()
    for impl in (ql, c_oracle):
        got = impl.gemv_broadcast_mat_int8(f16(gold["v_sm"]), gold["v_qm"], f16(gold["v_sv"]), gold["v_qv"])
        assert (got.view(np.uint16) == gold["v_out_int8"]).all()


def test_int8_gemm_against_cublaslt(gold, c_oracle):
    """The reference's cublasLt call sequence, for every storage order the library accepted on the B200."""
    seen = 0
    for aT in (0, 1):
        for bT in (0, 1):
            tag = "g_%d%d" % (aT, bT)
            if tag + "_out" not in gold.files:
                continue
            seen += 1
            A, B = gold[tag + "_A"], gold[tag + "_B"]
            for impl in (ql, c_oracle):
                assert (impl.gemm_int8(16, 32, 8, bool(aT), bool(bT), A, B) == gold[tag + "_out"]).all()
    assert seen >= 1


def test_gelu_restatements_match_the_reference_on_every_fp16_value():
    """tests/golden/reference_gelu_sm100.npz holds the reference's cu_gelu_forward on all 65536 fp16 bit patterns."""
    import os
    table = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_gelu_sm100.npz"))["gelu_of_every_fp16"]
    x = np.arange(65536, dtype=np.uint16).view(np.float16)
    assert (ql.gelu_forward(x).view(np.uint16) == table).all()
    assert (ql.COracle().gelu_forward(x).view(np.uint16) == table).all()


def test_layernorm_chain_restatement_matches_the_reference():
    """tests/golden/reference_layernorm_sm100.npz: the reference's layer norm -> affine -> column quantisation chain.
    The restatement reproduces the affine step, the scales and the codes exactly; the normalised tensor itself
    differs in at most a handful of elements by one fp16 step (the device's rsqrtf is not correctly rounded)."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_layernorm_sm100.npz"))
    cases = {"mean_bias": (1e-5, True), "rms": (1e-6, False), "ragged": (1e-5, True), "hidden4096": (1e-6, False),
             "ragged_rms_bias": (1e-5, False)}
    ln_mismatches = 0
    for name, (eps, rd_mean) in cases.items():
        x = g[name + "_x"].view(np.float16)
        alpha = g[name + "_alpha"].view(np.float16)
        beta = g[name + "_beta"].view(np.float16) if name + "_beta" in g else None
        ln = ql.layernorm_forward(x, eps, rd_mean)
        want_ln = g[name + "_ln"].view(np.float16)
        differ = ln.view(np.uint16) != want_ln.view(np.uint16)
        ln_mismatches += int(differ.sum())
        assert np.abs(ln[differ].view(np.int16).astype(np.int32) - want_ln[differ].view(np.int16).astype(np.int32)).max(initial=0) <= 1
        aff = ql.arith_ln_mul_add(want_ln, alpha, beta) if beta is not None else ql.arith_ln_mul(want_ln, alpha)
        assert (aff.view(np.uint16) == g[name + "_affine"]).all()
        scale, codes = ql.layernorm_quantize_cols(x, eps, rd_mean, alpha, beta)
        assert (scale.view(np.uint16) == g[name + "_scale"]).all()
        assert (codes == g[name + "_codes"]).all()
    assert ln_mismatches <= 3


def test_transpose_oracle_by_definition():
    """cuda/transpose.cu:6-22: out[b, c, r] = in[b, r, c], checked element by element on a small ragged case."""
    rng = np.random.default_rng(4)
    x = rng.integers(0, 65536, size=(3, 5, 7), dtype=np.uint16).view(np.float16)
    y = ql.transpose(x)
    assert y.shape == (3, 7, 5) and y.flags["C_CONTIGUOUS"]
    for b in range(3):
        for r in range(5):
            for c in range(7):
                assert y.view(np.uint16)[b, c, r] == x.view(np.uint16)[b, r, c]
