"""Pins the CPU oracle against the reference's own known-answer vectors (tests/golden/*.json,
generated from the reference tree by tests/golden/make_golden.py) and checks the oracle's two
implementations (NumPy and plain C) against each other."""
import ctypes as C
import json
import math
import os
import subprocess

import numpy as np
import pytest

from oracle import scaled_dot_oracle as o

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _val(s):
    return {"nan": math.nan, "inf": math.inf, "-inf": -math.inf}.get(s, None) if s in ("nan", "inf", "-inf") else float.fromhex(s)


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(HERE, "golden", "fp8_convert_roundtrip.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def c_oracle():
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle")], stdout=subprocess.DEVNULL)
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_build", "liboracle.so"))
    lib.oracle_fp8_decode.restype = C.c_float
    lib.oracle_fp8_decode.argtypes = [C.c_uint8, C.c_int]
    lib.oracle_fp8_encode.restype = C.c_uint8
    lib.oracle_fp8_encode.argtypes = [C.c_float, C.c_int]
    lib.oracle_f32_to_bf16.restype = C.c_uint16
    lib.oracle_f32_to_bf16.argtypes = [C.c_float]
    lib.oracle_scaled_dot_f8.restype = C.c_float
    lib.oracle_scaled_dot_f8.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_int, C.c_int, C.c_int64,
                                         C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_float, C.c_float, C.c_void_p,
                                         C.c_void_p, C.c_int, C.c_void_p]
    lib.oracle_dot_s8.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_void_p]
    return lib


@pytest.mark.parametrize("table", ["ConvertF16F8e5m2Roundtrip", "ConvertF32F8e5m2Roundtrip",
                                   "ConvertF16F8e4m3fnRoundtrip", "ConvertF32F8e4m3fnRoundtrip"])
def test_reference_roundtrip_tables(golden, c_oracle, table):
    """xla/tests/convert_test.cc: value -> FP8 -> value must give the listed result exactly."""
    t = golden["tables"][table]
    kind = t["fp8"]
    assert len(t["cases"]) >= 20
    for src, want in t["cases"]:
        x, w = _val(src), _val(want)
        xin = np.float32(np.float16(x)) if t["via"] == "f16" else np.float32(x)
        got = float(o.fp8_decode(o.fp8_encode(np.array([xin], np.float32), kind), kind)[0])
        got_c = c_oracle.oracle_fp8_decode(c_oracle.oracle_fp8_encode(float(xin), 0 if kind == "e4m3fn" else 1),
                                           0 if kind == "e4m3fn" else 1)
        for g in (got, got_c):
            if math.isnan(w):
                assert math.isnan(g), (table, src, g)
            else:
                assert g == w, (table, src, g, w)        # ErrorSpec(0.): value equality (-0 == 0)


def test_e8m0_roundtrip_table(golden):
    """xla/tests/convert_test.cc:2114-2152 (ConvertF32F8e8m0fnuRoundtrip): the block-scale type."""
    t = golden["tables"]["ConvertF32F8e8m0fnuRoundtrip"]
    assert t["fp8"] == "e8m0fnu" and len(t["cases"]) >= 14
    for src, want in t["cases"]:
        x, w = np.float32(_val(src)), _val(want)
        g = float(o.e8m0_decode(o.e8m0_encode(np.array([x], np.float32)))[0])
        assert (math.isnan(w) and math.isnan(g)) or g == w, (src, g, w)
    # ConvertF8e8m0fnuRoundtripExhaustive (:2154-2172): every code point survives f8 -> f32 -> f8.
    codes = np.arange(256, dtype=np.uint8)
    assert (o.e8m0_encode(o.e8m0_decode(codes)) == codes).all()
    assert o.e8m0_decode(np.array([0, 127, 254], np.uint8)).tolist() == [2.0 ** -127, 1.0, 2.0 ** 127]


def test_block_scaled_dot_is_the_expanded_hlo():
    """block_scaling_rewriter.cc:194-262: dequantize(a) . dequantize(b)^T with the scale broadcast over
    blocks of 32 along K; checked against a literal loop on a small case and against hand values."""
    a, b, sa, sb = o.make_mx_operands(9, 5, 3, 64, batch=2)
    got = o.block_scaled_dot(a, b, sa, sb)
    av, bv = o.fp8_decode(a).astype(np.float64), o.fp8_decode(b).astype(np.float64)
    for bt in range(2):
        for i in range(5):
            for j in range(3):
                acc = 0.0
                for kk in range(64):
                    acc += av[bt, i, kk] * 2.0 ** (int(sa[bt, i, kk // 32]) - 127) * bv[bt, j, kk] * 2.0 ** (int(sb[bt, j, kk // 32]) - 127)
                assert abs(got[bt, i, j] - acc) <= 1e-5 * max(1.0, abs(acc))
    one = o.fp8_encode(np.array([1.0], np.float32))[0]
    d = o.block_scaled_dot(np.full((1, 64), one, np.uint8), np.full((1, 64), one, np.uint8),
                           np.array([[128, 126]], np.uint8), np.array([[127, 130]], np.uint8))
    assert d.tolist() == [[32 * 2.0 + 32 * 0.5 * 8.0]]
    assert np.isnan(o.block_scaled_dot(np.full((1, 32), one, np.uint8), np.full((1, 32), one, np.uint8),
                                       np.array([[255]], np.uint8), np.array([[127]], np.uint8))).all()


@pytest.mark.parametrize("kind", ["e4m3fn", "e5m2"])
def test_exhaustive_roundtrips(c_oracle, kind):
    """ConvertF8e4m3fnRoundtripExhaustive{,2,3} / the e5m2 twins: all 256 code points survive
    FP8 -> f32 -> FP8, and FP8 -> bf16/f16 -> FP8 (every FP8 value is exact in those types)."""
    codes = np.arange(256, dtype=np.uint8)
    vals = o.fp8_decode(codes, kind)
    back = o.fp8_encode(vals, kind)
    nan = np.isnan(vals)
    assert np.array_equal(back[~nan], codes[~nan])
    assert np.isnan(o.fp8_decode(back[nan], kind)).all()
    ck = 0 if kind == "e4m3fn" else 1
    for c in range(256):
        v = c_oracle.oracle_fp8_decode(c, ck)
        assert (math.isnan(v) and nan[c]) or v == vals[c]
        if not nan[c]:
            assert c_oracle.oracle_fp8_encode(v, ck) == c
    via_bf16 = o.bf16_bits_to_f32(o.f32_to_bf16_bits(vals[~nan]))
    assert np.array_equal(via_bf16, vals[~nan])
    assert np.array_equal(vals[~nan].astype(np.float16).astype(np.float32), vals[~nan])


@pytest.mark.parametrize("kind", ["e4m3fn", "e5m2"])
def test_all_f16_inputs_numpy_vs_c(c_oracle, kind):
    """ConvertF8e4m3fnF16RoundtripExhaustive4: every f16 bit pattern -> FP8; the two oracle
    implementations must agree everywhere (a sample keeps the ctypes loop short)."""
    x = np.arange(0, 65536, 7, dtype=np.uint16).view(np.float16).astype(np.float32)
    enc = o.fp8_encode(x, kind)
    ck = 0 if kind == "e4m3fn" else 1
    for xi, e in zip(x.tolist(), enc.tolist()):
        g = c_oracle.oracle_fp8_encode(xi, ck)
        if math.isnan(xi):
            assert math.isnan(c_oracle.oracle_fp8_decode(g, ck))
        else:
            assert g == e, (xi, g, e)


def test_optional_cross_check_with_ml_dtypes():
    ml = pytest.importorskip("ml_dtypes")
    for kind, t in (("e4m3fn", ml.float8_e4m3fn), ("e5m2", ml.float8_e5m2)):
        rng = np.random.default_rng(0)
        x = np.concatenate([rng.standard_normal(50000).astype(np.float32) * 200,
                            rng.integers(0, 2 ** 32, 200000, dtype=np.uint64).astype(np.uint32).view(np.float32)])
        with np.errstate(all="ignore"):
            ref = x.astype(t).view(np.uint8)
        mine = o.fp8_encode(x, kind)
        ref_nan = np.isnan(ref.view(t).astype(np.float32))
        assert np.array_equal(ref_nan, np.isnan(o.fp8_decode(mine, kind)))
        assert np.array_equal(ref[~ref_nan], mine[~ref_nan])


def test_bf16_rounding_numpy_vs_c(c_oracle):
    x = np.random.default_rng(1).integers(0, 2 ** 32, 20000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    bits = o.f32_to_bf16_bits(x)
    for xi, b in zip(x.tolist(), bits.tolist()):
        if not math.isnan(xi):
            assert c_oracle.oracle_f32_to_bf16(xi) == b
    # ties to even
    assert o.f32_to_bf16_bits(np.array([1.00390625], np.float32))[0] == 0x3F80     # 1 + 2^-8 -> 1.0
    assert o.f32_to_bf16_bits(np.array([1.01171875], np.float32))[0] == 0x3F82     # 1 + 3*2^-8 -> 1 + 2^-6


def test_s8_known_answer():
    """cuda_blas_lt_test.cc:48-156 on the oracle: 32^3 all ones -> 32 everywhere."""
    with open(os.path.join(HERE, "golden", "s8_known_answer.json")) as f:
        ka = json.load(f)
    a = np.full((ka["m"], ka["k"]), ka["a_fill"], np.int8)
    b = np.full((ka["k"], ka["n"]), ka["b_fill"], np.int8)
    assert (o.dot_s8(a, b) == ka["expected_every_element"]).all()


@pytest.mark.parametrize("lc,rc", [(1, 0), (0, 0), (1, 1), (0, 1)])
def test_numpy_dot_matches_strict_c_interpreter_order(c_oracle, lc, rc):
    """BLAS order (used for big shapes) vs the strict sequential-k C restatement: 1e-5 relative."""
    m, k, n = 48, 160, 64
    a, b, sa, sb = o.make_f8_operands(70, m, k, n)
    a_st = a if lc == 1 else np.ascontiguousarray(a.T)
    b_st = b if rc == 0 else np.ascontiguousarray(b.T)
    bias = o.bf16_bits_to_f32(o.make_bias_bf16(70, n))
    out = np.zeros((m, n), np.float32)
    amax_c = c_oracle.oracle_scaled_dot_f8(a_st.ctypes.data, b_st.ctypes.data, float(sa), float(sb), 0, 0, m, n, k,
                                           lc, rc, 1.0, 0.0, None, bias.ctypes.data, 7, out.ctypes.data)
    exp, amax = o.scaled_dot_f8(a_st, b_st, sa, sb, lhs_contracting=lc, rhs_contracting=rc, bias=bias, epilogue=o.EPI_BIAS_GELU,
                                out_dtype=o.F32, want_amax=True)
    np.testing.assert_allclose(exp, out, rtol=1e-5, atol=1e-6)
    assert abs(amax - amax_c) <= 1e-5 * abs(amax_c)
    strict, _ = o.scaled_dot_f8(a_st, b_st, sa, sb, lhs_contracting=lc, rhs_contracting=rc, bias=bias, epilogue=o.EPI_BIAS_GELU,
                                out_dtype=o.F32, strict=True)
    np.testing.assert_allclose(strict, out, rtol=1e-5, atol=1e-6)


def test_s8_dot_numpy_vs_c(c_oracle):
    a, b, _, _ = o.make_s8_operands(3, 40, 96, 56)
    out = np.zeros((40, 56), np.int32)
    c_oracle.oracle_dot_s8(a.ctypes.data, b.ctypes.data, 40, 56, 96, 1, 0, out.ctypes.data)
    assert np.array_equal(out, o.dot_s8(a, b))
    assert np.array_equal(out, a.astype(np.int64) @ b.astype(np.int64))


def test_nan_rules():
    """maximum and clamp propagate NaN (hlo_evaluator_typed_visitor.h:594-613, 843-865)."""
    a, b, sa, sb = o.make_f8_operands(71, 16, 32, 16)
    a = a.copy()
    a[3, 4] = 0x7F
    d, amax = o.scaled_dot_f8(a, b, sa, sb, d_scale=1.0, out_dtype=o.F8E4M3FN, want_amax=True)
    assert np.isnan(amax)
    assert ((d[3] & 0x7F) == 0x7F).all() and ((d[2] & 0x7F) != 0x7F).all()
    assert o.fp8_encode_saturating(np.array([1e9, -1e9, np.inf, 500.0], np.float32)).tolist() == [0x7E, 0xFE, 0x7E, 0x7E]


def test_near_comparison_rule():
    """literal_comparison.cc:528-535: mismatch needs BOTH bounds exceeded; NaN == NaN; inf must match."""
    exp = np.array([1.0, 100.0, 0.0, np.nan, np.inf, 1.0], np.float32)
    act = np.array([1.005, 100.5, 0.005, np.nan, np.inf, 1.02], np.float32)
    bad, _, _ = o.near_mismatches(exp, act, 1e-2, 1e-2)
    assert bad == 1          # only 1.0 vs 1.02 exceeds both
    assert o.near_mismatches(np.array([np.inf]), np.array([1e30]), 1e-2, 1e-2)[0] == 1
    assert o.near_mismatches(np.array([1.0]), np.array([np.nan]), 1e-2, 1e-2)[0] == 1
    assert o.fp8_within_n_values(np.array([0x38, 0x38, 0x81], np.uint8), np.array([0x39, 0x3A, 0x01], np.uint8), 1) == 2


def _fill_unique(dims, start):
    """Array2D::FillUnique / Array3D::FillUnique (xla/array2d.h:78-85, xla/array3d.h:65-76): every index shifted into
    its own bit field, plus the start value."""
    def log2ceil(n):
        return int(math.ceil(math.log2(n))) if n > 1 else 0

    out = np.zeros(dims, np.float32)
    if len(dims) == 2:
        shift = log2ceil(dims[1])
        for i0 in range(dims[0]):
            for i1 in range(dims[1]):
                out[i0, i1] = ((i0 << shift) | i1) + start
    else:
        shift2, shift3 = log2ceil(dims[1]), log2ceil(dims[2])
        for i0 in range(dims[0]):
            for i1 in range(dims[1]):
                for i2 in range(dims[2]):
                    out[i0, i1, i2] = ((i0 << (shift3 + shift2)) | (i1 << shift2) | i2) + start
    return out


def test_scaled_dot_instruction_known_answers():
    """The `scaled-dot` known answers of xla/hlo/evaluator/hlo_evaluator_test.cc:2251-2409 (block scales in either
    contracting position, a scalar scale meaning none, a scale shared by the batch entries): the interpreter in
    oracle/hlo_eval.py must return exactly the reference's expected literal."""
    from oracle import hlo_eval

    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "scaled_dot_known_answers.json")) as f:
        golden = json.load(f)
    assert [t["name"] for t in golden["tests"]] == ["ScaledDot", "ScaledDotWithOneMissingScale", "ScaledDotWithBatchDim"]
    for t in golden["tests"]:
        lines, args = [], []
        for i, which in enumerate(("lhs", "rhs", "lhs_scale", "rhs_scale")):
            spec = t["operands"][which]
            if "scalar" in spec:
                lines.append(f"  {which} = bf16[] parameter({i})")
                args.append(o.f32_to_bf16_bits(np.float32(spec["scalar"])))
            else:
                lines.append(f"  {which} = bf16[{','.join(map(str, spec['dims']))}] parameter({i})")
                args.append(o.f32_to_bf16_bits(_fill_unique(spec["dims"], spec["start"])))
        d = t["dot_dimension_numbers"]
        attrs = ", ".join(f"{k.replace('_dimensions', '_dims')}={{{','.join(map(str, v))}}}" for k, v in d.items() if v)
        text = ("HloModule known_answer\nENTRY main {\n" + "\n".join(lines) +
                f"\n  ROOT d = bf16[{','.join(map(str, t['result_dims']))}] scaled-dot(lhs, rhs, lhs_scale, rhs_scale), {attrs}\n}}\n")
        got = hlo_eval.evaluate(text, args)
        want = o.f32_to_bf16_bits(np.asarray(t["expected_f32_before_rounding_to_bf16"], np.float32).reshape(t["result_dims"]))
        assert np.array_equal(np.asarray(got), want), (t["name"], o.bf16_bits_to_f32(np.asarray(got)).tolist())
    # the third test's exact sum is 1140, which is not a bf16 value: the expected literal is the rounded 1136
    assert golden["tests"][2]["expected_f32_before_rounding_to_bf16"] == [428.0, 1136.0]


def test_evaluator_known_answers_for_clamp_and_dot():
    """DoesClamp and DotRank2AndRank2 of xla/hlo/evaluator/hlo_evaluator_test.cc (the test fixture runs each in f32 and
    in bf16): the interpreter's clamp(low, value, high) operand order and its dot over `lhs_contracting_dims={1},
    rhs_contracting_dims={0}` must give the reference's expected literals exactly, in both types."""
    from oracle import hlo_eval

    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "evaluator_known_answers.json")) as f:
        golden = json.load(f)
    for t in ("f32", "bf16"):
        conv = (lambda x: np.asarray(x, np.float32)) if t == "f32" else (lambda x: o.f32_to_bf16_bits(np.asarray(x, np.float32)))
        back = (lambda x: np.asarray(x, np.float32)) if t == "f32" else (lambda x: o.bf16_bits_to_f32(np.asarray(x)))
        c = golden["DoesClamp"]
        text = f"""HloModule clamp
ENTRY main {{
  low = {t}[2,2] parameter(0)
  value = {t}[2,2] parameter(1)
  high = {t}[2,2] parameter(2)
  ROOT r = {t}[2,2] clamp(low, value, high)
}}
"""
        got = hlo_eval.evaluate(text, [conv(c["low"]), conv(c["value"]), conv(c["high"])])
        assert np.array_equal(back(got), np.asarray(c["expected"], np.float32)), t
        d = golden["DotRank2AndRank2"]
        lhs, rhs = _fill_unique(d["lhs"]["dims"], d["lhs"]["start"]), _fill_unique(d["rhs"]["dims"], d["rhs"]["start"])
        text = f"""HloModule dot
ENTRY main {{
  lhs = {t}[{d['lhs']['dims'][0]},{d['lhs']['dims'][1]}] parameter(0)
  rhs = {t}[{d['rhs']['dims'][0]},{d['rhs']['dims'][1]}] parameter(1)
  ROOT r = {t}[{d['lhs']['dims'][0]},{d['rhs']['dims'][1]}] dot(lhs, rhs), lhs_contracting_dims={{{d['lhs_contracting_dimensions'][0]}}}, rhs_contracting_dims={{{d['rhs_contracting_dimensions'][0]}}}
}}
"""
        got = hlo_eval.evaluate(text, [conv(lhs), conv(rhs)])
        assert np.array_equal(back(got), np.asarray(d["expected"], np.float32)), t


def test_within_n_values_rule_against_the_reference_cases():
    """CompareNear_NotEqual_1ulp / _4ulps of xla/literal_comparison_test.cc:54-102: next to 1.0, the neighbouring FP8
    value is a mismatch under ErrorSpec(0, 0) and accepted with within_n_values = 1; the value four steps away is a
    mismatch with within_n_values = 1 and accepted with 4.  `fp8_within_n_values` is what the FP8-output GPU tests
    judge by."""
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "within_n_values_known.json")) as f:
        golden = json.load(f)
    for kind, type_name in (("e4m3fn", "f8e4m3fn"), ("e5m2", "f8e5m2")):
        actual = o.fp8_encode(np.float32([golden["actual"]]), kind)
        for t in golden["tests"].values():
            expected = o.fp8_encode(np.float32([t["expected"][type_name]]), kind)
            assert float(o.fp8_decode(expected, kind)[0]) == t["expected"][type_name]        # representable as written
            assert o.fp8_within_n_values(expected, actual, t["accepted_with_within_n_values"]) == 0
            assert o.fp8_within_n_values(expected, actual, t["rejected_with_within_n_values"]) == 1
            assert abs(int(o.fp8_ordinal(expected)[0]) - int(o.fp8_ordinal(actual)[0])) == t["accepted_with_within_n_values"]
