"""Regenerates tests/golden/*.json from the reference checkout.

Run in the authoring container only (`python tests/golden/make_golden.py
[reference_root]`); the JSON it writes is committed so that the test-suite
never needs the reference tree at run time.

Sources, read as text:
  * xla/tests/convert_test.cc -- the `{input, expected_roundtrip}` tables of
    ConvertF16F8e5m2Roundtrip, ConvertF32F8e5m2Roundtrip,
    ConvertF16F8e4m3fnRoundtrip, ConvertF32F8e4m3fnRoundtrip and
    ConvertF32F8e8m0fnuRoundtrip (the block-scale type) (C hex-float literals,
    `nan`, `inf`).
  * xla/stream_executor/cuda/cuda_blas_lt_test.cc -- the S8S8S32 / S8S8F32
    known answer: m = n = k = 32, all-ones operands, every output == k.
  * xla/service/gpu/backend_configs.proto -- `enum Epilogue { ... }` of GemmBackendConfig, and
    xla/ffi/api/c_api.h -- `XLA_FFI_DataType`, `XLA_FFI_Error_Code`: the numbers the boundary
    (include/b200_scaled_dot.h) must use (interface_enums.json); with them the custom-call target names of
    xla/service/gpu/cublas_cudnn.h and xla/backends/gpu/transforms/block_scaling_rewriter.h and the MXFP8 block size.
  * xla/hlo/evaluator/hlo_evaluator_test.cc -- the three known-answer tests of the `scaled-dot` instruction
    (ScaledDot, ScaledDotWithOneMissingScale, ScaledDotWithBatchDim): operand extents and start values of the
    `FillUnique` arrays, dot dimension numbers and the expected result (scaled_dot_known_answers.json); and the
    DoesClamp and DotRank2AndRank2 known answers of the same file (evaluator_known_answers.json).
  * xla/literal_comparison_test.cc -- CompareNear_NotEqual_1ulp / _4ulps: for each FP8 type the value next to 1.0 that
    `within_n_values = 1` must accept and the value that needs `within_n_values = 4` (within_n_values_known.json).
  * xla/service/gpu/matmul_utils_test.cc -- the GetMatrixSizeRewriteThresholdTest cases: dot shapes, dimension numbers
    and whether IsMatrixMultiplicationTooSmallForRewriting(dot, 100) holds (rewrite_threshold_known.json).
"""
import json
import math
import os
import re
import sys

ROOT = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("XLA_ROOT", "")
if not os.path.isdir(os.path.join(ROOT, "xla")):
    sys.exit("usage: python " + os.path.basename(__file__) + " <xla checkout>   (or set XLA_ROOT)")
HERE = os.path.dirname(os.path.abspath(__file__))


def parse_literal(tok: str) -> float:
    tok = tok.strip()
    neg = tok.startswith("-")
    body = tok.lstrip("+-")
    if body == "nan":
        return math.nan
    if body == "inf":
        return -math.inf if neg else math.inf
    v = float.fromhex(body) if body.lower().startswith("0x") else float(body)
    return -v if neg else v


def table_of(src: str, test_name: str):
    start = src.index(f"TEST_F(ConvertTest, {test_name})")
    begin = src.index("test_cases[] = {", start)
    end = src.index("};", begin)
    rows = []
    for m in re.finditer(r"\{\s*([^,{}]+?)\s*,\s*([^,{}]+?)\s*\}", src[begin:end]):
        rows.append((parse_literal(m.group(1)), parse_literal(m.group(2))))
    return rows


def enc(v: float):
    """JSON-safe exact spelling of a double."""
    if math.isnan(v):
        return "nan"
    if math.isinf(v):
        return "-inf" if v < 0 else "inf"
    return v.hex()


def c_enum(src: str, start_marker: str, prefix: str):
    """`NAME = number` pairs of the C / proto enum that starts at `start_marker`."""
    begin = src.index(start_marker)
    end = src.index("}", begin)
    line = src[:begin].count("\n") + 1
    vals = {}
    for m in re.finditer(r"\b" + prefix + r"([A-Z0-9_a-z]+)\s*=\s*(\d+)\s*[,;]", src[begin:end]):
        vals[m.group(1)] = int(m.group(2))
    return line, src[:end].count("\n") + 1, vals


def write_interface_enums():
    proto = open(os.path.join(ROOT, "xla/service/gpu/backend_configs.proto")).read()
    gemm = proto.index("message GemmBackendConfig")
    l0, l1, epilogue = c_enum(proto[gemm:], "enum Epilogue {", "")
    base = proto[:gemm].count("\n")
    capi = open(os.path.join(ROOT, "xla/ffi/api/c_api.h")).read()
    d0, d1, dtypes = c_enum(capi, "  XLA_FFI_DataType_INVALID = 0", "XLA_FFI_DataType_")
    e0, e1, codes = c_enum(capi, "  XLA_FFI_Error_Code_OK = 0", "XLA_FFI_Error_Code_")
    scale_mode = re.search(r"int32 scale_mode = (\d+);", proto)
    # The custom-call target names this library stands in for or consumes.
    cudnn_h = open(os.path.join(ROOT, "xla/service/gpu/cublas_cudnn.h")).read()
    rewriter_h = open(os.path.join(ROOT, "xla/backends/gpu/transforms/block_scaling_rewriter.h")).read()
    call_targets = {}
    for text in (cudnn_h, rewriter_h):
        for m in re.finditer(r"absl::string_view (k\w+(?:CallTarget|CustomCallTarget)) =\s*\"([^\"]+)\";", text):
            if re.search(r"Matmul|Gemm|BlockScaledDot|Quantize", m.group(1)) and "Grouped" not in m.group(1):
                call_targets[m.group(1)] = m.group(2)
    assert call_targets["kCublasLtMatmulF8CallTarget"] and call_targets["kBlockScaledDotCustomCallTarget"]
    assert epilogue["DEFAULT"] == 0 and len(epilogue) == 10 and dtypes["F8E4M3FN"] == 20 and codes["UNIMPLEMENTED"] == 12
    out = {
        "epilogue": {"source": f"xla/service/gpu/backend_configs.proto:{base + l0}-{base + l1}", "values": epilogue},
        "data_type": {"source": f"xla/ffi/api/c_api.h:{d0}-{d1}", "values": dtypes},
        "error_code": {"source": f"xla/ffi/api/c_api.h:{e0}-{e1}", "values": codes},
        "scale_mode_field_number": int(scale_mode.group(1)),
        "call_targets": call_targets,
        "block_size_mxfp8": int(re.search(r"kBlockSizeMXFP8 = (\d+);", rewriter_h).group(1)),
    }
    with open(os.path.join(HERE, "interface_enums.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)


def write_scaled_dot_known_answers():
    """Each operand of the tests is `BF16Array2D(b, rows, cols, start)`, `BF16Array3D(b, batch, rows, cols, start)`
    (arrays filled by FillUnique, xla/array2d.h:78-85 and xla/array3d.h:65-76) or a BF16 scalar constant."""
    rel = "xla/hlo/evaluator/hlo_evaluator_test.cc"
    src = open(os.path.join(ROOT, rel)).read()
    tests = []
    for m in re.finditer(r"TEST_F\(HloEvaluatorTest, (ScaledDot\w*)\) \{(.*?)\n\}\n", src, flags=re.S):
        name, body = m.group(1), m.group(2)
        operands = {}
        for om in re.finditer(r"auto (\w+)_instr =\s*(.*?);", body, flags=re.S):
            which, expr = om.group(1), " ".join(om.group(2).split())
            a = re.search(r"BF16Array([23])D\(b, ([0-9, ]+), ([0-9.]+)f\)", expr)
            if a:
                operands[which] = {"dims": [int(x) for x in a.group(2).split(",")], "start": float(a.group(3))}
            else:
                c = re.search(r"CreateR0\(BF16, ([0-9.]+)f\)", expr)
                assert c, expr
                operands[which] = {"scalar": float(c.group(1))}
        assert sorted(operands) == ["lhs", "lhs_scale", "rhs", "rhs_scale"], (name, operands)
        dnums = {k: [int(x) for x in re.findall(r"add_%s\((\d+)\)" % k, body)]
                 for k in ("lhs_batch_dimensions", "rhs_batch_dimensions", "lhs_contracting_dimensions", "rhs_contracting_dimensions")}
        shape = [int(x) for x in re.search(r"MakeShape\(BF16, \{([0-9, ]+)\}\)", body).group(1).split(",")]
        exp = re.search(r"Array[23]D<float>\((\{.*?\})\);", body, flags=re.S).group(1)
        expected = [float(x) for x in re.findall(r"([0-9.]+)f", exp)]
        tests.append({"name": name, "line": src[: m.start()].count("\n") + 1, "operands": operands, "dot_dimension_numbers": dnums,
                      "result_type": "bf16", "result_dims": shape, "expected_f32_before_rounding_to_bf16": expected})
    assert [t["name"] for t in tests] == ["ScaledDot", "ScaledDotWithOneMissingScale", "ScaledDotWithBatchDim"], tests
    with open(os.path.join(HERE, "scaled_dot_known_answers.json"), "w") as f:
        json.dump({"source": rel, "operand_type": "bf16", "tests": tests}, f, indent=1)


def write_evaluator_known_answers():
    rel = "xla/hlo/evaluator/hlo_evaluator_test.cc"
    src = open(os.path.join(ROOT, rel)).read()

    def body_of(name):
        m = re.search(r"TEST_P\(HloEvaluatorBf16Test, %s\) \{(.*?)\n\}\n" % name, src, flags=re.S)
        return m.group(1), src[: m.start()].count("\n") + 1

    def matrix(text):
        return [[float(x.rstrip("f")) for x in re.findall(r"-?[0-9.]+f?", row)] for row in re.findall(r"\{([^{}]*)\}", text)]

    clamp, clamp_line = body_of("DoesClamp")
    lits = {k: matrix(re.search(r"auto %s = LiteralUtil::CreateR2<float>\((\{.*?\})\);" % k, clamp, flags=re.S).group(1))
            for k in ("low", "value", "high", "expected")}
    assert "HloOpcode::kClamp, c1, c2, c3" in clamp                      # clamp(low, value, high)
    dot, dot_line = body_of("DotRank2AndRank2")
    arrays = [(int(a), int(b), float(c)) for a, b, c in
              re.findall(r"Array2D<float>>\((\d+), (\d+)\);\s*\w+->FillUnique\(([0-9.]+)f\)", dot)]
    assert len(arrays) == 2, arrays
    expected = matrix(re.search(r"auto expected_array = Array2D<float>\((\{.*?\})\);", dot, flags=re.S).group(1))
    out = {
        "source": rel,
        "DoesClamp": dict(lits, line=clamp_line),
        "DotRank2AndRank2": {"line": dot_line, "lhs": {"dims": list(arrays[0][:2]), "start": arrays[0][2]},
                             "rhs": {"dims": list(arrays[1][:2]), "start": arrays[1][2]},
                             "lhs_contracting_dimensions": [int(x) for x in re.findall(r"add_lhs_contracting_dimensions\((\d+)\)", dot)],
                             "rhs_contracting_dimensions": [int(x) for x in re.findall(r"add_rhs_contracting_dimensions\((\d+)\)", dot)],
                             "expected": expected},
    }
    with open(os.path.join(HERE, "evaluator_known_answers.json"), "w") as f:
        json.dump(out, f, indent=1)


def write_within_n_values_known():
    rel = "xla/literal_comparison_test.cc"
    src = open(os.path.join(ROOT, rel)).read()
    out = {"source": rel, "actual": 1.0, "tests": {}}
    for name, accept_n in (("CompareNear_NotEqual_1ulp", 1), ("CompareNear_NotEqual_4ulps", 4)):
        m = re.search(r"TYPED_TEST\(LiteralComparisonTest, %s\) \{(.*?)\n\}\n" % name, src, flags=re.S)
        body = m.group(1)
        default = float(re.search(r"float expV = ([0-9.]+);", body).group(1))
        e5m2 = float(re.search(r"type == F8E5M2 \|\| type == F8E5M2FNUZ\)\s*expV = ([0-9.]+);", body).group(1))
        e8m0 = float(re.search(r"type == F8E8M0FNU\)\s*expV = ([0-9.]+);", body).group(1))
        out["tests"][name] = {"line": src[: m.start()].count("\n") + 1, "accepted_with_within_n_values": accept_n,
                              "rejected_with_within_n_values": 0 if accept_n == 1 else 1,
                              "expected": {"f8e4m3fn": default, "f8e5m2": e5m2, "f8e8m0fnu": e8m0}}
    with open(os.path.join(HERE, "within_n_values_known.json"), "w") as f:
        json.dump(out, f, indent=1)


def write_rewrite_threshold_known():
    rel = "xla/service/gpu/matmul_utils_test.cc"
    src = open(os.path.join(ROOT, rel)).read()
    cases = []
    heads = list(re.finditer(r"^TEST(?:_F|_P)?\(\s*(\w+)\s*,\s*(\w+)\s*\) \{", src, flags=re.M))
    for m, nxt in zip(heads, heads[1:] + [None]):
        if m.group(1) != "GetMatrixSizeRewriteThresholdTest":
            continue
        name, body = m.group(2), src[m.end(): nxt.start() if nxt else len(src)]      # the module text holds a "}" line of its own
        verdict = re.search(r"IsMatrixMultiplicationTooSmallForRewriting\(\*dot, (\d+)\),\s*absl_testing::IsOkAndHolds\((true|false)\)", body)
        if not verdict:
            continue
        x = re.search(r"x = \w+\[([0-9,]+)\] parameter\(0\)", body).group(1)
        y = re.search(r"y = \w+\[([0-9,]+)\] parameter\(1\)", body).group(1)
        dot = re.search(r"ROOT dot = \w+\[([0-9,]+)\] dot\(x, y\), (.*)", body)
        cases.append({"name": name, "line": src[: m.start()].count("\n") + 1, "threshold": int(verdict.group(1)),
                      "too_small": verdict.group(2) == "true", "x_dims": [int(v) for v in x.split(",")],
                      "y_dims": [int(v) for v in y.split(",")], "result_dims": [int(v) for v in dot.group(1).split(",")],
                      "dimension_numbers": dot.group(2).strip()})
    assert len(cases) == 4 and sum(c["too_small"] for c in cases) == 1, cases
    with open(os.path.join(HERE, "rewrite_threshold_known.json"), "w") as f:
        json.dump({"source": rel, "cases": cases}, f, indent=1)


def main():
    src = open(os.path.join(ROOT, "xla/tests/convert_test.cc")).read()
    out = {"source": "xla/tests/convert_test.cc", "tables": {}}
    for name, kind, via in [
        ("ConvertF16F8e5m2Roundtrip", "e5m2", "f16"),
        ("ConvertF32F8e5m2Roundtrip", "e5m2", "f32"),
        ("ConvertF16F8e4m3fnRoundtrip", "e4m3fn", "f16"),
        ("ConvertF32F8e4m3fnRoundtrip", "e4m3fn", "f32"),
        ("ConvertF32F8e8m0fnuRoundtrip", "e8m0fnu", "f32"),
    ]:
        rows = table_of(src, name)
        assert len(rows) >= 14, (name, len(rows))
        out["tables"][name] = {
            "fp8": kind,
            "via": via,
            "line": src[: src.index(f"TEST_F(ConvertTest, {name})")].count("\n") + 1,
            "cases": [[enc(a), enc(b)] for a, b in rows],
        }
    with open(os.path.join(HERE, "fp8_convert_roundtrip.json"), "w") as f:
        json.dump(out, f, indent=1)

    blas = open(os.path.join(ROOT, "xla/stream_executor/cuda/cuda_blas_lt_test.cc")).read()
    m = re.search(r"int64_t m = (\d+), n = (\d+), k = (\d+);", blas)
    dims = [int(g) for g in m.groups()]
    assert "std::vector<int8_t> host_a(m * k, 1)" in blas or "(m * k, 1)" in blas
    known = {
        "source": "xla/stream_executor/cuda/cuda_blas_lt_test.cc",
        "tests": ["S8S8S32Gemm", "S8S8F32Gemm"],
        "m": dims[0], "n": dims[1], "k": dims[2],
        "a_fill": 1, "b_fill": 1, "alpha": 1.0, "beta": 0.0,
        "expected_every_element": dims[2],
    }
    with open(os.path.join(HERE, "s8_known_answer.json"), "w") as f:
        json.dump(known, f, indent=1)
    write_interface_enums()
    write_scaled_dot_known_answers()
    write_evaluator_known_answers()
    write_within_n_values_known()
    write_rewrite_threshold_known()
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
