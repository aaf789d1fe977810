"""Extracts, as text, what the reference's own GemmRewriter tests hold for the scaled-dot path into
tests/golden/ref_rewrites.json: every test module and the rewrite its FileCheck lines expect.

Run in the authoring container only (`python tests/golden/make_ref_rewrites.py [reference_root]`);
the JSON is committed so that the test-suite never needs the reference tree at run time.

Sources, read as text (nothing is compiled or executed):
  * xla/backends/gpu/transforms/gemm_rewriter_fp8_test.cc -- every TEST_F of
    ParameterizedFp8GemmRewriteTest: the `R"( ... )"` HLO module(s), the `; CHECK` lines handed to
    RunAndFilecheckHloRewrite / MatchOptimizedHlo, and the ErrorSpec of the numeric comparison.  The
    placeholders <<F8E4M3>>, <<F8E5M2>>, <<F8E4M3_AMAX>> are expanded the way the fixture does for CUDA
    (:62-83); the two parameterised tests (:2825-2958) are expanded into their 32 + 32 layout
    combinations with the loops of the test restated below.
  * xla/backends/gpu/transforms/gemm_rewriter_test.cc -- the Int8Gemm* tests (:3182-3368).

From the CHECK lines of each test the script derives `expect`:
  rewritten      a line names custom_call_target="__cublas$lt$matmul$f8" (or "__cublas$lt$matmul" /
                 "__cublas$gemm" for the integer tests)
  operands       for every operand of the custom-call line, the chain of CHECK-defined instructions
                 from it back to a parameter / constant, as [opcode, ...] plus the root
                 ({"parameter": n} | {"constant": text} | {"unknown": capture-name})
  result         element types of the custom call's result tuple, dims of element 0
  backend_config alpha_real, alpha_imag, beta, epilogue (name), damax_output, contracting and
                 batch dimensions, operand_precision -- whichever of them the CHECK lines mention
A test without CHECK lines that asserts EXPECT_FALSE(changed) gets `expect = {"rewritten": false}`.
CHECK-GCN lines (ROCm only) are dropped; CHECK-PTX lines count as CHECK lines (CUDA).
The reference's tests run its rewriter for a Hopper target, which transposes B into the
column-major form cuBLASLt wants there; on Blackwell the rewriter inserts no transposes
(gemm_rewriter.cc:1535-1554, NoTransposeOnBlackwellF8 at gemm_rewriter_fp8_test.cc:3065-3108).
Consumers therefore compare operand roots and dimension numbers modulo `transpose`.

A second file, tests/golden/ref_block_scaled.json, holds the `__op$block_scaled_dot` modules of
  * xla/backends/gpu/transforms/block_scaling_rewriter_test.cc (what BlockScalingRewriter makes of each form) and
  * xla/backends/gpu/transforms/block_scaling_rewriter_cudnn_test.cc (a library run compared with the expansion
    under an ErrorSpec),
each with `library`: whether the reference, given a library that supports block-scaled dots, hands this module to it
(the test builds the pass with kCudnnSupportsBlockScaledDot / kCudnnVersion and its CHECK lines name
`__cudnn$blockScaledDot` or a custom call) or expands it into dequantize + dot.
The same file's `scaled_dot` list holds the modules built on the `scaled-dot` instruction:
  * the CudnnFusion* tests of block_scaling_rewriter_test.cc (`supported`: what the test expects of
    CudnnScaledDotHelper::IsSupported) and
  * xla/backends/gpu/autotuner/mx_scaled_dot_execution_test.cc, whose modules the test expects to end up as
    `__cublas$lt$matmul$mx` (or a Triton fusion) and compares with the expansion under an ErrorSpec (`mx_call`: true).
"""
import json
import os
import re
import sys

ROOT = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("XLA_ROOT", "")
if not os.path.isdir(os.path.join(ROOT, "xla")):
    sys.exit("usage: python " + os.path.basename(__file__) + " <xla checkout>   (or set XLA_ROOT)")
HERE = os.path.dirname(os.path.abspath(__file__))
FP8_TEST = "xla/backends/gpu/transforms/gemm_rewriter_fp8_test.cc"
GEMM_TEST = "xla/backends/gpu/transforms/gemm_rewriter_test.cc"
PLACEHOLDERS = {"<<F8E4M3>>": "f8e4m3fn", "<<F8E5M2>>": "f8e5m2", "<<F8E4M3_AMAX>>": "448."}


def expand(text):
    for k, v in PLACEHOLDERS.items():
        text = text.replace(k, v)
    return text


def split_tests(src, fixture_pattern):
    """[(name, first line, body text)] of every TEST_F / TEST_P whose fixture matches."""
    heads = [(m.start(), m.group(1), m.group(2)) for m in
             re.finditer(r"^TEST_[FP]\(\s*(\w+)\s*,\s*(\w+)\s*\)\s*\{", src, flags=re.M)]
    ends = [h[0] for h in heads[1:]] + [len(src)]
    out = []
    for (pos, fixture, name), end in zip(heads, ends):
        if re.fullmatch(fixture_pattern, fixture):
            out.append((name, src[:pos].count("\n") + 1, src[pos:end]))
    return out


def raw_strings(body):
    return [m.group(1) for m in re.finditer(r'R"\((.*?)\)"', body, flags=re.S)]


def is_checks(s):
    return "; CHECK" in s or ";CHECK" in s


def error_spec(body):
    m = re.search(r"ErrorSpec\s*\{\s*([0-9.e+-]+)\s*,\s*([0-9.e+-]+)\s*\}", body)
    return [float(m.group(1)), float(m.group(2))] if m else [1e-2, 1e-2]


# ---------------------------------------------------------------------------------- CHECK lines
CAPTURE = r"\[\[([A-Za-z0-9_]+)(?::[^\]]*\]?[^\]]*)?\]\]"


def check_lines(text):
    lines = []
    for raw in text.splitlines():
        m = re.match(r"\s*;\s*(CHECK(?:-[A-Z]+)*)\s*:\s?(.*)$", raw)
        if not m:
            continue
        kind, rest = m.group(1), m.group(2).strip()
        if "GCN" in kind:
            continue
        lines.append((kind.replace("-PTX", ""), rest))
    return lines


def names_in(text):
    """Capture names used in an operand list such as `[[P0]], [[P1_TRANSPOSE]], /*index=5*/[[CV2]]`."""
    text = re.sub(r"/\*.*?\*/", "", text)
    out = []
    depth, cur = 0, ""
    for c in text:
        if c in "([{":
            depth += 1
        if c in ")]}":
            depth -= 1
        if c == "," and depth == 0:
            out.append(cur.strip())
            cur = ""
        else:
            cur += c
    if cur.strip():
        out.append(cur.strip())
    names = []
    for o in out:
        m = re.search(r"\[\[([A-Za-z0-9_]+)", o)
        names.append(m.group(1) if m else o)
    return names


def parse_checks(text):
    lines = check_lines(text)
    defs = {}
    call = None
    cfg = {}
    target = None
    negative = []
    for kind, rest in lines:
        if kind.endswith("NOT"):
            negative.append(rest.strip())
            continue
        m = re.match(r"\[\[([A-Za-z0-9_]+):[^\]]*\]\+?\]\]\s*=\s*(\(.*?\)|\S+)\s+([a-z\-]+)\((.*)$", rest)
        if m:
            name, shape, opcode, tail = m.groups()
            depth, i = 1, 0
            while i < len(tail) and depth:
                depth += {"(": 1, ")": -1}.get(tail[i], 0)
                i += 1
            args, attrs = tail[: max(0, i - 1)], tail[i:]
            entry = {"shape": shape, "opcode": opcode, "args": args, "attrs": attrs.strip(" ,")}
            if opcode == "custom-call":
                call = dict(entry, name=name)
            elif name not in defs:
                defs[name] = entry
            if opcode != "custom-call":
                continue
        m = re.match(r"\{\{\.\*\}\}\s*(?:=\s*\{\{\.\*\}\}\s*)?custom-call\((.*?)\)?,?$", rest)
        if m and call is None and "custom-call(" in rest:
            call = {"shape": None, "opcode": "custom-call", "args": m.group(1), "attrs": "", "name": None}
        m = re.search(r'custom_call_target="([^"]+)"', rest)
        if m and target is None:
            target = m.group(1)
            if target == "$0":          # absl::Substitute placeholder of the integer tests: "__cublas$lt$matmul" or "__cublas$gemm"
                target = "__cublas$lt$matmul"
        for key in ("alpha_real", "alpha_imag", "beta"):
            m = re.search(r'"%s":([-0-9.e+]+)' % key, rest)
            if m:
                cfg[key] = float(m.group(1))
        m = re.search(r'"epilogue":"([A-Z_]+)"', rest)
        if m:
            cfg["epilogue"] = m.group(1)
        m = re.search(r'"damax_output":(true|false)', rest)
        if m:
            cfg["damax_output"] = m.group(1) == "true"
        for key in ("lhs_contracting_dimensions", "rhs_contracting_dimensions", "lhs_batch_dimensions", "rhs_batch_dimensions"):
            m = re.search(r'"%s":\[([^\]]*)\]' % key, rest)
            if m:
                cfg[key] = [int(x.strip().strip('"')) for x in m.group(1).split(",") if x.strip()]
        m = re.search(r'"operand_precision":\[([^\]]*)\]', rest)
        if m:
            cfg["operand_precision"] = [x.strip().strip('"') for x in m.group(1).split(",") if x.strip()]

    def resolve(name, seen=()):
        d = defs.get(name)
        if d is None or name in seen:
            return {"chain": [], "root": {"unknown": name}}
        if d["opcode"] == "parameter":
            return {"chain": [], "root": {"parameter": int(re.sub(r"\D", "", d["args"]) or -1)}, "shape": d["shape"]}
        if d["opcode"] == "constant":
            return {"chain": [], "root": {"constant": d["args"].strip()}, "shape": d["shape"]}
        ops = names_in(d["args"])
        first = ops[0] if ops else None
        # divide(1, scale): the value of interest is the divisor
        if d["opcode"] == "divide" and len(ops) == 2 and defs.get(ops[0], {}).get("opcode") == "constant":
            first = ops[1]
        inner = resolve(first, seen + (name,)) if first else {"chain": [], "root": {"unknown": name}}
        return {"chain": inner["chain"] + [d["opcode"]], "root": inner["root"], "shape": d["shape"]}

    expect = {"rewritten": bool(target and target.startswith("__cublas")), "target": target, "backend_config": cfg}
    if negative:
        expect["check_not"] = negative
    if call is not None:
        expect["operands"] = [dict(resolve(n), name=n) for n in names_in(call["args"])]
        if call["shape"]:
            shp = call["shape"]
            elems = re.findall(r"([a-z0-9]+)\[([^\]]*)\]", shp)
            expect["result"] = {"element_types": [e[0] for e in elems],
                                "dims": [int(x) for x in elems[0][1].split(",") if x.strip().isdigit()] if elems else None,
                                "shape": shp}
    return expect


# ---------------------------------------------------------------------------------- the two layout sweeps
def sweep_2d(template):
    out = []
    for d_is_col in (False, True):
        for a_is_col in (False, True):
            for b_is_col in (False, True):
                for lcd in (0, 1):
                    for rcd in (0, 1):
                        rep = {"<<Lcd>>": "{1}" if lcd == 1 else "{0}", "<<Rcd>>": "{1}" if rcd == 1 else "{0}",
                               "<<Ashape>>": "[64,32]" if lcd == 1 else "[32,64]",
                               "<<Bshape>>": "[32,16]" if rcd == 0 else "[16,32]",
                               "<<Alayout>>": "{0,1}" if a_is_col else "{1,0}", "<<Blayout>>": "{0,1}" if b_is_col else "{1,0}",
                               "<<Olayout>>": "{0,1}" if d_is_col else "{1,0}"}
                        text = template
                        for k, v in rep.items():
                            text = text.replace(k, v)
                        out.append((f"d{'col' if d_is_col else 'row'}_a{'col' if a_is_col else 'row'}_b{'col' if b_is_col else 'row'}_l{lcd}_r{rcd}", text))
    return out


def sweep_batched(template):
    out = []
    for o_is_col in (False, True):
        for lcd in (2, 1):
            for rcd in (2, 1):
                for a_layout in ("{2,1,0}", "{1,2,0}"):
                    for b_layout in ("{2,1,0}", "{1,2,0}"):
                        rep = {"<<Lcd>>": "{%d}" % lcd, "<<Rcd>>": "{%d}" % rcd,
                               "<<Ashape>>": "[2,64,32]" if lcd == 2 else "[2,32,64]",
                               "<<Bshape>>": "[2,32,16]" if rcd == 1 else "[2,16,32]",
                               "<<Alayout>>": a_layout, "<<Blayout>>": b_layout,
                               "<<Olayout>>": "{2, 0, 1}" if o_is_col else "{2, 1, 0}"}
                        text = template
                        for k, v in rep.items():
                            text = text.replace(k, v)
                        out.append((f"o{'col' if o_is_col else 'row'}_l{lcd}_r{rcd}_a{a_layout.strip('{}').replace(',', '')}_b{b_layout.strip('{}').replace(',', '')}", text))
    return out


def skip_note(body):
    notes = re.findall(r'GTEST_SKIP\(\)\s*<<\s*"([^"]*)"', body)
    return notes


def cases_of(rel_path, fixture_pattern, name_filter=None):
    src = open(os.path.join(ROOT, rel_path)).read()
    cases = []
    for name, line, body in split_tests(src, fixture_pattern):
        if name_filter and not re.search(name_filter, name):
            continue
        strings = raw_strings(body)
        modules = [s for s in strings if not is_checks(s) and re.search(r"\bparameter\(", s)]
        checks = [s for s in strings if is_checks(s)]
        if not modules:
            continue
        spec = error_spec(body)
        numeric = "RunAndCompare" in body or "CheckFp8IfSupported" in body
        base = {"source": f"{rel_path}:{line}", "test": name, "error_spec": spec, "numeric": numeric, "skip_notes": skip_note(body)}
        if name == "ScaledABUnscaledDF8Parameterized":
            for tag, text in sweep_2d(modules[0]):
                cases.append(dict(base, name=f"{name}/{tag}", hlo=expand(text), checks=expand(checks[0]), expect=parse_checks(expand(checks[0]))))
            continue
        if name == "ScaledABUnscaledDF8ParameterizedBatched":
            for tag, text in sweep_batched(modules[0]):
                cases.append(dict(base, name=f"{name}/{tag}", hlo=expand(text), checks=expand(checks[0]), expect=parse_checks(expand(checks[0]))))
            continue
        # one module, possibly several check blocks (rewriter output, optimised output): the first block that
        # names a custom call is the rewrite expectation.  A test that assembles its pattern from pieces
        # (`checks.append(...)`, `checks += ...`; the ROCm-only pieces are CHECK-GCN lines and drop out) is
        # read as the concatenation of the pieces.
        chosen = None
        if re.search(r"checks\s*(\.append\(|\+=)", body) and checks:
            merged = "\n".join(checks)
            chosen = (merged, parse_checks(expand(merged)))
            checks = []
        for c in checks:
            e = parse_checks(expand(c))
            if chosen is None or (not chosen[1].get("operands") and e.get("operands")):
                chosen = (c, e)
        for i, mod in enumerate(modules):
            case = dict(base, name=name if len(modules) == 1 else f"{name}/{i}", hlo=expand(mod))
            if chosen is not None and i == 0:
                case["checks"] = expand(chosen[0])
                case["expect"] = chosen[1]
            else:
                case["checks"] = None
                case["expect"] = None
                # tests that only assert whether the pass changed the module
                if re.search(r"EXPECT_FALSE\(changed\)", body):
                    case["expect"] = {"rewritten": False, "target": None, "backend_config": {}}
            cases.append(case)
    return cases


BLOCK_TESTS = ("xla/backends/gpu/transforms/block_scaling_rewriter_test.cc",
               "xla/backends/gpu/transforms/block_scaling_rewriter_cudnn_test.cc")


def block_scaled_cases():
    cases = []
    for rel_path in BLOCK_TESTS:
        src = open(os.path.join(ROOT, rel_path)).read()
        for name, line, body in split_tests(src, r"BlockScalingRewriter\w*Test"):
            modules = [m for m in raw_strings(body) if "__op$block_scaled_dot" in m and re.search(r"\bparameter\(", m)]
            if not modules:
                continue
            with_library = bool(re.search(r"kCudnnSupportsBlockScaledDot|kCudnnVersion\b", body))
            library = with_library and bool(re.search(r"CHECK[^\n]*(__cudnn\$blockScaledDot|custom-call\()", body))
            m = re.search(r"ErrorSpec\(\s*/\*aabs=\*/\s*([0-9.e+-]+)\s*,\s*/\*arel=\*/\s*([0-9.e+-]+)\s*\)", body)
            cases.append({"name": name, "source": f"{rel_path}:{line}", "hlo": modules[0].strip() + "\n",
                          "library": library, "numeric": "RunAndCompare" in body,
                          "error_spec": [float(m.group(1)), float(m.group(2))] if m else None})
    return cases


MX_EXECUTION_TEST = "xla/backends/gpu/autotuner/mx_scaled_dot_execution_test.cc"
ERROR_SPEC = r"ErrorSpec\(\s*/\*aabs=\*/\s*([0-9.e+-]+)\s*,\s*/\*arel=\*/\s*([0-9.e+-]+)\s*\)"


def scaled_dot_cases():
    cases = []
    src = open(os.path.join(ROOT, BLOCK_TESTS[0])).read()
    for name, line, body in split_tests(src, r"BlockScalingRewriter\w*Test"):
        modules = [m for m in raw_strings(body) if "scaled-dot(" in m]
        expected = re.search(r"EXPECT_(TRUE|FALSE)\(\s*CudnnScaledDotHelper::IsSupported", body)
        if modules and expected:
            cases.append({"name": name, "source": f"{BLOCK_TESTS[0]}:{line}", "hlo": modules[0].strip() + "\n",
                          "supported": expected.group(1) == "TRUE", "mx_call": None, "error_spec": None})
    # Modules held in named constants, each used by one TEST_F through RunMxCorrectnessTest(constant, ErrorSpec(..)).
    src = open(os.path.join(ROOT, MX_EXECUTION_TEST)).read()
    constants = {m.group(1): (m.group(2), src[:m.start()].count("\n") + 1)
                 for m in re.finditer(r'constexpr absl::string_view (k\w+) =\s*R"\((.*?)\)";', src, flags=re.S)}
    for name, line, body in split_tests(src, r"MxScaledDotExecutionTest"):
        use = re.search(r"RunMxCorrectnessTest\(\s*(k\w+)\s*,\s*" + ERROR_SPEC, body)
        if not use or use.group(1) not in constants:
            continue
        text, at = constants[use.group(1)]
        cases.append({"name": name, "source": f"{MX_EXECUTION_TEST}:{at}", "hlo": text.strip() + "\n", "supported": None,
                      "mx_call": True, "error_spec": [float(use.group(2)), float(use.group(3))]})
    return cases


def main():
    blocks = block_scaled_cases()
    scaled = scaled_dot_cases()
    with open(os.path.join(HERE, "ref_block_scaled.json"), "w") as f:
        json.dump({"sources": list(BLOCK_TESTS),
                   "sources_scaled_dot": [BLOCK_TESTS[0], MX_EXECUTION_TEST],
                   "note": "`__op$block_scaled_dot` modules of the reference's BlockScalingRewriter tests, extracted as text; "
                           "`library` = handed to a block-scaled library kernel rather than expanded, see the generating script",
                   "cases": blocks, "scaled_dot": scaled}, f, indent=1)
    print(f"{len(blocks)} block-scaled cases, {sum(c['library'] for c in blocks)} taken by the library path; "
          f"{len(scaled)} scaled-dot cases")
    fp8 = cases_of(FP8_TEST, r"ParameterizedFp8GemmRewriteTest")
    int8 = cases_of(GEMM_TEST, r"\w*GemmRewriteTest\w*", name_filter=r"^Int8Gemm")
    out = {
        "sources": {"fp8": FP8_TEST, "int8": GEMM_TEST},
        "placeholders": PLACEHOLDERS,
        "note": "HLO modules and FileCheck expectations of the reference's GemmRewriter tests, extracted as text; "
                "the expectations are for a Hopper target (B transposed to column-major), see the generating script",
        "fp8": fp8,
        "int8": int8,
    }
    with open(os.path.join(HERE, "ref_rewrites.json"), "w") as f:
        json.dump(out, f, indent=1)
    print(f"{len(fp8)} FP8 cases, {len(int8)} int8 cases; "
          f"{sum(1 for c in fp8 if c['expect'] and c['expect'].get('operands'))} with an operand list")


if __name__ == "__main__":
    main()
