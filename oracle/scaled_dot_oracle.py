"""CPU oracle for XLA's quantized scaled-dot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in NumPy, the arithmetic XLA assigns to the HLO pattern
that `GemmRewriter` turns into `__cublas$lt$matmul$f8` (and the s8 x s8 -> s32
sibling).  It is the checker that the CUDA path is compared with; nothing in
the product package may import it.

Parity status: the FP8 / bf16 conversion routines are pinned against the
reference's own known-answer tables (xla/tests/convert_test.cc:1093-1257 and
the e5m2 tables in the same file) and the int8 path against the all-ones
known answer of xla/stream_executor/cuda/cuda_blas_lt_test.cc:48-156, through
the fixtures under tests/golden/.  The scaled dot itself has no stored golden
output in the reference (its tests compare a GPU run with the HLO interpreter
on random inputs under ErrorSpec{1e-2, 1e-2}); XLA's CPU backend cannot be
built in this environment, so for the dot the oracle is a restatement of the
interpreter's rules and not an execution of the reference.

What is followed, by reference file:line:
  * FP8 formats: arithmetic of the third-party `ml_dtypes` float8 types
    (pinned by third_party/py/ml_dtypes/workspace.bzl:25) as reached through
    `Literal::Convert`; published format definition: e4m3fn = 1-4-3 bits,
    bias 7, no infinities, S.1111.111 is NaN, max 448; e5m2 = 1-5-2 bits,
    bias 15, IEEE-style inf/NaN, max 57344.  Conversion from f32 rounds to
    nearest even; e4m3fn overflow gives NaN, e5m2 overflow gives inf.
  * dot: xla/hlo/evaluator/hlo_evaluator_typed_visitor.h:1271-1340 --
    operands are converted to the f32 element-wise type, products are
    accumulated over k in f32, one cast at the end.
  * maximum / clamp propagate NaN: same file :594-613 and :843-865.
  * GELU (tanh form) exactly as the rewriter matches it:
    xla/backends/gpu/transforms/gemm_rewriter.cc:924-971.
  * scaled FP8 output cast and amax: gemm_rewriter.cc:1635-1794; the HLO the
    reference's tests use is gemm_rewriter_fp8_test.cc:2559-2596.
  * comparison rule: xla/literal_comparison.cc:456-556 (an element is a
    mismatch only when BOTH the absolute and the relative bound are
    exceeded) and the n-representable-values rule of :434-453, :518-526.
"""

from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------
# XLA PrimitiveType numbering (xla/ffi/api/c_api.h:233-266 mirrors it).
# ----------------------------------------------------------------------------
S8, S32, F16, F32, BF16, F8E5M2, F8E4M3FN = 2, 4, 10, 11, 16, 19, 20
F8E8M0FNU = 33

# GemmBackendConfig.Epilogue values (xla/service/gpu/backend_configs.proto:106-117).
EPI_DEFAULT, EPI_BIAS, EPI_RELU, EPI_BIAS_RELU = 0, 1, 2, 3
EPI_GELU, EPI_GELU_AUX, EPI_BIAS_GELU, EPI_BIAS_GELU_AUX = 4, 5, 6, 7

_FP8 = {
    # name: (exponent bits, mantissa bits, bias, finite-only "fn" flavour)
    "e4m3fn": (4, 3, 7, True),
    "e5m2": (5, 2, 15, False),
}


def _fp8_table(kind: str) -> np.ndarray:
    """All 256 code points of an FP8 format as f32."""
    ebits, mbits, bias, fn = _FP8[kind]
    out = np.empty(256, dtype=np.float32)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        e = (code >> mbits) & ((1 << ebits) - 1)
        m = code & ((1 << mbits) - 1)
        emax = (1 << ebits) - 1
        if fn and e == emax and m == (1 << mbits) - 1:
            v = np.nan
        elif (not fn) and e == emax:
            v = np.inf if m == 0 else np.nan
        elif e == 0:
            v = m * 2.0 ** (1 - bias - mbits)
        else:
            v = (1.0 + m / (1 << mbits)) * 2.0 ** (e - bias)
        out[code] = sign * v if not np.isnan(v) else np.nan
    return out


_TABLES = {k: _fp8_table(k) for k in _FP8}


def fp8_decode(codes: np.ndarray, kind: str = "e4m3fn") -> np.ndarray:
    """uint8 code points -> f32 values (exact)."""
    return _TABLES[kind][np.asarray(codes, dtype=np.uint8)]


def fp8_max(kind: str) -> float:
    return 448.0 if kind == "e4m3fn" else 57344.0


def fp8_encode(x: np.ndarray, kind: str = "e4m3fn") -> np.ndarray:
    """f32 -> FP8 code points, round-to-nearest-even, no saturation.

    e4m3fn: anything that rounds above 448 (|x| > 464) and +-inf become NaN
    (0x7f / 0xff).  e5m2: overflow becomes +-inf (0x7c / 0xfc).  Pinned by
    xla/tests/convert_test.cc:1144-1194.
    """
    ebits, mbits, bias, fn = _FP8[kind]
    x = np.asarray(x, dtype=np.float32)
    sign = (x.view(np.uint32) >> 31).astype(np.uint8) << 7
    with np.errstate(invalid="ignore"):
        a = np.abs(x).astype(np.float64)
    nan = np.isnan(a)
    inf = np.isinf(a)
    a = np.where(nan | inf, 0.0, a)
    emin = 1 - bias  # exponent of the smallest normal
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0))).astype(np.int64)
    # log2 may be off by one ulp at powers of two; fix by direct comparison.
    e = np.where(2.0 ** e > a, e - 1, e)
    e = np.where(2.0 ** (e + 1) <= a, e + 1, e)
    e = np.maximum(e, emin)
    quantum = 2.0 ** (e - mbits)
    r = np.rint(a / quantum) * quantum  # np.rint rounds half to even
    # Re-derive the exponent after rounding (mantissa carry).
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(r > 0, r, 1.0))).astype(np.int64)
    e2 = np.where(2.0 ** e2 > r, e2 - 1, e2)
    e2 = np.where(2.0 ** (e2 + 1) <= r, e2 + 1, e2)
    is_sub = r < 2.0 ** emin
    exp_field = np.where(is_sub, 0, e2 + bias).astype(np.int64)
    man_field = np.where(
        is_sub,
        np.rint(r / 2.0 ** (emin - mbits)),
        np.rint((r / 2.0 ** e2 - 1.0) * (1 << mbits)),
    ).astype(np.int64)
    code = (exp_field << mbits) | man_field
    over = r > fp8_max(kind)
    if fn:
        nan_code = (1 << (ebits + mbits)) - 1  # 0x7f
        code = np.where(over | inf | nan, nan_code, code)
    else:
        inf_code = ((1 << ebits) - 1) << mbits  # 0x7c
        code = np.where(over | inf, inf_code, code)
        code = np.where(nan, inf_code | (1 << (mbits - 1)), code)  # quiet NaN 0x7e
    return (code.astype(np.uint8) | sign).astype(np.uint8)


# ----------------------------------------------------------------------------
# f8e8m0fnu: the scale type of MX block-scaled operands.  Eight exponent bits and nothing else:
# code c is 2^(c-127), 0xff is NaN; no zero, no sign, no infinity.
# Pinned by xla/tests/convert_test.cc:2114-2152 (ConvertF32F8e8m0fnuRoundtrip).
# ----------------------------------------------------------------------------
def e8m0_decode(codes: np.ndarray) -> np.ndarray:
    """uint8 code points -> f32 values (exact; code 0 is the f32 denormal 2^-127)."""
    c = np.asarray(codes, dtype=np.uint8).astype(np.int64)
    v = np.ldexp(np.float64(1.0), np.minimum(c, 254) - 127).astype(np.float32)
    return np.where(c == 255, np.float32(np.nan), v).astype(np.float32)


def e8m0_encode(x: np.ndarray) -> np.ndarray:
    """f32 -> f8e8m0fnu code points.  Zero, negative values, infinities and NaN become NaN (0xff);
    a positive value rounds to the nearest power of two (a mantissa of exactly 1.5 rounds up, there
    being no even neighbour to prefer); anything that rounds above 2^127 is NaN.  Below 2^-126 the
    destination has one step of 2^-126: the value rounds, ties to even, to 2^-126 (code 1) or to
    code 0."""
    x = np.asarray(x, dtype=np.float32)
    a = x.astype(np.float64)
    bad = ~np.isfinite(a) | (a <= 0)
    a = np.where(bad, 1.0, a)
    m, e = np.frexp(a)                       # a = m * 2^e, m in [0.5, 1)
    e = e - 1                                # a = (2m) * 2^e, 2m in [1, 2)
    e = np.where(2.0 * m >= 1.5, e + 1, e)
    tiny = a < 2.0 ** -126
    q = np.rint(a / 2.0 ** -126)             # 0 or 1, ties to even
    code = np.where(tiny, q, e + 127)
    code = np.where(bad | (code > 254), 255, code)
    return code.astype(np.uint8)


MX_BLOCK = 32


def mx_dequantize(codes: np.ndarray, scale_codes: np.ndarray, kind: str = "e4m3fn",
                  out_dtype=np.float32) -> np.ndarray:
    """One operand of a block-scaled dot as the reference expands it
    (xla/backends/gpu/transforms/block_scaling_rewriter.cc:194-220, BuildDequantize): the input
    and the scale are each converted to the result type, the scale is broadcast over its block
    along the minor (contracting) dimension, and the two are multiplied.  `codes` is
    [..., rows, k] FP8 code points, `scale_codes` is [..., rows, k / block] f8e8m0fnu code points;
    the block size is the ratio of the two minor extents (32 for MX)."""
    codes = np.asarray(codes, dtype=np.uint8)
    scale_codes = np.asarray(scale_codes, dtype=np.uint8)
    k, kb = codes.shape[-1], scale_codes.shape[-1]
    assert codes.shape[:-1] == scale_codes.shape[:-1] and kb > 0 and k % kb == 0, (codes.shape, scale_codes.shape)
    block = k // kb
    v = fp8_decode(codes, kind).astype(out_dtype)
    s = np.repeat(e8m0_decode(scale_codes).astype(out_dtype), block, axis=-1)
    with np.errstate(over="ignore", invalid="ignore", under="ignore"):
        return (v * s).astype(out_dtype)


def block_scaled_dot(a, b, a_scale, b_scale, *, a_kind="e4m3fn", b_kind="e4m3fn", out_dtype=F32,
                     alpha=1.0, block_size=None):
    """`__op$block_scaled_dot` / `__cublas$lt$matmul$mx`
    (xla/backends/gpu/transforms/block_scaling_rewriter.h:30-77, xla/service/gpu/thunk_emitter.cc:939-988):

        D[b, m, n] = sum_k dequant(a)[b, m, k] * dequant(b)[b, n, k]

    with both operands stored contracting-dimension-minor and an optional leading batch dimension.
    The reference's expansion (block_scaling_rewriter.cc:222-262) dequantizes into the RESULT type
    and then takes an ordinary dot, whose products the interpreter accumulates in f32
    (hlo_evaluator_typed_visitor.h:1271-1340).  Scale arrays may be padded
    (BuildBlockScaledDotInput, block_scaling_rewriter.cc:469-518): extra rows are always sliced
    off; extra columns only when `block_size` is given explicitly (the backend config's
    block_scaled_dot_backend_config.block_size), since otherwise the block size is the ratio of
    the minor extents.  Returns D in the spelling of cast_output()."""
    a = np.asarray(a, dtype=np.uint8)
    b = np.asarray(b, dtype=np.uint8)
    a_scale = np.asarray(a_scale, dtype=np.uint8)
    b_scale = np.asarray(b_scale, dtype=np.uint8)
    for x, s in ((a, a_scale), (b, b_scale)):
        if s.shape[-2] < x.shape[-2] or s.shape[:-2] != x.shape[:-2]:
            raise ValueError("scale rows must cover the operand's rows (block_scaling_rewriter.cc:489-493)")
        if block_size is not None and s.shape[-1] * block_size < x.shape[-1]:
            raise ValueError("scale columns must cover k / block_size (block_scaling_rewriter.cc:496-505)")
    a_scale = a_scale[..., : a.shape[-2], :]
    b_scale = b_scale[..., : b.shape[-2], :]
    if block_size is not None:
        a_scale = a_scale[..., : -(-a.shape[-1] // block_size)]
        b_scale = b_scale[..., : -(-b.shape[-1] // block_size)]
    np_type = {F32: np.float32, F16: np.float16, BF16: None}[out_dtype]
    if np_type is None:      # bf16: dequantized values rounded to bf16, then widened for the dot
        a_dq = bf16_bits_to_f32(f32_to_bf16_bits(mx_dequantize(a, a_scale, a_kind)))
        b_dq = bf16_bits_to_f32(f32_to_bf16_bits(mx_dequantize(b, b_scale, b_kind)))
    else:
        a_dq = mx_dequantize(a, a_scale, a_kind, np_type).astype(np.float32)
        b_dq = mx_dequantize(b, b_scale, b_kind, np_type).astype(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        x = np.matmul(a_dq, np.swapaxes(b_dq, -1, -2), dtype=np.float32)
        if alpha != 1.0:
            x = (x * np.float32(alpha)).astype(np.float32)
    return cast_output(x, out_dtype)


def make_mx_operands(seed: int, m: int, n: int, k: int, batch: int = 0, kind_a="e4m3fn", kind_b="e4m3fn",
                     scale_lo: int = 119, scale_hi: int = 135):
    """Seeded MX operands: FP8 codes of N(0,1) values scaled into the format's range and one
    f8e8m0fnu exponent per 32 values drawn uniformly from [scale_lo, scale_hi] (2^-8 .. 2^8)."""
    rng = np.random.default_rng(seed)
    lead = (batch,) if batch > 0 else ()
    a = fp8_encode(np.clip(rng.standard_normal(lead + (m, k), dtype=np.float32) * 4, -400, 400), kind_a)
    b = fp8_encode(np.clip(rng.standard_normal(lead + (n, k), dtype=np.float32) * 4, -400, 400), kind_b)
    sa = rng.integers(scale_lo, scale_hi + 1, size=lead + (m, k // MX_BLOCK), dtype=np.uint8)
    sb = rng.integers(scale_lo, scale_hi + 1, size=lead + (n, k // MX_BLOCK), dtype=np.uint8)
    return a, b, sa, sb


def fp8_encode_saturating(x: np.ndarray, kind: str = "e4m3fn") -> np.ndarray:
    """clamp(-max, x, max) then convert: the HLO spelling of a saturating cast
    (gemm_rewriter.cc:1644-1657 requires exactly these clamp bounds).  clamp
    propagates NaN (hlo_evaluator_typed_visitor.h:843-865)."""
    x = np.asarray(x, dtype=np.float32)
    mx = np.float32(fp8_max(kind))
    with np.errstate(invalid="ignore"):
        c = np.where(np.isnan(x), x, np.minimum(np.maximum(x, -mx), mx))
    return fp8_encode(c, kind)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 (uint16 bit pattern), round-to-nearest-even, NaN stays NaN."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    nan = np.isnan(np.asarray(x, dtype=np.float32))
    rounded = np.where(nan, (u >> 16) | 0x40, rounded)
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


# ----------------------------------------------------------------------------
# Input builders shared by tests and benchmarks (BASELINE configs: values from
# N(0,1), per-tensor scale = amax/448, divide, convert to e4m3fn).
# ----------------------------------------------------------------------------
def quantize_per_tensor(x: np.ndarray, kind: str = "e4m3fn"):
    """Returns (codes uint8, scale f32) with x ~= decode(codes) * scale."""
    x = np.asarray(x, dtype=np.float32)
    scale = np.float32(np.max(np.abs(x)) / np.float32(fp8_max(kind)))
    if scale == 0:
        scale = np.float32(1.0)
    return fp8_encode(x / scale, kind), scale


# ----------------------------------------------------------------------------
# The epilogue chain, element-wise in f32, operation by operation.
# ----------------------------------------------------------------------------
def gelu_tanh_f32(x: np.ndarray) -> np.ndarray:
    """0.5*x*(1+tanh(sqrt(2/pi)*(x+0.044715*x^3))) with every intermediate
    rounded to f32 in the order the matched HLO spells it
    (gemm_rewriter.cc:924-971)."""
    x = np.asarray(x, dtype=np.float32)
    x2 = x * x
    x3 = x * x2
    t0 = x3 * np.float32(0.044715)
    t1 = x + t0
    t2 = t1 * np.float32(0.797884583)
    th = np.tanh(t2).astype(np.float32)
    t3 = th + np.float32(1.0)
    cdf = t3 * np.float32(0.5)
    return (x * cdf).astype(np.float32)


def _max_propagating_nan(x: np.ndarray) -> np.float32:
    if x.size == 0:
        return np.float32(-np.inf)
    if np.isnan(x).any():
        return np.float32(np.nan)
    return np.float32(x.max())


def dequantize(codes: np.ndarray, scale, kind: str) -> np.ndarray:
    """convert(f8 -> f32) * broadcast(scale), rounded to f32 like the HLO."""
    return (fp8_decode(codes, kind) * np.float32(scale)).astype(np.float32)


def dot_f32(a: np.ndarray, b: np.ndarray, lhs_contracting: int = 1,
            rhs_contracting: int = 0, strict: bool = False) -> np.ndarray:
    """f32 dot with f32 accumulation.  `strict` accumulates sequentially over
    k exactly like the interpreter (small shapes only); otherwise the host
    BLAS is used, which differs only in f32 summation order."""
    a2 = a if lhs_contracting == 1 else a.T
    b2 = b if rhs_contracting == 0 else b.T
    if not strict:
        return np.matmul(a2, b2, dtype=np.float32)
    m, k = a2.shape
    n = b2.shape[1]
    acc = np.zeros((m, n), dtype=np.float32)
    for kk in range(k):
        acc += np.outer(a2[:, kk], b2[kk, :]).astype(np.float32)
    return acc


def scaled_dot_f8(a, b, a_scale, b_scale, *, a_kind="e4m3fn", b_kind="e4m3fn",
                  lhs_contracting=1, rhs_contracting=0, c=None, beta=0.0,
                  alpha=1.0, bias=None, epilogue=EPI_DEFAULT, d_scale=None,
                  out_dtype=BF16, want_amax=False, strict=False):
    """The complete `__cublas$lt$matmul$f8` semantics, as HLO:

        D = cast( d_scale * epi(alpha * dot(a*a_scale, b*b_scale) + beta*C + bias) )
        amax = max |epi(...)|   (before d_scale)

    a, b: uint8 FP8 code points.  bias: f32 values (the caller converts the
    bf16/f16 bias, as `convert(bias)` does in the HLO).  c: f32 values.
    Returns (D, amax) where D is f32 values for F32, uint16 bit patterns for
    BF16/F16, uint8 code points for FP8 outputs; amax is None unless asked.
    Operand order and meaning: xla/service/gpu/thunk_emitter.cc:776-862.
    """
    a_dq = dequantize(a, a_scale, a_kind)
    b_dq = dequantize(b, b_scale, b_kind)
    x = dot_f32(a_dq, b_dq, lhs_contracting, rhs_contracting, strict)
    if alpha != 1.0:
        x = (x * np.float32(alpha)).astype(np.float32)
    if c is not None and beta != 0.0:
        x = (x + np.float32(beta) * np.asarray(c, dtype=np.float32)).astype(np.float32)
    if epilogue in (EPI_BIAS, EPI_BIAS_RELU, EPI_BIAS_GELU, EPI_BIAS_GELU_AUX):
        x = (x + np.asarray(bias, dtype=np.float32)[None, :]).astype(np.float32)
    if epilogue in (EPI_RELU, EPI_BIAS_RELU):
        with np.errstate(invalid="ignore"):
            x = np.where(np.isnan(x), x, np.maximum(x, np.float32(0)))
    elif epilogue in (EPI_GELU, EPI_BIAS_GELU, EPI_GELU_AUX, EPI_BIAS_GELU_AUX):
        x = gelu_tanh_f32(x)
    amax = _max_propagating_nan(np.abs(x)) if want_amax else None
    if d_scale is not None:
        x = (x * np.float32(d_scale)).astype(np.float32)
    return cast_output(x, out_dtype), amax


def cast_output(x: np.ndarray, out_dtype: int):
    if out_dtype == F32:
        return np.asarray(x, dtype=np.float32)
    if out_dtype == BF16:
        return f32_to_bf16_bits(x)
    if out_dtype == F16:
        return f32_to_f16_bits(x)
    if out_dtype == F8E4M3FN:
        return fp8_encode_saturating(x, "e4m3fn")
    if out_dtype == F8E5M2:
        return fp8_encode_saturating(x, "e5m2")
    raise ValueError(f"unsupported output type {out_dtype}")


def output_to_f32(d: np.ndarray, out_dtype: int) -> np.ndarray:
    if out_dtype == F32:
        return np.asarray(d, dtype=np.float32)
    if out_dtype == BF16:
        return bf16_bits_to_f32(d)
    if out_dtype == F16:
        return np.asarray(d, dtype=np.uint16).view(np.float16).astype(np.float32)
    if out_dtype == F8E4M3FN:
        return fp8_decode(d, "e4m3fn")
    if out_dtype == F8E5M2:
        return fp8_decode(d, "e5m2")
    if out_dtype == S32:
        return np.asarray(d).astype(np.float32)
    raise ValueError(f"unsupported output type {out_dtype}")


def dot_s8(a: np.ndarray, b: np.ndarray, lhs_contracting=1, rhs_contracting=0) -> np.ndarray:
    """s8 x s8 -> s32, exact (hlo_evaluator_typed_visitor.h:1330-1336).
    Evaluated through an f64 BLAS GEMM, exact while K*127^2 < 2^53."""
    a2 = a if lhs_contracting == 1 else a.T
    b2 = b if rhs_contracting == 0 else b.T
    assert a2.shape[1] * 127 * 127 < 2 ** 53
    acc = np.matmul(a2.astype(np.float64), b2.astype(np.float64))
    return acc.astype(np.int64).astype(np.int32)


def dequant_s32_to_bf16(acc: np.ndarray, a_row_scale: np.ndarray, b_col_scale: np.ndarray) -> np.ndarray:
    """convert(s32 -> f32) * a_scale[m] * b_scale[n] -> bf16, the two f32
    multiplies in that order (the loop fusion XLA emits after the s32 GEMM;
    gemm_rewriter.cc:897-901 refuses to fuse it)."""
    y = acc.astype(np.float32)
    y = (y * np.asarray(a_row_scale, dtype=np.float32)[:, None]).astype(np.float32)
    y = (y * np.asarray(b_col_scale, dtype=np.float32)[None, :]).astype(np.float32)
    return f32_to_bf16_bits(y)


# ----------------------------------------------------------------------------
# Comparison, the reference's way.
# ----------------------------------------------------------------------------
def fp8_ordinal(codes: np.ndarray) -> np.ndarray:
    """Maps sign-magnitude FP8 code points onto a monotone integer line so that
    the distance between two values in representable steps is a subtraction
    (literal_comparison.cc:434-453 `CalculateDistanceInFloats`)."""
    c = np.asarray(codes, dtype=np.uint8).astype(np.int32)
    mag = c & 0x7F
    return np.where(c & 0x80, -mag, mag)


def near_mismatches(expected: np.ndarray, actual: np.ndarray, abs_tol: float, rel_tol: float):
    """Count of mismatching elements under xla/literal_comparison.cc:456-556:
    equal values and NaN pairs match; a NaN on one side only or an inf on one
    side only mismatches; otherwise mismatch iff abs_err > abs AND rel_err > rel.
    Returns (count, max_abs_err, max_rel_err over finite pairs)."""
    e = np.asarray(expected, dtype=np.float64).ravel()
    a = np.asarray(actual, dtype=np.float64).ravel()
    both_nan = np.isnan(e) & np.isnan(a)
    one_nan = np.isnan(e) ^ np.isnan(a)
    equal = (e == a) | both_nan
    one_inf = (np.isinf(e) | np.isinf(a)) & ~equal & ~one_nan
    with np.errstate(invalid="ignore", divide="ignore"):
        abs_err = np.abs(a - e)
        rel_err = np.where(e != 0, abs_err / np.abs(e), np.inf)
    finite = ~(equal | one_nan | one_inf)
    bad = one_nan | one_inf | (finite & (abs_err > abs_tol) & (rel_err > rel_tol))
    max_abs = float(abs_err[finite].max()) if finite.any() else 0.0
    fin_rel = finite & (e != 0)
    max_rel = float(rel_err[fin_rel].max()) if fin_rel.any() else 0.0
    return int(bad.sum()), max_abs, max_rel


def fp8_within_n_values(expected_codes, actual_codes, n: int = 1) -> int:
    """Number of elements further than n representable values apart (NaN must
    match NaN).  The reference's `low_precision_fp_error_spec{within_n_values}`
    (xla/error_spec.h:58-78)."""
    e = np.asarray(expected_codes, dtype=np.uint8).ravel()
    a = np.asarray(actual_codes, dtype=np.uint8).ravel()
    e_nan = (e & 0x7F) == 0x7F
    a_nan = (a & 0x7F) == 0x7F
    dist = np.abs(fp8_ordinal(e) - fp8_ordinal(a))
    bad = (e_nan ^ a_nan) | (~e_nan & ~a_nan & (dist > n))
    return int(bad.sum())


# ----------------------------------------------------------------------------
# Seeded inputs of the five BASELINE configurations (seed = 1000*config + index).
# ----------------------------------------------------------------------------
def make_f8_operands(cfg: int, m: int, k: int, n: int, kind_a="e4m3fn", kind_b="e4m3fn"):
    rng_a = np.random.default_rng(1000 * cfg + 0)
    rng_b = np.random.default_rng(1000 * cfg + 1)
    a, a_scale = quantize_per_tensor(rng_a.standard_normal((m, k), dtype=np.float32), kind_a)
    b, b_scale = quantize_per_tensor(rng_b.standard_normal((k, n), dtype=np.float32), kind_b)
    return a, b, a_scale, b_scale


def make_bias_bf16(cfg: int, n: int) -> np.ndarray:
    rng = np.random.default_rng(1000 * cfg + 4)
    return f32_to_bf16_bits((rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)))


def make_s8_operands(cfg: int, m: int, k: int, n: int):
    rng = np.random.default_rng(1000 * cfg + 0)
    a = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    b = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
    a_scale = rng.uniform(0.001, 0.02, size=m).astype(np.float32)
    b_scale = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
    return a, b, a_scale, b_scale
