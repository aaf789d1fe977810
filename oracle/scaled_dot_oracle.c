/* CPU oracle for XLA's quantized scaled-dot path, plain C.  TEST INFRASTRUCTURE ONLY.
 *
 * A strict restatement of the HLO interpreter's arithmetic for the pattern that
 * GemmRewriter lowers to `__cublas$lt$matmul$f8` and for the s8 x s8 -> s32 dot:
 * operands are dequantised element by element into f32, products are accumulated
 * sequentially over k in f32 and the result is cast once at the end
 * (xla/hlo/evaluator/hlo_evaluator_typed_visitor.h:1271-1340).  The product
 * library never links or loads this file; tests and the benchmark's CPU-baseline
 * leg are its only users.
 *
 * Parity status: conversions pinned against xla/tests/convert_test.cc:1093-1257
 * through tests/golden/; the dot has no stored golden output in the reference
 * (see the header of scaled_dot_oracle.py) and XLA's CPU backend is not buildable
 * in this environment.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

/* kind: 0 = e4m3fn (1-4-3, bias 7, no inf, 0x7f NaN), 1 = e5m2 (1-5-2, bias 15, IEEE). */
float oracle_fp8_decode(uint8_t code, int kind) {
  const int mbits = kind == 0 ? 3 : 2, ebits = kind == 0 ? 4 : 5, bias = kind == 0 ? 7 : 15;
  const int e = (code >> mbits) & ((1 << ebits) - 1), m = code & ((1 << mbits) - 1);
  const int emax = (1 << ebits) - 1;
  float v;
  if (kind == 0 && e == emax && m == 7) v = NAN;
  else if (kind == 1 && e == emax) v = m ? NAN : INFINITY;
  else if (e == 0) v = ldexpf((float)m, 1 - bias - mbits);
  else v = ldexpf(1.0f + (float)m / (float)(1 << mbits), e - bias);
  return (code & 0x80) ? -v : v;
}

/* f32 -> FP8, round to nearest even; e4m3fn overflow -> NaN, e5m2 overflow -> inf
 * (xla/tests/convert_test.cc:1144-1194). */
uint8_t oracle_fp8_encode(float x, int kind) {
  const int mbits = kind == 0 ? 3 : 2, ebits = kind == 0 ? 4 : 5, bias = kind == 0 ? 7 : 15;
  const float vmax = kind == 0 ? 448.0f : 57344.0f;
  uint32_t bits; memcpy(&bits, &x, 4);
  const uint8_t sign = (uint8_t)((bits >> 31) << 7);
  const uint8_t nan_code = kind == 0 ? 0x7f : 0x7e, inf_code = kind == 0 ? 0x7f : 0x7c;
  if (isnan(x)) return sign | nan_code;
  if (isinf(x)) return sign | inf_code;
  double a = fabs((double)x);
  if (a == 0.0) return sign;
  int e; frexp(a, &e); e -= 1;                 /* a = f * 2^e, f in [1,2) */
  const int emin = 1 - bias;
  if (e < emin) e = emin;
  const double quantum = ldexp(1.0, e - mbits);
  double r = nearbyint(a / quantum) * quantum; /* default rounding mode: half to even */
  if (r > vmax) return sign | inf_code;
  if (r == 0.0) return sign;
  int e2; frexp(r, &e2); e2 -= 1;
  if (r < ldexp(1.0, emin)) return sign | (uint8_t)nearbyint(r / ldexp(1.0, emin - mbits));
  const int man = (int)nearbyint((r / ldexp(1.0, e2) - 1.0) * (1 << mbits));
  return sign | (uint8_t)(((e2 + bias) << mbits) | man);
}

uint16_t oracle_f32_to_bf16(float x) {
  uint32_t u; memcpy(&u, &x, 4);
  if (isnan(x)) return (uint16_t)((u >> 16) | 0x40);
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

static float gelu_tanh(float x) { /* gemm_rewriter.cc:924-971, every step in f32 */
  float x2 = x * x, x3 = x * x2, t0 = x3 * 0.044715f, t1 = x + t0, t2 = t1 * 0.797884583f;
  float th = tanhf(t2), t3 = th + 1.0f, cdf = t3 * 0.5f;
  return x * cdf;
}

/* out_f32[m,n] = epi(alpha * sum_k (A*a_scale)(B*b_scale) + beta*C + bias), sequential k in f32.
 * a is [m,k] when lhs_contracting == 1 else [k,m]; b is [k,n] when rhs_contracting == 0 else
 * [n,k]; all row-major.  epilogue uses GemmBackendConfig.Epilogue numbering
 * (xla/service/gpu/backend_configs.proto:106-117).  Returns amax = max|out| with NaN
 * propagation (hlo_evaluator_typed_visitor.h:594-613). */
float oracle_scaled_dot_f8(const uint8_t* a, const uint8_t* b, float a_scale, float b_scale,
                           int a_kind, int b_kind, int64_t m, int64_t n, int64_t k,
                           int lhs_contracting, int rhs_contracting, float alpha, float beta,
                           const float* c, const float* bias, int epilogue, float* out_f32) {
  float amax = -INFINITY; int saw_nan = 0;
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      float acc = 0.0f;
      for (int64_t kk = 0; kk < k; ++kk) {
        const uint8_t ca = lhs_contracting == 1 ? a[i * k + kk] : a[kk * m + i];
        const uint8_t cb = rhs_contracting == 0 ? b[kk * n + j] : b[j * k + kk];
        const float av = oracle_fp8_decode(ca, a_kind) * a_scale;
        const float bv = oracle_fp8_decode(cb, b_kind) * b_scale;
        const float prod = av * bv;
        acc = acc + prod;
      }
      float x = acc;
      if (alpha != 1.0f) x = x * alpha;
      if (c && beta != 0.0f) x = x + beta * c[i * n + j];
      if (epilogue == 2 || epilogue == 4 || epilogue == 7 || epilogue == 8) x = x + bias[j];
      if (epilogue == 3 || epilogue == 4) x = isnan(x) ? x : (x > 0.0f ? x : 0.0f);
      else if (epilogue >= 5 && epilogue <= 8) x = gelu_tanh(x);
      out_f32[i * n + j] = x;
      if (isnan(x)) saw_nan = 1; else if (fabsf(x) > amax) amax = fabsf(x);
    }
  }
  return saw_nan ? NAN : amax;
}

/* s8 x s8 -> s32, exact (hlo_evaluator_typed_visitor.h:1330-1336). */
void oracle_dot_s8(const int8_t* a, const int8_t* b, int64_t m, int64_t n, int64_t k,
                   int lhs_contracting, int rhs_contracting, int32_t* out) {
  for (int64_t i = 0; i < m; ++i)
    for (int64_t j = 0; j < n; ++j) {
      int32_t acc = 0;
      for (int64_t kk = 0; kk < k; ++kk) {
        const int32_t av = lhs_contracting == 1 ? a[i * k + kk] : a[kk * m + i];
        const int32_t bv = rhs_contracting == 0 ? b[kk * n + j] : b[j * k + kk];
        acc += av * bv;
      }
      out[i * n + j] = acc;
    }
}
