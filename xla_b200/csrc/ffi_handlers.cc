// XLA FFI handlers: the drop-in boundary.  An XLA process registers these under the custom-call
// targets "b200$scaled_dot$f8" and "b200$dot$s8"; a GemmRewriter that emits those targets instead
// of "__cublas$lt$matmul$f8" / "__cublas$lt$matmul" (xla/service/gpu/cublas_cudnn.h) gets this
// library in place of CublasLtMatmulThunk + cuBLASLt.
//
// Call-frame contract (operand order of ThunkEmitter::EmitCublasLtMatmulF8,
// xla/service/gpu/thunk_emitter.cc:776-862):
//   operands  a, b, [c iff beta != 0], a_scale, b_scale, [bias iff the epilogue adds one],
//             [d_scale iff D is F8E4M3FN / F8E5M2; may be left out when there is no bias, b_scale then
//             doubles as d_scale]
//   results   D, [amax f32[] iff damax_output], [workspace s8[n]]
//   attrs     GemmBackendConfig fields (xla/service/gpu/backend_configs.proto:88-135) as a flat
//             dictionary: alpha_real, beta (f64 or f32), epilogue (i32/i64, enum number),
//             lhs_contracting_dim, rhs_contracting_dim (i64/i32), damax_output (bool),
//             lhs_batch_dims, rhs_batch_dims (i64 arrays, {0} for rank-3 operands),
//             selected_config (i64, optional; 0 = automatic kernel choice).
// XLA_FFI_Buffer carries no layout (xla/ffi/api/c_api.h:273-281): every buffer is row-major and
// transposition is expressed by the contracting dimensions alone.
//
// Stages (xla/ffi/api/c_api.h:413-455): `instantiate` checks types, shapes and attributes with
// no device access; `initialize` does the per-device set-up; `execute` only enqueues work on the
// stream XLA provides -- no allocation and no synchronisation, so the handler is declared
// command-buffer compatible (xla/ffi/api/api.h:251-268).
#include <cuda_runtime.h>

#include <cstdint>
#include <optional>
#include <string>

#define B200SD_NO_FFI_DECLS 1
#include "../../include/b200_scaled_dot.h"
#include <vector>

#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error MakeError(int code, const std::string& msg) {
  return ffi::Error(static_cast<ffi::ErrorCode>(code), msg);
}

// Integer attributes arrive as i64 or i32 depending on how the backend_config was spelled.
std::optional<int64_t> GetInt(const ffi::Dictionary& attrs, std::string_view name) {
  if (attrs.contains<int64_t>(name)) return *attrs.get<int64_t>(name);
  if (attrs.contains<int32_t>(name)) return static_cast<int64_t>(*attrs.get<int32_t>(name));
  return std::nullopt;
}
std::optional<double> GetFloat(const ffi::Dictionary& attrs, std::string_view name) {
  if (attrs.contains<double>(name)) return *attrs.get<double>(name);
  if (attrs.contains<float>(name)) return static_cast<double>(*attrs.get<float>(name));
  return std::nullopt;
}
std::optional<std::vector<int64_t>> GetIntArray(const ffi::Dictionary& attrs, std::string_view name) {
  auto span = attrs.get<ffi::Span<const int64_t>>(name);     // absent (or not an i64 array): no value
  if (!span.has_value()) return std::nullopt;
  return std::vector<int64_t>(span->begin(), span->end());
}
bool GetBool(const ffi::Dictionary& attrs, std::string_view name, bool dflt) {
  if (attrs.contains<bool>(name)) return *attrs.get<bool>(name);
  return dflt;
}

bool EpilogueAddsVectorBias(int64_t e) {
  return e == B200SD_EPILOGUE_BIAS || e == B200SD_EPILOGUE_BIAS_RELU || e == B200SD_EPILOGUE_BIAS_GELU ||
         e == B200SD_EPILOGUE_BIAS_GELU_AUX;
}
bool IsF8(ffi::DataType t) { return t == ffi::DataType::F8E4M3FN || t == ffi::DataType::F8E5M2; }
bool IsScalar(const ffi::AnyBuffer& b) { return b.element_count() == 1; }

struct DecodedF8 {
  B200SD_ScaledDotF8 args;
};

// GemmBackendConfig.lhs_stride / rhs_stride (backend_configs.proto:121-122): the reference's rewriter always writes the
// dense extent of one batch entry, rows * cols (gemm_rewriter.cc:705-721).  Accepted when they say exactly that;
// batches that are not packed back to back are not implemented.
ffi::Error CheckDenseStrides(const ffi::Dictionary& attrs, const ffi::AnyBuffer& lhs, const ffi::AnyBuffer& rhs, size_t bo) {
  const auto ls = GetInt(attrs, "lhs_stride"), rs = GetInt(attrs, "rhs_stride");
  if (ls.has_value() && *ls != lhs.dimensions()[bo] * lhs.dimensions()[bo + 1])
    return MakeError(12, "lhs_stride must be the dense extent of one batch entry of a (rows * cols)");
  if (rs.has_value() && *rs != rhs.dimensions()[bo] * rhs.dimensions()[bo + 1])
    return MakeError(12, "rhs_stride must be the dense extent of one batch entry of b (rows * cols)");
  return ffi::Error::Success();
}

// Decodes and checks a scaled-dot call frame.  Works with null data pointers (instantiate stage).
ffi::Error DecodeF8(ffi::RemainingArgs operands, ffi::RemainingRets results, const ffi::Dictionary& attrs,
                    B200SD_ScaledDotF8* out) {
  B200SD_ScaledDotF8 a{};
  a.struct_size = sizeof(a);
  a.alpha = static_cast<float>(GetFloat(attrs, "alpha_real").value_or(1.0));
  a.beta = static_cast<float>(GetFloat(attrs, "beta").value_or(0.0));
  if (GetFloat(attrs, "alpha_imag").value_or(0.0) != 0.0)
    return MakeError(3, "alpha_imag must be 0 for an FP8 dot");
  a.epilogue = static_cast<int32_t>(GetInt(attrs, "epilogue").value_or(B200SD_EPILOGUE_DEFAULT));
  a.lhs_contracting_dim = static_cast<int32_t>(GetInt(attrs, "lhs_contracting_dim").value_or(1));
  a.rhs_contracting_dim = static_cast<int32_t>(GetInt(attrs, "rhs_contracting_dim").value_or(0));
  a.kernel = static_cast<int32_t>(GetInt(attrs, "selected_config").value_or(B200SD_KERNEL_AUTO));
  const bool damax = GetBool(attrs, "damax_output", false);
  const bool has_c = a.beta != 0.0f;
  const bool has_bias = EpilogueAddsVectorBias(a.epilogue);

  if (results.size() < 1) return MakeError(3, "expected at least one result (D)");
  auto d = results.get<ffi::AnyBuffer>(0);
  if (!d.has_value()) return d.error();
  const bool d_is_f8 = IsF8((*d)->element_type());
  size_t want_operands = 4 + (has_c ? 1 : 0) + (has_bias ? 1 : 0) + (d_is_f8 ? 1 : 0);
  // An FP8 result without a separate d_scale operand: the reference's emitter takes "the last operand" as d_scale
  // whenever D is FP8 (thunk_emitter.cc:812-818), which for the call the rewriter emits for a bare FP8 dot
  // (a, b, 1, 1 -- gemm_rewriter_fp8_test.cc:313-350) is b_scale.  Accepted in exactly that form.
  const bool d_scale_is_last_scale = d_is_f8 && !has_bias && operands.size() + 1 == want_operands;
  if (d_scale_is_last_scale) --want_operands;
  if (operands.size() != want_operands)
    return MakeError(3, "expected " + std::to_string(want_operands) + " operands (a, b, [c], a_scale, b_scale, [bias], [d_scale]) for this "
                        "backend_config, got " + std::to_string(operands.size()));
  const size_t want_results_min = 1 + (damax ? 1 : 0);
  if (results.size() < want_results_min || results.size() > want_results_min + 1)
    return MakeError(3, "expected results (D, [amax], [workspace]), got " + std::to_string(results.size()));

  size_t idx = 0;
  auto lhs = operands.get<ffi::AnyBuffer>(idx++);
  auto rhs = operands.get<ffi::AnyBuffer>(idx++);
  if (!lhs.has_value()) return lhs.error();
  if (!rhs.has_value()) return rhs.error();
  // Rank 2, or rank 3 with ONE leading batch dimension on a, b and D (lhs_batch_dims = rhs_batch_dims = {0},
  // the canonical form the rewriter produces, gemm_rewriter_fp8_test.cc:941-991).  Contracting
  // dimensions are given in the operand's own index space, as DotDimensionNumbers does.
  const size_t rank = lhs->dimensions().size();
  if ((rank != 2 && rank != 3) || rhs->dimensions().size() != rank || (*d)->dimensions().size() != rank)
    return MakeError(12, "operands and result must all have rank 2, or rank 3 with one leading batch dimension");
  const int64_t bo = rank == 3 ? 1 : 0;                  // offset of the matrix dimensions
  {
    auto lb = GetIntArray(attrs, "lhs_batch_dims"), rb = GetIntArray(attrs, "rhs_batch_dims");
    const bool want = rank == 3;
    auto ok = [&](const std::optional<std::vector<int64_t>>& v) {
      if (!v.has_value()) return !want;
      return want ? (v->size() == 1 && (*v)[0] == 0) : v->empty();
    };
    if (!ok(lb) || !ok(rb)) return MakeError(want ? 12 : 3, "lhs_batch_dims and rhs_batch_dims must be {0} for rank-3 operands and empty for rank-2");
  }
  a.batch_count = rank == 3 ? static_cast<int32_t>(lhs->dimensions()[0]) : 1;
  if (rank == 3 && (rhs->dimensions()[0] != lhs->dimensions()[0] || (*d)->dimensions()[0] != lhs->dimensions()[0]))
    return MakeError(3, "batch dimensions of a, b and the result differ");
  if (ffi::Error e = CheckDenseStrides(attrs, *lhs, *rhs, static_cast<size_t>(bo)); e.failure()) return e;
  a.lhs_contracting_dim = static_cast<int32_t>(GetInt(attrs, "lhs_contracting_dim").value_or(bo + 1) - bo);
  a.rhs_contracting_dim = static_cast<int32_t>(GetInt(attrs, "rhs_contracting_dim").value_or(bo) - bo);
  if (a.lhs_contracting_dim != 0 && a.lhs_contracting_dim != 1) return MakeError(3, "lhs_contracting_dim must be one of the two matrix dimensions");
  if (a.rhs_contracting_dim != 0 && a.rhs_contracting_dim != 1) return MakeError(3, "rhs_contracting_dim must be one of the two matrix dimensions");
  a.k = lhs->dimensions()[bo + a.lhs_contracting_dim];
  a.m = lhs->dimensions()[bo + 1 - a.lhs_contracting_dim];
  a.n = rhs->dimensions()[bo + 1 - a.rhs_contracting_dim];
  if (rhs->dimensions()[bo + a.rhs_contracting_dim] != a.k) return MakeError(3, "contracting dimensions of a and b differ");
  if ((*d)->dimensions()[bo] != a.m || (*d)->dimensions()[bo + 1] != a.n) return MakeError(3, "result shape is not [m, n]");
  a.a = lhs->untyped_data();
  a.b = rhs->untyped_data();
  a.a_dtype = static_cast<int32_t>(lhs->element_type());
  a.b_dtype = static_cast<int32_t>(rhs->element_type());
  a.d = (*d)->untyped_data();
  a.d_dtype = static_cast<int32_t>((*d)->element_type());

  if (has_c) {
    auto c = operands.get<ffi::AnyBuffer>(idx++);
    if (!c.has_value()) return c.error();
    if (c->dimensions().size() != rank || c->dimensions()[bo] != a.m || c->dimensions()[bo + 1] != a.n ||
        (rank == 3 && c->dimensions()[0] != a.batch_count))
      return MakeError(3, "matrix bias c must have the result's shape");
    a.c = c->untyped_data();
    a.c_dtype = static_cast<int32_t>(c->element_type());
  }
  auto a_scale = operands.get<ffi::AnyBuffer>(idx++);
  auto b_scale = operands.get<ffi::AnyBuffer>(idx++);
  if (!a_scale.has_value()) return a_scale.error();
  if (!b_scale.has_value()) return b_scale.error();
  if (a_scale->element_type() != ffi::DataType::F32 || b_scale->element_type() != ffi::DataType::F32 ||
      !IsScalar(*a_scale) || !IsScalar(*b_scale))
    return MakeError(3, "a_scale and b_scale must be f32 scalars");
  a.a_scale = static_cast<const float*>(a_scale->untyped_data());
  a.b_scale = static_cast<const float*>(b_scale->untyped_data());
  if (has_bias) {
    auto bias = operands.get<ffi::AnyBuffer>(idx++);
    if (!bias.has_value()) return bias.error();
    if (bias->element_count() != static_cast<size_t>(a.n)) return MakeError(3, "vector bias must have n elements");
    a.bias = bias->untyped_data();
    a.bias_dtype = static_cast<int32_t>(bias->element_type());
  }
  if (d_scale_is_last_scale) {
    a.d_scale = a.b_scale;
  } else if (d_is_f8) {
    auto d_scale = operands.get<ffi::AnyBuffer>(idx++);
    if (!d_scale.has_value()) return d_scale.error();
    if (d_scale->element_type() != ffi::DataType::F32 || !IsScalar(*d_scale))
      return MakeError(3, "d_scale must be an f32 scalar");
    a.d_scale = static_cast<const float*>(d_scale->untyped_data());
  }
  size_t ridx = 1;
  if (damax) {
    auto amax = results.get<ffi::AnyBuffer>(ridx++);
    if (!amax.has_value()) return amax.error();
    if ((*amax)->element_type() != ffi::DataType::F32 || !IsScalar(**amax))
      return MakeError(3, "amax result must be an f32 scalar");
    a.amax = static_cast<float*>((*amax)->untyped_data());
  }
  if (ridx < results.size()) {
    auto ws = results.get<ffi::AnyBuffer>(ridx++);
    if (!ws.has_value()) return ws.error();
    a.workspace = (*ws)->untyped_data();
    a.workspace_bytes = (*ws)->size_bytes();
  }
  *out = a;
  return ffi::Error::Success();
}

ffi::Error DecodeS8(ffi::RemainingArgs operands, ffi::RemainingRets results, const ffi::Dictionary& attrs,
                    B200SD_DotS8* out) {
  B200SD_DotS8 a{};
  a.struct_size = sizeof(a);
  a.kernel = static_cast<int32_t>(GetInt(attrs, "selected_config").value_or(B200SD_KERNEL_AUTO));
  const bool emit_s32 = GetBool(attrs, "emit_s32", false);
  if (GetFloat(attrs, "alpha_real").value_or(1.0) != 1.0 || GetFloat(attrs, "beta").value_or(0.0) != 0.0)
    return MakeError(12, "alpha and beta are not fused into integer dots (the reference does not either)");
  if (operands.size() != 2 && operands.size() != 4)
    return MakeError(3, "expected operands (a, b) or (a, b, a_row_scale, b_col_scale), got " + std::to_string(operands.size()));
  const size_t want_results = 1 + (emit_s32 ? 1 : 0);
  if (results.size() < want_results || results.size() > want_results + 1)
    return MakeError(3, "expected results (D, [acc s32 iff emit_s32], [workspace]), got " + std::to_string(results.size()));
  auto lhs = operands.get<ffi::AnyBuffer>(0);
  auto rhs = operands.get<ffi::AnyBuffer>(1);
  auto d = results.get<ffi::AnyBuffer>(0);
  if (!lhs.has_value()) return lhs.error();
  if (!rhs.has_value()) return rhs.error();
  if (!d.has_value()) return d.error();
  if (lhs->element_type() != ffi::DataType::S8 || rhs->element_type() != ffi::DataType::S8)
    return MakeError(3, "operands must be S8");
  // Rank 2, or rank 3 with one leading batch dimension on a, b, D and the s32 copy (lhs_batch_dims = rhs_batch_dims
  // = {0}), exactly as for the FP8 call; contracting dimensions index the operand as it is.
  const size_t rank = lhs->dimensions().size();
  if ((rank != 2 && rank != 3) || rhs->dimensions().size() != rank || (*d)->dimensions().size() != rank)
    return MakeError(12, "operands and result must all have rank 2, or rank 3 with one leading batch dimension");
  const int64_t bo = rank == 3 ? 1 : 0;
  {
    auto lb = GetIntArray(attrs, "lhs_batch_dims"), rb = GetIntArray(attrs, "rhs_batch_dims");
    const bool want = rank == 3;
    auto ok = [&](const std::optional<std::vector<int64_t>>& v) {
      if (!v.has_value()) return !want;
      return want ? (v->size() == 1 && (*v)[0] == 0) : v->empty();
    };
    if (!ok(lb) || !ok(rb)) return MakeError(want ? 12 : 3, "lhs_batch_dims and rhs_batch_dims must be {0} for rank-3 operands and empty for rank-2");
  }
  a.batch_count = rank == 3 ? lhs->dimensions()[0] : 1;
  if (rank == 3 && (rhs->dimensions()[0] != lhs->dimensions()[0] || (*d)->dimensions()[0] != lhs->dimensions()[0]))
    return MakeError(3, "batch dimensions of a, b and the result differ");
  if (ffi::Error e = CheckDenseStrides(attrs, *lhs, *rhs, static_cast<size_t>(bo)); e.failure()) return e;
  a.lhs_contracting_dim = static_cast<int32_t>(GetInt(attrs, "lhs_contracting_dim").value_or(bo + 1) - bo);
  a.rhs_contracting_dim = static_cast<int32_t>(GetInt(attrs, "rhs_contracting_dim").value_or(bo) - bo);
  if ((a.lhs_contracting_dim | 1) != 1 || (a.rhs_contracting_dim | 1) != 1) return MakeError(3, "contracting dimensions must be the two matrix dimensions");
  a.k = lhs->dimensions()[bo + a.lhs_contracting_dim];
  a.m = lhs->dimensions()[bo + 1 - a.lhs_contracting_dim];
  a.n = rhs->dimensions()[bo + 1 - a.rhs_contracting_dim];
  if (rhs->dimensions()[bo + a.rhs_contracting_dim] != a.k) return MakeError(3, "contracting dimensions of a and b differ");
  if ((*d)->dimensions()[bo] != a.m || (*d)->dimensions()[bo + 1] != a.n) return MakeError(3, "result shape is not [m, n]");
  a.a = lhs->untyped_data();
  a.b = rhs->untyped_data();
  a.d = (*d)->untyped_data();
  a.d_dtype = static_cast<int32_t>((*d)->element_type());
  if (operands.size() == 4) {
    if ((*d)->element_type() == ffi::DataType::S32)
      return MakeError(3, "dequantisation scales need a floating-point output type");
    auto rs = operands.get<ffi::AnyBuffer>(2);
    auto cs = operands.get<ffi::AnyBuffer>(3);
    if (!rs.has_value()) return rs.error();
    if (!cs.has_value()) return cs.error();
    if (rs->element_type() != ffi::DataType::F32 || cs->element_type() != ffi::DataType::F32 ||
        rs->element_count() != static_cast<size_t>(a.m) || cs->element_count() != static_cast<size_t>(a.n))
      return MakeError(3, "a_row_scale must be f32[m] and b_col_scale f32[n]");
    a.a_row_scale = static_cast<const float*>(rs->untyped_data());
    a.b_col_scale = static_cast<const float*>(cs->untyped_data());
  }
  if (emit_s32) {
    auto acc = results.get<ffi::AnyBuffer>(1);
    if (!acc.has_value()) return acc.error();
    if ((*acc)->element_type() != ffi::DataType::S32 || (*acc)->dimensions().size() != rank ||
        (*acc)->dimensions()[bo] != a.m || (*acc)->dimensions()[bo + 1] != a.n ||
        (rank == 3 && (*acc)->dimensions()[0] != lhs->dimensions()[0]))
      return MakeError(3, "the emit_s32 result must be s32[(batch,) m, n]");
    a.acc_out = static_cast<int32_t*>((*acc)->untyped_data());
  }
  if (results.size() == want_results + 1) {       // trailing s8[workspace], as GemmWorkspaceRewriteVisitor appends
    auto ws = results.get<ffi::AnyBuffer>(want_results);
    if (!ws.has_value()) return ws.error();
    a.workspace = (*ws)->untyped_data();
    a.workspace_bytes = (*ws)->size_bytes();
  }
  *out = a;
  return ffi::Error::Success();
}

ffi::Error FromCode(int code, const char* msg) {
  return code == 0 ? ffi::Error::Success() : MakeError(code, msg);
}

// ---- b200$scaled_dot$f8 --------------------------------------------------------------------
ffi::Error ScaledDotF8Instantiate(ffi::RemainingArgs operands, ffi::RemainingRets results, ffi::Dictionary attrs) {
  B200SD_ScaledDotF8 a;
  ffi::Error e = DecodeF8(operands, results, attrs, &a);
  if (e.failure()) return e;
  char msg[512];
  return FromCode(b200sd_check_scaled_dot_f8(&a, msg, sizeof(msg)), msg);
}
ffi::Error InitializeDevice() {
  char msg[512];
  return FromCode(b200sd_init_device(msg, sizeof(msg)), msg);
}
ffi::Error ScaledDotF8Execute(cudaStream_t stream, ffi::RemainingArgs operands, ffi::RemainingRets results,
                              ffi::Dictionary attrs) {
  B200SD_ScaledDotF8 a;
  ffi::Error e = DecodeF8(operands, results, attrs, &a);
  if (e.failure()) return e;
  char msg[512];
  return FromCode(b200sd_scaled_dot_f8(&a, stream, msg, sizeof(msg)), msg);
}

// ---- b200$dot$s8 ---------------------------------------------------------------------------
ffi::Error DotS8Instantiate(ffi::RemainingArgs operands, ffi::RemainingRets results, ffi::Dictionary attrs) {
  B200SD_DotS8 a;
  ffi::Error e = DecodeS8(operands, results, attrs, &a);
  if (e.failure()) return e;
  char msg[512];
  return FromCode(b200sd_check_dot_s8(&a, msg, sizeof(msg)), msg);
}
ffi::Error DotS8Execute(cudaStream_t stream, ffi::RemainingArgs operands, ffi::RemainingRets results,
                        ffi::Dictionary attrs) {
  B200SD_DotS8 a;
  ffi::Error e = DecodeS8(operands, results, attrs, &a);
  if (e.failure()) return e;
  char msg[512];
  return FromCode(b200sd_dot_s8(&a, stream, msg, sizeof(msg)), msg);
}

// ---- b200$block_scaled_dot$mx --------------------------------------------------------------
// Operands (a, b, a_scale, b_scale), results (D, [workspace]): the call ThunkEmitter::EmitCublasLtMatmulMx
// accepts (xla/service/gpu/thunk_emitter.cc:939-988).  Shapes are those of `__op$block_scaled_dot`
// (xla/backends/gpu/transforms/block_scaling_rewriter.h:30-77): a [b, m, k], b [b, n, k], scales
// [b, rows, k / 32], D [b, m, n], the batch dimension optional.  Attribute `alpha_real` is optional.
ffi::Error DecodeMx(ffi::RemainingArgs operands, ffi::RemainingRets results, ffi::Dictionary attrs,
                    B200SD_BlockScaledDotMx* out) {
  B200SD_BlockScaledDotMx a{};
  a.struct_size = sizeof(a);
  a.alpha = static_cast<float>(GetFloat(attrs, "alpha_real").value_or(1.0));
  a.kernel = static_cast<int32_t>(GetInt(attrs, "selected_config").value_or(0));
  if (operands.size() != 4) return MakeError(3, "expected operands (a, b, a_scale, b_scale), got " + std::to_string(operands.size()));
  if (results.size() < 1 || results.size() > 2) return MakeError(3, "expected results (D, [workspace]), got " + std::to_string(results.size()));
  auto lhs = operands.get<ffi::AnyBuffer>(0);
  auto rhs = operands.get<ffi::AnyBuffer>(1);
  auto ls = operands.get<ffi::AnyBuffer>(2);
  auto rs = operands.get<ffi::AnyBuffer>(3);
  auto d = results.get<ffi::AnyBuffer>(0);
  if (!lhs.has_value()) return lhs.error();
  if (!rhs.has_value()) return rhs.error();
  if (!ls.has_value()) return ls.error();
  if (!rs.has_value()) return rs.error();
  if (!d.has_value()) return d.error();
  const size_t rank = lhs->dimensions().size();
  if (rank != 2 && rank != 3) return MakeError(12, "operands must have rank 2, or rank 3 with a leading batch dimension");
  if (rhs->dimensions().size() != rank || ls->dimensions().size() != rank || rs->dimensions().size() != rank ||
      (*d)->dimensions().size() != rank)
    return MakeError(3, "operands, scales and result must all have the same rank");
  const size_t o = rank - 2;
  const int64_t batch = rank == 3 ? lhs->dimensions()[0] : 1;
  a.m = lhs->dimensions()[o];
  a.k = lhs->dimensions()[o + 1];
  a.n = rhs->dimensions()[o];
  if (rhs->dimensions()[o + 1] != a.k) return MakeError(3, "contracting (minor) dimensions of a and b differ");
  // Padded scale arrays are taken as they are: the kernel reads the leading [rows, k / 32] corner.  Extra rows are
  // always allowed; extra columns only when the call states its block size (the `block_size` attribute, from
  // block_scaled_dot_backend_config), because otherwise the block size is the ratio of the minor extents
  // (block_scaling_rewriter.cc:98-113, 489-505).
  const auto block_size = GetInt(attrs, "block_size");
  if (block_size.has_value() && *block_size != 32) return MakeError(12, "block_size must be 32 (MX)");
  const bool cols_ok = block_size.has_value()
                           ? (ls->dimensions()[o + 1] >= a.k / 32 && rs->dimensions()[o + 1] >= a.k / 32)
                           : (ls->dimensions()[o + 1] == a.k / 32 && rs->dimensions()[o + 1] == a.k / 32);
  if (a.k % 32 != 0 || ls->dimensions()[o] < a.m || rs->dimensions()[o] < a.n || !cols_ok)
    return MakeError(3, "scales must cover [rows, k / 32]: one scale per block of 32 along the contracting dimension");
  a.a_scale_rows = ls->dimensions()[o];
  a.a_scale_cols = ls->dimensions()[o + 1];
  a.b_scale_rows = rs->dimensions()[o];
  a.b_scale_cols = rs->dimensions()[o + 1];
  if ((*d)->dimensions()[o] != a.m || (*d)->dimensions()[o + 1] != a.n) return MakeError(3, "result shape is not [m, n]");
  if (rank == 3 && (rhs->dimensions()[0] != batch || ls->dimensions()[0] != batch || rs->dimensions()[0] != batch ||
                    (*d)->dimensions()[0] != batch))
    return MakeError(3, "batch dimensions differ");
  if (ls->element_type() != rs->element_type()) return MakeError(3, "a_scale and b_scale must have the same type");
  a.batch_count = static_cast<int32_t>(batch);
  a.a_dtype = static_cast<int32_t>(lhs->element_type());
  a.b_dtype = static_cast<int32_t>(rhs->element_type());
  a.scale_dtype = static_cast<int32_t>(ls->element_type());
  a.d_dtype = static_cast<int32_t>((*d)->element_type());
  a.a = lhs->untyped_data();
  a.b = rhs->untyped_data();
  a.a_scale = ls->untyped_data();
  a.b_scale = rs->untyped_data();
  a.d = (*d)->untyped_data();
  *out = a;
  return ffi::Error::Success();
}
ffi::Error BlockScaledDotMxInstantiate(ffi::RemainingArgs operands, ffi::RemainingRets results, ffi::Dictionary attrs) {
  B200SD_BlockScaledDotMx a;
  ffi::Error e = DecodeMx(operands, results, attrs, &a);
  if (e.failure()) return e;
  char msg[512];
  return FromCode(b200sd_check_block_scaled_dot_mx(&a, msg, sizeof(msg)), msg);
}
ffi::Error BlockScaledDotMxExecute(cudaStream_t stream, ffi::RemainingArgs operands, ffi::RemainingRets results,
                                   ffi::Dictionary attrs) {
  B200SD_BlockScaledDotMx a;
  ffi::Error e = DecodeMx(operands, results, attrs, &a);
  if (e.failure()) return e;
  char msg[512];
  return FromCode(b200sd_block_scaled_dot_mx(&a, stream, msg, sizeof(msg)), msg);
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(b200sd_ffi_block_scaled_dot_mx_instantiate, BlockScaledDotMxInstantiate,
                              ffi::Ffi::BindInstantiate().RemainingArgs().RemainingRets().Attrs());
XLA_FFI_DEFINE_HANDLER_SYMBOL(b200sd_ffi_block_scaled_dot_mx_initialize, InitializeDevice, ffi::Ffi::BindInitialize());
XLA_FFI_DEFINE_HANDLER_SYMBOL(b200sd_ffi_block_scaled_dot_mx, BlockScaledDotMxExecute,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .RemainingArgs()
                                  .RemainingRets()
                                  .Attrs(),
                              {ffi::Traits::kCmdBufferCompatible});

XLA_FFI_DEFINE_HANDLER_SYMBOL(b200sd_ffi_scaled_dot_f8_instantiate, ScaledDotF8Instantiate,
                              ffi::Ffi::BindInstantiate().RemainingArgs().RemainingRets().Attrs());
XLA_FFI_DEFINE_HANDLER_SYMBOL(b200sd_ffi_scaled_dot_f8_initialize, InitializeDevice, ffi::Ffi::BindInitialize());
XLA_FFI_DEFINE_HANDLER_SYMBOL(b200sd_ffi_scaled_dot_f8, ScaledDotF8Execute,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .RemainingArgs()
                                  .RemainingRets()
                                  .Attrs(),
                              {ffi::Traits::kCmdBufferCompatible});

XLA_FFI_DEFINE_HANDLER_SYMBOL(b200sd_ffi_dot_s8_instantiate, DotS8Instantiate,
                              ffi::Ffi::BindInstantiate().RemainingArgs().RemainingRets().Attrs());
XLA_FFI_DEFINE_HANDLER_SYMBOL(b200sd_ffi_dot_s8_initialize, InitializeDevice, ffi::Ffi::BindInitialize());
XLA_FFI_DEFINE_HANDLER_SYMBOL(b200sd_ffi_dot_s8, DotS8Execute,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .RemainingArgs()
                                  .RemainingRets()
                                  .Attrs(),
                              {ffi::Traits::kCmdBufferCompatible});

extern "C" int b200sd_ffi_register(const void* xla_ffi_api, char* err, size_t err_len) {
  const XLA_FFI_Api* api = static_cast<const XLA_FFI_Api*>(xla_ffi_api);
  if (api == nullptr) {
    if (err && err_len) snprintf(err, err_len, "XLA_FFI_Api pointer is null");
    return 3;
  }
  struct Target {
    const char* name;
    XLA_FFI_Handler_Bundle bundle;
  } targets[] = {
      {"b200$scaled_dot$f8",
       {b200sd_ffi_scaled_dot_f8_instantiate, nullptr, b200sd_ffi_scaled_dot_f8_initialize, b200sd_ffi_scaled_dot_f8}},
      {"b200$dot$s8", {b200sd_ffi_dot_s8_instantiate, nullptr, b200sd_ffi_dot_s8_initialize, b200sd_ffi_dot_s8}},
      {"b200$block_scaled_dot$mx",
       {b200sd_ffi_block_scaled_dot_mx_instantiate, nullptr, b200sd_ffi_block_scaled_dot_mx_initialize,
        b200sd_ffi_block_scaled_dot_mx}},
  };
  for (const Target& t : targets) {
    XLA_FFI_Error* e = ffi::Ffi::RegisterStaticHandler(api, t.name, "CUDA", t.bundle,
                                                       XLA_FFI_HANDLER_TRAITS_COMMAND_BUFFER_COMPATIBLE);
    if (e != nullptr) {
      XLA_FFI_Error_GetDetails_Args details{};
      details.struct_size = XLA_FFI_Error_GetDetails_Args_STRUCT_SIZE;
      details.error = e;
      api->XLA_FFI_Error_GetDetails(&details);
      if (err && err_len) snprintf(err, err_len, "registering %s: %s", t.name, details.message ? details.message : "?");
      const int code = static_cast<int>(details.errc);
      XLA_FFI_Error_Destroy_Args destroy{};
      destroy.struct_size = XLA_FFI_Error_Destroy_Args_STRUCT_SIZE;
      destroy.error = e;
      api->XLA_FFI_Error_Destroy(&destroy);
      return code ? code : 13;
    }
  }
  return 0;
}
