// Plain C entry points of libb200_scaled_dot.so: argument validation (the checks the reference
// spreads over GemmRewriter::CreateF8CustomCall, TypesAreSupportedByCublasLt and
// cuda::BlasLt::GetMatmulPlan), kernel selection (instead of the cuBLASLt autotuner) and launch.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <shared_mutex>
#include <tuple>
#include <cstddef>
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/b200_scaled_dot.h"
#include "kernels.h"
#include "ptx.cuh"

namespace b200sd {

// Status word the kernels OR their error bits into (one instance per device that loads the
// library).  Kernels receive its device address as an argument.
__device__ uint32_t g_device_status;

Status InitDenseKernels();
Status InitSkinnyKernels();
Status InitMxKernels();

namespace {

struct DeviceState {
  std::once_flag once;
  Status init_status;
  int sm_count = 0;
  uint32_t* status_word = nullptr;
};
DeviceState g_state[64];
std::atomic<uint64_t> g_launches{0};

int CopyStatus(const Status& s, char* err, size_t err_len) {
  if (err != nullptr && err_len > 0) {
    const size_t n = s.message.size() < err_len - 1 ? s.message.size() : err_len - 1;
    std::memcpy(err, s.message.data(), n);
    err[n] = '\0';
  }
  return s.code;
}

bool IsF8(int32_t t) { return t == kF8E4M3FN || t == kF8E5M2; }

__global__ void wait_probe_kernel(uint64_t limit_ns, uint32_t* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
    // Nobody ever arrives on `bar`: the wait below can only end through its time limit.
    (void)mbar_wait(&bar, 0, &abort_flag, status, kStatusProbeTimeout, limit_ns);
  }
}

}  // namespace

extern "C" int b200sd_load_config_table(const char* path, int32_t* entries, char* err, size_t err_len);

Status InitDevice(int device) {
  if (device < 0 || device >= 64) return Status::Error(kInvalidArgument, "device ordinal out of range");
  DeviceState& st = g_state[device];
  std::call_once(st.once, [&] {
    cudaDeviceProp prop{};
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) {
      st.init_status = Status::Error(kInternal, std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e));
      return;
    }
    if (prop.major != 10) {
      st.init_status = Status::Error(kFailedPrecondition,
                                     "libb200_scaled_dot needs an sm_100 (Blackwell B200) device, found sm_" +
                                         std::to_string(prop.major) + std::to_string(prop.minor));
      return;
    }
    st.sm_count = prop.multiProcessorCount;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&st.status_word), g_device_status);
    if (e != cudaSuccess) {
      st.init_status = Status::Error(kInternal, std::string("cudaGetSymbolAddress(status): ") + cudaGetErrorString(e));
      return;
    }
    st.init_status = InitDenseKernels();
    if (st.init_status.ok()) st.init_status = InitSkinnyKernels();
    if (st.init_status.ok()) st.init_status = InitMxKernels();
    // A persisted tuning result named by the environment is loaded with the first device (a file
    // that cannot be read or parsed makes the first call fail loudly instead of being ignored).
    static std::once_flag table_once;
    std::call_once(table_once, [&] {
      const char* path = std::getenv("B200SD_CONFIG_TABLE");
      if (path == nullptr || path[0] == 0 || !st.init_status.ok()) return;
      char msg[512] = {0};
      const int rc = b200sd_load_config_table(path, nullptr, msg, sizeof msg);
      if (rc != 0) st.init_status = Status::Error(rc, std::string("B200SD_CONFIG_TABLE: ") + msg);
    });
  });
  return st.init_status;
}

int DeviceSmCount() {
  int device = 0;
  cudaGetDevice(&device);
  return (device >= 0 && device < 64 && g_state[device].sm_count > 0) ? g_state[device].sm_count : 148;
}

uint32_t* StatusWordPtr() {
  int device = 0;
  cudaGetDevice(&device);
  return (device >= 0 && device < 64) ? g_state[device].status_word : nullptr;
}

Status ReadDeviceStatus(uint32_t* bits) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return Status::Error(kInternal, std::string("cudaDeviceSynchronize: ") + cudaGetErrorString(e));
  uint32_t v = 0, zero = 0;
  e = cudaMemcpyFromSymbol(&v, g_device_status, sizeof(v));
  if (e == cudaSuccess && v != 0) e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero));
  if (e != cudaSuccess) return Status::Error(kInternal, std::string("status word copy: ") + cudaGetErrorString(e));
  *bits = v;
  return Status::Ok();
}

Status LaunchWaitProbe(uint64_t limit_ns, cudaStream_t stream) {
  if (limit_ns > 1000000000ull) return Status::Error(kInvalidArgument, "probe limit above one second");
  int device = 0;
  cudaGetDevice(&device);
  Status st = InitDevice(device);
  if (!st.ok()) return st;
  wait_probe_kernel<<<1, 32, 0, stream>>>(limit_ns, StatusWordPtr());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return Status::Error(kInternal, std::string("wait_probe_kernel launch: ") + cudaGetErrorString(e));
  return Status::Ok();
}

// Tuned kernel choices keyed by (type: 0 f8, 1 s8, 2 mx; m, n, k): what `selected_algorithm` of a persisted
// autotuning result is to the reference (xla/backends/gpu/autotuner/cublaslt.cc:84-189 picks an
// algorithm by timing, docs/persisted_autotuning.md stores it).  Filled by b200sd_load_config_table;
// read-mostly, so lookups take a shared lock only.
struct ConfigKey {
  int32_t int8;
  int64_t m, n, k;
  bool operator<(const ConfigKey& o) const { return std::tie(int8, m, n, k) < std::tie(o.int8, o.m, o.n, o.k); }
};
std::shared_mutex g_config_mutex;
std::map<ConfigKey, int32_t> g_config_table;

// Kernel choice for B200SD_KERNEL_AUTO: the tuned table first, then the static rule -- decode-shaped
// problems (few rows of A, a weight matrix that has to be streamed once from HBM) go to the split-K
// kernel, everything else to the dense kernel.
int SelectKernelFor(bool int8, int64_t m, int64_t n, int64_t k) {
  {
    std::shared_lock<std::shared_mutex> lock(g_config_mutex);
    auto it = g_config_table.find(ConfigKey{int8 ? 1 : 0, m, n, k});
    if (it != g_config_table.end()) return it->second;
  }
  if (!int8 && m <= 128 && n >= 1024 && k >= 1024 && SkinnyWorkspaceBytes(m, n, k) > 0) {
    // Decode shapes are bound by streaming the weights.  When the 256-column strips of the dense
    // single-CTA kernel fill one wave of the 148 SMs well (or many waves), each CTA streams its own
    // strip over all of K with nothing to combine afterwards, which measures faster than splitting K
    // (8192 x 28672, 112 strips: 5.56 / 5.47 / 5.32 TB/s against 5.35 / 5.46 / 4.89 at M = 16 / 64 / 128).
    // Few strips (the per-GPU shards of an N-split) leave SMs without work: split K then.
    constexpr int64_t kSms = 148;
    const int64_t strips = (n + 255) / 256;
    const int64_t last_wave = strips % kSms == 0 ? kSms : strips % kSms;
    if (strips >= 4 * kSms || (strips >= (kSms * 7) / 10 && last_wave >= (kSms * 7) / 10)) return kKernelDense;
    return kKernelSkinny;
  }
  return kKernelDense;
}
int SelectKernel(int64_t m, int64_t n, int64_t k) { return SelectKernelFor(false, m, n, k); }

// The tuned tile form of the block-scaled kernel for this shape, or kKernelAuto when the table has no entry (the
// launch then decides from the number of CTA pairs the device runs at once).
int TunedMxKernel(int64_t m, int64_t n, int64_t k) {
  std::shared_lock<std::shared_mutex> lock(g_config_mutex);
  auto it = g_config_table.find(ConfigKey{2, m, n, k});
  return it != g_config_table.end() ? it->second : kKernelAuto;
}

Status ValidateF8(const B200SD_ScaledDotF8& in, GemmProblem* g, bool check_pointers = true) {
  // The struct grew by batch_count; older callers pass the shorter size and get a plain matrix product.
  if (in.struct_size < offsetof(B200SD_ScaledDotF8, batch_count)) return Status::Error(kInvalidArgument, "B200SD_ScaledDotF8.struct_size is smaller than this library's struct");
  B200SD_ScaledDotF8 a{};
  memcpy(&a, &in, in.struct_size < sizeof(a) ? in.struct_size : sizeof(a));
  if (a.batch_count == 0) a.batch_count = 1;
  if (a.batch_count < 0 || a.batch_count > (1 << 20)) return Status::Error(kInvalidArgument, "batch_count out of range");
  if (check_pointers && (a.a == nullptr || a.b == nullptr || a.d == nullptr)) return Status::Error(kInvalidArgument, "a, b and d must not be null");
  if (!IsF8(a.a_dtype) || !IsF8(a.b_dtype)) return Status::Error(kInvalidArgument, "operands must be F8E4M3FN or F8E5M2");
  if (a.a_dtype == kF8E5M2 && a.b_dtype == kF8E5M2) return Status::Error(kUnimplemented, "F8E5M2 x F8E5M2 is not a supported FP8 dot (one operand must be F8E4M3FN)");
  const int32_t d = a.d_dtype;
  if (!(d == kBF16 || d == kF16 || d == kF32 || d == kF8E4M3FN || d == kF8E5M2)) return Status::Error(kInvalidArgument, "output type must be BF16, F16, F32, F8E4M3FN or F8E5M2");
  if (d == kF8E5M2 && a.a_dtype == kF8E4M3FN && a.b_dtype == kF8E4M3FN) return Status::Error(kUnimplemented, "F8E4M3FN x F8E4M3FN -> F8E5M2 is not in the supported type table");
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return Status::Error(kInvalidArgument, "m, n and k must be positive");
  if (a.m % 16 || a.n % 16 || a.k % 16) return Status::Error(kInvalidArgument, "m, n and k must be multiples of 16 (pad as the rewriter does)");
  if (a.m > (1ll << 30) || a.n > (1ll << 30) || a.k > (1ll << 30)) return Status::Error(kInvalidArgument, "dimension too large");
  if ((a.lhs_contracting_dim | 1) != 1 || (a.rhs_contracting_dim | 1) != 1) return Status::Error(kInvalidArgument, "contracting dimensions must be 0 or 1");
  if (a.kernel < B200SD_KERNEL_AUTO || a.kernel > B200SD_KERNEL_DENSE_STREAMK) return Status::Error(kInvalidArgument, "unknown kernel selection " + std::to_string(a.kernel));
  bool has_bias = false;
  int32_t act = kActNone;
  switch (a.epilogue) {
    case B200SD_EPILOGUE_DEFAULT: break;
    case B200SD_EPILOGUE_BIAS: has_bias = true; break;
    case B200SD_EPILOGUE_RELU: act = kActRelu; break;
    case B200SD_EPILOGUE_BIAS_RELU: has_bias = true; act = kActRelu; break;
    case B200SD_EPILOGUE_GELU: act = kActGelu; break;
    case B200SD_EPILOGUE_BIAS_GELU: has_bias = true; act = kActGelu; break;
    case B200SD_EPILOGUE_GELU_AUX:
    case B200SD_EPILOGUE_BIAS_GELU_AUX: return Status::Error(kUnimplemented, "epilogues with an auxiliary output are not implemented");
    case B200SD_EPILOGUE_SILU:
    case B200SD_EPILOGUE_BIAS_SILU: return Status::Error(kUnimplemented, "SILU epilogues are not supported");
    default: return Status::Error(kInvalidArgument, "unknown epilogue " + std::to_string(a.epilogue));
  }
  if (has_bias) {
    if (check_pointers && a.bias == nullptr) return Status::Error(kInvalidArgument, "epilogue adds a vector bias but bias is null");
    if (!(a.bias_dtype == kBF16 || a.bias_dtype == kF16 || a.bias_dtype == kF32)) return Status::Error(kInvalidArgument, "bias must be BF16, F16 or F32");
  }
  if (a.beta != 0.0f) {
    if (check_pointers && a.c == nullptr) return Status::Error(kInvalidArgument, "beta != 0 but c is null");
    if (!(a.c_dtype == kBF16 || a.c_dtype == kF16 || a.c_dtype == kF32)) return Status::Error(kInvalidArgument, "c must be BF16, F16 or F32");
  }
  g->m = a.m; g->n = a.n; g->k = a.k;
  g->int8 = false;
  g->a_dtype = a.a_dtype; g->b_dtype = a.b_dtype;
  g->a_mn_major = a.lhs_contracting_dim == 0;
  g->b_mn_major = a.rhs_contracting_dim == 0;
  g->a = a.a; g->b = a.b;
  g->a_scale = a.a_scale; g->b_scale = a.b_scale; g->d_scale = a.d_scale;
  g->alpha = a.alpha; g->beta = a.beta;
  g->c = a.beta != 0.0f ? a.c : nullptr; g->c_dtype = a.c_dtype;
  g->bias = has_bias ? a.bias : nullptr; g->bias_dtype = a.bias_dtype;
  g->activation = act;
  g->amax = a.amax;
  g->d = a.d; g->d_dtype = a.d_dtype;
  g->workspace = a.workspace; g->workspace_bytes = a.workspace_bytes;
  g->batch = a.batch_count;
  return Status::Ok();
}

Status ValidateS8(const B200SD_DotS8& in, GemmProblem* g, bool check_pointers = true) {
  // The struct grew by the workspace fields; older callers pass the shorter size and get none.
  if (in.struct_size < offsetof(B200SD_DotS8, workspace)) return Status::Error(kInvalidArgument, "B200SD_DotS8.struct_size is smaller than this library's struct");
  B200SD_DotS8 a{};
  memcpy(&a, &in, in.struct_size < sizeof(a) ? in.struct_size : sizeof(a));
  if (check_pointers && (a.a == nullptr || a.b == nullptr || a.d == nullptr)) return Status::Error(kInvalidArgument, "a, b and d must not be null");
  if (!(a.d_dtype == kS32 || a.d_dtype == kF32 || a.d_dtype == kBF16)) return Status::Error(kInvalidArgument, "output type must be S32, F32 or BF16");
  if (a.d_dtype == kS32 && (a.a_row_scale || a.b_col_scale)) return Status::Error(kInvalidArgument, "dequantisation scales need a floating-point output type");
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return Status::Error(kInvalidArgument, "m, n and k must be positive");
  if (a.m % 16 || a.n % 16 || a.k % 16) return Status::Error(kInvalidArgument, "m, n and k must be multiples of 16");
  if (a.m > (1ll << 30) || a.n > (1ll << 30) || a.k > (1ll << 30)) return Status::Error(kInvalidArgument, "dimension too large");
  if (a.kernel == B200SD_KERNEL_SKINNY || a.kernel < B200SD_KERNEL_AUTO || a.kernel > B200SD_KERNEL_DENSE_STREAMK) return Status::Error(kInvalidArgument, "integer dots run on the dense kernel only");
  // |sum| <= k * (-128 * -128) = k * 2^14 must stay below 2^31.
  if (a.k >= 131072) return Status::Error(kInvalidArgument, "k too large for exact s32 accumulation of s8 products (k must be below 131072)");
  if ((a.lhs_contracting_dim | 1) != 1 || (a.rhs_contracting_dim | 1) != 1) return Status::Error(kInvalidArgument, "contracting dimensions must be 0 or 1");
  g->m = a.m; g->n = a.n; g->k = a.k;
  g->int8 = true;
  g->a_dtype = kS8; g->b_dtype = kS8;
  g->a_mn_major = a.lhs_contracting_dim == 0;
  g->b_mn_major = a.rhs_contracting_dim == 0;
  g->a = a.a; g->b = a.b;
  g->a_row_scale = a.a_row_scale; g->b_col_scale = a.b_col_scale;
  g->d_s32 = a.acc_out;
  g->d = a.d; g->d_dtype = a.d_dtype;
  g->workspace = a.workspace; g->workspace_bytes = a.workspace_bytes;
  g->batch = a.batch_count > 0 ? a.batch_count : 1;
  if (a.batch_count < 0 || a.batch_count > (1 << 20)) return Status::Error(kInvalidArgument, "batch_count out of range");
  return Status::Ok();
}

}  // namespace b200sd

using namespace b200sd;

extern "C" {

int b200sd_init_device(char* err, size_t err_len) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return CopyStatus(Status::Error(kInternal, std::string("cudaGetDevice: ") + cudaGetErrorString(e)), err, err_len);
  return CopyStatus(InitDevice(device), err, err_len);
}

int b200sd_scaled_dot_f8(const B200SD_ScaledDotF8* args, void* cuda_stream, char* err, size_t err_len) {
  if (args == nullptr) return CopyStatus(Status::Error(kInvalidArgument, "args is null"), err, err_len);
  GemmProblem g;
  Status st = ValidateF8(*args, &g);
  if (!st.ok()) return CopyStatus(st, err, err_len);
  int kernel = args->kernel;
  if (kernel == B200SD_KERNEL_AUTO) kernel = g.batch > 1 ? B200SD_KERNEL_DENSE : SelectKernel(g.m, g.n, g.k);
  if (kernel == B200SD_KERNEL_SKINNY && g.batch > 1) return CopyStatus(Status::Error(kInvalidArgument, "the split-K kernel does not take batched dots"), err, err_len);
  if (kernel == B200SD_KERNEL_SKINNY) {
    // The split-K kernel covers the plain scaled dot only; fall back to the dense kernel for the rest
    // or when the caller's workspace is too small.
    // ... with a bf16 / f16 / f32 result: its store path knows no FP8 cast and no d_scale.
    const bool plain = g.c == nullptr && g.bias == nullptr && g.activation == kActNone && g.amax == nullptr &&
                       g.d_scale == nullptr && (g.d_dtype == kBF16 || g.d_dtype == kF16 || g.d_dtype == kF32) &&
                       !g.a_mn_major && g.b_mn_major && g.m <= 128 && g.a_dtype == kF8E4M3FN &&
                       g.b_dtype == kF8E4M3FN;
    const size_t need = SkinnyWorkspaceBytes(g.m, g.n, g.k);
    if (!plain || need == 0 || g.workspace == nullptr || g.workspace_bytes < need) {
      if (args->kernel == B200SD_KERNEL_SKINNY)
        return CopyStatus(Status::Error(kInvalidArgument, "the split-K kernel needs m <= 128, row-major A[m,k] and B[k,n], e4m3 operands, "
                                                          "a bf16/f16/f32 result, no bias/activation/amax/d_scale and a workspace of "
                                                          "b200sd_workspace_bytes()"),
                          err, err_len);
      kernel = B200SD_KERNEL_DENSE;
    }
  }
  LaunchStats stats;
  st = kernel == B200SD_KERNEL_SKINNY ? LaunchSkinny(g, static_cast<cudaStream_t>(cuda_stream), &stats)
                                      : LaunchDense(g, static_cast<cudaStream_t>(cuda_stream), &stats, kernel);
  if (st.ok()) g_launches.fetch_add(stats.launches, std::memory_order_relaxed);
  return CopyStatus(st, err, err_len);
}

namespace {
Status ConvertMx(const B200SD_BlockScaledDotMx& a, MxProblem* g) {
  if (a.struct_size < offsetof(B200SD_BlockScaledDotMx, a_scale_rows)) return Status::Error(kInvalidArgument, "B200SD_BlockScaledDotMx.struct_size is smaller than this library's struct");
  if (a.struct_size >= sizeof(B200SD_BlockScaledDotMx)) {
    g->a_scale_rows = a.a_scale_rows; g->a_scale_cols = a.a_scale_cols;
    g->b_scale_rows = a.b_scale_rows; g->b_scale_cols = a.b_scale_cols;
  }
  g->m = a.m; g->n = a.n; g->k = a.k;
  g->batch = a.batch_count > 1 ? a.batch_count : 1;
  g->a_dtype = a.a_dtype; g->b_dtype = a.b_dtype;
  g->scale_dtype = a.scale_dtype;
  g->a = a.a; g->b = a.b;
  g->a_scale = a.a_scale; g->b_scale = a.b_scale;
  g->alpha = a.alpha;
  g->d = a.d; g->d_dtype = a.d_dtype;
  g->kernel = a.kernel;
  if (a.batch_count < 0) return Status::Error(kInvalidArgument, "batch_count must not be negative");
  return ValidateMx(*g);
}
}  // namespace

int b200sd_check_block_scaled_dot_mx(const B200SD_BlockScaledDotMx* args, char* err, size_t err_len) {
  if (args == nullptr) return CopyStatus(Status::Error(kInvalidArgument, "args is null"), err, err_len);
  MxProblem g;
  return CopyStatus(ConvertMx(*args, &g), err, err_len);
}

int b200sd_block_scaled_dot_mx(const B200SD_BlockScaledDotMx* args, void* cuda_stream, char* err, size_t err_len) {
  if (args == nullptr) return CopyStatus(Status::Error(kInvalidArgument, "args is null"), err, err_len);
  MxProblem g;
  Status st = ConvertMx(*args, &g);
  if (!st.ok()) return CopyStatus(st, err, err_len);
  LaunchStats stats;
  st = LaunchMx(g, static_cast<cudaStream_t>(cuda_stream), &stats);
  if (st.ok()) g_launches.fetch_add(stats.launches, std::memory_order_relaxed);
  return CopyStatus(st, err, err_len);
}

int b200sd_scaled_dot_f8_progress(const B200SD_ScaledDotF8* args, B200SD_Progress* progress, void* cuda_stream, char* err,
                                  size_t err_len) {
  if (args == nullptr || progress == nullptr) return CopyStatus(Status::Error(kInvalidArgument, "args or progress is null"), err, err_len);
  if (progress->struct_size < sizeof(B200SD_Progress)) return CopyStatus(Status::Error(kInvalidArgument, "B200SD_Progress.struct_size is smaller than this library's struct"), err, err_len);
  GemmProblem g;
  Status st = ValidateF8(*args, &g);
  if (!st.ok()) return CopyStatus(st, err, err_len);
  if (args->kernel != B200SD_KERNEL_AUTO && args->kernel != B200SD_KERNEL_DENSE) return CopyStatus(Status::Error(kInvalidArgument, "progress reporting exists for the dense kernel only (kernel AUTO or DENSE)"), err, err_len);
  if (progress->counters == nullptr) return CopyStatus(Status::Error(kInvalidArgument, "progress counters must not be null"), err, err_len);
  if (progress->rows_per_block <= 0 || progress->rows_per_block % 256 != 0) return CopyStatus(Status::Error(kInvalidArgument, "rows_per_block must be a positive multiple of 256"), err, err_len);
  if (progress->max_ctas < 0) return CopyStatus(Status::Error(kInvalidArgument, "max_ctas must not be negative"), err, err_len);
  g.progress = progress->counters;
  g.progress_rows = progress->rows_per_block;
  g.max_ctas = progress->max_ctas;
  progress->num_blocks = int32_t((g.m + g.progress_rows - 1) / g.progress_rows);
  progress->increment = ProgressIncrement(g, 0);
  progress->last_increment = ProgressIncrement(g, progress->num_blocks - 1);
  LaunchStats stats;
  st = LaunchDense(g, static_cast<cudaStream_t>(cuda_stream), &stats, B200SD_KERNEL_DENSE);
  if (st.ok()) g_launches.fetch_add(stats.launches, std::memory_order_relaxed);
  return CopyStatus(st, err, err_len);
}

int b200sd_scaled_dot_f8_peer_reduce(const B200SD_ScaledDotF8* args, const B200SD_PeerReduce* peers, void* cuda_stream, char* err,
                                     size_t err_len) {
  if (args == nullptr || peers == nullptr) return CopyStatus(Status::Error(kInvalidArgument, "args or peers is null"), err, err_len);
  if (peers->struct_size < offsetof(B200SD_PeerReduce, peer_wait_ms)) return CopyStatus(Status::Error(kInvalidArgument, "B200SD_PeerReduce.struct_size is smaller than this library's struct"), err, err_len);
  GemmProblem g;
  Status st = ValidateF8(*args, &g);
  if (!st.ok()) return CopyStatus(st, err, err_len);
  PeerReduceProblem r;
  r.world = peers->world;
  r.rank = peers->rank;
  r.emulate = peers->emulate_ranks;
  r.epoch = peers->epoch;
  r.d_multicast = peers->d_multicast;
  r.peer_wait_ms = peers->struct_size >= offsetof(B200SD_PeerReduce, pull) ? peers->peer_wait_ms : 0;
  if (peers->struct_size >= sizeof(B200SD_PeerReduce)) {
    r.pull = peers->pull;
    r.stage_multicast = peers->stage_multicast;
  }
  if (r.peer_wait_ms > 600000u) return CopyStatus(Status::Error(kInvalidArgument, "peer_wait_ms above ten minutes"), err, err_len);
  for (int i = 0; i < kMaxPeers; ++i) {
    r.d[i] = peers->d[i];
    r.stage[i] = peers->stage[i];
    r.flags[i] = peers->flags[i];
    r.emu_a[i] = peers->emu_a[i];
    r.emu_b[i] = peers->emu_b[i];
  }
  LaunchStats stats;
  st = LaunchDenseReduce(g, r, static_cast<cudaStream_t>(cuda_stream), &stats);
  if (st.ok()) g_launches.fetch_add(stats.launches, std::memory_order_relaxed);
  return CopyStatus(st, err, err_len);
}

size_t b200sd_peer_reduce_flag_words(int64_t m, int64_t n, int32_t world) { return PeerReduceFlagWords(m, n, world); }

int b200sd_stream_wait_counter(void* cuda_stream, const uint32_t* counter, uint32_t target, char* err, size_t err_len) {
  // A stream memory operation, not a kernel: the waiting stream holds no SM while it waits and the
  // producer never waits for it.
  typedef CUresult (*WaitValueFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
  static WaitValueFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return reinterpret_cast<WaitValueFn>(p);
  }();
  if (fn == nullptr) return CopyStatus(Status::Error(kInternal, "cuStreamWaitValue32 is not available from this driver"), err, err_len);
  if (counter == nullptr) return CopyStatus(Status::Error(kInvalidArgument, "counter is null"), err, err_len);
  const CUresult r = fn(static_cast<CUstream>(cuda_stream), reinterpret_cast<CUdeviceptr>(counter), target, CU_STREAM_WAIT_VALUE_GEQ);
  if (r != CUDA_SUCCESS) return CopyStatus(Status::Error(kInternal, "cuStreamWaitValue32 failed with CUresult " + std::to_string(int(r))), err, err_len);
  return CopyStatus(Status::Ok(), err, err_len);
}

int b200sd_dot_s8(const B200SD_DotS8* args, void* cuda_stream, char* err, size_t err_len) {
  if (args == nullptr) return CopyStatus(Status::Error(kInvalidArgument, "args is null"), err, err_len);
  GemmProblem g;
  Status st = ValidateS8(*args, &g);
  if (!st.ok()) return CopyStatus(st, err, err_len);
  LaunchStats stats;
  int kernel = args->kernel;
  if (kernel == B200SD_KERNEL_AUTO) {
    kernel = g.batch > 1 ? B200SD_KERNEL_DENSE : SelectKernelFor(true, g.m, g.n, g.k);
    if (kernel == B200SD_KERNEL_SKINNY) kernel = B200SD_KERNEL_DENSE;       // a table entry cannot send an integer dot there
  }
  st = LaunchDense(g, static_cast<cudaStream_t>(cuda_stream), &stats, kernel);
  if (st.ok()) g_launches.fetch_add(stats.launches, std::memory_order_relaxed);
  return CopyStatus(st, err, err_len);
}

int b200sd_check_scaled_dot_f8(const B200SD_ScaledDotF8* args, char* err, size_t err_len) {
  if (args == nullptr) return CopyStatus(Status::Error(kInvalidArgument, "args is null"), err, err_len);
  GemmProblem g;
  return CopyStatus(ValidateF8(*args, &g, /*check_pointers=*/false), err, err_len);
}

int b200sd_check_dot_s8(const B200SD_DotS8* args, char* err, size_t err_len) {
  if (args == nullptr) return CopyStatus(Status::Error(kInvalidArgument, "args is null"), err, err_len);
  GemmProblem g;
  return CopyStatus(ValidateS8(*args, &g, /*check_pointers=*/false), err, err_len);
}

size_t b200sd_workspace_bytes(int64_t m, int64_t n, int64_t k) {
  return SelectKernel(m, n, k) == kKernelSkinny ? SkinnyWorkspaceBytes(m, n, k) : 0;
}

int b200sd_select_kernel(int64_t m, int64_t n, int64_t k) { return SelectKernel(m, n, k); }

int b200sd_tuned_kernel_mx(int64_t m, int64_t n, int64_t k) { return TunedMxKernel(m, n, k); }

int b200sd_load_config_table(const char* path, int32_t* entries, char* err, size_t err_len) {
  if (entries != nullptr) *entries = 0;
  if (path == nullptr) return CopyStatus(Status::Error(kInvalidArgument, "path is null"), err, err_len);
  FILE* f = std::fopen(path, "r");
  if (f == nullptr) return CopyStatus(Status::Error(kInvalidArgument, std::string("cannot open ") + path), err, err_len);
  std::map<ConfigKey, int32_t> table;
  char line[256];
  int lineno = 0;
  Status st = Status::Ok();
  while (std::fgets(line, sizeof line, f) != nullptr) {
    ++lineno;
    char* p = line;
    while (*p == ' ' || *p == '\t') ++p;
    if (*p == '#' || *p == '\n' || *p == '\r' || *p == 0) continue;
    char type[8];
    long long m, n, k;
    int kernel;
    const bool parsed = std::sscanf(p, "%7s %lld %lld %lld %d", type, &m, &n, &k, &kernel) == 5;
    const int type_code = !parsed ? -1 : std::strcmp(type, "f8") == 0 ? 0 : std::strcmp(type, "s8") == 0 ? 1 : std::strcmp(type, "mx") == 0 ? 2 : -1;
    const bool kernel_ok = type_code == 2 ? (kernel == B200SD_KERNEL_MX_256 || kernel == B200SD_KERNEL_MX_224)
                                          : (kernel >= B200SD_KERNEL_DENSE && kernel <= B200SD_KERNEL_DENSE_STREAMK &&
                                             !(type_code == 1 && kernel == B200SD_KERNEL_SKINNY));
    if (type_code < 0 || m <= 0 || n <= 0 || k <= 0 || !kernel_ok) {
      st = Status::Error(kInvalidArgument, std::string(path) + ":" + std::to_string(lineno) +
                                               ": expected `f8|s8 m n k kernel` with kernel 1..5, or `mx m n k kernel` with kernel 6 or 7");
      break;
    }
    table[ConfigKey{type_code, m, n, k}] = kernel;
  }
  std::fclose(f);
  if (!st.ok()) return CopyStatus(st, err, err_len);          // a bad file changes nothing
  {
    std::unique_lock<std::shared_mutex> lock(g_config_mutex);
    g_config_table.swap(table);
    if (entries != nullptr) *entries = int32_t(g_config_table.size());
  }
  return CopyStatus(Status::Ok(), err, err_len);
}

uint64_t b200sd_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int b200sd_device_status(uint32_t* bits, char* err, size_t err_len) {
  if (bits == nullptr) return CopyStatus(Status::Error(kInvalidArgument, "bits is null"), err, err_len);
  return CopyStatus(ReadDeviceStatus(bits), err, err_len);
}

int b200sd_wait_probe(uint64_t limit_ns, void* cuda_stream, char* err, size_t err_len) {
  return CopyStatus(LaunchWaitProbe(limit_ns, static_cast<cudaStream_t>(cuda_stream)), err, err_len);
}

}  // extern "C"
