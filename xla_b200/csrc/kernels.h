// Internal host-side interface between the C-ABI layer and the CUDA kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <string>

struct CUtensorMap_st;   // CUtensorMap of <cuda.h>

// B200SD_TUNING=1 (make TUNING=1 -> libb200_scaled_dot_tuning.so) compiles in what the product
// library leaves out: the per-CTA wait counters the kernels' roles keep (read back with
// b200sd_debug_read_timing / b200sd_debug_read_skinny_timing, switched on by B200SD_TIMING=1) and the
// environment overrides of tile order and pipeline depths.  The product build carries neither.
#ifndef B200SD_TUNING
#define B200SD_TUNING 0
#endif

namespace b200sd {

constexpr bool kTiming = B200SD_TUNING != 0;

// An integer tuning knob: read from the environment in a tuning build, `dflt` in the product build.
inline int TuningEnvInt(const char* name, int dflt) {
#if B200SD_TUNING
  const char* e = std::getenv(name);
  return e != nullptr ? std::atoi(e) : dflt;
#else
  (void)name;
  return dflt;
#endif
}

// xla::PrimitiveType numbers (mirrored by XLA_FFI_DataType, xla/ffi/api/c_api.h:233-266).
enum PrimitiveType : int32_t {
  kInvalidType = 0,
  kS8 = 2,
  kS32 = 4,
  kF16 = 10,
  kF32 = 11,
  kBF16 = 16,
  kF8E5M2 = 19,
  kF8E4M3FN = 20,
  kF8E8M0FNU = 33,
};

// Activation applied after the optional bias.
enum Activation : int32_t { kActNone = 0, kActRelu = 1, kActGelu = 2 };

// Status codes use the numbering of XLA_FFI_Error_Code (xla/ffi/api/c_api.h:168-186), which is
// absl::StatusCode's.
enum Code : int32_t {
  kOk = 0,
  kInvalidArgument = 3,
  kDeadlineExceeded = 4,
  kResourceExhausted = 8,
  kFailedPrecondition = 9,
  kUnimplemented = 12,
  kInternal = 13,
};

struct Status {
  int32_t code = kOk;
  std::string message;
  bool ok() const { return code == kOk; }
  static Status Ok() { return {}; }
  static Status Error(int32_t c, std::string m) { return Status{c, std::move(m)}; }
};

// A fully validated GEMM: D[m,n] = epilogue(sum_k A(m,k) * B(k,n)).  All matrices are dense
// row-major in memory; `a_mn_major` says A is stored [k,m] (contracting dimension 0) and
// `b_mn_major` that B is stored [k,n] (contracting dimension 0).
struct GemmProblem {
  int64_t m = 0, n = 0, k = 0;
  int64_t batch = 1;                 // leading batch dimension shared by A, B, C and D (dense kernel only)
  bool int8 = false;                 // s8 x s8 -> s32 accumulate, else FP8 -> f32 accumulate
  int32_t a_dtype = kF8E4M3FN, b_dtype = kF8E4M3FN;
  bool a_mn_major = false, b_mn_major = true;
  const void* a = nullptr;
  const void* b = nullptr;

  // FP8 epilogue: x = alpha * a_scale * b_scale * acc + beta * C + bias; act; amax; * d_scale; cast.
  const float* a_scale = nullptr;    // device scalars, nullptr = 1.0
  const float* b_scale = nullptr;
  const float* d_scale = nullptr;
  float alpha = 1.0f, beta = 0.0f;
  const void* c = nullptr;
  int32_t c_dtype = kInvalidType;
  const void* bias = nullptr;        // [n]
  int32_t bias_dtype = kInvalidType;
  int32_t activation = kActNone;
  float* amax = nullptr;             // device scalar, overwritten

  // int8 epilogue: y = float(acc) * a_row_scale[m] * b_col_scale[n] (either may be nullptr).
  const float* a_row_scale = nullptr;
  const float* b_col_scale = nullptr;
  int32_t* d_s32 = nullptr;          // optional raw accumulator output

  void* d = nullptr;
  int32_t d_dtype = kBF16;

  void* workspace = nullptr;         // caller-owned scratch for the split-K kernel
  size_t workspace_bytes = 0;

  // Optional progress reporting of the dense kernel, for a consumer on another stream that wants
  // to start on finished row blocks of D (the all-reduce of a K-split dot) before the kernel ends.
  // counters[i] is incremented (never reset) as tiles of rows [i*progress_rows, (i+1)*progress_rows)
  // are stored; ProgressIncrement() is what one launch adds to each counter.
  uint32_t* progress = nullptr;
  int32_t progress_rows = 0;         // multiple of 256
  int32_t max_ctas = 0;              // > 0: use at most this many SMs, leaving the rest to the consumer
};

// A contracting-dimension split over `world` GPUs whose sum is formed inside the dense kernel:
// every rank pushes its bf16 partial of the row blocks it does not own into the owner's staging
// buffer over peer memory, computes its own block last, adds what the others pushed and writes
// the finished rows into every rank's D.  All pointers are indexed by rank and peer-mapped.
constexpr int kMaxPeers = 8;
constexpr uint32_t kDefaultPeerWaitMs = 10000;   // covers launch skew between processes and a first call's lazy loading
struct PeerReduceProblem {
  int32_t world = 1, rank = 0;
  int32_t emulate = 0;               // one launch on one GPU plays all ranks (single-GPU testing)
  uint32_t epoch = 1;                // 1, 2, 3, ...; the same on every rank for the same call
  uint32_t peer_wait_ms = 0;         // limit of a wait for another rank; 0 = kDefaultPeerWaitMs
  void* d[kMaxPeers] = {};
  void* d_multicast = nullptr;       // optional NVSwitch multicast mapping of all the d[i]
  int32_t pull = 0;                  // 1 / 2: partials stay with their producer; the owner of the rows fetches their sum (1: the own tile's warp, 2: reducer warps)
  void* stage_multicast = nullptr;   // pull: optional NVSwitch multicast mapping of all the stage[i] (in-switch sum)
  void* stage[kMaxPeers] = {};       // m*n bf16 each
  uint32_t* flags[kMaxPeers] = {};   // PeerReduceFlagWords() u32 each, zeroed once
  const void* emu_a[kMaxPeers] = {};
  const void* emu_b[kMaxPeers] = {};
};
size_t PeerReduceFlagWords(int64_t m, int64_t n, int32_t world);
struct LaunchStats;
Status LaunchDenseReduce(const GemmProblem& g, const PeerReduceProblem& r, cudaStream_t stream, LaunchStats* stats);

// What one dense launch adds to progress counter `block` (0 when the block is past the last row).
uint32_t ProgressIncrement(const GemmProblem& g, int32_t block);

// Kernel selection (stands in for cuBLASLt's algorithm index).
enum KernelKind : int32_t { kKernelAuto = 0, kKernelDense = 1, kKernelSkinny = 2, kKernelDenseSingle = 3, kKernelDensePair = 4,
                            kKernelDenseStreamK = 5, kKernelMxPair256 = 6, kKernelMxPair224 = 7 };

struct LaunchStats {
  int32_t kernel = 0;     // KernelKind actually used
  int32_t grid = 0;
  int32_t launches = 0;   // kernels launched (memset nodes not counted)
};

// One-time per-device set-up (function attributes, SM count).  Not a stream operation; must not
// be called for the first time while the stream is being captured.
Status InitDevice(int device);

// `variant`: kKernelDense picks between the CTA-pair and the single-CTA instantiation.
Status LaunchDense(const GemmProblem& p, cudaStream_t stream, LaunchStats* stats, int variant = kKernelDense);
Status LaunchSkinny(const GemmProblem& p, cudaStream_t stream, LaunchStats* stats);
size_t SkinnyWorkspaceBytes(int64_t m, int64_t n, int64_t k);

// An MX block-scaled dot: D[b,m,n] = alpha * sum_k A[b,m,k] * 2^(SA[b,m,k/32]-127) * B[b,n,k] * 2^(SB[b,n,k/32]-127).
// Both operands are stored contracting-dimension-minor, the scales row-major [rows, k/32].
struct MxProblem {
  int64_t m = 0, n = 0, k = 0;
  int64_t batch = 1;
  int32_t a_dtype = kF8E4M3FN, b_dtype = kF8E4M3FN;
  int32_t scale_dtype = kF8E8M0FNU;
  const void* a = nullptr;
  const void* b = nullptr;
  const void* a_scale = nullptr;
  const void* b_scale = nullptr;
  // Extents of the scale arrays when they are padded ([batch, rows >= m | n, cols >= k / 32], the form the reference's
  // BuildBlockScaledDotInput slices, block_scaling_rewriter.cc:469-518); 0 = exactly [rows, k / 32].
  int64_t a_scale_rows = 0, a_scale_cols = 0;
  int64_t b_scale_rows = 0, b_scale_cols = 0;
  float alpha = 1.0f;
  void* d = nullptr;
  int32_t d_dtype = kF32;
  int32_t kernel = kKernelAuto;      // kKernelAuto, kKernelMxPair256 or kKernelMxPair224
};
int TunedMxKernel(int64_t m, int64_t n, int64_t k);      // the tuned table's tile form for this shape, or kKernelAuto
Status ValidateMx(const MxProblem& g);      // everything but the pointers
Status LaunchMx(const MxProblem& g, cudaStream_t stream, LaunchStats* stats);

// Reads (and clears) the device status word the kernels OR their error bits into.  Synchronises
// the device.
Status ReadDeviceStatus(uint32_t* bits);

// Runs a tiny kernel whose only wait is on a barrier nobody arrives at, with the given limit, and
// reports through the status word.  Exercises the bounded-wait path without any fault.
Status LaunchWaitProbe(uint64_t limit_ns, cudaStream_t stream);

int DeviceSmCount();

// True while `stream` is being captured into a CUDA graph (an XLA command buffer records a custom
// call this way).  A recorded launch replays with the SAME kernel arguments, so the per-launch epoch
// values that normally stand in for clearing flags and amax cannot tell one replay from the next;
// launches made during capture therefore put a memset node in front of the kernel instead.
inline bool StreamIsCapturing(cudaStream_t stream) {
  cudaStreamCaptureStatus s = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &s) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return s != cudaStreamCaptureStatusNone;
}

// Tensor map of a row-major [rows, cols] byte matrix, `cols` innermost; box = box_cols x box_rows bytes,
// 128-byte swizzle, out-of-range elements read as zero.  `l2_promotion`: 0 none, 1 = 64 B, 2 = 128 B, 3 = 256 B.
Status MakeByteMatrixMap(::CUtensorMap_st* map, const void* base, int64_t rows, int64_t cols, uint32_t box_cols,
                         uint32_t box_rows, int l2_promotion = 3);

// Device address of the current device's status word (valid after InitDevice).
uint32_t* StatusWordPtr();

}  // namespace b200sd
