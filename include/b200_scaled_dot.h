/* b200_scaled_dot.h -- C ABI of libb200_scaled_dot.so.
 *
 * A B200 (sm_100a) replacement for the GPU half of XLA's quantized scaled dot: the work that
 * `CublasLtMatmulThunk::ExecuteOnStream` hands to cuBLASLt for the custom calls
 * `__cublas$lt$matmul$f8` and (s8 x s8) `__cublas$lt$matmul`.
 *
 * Two layers are exported:
 *   1. plain entry points taking a parameter struct of raw device pointers and sizes;
 *   2. XLA FFI handlers (`XLA_FFI_Error* fn(XLA_FFI_CallFrame*)`) that decode a call frame and
 *      call layer 1 -- these are what an XLA process registers as custom-call targets.
 *
 * Conventions: every matrix is dense and row-major; transposition is expressed through the
 * contracting-dimension index exactly as `DotDimensionNumbers` does.  Pointers are device
 * pointers valid on the current CUDA device; the caller owns every buffer.  Work is enqueued on
 * the given stream and nothing synchronises.  Return value: 0 on success, otherwise an
 * `absl::StatusCode` / `XLA_FFI_Error_Code` number (3 INVALID_ARGUMENT, 12 UNIMPLEMENTED,
 * 13 INTERNAL ...), with a message copied into `err` when `err_len > 0`.
 */
#ifndef B200_SCALED_DOT_H_
#define B200_SCALED_DOT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types use xla::PrimitiveType numbers (= XLA_FFI_DataType, xla/ffi/api/c_api.h:233-266). */
enum {
  B200SD_S8 = 2,
  B200SD_S32 = 4,
  B200SD_F16 = 10,
  B200SD_F32 = 11,
  B200SD_BF16 = 16,
  B200SD_F8E5M2 = 19,
  B200SD_F8E4M3FN = 20,
  B200SD_F8E8M0FNU = 33          /* the scale type of MX block-scaled operands */
};

/* GemmBackendConfig.Epilogue, with the enum's own (0-based) numbers
 * (xla/service/gpu/backend_configs.proto:106-117), so that a backend_config written by
 * GemmRewriter is understood as it stands. */
enum {
  B200SD_EPILOGUE_DEFAULT = 0,
  B200SD_EPILOGUE_BIAS = 1,
  B200SD_EPILOGUE_RELU = 2,
  B200SD_EPILOGUE_BIAS_RELU = 3,
  B200SD_EPILOGUE_GELU = 4,
  B200SD_EPILOGUE_GELU_AUX = 5,       /* not implemented: returns UNIMPLEMENTED (as thunk_emitter.cc:842 for FP8) */
  B200SD_EPILOGUE_BIAS_GELU = 6,
  B200SD_EPILOGUE_BIAS_GELU_AUX = 7,  /* not implemented: returns UNIMPLEMENTED */
  B200SD_EPILOGUE_SILU = 8,           /* not implemented: returns UNIMPLEMENTED (as cuda_blas_lt.cc:142-146) */
  B200SD_EPILOGUE_BIAS_SILU = 9       /* not implemented: returns UNIMPLEMENTED */
};

/* Kernel choice; plays the role of GemmBackendConfig.selected_algorithm. */
enum {
  B200SD_KERNEL_AUTO = 0,
  B200SD_KERNEL_DENSE = 1,        /* dense kernel, pair or single-CTA instantiation chosen by shape */
  B200SD_KERNEL_SKINNY = 2,       /* split-K kernel for decode shapes */
  B200SD_KERNEL_DENSE_SINGLE = 3, /* one CTA per 128 x 256 tile */
  B200SD_KERNEL_DENSE_PAIR = 4,   /* two-CTA clusters on 256 x 256 tiles (tcgen05 cta_group::2) */
  B200SD_KERNEL_DENSE_STREAMK = 5,/* DENSE_PAIR whose tiles past the last full wave are cut along K, one equal share per
                                     cluster (needs the workspace; plain DENSE_PAIR when the shape has no such tail) */
  B200SD_KERNEL_MX_256 = 6,       /* block-scaled dot only: 256 x 256 tiles, one accumulator in TMEM */
  B200SD_KERNEL_MX_224 = 7        /* block-scaled dot only: 256 x 224 tiles, two accumulators (epilogue under the next main loop) */
};

/* Arguments of one FP8 scaled dot.
 *
 *   D = cast( d_scale * act( alpha * a_scale * b_scale * dot(A, B) + beta * C + bias ) )
 *   amax = max | act(...) |                     (value before d_scale, f32)
 *
 * Mirrors what `cuda::BlasLt::MatmulPlan::ExecuteOnStream` passes to cublasLtMatmul
 * (xla/stream_executor/cuda/cuda_blas_lt.cc:456-576) and the operand meaning fixed by
 * `ThunkEmitter::EmitCublasLtMatmulF8` (xla/service/gpu/thunk_emitter.cc:776-862).
 * A is [m,k] when lhs_contracting_dim == 1, [k,m] when 0; B is [k,n] when rhs_contracting_dim
 * == 0, [n,k] when 1.  m, n and k must be multiples of 16 (the rewriter pads to 16,
 * xla/backends/gpu/transforms/gemm_rewriter.cc:1556-1580).
 */
typedef struct B200SD_ScaledDotF8 {
  size_t struct_size;            /* sizeof(B200SD_ScaledDotF8), for forward compatibility */
  const void* a;
  const void* b;
  const void* c;                 /* optional matrix bias [m,n], used when beta != 0 */
  const void* bias;              /* optional vector bias [n] */
  const float* a_scale;          /* device scalars; NULL means 1.0 */
  const float* b_scale;
  const float* d_scale;
  void* d;                       /* [m,n] */
  float* amax;                   /* optional device scalar, overwritten */
  void* workspace;               /* scratch owned by the caller (the custom call's s8[] result) */
  size_t workspace_bytes;
  int64_t m, n, k;
  int32_t a_dtype, b_dtype;      /* B200SD_F8E4M3FN or B200SD_F8E5M2, not both e5m2 */
  int32_t c_dtype, bias_dtype;   /* B200SD_BF16, B200SD_F16 or B200SD_F32 */
  int32_t d_dtype;               /* BF16, F16, F32, F8E4M3FN or F8E5M2 */
  int32_t lhs_contracting_dim;   /* 0 or 1 */
  int32_t rhs_contracting_dim;   /* 0 or 1 */
  int32_t epilogue;              /* B200SD_EPILOGUE_* */
  float alpha, beta;
  int32_t kernel;                /* B200SD_KERNEL_* */
  int32_t batch_count;           /* 0 or 1: plain matrices.  > 1: A, B, C and D carry this leading batch dimension ([batch, m, k] ...,
                                    dense row-major, lhs/rhs_batch_dims = {0} as in gemm_rewriter_fp8_test.cc:941-991);
                                    the bias vector, the scales and amax are shared by all batches */
} B200SD_ScaledDotF8;

/* Arguments of one s8 x s8 dot with s32 accumulation, optionally followed by the dequantising
 * multiply XLA emits as a separate loop fusion (gemm_rewriter.cc:897-901 refuses to fuse it):
 *   acc = dot(A, B)                                  exact, s32
 *   D   = cast( f32(acc) * a_row_scale[m] * b_col_scale[n] )
 * d_dtype S32 returns acc itself (what `__cublas$lt$matmul` with I32 compute returns,
 * xla/stream_executor/cuda/cuda_blas_lt.cc:444-445).  `acc_out`, when not NULL, additionally
 * receives acc so that the s32 intermediate can be checked bit for bit.
 */
typedef struct B200SD_DotS8 {
  size_t struct_size;
  const void* a;
  const void* b;
  const float* a_row_scale;      /* optional [m] */
  const float* b_col_scale;      /* optional [n] */
  void* d;
  int32_t* acc_out;              /* optional s32 [m,n] */
  int64_t m, n, k;
  int32_t d_dtype;               /* S32, F32 or BF16 */
  int32_t lhs_contracting_dim;
  int32_t rhs_contracting_dim;
  int32_t kernel;                /* B200SD_KERNEL_AUTO, _DENSE, _DENSE_SINGLE or _DENSE_PAIR */
  /* Fields below were added later: a caller whose struct_size stops before them gets NULL / 0. */
  void* workspace;               /* optional scratch (the custom call's s8[] result); lets the kernel balance its last wave */
  size_t workspace_bytes;
  int64_t batch_count;           /* > 1: leading batch dimension of A, B, D and acc_out; the scale vectors are shared */
} B200SD_DotS8;

/* Arguments of one MX block-scaled dot (`scale_mode = BLOCK_SCALING` of GemmBackendConfig):
 *
 *   D[b,m,n] = alpha * sum_k  A[b,m,k] * 2^(SA[b,m,k/32] - 127)  *  B[b,n,k] * 2^(SB[b,n,k/32] - 127)
 *
 * The operand list is that of `ThunkEmitter::EmitCublasLtMatmulMx`
 * (xla/service/gpu/thunk_emitter.cc:939-988): a, b, a_scale, b_scale and one result (plus the
 * workspace XLA appends, which this kernel does not need); no bias, no matrix C, no d_scale, no
 * amax.  Layout is the one `__op$block_scaled_dot` fixes
 * (xla/backends/gpu/transforms/block_scaling_rewriter.h:30-77): the contracting dimension is
 * the minor one of BOTH operands (A is [m,k], B is [n,k]), an optional batch dimension is the
 * major one, and each scale tensor is row-major [rows, k/32] of f8e8m0fnu -- the plain HLO
 * operand, not a library-specific swizzled form.  k must be a multiple of 32; m and n are free.
 * The scale arrays may be padded ([batch, rows >= m|n, cols >= k/32], given by the *_scale_rows /
 * *_scale_cols fields): only the leading [rows, k/32] corner is read, exactly the slice
 * `BuildBlockScaledDotInput` takes (xla/backends/gpu/transforms/block_scaling_rewriter.cc:469-518).
 */
typedef struct B200SD_BlockScaledDotMx {
  size_t struct_size;            /* sizeof(B200SD_BlockScaledDotMx) */
  const void* a;                 /* [batch, m, k] FP8 */
  const void* b;                 /* [batch, n, k] FP8 */
  const void* a_scale;           /* [batch, m, k/32] f8e8m0fnu */
  const void* b_scale;           /* [batch, n, k/32] f8e8m0fnu */
  void* d;                       /* [batch, m, n] */
  int64_t m, n, k;
  int32_t a_dtype, b_dtype;      /* B200SD_F8E4M3FN or B200SD_F8E5M2 */
  int32_t scale_dtype;           /* B200SD_F8E8M0FNU */
  int32_t d_dtype;               /* F32, BF16 or F16 */
  float alpha;                   /* GemmBackendConfig.alpha_real; XLA writes 1 */
  int32_t batch_count;           /* 0 or 1: plain matrices */
  int32_t kernel;                /* B200SD_KERNEL_AUTO, B200SD_KERNEL_MX_256 or B200SD_KERNEL_MX_224 */
  /* Fields below were added later: a caller whose struct_size stops before them gets 0 (no padding). */
  int64_t a_scale_rows;          /* extents of a padded a_scale, [batch, a_scale_rows, a_scale_cols]; 0 = m and k/32 */
  int64_t a_scale_cols;
  int64_t b_scale_rows;          /* the same for b_scale; 0 = n and k/32 */
  int64_t b_scale_cols;
} B200SD_BlockScaledDotMx;

/* One-time set-up for the current device (kernel attributes, SM count).  Called implicitly by the
 * first launch on a device; call it yourself before capturing a stream into a CUDA graph. */
int b200sd_init_device(char* err, size_t err_len);

/* Replaces the cublasLtMatmul call of xla/stream_executor/cuda/cuda_blas_lt.cc:559-564 (FP8). */
int b200sd_scaled_dot_f8(const B200SD_ScaledDotF8* args, void* cuda_stream, char* err, size_t err_len);

/* Replaces the same call for s8 x s8 -> s32 (type table at cuda_blas_lt.cc:444-445). */
int b200sd_dot_s8(const B200SD_DotS8* args, void* cuda_stream, char* err, size_t err_len);

/* Replaces the library call behind `__cublas$lt$matmul$mx` (CublasLtMatmulThunk built by
 * xla/service/gpu/thunk_emitter.cc:939-988 with GemmConfig::scale_mode == BLOCK_SCALING). */
int b200sd_block_scaled_dot_mx(const B200SD_BlockScaledDotMx* args, void* cuda_stream, char* err, size_t err_len);
int b200sd_check_block_scaled_dot_mx(const B200SD_BlockScaledDotMx* args, char* err, size_t err_len);

/* Validate everything about a call except the pointer values (which may be NULL): types, shapes,
 * epilogue, the supported type table (`TypesAreSupportedByCublasLt`,
 * xla/backends/gpu/transforms/gemm_rewriter.cc:2425-2677).  No device access; this is what the FFI
 * handlers run in the `instantiate` stage. */
int b200sd_check_scaled_dot_f8(const B200SD_ScaledDotF8* args, char* err, size_t err_len);
int b200sd_check_dot_s8(const B200SD_DotS8* args, char* err, size_t err_len);

/* Bytes of workspace the split-K kernel wants for a problem (0 when the dense kernel is used).
 * XLA always provides 32 MiB (xla/service/gpu/matmul_utils.h:103), which covers every case. */
size_t b200sd_workspace_bytes(int64_t m, int64_t n, int64_t k);

/* Which kernel B200SD_KERNEL_AUTO picks; the static stand-in for the cuBLASLt autotuner
 * (xla/backends/gpu/autotuner/cublaslt.cc:84-189). */
int b200sd_select_kernel(int64_t m, int64_t n, int64_t k);

/* The tile form (B200SD_KERNEL_MX_256 / _224) the tuned table holds for an MX block-scaled dot of
 * this shape, or B200SD_KERNEL_AUTO when it has no entry: the launch then chooses from the tile
 * counts and the number of CTA pairs the device runs at once. */
int b200sd_tuned_kernel_mx(int64_t m, int64_t n, int64_t k);

/* Replaces the tuned kernel choices of this process with those in a text file, one per line:
 *     f8|s8  m  n  k  kernel          (kernel = B200SD_KERNEL_* 1..5; `#` starts a comment)
 *     mx     m  n  k  kernel          (kernel = B200SD_KERNEL_MX_256 or _MX_224)
 * B200SD_KERNEL_AUTO then uses an entry whose (type, m, n, k) matches exactly and the static rule
 * otherwise.  The file is what a persisted autotuning result is to the reference
 * (docs/persisted_autotuning.md; the cuBLASLt backend of the autotuner,
 * xla/backends/gpu/autotuner/cublaslt.cc:84-189, times the algorithms and keeps the best);
 * `python -m xla_b200.autotune` writes one.  A malformed file is rejected as a whole. */
int b200sd_load_config_table(const char* path, int32_t* entries, char* err, size_t err_len);

/* Number of kernels this library has launched in the calling process (for benchmarks). */
uint64_t b200sd_launch_count(void);

/* Synchronises the device, then returns and clears the bit mask kernels set when one of their
 * bounded waits expired (0 = healthy).  The host-visible half of failure detection; stands where
 * the reference relies on its execution watchdog (xla/service/gpu/execution_watchdog.h:43-61). */
int b200sd_device_status(uint32_t* bits, char* err, size_t err_len);

/* Launches a one-thread kernel that waits `limit_ns` on a barrier nobody signals and then reports
 * through the status word (value 16).  Lets a test watch a wait expire without faulting anything. */
int b200sd_wait_probe(uint64_t limit_ns, void* cuda_stream, char* err, size_t err_len);

/* Row-block progress of a dense scaled dot, for overlapping the all-reduce of a contracting-
 * dimension split (xla/service/spmd/dot_handler.cc:2815-2951 emits dot -> all-reduce; XLA's own
 * overlap of that pair is the async collective scheduling of
 * xla/backends/gpu/runtime/all_reduce_thunk.cc:89-150, which cannot start before the dot ends).
 * `counters[i]` (u32, device memory, caller-owned, at least `num_blocks` entries, zeroed once by
 * the caller and never reset by the library) grows by `increment` per launch as rows
 * [i*rows_per_block, (i+1)*rows_per_block) of D are stored (`last_increment` for the last, possibly
 * shorter, block).  A consumer stream calls b200sd_stream_wait_counter() with the running total it
 * expects and may then read those rows.  `max_ctas` > 0 caps the SMs the kernel occupies so the
 * consumer's kernels can run beside it.  The three outputs are filled in by the call. */
typedef struct B200SD_Progress {
  size_t struct_size;
  uint32_t* counters;
  int32_t rows_per_block;   /* positive multiple of 256 */
  int32_t max_ctas;         /* 0 = all SMs */
  int32_t num_blocks;       /* out */
  uint32_t increment;       /* out */
  uint32_t last_increment;  /* out */
} B200SD_Progress;

/* b200sd_scaled_dot_f8 on the dense kernel, reporting progress as described above. */
int b200sd_scaled_dot_f8_progress(const B200SD_ScaledDotF8* args, B200SD_Progress* progress, void* cuda_stream,
                                  char* err, size_t err_len);

/* Enqueues on `cuda_stream` a wait (a stream memory operation, no kernel) until
 * (int32)(*counter - target) >= 0. */
int b200sd_stream_wait_counter(void* cuda_stream, const uint32_t* counter, uint32_t target, char* err, size_t err_len);

/* Contracting-dimension split over `world` GPUs of one box with the sum formed inside the dot's
 * kernel, over peer memory, instead of by a separate all-reduce.  Replaces the pair
 * dot -> all-reduce that xla/service/spmd/dot_handler.cc:2815-2951 emits and
 * xla/backends/gpu/runtime/all_reduce_thunk.cc:89-150 /
 * xla/backends/gpu/collectives/nccl_communicator.cc:557-592 execute.
 *
 * Every rank calls this with its own K-shard in `args` (a, b, scales; args->d = d[rank]; bf16
 * result, no epilogue).  The rows are dealt out to the ranks in sub-blocks.  (Default, push mode:) rank r pushes the bf16
 * partial of the sub-blocks it does not own into the owner's `stage` buffer while its tensor cores
 * work on the next tile; for a sub-block it owns it adds the partials the others pushed (in rank
 * order, in f32, rounded once) and writes the finished rows into every rank's `d`.  When the
 * kernel ends on a rank, that rank's `d` is complete.  m must be a multiple of 256*world.
 *
 * d[i], stage[i] (m*n*2 bytes) and flags[i] (b200sd_peer_reduce_flag_words() u32, zeroed once when
 * allocated, never by the library) are rank i's buffers as mapped into THIS process (peer memory:
 * symmetric-memory or IPC mappings); the same buffers must be passed on every call of a sequence
 * and `epoch` must count the calls 1, 2, 3, ... identically on every rank.
 *
 * Failure and recovery.  Waits between ranks are bounded: `peer_wait_ms` milliseconds (0 = 10 s,
 * long enough for the launch skew of separate processes and the lazy loading of a first call).  A
 * wait that gives up sets bit 32 of the status word and the kernel drains; the call has still
 * returned 0 when it was enqueued, and D then holds incomplete sums.  So a caller MUST read
 * b200sd_device_status() after a call (or a step of calls) before it trusts D.  The flag counters
 * only grow and their targets are multiples of `epoch`, so after one such failure every later
 * call would miss its targets too: re-arm before going on -- every rank synchronises its device,
 * zeroes its own flags buffer, all ranks meet in a barrier (any host-side one), and the epoch
 * restarts at 1.  Because the epoch is an argument fixed at enqueue time, this call is not meant to
 * be recorded into a CUDA graph.
 *
 * emulate_ranks == world makes ONE launch on ONE GPU play every rank (each with its own operands
 * emu_a[i], emu_b[i] and 1/world of the SMs): the way to exercise the protocol without a second
 * GPU.  It synchronises the stream once before the launch. */
typedef struct B200SD_PeerReduce {
  size_t struct_size;
  int32_t world;
  int32_t rank;
  int32_t emulate_ranks;
  uint32_t epoch;
  void* d[8];
  void* stage[8];
  uint32_t* flags[8];
  const void* emu_a[8];
  const void* emu_b[8];
  void* d_multicast;   /* optional: an NVSwitch multicast address bound to every rank's d (same offset);
                          finished rows then leave this GPU once and the switch replicates them */
  /* Added later: a caller whose struct_size stops before this field gets the default. */
  uint32_t peer_wait_ms; /* limit of every wait for another rank, milliseconds; 0 = 10000 */
  int32_t pull;          /* 1 or 2: partials stay in the producing rank's own `stage` buffer (at the rows of the block's owner) and
                            the owner fetches them when it reaches its rows -- the reduce-scatter half of the multimem
                            all-reduce of xla/stream_executor/gpu/all_reduce_kernel_lib.cu.h:99-357 done inside the dot's
                            kernel.  Nothing is pushed from the epilogue of a foreign tile and, with `stage_multicast`, each
                            partial crosses NVLink once and is added inside the switch.  1: the warp that computed a tile of
                            own rows fetches that tile's sum; 2: the sums of one round's own rows are fetched in pieces of
                            8 rows x 64 columns by all warps of the rank during the next round (two pieces per tile, loads
                            issued before the tile's epilogue and sent on after it), so the reduction's traffic is spread
                            over the kernel and only the last round's is left for its end */
  void* stage_multicast; /* pull: optional NVSwitch multicast address bound to every rank's stage (same offset): the owner's
                            fetch is one multimem.ld_reduce (f32 accumulation in the switch, one rounding to bf16; the order
                            of the additions is the switch's).  NULL: plain peer loads added in rank order */
} B200SD_PeerReduce;

int b200sd_scaled_dot_f8_peer_reduce(const B200SD_ScaledDotF8* args, const B200SD_PeerReduce* peers, void* cuda_stream,
                                     char* err, size_t err_len);

/* Number of u32 flag words each rank must provide for the call above (0 if the shape is not supported). */
size_t b200sd_peer_reduce_flag_words(int64_t m, int64_t n, int32_t world);

/* Decode-shaped scaled dot that allocates nothing and needs no workspace from the caller.
 * (No counterpart in the reference, whose cuBLASLt call always receives a workspace buffer.)
 *
 * For callers that cannot hand over scratch memory and are not allowed to create any: an XLA
 * executable runs on a memory plan that was fixed when it was compiled, the runtime's allocator
 * has usually taken nearly all of the GPU's memory already, and a handler that declares itself
 * safe to record into a command buffer must not allocate while it runs -- so if the custom call
 * was emitted without its trailing workspace result, the regular split-K kernel has nowhere to
 * put its partial sums.  This variant keeps that scratch in a fixed array inside the library
 * image: b200sd_noalloc_scratch_bytes() bytes (about 10 MiB) stay resident on every GPU that
 * loads the library until the process exits.
 *
 * Same arguments as b200sd_scaled_dot_f8, of which it computes the plain case only: e4m3 A[m,k]
 * and B[k,n] (row-major, contracting dims 1 and 0), per-tensor a_scale / b_scale, bf16 / f16 /
 * f32 output, no c, bias, activation, amax or d_scale; `workspace` is not used and `kernel` has
 * no effect.
 * Limit: m <= 128; anything larger is refused with INVALID_ARGUMENT and a message naming the
 * limit.  It calls no cudaMalloc / cudaFree nor any allocating library routine.
 * The first call on a device looks up the array's device address (and does the one-time
 * per-device set-up of b200sd_init_device); make that first call before capturing the stream.
 * All calls on a device share the one array, which still holds the previous call's contents --
 * the part that must start at zero is cleared on the stream at the start of every call -- so two
 * calls that overlap on the same GPU (different streams) race; serialise them. */
int b200sd_scaled_dot_f8_decode_noalloc(const B200SD_ScaledDotF8* args, void* cuda_stream, char* err,
                                        size_t err_len);
size_t b200sd_noalloc_scratch_bytes(void);

/* Rewriter-lite: applies GemmRewriter's decisions for this path
 * (xla/backends/gpu/transforms/gemm_rewriter.cc:190-336 MatchFp8Param, :1235-1591 CreateF8CustomCall,
 * :1829-2249 bias / ReLU / GELU fusion, :1635-1794 FP8 output cast and amax, :2774-2892 workspace) to an
 * HLO module given as text, over the subset of HLO the fixtures under tests/golden/hlo use, and emits
 * the custom calls "b200$scaled_dot$f8" / "b200$dot$s8" where the reference would emit
 * "__cublas$lt$matmul$f8" / "__cublas$lt$matmul".  `out_hlo` receives the rewritten module text,
 * `plan_json` a description of the custom call (operand sources in terms of the module's parameters,
 * results, attributes).  Returns 0 when the text was understood (plan_json says whether anything was
 * rewritten and, if not, why), 3 for unparsable text, 8 when a buffer is too small. */
int b200sd_rewrite_hlo(const char* hlo_text, char* out_hlo, size_t out_hlo_len, char* plan_json,
                       size_t plan_json_len, char* err, size_t err_len);

/* ---- XLA FFI handlers (typed FFI, api_version = API_VERSION_TYPED_FFI) -----------------------
 * Signature: XLA_FFI_Error* (*)(XLA_FFI_CallFrame*), xla/ffi/api/c_api.h:517.  Declared with
 * void* here so that this header does not depend on XLA's.  Register them under the custom-call
 * targets "b200$scaled_dot$f8", "b200$dot$s8" and "b200$block_scaled_dot$mx" (platform "CUDA"); the first two accept the operand and
 * result arrangements of `__cublas$lt$matmul$f8` (xla/service/gpu/thunk_emitter.cc:776-862).
 * The *_instantiate / *_initialize symbols are the optional stages of the handler bundle
 * (c_api.h:520-526). */
#ifndef B200SD_NO_FFI_DECLS
void* b200sd_ffi_scaled_dot_f8(void* call_frame);
void* b200sd_ffi_scaled_dot_f8_instantiate(void* call_frame);
void* b200sd_ffi_scaled_dot_f8_initialize(void* call_frame);
void* b200sd_ffi_dot_s8(void* call_frame);
void* b200sd_ffi_dot_s8_instantiate(void* call_frame);
void* b200sd_ffi_dot_s8_initialize(void* call_frame);
/* Target "b200$block_scaled_dot$mx": operands (a, b, a_scale, b_scale), results (D, [workspace]) -- the
 * arrangement of `__cublas$lt$matmul$mx` (xla/service/gpu/thunk_emitter.cc:939-988). */
void* b200sd_ffi_block_scaled_dot_mx(void* call_frame);
void* b200sd_ffi_block_scaled_dot_mx_instantiate(void* call_frame);
void* b200sd_ffi_block_scaled_dot_mx_initialize(void* call_frame);
#endif

/* Registers the three bundles with the given `const XLA_FFI_Api*` (what XLA_FFI_REGISTER_HANDLER does,
 * xla/ffi/api/api.h:2881-2893).  Returns 0 or an error code. */
int b200sd_ffi_register(const void* xla_ffi_api, char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
#endif /* B200_SCALED_DOT_H_ */
