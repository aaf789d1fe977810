// Dense quantized GEMM for sm_100a: the kernel behind XLA's `__cublas$lt$matmul$f8` pattern
// (FP8 e4m3fn / e5m2 operands, f32 accumulate) and the s8 x s8 -> s32 dot, with the whole epilogue
// fused.  Replaces the library call at xla/stream_executor/cuda/cuda_blas_lt.cc:559-564.
//
// Two instantiations of one persistent, warp-specialised kernel (320 threads per CTA):
//   pair   clusters of two CTAs work on 256 x 256 tiles with tcgen05.mma cta_group::2: each CTA
//          streams its own 128 rows of A and its own 128 columns of B (32 KiB per 128-deep
//          k-block, six stages), the leader CTA issues M=256, N=256, K=32 MMAs that read both
//          CTAs' shared memory, and each CTA ends up with its 128 x 256 slice of the accumulator
//          in its own TMEM.  Halving the B traffic per SM is what lets the shared-memory fill
//          rate keep up with the tensor pipe.
//   single one CTA per 128 x 256 tile (48 KiB per k-block, four stages); used when M <= 128.
// Roles: warp 0 = TMA producer, warp 1 = TMEM allocator + MMA issuer, warps 2-9 = epilogue
// (tcgen05.ld, scale / beta*C / bias / ReLU or GELU / amax / d_scale / cast, vector stores).
// TMEM holds two 256-column accumulators so the epilogue of one tile overlaps the main loop of the
// next.  Every wait is bounded; on expiry the kernel records a status bit and drains.
// A third instantiation (pair, reduce) forms the sum of a contracting-dimension split over the GPUs of one box
// inside the kernel, over peer memory: partials pushed to the rows' owner, or parked locally and fetched by the
// owner -- with multimem.ld_reduce the NVSwitch adds them up -- by two extra reducer warps (384 threads).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <atomic>
#include <random>
#include <cstdlib>
#include <string>

#include "kernels.h"
#include "ptx.cuh"

namespace b200sd {
namespace {

constexpr int kBM = 128;          // rows of D per CTA per tile (= TMEM lanes)
constexpr int kBN = 256;          // columns of D per tile (= TMEM columns per accumulator)
constexpr int kBK = 128;          // bytes (= 8-bit elements) of K per stage: one 128B swizzle row
constexpr int kUmmaK = 32;        // K per tcgen05.mma for 8-bit operands
constexpr int kAccBufs = 2;
constexpr int kAStageBytes = kBM * kBK;          // 16 KiB
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kReducerWarps = 2;                     // peer-reduce instantiation only: warps that fetch and forward the sums of own rows
constexpr int kReduceThreads = kThreads + 32 * kReducerWarps;
constexpr int kColsPerEpilogueWarp = kBN / 2;    // warps 2-5 take columns 0-127, warps 6-9 columns 128-255
constexpr int kTmemCols = 512;

template <bool kPair>
struct Shape {
  static constexpr int kStages = kPair ? 6 : 4;
  static constexpr int kBStageBytes = (kPair ? kBN / 2 : kBN) * kBK;   // 16 or 32 KiB
  static constexpr int kStageBytes = kAStageBytes + kBStageBytes;
  static constexpr int kTileRows = kPair ? 2 * kBM : kBM;
};

template <bool kPair>
struct __align__(16) DenseAux {
  uint64_t full_bar[Shape<kPair>::kStages];
  uint64_t empty_bar[Shape<kPair>::kStages];
  uint64_t acc_full_bar[kAccBufs];
  uint64_t acc_empty_bar[kAccBufs];
  uint64_t pad_;
  uint32_t tmem_base;
  int abort_flag;
};

// Per-column vectors staged per epilogue warp (private copies: no CTA-level barrier).  Not present
// in the peer-reduce instantiation, which has no bias and spends the space on its store stages.
struct __align__(16) EpilogueVectors {
  float bias_s[kEpilogueWarps][kColsPerEpilogueWarp];
  float colscale_s[kEpilogueWarps][kColsPerEpilogueWarp];
};

// Peer-reduce mode stages 32 rows x 64 bf16 columns per epilogue warp in shared memory, in the
// 128-byte-swizzled layout a TMA store reads, so that what crosses NVLink are bulk stores of
// full lines issued by one lane instead of 16-byte stores from every lane.
constexpr int kStoreStageBytes = 32 * 128;

// Every other instantiation stages 32 rows x 64 bytes of converted output per epilogue warp, so that what
// goes to global memory are 64-byte row segments from four neighbouring lanes instead of one 16-byte
// piece per lane and row (a warp-wide store then touches 8 lines instead of 32).
constexpr int kOutStageRowBytes = 64;
constexpr int kOutStageBytes = 32 * kOutStageRowBytes;

// Layout: [pipeline stages][peer-reduce: eight 4 KiB store stages][aux][others: epilogue vectors, eight 2 KiB output stages].
template <bool kPair, bool kReduce = false>
constexpr size_t DenseSmemBytes() {
  return 1024 /*alignment slack*/ + size_t(Shape<kPair>::kStages) * Shape<kPair>::kStageBytes + sizeof(DenseAux<kPair>) +
         (kReduce ? size_t(kEpilogueWarps) * kStoreStageBytes : sizeof(EpilogueVectors) + size_t(kEpilogueWarps) * kOutStageBytes);
}
static_assert(DenseSmemBytes<true, true>() <= 232448 && DenseSmemBytes<true, false>() <= 232448, "shared memory budget");

// Peer-reduce mode (see PeerReduceProblem): what the kernel needs of it.
struct ReduceArgs {
  int32_t world, rank, emulate;
  int32_t m_tiles_per_block;      // 256-row tiles each rank owns in all (its rows of the staging buffers)
  int32_t stages;                 // the rows are dealt out in `stages` rounds of world sub-blocks (see tile_coords_reduce)
  int32_t col_rounds;             // ... each of which is further cut into this many groups of column tiles (a divisor of num_n_tiles)
  int32_t debug;                  // tuning build only: 1 = reducers skip the fetches, 2 = skip the stores too (results are then wrong)
  uint32_t flag_target;           // value a (tile, warp) flag reaches when every other rank has pushed: epoch * (world - 1)
  uint32_t done_target;           // value the end-of-call counter reaches when every rank is through: epoch * world
  uint32_t done_local_target;     // value this rank's own CTA counter (the word behind it) reaches with its last CTA: epoch * CTAs
  int32_t done_index;             // index of that counter in the flag array
  uint64_t peer_wait_ns;          // limit of a wait for another rank
  uint16_t* d[kMaxPeers];
  uint16_t* d_multicast;          // optional: NVSwitch multicast address covering every rank's D
  int32_t pull;                   // partials stay in the producing rank's staging buffer; the owner of the rows fetches them
  uint16_t* stage_multicast;      // pull: optional multicast address covering every rank's staging buffer (in-switch sum)
  uint16_t* stage[kMaxPeers];
  uint32_t* flags[kMaxPeers];
  const CUtensorMap* emu_maps;    // emulate: A and B maps of rank r at [2r], [2r+1]
};

// Peer-reduce mode: byte-matrix maps ([m, 2n] bytes, 128 B x 32 row boxes, 128-byte swizzle) of
// every rank's staging buffer and output, for the epilogue's bulk stores.
struct ReduceMaps {
  CUtensorMap stage[kMaxPeers];
  CUtensorMap d[kMaxPeers];
};

struct DenseArgs {
  int64_t m, n, k;
  int32_t batch;                 // leading batch dimension of A, B, C and D (1 = plain matrices)
  int32_t num_m_tiles, num_n_tiles, num_k_blocks, raster_group;
  int32_t a_mn_major, b_mn_major;
  uint32_t idesc;
  const float* a_scale;
  const float* b_scale;
  const float* d_scale;
  float alpha, beta;
  const void* c;
  int32_t c_dtype;
  const void* bias;
  int32_t bias_dtype;
  int32_t activation;
  float* amax;
  const float* a_row_scale;
  const float* b_col_scale;
  int32_t* d_s32;
  void* d;
  int32_t d_dtype;
  int32_t vec_store_ok;  // D rows start 16-byte aligned and N is a multiple of the vector width
  uint32_t* status;      // device status word (error bits)
  uint32_t* progress;    // optional per-row-block completion counters, else nullptr
  int32_t progress_tiles;   // row-tiles per progress counter
  unsigned long long* timing;   // optional per-CTA wait-time counters (tuning aid), else nullptr
  ReduceArgs red;               // read by the peer-reduce instantiation only
  // Stream-K tail (pair kernel): the tiles past the last full wave are cut along K into equal
  // shares, one per cluster.  dp_tiles tiles are worked one per cluster per round; sk_tiles follow.
  int32_t dp_tiles, sk_tiles;
  unsigned long long sk_epoch;          // value that marks a partial of THIS launch as written
  unsigned long long* sk_flags;         // [clusters][2 CTAs][8 warps]
  uint4* sk_partials;                   // [clusters] raw accumulator tiles, 256 KiB each
  // amax without a memset in front of the launch: two words in the caller's workspace.  The first warp
  // of THIS launch to finish (it swaps the launch's epoch into word 0 and finds another value there)
  // stores 0 to amax and then publishes the epoch in word 1; every other warp waits for word 1.
  unsigned long long* amax_sync;        // nullptr: the host cleared amax with a memset node
  unsigned long long amax_epoch;
};

constexpr size_t kSkFlagBytes = 16384;                                 // up to 128 clusters x 16 flags x 8 B
constexpr size_t kSkPartialBytes = size_t(2 * kBM) * kBN * 4;          // one 256 x 256 accumulator tile


// Tuning aid: per CTA, [0] cycles the MMA issuer waited for operands, [1] cycles it waited for a
// free accumulator, [2] its total cycles, [3] cycles the producer waited for a free stage,
// [4] the issuer's wall time in ns, [5]/[6] cycles epilogue warp 2 waited for / worked on accumulators,
// [7] cycles the issuer waited for the stream-K preload; then absolute %globaltimer values (ns):
// [8] CTA entry, [9] set-up done (after the cluster barrier), [10] first operands landed, [11] issuer done,
// [12] epilogue warp 2 done, [13] CTA exit, [14] last accumulator complete (seen by epilogue warp 2), [15] that warp's
// last tile stored (before the amax hand-shake), [16] cycles epilogue warp 2 spent waiting for its TMEM loads, [17] in the
// arithmetic and conversion of chunks, [18] in the flushes of its output stage.
constexpr int kTimingSlots = 24;
// Tuning builds only; filled when B200SD_TIMING=1 was set at load time.
#if B200SD_TUNING
__device__ unsigned long long g_dense_timing[kTimingSlots * 512];
#endif

__device__ __forceinline__ float load_as_f32(const void* base, int32_t dtype, int64_t idx) {
  switch (dtype) {
    case kF32: return static_cast<const float*>(base)[idx];
    case kBF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
    case kF16: return __half2float(static_cast<const __half*>(base)[idx]);
    default: return 0.0f;
  }
}

// tanh-form GELU as matched by the rewriter (xla/backends/gpu/transforms/gemm_rewriter.cc:924-971):
// 0.5 x (1 + tanh(u)), u = sqrt(2/pi) (x + 0.044715 x^3).  Evaluated through the identity
// 0.5 (1 + tanh(u)) = 1 / (1 + exp(-2u)) with the hardware exponential and reciprocal
// (relative error about 2^-21, far inside bf16 / e4m3 output resolution); the limits
// exp -> inf and exp -> 0 give exactly 0 and x.
__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.797884583f * (x + 0.044715f * (x * x * x));
  return __fdividef(x, 1.0f + __expf(-2.0f * u));
}

__device__ __forceinline__ void tile_coords(int32_t tile, const DenseArgs& p, int32_t* mt, int32_t* nt, int32_t* batch) {
  // Batches one after the other; inside a batch, groups of `raster_group` row-tiles are swept
  // column by column so that the CTAs running at the same time share A row-panels and B
  // column-panels in L2.
  const int32_t per_batch = p.num_m_tiles * p.num_n_tiles;
  *batch = tile / per_batch;
  tile -= *batch * per_batch;
  const int32_t per_group = p.raster_group * p.num_n_tiles;
  const int32_t g = tile / per_group;
  const int32_t first_m = g * p.raster_group;
  const int32_t gsize = min(p.raster_group, p.num_m_tiles - first_m);
  const int32_t r = tile - g * per_group;
  *mt = first_m + r % gsize;
  *nt = r / gsize;
}

// What one cluster does, in order: its share of the stream-K tail that does NOT finish a tile
// (accumulator dumped to the workspace), then the share that finishes a tile (the earlier shares of
// that tile, dumped by lower-numbered clusters as the first thing they did, are added in its
// epilogue), then its whole tiles.  Finishers therefore never wait for work that has not started,
// and both short epilogues run under the main loop of a following item: the one epilogue left
// exposed at the end of the kernel is that of an ordinary tile.
struct WorkItem {
  int32_t tile, kb0, kb1;
  int32_t mode;            // 0 whole tile, 1 dump a partial, 2 finish a tile others contributed to
};
struct WorkList {
  int32_t n_items, dp_count, first_tile, tile_step;
  int32_t nf_tile, nf_kb0, nf_kb1;     // share that does not finish its tile (nf_tile < 0: none)
  int32_t fin_tile, fin_kb0;           // share that finishes its tile (fin_tile < 0: none)
};

__device__ __forceinline__ int64_t sk_bound(const DenseArgs& p, int32_t cluster, int32_t clusters) {
  return int64_t(cluster) * (int64_t(p.sk_tiles) * p.num_k_blocks) / clusters;
}

__device__ __forceinline__ WorkList make_work_list(const DenseArgs& p, int32_t cluster, int32_t clusters, int32_t first_tile,
                                                   int32_t tile_step) {
  WorkList w;
  w.first_tile = first_tile;
  w.tile_step = tile_step;
  w.dp_count = first_tile < p.dp_tiles ? (p.dp_tiles - first_tile + tile_step - 1) / tile_step : 0;
  w.nf_tile = -1;
  w.fin_tile = -1;
  w.nf_kb0 = w.nf_kb1 = w.fin_kb0 = 0;
  if (p.sk_tiles > 0) {
    const int64_t u0 = sk_bound(p, cluster, clusters), u1 = sk_bound(p, cluster + 1, clusters);
    if (u1 > u0) {
      const int32_t kb = p.num_k_blocks;
      const int32_t t_lo = int32_t(u0 / kb), t_hi = int32_t((u1 - 1) / kb);
      if (t_lo == t_hi) {
        const int32_t k0 = int32_t(u0 - int64_t(t_lo) * kb), k1 = int32_t(u1 - int64_t(t_lo) * kb);
        if (k1 == kb) {
          w.fin_tile = p.dp_tiles + t_lo;
          w.fin_kb0 = k0;
        } else {
          w.nf_tile = p.dp_tiles + t_lo;
          w.nf_kb0 = k0;
          w.nf_kb1 = k1;
        }
      } else {
        w.fin_tile = p.dp_tiles + t_lo;
        w.fin_kb0 = int32_t(u0 - int64_t(t_lo) * kb);
        w.nf_tile = p.dp_tiles + t_hi;
        w.nf_kb0 = 0;
        w.nf_kb1 = int32_t(u1 - int64_t(t_hi) * kb);
      }
    }
  }
  w.n_items = w.dp_count + (w.nf_tile >= 0 ? 1 : 0) + (w.fin_tile >= 0 ? 1 : 0);
  return w;
}

__device__ __forceinline__ WorkItem get_item(const WorkList& w, const DenseArgs& p, int32_t it) {
  WorkItem x;
  if (w.nf_tile >= 0) {
    if (it == 0) {
      x.tile = w.nf_tile; x.kb0 = w.nf_kb0; x.kb1 = w.nf_kb1; x.mode = 1;
      return x;
    }
    --it;
  }
  if (w.fin_tile >= 0) {
    if (it == 0) {
      x.tile = w.fin_tile; x.kb0 = w.fin_kb0; x.kb1 = p.num_k_blocks; x.mode = w.fin_kb0 > 0 ? 2 : 0;
      return x;
    }
    --it;
  }
  x.tile = w.first_tile + it * w.tile_step; x.kb0 = 0; x.kb1 = p.num_k_blocks; x.mode = 0;
  return x;
}

__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Peer-reduce order.  The rows are cut into stages x world sub-blocks; sub-block s*world + j belongs to
// rank j (and, with col_rounds > 1, each sub-block's column tiles into that many groups, one round each).  In every stage rank r walks the sub-blocks of ranks r+1, r+2, ..., r (its own last): what it
// pushes first is what its neighbours need last, and when it reaches its own sub-block the others'
// partials of it have arrived.  Several stages spread the broadcasts of finished rows over the
// kernel instead of leaving them all for its end.  `blk` is the owner of the tile's rows, `own_mt`
// the tile's row-tile index within the owner's rows (staging buffer, flags), `slot` names its flags.
__device__ __forceinline__ void tile_coords_reduce(int32_t tile, const DenseArgs& p, int32_t my_rank, int32_t* mt,
                                                   int32_t* nt, int32_t* blk, int32_t* slot, int32_t* own_mt) {
  const int32_t mtps = p.red.m_tiles_per_block / p.red.stages;       // row tiles per sub-block
  const int32_t ntps = p.num_n_tiles / p.red.col_rounds;             // column tiles per sub-block
  const int32_t per_sub = mtps * ntps;
  const int32_t per_round = per_sub * p.red.world;
  const int32_t round = tile / per_round;                            // row round major, column round minor
  const int32_t rs = round / p.red.col_rounds, cs = round - rs * p.red.col_rounds;
  const int32_t within = tile - round * per_round;
  const int32_t b = within / per_sub;
  const int32_t local = within - b * per_sub;
  int32_t owner = my_rank + 1 + b;
  if (owner >= p.red.world) owner -= p.red.world;
  const int32_t rg = min(p.raster_group, mtps);
  const int32_t per_group = rg * ntps;
  const int32_t g = local / per_group;
  const int32_t first_m = g * rg;
  const int32_t gsize = min(rg, mtps - first_m);
  const int32_t r = local - g * per_group;
  const int32_t mt_local = first_m + r % gsize;
  *nt = cs * ntps + r / gsize;
  *mt = (rs * p.red.world + owner) * mtps + mt_local;
  *blk = owner;
  *own_mt = rs * mtps + mt_local;
  *slot = *own_mt * p.num_n_tiles + *nt;
}

constexpr int kChunk = 16;   // accumulator columns handled per epilogue step

// Peer-reduce epilogue for kChunk columns of one row.  The partial is rounded to bf16 (the dot's
// result type).  For a row this rank owns, the bf16 partials of all ranks are added in rank order
// in f32 and rounded once.  Either way the 16 values go into the warp's store stage (row = lane,
// 16-byte units XOR-swizzled by the row to spread the banks); flush_store_stage writes them out.
__device__ __forceinline__ void reduce_chunk(const DenseArgs& p, const uint32_t (&r)[kChunk], float scale, int32_t my_rank,
                                             int32_t blk, int64_t row_in_block, int64_t rows_per_block, int64_t col0,
                                             uint4* stage_row, int unit0, int lane) {
  uint32_t w[kChunk / 2];
#pragma unroll
  for (int i = 0; i < kChunk / 2; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * i]) * scale, __uint_as_float(r[2 * i + 1]) * scale);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  if (blk == my_rank && p.red.world > 1 && !p.red.pull) {
    // The other ranks' partials are requested four ranks at a time before any is used: one memory
    // latency per group instead of one per rank.
    float acc[kChunk];
#pragma unroll
    for (int i = 0; i < kChunk; ++i) acc[i] = 0.0f;
    const uint16_t* const mine = p.red.stage[my_rank] + row_in_block * p.n + col0;
    const int64_t slot_stride = rows_per_block * p.n;
#pragma unroll 1
    for (int32_t s0 = 0; s0 < p.red.world; s0 += 4) {
      uint4 lo[4], hi[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int32_t s = s0 + j;
        if (s < p.red.world && s != my_rank) {
          const uint4* src = reinterpret_cast<const uint4*>(mine + s * slot_stride);
          lo[j] = __ldcg(src);           // written by another GPU: never through L1
          hi[j] = __ldcg(src + 1);
        } else {                         // this rank's own partial takes its place in the rank order
          lo[j] = make_uint4(w[0], w[1], w[2], w[3]);
          hi[j] = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (s0 + j < p.red.world) {
          const uint32_t x[kChunk / 2] = {lo[j].x, lo[j].y, lo[j].z, lo[j].w, hi[j].x, hi[j].y, hi[j].z, hi[j].w};
#pragma unroll
          for (int i = 0; i < kChunk / 2; ++i) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x[i]));
            acc[2 * i] += f.x;
            acc[2 * i + 1] += f.y;
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kChunk / 2; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  stage_row[(unit0) ^ (lane & 7)] = make_uint4(w[0], w[1], w[2], w[3]);
  stage_row[(unit0 + 1) ^ (lane & 7)] = make_uint4(w[4], w[5], w[6], w[7]);
}

// Sends the warp's 32 x 64 staged values on their way.  Rows another rank owns go to that rank's
// staging buffer, own rows to every rank's D: one bulk tensor store per destination, issued by
// lane 0 (or, with an NVSwitch multicast mapping of D, multimem stores from every lane).
// `byte_col` / `row` are the coordinates of the stage's first element in the destination matrix.
__device__ __forceinline__ void flush_store_stage(const DenseArgs& p, const ReduceMaps& maps, const uint4* stage,
                                                  int32_t my_rank, int32_t blk, int64_t row0, int64_t row0_in_block,
                                                  int64_t rows_per_block, int64_t col0, int lane, bool partial_to_own_stage = false) {
  if (partial_to_own_stage) {
    // Pull mode: every partial, of foreign rows and of own rows alike, goes to THIS rank's staging buffer, at the
    // rows of the block's owner; the owner fetches it from there.
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (col0 < p.n) tma_store_2d(&maps.stage[my_rank], stage, int32_t(col0 * 2), int32_t(int64_t(blk) * rows_per_block + row0_in_block));
      tma_store_commit();
    }
    return;
  }
  if (blk == my_rank && p.red.d_multicast != nullptr) {
    __syncwarp();
    const int unit = lane & 7;
    const int64_t col = col0 + unit * 8;
    if (col < p.n) {
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int rrow = it * 4 + (lane >> 3);
        multimem_st_v4(p.red.d_multicast + (row0 + rrow) * p.n + col, stage[rrow * 8 + (unit ^ (rrow & 7))]);
      }
    }
    __syncwarp();
    return;
  }
  fence_proxy_async_smem();        // this lane's writes to the stage become visible to the bulk-copy engine
  __syncwarp();
  if (lane == 0) {
    if (col0 < p.n) {
      if (blk != my_rank) {
        tma_store_2d(&maps.stage[blk], stage, int32_t(col0 * 2), int32_t(int64_t(my_rank) * rows_per_block + row0_in_block));
      } else {
        for (int32_t j = 0; j < p.red.world; ++j) tma_store_2d(&maps.d[j], stage, int32_t(col0 * 2), int32_t(row0));
      }
    }
    tma_store_commit();          // also when empty: every tile adds exactly two groups
  }
}

// Converts and stores kChunk consecutive columns of one row straight from the lane's registers.  The path
// for outputs whose rows are not 16-byte aligned; kept out of line so that it does not widen the epilogue loop.
__device__ __noinline__ void store_row_chunk(void* d, int32_t d_dtype, bool vec_ok, const float (&v)[kChunk], int64_t off,
                                             int32_t ncols) {
  const bool vec = ncols == kChunk && vec_ok;
  if (d_dtype == kF8E4M3FN || d_dtype == kF8E5M2) {
    const __nv_fp8_interpretation_t fmt = d_dtype == kF8E4M3FN ? __NV_E4M3 : __NV_E5M2;
    uint8_t* out = static_cast<uint8_t*>(d) + off;
    uint32_t w[kChunk / 4];
#pragma unroll
    for (int i = 0; i < kChunk / 4; ++i) {
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i], v[4 * i + 1]), __NV_SATFINITE, fmt);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i + 2], v[4 * i + 3]), __NV_SATFINITE, fmt);
      w[i] = lo | (hi << 16);
    }
    if (vec) {
      *reinterpret_cast<uint4*>(out) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
#pragma unroll
      for (int i = 0; i < kChunk; ++i)
        if (i < ncols) out[i] = static_cast<uint8_t>(w[i >> 2] >> (8 * (i & 3)));
    }
  } else if (d_dtype == kBF16 || d_dtype == kF16) {
    uint16_t* out = static_cast<uint16_t*>(d) + off;
    uint32_t w[kChunk / 2];
    if (d_dtype == kBF16) {
#pragma unroll
      for (int i = 0; i < kChunk / 2; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    } else {
#pragma unroll
      for (int i = 0; i < kChunk / 2; ++i) {
        const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    if (vec) {
      reinterpret_cast<uint4*>(out)[0] = make_uint4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<uint4*>(out)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
#pragma unroll
      for (int i = 0; i < kChunk; ++i)
        if (i < ncols) out[i] = static_cast<uint16_t>(w[i >> 1] >> (16 * (i & 1)));
    }
  } else {  // kF32
    float* out = static_cast<float*>(d) + off;
    if (vec) {
#pragma unroll
      for (int i = 0; i < kChunk / 4; ++i)
        reinterpret_cast<float4*>(out)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < kChunk; ++i)
        if (i < ncols) out[i] = v[i];
    }
  }
}

// v += beta * C for kChunk columns of one row.  Out of line: a matrix bias is the rare case and its three
// element types would otherwise triple this code inside the epilogue loop.
__device__ __noinline__ void add_matrix_bias(const void* c, int32_t c_dtype, float beta, int64_t off, int32_t ncols, float (&v)[kChunk]) {
#pragma unroll
  for (int i = 0; i < kChunk; ++i)
    if (i < ncols) v[i] += beta * load_as_f32(c, c_dtype, off + i);
}

// The warp's output stage: 32 rows (one per lane) x four 16-byte pieces, the piece index XOR-swizzled
// by the row pair so that neither the row-per-lane writes nor the piece-per-lane reads collide on banks.
__device__ __forceinline__ void stage_put(uint4* stage, int lane, int piece, uint4 v) {
  stage[lane * 4 + (piece ^ ((lane >> 1) & 3))] = v;
}

// Converts kChunk values of this lane's row to the output type and puts them into the stage at
// piece `piece0` (1, 2 or 4 pieces for 1-, 2- and 4-byte output elements).
__device__ __forceinline__ void stage_row_chunk(const DenseArgs& p, const float (&v)[kChunk], uint4* stage, int lane, int piece0) {
  if (p.d_dtype == kF8E4M3FN || p.d_dtype == kF8E5M2) {
    const __nv_fp8_interpretation_t fmt = p.d_dtype == kF8E4M3FN ? __NV_E4M3 : __NV_E5M2;
    uint32_t w[kChunk / 4];
#pragma unroll
    for (int i = 0; i < kChunk / 4; ++i) {
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i], v[4 * i + 1]), __NV_SATFINITE, fmt);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i + 2], v[4 * i + 3]), __NV_SATFINITE, fmt);
      w[i] = lo | (hi << 16);
    }
    stage_put(stage, lane, piece0, make_uint4(w[0], w[1], w[2], w[3]));
  } else if (p.d_dtype == kBF16 || p.d_dtype == kF16) {
    uint32_t w[kChunk / 2];
    if (p.d_dtype == kBF16) {
#pragma unroll
      for (int i = 0; i < kChunk / 2; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    } else {
#pragma unroll
      for (int i = 0; i < kChunk / 2; ++i) {
        const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    stage_put(stage, lane, piece0, make_uint4(w[0], w[1], w[2], w[3]));
    stage_put(stage, lane, piece0 + 1, make_uint4(w[4], w[5], w[6], w[7]));
  } else {  // kF32
#pragma unroll
    for (int i = 0; i < kChunk / 4; ++i)
      stage_put(stage, lane, piece0 + i, make_uint4(__float_as_uint(v[4 * i]), __float_as_uint(v[4 * i + 1]),
                                                      __float_as_uint(v[4 * i + 2]), __float_as_uint(v[4 * i + 3])));
  }
}

// Writes the warp's staged 32 x 64-byte block out: four store instructions, each covering 8 rows x 64
// contiguous bytes.  `row0` is the warp's first row in the [batch * m, n] view of D, `rows_valid` how many
// of its rows exist, `byte_col0` the block's first byte within a row, `row_bytes` the row pitch.
__device__ __forceinline__ void stage_flush(const DenseArgs& p, const uint4* stage, int lane, int64_t row0, int32_t rows_valid,
                                            int64_t byte_col0, int64_t row_bytes) {
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int q = i * 32 + lane;
    const int r = q >> 2, piece = q & 3;
    const uint4 v = stage[r * 4 + (piece ^ ((r >> 1) & 3))];
    const int64_t bc = byte_col0 + piece * 16;
    if (r < rows_valid && bc < row_bytes) *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.d) + (row0 + r) * row_bytes + bc) = v;
  }
  __syncwarp();
}

// Epilogue arithmetic and store for kChunk columns of one accumulator row.  Every option is
// tested once per chunk, outside the per-element loops, which keeps the unrolled code small
// enough to stay resident in the instruction cache while eight warps run it.
// With `stage` the converted values go to the warp's output stage (piece `piece0`) for a coalesced flush by
// the caller; without it they are stored directly (unaligned or ragged outputs).
template <bool kInt8>
__device__ __forceinline__ void finish_chunk(const DenseArgs& p, const uint32_t (&r)[kChunk], int64_t row, int64_t col0,
                                             int32_t ncols, float scale, float d_scale, float row_scale,
                                             const float* bias_c, const float* colscale_c, uint32_t* amax_bits,
                                             uint4* stage, int lane, int piece0) {
  float v[kChunk];
  if (kInt8) {
    if (p.d_s32) {
      int32_t* out = p.d_s32 + row * p.n + col0;
      if (ncols == kChunk && p.vec_store_ok) {
#pragma unroll
        for (int i = 0; i < kChunk / 4; ++i)
          reinterpret_cast<uint4*>(out)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < kChunk; ++i)
          if (i < ncols) out[i] = static_cast<int32_t>(r[i]);
      }
    }
    if (p.d == nullptr) return;
#pragma unroll
    for (int i = 0; i < kChunk; ++i) v[i] = __int2float_rn(static_cast<int32_t>(r[i]));
    if (p.a_row_scale) {
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] = v[i] * row_scale;
    }
    if (p.b_col_scale) {
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] = v[i] * colscale_c[i];
    }
  } else {
#pragma unroll
    for (int i = 0; i < kChunk; ++i) v[i] = __uint_as_float(r[i]) * scale;
    if (p.c != nullptr) {
      // through a copy: an array handed to an out-of-line function lives in local memory, and `v` must not
      float t[kChunk];
#pragma unroll
      for (int i = 0; i < kChunk; ++i) t[i] = v[i];
      add_matrix_bias(p.c, p.c_dtype, p.beta, row * p.n + col0, ncols, t);
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] = t[i];
    }
    if (p.bias) {
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] += bias_c[i];
    }
    if (p.activation == kActRelu) {
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] = (v[i] != v[i]) ? v[i] : fmaxf(v[i], 0.0f);
    } else if (p.activation == kActGelu) {
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] = gelu_tanh(v[i]);
    }
    if (p.amax != nullptr) {
      // Columns past N hold act(0 + 0) = 0 (zero-filled operands, zero-staged bias) and cannot raise the maximum.
      uint32_t m = *amax_bits;
#pragma unroll
      for (int i = 0; i < kChunk; ++i) m = max(m, __float_as_uint(fabsf(v[i])));
      *amax_bits = m;
    }
    if (d_scale != 1.0f) {
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] *= d_scale;
    }
  }
  if (stage != nullptr) {
    stage_row_chunk(p, v, stage, lane, piece0);
  } else {
    float t[kChunk];                 // see add_matrix_bias above
#pragma unroll
    for (int i = 0; i < kChunk; ++i) t[i] = v[i];
    store_row_chunk(p.d, p.d_dtype, p.vec_store_ok != 0, t, row * p.n + col0, ncols);
  }
}

// Peer reduce, pull == 2: fetches the sums of the (tile, warp) parts first, first + step, ... of one round's own rows
// and writes them to every rank's D.  A part is the 32 rows x 128 columns one epilogue warp produces; it is complete
// when every rank -- this one included -- has raised its flag.  Per part: one flag wait, sixteen 16-byte fetches
// per lane (multimem.ld_reduce through the switch when the staging buffers have a multicast mapping, else peer
// loads added in rank order), sixteen stores (multimem.st, else one store per rank).  Returns false when a wait
// gave up.
__device__ __forceinline__ bool reduce_parts(const DenseArgs& p, int32_t my_rank, int32_t round, int32_t first, int32_t step,
                                             int lane, volatile int* abort_flag) {
  constexpr int kTileRows = 2 * kBM;
  const int32_t mtps = p.red.m_tiles_per_block / p.red.stages;
  const int32_t ntps = p.num_n_tiles / p.red.col_rounds;
  const int32_t rs = round / p.red.col_rounds, cs = round - rs * p.red.col_rounds;      // row round, column round
  const int64_t rows_per_block = int64_t(p.red.m_tiles_per_block) * kTileRows;
  const int32_t parts = mtps * ntps * 2 * kEpilogueWarps;
  bool ok = true;
  for (int32_t q = first; q < parts && ok; q += step) {
    const int32_t t = q / (2 * kEpilogueWarps), w16 = q - t * 2 * kEpilogueWarps;
    const int32_t cta = w16 / kEpilogueWarps, ew = w16 - cta * kEpilogueWarps;
    const int32_t mt_local = t / ntps, nt = cs * ntps + (t - mt_local * ntps);
    const int32_t own_mt = rs * mtps + mt_local;
    const int32_t f_index = ((own_mt * p.num_n_tiles + nt) * 2 + cta) * kEpilogueWarps + ew;
    if (lane == 0) ok = counter_wait(p.red.flags[my_rank] + f_index, p.red.flag_target, abort_flag, p.status, kStatusPeerTimeout, p.red.peer_wait_ns);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) break;
    const int32_t row_in_tile = cta * kBM + (((ew & 3) + 2) & 3) * 32;
    const int64_t own_row0 = int64_t(own_mt) * kTileRows + row_in_tile;
    const int64_t d_row0 = (int64_t(rs) * p.red.world + my_rank) * mtps * kTileRows + int64_t(mt_local) * kTileRows + row_in_tile;
    const int64_t col0 = int64_t(nt) * kBN + (ew >> 2) * kColsPerEpilogueWarp + (lane & 7) * 8;
    uint4 v[16];
#pragma unroll
    for (int it = 0; it < 16; ++it) {
      const int rrow = (it & 7) * 4 + (lane >> 3);
      const int64_t col = col0 + (it >> 3) * 64;
      if (col >= p.n) continue;
      const int64_t off = (int64_t(my_rank) * rows_per_block + own_row0 + rrow) * p.n + col;
      if (kTiming && p.red.debug >= 1) {
        v[it] = make_uint4(0u, 0u, 0u, 0u);
      } else if (p.red.stage_multicast != nullptr) {
        v[it] = multimem_ld_reduce_bf16x8(p.red.stage_multicast + off);
      } else {
        float acc8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc8[i] = 0.0f;
        for (int32_t sr = 0; sr < p.red.world; ++sr) {
          const uint4 x = __ldcg(reinterpret_cast<const uint4*>(p.red.stage[sr] + off));
          const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xw[i]));
            acc8[2 * i] += f.x;
            acc8[2 * i + 1] += f.y;
          }
        }
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 hh = __floats2bfloat162_rn(acc8[2 * i], acc8[2 * i + 1]);
          o[i] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        v[it] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
#pragma unroll
    for (int it = 0; it < 16; ++it) {
      const int rrow = (it & 7) * 4 + (lane >> 3);
      const int64_t col = col0 + (it >> 3) * 64;
      if (col >= p.n) continue;
      const int64_t off = (d_row0 + rrow) * p.n + col;
      if (kTiming && p.red.debug >= 2) {
      } else if (p.red.d_multicast != nullptr) {
        multimem_st_v4(p.red.d_multicast + off, v[it]);
      } else {
        for (int32_t j = 0; j < p.red.world; ++j) *reinterpret_cast<uint4*>(p.red.d[j] + off) = v[it];
      }
    }
  }
  return ok;
}

template <bool kInt8, bool kPair, bool kReduce = false>
__global__ void __launch_bounds__(kReduce ? kReduceThreads : kThreads, 1)
dense_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a_param, const __grid_constant__ CUtensorMap tmap_b_param,
                  const DenseArgs p, const __grid_constant__ ReduceMaps rmaps) {
  static_assert(!kReduce || (kPair && !kInt8), "peer-reduce mode exists for the FP8 pair kernel only");
  using S = Shape<kPair>;
  constexpr int kStages = S::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kAStageBytes;
  uint8_t* const after_stages = smem + kStages * S::kStageBytes;                  // 1024-byte aligned
  DenseAux<kPair>* aux = reinterpret_cast<DenseAux<kPair>*>(after_stages + (kReduce ? kEpilogueWarps * kStoreStageBytes : 0));
  volatile int* abort_flag = &aux->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const unsigned long long t_entry = (kTiming && p.timing) ? global_timer_ns() : 0;
  // The kernel behind this one in the stream may be scheduled as this one's CTAs retire (it sets itself up
  // and then waits for this grid to complete before it touches global memory).
  if (threadIdx.x == 0) griddep_launch_dependents();
  const uint32_t rank = kPair ? cluster_cta_rank() : 0u;        // 0 = leader of the pair
  int32_t first_tile = kPair ? int32_t(blockIdx.x >> 1) : int32_t(blockIdx.x);
  int32_t tile_step = kPair ? int32_t(gridDim.x >> 1) : int32_t(gridDim.x);
  // Which rank of a contracting-dimension split this CTA works for, and on whose operands.
  int32_t my_rank = 0;
  const CUtensorMap* tmap_a_ptr = &tmap_a_param;
  const CUtensorMap* tmap_b_ptr = &tmap_b_param;
  if constexpr (kReduce) {
    my_rank = p.red.rank;
    if (p.red.emulate) {
      tile_step /= p.red.world;                   // clusters per emulated rank
      my_rank = first_tile / tile_step;
      first_tile -= my_rank * tile_step;
      tmap_a_ptr = p.red.emu_maps + 2 * my_rank;
      tmap_b_ptr = p.red.emu_maps + 2 * my_rank + 1;
    }
  }
  const CUtensorMap& tmap_a = *tmap_a_ptr;
  const CUtensorMap& tmap_b = *tmap_b_ptr;
  const int32_t cluster_id = kPair ? int32_t(blockIdx.x >> 1) : int32_t(blockIdx.x);
  const WorkList work = make_work_list(p, cluster_id, kPair ? int32_t(gridDim.x >> 1) : int32_t(gridDim.x), first_tile, tile_step);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&aux->full_bar[s], 1);
      mbar_init(&aux->empty_bar[s], 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      mbar_init(&aux->acc_full_bar[b], 1);
      mbar_init(&aux->acc_empty_bar[b], kPair ? 2 * kEpilogueWarps : kEpilogueWarps);
    }
    aux->abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    if (kPair) {
      tmem_alloc_pair(&aux->tmem_base, kTmemCols);
      tmem_relinquish_alloc_pair();
    } else {
      tmem_alloc(&aux->tmem_base, kTmemCols);
      tmem_relinquish_alloc();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (kPair) cluster_sync_all();          // the peer's barriers exist before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = aux->tmem_base;
  // Everything above touched only this CTA's shared memory, TMEM and the kernel parameters.  From here on
  // global memory is read and written: the kernel in front of this one must have completed.
  griddep_wait();
  if (kTiming && p.timing && threadIdx.x == 0) {
    p.timing[blockIdx.x * kTimingSlots + 9] = global_timer_ns();
    p.timing[blockIdx.x * kTimingSlots + 8] = t_entry;
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long prod_wait = 0;
      for (int32_t it = 0; it < work.n_items && ok; ++it) {
        const WorkItem item = get_item(work, p, it);
        const int32_t tile = item.tile;
        int32_t mt, nt, bt = 0;
        if constexpr (kReduce) {
          int32_t blk, slot, own_mt;
          tile_coords_reduce(tile, p, my_rank, &mt, &nt, &blk, &slot, &own_mt);
        } else {
          tile_coords(tile, p, &mt, &nt, &bt);
        }
        const int32_t row0 = mt * S::kTileRows + int32_t(rank) * kBM;
        const int32_t col0 = nt * kBN + (kPair ? int32_t(rank) * (kBN / 2) : 0);
        for (int32_t kb = item.kb0; kb < item.kb1; ++kb) {
          const long long tw = (kTiming && p.timing) ? clock64() : 0;
          ok = mbar_wait(&aux->empty_bar[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout);
          if (kTiming && p.timing) prod_wait += clock64() - tw;
          if (!ok) break;
          uint8_t* sa = smem_a + stage * kAStageBytes;
          uint8_t* sb = smem_b + stage * S::kBStageBytes;
          if (kPair) {
            // Both CTAs' loads count on the leader's barrier; the leader announces the bytes of both.
            if (rank == 0) mbar_arrive_expect_tx(&aux->full_bar[stage], 2 * S::kStageBytes);
            const uint32_t full = map_to_cta(&aux->full_bar[stage], 0);
            if (p.a_mn_major) {
              tma_load_3d_pair(sa, &tmap_a, full, row0, kb * kBK, bt);
            } else {
              tma_load_3d_pair(sa, &tmap_a, full, kb * kBK, row0, bt);
            }
            if (p.b_mn_major) {
              tma_load_3d_pair(sb, &tmap_b, full, col0, kb * kBK, bt);
            } else {
              tma_load_3d_pair(sb, &tmap_b, full, kb * kBK, col0, bt);
            }
          } else {
            uint64_t* full = &aux->full_bar[stage];
            mbar_arrive_expect_tx(full, S::kStageBytes);
            if (p.a_mn_major) {
              tma_load_3d(sa, &tmap_a, full, row0, kb * kBK, bt);
            } else {
              tma_load_3d(sa, &tmap_a, full, kb * kBK, row0, bt);
            }
            if (p.b_mn_major) {
              tma_load_3d(sb, &tmap_b, full, col0, kb * kBK, bt);
              tma_load_3d(sb + S::kBStageBytes / 2, &tmap_b, full, col0 + 128, kb * kBK, bt);
            } else {
              tma_load_3d(sb, &tmap_b, full, kb * kBK, col0, bt);
            }
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (kTiming && p.timing) p.timing[blockIdx.x * kTimingSlots + 3] = prod_wait;
      if (!ok && !kPair) {
        // Abort path: let loads that were already issued land before the CTA's memory is released.
        for (int s = 0; s < kStages; ++s) {
          for (int i = 0; i < 100000 && !mbar_try_wait(&aux->full_bar[s], 0) && !mbar_try_wait(&aux->full_bar[s], 1); ++i) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && elect_one()) {
      const long long t_begin = (kTiming && p.timing) ? clock64() : 0;
      const unsigned long long ns_begin = (kTiming && p.timing) ? global_timer_ns() : 0;
      long long wait_full = 0, wait_acc = 0;
      unsigned long long first_data_ns = 0;
      const uint32_t sbo = 1024, lbo = 16384;
      const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem_a), lbo, sbo);
      const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(smem_b), lbo, sbo);
      // Encoded (>>4) advance of the start address per K=32 step: 32 bytes along a K-major row,
      // 32 rows of 128 bytes for an MN-major operand.
      const uint32_t a_kstep = p.a_mn_major ? (kUmmaK * 128) >> 4 : kUmmaK >> 4;
      const uint32_t b_kstep = p.b_mn_major ? (kUmmaK * 128) >> 4 : kUmmaK >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int32_t it = 0; it < work.n_items && ok; ++it) {
        const WorkItem item = get_item(work, p, it);
        const long long tw0 = (kTiming && p.timing) ? clock64() : 0;
        ok = mbar_wait(&aux->acc_empty_bar[acc], acc_phase ^ 1, abort_flag, p.status, kStatusMmaTimeout);
        if (kTiming && p.timing) wait_acc += clock64() - tw0;
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        constexpr bool preloaded = false;
        for (int32_t kb = item.kb0; kb < item.kb1; ++kb) {
          const long long tw1 = (kTiming && p.timing) ? clock64() : 0;
          ok = mbar_wait(&aux->full_bar[stage], phase, abort_flag, p.status, kStatusMmaTimeout);
          if (kTiming && p.timing) {
            wait_full += clock64() - tw1;
            if (first_data_ns == 0) first_data_ns = global_timer_ns();
          }
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t a_desc = a_desc0 + uint64_t((stage * kAStageBytes) >> 4);
          const uint64_t b_desc = b_desc0 + uint64_t((stage * S::kBStageBytes) >> 4);
#pragma unroll
          for (int j = 0; j < kBK / kUmmaK; ++j) {
            const uint32_t accumulate = (preloaded || kb > item.kb0 || j > 0) ? 1u : 0u;
            const uint64_t ad = a_desc + uint64_t(j * a_kstep), bd = b_desc + uint64_t(j * b_kstep);
            if (kPair) {
              if (kInt8) umma_i8_pair(d_tmem, ad, bd, p.idesc, accumulate);
              else umma_f8_pair(d_tmem, ad, bd, p.idesc, accumulate);
            } else {
              if (kInt8) umma_i8(d_tmem, ad, bd, p.idesc, accumulate);
              else umma_f8(d_tmem, ad, bd, p.idesc, accumulate);
            }
          }
          // The stage may be refilled once these MMAs have read it -- in both CTAs of a pair.
          if (kPair) {
            umma_commit_pair(map_to_cta(&aux->empty_bar[stage], 0));
            umma_commit_pair(map_to_cta(&aux->empty_bar[stage], 1));
          } else {
            umma_commit(&aux->empty_bar[stage]);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (kPair) {                                   // accumulator complete (each CTA has its rows)
          umma_commit_pair(map_to_cta(&aux->acc_full_bar[acc], 0));
          umma_commit_pair(map_to_cta(&aux->acc_full_bar[acc], 1));
        } else {
          umma_commit(&aux->acc_full_bar[acc]);
        }
        if (++acc == kAccBufs) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
      if (kTiming && p.timing) {
        p.timing[blockIdx.x * kTimingSlots + 0] = wait_full;
        p.timing[blockIdx.x * kTimingSlots + 1] = wait_acc;
        p.timing[blockIdx.x * kTimingSlots + 2] = clock64() - t_begin;
        p.timing[blockIdx.x * kTimingSlots + 4] = global_timer_ns() - ns_begin;
        p.timing[blockIdx.x * kTimingSlots + 10] = first_data_ns;
        p.timing[blockIdx.x * kTimingSlots + 11] = global_timer_ns();
      }
    }
  } else if (kReduce && warp >= 2 + kEpilogueWarps) {
    // ------------------------------------------------------------------ reducer warps (peer reduce, pull == 2)
    // They fetch and forward the sums of this rank's own rows (reduce_parts) round by round, as the flags of the
    // parts complete.  Nothing of this touches the accumulators, so the tensor cores never wait for NVLink: the
    // traffic of round r flows while round r + 1 is computed.  The LAST round's parts, which only complete when
    // every rank has finished its last tiles, are shared out among all ten warps of every CTA: the epilogue warps
    // take theirs when their tile loop ends.
    if constexpr (kReduce) {
      if (p.red.pull == 2 && p.red.world > 1) {
        const int32_t n_ctas = tile_step * 2;                                          // CTAs of this rank
        const int32_t cta_of_rank = first_tile * 2 + int32_t(rank);
        const int32_t rw = warp - 2 - kEpilogueWarps;
        bool ok = true;
        const int32_t rounds = p.red.stages * p.red.col_rounds;
        for (int32_t round = 0; round + 1 < rounds && ok; ++round)
          ok = reduce_parts(p, my_rank, round, cta_of_rank * kReducerWarps + rw, n_ctas * kReducerWarps, lane, abort_flag);
        if (ok) ok = reduce_parts(p, my_rank, rounds - 1, cta_of_rank * (kEpilogueWarps + kReducerWarps) + kEpilogueWarps + rw,
                                  n_ctas * (kEpilogueWarps + kReducerWarps), lane, abort_flag);
        __threadfence_system();     // this warp's rows are in every rank's D before the CTA reports (end of the kernel)
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int q = warp & 3;                      // TMEM lane quarter this warp may access
    const int ew = warp - 2;                     // 0..7
    const int col_half = ew >> 2;                // which 128 columns of the tile
    EpilogueVectors* const vecs = reinterpret_cast<EpilogueVectors*>(aux + 1);        // absent in peer-reduce mode
    float* bias_w = kReduce ? nullptr : vecs->bias_s[ew];
    float* colscale_w = kReduce ? nullptr : vecs->colscale_s[ew];
    float scale = p.alpha;
    float d_scale = 1.0f;
    if (!kInt8) {
      if (p.a_scale) scale *= __ldg(p.a_scale);
      if (p.b_scale) scale *= __ldg(p.b_scale);
      if (p.d_scale) d_scale = __ldg(p.d_scale);
    }
    const int64_t rows_per_block = kReduce ? int64_t(p.red.m_tiles_per_block) * S::kTileRows : 0;
    uint32_t* pending_flag = nullptr;     // peer-reduce, lane 0: flag of the pushed tile whose stores are still in flight
    uint4* const store_stage = reinterpret_cast<uint4*>(after_stages + ew * kStoreStageBytes);   // 1024-byte aligned
    uint32_t amax_bits = 0;
    long long ep_wait = 0, ep_busy = 0, ep_ld = 0, ep_math = 0, ep_flush = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    // Peer reduce, pull == 2: the sums of own rows are fetched by the CTA's two reducer warps (below), not here;
    // the epilogue only parks every partial in this rank's staging buffer and raises the flag -- also its own.
    [[maybe_unused]] const bool spread = kReduce && p.red.pull == 2 && p.red.world > 1;

    for (int32_t it = 0; it < work.n_items; ++it) {
      const WorkItem item = get_item(work, p, it);
      const int32_t tile = item.tile;
      int32_t mt, nt, bt = 0;
      int32_t blk = 0, slot = 0, own_mt = 0;
      if constexpr (kReduce) tile_coords_reduce(tile, p, my_rank, &mt, &nt, &blk, &slot, &own_mt);
      else tile_coords(tile, p, &mt, &nt, &bt);
      const int64_t col_base = int64_t(nt) * kBN + col_half * kColsPerEpilogueWarp;
      // Stage the per-column vectors of this warp's columns.
      __syncwarp();
      for (int i = lane; i < kColsPerEpilogueWarp; i += 32) {
        const int64_t col = col_base + i;
        if (p.bias) bias_w[i] = col < p.n ? load_as_f32(p.bias, p.bias_dtype, col) : 0.0f;
        if (kInt8 && p.b_col_scale) colscale_w[i] = col < p.n ? __ldg(p.b_col_scale + col) : 0.0f;
      }
      __syncwarp();

      // Flag of this warp's part of the tile: raised once by the same warp of every other rank.
      uint32_t* const my_flag_base = kReduce ? p.red.flags[my_rank] : nullptr;
      const int32_t flag_index = (slot * 2 + int32_t(rank)) * kEpilogueWarps + ew;
      if constexpr (kReduce) {
        if (blk == my_rank && p.red.world > 1 && !spread) {
          // An own tile: the other ranks pushed their partials long ago.  Confirm that, and pull
          // them towards the L2 while the tensor cores are still busy with this tile.  A flag this
          // warp still owes another rank goes out first: no rank may wait for a peer while it
          // holds back something a peer waits for.
          if (lane == 0 && pending_flag != nullptr) {
            tma_store_wait_all<0>();
            asm volatile("fence.proxy.async.global;" ::: "memory");
            red_relaxed_sys_add_u32(pending_flag, 1u);
            pending_flag = nullptr;
          }
          if (lane == 0) ok = counter_wait(my_flag_base + flag_index, p.red.flag_target, abort_flag, p.status, kStatusPeerTimeout, p.red.peer_wait_ns);
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
          const int64_t prow = int64_t(own_mt) * S::kTileRows + int64_t(rank) * kBM + q * 32 + lane;
          for (int32_t s = 0; s < p.red.world && !p.red.pull; ++s) {
            if (s == my_rank) continue;
            const uint16_t* line = p.red.stage[my_rank] + (int64_t(s) * rows_per_block + prow) * p.n + col_base;
            if (col_base < p.n) asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
            if (col_base + 64 < p.n) asm volatile("prefetch.global.L2 [%0];" ::"l"(line + 64));
          }
        }
      }
      // Lane 0 does the bounded wait; the warp then agrees on the outcome so that the
      // warp-collective TMEM loads below never run with a partial warp.
      const long long te0 = (kTiming && p.timing) ? clock64() : 0;
      if (lane == 0) ok = mbar_wait(&aux->acc_full_bar[acc], acc_phase, abort_flag, p.status, kStatusEpilogueTimeout);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      const long long te1 = (kTiming && p.timing) ? clock64() : 0;
      ep_wait += te1 - te0;
      if (kTiming && p.timing && warp == 2 && lane == 0) p.timing[blockIdx.x * kTimingSlots + 14] = global_timer_ns();   // last accumulator complete
      if (!ok) break;
      (void)mbar_try_wait(&aux->acc_full_bar[acc], acc_phase);   // every lane observes the completed phase
      tc_fence_after_sync();

      // Stream-K: where this warp's part of a dumped accumulator lives (same lane mapping for the
      // writer and the reader, 512 contiguous bytes per store instruction), and who contributed.
      constexpr int kWarpPartU4 = kColsPerEpilogueWarp * 32 / 4;                     // uint4 per warp part
      constexpr size_t kSlotU4 = kSkPartialBytes / sizeof(uint4);
      const int warp_part = int(rank) * kEpilogueWarps + ew;
      auto sk_dump = [&](const uint32_t (&r)[kChunk], int c0) {
        uint4* dst = p.sk_partials + size_t(cluster_id) * kSlotU4 + warp_part * kWarpPartU4 + (c0 / kChunk) * 128 + lane;
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j * 32] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
      };
      // The finishing share: the clusters [first_contrib, cluster_id) dumped the earlier shares of this tile as the
      // first thing they did; their flags are confirmed here and their values added chunk by chunk below.
      int32_t first_contrib = cluster_id;
      if (!kReduce && item.mode == 2) {
        const int32_t clusters = kPair ? int32_t(gridDim.x >> 1) : int32_t(gridDim.x);
        const int64_t tile_start = int64_t(item.tile - p.dp_tiles) * p.num_k_blocks;
        while (first_contrib > 0 && sk_bound(p, first_contrib, clusters) > tile_start) --first_contrib;
        if (lane == 0) {
          for (int32_t c = cluster_id - 1; c >= first_contrib && ok; --c) {
            const unsigned long long* f = p.sk_flags + c * 2 * kEpilogueWarps + warp_part;
            uint64_t t0 = 0;
            uint32_t polls = 0;
            while (ld_acquire_gpu_u64(f) != p.sk_epoch) {
              if ((++polls & 1023u) == 0) {
                const uint64_t now = global_timer_ns();
                if (t0 == 0) t0 = now;
                if (*abort_flag || now - t0 > kWaitLimitNs) {
                  *abort_flag = 1;
                  atomicOr(p.status, kStatusFixupTimeout);
                  ok = false;
                  break;
                }
              }
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        for (int32_t c = cluster_id - 1; c >= first_contrib; --c)    // every lane acquires before it reads the partials
          (void)ld_acquire_gpu_u64(p.sk_flags + c * 2 * kEpilogueWarps + warp_part);
      }
      auto sk_add = [&](uint32_t (&r)[kChunk], int c0) {
        for (int32_t c = first_contrib; c < cluster_id; ++c) {
          const uint4* src = p.sk_partials + size_t(c) * kSlotU4 + warp_part * kWarpPartU4 + (c0 / kChunk) * 128 + lane;
          uint4 v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) v[j] = __ldcg(src + j * 32);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (kInt8) {
              r[4 * j] += v[j].x; r[4 * j + 1] += v[j].y; r[4 * j + 2] += v[j].z; r[4 * j + 3] += v[j].w;
            } else {
              r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + __uint_as_float(v[j].x));
              r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + __uint_as_float(v[j].y));
              r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + __uint_as_float(v[j].z));
              r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + __uint_as_float(v[j].w));
            }
          }
        }
      };

      const int64_t row_in_batch = int64_t(mt) * S::kTileRows + int64_t(rank) * kBM + q * 32 + lane;
      const bool row_ok = row_in_batch < p.m;
      float row_scale = 1.0f;
      if (kInt8 && p.a_row_scale && row_ok) row_scale = __ldg(p.a_row_scale + row_in_batch);
      const int64_t row = int64_t(bt) * p.m + row_in_batch;        // row of the [batch * m, n] view of C and D
      const int64_t own_row = int64_t(own_mt) * S::kTileRows + int64_t(rank) * kBM + q * 32 + lane;   // peer reduce: row within the owner's rows
      const uint32_t taddr =
          tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * kBN + col_half * kColsPerEpilogueWarp);

      // Converted output goes through the warp's 32 x 64-byte stage and leaves in 64-byte row segments (direct
      // 16-byte stores per lane only when D's rows are not 16-byte aligned).  One stage holds `group` chunks.
      const int out_elt = (p.d_dtype == kF8E4M3FN || p.d_dtype == kF8E5M2) ? 1 : (p.d_dtype == kF32 ? 4 : 2);
      uint4* const out_stage = (!kReduce && p.vec_store_ok && p.d != nullptr && item.mode != 1)
                                   ? reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(vecs + 1) + ew * kOutStageBytes) : nullptr;
      const int group = 4 / out_elt;
      const int64_t warp_row0 = row - lane, out_row_bytes = p.n * out_elt;
      const int32_t rows_valid = int32_t(max(int64_t(0), min(int64_t(32), p.m - (row_in_batch - lane))));
      auto flush_group = [&](int ci) {         // after chunk ci: the group it completes, if any, goes out
        if (out_stage == nullptr || ((ci + 1) % group) != 0) return;
        const int64_t gcol0 = col_base + int64_t(ci + 1 - group) * kChunk;
        if (gcol0 < p.n) stage_flush(p, out_stage, lane, warp_row0, rows_valid, gcol0 * out_elt, out_row_bytes);
      };

      // kChunk columns at a time; the load of the next chunk is in flight while this one is processed.  One copy of
      // the loop body (the chunk just loaded is moved into `cur`) keeps the epilogue's code small: eight warps run
      // it and it has to stay in the instruction cache.
      constexpr int kChunks = kColsPerEpilogueWarp / kChunk;
      uint32_t cur[kChunk], nxt[kChunk];
      tmem_ld_32x16(taddr, nxt);
#pragma unroll 1
      for (int ci = 0; ci < kChunks; ++ci) {
        const int c0 = ci * kChunk;
        const long long tl0 = (kTiming && p.timing) ? clock64() : 0;
        tmem_ld_wait_16(nxt);
#pragma unroll
        for (int i = 0; i < kChunk; ++i) cur[i] = nxt[i];
        if (ci + 1 < kChunks) tmem_ld_32x16(taddr + c0 + kChunk, nxt);
        const long long tl1 = (kTiming && p.timing) ? clock64() : 0;
        ep_ld += tl1 - tl0;
        const int64_t col0 = col_base + c0;
        if (!kReduce && item.mode == 2) sk_add(cur, c0);
        if (!kReduce && item.mode == 1) {
          sk_dump(cur, c0);
        } else if (col0 < p.n && row_ok) {
          const int32_t ncols = static_cast<int32_t>(min(int64_t(kChunk), p.n - col0));
          if constexpr (kReduce) {
            if ((ci & 3) == 0) {           // a new 64-column group: the bulk store of the previous one must have read the stage
              if (lane == 0) tma_store_wait_read<0>();
              __syncwarp();
            }
            reduce_chunk(p, cur, scale, my_rank, blk, own_row, rows_per_block, col0, store_stage + lane * 8, (ci * 2) & 7, lane);
          } else {
            finish_chunk<kInt8>(p, cur, row, col0, ncols, scale, d_scale, row_scale, bias_w + c0, colscale_w + c0, &amax_bits,
                                out_stage, lane, (ci % group) * out_elt);
          }
        }
        const long long tl2 = (kTiming && p.timing) ? clock64() : 0;
        ep_math += tl2 - tl1;
        if constexpr (kReduce) {
          if ((ci & 3) == 3) {             // 64 columns staged: write them out as full lines
            const int64_t warp_row0r = row - lane;
            flush_store_stage(p, rmaps, store_stage, my_rank, blk, warp_row0r, own_row - lane, rows_per_block,
                              col_base + c0 - 3 * kChunk, lane, p.red.pull != 0 && p.red.world > 1);
          }
        } else {
          flush_group(ci);
        }
        if (kTiming && p.timing) ep_flush += clock64() - tl2;
      }
      if constexpr (kReduce) {
        // Lane 0 issued this tile's bulk stores (two groups).  Waiting for them here would put an
        // NVLink round trip into every tile, so the owner's flag for a pushed tile is raised one
        // tile later, when its stores have long been performed.
        if (lane == 0) {
          if (pending_flag != nullptr) {
            if (blk == my_rank && p.red.d_multicast != nullptr && !p.red.pull) tma_store_wait_all<0>();   // this tile added no groups
            else tma_store_wait_all<2>();                                                  // all but this tile's two
            asm volatile("fence.proxy.async.global;" ::: "memory");
            red_relaxed_sys_add_u32(pending_flag, 1u);
            pending_flag = nullptr;
          }
          if (blk != my_rank || spread) pending_flag = p.red.flags[blk] + flag_index;
        }
      }
      if (!kReduce && item.mode == 1) {
        // The dumped part is complete: publish it to the cluster that finishes this tile.
        __threadfence();
        __syncwarp();
        if (lane == 0) st_release_gpu_u64(p.sk_flags + cluster_id * 2 * kEpilogueWarps + warp_part, p.sk_epoch);
      }
      if (p.progress != nullptr) {
        // Publish this warp's part of the tile: each lane orders its own stores device-wide, the
        // warp agrees, one lane counts.  A consumer that sees the full count sees the stores.
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(p.progress + mt / p.progress_tiles, 1u);
      }
      // Hand the accumulator back to the MMA issuer (in the leader CTA): one arrival per warp.
      tc_fence_before_sync();
      __syncwarp();
      if (kTiming && p.timing) ep_busy += clock64() - te1;
      if (lane == 0) {
        if (kPair && rank != 0) mbar_arrive_cluster(map_to_cta(&aux->acc_empty_bar[acc], 0));
        else mbar_arrive(&aux->acc_empty_bar[acc]);
      }
      if (++acc == kAccBufs) {
        acc = 0;
        acc_phase ^= 1;
      }
      if constexpr (kReduce) {
        if (p.red.pull == 1 && blk == my_rank && p.red.world > 1) {
          // Pull mode, own rows.  The accumulator is back with the issuer, this rank's partial is on its way to its
          // own staging buffer, and every other rank has said (flag wait above) that its partial is in ITS staging
          // buffer.  Fetch the sum -- one multimem.ld_reduce per 16 bytes when the staging buffers are bound to an
          // NVSwitch multicast address, else plain peer loads added in rank order -- and send the finished rows
          // to every rank's D the same way the push mode does.
          if (lane == 0) {
            tma_store_wait_all<0>();                                   // own partial (and everything before it) is in memory
            asm volatile("fence.proxy.async.global;" ::: "memory");
            if (pending_flag != nullptr) {
              red_relaxed_sys_add_u32(pending_flag, 1u);
              pending_flag = nullptr;
            }
          }
          __syncwarp();
          const int unit = lane & 7;
          const int64_t stage_row0 = int64_t(my_rank) * rows_per_block + own_row - lane;
          const int64_t d_row0 = row - lane;
#pragma unroll 1
          for (int gi = 0; gi < kColsPerEpilogueWarp / 64; ++gi) {
            const int64_t gcol0 = col_base + gi * 64;
            const int64_t col = gcol0 + unit * 8;
            uint4 v[8];
            if (col < p.n) {
              if (p.red.stage_multicast != nullptr) {
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                  const int rrow = it * 4 + (lane >> 3);
                  v[it] = multimem_ld_reduce_bf16x8(p.red.stage_multicast + (stage_row0 + rrow) * p.n + col);
                }
              } else {
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                  const int rrow = it * 4 + (lane >> 3);
                  float acc8[8];
#pragma unroll
                  for (int i = 0; i < 8; ++i) acc8[i] = 0.0f;
                  for (int32_t s = 0; s < p.red.world; ++s) {
                    const uint4 x = __ldcg(reinterpret_cast<const uint4*>(p.red.stage[s] + (stage_row0 + rrow) * p.n + col));
                    const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xw[i]));
                      acc8[2 * i] += f.x;
                      acc8[2 * i + 1] += f.y;
                    }
                  }
                  uint32_t o[4];
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(acc8[2 * i], acc8[2 * i + 1]);
                    o[i] = *reinterpret_cast<const uint32_t*>(&h);
                  }
                  v[it] = make_uint4(o[0], o[1], o[2], o[3]);
                }
              }
            }
            if (lane == 0) tma_store_wait_read<0>();      // the stage's previous contents have left
            __syncwarp();
            if (col < p.n) {
#pragma unroll
              for (int it = 0; it < 8; ++it) {
                const int rrow = it * 4 + (lane >> 3);
                store_stage[rrow * 8 + (unit ^ (rrow & 7))] = v[it];
              }
            }
            flush_store_stage(p, rmaps, store_stage, my_rank, blk, d_row0, own_row - lane, rows_per_block, gcol0, lane);
          }
        }
      }
    }
    if constexpr (kReduce) {
      if (lane == 0) {
        tma_store_wait_all<0>();
        asm volatile("fence.proxy.async.global;" ::: "memory");
        if (pending_flag != nullptr) red_relaxed_sys_add_u32(pending_flag, 1u);
        pending_flag = nullptr;
      }
      if (spread && ok) {          // this warp's share of the last round's sums (the reducer warps take the other rounds)
        __syncwarp();
        ok = reduce_parts(p, my_rank, p.red.stages * p.red.col_rounds - 1, (first_tile * 2 + int32_t(rank)) * (kEpilogueWarps + kReducerWarps) + ew,
                          tile_step * 2 * (kEpilogueWarps + kReducerWarps), lane, abort_flag);
      }
      __threadfence_system();       // this warp's rows are in every rank's D before the CTA reports (end of the kernel)
    }
    if (kTiming && p.timing && warp == 2 && lane == 0) {
      p.timing[blockIdx.x * kTimingSlots + 15] = global_timer_ns();        // column loops done, before the amax hand-shake
      p.timing[blockIdx.x * kTimingSlots + 5] = ep_wait;
      p.timing[blockIdx.x * kTimingSlots + 6] = ep_busy;
      p.timing[blockIdx.x * kTimingSlots + 16] = ep_ld;
      p.timing[blockIdx.x * kTimingSlots + 17] = ep_math;
      p.timing[blockIdx.x * kTimingSlots + 18] = ep_flush;
    }
    if (!kInt8 && p.amax != nullptr) {
      // The bit pattern of a non-negative float orders like the float; NaN patterns sit above
      // +inf, so an integer max propagates NaN the way XLA's `maximum` does.
      amax_bits = __reduce_max_sync(0xffffffffu, amax_bits);
      if (lane == 0) {
        if (p.amax_sync != nullptr) {
          const unsigned long long old = atomicExch(p.amax_sync, p.amax_epoch);
          if (old != p.amax_epoch) {
            *reinterpret_cast<volatile unsigned int*>(p.amax) = 0u;
            __threadfence();
            st_release_gpu_u64(p.amax_sync + 1, p.amax_epoch);
          } else {
            uint64_t t0 = 0;
            uint32_t polls = 0;
            while (ld_acquire_gpu_u64(p.amax_sync + 1) != p.amax_epoch) {
              if ((++polls & 1023u) == 0) {
                const uint64_t now = global_timer_ns();
                if (t0 == 0) t0 = now;
                if (now - t0 > kWaitLimitNs) {
                  atomicOr(p.status, kStatusEpilogueTimeout);
                  break;
                }
              }
            }
          }
        }
        atomicMax(reinterpret_cast<unsigned int*>(p.amax), amax_bits);
      }
    }
    if (kTiming && p.timing && warp == 2 && lane == 0) p.timing[blockIdx.x * kTimingSlots + 12] = global_timer_ns();
  }

  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kReduce) {
    // End of call.  Every warp of this CTA has put its rows into every rank's D and fenced them system-wide.  The CTAs
    // of a rank count themselves on a word of their own GPU; the last one tells every rank (one remote add per rank and
    // call -- warps reporting one by one meant world x 1480 system-scope adds onto one word of every GPU), and every
    // CTA stays until all ranks have reported, so that D is complete here when the kernel ends and nobody overwrites
    // a staging buffer that is still being read.
    if (threadIdx.x == 0) {
      uint32_t* const local = p.red.flags[my_rank] + p.red.done_index + 1;
      uint32_t old;
      asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(local) : "memory");
      if (old + 1 == p.red.done_local_target) {
        for (int32_t j = 0; j < p.red.world; ++j) red_release_sys_add_u32(p.red.flags[j] + p.red.done_index, 1u);
      }
      (void)counter_wait(p.red.flags[my_rank] + p.red.done_index, p.red.done_target, abort_flag, p.status, kStatusPeerTimeout, p.red.peer_wait_ns);
    }
    __syncthreads();
  }
  if (kPair) cluster_sync_all();   // nobody leaves while the peer may still read this CTA's shared memory
  if (kTiming && p.timing && threadIdx.x == 0) p.timing[blockIdx.x * kTimingSlots + 13] = global_timer_ns();
  if (warp == 1) {
    tc_fence_after_sync();
    if (kPair) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn GetEncodeTiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      p = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int g_max_pair_clusters[64];   // co-resident 2-CTA clusters per device, filled by InitDenseKernels

template <bool kInt8, bool kPair, bool kReduce = false>
cudaError_t LaunchOne(int grid, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb, const DenseArgs& p,
                      const ReduceMaps* rmaps = nullptr) {
  static const ReduceMaps no_maps{};
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kReduce ? kReduceThreads : kThreads, 1, 1);
  cfg.dynamicSmemBytes = DenseSmemBytes<kPair, kReduce>();
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kPair ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // Programmatic dependent launch: this kernel's set-up (barriers, TMEM, descriptor prefetch) overlaps the tail
  // of the kernel in front of it; its griddep_wait() orders every global access behind that kernel's end.
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = kReduce ? 1 : 2;       // the peer-reduce form waits on other GPUs: it keeps plain stream order
  return cudaLaunchKernelEx(&cfg, dense_gemm_kernel<kInt8, kPair, kReduce>, ta, tb, p, rmaps ? *rmaps : no_maps);
}

}  // namespace

// A row-major [rows, cols] byte matrix viewed as a 2-D tensor with `cols` innermost; box =
// box_cols x box_rows, 128-byte swizzle, out-of-range elements read as zero.
Status MakeByteMatrixMap(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, uint32_t box_cols,
                         uint32_t box_rows, int l2_promotion) {
  EncodeTiledFn encode = GetEncodeTiled();
  if (encode == nullptr) return Status::Error(kInternal, "cuTensorMapEncodeTiled is not available from this driver");
  if (cols % 16 != 0) return Status::Error(kInvalidArgument, "the minor dimension of an 8-bit operand must be a multiple of 16");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return Status::Error(kInvalidArgument, "operand base address must be 16-byte aligned");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols)};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                            elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            l2_promotion == 0   ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                            : l2_promotion == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                            : l2_promotion == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                                : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Status::Error(kInternal, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(r)));
  return Status::Ok();
}

int MaxPairClusters();

// `batch` row-major [rows, cols] byte matrices stored one after the other, as a 3-D tensor
// (cols innermost); box = box_cols x box_rows x 1, 128-byte swizzle, out-of-range elements read
// as zero -- also past the last row of a batch, so tiles never see the next batch's data.
Status MakeBatchedByteMatrixMap(CUtensorMap* map, const void* base, int64_t batch, int64_t rows, int64_t cols,
                                uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn encode = GetEncodeTiled();
  if (encode == nullptr) return Status::Error(kInternal, "cuTensorMapEncodeTiled is not available from this driver");
  if (cols % 16 != 0) return Status::Error(kInvalidArgument, "the minor dimension of an 8-bit operand must be a multiple of 16");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return Status::Error(kInvalidArgument, "operand base address must be 16-byte aligned");
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows) * static_cast<cuuint64_t>(cols)};
  const cuuint32_t box[3] = {box_cols, box_rows, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem_strides,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Status::Error(kInternal, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(r)));
  return Status::Ok();
}

// A 3-D byte view [batch, rows, cols] without a shared-memory swizzle: the box lands row after row, box_cols bytes
// each.  Rows are row_stride bytes apart and batches batch_stride (both multiples of 16); cols itself may be anything,
// bytes past it read as zero.
Status MakeBatchedPlainByteMap(CUtensorMap* map, const void* base, int64_t batch, int64_t rows, int64_t cols,
                               int64_t row_stride, int64_t batch_stride, uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn encode = GetEncodeTiled();
  if (encode == nullptr) return Status::Error(kInternal, "cuTensorMapEncodeTiled is not available from this driver");
  if (row_stride % 16 != 0 || batch_stride % 16 != 0 || box_cols % 16 != 0 || cols > row_stride)
    return Status::Error(kInvalidArgument, "the row and batch strides and the box width must be multiples of 16 bytes");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return Status::Error(kInvalidArgument, "base address must be 16-byte aligned");
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_stride), static_cast<cuuint64_t>(batch_stride)};
  const cuuint32_t box[3] = {box_cols, box_rows, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem_strides,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Status::Error(kInternal, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(r)));
  return Status::Ok();
}

Status InitDenseKernels() {
  int device = 0;
  cudaGetDevice(&device);
  cudaError_t e = cudaSuccess;
  auto set = [&](const void* fn, size_t bytes) {
    if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
  };
  set(reinterpret_cast<const void*>(dense_gemm_kernel<false, false>), DenseSmemBytes<false>());
  set(reinterpret_cast<const void*>(dense_gemm_kernel<true, false>), DenseSmemBytes<false>());
  set(reinterpret_cast<const void*>(dense_gemm_kernel<false, true>), DenseSmemBytes<true>());
  set(reinterpret_cast<const void*>(dense_gemm_kernel<true, true>), DenseSmemBytes<true>());
  set(reinterpret_cast<const void*>(dense_gemm_kernel<false, true, true>), (DenseSmemBytes<true, true>()));
  if (e != cudaSuccess) return Status::Error(kInternal, std::string("cudaFuncSetAttribute(dense): ") + cudaGetErrorString(e));
  // How many CTA pairs fit on the device at once bounds the persistent grid of the pair kernel.
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2 * 148, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = DenseSmemBytes<true>();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  e = cudaOccupancyMaxActiveClusters(&clusters, dense_gemm_kernel<false, true>, &cfg);
  if (e != cudaSuccess || clusters <= 0) {
    cudaGetLastError();
    clusters = 0;             // the pair kernel is then never selected
  }
  if (device >= 0 && device < 64) g_max_pair_clusters[device] = clusters;
  return Status::Ok();
}

uint32_t FormatCode(int32_t dtype) {
  // kind::f8f6f4: e4m3 = 0, e5m2 = 1; kind::i8: s8 = 1.
  return dtype == kF8E5M2 ? 1u : (dtype == kS8 ? 1u : 0u);
}

#if B200SD_TUNING
// Copies the tuning counters of the last dense launch on the current device (8 per CTA).
extern "C" int b200sd_debug_read_timing(unsigned long long* out, int count) {
  cudaDeviceSynchronize();
  return int(cudaMemcpyFromSymbol(out, g_dense_timing, sizeof(unsigned long long) * size_t(count)));
}
#endif

// A 64-bit value no earlier launch of this process has used and that stale workspace contents will
// not equal by accident: a per-process random tag in the high half, a launch counter in the low half.
unsigned long long NextDenseEpoch() {
  static const uint64_t tag = [] {
    std::random_device rd;
    const uint64_t t = (uint64_t(rd()) << 32) ^ uint64_t(rd());
    return (t | (1ull << 62)) & 0xFFFFFFFF00000000ull;
  }();
  static std::atomic<uint64_t> counter{1};
  return tag | (counter.fetch_add(1, std::memory_order_relaxed) & 0xFFFFFFFFull);
}

uint32_t ProgressIncrement(const GemmProblem& g, int32_t block) {
  // Every epilogue warp of every CTA working on a tile counts once: 8 warps x (2 CTAs for the pair kernel).
  if (g.progress_rows <= 0 || block < 0 || int64_t(block) * g.progress_rows >= g.m) return 0;
  int device = 0;
  cudaGetDevice(&device);
  if (!InitDevice(device).ok()) return 0;
  const bool pair = g.m > kBM && MaxPairClusters() > 0;
  const int tile_rows = pair ? 2 * kBM : kBM;
  const int64_t rows = std::min<int64_t>(g.progress_rows, g.m - int64_t(block) * g.progress_rows);
  const int64_t row_tiles = (rows + tile_rows - 1) / tile_rows;
  const int64_t col_tiles = (g.n + kBN - 1) / kBN;
  return uint32_t(row_tiles * col_tiles * kEpilogueWarps * (pair ? 2 : 1));
}

int MaxPairClusters() {
  int device = 0;
  cudaGetDevice(&device);
  return (device >= 0 && device < 64) ? g_max_pair_clusters[device] : 0;
}

Status LaunchDense(const GemmProblem& g, cudaStream_t stream, LaunchStats* stats, int variant) {
  int device = 0;
  cudaGetDevice(&device);
  Status st = InitDevice(device);
  if (!st.ok()) return st;
  const int max_pairs = MaxPairClusters();
  bool pair = g.m > kBM && max_pairs > 0;           // a second CTA would only compute padding when M <= 128
  if (variant == kKernelDenseSingle) pair = false;
  if (variant == kKernelDensePair || variant == kKernelDenseStreamK) {
    if (max_pairs <= 0) return Status::Error(kFailedPrecondition, "this device cannot co-schedule CTA pairs for the pair kernel");
    pair = true;
  }

  const int64_t batch = g.batch > 0 ? g.batch : 1;
  if (batch > 1 && g.progress != nullptr) return Status::Error(kInvalidArgument, "progress reporting is not available for batched dots");
  if (batch * ((g.m + kBM - 1) / kBM) * ((g.n + kBN - 1) / kBN) > (1ll << 30)) return Status::Error(kInvalidArgument, "too many tiles");
  CUtensorMap tmap_a, tmap_b;
  if (g.a_mn_major) {
    st = MakeBatchedByteMatrixMap(&tmap_a, g.a, batch, g.k, g.m, 128, kBK);       // [k, m], box 128(m) x 128(k)
  } else {
    st = MakeBatchedByteMatrixMap(&tmap_a, g.a, batch, g.m, g.k, kBK, kBM);       // [m, k], box 128(k) x 128(m)
  }
  if (!st.ok()) return st;
  if (g.b_mn_major) {
    st = MakeBatchedByteMatrixMap(&tmap_b, g.b, batch, g.k, g.n, 128, kBK);       // [k, n], box 128(n) x 128(k)
  } else {
    st = MakeBatchedByteMatrixMap(&tmap_b, g.b, batch, g.n, g.k, kBK, pair ? kBN / 2 : kBN);   // [n, k], box 128(k) x 128|256(n)
  }
  if (!st.ok()) return st;

  DenseArgs p{};
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.batch = int32_t(batch);
  const int tile_rows = pair ? 2 * kBM : kBM;
  p.num_m_tiles = int32_t((g.m + tile_rows - 1) / tile_rows);
  p.num_n_tiles = int32_t((g.n + kBN - 1) / kBN);
  p.num_k_blocks = int32_t((g.k + kBK - 1) / kBK);
  static const int env_raster = TuningEnvInt("B200SD_RASTER", 0);
  p.raster_group = env_raster > 0 ? env_raster : 16;   // 16 measured best at 8192^3
  p.progress = nullptr;
  p.progress_tiles = 1;
  if (g.progress != nullptr) {
    if (g.progress_rows <= 0 || g.progress_rows % (2 * kBM) != 0) return Status::Error(kInvalidArgument, "progress_rows must be a positive multiple of 256");
    p.progress = g.progress;
    p.progress_tiles = g.progress_rows / tile_rows;
    p.raster_group = p.progress_tiles;   // row blocks then finish one after the other, not all at the end
  }
  p.a_mn_major = g.a_mn_major; p.b_mn_major = g.b_mn_major;
  p.idesc = make_idesc(g.int8 ? 2u : 1u, FormatCode(g.a_dtype), FormatCode(g.b_dtype), g.a_mn_major, g.b_mn_major,
                       uint32_t(tile_rows), kBN);
  p.a_scale = g.a_scale; p.b_scale = g.b_scale; p.d_scale = g.d_scale;
  p.alpha = g.alpha; p.beta = g.beta;
  p.c = (g.beta != 0.0f) ? g.c : nullptr; p.c_dtype = g.c_dtype;
  p.bias = g.bias; p.bias_dtype = g.bias_dtype;
  p.activation = g.activation;
  p.amax = g.amax;
  p.a_row_scale = g.a_row_scale; p.b_col_scale = g.b_col_scale;
  p.d_s32 = g.d_s32;
  p.d = g.d; p.d_dtype = g.d_dtype;
  if (g.int8 && g.d_dtype == kS32) {   // the accumulator itself is the result
    p.d_s32 = static_cast<int32_t*>(g.d);
    p.d = nullptr;
  }
  // Vector stores need 16-byte aligned row starts for every output that is written.
  auto aligned = [&](const void* ptr, int64_t elt) {
    return ptr == nullptr || ((reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (g.n * elt) % 16 == 0);
  };
  const int64_t d_elt = (g.d_dtype == kF8E4M3FN || g.d_dtype == kF8E5M2) ? 1 : (g.d_dtype == kF32 || g.d_dtype == kS32) ? 4 : 2;
  p.vec_store_ok = aligned(p.d, d_elt) && aligned(p.d_s32, 4);
  p.status = StatusWordPtr();
  p.timing = nullptr;
#if B200SD_TUNING
  static const bool timing_on = TuningEnvInt("B200SD_TIMING", 0) == 1;
  if (timing_on) {
    cudaGetSymbolAddress(reinterpret_cast<void**>(&p.timing), g_dense_timing);
    cudaMemsetAsync(p.timing, 0, sizeof(unsigned long long) * kTimingSlots * 512, stream);
  }
#endif

  const int64_t tiles = batch * p.num_m_tiles * p.num_n_tiles;
  int grid;
  if (pair) {
    grid = 2 * int(tiles < max_pairs ? tiles : max_pairs);
  } else {
    grid = int(tiles < DeviceSmCount() ? tiles : DeviceSmCount());
  }
  if (g.max_ctas > 0 && grid > g.max_ctas) grid = pair ? (g.max_ctas >= 2 ? g.max_ctas & ~1 : 2) : g.max_ctas;
  // Stream-K tail: when the tiles do not fill the last wave, cut the leftover tiles along K so
  // that every cluster gets the same number of k-blocks.  Needs the caller's workspace for the
  // partial accumulators and at least one full wave (or a long K) to be worth the extra traffic.
  p.dp_tiles = int32_t(tiles);
  p.sk_tiles = 0;
  const bool capturing = StreamIsCapturing(stream);
  // Opt-in (kernel variant DENSE_STREAMK): measured on B200 it does not pay under the 1 kW power cap,
  // where SMs idling in the last wave let the others clock higher (8192 x 1024 x 8192: 64 us against
  // 62 us without; 4096^3: 73 against 62).
  if (pair && variant == kKernelDenseStreamK && g.progress == nullptr && g.workspace != nullptr) {
    const int clusters = grid / 2;
    const int64_t rem = tiles % clusters;
    const int64_t share = rem * p.num_k_blocks / clusters;              // k-blocks per cluster in the tail
    const size_t need = kSkFlagBytes + size_t(clusters) * kSkPartialBytes;
    if (tiles > clusters && rem != 0 && share >= 8 && g.workspace_bytes >= need && clusters <= 128 &&
        (reinterpret_cast<uintptr_t>(g.workspace) & 15) == 0) {
      p.sk_tiles = int32_t(rem);
      p.dp_tiles = int32_t(tiles - rem);
      p.sk_epoch = NextDenseEpoch();
      p.sk_flags = static_cast<unsigned long long*>(g.workspace);
      p.sk_partials = reinterpret_cast<uint4*>(static_cast<uint8_t*>(g.workspace) + kSkFlagBytes);
      if (capturing) {   // replays repeat sk_epoch: the previous replay's flags must be cleared by a node of the graph
        cudaError_t me = cudaMemsetAsync(p.sk_flags, 0, kSkFlagBytes, stream);
        if (me != cudaSuccess) return Status::Error(kInternal, std::string("cudaMemsetAsync(stream-K flags): ") + cudaGetErrorString(me));
      }
    }
  }
  p.amax_sync = nullptr;
  if (g.amax != nullptr) {
    // The last 64 bytes of the caller's workspace hold the two words that let the kernel clear amax
    // itself (the stream-K scratch, when used, sits at the front); without a workspace, or while the stream is
    // being captured (every replay would carry the same epoch), a memset node does it.
    const size_t front = p.sk_tiles > 0 ? kSkFlagBytes + size_t(grid / 2) * kSkPartialBytes : 0;
    if (!capturing && g.workspace != nullptr && g.workspace_bytes >= front + 128) {
      uintptr_t end = (reinterpret_cast<uintptr_t>(g.workspace) + g.workspace_bytes) & ~uintptr_t(63);
      p.amax_sync = reinterpret_cast<unsigned long long*>(end - 64);
      p.amax_epoch = NextDenseEpoch();
    } else {
      cudaError_t e = cudaMemsetAsync(g.amax, 0, sizeof(float), stream);
      if (e != cudaSuccess) return Status::Error(kInternal, std::string("cudaMemsetAsync(amax): ") + cudaGetErrorString(e));
    }
  }
  cudaError_t e;
  if (pair) {
    e = g.int8 ? LaunchOne<true, true>(grid, stream, tmap_a, tmap_b, p) : LaunchOne<false, true>(grid, stream, tmap_a, tmap_b, p);
  } else {
    e = g.int8 ? LaunchOne<true, false>(grid, stream, tmap_a, tmap_b, p) : LaunchOne<false, false>(grid, stream, tmap_a, tmap_b, p);
  }
  if (e != cudaSuccess) return Status::Error(kInternal, std::string("dense_gemm_kernel launch: ") + cudaGetErrorString(e));
  if (stats) {
    stats->kernel = pair ? kKernelDensePair : kKernelDenseSingle;
    stats->grid = grid;
    stats->launches = 1;
  }
  return Status::Ok();
}

// Tensor maps of the emulated ranks (single-GPU testing of the peer-reduce protocol).
__device__ __align__(64) CUtensorMap g_emu_maps[2 * kMaxPeers];

size_t PeerReduceFlagWords(int64_t m, int64_t n, int32_t world) {
  if (world < 1 || m <= 0 || n <= 0 || m % (int64_t(world) * 2 * kBM) != 0) return 0;
  const int64_t tiles_per_block = (m / world / (2 * kBM)) * ((n + kBN - 1) / kBN);
  return size_t(tiles_per_block) * 2 * kEpilogueWarps + 64;   // one flag per (tile, CTA of the pair, warp); then the end-of-call counter
}

Status LaunchDenseReduce(const GemmProblem& g, const PeerReduceProblem& r, cudaStream_t stream, LaunchStats* stats) {
  int device = 0;
  cudaGetDevice(&device);
  Status st = InitDevice(device);
  if (!st.ok()) return st;
  const int max_pairs = MaxPairClusters();
  if (max_pairs <= 0) return Status::Error(kFailedPrecondition, "this device cannot co-schedule CTA pairs for the pair kernel");
  if (r.world < 1 || r.world > kMaxPeers || r.rank < 0 || r.rank >= r.world) return Status::Error(kInvalidArgument, "world must be 1..8 and rank inside it");
  if (g.batch > 1) return Status::Error(kInvalidArgument, "the peer-reduced dot does not take batched dots");
  if (g.int8 || g.d_dtype != kBF16 || g.c != nullptr || g.bias != nullptr || g.activation != kActNone || g.amax != nullptr || g.d_scale != nullptr)
    return Status::Error(kInvalidArgument, "the peer-reduced dot is the plain FP8 scaled dot with a bf16 result");
  if (g.m % (int64_t(r.world) * 2 * kBM) != 0) return Status::Error(kInvalidArgument, "m must be a multiple of 256 x world for the peer-reduced dot");
  if (g.n % 16 != 0) return Status::Error(kInvalidArgument, "n must be a multiple of 16");
  if (r.epoch == 0) return Status::Error(kInvalidArgument, "epoch counts calls from 1");
  if (r.emulate && r.emulate != r.world) return Status::Error(kInvalidArgument, "emulate must be 0 or equal to world");
  for (int i = 0; i < r.world; ++i) {
    if (r.d[i] == nullptr || r.stage[i] == nullptr || r.flags[i] == nullptr) return Status::Error(kInvalidArgument, "d, stage and flags are needed for every rank");
    if ((reinterpret_cast<uintptr_t>(r.d[i]) | reinterpret_cast<uintptr_t>(r.stage[i])) & 15) return Status::Error(kInvalidArgument, "d and stage must be 16-byte aligned");
    if (r.emulate && (r.emu_a[i] == nullptr || r.emu_b[i] == nullptr)) return Status::Error(kInvalidArgument, "emulation needs every rank's operands");
  }

  DenseArgs p{};
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.batch = 1;
  p.num_m_tiles = int32_t(g.m / (2 * kBM));
  p.num_n_tiles = int32_t((g.n + kBN - 1) / kBN);
  p.num_k_blocks = int32_t((g.k + kBK - 1) / kBK);
  p.raster_group = 16;
  p.a_mn_major = g.a_mn_major; p.b_mn_major = g.b_mn_major;
  p.idesc = make_idesc(1u, FormatCode(g.a_dtype), FormatCode(g.b_dtype), g.a_mn_major, g.b_mn_major, 2 * kBM, kBN);
  p.a_scale = g.a_scale; p.b_scale = g.b_scale;
  p.alpha = g.alpha;
  p.d = r.d[r.rank]; p.d_dtype = kBF16;
  p.vec_store_ok = 1;
  p.status = StatusWordPtr();
  p.progress_tiles = 1;

  const int64_t tiles = int64_t(p.num_m_tiles) * p.num_n_tiles;
  p.dp_tiles = int32_t(tiles);
  p.sk_tiles = 0;
  int clusters_per_rank = r.emulate ? max_pairs / r.world : max_pairs;
  if (clusters_per_rank > tiles) clusters_per_rank = int(tiles);
  if (clusters_per_rank < 1) return Status::Error(kFailedPrecondition, "not enough SMs to emulate this many ranks");
  const int grid = 2 * clusters_per_rank * (r.emulate ? r.world : 1);

  ReduceArgs& q = p.red;
  q.world = r.world; q.rank = r.rank; q.emulate = r.emulate;
  q.m_tiles_per_block = p.num_m_tiles / r.world;
  // Rounds in which the rows are dealt out: two when each rank's row tiles divide (measured at 4 GPUs on
  // 8192 x 28672 x 8192: 0.515 / 0.487 / 0.520 / 0.580 ms for 1 / 2 / 4 / 8 rounds -- more rounds spread the
  // broadcasts but add a rendezvous each).
  static const int env_stages = TuningEnvInt("B200SD_REDUCE_STAGES", 0);
  q.stages = q.m_tiles_per_block % 2 == 0 ? 2 : 1;
  q.col_rounds = 1;
  q.debug = TuningEnvInt("B200SD_REDUCE_DEBUG", 0);
  if (env_stages > 0 && q.m_tiles_per_block % env_stages == 0) q.stages = env_stages;
  q.flag_target = r.epoch * uint32_t(r.world - 1);
  q.done_index = int32_t(PeerReduceFlagWords(g.m, g.n, r.world)) - 32;
  q.done_target = r.epoch * uint32_t(r.world);
  q.done_local_target = r.epoch * uint32_t(2 * clusters_per_rank);
  q.peer_wait_ns = uint64_t(r.peer_wait_ms ? r.peer_wait_ms : kDefaultPeerWaitMs) * 1000000ull;
  for (int i = 0; i < r.world; ++i) {
    q.d[i] = static_cast<uint16_t*>(r.d[i]);
    q.stage[i] = static_cast<uint16_t*>(r.stage[i]);
    q.flags[i] = r.flags[i];
  }
#if B200SD_TUNING
  static const bool timing_on = TuningEnvInt("B200SD_TIMING", 0) == 1;
  if (timing_on) {
    cudaGetSymbolAddress(reinterpret_cast<void**>(&p.timing), g_dense_timing);
    cudaMemsetAsync(p.timing, 0, sizeof(unsigned long long) * kTimingSlots * 512, stream);
  }
#endif
  q.emu_maps = nullptr;
  q.d_multicast = r.emulate ? nullptr : static_cast<uint16_t*>(r.d_multicast);
  q.pull = ((r.pull == 1 || r.pull == 2) && r.world > 1) ? r.pull : 0;
  if (q.pull == 2) {
    q.flag_target = r.epoch * uint32_t(r.world);      // a rank's own partial counts like every other
    // Rounds: no warp waits for a peer inside the tile loop in this form, so rounds cost no rendezvous, and only the last
    // round's sums (1 / rounds of the traffic) are left for the end of the kernel.  A round gives every owner a
    // sub-block of mtps x ntps tiles; the sub-block is kept as square as its 64 / world tiles allow, because the tiles
    // of a round run at the same time and share the mtps row panels of A and ntps column panels of B in L2.
    {
      const int64_t want = std::max<int64_t>(1, 64 / r.world);
      int best_m = q.m_tiles_per_block, best_n = p.num_n_tiles;
      for (int mt = 1; mt <= q.m_tiles_per_block; ++mt) {
        if (q.m_tiles_per_block % mt) continue;
        for (int nt = 1; nt <= p.num_n_tiles; ++nt) {
          if (p.num_n_tiles % nt || int64_t(mt) * nt < want) continue;
          const bool better = mt + nt < best_m + best_n || (mt + nt == best_m + best_n && mt * nt < best_m * best_n);
          if (better) { best_m = mt; best_n = nt; }
        }
      }
      q.stages = q.m_tiles_per_block / best_m;
      q.col_rounds = p.num_n_tiles / best_n;
    }
    static const int env_cols = TuningEnvInt("B200SD_REDUCE_COL_ROUNDS", 0);
    if (env_stages > 0 && q.m_tiles_per_block % env_stages == 0) q.stages = env_stages;
    if (env_cols > 0 && p.num_n_tiles % env_cols == 0) q.col_rounds = env_cols;
  }
  q.stage_multicast = (r.emulate || !r.pull) ? nullptr : static_cast<uint16_t*>(r.stage_multicast);

  auto make_maps = [&](const void* a, const void* b, CUtensorMap* ta, CUtensorMap* tb) {
    Status s = g.a_mn_major ? MakeBatchedByteMatrixMap(ta, a, 1, g.k, g.m, 128, kBK) : MakeBatchedByteMatrixMap(ta, a, 1, g.m, g.k, kBK, kBM);
    if (!s.ok()) return s;
    return g.b_mn_major ? MakeBatchedByteMatrixMap(tb, b, 1, g.k, g.n, 128, kBK) : MakeBatchedByteMatrixMap(tb, b, 1, g.n, g.k, kBK, kBN / 2);
  };
  CUtensorMap tmap_a, tmap_b;
  if (r.emulate) {
    CUtensorMap maps[2 * kMaxPeers];
    for (int i = 0; i < r.world; ++i) {
      st = make_maps(r.emu_a[i], r.emu_b[i], &maps[2 * i], &maps[2 * i + 1]);
      if (!st.ok()) return st;
    }
    cudaError_t e = cudaMemcpyToSymbolAsync(g_emu_maps, maps, sizeof(CUtensorMap) * 2 * r.world, 0, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);   // `maps` lives on this stack frame
    if (e != cudaSuccess) return Status::Error(kInternal, std::string("copying the emulated ranks' tensor maps: ") + cudaGetErrorString(e));
    cudaGetSymbolAddress(reinterpret_cast<void**>(const_cast<CUtensorMap**>(&q.emu_maps)), g_emu_maps);
    tmap_a = maps[0];
    tmap_b = maps[1];
  } else {
    st = make_maps(g.a, g.b, &tmap_a, &tmap_b);
    if (!st.ok()) return st;
  }
  // Maps for the epilogue's bulk stores: each rank's staging buffer and output as [m, 2n]-byte matrices.
  ReduceMaps rmaps{};
  for (int i = 0; i < r.world; ++i) {
    st = MakeByteMatrixMap(&rmaps.stage[i], r.stage[i], g.m, 2 * g.n, 128, 32);
    if (st.ok()) st = MakeByteMatrixMap(&rmaps.d[i], r.d[i], g.m, 2 * g.n, 128, 32);
    if (!st.ok()) return st;
  }
  cudaError_t e = LaunchOne<false, true, true>(grid, stream, tmap_a, tmap_b, p, &rmaps);
  if (e != cudaSuccess) return Status::Error(kInternal, std::string("dense_gemm_kernel (peer reduce) launch: ") + cudaGetErrorString(e));
  if (stats) {
    stats->kernel = kKernelDensePair;
    stats->grid = grid;
    stats->launches = 1;
  }
  return Status::Ok();
}

}  // namespace b200sd
