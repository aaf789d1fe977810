// MX block-scaled dot for sm_100a: the kernel behind XLA's `__cublas$lt$matmul$mx` custom call
// (operand meaning: ThunkEmitter::EmitCublasLtMatmulMx, xla/service/gpu/thunk_emitter.cc:939-988; the
// arithmetic: `__op$block_scaled_dot`, xla/backends/gpu/transforms/block_scaling_rewriter.h:30-77):
//
//     D[b, m, n] = alpha * sum_k  A[b, m, k] * 2^(SA[b, m, k/32] - 127)  *  B[b, n, k] * 2^(SB[b, n, k/32] - 127)
//
// A and B are FP8 (e4m3fn / e5m2), stored with the contracting dimension minor; SA and SB are
// f8e8m0fnu, one per 32 values along K, stored row-major exactly as the HLO operand is -- no
// pre-swizzled scale layout is asked of the caller.
//
// One persistent, warp-specialised kernel run by clusters of two CTAs on 256 x 256 tiles
// (tcgen05.mma cta_group::2, kind::mxf8f6f4.block_scale), 384 threads per CTA:
//   warp 0      TMA producer: per 128-deep k-block its CTA's 128 rows of A and 128 rows of B.
//   warp 1      TMEM allocator; in the leader CTA the MMA issuer: per k-block three tcgen05.cp that
//               move the block's scales from shared memory into TMEM, then four K=32 MMAs, each
//               naming the byte of the scale columns that belongs to its 32 values.
//   warps 2-3   scale loaders (alternate groups).  Scales travel in groups of four k-blocks through a ring of their own:
//               one TMA box brings 16 scale bytes (four k-blocks) of each of the CTA's 128 A rows and
//               of all 256 B rows of the tile (every CTA of the pair multiplies by every column's
//               scale); the warp then rewrites the slot in place into the layout tcgen05.cp wants: per
//               k-block and per 128 rows a block of 32 x 16 bytes, byte (r % 32) * 16 + (r / 32) * 4 + j
//               holding the scale of row r and 32-value sub-block j.  One proxy fence and one arrival
//               per group.  Scale rows that do not start on 16-byte boundaries (k not a multiple of
//               512) are gathered with plain loads instead of the box.
//   warps 4-11  epilogue: the whole 128 x 256 accumulator slice is pulled into registers (128 per
//               thread), TMEM is handed back to the issuer at once, and only then are the values
//               scaled, converted and stored.
// TMEM holds ONE 256-column accumulator: with the scale columns there is no room for a second, so
// what the epilogue keeps the tensor pipe waiting for is the register read-out, not the stores.
// Every wait is bounded; on expiry the kernel records a status bit and drains.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <string>

#include "kernels.h"
#include "ptx.cuh"

namespace b200sd {

Status MakeBatchedByteMatrixMap(CUtensorMap* map, const void* base, int64_t batch, int64_t rows, int64_t cols,
                                uint32_t box_cols, uint32_t box_rows);
Status MakeBatchedPlainByteMap(CUtensorMap* map, const void* base, int64_t batch, int64_t rows, int64_t cols,
                               int64_t row_stride, int64_t batch_stride, uint32_t box_cols, uint32_t box_rows);
int MaxPairClusters();

namespace {

constexpr int kMxBM = 128;                 // rows of D per CTA per tile (= TMEM lanes)
constexpr int kMxTileM = 2 * kMxBM;        // rows of D per pair per tile
// Two tile widths.  256 columns: one accumulator (the scale columns leave no room for a second), the tensor pipe
// waits while the epilogue reads it out.  224 columns: two accumulators (2 x 224 + 24 scale columns <= 512), the
// epilogue of one tile runs under the main loop of the next, at the price of 14 % more A traffic per flop and a
// ragged last column tile.  The host picks per shape; 256 wins wherever it does not need more rounds of tiles.
constexpr int kMxBK = 128;                 // values of K per stage: one 128-byte swizzle row
constexpr int kMxUmmaK = 32;               // K per MMA = one scale block
constexpr int kMxStages = 6;
constexpr int kMxAStageBytes = kMxBM * kMxBK;            // 16 KiB
constexpr int kMxSfBlockBytes = 512;                     // scales of 128 rows x 4 sub-blocks
constexpr int kMxSfaStageBytes = kMxSfBlockBytes;        // this CTA's 128 rows of A
constexpr int kMxSfbStageBytes = 2 * kMxSfBlockBytes;    // all 256 rows of B
constexpr int kMxSfStageBytes = kMxSfaStageBytes + kMxSfbStageBytes;
constexpr int kMxEpilogueWarps = 8;
constexpr int kMxFirstEpilogueWarp = 4;
constexpr int kMxThreads = 32 * (kMxFirstEpilogueWarp + kMxEpilogueWarps);
constexpr int kMxTmemCols = 512;
template <int kBN_>
struct MxCfg {
  static constexpr int kBN = kBN_;                            // columns of D per tile
  static constexpr int kAccBufs = kBN_ == 256 ? 1 : 2;
  static constexpr int kBStageBytes = (kBN_ / 2) * kMxBK;     // this CTA's half of the tile's B rows: 16 or 14 KiB
  static constexpr int kRawSfbBytes = kBN_ * 16;              // 16 scale bytes of every B row of the tile
  // TMEM columns: accumulators at 0 and 256; scale columns in two alternating sets so that the copy for one
  // k-block never lands on columns the MMAs of the block before may still be reading (A: 4 columns, B: 8).
  static constexpr int kTmemAccStride = 256;
  static constexpr int kTmemSfa = kAccBufs == 1 ? 256 : 480, kTmemSfaSet = kAccBufs == 1 ? 16 : 4;
  static constexpr int kTmemSfb = kAccBufs == 1 ? 288 : 488, kTmemSfbSet = kAccBufs == 1 ? 16 : 8;
  static constexpr int kColsHalf1 = kBN_ - 128;               // columns of the second group of epilogue warps: 128 or 96
  static_assert(kBN_ == 256 || kBN_ == 224, "tile widths the epilogue is written for");
};
// Scales travel in groups of four k-blocks (16 bytes per row: what one TMA box can bring), one group
// per slot of their own ring, so the loader runs well ahead of the operand stages.
constexpr int kMxSfSlots = 5;
constexpr int kMxRawSfaBytes = kMxBM * 16;               // 2 KiB: 128 rows of A
constexpr int kMxSfSlotBytes = 4 * kMxSfStageBytes;      // 6 KiB: a landed box (2 KiB + 16 bytes per B row) and four rearranged k-blocks

struct MxAux {
  uint64_t full_bar[kMxStages];    // leader's: both CTAs' operand bytes have landed
  uint64_t empty_bar[kMxStages];   // each CTA's: the MMAs that read the stage have completed
  uint64_t acc_full_bar[2];        // each CTA's: the tile's accumulator is complete
  uint64_t acc_empty_bar[2];       // leader's: all 16 epilogue warps of the pair have read the accumulator out
  uint64_t raw_full_bar[kMxSfSlots];    // each CTA's: a box of scales has landed in the slot
  uint64_t sf_full_bar[kMxSfSlots];     // leader's: both CTAs have rearranged the slot's scales
  uint64_t sf_empty_bar[kMxSfSlots];    // each CTA's: the copies and MMAs that read the slot have completed
  uint32_t tmem_base;
  int abort_flag;
};

template <int kBN>
constexpr size_t MxSmemBytes() {
  return 1024 + size_t(kMxStages) * (kMxAStageBytes + MxCfg<kBN>::kBStageBytes) + kMxSfSlots * kMxSfSlotBytes + sizeof(MxAux);
}

struct MxArgs {
  int64_t m, n, k;
  int64_t scale_cols;              // k / 32: scales in use per row of SA and SB
  int64_t sfa_ld, sfb_ld;          // bytes between rows of SA / SB (>= scale_cols; more when the arrays are padded)
  int64_t sfa_batch, sfb_batch;    // bytes between batches
  int32_t batch;
  int32_t num_m_tiles, num_n_tiles, num_k_blocks;
  int32_t raster_group;
  uint32_t idesc;
  const uint8_t* sfa;
  const uint8_t* sfb;
  int32_t sf_words_ok;             // rows of SA / SB start on 4-byte boundaries and hold whole 4-byte groups
  int32_t sf_bulk_ok;              // ... on 16-byte boundaries: the scales come by TMA, four k-blocks per box
  float alpha;
  void* d;
  int32_t d_dtype;
  int32_t vec_store_ok;
  uint32_t* status;
  unsigned long long* timing;      // tuning build: kMxTimingSlots counters per CTA, else nullptr
};

// Tuning counters per CTA (cycles unless said otherwise): [0] issuer waiting for a full stage, [1] issuer
// waiting for the accumulator to be read out, [2] issuer total, [3] producer waiting for a free stage,
// [4] scale loader waiting for its box, [5] scale loader waiting for a free slot, [6] scale loader writing,
// fencing and signalling, [7] epilogue waiting for the accumulator, [8] epilogue read-out, [9] epilogue stores,
// [10] issuer waiting for a group of scales.
constexpr int kMxTimingSlots = 16;
#if B200SD_TUNING
__device__ unsigned long long g_mx_timing[kMxTimingSlots * 512];
#endif

// Tile order: groups of `raster_group` row tiles are swept column by column, so the clusters that run at
// the same time share a few row panels of A and a few column panels of B in L2.
__device__ __forceinline__ void mx_tile_coords(int32_t tile, const MxArgs& p, int32_t* mt, int32_t* nt, int32_t* bt) {
  const int32_t per_batch = p.num_m_tiles * p.num_n_tiles;
  *bt = tile / per_batch;
  const int32_t t = tile - *bt * per_batch;
  const int32_t group_tiles = p.raster_group * p.num_n_tiles;
  const int32_t g = t / group_tiles;
  const int32_t r = t - g * group_tiles;
  const int32_t rows = min(p.raster_group, p.num_m_tiles - g * p.raster_group);
  *mt = g * p.raster_group + r % rows;
  *nt = r / rows;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Stores 32 consecutive f32 values of one row of D, columns [col, col + 32), as `dtype`.
__device__ __forceinline__ void mx_store_chunk(const MxArgs& p, int64_t row_off, int32_t col, const uint32_t (&r)[32]) {
  const float alpha = p.alpha;
  if (p.vec_store_ok && col + 32 <= p.n) {
    if (p.d_dtype == kF32) {
      float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.d) + row_off + col);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dst[i] = make_float4(__uint_as_float(r[4 * i]) * alpha, __uint_as_float(r[4 * i + 1]) * alpha,
                             __uint_as_float(r[4 * i + 2]) * alpha, __uint_as_float(r[4 * i + 3]) * alpha);
      }
    } else {
      uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.d) + row_off + col);
      const bool bf = p.d_dtype == kBF16;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = __uint_as_float(r[8 * i + 2 * j]) * alpha, hi = __uint_as_float(r[8 * i + 2 * j + 1]) * alpha;
          w[j] = bf ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
        }
        dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    if (col + i < p.n) {
      const float v = __uint_as_float(r[i]) * alpha;
      if (p.d_dtype == kF32) static_cast<float*>(p.d)[row_off + col + i] = v;
      else if (p.d_dtype == kBF16) static_cast<__nv_bfloat16*>(p.d)[row_off + col + i] = __float2bfloat16_rn(v);
      else static_cast<__half*>(p.d)[row_off + col + i] = __float2half_rn(v);
    }
  }
}

template <int kBN>
__global__ void __launch_bounds__(kMxThreads, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb, const MxArgs p) {
  using Cfg = MxCfg<kBN>;
  constexpr int kMxBN = Cfg::kBN;
  constexpr int kMxBStageBytes = Cfg::kBStageBytes;
  constexpr int kAccBufs = Cfg::kAccBufs;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem_a + kMxStages * kMxAStageBytes;
  uint8_t* smem_sf = smem_b + kMxStages * kMxBStageBytes;
  MxAux* aux = reinterpret_cast<MxAux*>(smem_sf + kMxSfSlots * kMxSfSlotBytes);
  volatile int* abort_flag = &aux->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();                 // 0 = leader of the pair
  const int32_t cluster_id = int32_t(blockIdx.x >> 1);
  const int32_t num_clusters = int32_t(gridDim.x >> 1);
  const int32_t num_tiles = p.batch * p.num_m_tiles * p.num_n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMxStages; ++s) {
      mbar_init(&aux->full_bar[s], 1);        // the leader's producer, with the byte count of both CTAs' loads
      mbar_init(&aux->empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&aux->acc_full_bar[b], 1);
      mbar_init(&aux->acc_empty_bar[b], 2 * kMxEpilogueWarps);
    }
    for (int s = 0; s < kMxSfSlots; ++s) {
      mbar_init(&aux->raw_full_bar[s], 1);
      mbar_init(&aux->sf_full_bar[s], 2);     // one scale loader per CTA
      mbar_init(&aux->sf_empty_bar[s], 1);
    }
    aux->abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(&aux->tmem_base, kMxTmemCols);
    tmem_relinquish_alloc_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                         // the peer's barriers exist before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = aux->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long prod_wait = 0;
      for (int32_t tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        int32_t mt, nt, bt;
        mx_tile_coords(tile, p, &mt, &nt, &bt);
        const int32_t row0 = mt * kMxTileM + int32_t(rank) * kMxBM;
        const int32_t col0 = nt * kMxBN + int32_t(rank) * (kMxBN / 2);
        for (int32_t kb = 0; kb < p.num_k_blocks; ++kb) {
          const long long tw = (kTiming && p.timing) ? clock64() : 0;
          ok = mbar_wait(&aux->empty_bar[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout);
          if (kTiming && p.timing) prod_wait += clock64() - tw;
          if (!ok) break;
          // Both CTAs' loads count on the leader's barrier; the leader announces the bytes of both.
          if (rank == 0) mbar_arrive_expect_tx(&aux->full_bar[stage], 2 * (kMxAStageBytes + kMxBStageBytes));
          const uint32_t full = map_to_cta(&aux->full_bar[stage], 0);
          tma_load_3d_pair(smem_a + stage * kMxAStageBytes, &tmap_a, full, kb * kMxBK, row0, bt);
          tma_load_3d_pair(smem_b + stage * kMxBStageBytes, &tmap_b, full, kb * kMxBK, col0, bt);
          if (++stage == kMxStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (kTiming && p.timing) p.timing[blockIdx.x * kMxTimingSlots + 3] = prod_wait;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && elect_one()) {
      const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem_a), 16384, 1024);
      const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(smem_b), 16384, 1024);
      const uint64_t sf_desc0 = make_smem_desc_noswizzle(smem_u32(smem_sf), 128);
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0, set = 0;
      int acc = 0;
      uint32_t sf_group = 0;                     // groups of four k-blocks taken from the scale ring so far
      bool ok = true;
      const bool timed = kTiming && p.timing != nullptr;
      const long long t_begin = timed ? clock64() : 0;
      long long wait_full = 0, wait_acc = 0, wait_sf = 0;
      for (int32_t tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const long long ta = timed ? clock64() : 0;
        ok = mbar_wait(&aux->acc_empty_bar[acc], acc_phase ^ 1, abort_flag, p.status, kStatusMmaTimeout);
        if (timed) wait_acc += clock64() - ta;
        if (!ok) break;
        tc_fence_after_sync();
        for (int32_t kb = 0; kb < p.num_k_blocks; ++kb) {
          const uint32_t sf_slot = sf_group % kMxSfSlots;
          if ((kb & 3) == 0) {                   // a new group of scales
            const long long tq = timed ? clock64() : 0;
            ok = mbar_wait(&aux->sf_full_bar[sf_slot], (sf_group / kMxSfSlots) & 1, abort_flag, p.status, kStatusMmaTimeout);
            if (timed) wait_sf += clock64() - tq;
            if (!ok) break;
          }
          const long long tf = timed ? clock64() : 0;
          ok = mbar_wait(&aux->full_bar[stage], phase, abort_flag, p.status, kStatusMmaTimeout);
          if (timed) wait_full += clock64() - tf;
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t a_desc = a_desc0 + uint64_t((stage * kMxAStageBytes) >> 4);
          const uint64_t b_desc = b_desc0 + uint64_t((stage * kMxBStageBytes) >> 4);
          const uint64_t sf_desc = sf_desc0 + uint64_t((sf_slot * kMxSfSlotBytes + uint32_t(kb & 3) * kMxSfStageBytes) >> 4);
          const uint32_t sfa_t = tmem_base + Cfg::kTmemSfa + Cfg::kTmemSfaSet * set;
          const uint32_t sfb_t = tmem_base + Cfg::kTmemSfb + Cfg::kTmemSfbSet * set;
          tmem_cp_32x128b_pair(sfa_t, sf_desc);                                             // A rows of this CTA
          tmem_cp_32x128b_pair(sfb_t, sf_desc + uint64_t(kMxSfaStageBytes >> 4));           // B rows 0-127
          tmem_cp_32x128b_pair(sfb_t + 4, sf_desc + uint64_t((kMxSfaStageBytes + kMxSfBlockBytes) >> 4));   // B rows 128-255
#pragma unroll
          for (int j = 0; j < kMxBK / kMxUmmaK; ++j) {
            const uint32_t accumulate = (kb > 0 || j > 0) ? 1u : 0u;
            umma_mxf8_pair(tmem_base + uint32_t(acc * Cfg::kTmemAccStride), a_desc + uint64_t((j * kMxUmmaK) >> 4), b_desc + uint64_t((j * kMxUmmaK) >> 4),
                           idesc_mx_with_scale_byte(p.idesc, uint32_t(j)), sfa_t, sfb_t, accumulate);
          }
          // The stage may be refilled once these copies and MMAs have read it -- in both CTAs.
          umma_commit_pair(map_to_cta(&aux->empty_bar[stage], 0));
          umma_commit_pair(map_to_cta(&aux->empty_bar[stage], 1));
          if ((kb & 3) == 3 || kb == p.num_k_blocks - 1) {       // the group's scales have been copied out -- in both CTAs
            umma_commit_pair(map_to_cta(&aux->sf_empty_bar[sf_slot], 0));
            umma_commit_pair(map_to_cta(&aux->sf_empty_bar[sf_slot], 1));
            ++sf_group;
          }
          set ^= 1;
          if (++stage == kMxStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(map_to_cta(&aux->acc_full_bar[acc], 0));     // accumulator complete (each CTA has its rows)
        umma_commit_pair(map_to_cta(&aux->acc_full_bar[acc], 1));
        if (++acc == kAccBufs) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
      if (timed) {
        p.timing[blockIdx.x * kMxTimingSlots + 0] = wait_full;
        p.timing[blockIdx.x * kMxTimingSlots + 1] = wait_acc;
        p.timing[blockIdx.x * kMxTimingSlots + 2] = clock64() - t_begin;
        p.timing[blockIdx.x * kMxTimingSlots + 10] = wait_sf;
      }
    }
  } else if (warp == 2 || warp == 3) {
    // ------------------------------------------------------------------ scale loader
    // Works in groups of four k-blocks, one group per slot of a ring of kMxSfSlots.  A slot goes
    // free -> box requested -> box landed -> rearranged (sf_full) -> read by tcgen05.cp -> free (sf_empty).
    // Bulk path: lane 0 keeps boxes in flight (16 scale bytes = four k-blocks of each of this CTA's
    // 128 A rows and of the tile's 256 B rows, row after row); when one has landed every lane
    // reads the 16 bytes of its twelve rows and, once all lanes have read, writes them back into the
    // same slot in the layout tcgen05.cp wants.  Gather path (rows of scales that do not start on
    // 16-byte boundaries): the lanes fetch the bytes themselves.
    // Warps 2 and 3 take alternate groups, so each has eight k-blocks' worth of time for one group.
    const uint32_t groups_per_tile = uint32_t(p.num_k_blocks + 3) / 4;
    const uint32_t my_tiles = cluster_id < num_tiles ? uint32_t(num_tiles - cluster_id + num_clusters - 1) / uint32_t(num_clusters) : 0u;
    const uint32_t total_groups = my_tiles * groups_per_tile;
    const uint32_t first_group = uint32_t(warp - 2);
    uint32_t gi_issue = first_group;                        // next group whose box lane 0 asks for (bulk path)
    bool ok = true;
    const bool timed = kTiming && p.timing != nullptr;
    long long sf_wait_box = 0, sf_wait_slot = 0, sf_work = 0;
    if (lane == 0 && p.sf_bulk_ok) {
      tma_prefetch_desc(&tmap_sfa);
      tma_prefetch_desc(&tmap_sfb);
    }
    for (uint32_t gi = first_group; gi < total_groups && ok; gi += 2) {
      {
        const uint32_t slot = gi % kMxSfSlots;
        const uint32_t use = gi / kMxSfSlots;
        const uint32_t slot_addr = smem_u32(smem_sf) + slot * kMxSfSlotBytes + uint32_t(lane) * 16;
        uint32_t w[12][4];
        if (p.sf_bulk_ok) {
          if (lane == 0) {
            while (gi_issue < total_groups && gi_issue - gi < uint32_t(kMxSfSlots)) {
              const uint32_t islot = gi_issue % kMxSfSlots;
              const uint32_t ipar = ((gi_issue / kMxSfSlots) & 1) ^ 1;
              const long long ts = timed ? clock64() : 0;
              if (gi_issue != gi) {              // this group's own box is already on its way: do not stall on a slot still in use
                if (!mbar_try_wait(&aux->sf_empty_bar[islot], ipar)) break;
              } else {
                ok = mbar_wait(&aux->sf_empty_bar[islot], ipar, abort_flag, p.status, kStatusProducerTimeout);
                if (!ok) break;
              }
              if (timed) sf_wait_slot += clock64() - ts;
              int32_t imt, int_, ibt;
              mx_tile_coords(cluster_id + int32_t(gi_issue / groups_per_tile) * num_clusters, p, &imt, &int_, &ibt);
              const int32_t igrp = int32_t(gi_issue % groups_per_tile);
              uint8_t* raw = smem_sf + islot * kMxSfSlotBytes;
              mbar_arrive_expect_tx(&aux->raw_full_bar[islot], kMxRawSfaBytes + Cfg::kRawSfbBytes);
              tma_load_3d(raw, &tmap_sfa, &aux->raw_full_bar[islot], igrp * 16, imt * kMxTileM + int32_t(rank) * kMxBM, ibt);
              tma_load_3d(raw + kMxRawSfaBytes, &tmap_sfb, &aux->raw_full_bar[islot], igrp * 16, int_ * kMxBN, ibt);
              gi_issue += 2;
            }
            if (ok) {
              const long long tb = timed ? clock64() : 0;
              ok = mbar_wait(&aux->raw_full_bar[slot], use & 1, abort_flag, p.status, kStatusProducerTimeout);
              if (timed) sf_wait_box += clock64() - tb;
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
          (void)mbar_try_wait(&aux->raw_full_bar[slot], use & 1);   // every lane observes the phase
#pragma unroll
          for (int g = 0; g < 12; ++g) {      // row lane + 32 g of the box: g 0-3 rows of A, g 4-11 rows of B
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[g][0]), "=r"(w[g][1]), "=r"(w[g][2]), "=r"(w[g][3])
                         : "r"(slot_addr + uint32_t(g) * 512)
                         : "memory");
          }
          __syncwarp();                        // every lane has read the box before anyone overwrites it
        } else {
          const long long ts = timed ? clock64() : 0;
          if (lane == 0) ok = mbar_wait(&aux->sf_empty_bar[slot], (use & 1) ^ 1, abort_flag, p.status, kStatusProducerTimeout);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (timed) sf_wait_slot += clock64() - ts;
          if (!ok) break;
          int32_t mt, nt, bt;
          mx_tile_coords(cluster_id + int32_t(gi / groups_per_tile) * num_clusters, p, &mt, &nt, &bt);
          const int64_t a_row0 = int64_t(mt) * kMxTileM + int64_t(rank) * kMxBM + lane;
          const int64_t b_row0 = int64_t(nt) * kMxBN + lane;
          const uint8_t* sfa_b = p.sfa + int64_t(bt) * p.sfa_batch;
          const uint8_t* sfb_b = p.sfb + int64_t(bt) * p.sfb_batch;
          const int64_t col0 = int64_t(gi % groups_per_tile) * 16;
#pragma unroll
          for (int g = 0; g < 12; ++g) {
            const bool is_a = g < 4;
            const int64_t row = is_a ? a_row0 + 32 * g : b_row0 + 32 * (g - 4);
            const bool valid = row < (is_a ? p.m : p.n);
            const uint8_t* src = (is_a ? sfa_b : sfb_b) + (valid ? row * (is_a ? p.sfa_ld : p.sfb_ld) + col0 : 0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t v = 0;
              if (valid && col0 + 4 * j < p.scale_cols) {
                if (p.sf_words_ok) {
                  v = __ldg(reinterpret_cast<const uint32_t*>(src + 4 * j));
                } else {
#pragma unroll
                  for (int b = 0; b < 4; ++b) {
                    if (col0 + 4 * j + b < p.scale_cols) v |= uint32_t(__ldg(src + 4 * j + b)) << (8 * b);
                  }
                }
              }
              w[g][j] = v;
            }
          }
        }
        const long long tw = timed ? clock64() : 0;
        // Slot layout read by the issuer: k-block j at j * 1536; there the A rows' block, then the two B blocks;
        // in a block this lane's 16 bytes are the j-th words of its four rows.
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int blk = 0; blk < 3; ++blk) {
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(slot_addr + uint32_t(j) * kMxSfStageBytes + uint32_t(blk) * kMxSfBlockBytes),
                         "r"(w[4 * blk][j]), "r"(w[4 * blk + 1][j]), "r"(w[4 * blk + 2][j]), "r"(w[4 * blk + 3][j])
                         : "memory");
          }
        }
        fence_proxy_async_smem();              // the tensor core reads these bytes through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(&aux->sf_full_bar[slot], 0));
        if (timed) sf_work += clock64() - tw;
      }
    }
    if (timed && lane == 0 && warp == 2) {
      p.timing[blockIdx.x * kMxTimingSlots + 4] = sf_wait_box;
      p.timing[blockIdx.x * kMxTimingSlots + 5] = sf_wait_slot;
      p.timing[blockIdx.x * kMxTimingSlots + 6] = sf_work;
    }
    if (!ok && lane == 0 && p.sf_bulk_ok) {
      // Abort path: let boxes that were already requested land before the CTA's memory is released.
      for (int sl = 0; sl < kMxSfSlots; ++sl) {
        for (int i = 0; i < 100000 && !mbar_try_wait(&aux->raw_full_bar[sl], 0) && !mbar_try_wait(&aux->raw_full_bar[sl], 1); ++i) {
        }
      }
    }
  } else if (warp >= kMxFirstEpilogueWarp) {
    // ------------------------------------------------------------------ epilogue (warps 4..11)
    const int q = warp & 3;                               // TMEM lane quarter this warp may access
    const int col_half = (warp - kMxFirstEpilogueWarp) >> 2;
    const uint32_t t_addr0 = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(col_half * 128);
    uint32_t acc_phase = 0;
    int acc = 0;
    bool ok = true;
    const bool timed = kTiming && p.timing != nullptr;
    long long ep_wait = 0, ep_read = 0, ep_store = 0;
    for (int32_t tile = cluster_id; tile < num_tiles; tile += num_clusters) {
      int32_t mt, nt, bt;
      mx_tile_coords(tile, p, &mt, &nt, &bt);
      const long long t0 = timed ? clock64() : 0;
      if (lane == 0) ok = mbar_wait(&aux->acc_full_bar[acc], acc_phase, abort_flag, p.status, kStatusEpilogueTimeout);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      const long long t1 = timed ? clock64() : 0;
      if (!ok) break;
      (void)mbar_try_wait(&aux->acc_full_bar[acc], acc_phase);     // every lane observes the completed phase
      const uint32_t t_addr = t_addr0 + uint32_t(acc * Cfg::kTmemAccStride);
      const bool four = col_half == 0 || Cfg::kColsHalf1 == 128;      // this warp's group has 128 columns (else 96)
      tc_fence_after_sync();
      uint32_t r0[32], r1[32], r2[32], r3[32];
      tmem_ld_32x32(t_addr, r0);
      tmem_ld_32x32(t_addr + 32, r1);
      tmem_ld_32x32(t_addr + 64, r2);
      if (four) tmem_ld_32x32(t_addr + 96, r3);
      tmem_ld_wait_for(r0);
      tmem_ld_wait_for(r1);
      tmem_ld_wait_for(r2);
      if (four) tmem_ld_wait_for(r3);
      // The accumulator is in registers: the issuer may start the next tile.
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank != 0) mbar_arrive_cluster(map_to_cta(&aux->acc_empty_bar[acc], 0));
        else mbar_arrive(&aux->acc_empty_bar[acc]);
      }
      if (++acc == kAccBufs) {
        acc = 0;
        acc_phase ^= 1;
      }
      const long long t2 = timed ? clock64() : 0;
      const int64_t row = int64_t(mt) * kMxTileM + int64_t(rank) * kMxBM + q * 32 + lane;
      if (row < p.m) {
        const int64_t row_off = (int64_t(bt) * p.m + row) * p.n;
        const int32_t col = nt * kMxBN + col_half * 128;
        mx_store_chunk(p, row_off, col, r0);
        mx_store_chunk(p, row_off, col + 32, r1);
        mx_store_chunk(p, row_off, col + 64, r2);
        if (four) mx_store_chunk(p, row_off, col + 96, r3);
      }
      if (timed) {
        ep_wait += t1 - t0;
        ep_read += t2 - t1;
        ep_store += clock64() - t2;
      }
    }
    if (timed && warp == kMxFirstEpilogueWarp && lane == 0) {
      p.timing[blockIdx.x * kMxTimingSlots + 7] = ep_wait;
      p.timing[blockIdx.x * kMxTimingSlots + 8] = ep_read;
      p.timing[blockIdx.x * kMxTimingSlots + 9] = ep_store;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();      // nobody leaves while the peer may still read this CTA's shared memory
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kMxTmemCols);
  }
}

}  // namespace

// ----------------------------------------------------------------------------- host side
Status InitMxKernels() {
  cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(mx_gemm_kernel<256>),
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, int(MxSmemBytes<256>()));
  if (e == cudaSuccess) e = cudaFuncSetAttribute(reinterpret_cast<const void*>(mx_gemm_kernel<224>),
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, int(MxSmemBytes<224>()));
  if (e != cudaSuccess) return Status::Error(kInternal, std::string("cudaFuncSetAttribute(mx): ") + cudaGetErrorString(e));
  return Status::Ok();
}

#if B200SD_TUNING
// Copies the tuning counters of the last block-scaled launch on the current device (kMxTimingSlots per CTA).
extern "C" int b200sd_debug_read_mx_timing(unsigned long long* out, int count) {
  cudaDeviceSynchronize();
  return int(cudaMemcpyFromSymbol(out, g_mx_timing, sizeof(unsigned long long) * size_t(count)));
}
#endif

Status ValidateMx(const MxProblem& g) {
  auto f8 = [](int32_t t) { return t == kF8E4M3FN || t == kF8E5M2; };
  if (!f8(g.a_dtype) || !f8(g.b_dtype)) {
    return Status::Error(kUnimplemented, "block-scaled dot: operands must be f8e4m3fn or f8e5m2 (4- and 6-bit MX element types are not implemented)");
  }
  if (g.scale_dtype != kF8E8M0FNU) return Status::Error(kUnimplemented, "block-scaled dot: scales must be f8e8m0fnu (block size 32)");
  if (g.d_dtype != kF32 && g.d_dtype != kBF16 && g.d_dtype != kF16) {
    return Status::Error(kInvalidArgument, "block-scaled dot: the result must be f32, bf16 or f16");
  }
  if (g.m <= 0 || g.n <= 0 || g.k <= 0 || g.batch < 0) return Status::Error(kInvalidArgument, "block-scaled dot: empty or negative dimension");
  if (g.k % 32 != 0) return Status::Error(kInvalidArgument, "block-scaled dot: the contracting dimension must be a multiple of the block size 32");
  if (g.a_scale_rows < 0 || g.a_scale_cols < 0 || g.b_scale_rows < 0 || g.b_scale_cols < 0 ||
      (g.a_scale_rows > 0 && g.a_scale_rows < g.m) || (g.b_scale_rows > 0 && g.b_scale_rows < g.n) ||
      (g.a_scale_cols > 0 && g.a_scale_cols < g.k / 32) || (g.b_scale_cols > 0 && g.b_scale_cols < g.k / 32))
    return Status::Error(kInvalidArgument, "block-scaled dot: padded scale extents must cover [rows, k / 32]");
  if (g.kernel != kKernelAuto && g.kernel != kKernelMxPair256 && g.kernel != kKernelMxPair224)
    return Status::Error(kInvalidArgument, "block-scaled dot: kernel must be AUTO, MX_256 or MX_224");
  if (g.m >= (1ll << 31) || g.n >= (1ll << 31) || g.k >= (1ll << 31)) return Status::Error(kInvalidArgument, "block-scaled dot: dimension too large");
  return Status::Ok();
}

Status LaunchMx(const MxProblem& g, cudaStream_t stream, LaunchStats* stats) {
  Status st = ValidateMx(g);
  if (!st.ok()) return st;
  int device = 0;
  cudaGetDevice(&device);
  st = InitDevice(device);
  if (!st.ok()) return st;
  const int max_pairs = MaxPairClusters();
  if (max_pairs <= 0) return Status::Error(kFailedPrecondition, "this device cannot co-schedule the CTA pairs the block-scaled kernel runs as");
  if (g.a == nullptr || g.b == nullptr || g.a_scale == nullptr || g.b_scale == nullptr || g.d == nullptr) {
    return Status::Error(kInvalidArgument, "block-scaled dot: null operand, scale or result pointer");
  }
  const int64_t batch = g.batch > 0 ? g.batch : 1;
  CUtensorMap tmap_a, tmap_b;
  st = MakeBatchedByteMatrixMap(&tmap_a, g.a, batch, g.m, g.k, kMxBK, kMxBM);          // [m, k], box 128(k) x 128(m)
  if (!st.ok()) return st;
  // Tile width.  Measured (bf16 result): 8192^3 398 us with 256-column tiles against 415 us with 224 (16 rounds instead
  // of 14, and 14 % more A traffic per flop on a kernel whose limit is the shared-memory fill rate); 4096^3 62.8 against
  // 68.1; 2048 x 8192 x 4096, where both widths need four rounds, 80.1 against 74.6.  The accumulator read-out that
  // the second accumulator hides costs the 256-column form about 800 cycles per tile in the end (the MMAs already
  // queued cover the rest); the narrower tile costs 8 % per flop.
  const int max_clusters = max_pairs;
  auto rounds = [&](int bn) {
    const int64_t t = batch * ((g.m + kMxTileM - 1) / kMxTileM) * ((g.n + bn - 1) / bn);
    return double((t + max_clusters - 1) / max_clusters);
  };
  const double k_cycles = 512.0 * double((g.k + kMxBK - 1) / kMxBK);
  const double cost256 = rounds(256) * (k_cycles + 800.0), cost224 = rounds(224) * k_cycles * (224.0 / 256.0) * 1.08;
  // A tuned table entry for exactly this shape (single dots only) wins over the cost estimate.
  const int want = g.kernel != kKernelAuto ? g.kernel : (batch == 1 ? TunedMxKernel(g.m, g.n, g.k) : kKernelAuto);
  const int bn = want == kKernelMxPair256 ? 256 : want == kKernelMxPair224 ? 224 : (cost224 < cost256 ? 224 : 256);
  st = MakeBatchedByteMatrixMap(&tmap_b, g.b, batch, g.n, g.k, kMxBK, uint32_t(bn / 2));      // [n, k], box 128(k) x 128|112(n)
  if (!st.ok()) return st;

  MxArgs p{};
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.scale_cols = g.k / 32;
  // Padded scale arrays: only the leading [rows, k / 32] corner is read, the rest is stepped over.
  p.sfa_ld = g.a_scale_cols > 0 ? g.a_scale_cols : p.scale_cols;
  p.sfb_ld = g.b_scale_cols > 0 ? g.b_scale_cols : p.scale_cols;
  p.sfa_batch = (g.a_scale_rows > 0 ? g.a_scale_rows : g.m) * p.sfa_ld;
  p.sfb_batch = (g.b_scale_rows > 0 ? g.b_scale_rows : g.n) * p.sfb_ld;
  // Scale rows that start on 16-byte boundaries can be fetched as TMA boxes of 16 bytes x 128 / 256 rows (the map's
  // extents are the corner in use, so padding reads as zero like everything else outside it).
  p.sf_bulk_ok = (p.sfa_ld % 16 == 0 && p.sfb_ld % 16 == 0 && p.sfa_batch % 16 == 0 && p.sfb_batch % 16 == 0 &&
                  (reinterpret_cast<uintptr_t>(g.a_scale) & 15) == 0 && (reinterpret_cast<uintptr_t>(g.b_scale) & 15) == 0) ? 1 : 0;
  CUtensorMap tmap_sfa = tmap_a, tmap_sfb = tmap_b;       // placeholders the gather path never touches
  if (p.sf_bulk_ok) {
    st = MakeBatchedPlainByteMap(&tmap_sfa, g.a_scale, batch, g.m, p.scale_cols, p.sfa_ld, p.sfa_batch, 16, kMxBM);
    if (!st.ok()) return st;
    st = MakeBatchedPlainByteMap(&tmap_sfb, g.b_scale, batch, g.n, p.scale_cols, p.sfb_ld, p.sfb_batch, 16, uint32_t(bn));
    if (!st.ok()) return st;
  }
  p.batch = int32_t(batch);
  p.num_m_tiles = int32_t((g.m + kMxTileM - 1) / kMxTileM);
  p.num_n_tiles = int32_t((g.n + bn - 1) / bn);
  p.num_k_blocks = int32_t((g.k + kMxBK - 1) / kMxBK);
  const int64_t tiles = batch * p.num_m_tiles * p.num_n_tiles;
  if (tiles > (1ll << 30)) return Status::Error(kInvalidArgument, "block-scaled dot: too many tiles");
  p.raster_group = 16;
  p.idesc = make_idesc_mx(g.a_dtype == kF8E5M2 ? 1u : 0u, g.b_dtype == kF8E5M2 ? 1u : 0u, kMxTileM, uint32_t(bn));
  p.sfa = static_cast<const uint8_t*>(g.a_scale);
  p.sfb = static_cast<const uint8_t*>(g.b_scale);
  p.sf_words_ok = (p.scale_cols % 4 == 0 && p.sfa_ld % 4 == 0 && p.sfb_ld % 4 == 0 && (reinterpret_cast<uintptr_t>(g.a_scale) & 3) == 0 &&
                   (reinterpret_cast<uintptr_t>(g.b_scale) & 3) == 0) ? 1 : 0;
  p.alpha = g.alpha;
  p.d = g.d;
  p.d_dtype = g.d_dtype;
  const int64_t d_elt = g.d_dtype == kF32 ? 4 : 2;
  p.vec_store_ok = ((reinterpret_cast<uintptr_t>(g.d) & 15) == 0 && (g.n * d_elt) % 16 == 0) ? 1 : 0;
  p.status = StatusWordPtr();
  p.timing = nullptr;
#if B200SD_TUNING
  static const bool timing_on = TuningEnvInt("B200SD_TIMING", 0) == 1;
  if (timing_on) {
    cudaGetSymbolAddress(reinterpret_cast<void**>(&p.timing), g_mx_timing);
    cudaMemsetAsync(p.timing, 0, sizeof(unsigned long long) * kMxTimingSlots * 512, stream);
  }
#endif

  const int grid = 2 * int(tiles < max_pairs ? tiles : max_pairs);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kMxThreads, 1, 1);
  cfg.dynamicSmemBytes = bn == 224 ? MxSmemBytes<224>() : MxSmemBytes<256>();
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = bn == 224 ? cudaLaunchKernelEx(&cfg, mx_gemm_kernel<224>, tmap_a, tmap_b, tmap_sfa, tmap_sfb, p)
                                  : cudaLaunchKernelEx(&cfg, mx_gemm_kernel<256>, tmap_a, tmap_b, tmap_sfa, tmap_sfb, p);
  if (e != cudaSuccess) return Status::Error(kInternal, std::string("mx_gemm_kernel launch: ") + cudaGetErrorString(e));
  if (stats) {
    stats->kernel = bn == 224 ? kKernelMxPair224 : kKernelMxPair256;
    stats->grid = grid;
    stats->launches = 1;
  }
  return Status::Ok();
}

}  // namespace b200sd
