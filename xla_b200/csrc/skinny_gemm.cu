// Decode-shaped FP8 scaled dot for sm_100a: D[m,n] = (a_scale*b_scale) * A[m,k] . W[k,n] with
// m <= 128 rows of activations and a weight matrix that is read from HBM exactly once.  The same
// `__cublas$lt$matmul$f8` call (xla/stream_executor/cuda/cuda_blas_lt.cc:559-564) in the regime
// where it is bound by memory bandwidth.
//
// The roles of the operands are swapped so that W fills the 128-row side of the tensor-core
// instruction: D^T[128 n, m] = W^T . A^T, with W taken MN-major straight from its row-major [k,n]
// storage and A as the (narrow) N operand.  A CTA works on a "strip" of `n_sub` adjacent 128-column
// tiles at once (n_sub accumulators), so that every k-row it fetches is n_sub*128 contiguous
// bytes of W -- long enough runs for the DRAM pages to be used well.  Work is split stream-K
// style: the (strip, k-block) units are dealt out evenly to one persistent CTA per SM, so every SM
// streams the same number of W bytes.  A CTA whose range ends inside a strip computes that piece
// FIRST, writes the f32 partial to the caller's workspace and raises a flag; the CTA that owns
// the strip's last k-block adds the partials of the (lower-numbered) CTAs before it and writes D.
// Waiting therefore only ever targets CTAs that were scheduled earlier and finished that piece
// long ago; the wait is bounded all the same.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <random>
#include <string>

#include "../../include/b200_scaled_dot.h"
#include "kernels.h"
#include "ptx.cuh"

namespace b200sd {
namespace {

constexpr int kTileN = 128;        // weight columns per accumulator (= TMEM lanes)
constexpr int kBK = 128;           // k per stage
constexpr int kUmmaK = 32;
constexpr int kMaxStages = 12;
constexpr int kMaxSub = 4;
constexpr int kWBoxBytes = kBK * kTileN;     // 16 KiB per 128-column tile per stage
constexpr int kThreads = 320;            // producer warp, MMA warp, eight epilogue warps
constexpr int kAccBufs = 2;
constexpr int kTmemCols = 512;
constexpr int kMaxCtas = 160;
constexpr size_t kFlagBytes = size_t(kMaxCtas) * 8 * sizeof(uint64_t);   // one flag per CTA per epilogue warp
constexpr size_t kSmemBudget = 227 * 1024;

struct __align__(16) SkinnyAux {
  uint64_t full_bar[kMaxStages];
  uint64_t empty_bar[kMaxStages];
  uint64_t acc_full_bar[kAccBufs];
  uint64_t acc_empty_bar[kAccBufs];
  uint32_t tmem_base;
  int abort_flag;
};

struct SkinnyArgs {
  int32_t m;                 // activation rows (multiple of 16, <= 128)
  int64_t n, k;
  int32_t n_sub;             // 128-column tiles per CTA per strip
  int32_t group;             // CTAs that walk the same unit range side by side
  int32_t stages;
  int32_t a_stage_bytes;     // m * 128 rounded up to 1 KiB
  int32_t num_strips, num_k_blocks;
  int64_t total_units;       // num_strips * num_k_blocks
  uint32_t idesc;
  const float* a_scale;
  const float* b_scale;
  float alpha;
  void* d;
  int32_t d_dtype;
  uint64_t* flags;           // [grid][8]; a flag is raised by storing this launch's epoch
  uint64_t epoch;            // unique per launch, so stale or foreign workspace contents never look raised
  float* partials;           // [grid][n_sub][m][128]
  uint32_t* status;
  unsigned long long* timing;   // optional per-CTA wait counters (tuning aid), else nullptr
};

// Tuning aid, 8 counters per CTA: [0] cycles the MMA issuer waited for operands, [1] for a free
// accumulator, [2] its total cycles, [3] cycles the producer waited for a free stage, [4] the CTA's
// wall time in ns, [5] time the first operands landed, [6] cycles epilogue warp 2 was busy, [7] CTA exit time.
// Tuning builds only; filled when B200SD_TIMING=1.
#if B200SD_TUNING
__device__ unsigned long long g_skinny_timing[16 * 256];
#endif

__device__ __forceinline__ int64_t unit_begin(int64_t cta, int64_t total, int64_t grid) { return cta * total / grid; }

__device__ __forceinline__ uint64_t ld_acquire_gpu(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint64_t* p, uint64_t v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void store_out(const SkinnyArgs& p, int64_t idx, float x) {
  if (p.d_dtype == kBF16) {
    static_cast<__nv_bfloat16*>(p.d)[idx] = __float2bfloat16_rn(x);
  } else if (p.d_dtype == kF16) {
    static_cast<__half*>(p.d)[idx] = __float2half_rn(x);
  } else {
    static_cast<float*>(p.d)[idx] = x;
  }
}

__global__ void __launch_bounds__(kThreads, 1)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                   const SkinnyArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int w_stage_bytes = p.n_sub * kWBoxBytes;
  const int stage_bytes = w_stage_bytes + p.a_stage_bytes;
  SkinnyAux* aux = reinterpret_cast<SkinnyAux*>(smem + p.stages * stage_bytes);
  volatile int* abort_flag = &aux->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // CTAs work in lock-step groups of `p.group`: the members of a group walk the same range of
  // (strip, k-block) units, member j on the j-th tile set of each strip, so that at any moment they
  // fetch neighbouring 128-byte pieces of the same rows of W (long contiguous runs for the DRAM).
  const int64_t cta = blockIdx.x;                      // physical CTA: owns workspace slot and flags
  const int64_t side = cta % p.group;                  // position inside the group
  const int64_t member = cta / p.group;                // which unit range
  const int64_t grid = gridDim.x / p.group;            // number of unit ranges
  const int64_t u_begin = unit_begin(member, p.total_units, grid);
  const int64_t u_end = unit_begin(member + 1, p.total_units, grid);
  const uint32_t stage_tx_bytes = uint32_t(w_stage_bytes) + uint32_t(p.m) * kBK;
  const int acc_cols = p.n_sub * p.m;            // TMEM columns of one accumulator set
  // Eight epilogue warps split the m columns in two halves when that leaves whole 16-column
  // chunks; otherwise four warps take all columns and the other four stay out of the way.
  const int ep_halves = (p.m % 32 == 0) ? 2 : 1;
  const int cols_per_warp = p.m / ep_halves;
  if (kTiming && p.timing && threadIdx.x == 64) p.timing[blockIdx.x * 16 + 1] = global_timer_ns();
  // Programmatic dependent launch: the kernel behind this one in the stream may be scheduled as this one's CTAs
  // retire; every role of this kernel sets itself up first and passes griddep_wait() before it touches global
  // memory, so the set-up overlaps the tail of the kernel in front.
  if (threadIdx.x == 0) griddep_launch_dependents();

  // The CTA walks its unit range [u_begin, u_end) backwards, one strip-segment at a time:
  //   segment = units of one strip, [max(u_begin, strip*KB), min(u_end, (strip+1)*KB)).
  // All three roles derive the same segment sequence from these two numbers.
  const int64_t kb_per_strip = p.num_k_blocks;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // Starts streaming before the rest of the CTA has finished setting up: it only needs its
    // own barriers, which it initialises itself.
    if (lane == 0) {
      for (int s = 0; s < p.stages; ++s) {
        mbar_init(&aux->full_bar[s], 1);
        mbar_init(&aux->empty_bar[s], 1);
      }
      for (int b = 0; b < kAccBufs; ++b) {
        mbar_init(&aux->acc_full_bar[b], 1);
        mbar_init(&aux->acc_empty_bar[b], 4 * ep_halves);
      }
      aux->abort_flag = 0;
      fence_mbar_init();
      fence_proxy_async_smem();
    }
    __syncwarp();
    named_bar_arrive(1, kThreads);               // barriers are ready: release the other warps
    if (elect_one()) {
      tma_prefetch_desc(&tmap_w);
      tma_prefetch_desc(&tmap_a);
      griddep_wait();                                         // operands may be the previous kernel's results
      const uint64_t stream_once = l2_policy_evict_first();   // W passes through L2 exactly once
      const uint64_t keep = l2_policy_evict_last();           // A is re-read by every CTA
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long prod_wait = 0;
      int64_t seg_end = u_end;
      while (seg_end > u_begin && ok) {
        const int64_t strip = (seg_end - 1) / kb_per_strip;
        const int64_t seg_begin = max(u_begin, strip * kb_per_strip);
        for (int64_t u = seg_begin; u < seg_end; ++u) {
          const int32_t kb = int32_t(u - strip * kb_per_strip);
          const long long tw = (kTiming && p.timing) ? clock64() : 0;
          ok = mbar_wait(&aux->empty_bar[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout);
          if (kTiming && p.timing) prod_wait += clock64() - tw;
          if (!ok) break;
          uint64_t* full = &aux->full_bar[stage];
          mbar_arrive_expect_tx(full, stage_tx_bytes);
          uint8_t* sw = smem + stage * stage_bytes;
          for (int s = 0; s < p.n_sub; ++s)
            tma_load_2d_hint(sw + s * kWBoxBytes, &tmap_w, full, int32_t((strip * p.group + side) * p.n_sub + s) * kTileN, kb * kBK,
                             stream_once);
          tma_load_2d_hint(sw + w_stage_bytes, &tmap_a, full, kb * kBK, 0, keep);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        seg_end = seg_begin;
      }
      if (kTiming && p.timing) p.timing[blockIdx.x * 16 + 3] = prod_wait;
      if (!ok) {
        for (int s = 0; s < p.stages; ++s) {
          for (int i = 0; i < 100000 && !mbar_try_wait(&aux->full_bar[s], 0) && !mbar_try_wait(&aux->full_bar[s], 1); ++i) {
          }
        }
      }
    }
  } else {
    if (warp == 1) {
      tmem_alloc(&aux->tmem_base, kTmemCols);
      tmem_relinquish_alloc();
      tc_fence_before_sync();
    }
    named_bar_sync(1, kThreads);                 // barriers initialised (warp 0) and TMEM allocated (warp 1)
    tc_fence_after_sync();
    const uint32_t tmem_base = aux->tmem_base;
    griddep_wait();                              // from here on: scales, flags, partials and D in global memory

    if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (elect_one()) {
        const uint64_t w_desc0 = make_smem_desc_sw128(smem_u32(smem), 16384, 1024);                    // MN-major
        const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem + w_stage_bytes), 16, 1024);       // K-major
        const uint32_t w_kstep = (kUmmaK * 128) >> 4;
        const uint32_t a_kstep = kUmmaK >> 4;
        const long long t_begin = (kTiming && p.timing) ? clock64() : 0;
        const unsigned long long ns_begin = (kTiming && p.timing) ? global_timer_ns() : 0;
        long long wait_full = 0, wait_acc = 0;
        unsigned long long first_data_ns = 0;
        int stage = 0;
        uint32_t phase = 0;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        int64_t seg_end = u_end;
        while (seg_end > u_begin && ok) {
          const int64_t strip = (seg_end - 1) / kb_per_strip;
          const int64_t seg_begin = max(u_begin, strip * kb_per_strip);
          const long long tw0 = (kTiming && p.timing) ? clock64() : 0;
          ok = mbar_wait(&aux->acc_empty_bar[acc], acc_phase ^ 1, abort_flag, p.status, kStatusMmaTimeout);
          if (kTiming && p.timing) wait_acc += clock64() - tw0;
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + acc * acc_cols;
          for (int64_t u = seg_begin; u < seg_end; ++u) {
            const long long tw1 = (kTiming && p.timing) ? clock64() : 0;
            ok = mbar_wait(&aux->full_bar[stage], phase, abort_flag, p.status, kStatusMmaTimeout);
            if (kTiming && p.timing) {
              wait_full += clock64() - tw1;
              if (first_data_ns == 0) first_data_ns = global_timer_ns();   // first operands have landed
            }
            if (!ok) break;
            tc_fence_after_sync();
            const uint64_t stage_off = uint64_t((stage * stage_bytes) >> 4);
            for (int s = 0; s < p.n_sub; ++s) {
              const uint64_t w_desc = w_desc0 + stage_off + uint64_t((s * kWBoxBytes) >> 4);
#pragma unroll
              for (int j = 0; j < kBK / kUmmaK; ++j) {
                umma_f8(d_tmem + s * p.m, w_desc + uint64_t(j * w_kstep), a_desc0 + stage_off + uint64_t(j * a_kstep),
                        p.idesc, (u > seg_begin || j > 0) ? 1u : 0u);
              }
            }
            umma_commit(&aux->empty_bar[stage]);
            if (++stage == p.stages) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (!ok) break;
          umma_commit(&aux->acc_full_bar[acc]);
          if (++acc == kAccBufs) {
            acc = 0;
            acc_phase ^= 1;
          }
          seg_end = seg_begin;
        }
        if (kTiming && p.timing) {
          p.timing[blockIdx.x * 16 + 0] = wait_full;
          p.timing[blockIdx.x * 16 + 5] = first_data_ns;
          p.timing[blockIdx.x * 16 + 8] = wait_acc;
          p.timing[blockIdx.x * 16 + 2] = clock64() - t_begin;
          p.timing[blockIdx.x * 16 + 4] = global_timer_ns() - ns_begin;
        }
      }
    } else if ((warp - 2) / 4 < ep_halves) {
      // ------------------------------------------------------------------ epilogue (warps 2..9)
      const int q = warp & 3;                    // TMEM lane quarter
      const int half = (warp - 2) >> 2;          // which half of the m columns
      const int fq = half * 4 + q;               // flag / partial ownership index within a CTA
      const int col_lo = half * cols_per_warp;
      float scale = p.alpha;
      if (p.a_scale) scale *= __ldg(p.a_scale);
      if (p.b_scale) scale *= __ldg(p.b_scale);
      const uint64_t keep = l2_policy_evict_last();            // partial tiles should still be in L2 when they are summed
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      long long ep_accwait = 0, ep_flagwait = 0, ep_busy = 0;
      int64_t seg_end = u_end;
      while (seg_end > u_begin) {
        const int64_t strip = (seg_end - 1) / kb_per_strip;
        const int64_t strip_first = strip * kb_per_strip;
        const int64_t seg_begin = max(u_begin, strip_first);
        const bool owns_tail = seg_end == strip_first + kb_per_strip;   // holds the strip's last k-block
        const bool owns_head = seg_begin == strip_first;

        const int nl = q * 32 + lane;                          // lane of the accumulator = column within a tile
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * acc_cols);
        const int64_t slot_floats = int64_t(p.n_sub) * p.m * kTileN;
        const int chunks_per_sub = cols_per_warp / 16;
        const int nchunks = p.n_sub * chunks_per_sub;
        const bool finisher = owns_tail && !owns_head;       // must add other CTAs' partial sums
        int64_t first_contrib = member;                      // lowest unit range that contributed to this strip
        float pre0[16], pre1[16], pre2[16], pre3[16];        // other CTAs' partial sums, fetched four chunks ahead

        // Sum of the lower-numbered CTAs' partials for chunk `ci` (requested early, consumed later).
        auto load_partials = [&](int ci, float (&pre)[16]) {
          const int s = ci / chunks_per_sub, c0 = col_lo + (ci % chunks_per_sub) * 16;
          const float* slot =
              p.partials + (first_contrib * p.group + side) * slot_floats + (int64_t(s) * p.m + c0) * kTileN + nl;
#pragma unroll
          for (int i = 0; i < 16; ++i) pre[i] = __ldcg(slot + i * kTileN);
          for (int64_t c = first_contrib + 1; c < member; ++c) {
            slot += p.group * slot_floats;
#pragma unroll
            for (int i = 0; i < 16; ++i) pre[i] += __ldcg(slot + i * kTileN);
          }
        };

        if (finisher) {
          // The CTAs holding the earlier k-blocks of this strip finished their piece long ago (it was
          // the first thing they did).  Their flags and partials are fetched now, while this CTA's own
          // MMAs for the strip are still running, so that nothing but arithmetic is left for the end.
          first_contrib = member - 1;
          while (unit_begin(first_contrib, p.total_units, grid) > strip_first) --first_contrib;
          const long long tf0 = (kTiming && p.timing) ? clock64() : 0;
          if (lane == 0) {
            for (int64_t c = member - 1; c >= first_contrib && ok; --c) {
              const uint64_t* f = p.flags + (c * p.group + side) * 8 + fq;
              uint64_t t0 = 0;
              uint32_t polls = 0;
              while (ld_acquire_gpu(f) != p.epoch) {
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
          if (kTiming && p.timing) ep_flagwait += clock64() - tf0;
          if (!ok) break;
          // Every lane acquires the (already raised) flags itself before it reads the partials.
          for (int64_t c = member - 1; c >= first_contrib; --c)
            (void)ld_acquire_gpu(p.flags + (c * p.group + side) * 8 + fq);
          load_partials(0, pre0);
          if (nchunks > 1) load_partials(1, pre1);
          if (nchunks > 2) load_partials(2, pre2);
          if (nchunks > 3) load_partials(3, pre3);
        }

        const long long te0 = (kTiming && p.timing) ? clock64() : 0;
        if (lane == 0) ok = mbar_wait(&aux->acc_full_bar[acc], acc_phase, abort_flag, p.status, kStatusEpilogueTimeout);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        (void)mbar_try_wait(&aux->acc_full_bar[acc], acc_phase);
        tc_fence_after_sync();
        const long long te1 = (kTiming && p.timing) ? clock64() : 0;
        ep_accwait += te1 - te0;

        if (!owns_tail) {
          // Partial piece: park it in this CTA's workspace slot and publish.
          float* slot = p.partials + cta * slot_floats;
          uint32_t r[16];
          tmem_ld_32x16(taddr + col_lo, r);
#pragma unroll 1
          for (int ci = 0; ci < nchunks; ++ci) {
            const int s = ci / chunks_per_sub, c0 = col_lo + (ci % chunks_per_sub) * 16;
            float* out = slot + (int64_t(s) * p.m + c0) * kTileN + nl;
            tmem_ld_wait_16(r);
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
            if (ci + 1 < nchunks) {
              const int s1 = (ci + 1) / chunks_per_sub, c1 = col_lo + ((ci + 1) % chunks_per_sub) * 16;
              tmem_ld_32x16(taddr + s1 * p.m + c1, r);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) st_global_f32_hint(out + i * kTileN, v[i], keep);
          }
          __threadfence();
          __syncwarp();
          if (lane == 0) st_release_gpu(p.flags + cta * 8 + fq, p.epoch);
        } else {
          // Finishing piece: accumulator (+ the other CTAs' partials) -> scale -> cast -> D.
          uint32_t r[16];
          tmem_ld_32x16(taddr + col_lo, r);
          auto finish_chunk = [&](int ci, float (&pre)[16]) {
            const int s = ci / chunks_per_sub, c0 = col_lo + (ci % chunks_per_sub) * 16;
            const int64_t col = ((strip * p.group + side) * p.n_sub + s) * kTileN + nl;
            float v[16];
            if (finisher) {
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] = pre[i];
              if (ci + 4 < nchunks) load_partials(ci + 4, pre);
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] = 0.0f;
            }
            tmem_ld_wait_16(r);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = (v[i] + __uint_as_float(r[i])) * scale;
            if (ci + 1 < nchunks) {
              const int s1 = (ci + 1) / chunks_per_sub, c1 = col_lo + ((ci + 1) % chunks_per_sub) * 16;
              tmem_ld_32x16(taddr + s1 * p.m + c1, r);
            }
            if (col < p.n) {
#pragma unroll
              for (int i = 0; i < 16; ++i) store_out(p, int64_t(c0 + i) * p.n + col, v[i]);
            }
          };
#pragma unroll 1
          for (int ci = 0; ci < nchunks; ci += 4) {
            finish_chunk(ci, pre0);
            if (ci + 1 < nchunks) finish_chunk(ci + 1, pre1);
            if (ci + 2 < nchunks) finish_chunk(ci + 2, pre2);
            if (ci + 3 < nchunks) finish_chunk(ci + 3, pre3);
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (kTiming && p.timing) ep_busy += clock64() - te1;
        if (lane == 0) mbar_arrive(&aux->acc_empty_bar[acc]);
        if (++acc == kAccBufs) {
          acc = 0;
          acc_phase ^= 1;
        }
        seg_end = seg_begin;
      }
      if (kTiming && p.timing && warp == 2 && lane == 0) {
        p.timing[blockIdx.x * 16 + 6] = ep_busy;
        p.timing[blockIdx.x * 16 + 9] = ep_flagwait;
        p.timing[blockIdx.x * 16 + 10] = ep_accwait;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (kTiming && p.timing && threadIdx.x == 64) p.timing[blockIdx.x * 16 + 7] = global_timer_ns();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(aux->tmem_base, kTmemCols);
  }
}

// A 64-bit value no earlier launch of this process has used and that arbitrary memory contents will
// not equal by accident: a per-process random tag in the high half, a launch counter in the low half.
uint64_t NextEpoch() {
  static const uint64_t tag = [] {
    std::random_device rd;
    uint64_t t = (uint64_t(rd()) << 32) ^ uint64_t(rd());
    return (t | (1ull << 63)) & 0xFFFFFFFF00000000ull;
  }();
  static std::atomic<uint64_t> counter{1};
  return tag | (counter.fetch_add(1, std::memory_order_relaxed) & 0xFFFFFFFFull);
}

// Strip width: as wide as the two accumulator sets allow (2 * n_sub * m <= 512 TMEM columns).
int StripTiles(int64_t m) {
  static const int forced = TuningEnvInt("B200SD_SKINNY_NSUB", 0);   // 1, 2 or 4
  int n_sub = 1;   // measured fastest: wider strips lengthen the exposed last epilogue more than they help DRAM
  if (forced == 1 || forced == 2 || forced == 4) n_sub = forced;
  while (2 * n_sub * m > kTmemCols) n_sub >>= 1;
  return n_sub;
}

}  // namespace

Status InitSkinnyKernels() {
  cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       int(kSmemBudget));
  if (e != cudaSuccess) return Status::Error(kInternal, std::string("cudaFuncSetAttribute(skinny): ") + cudaGetErrorString(e));
  return Status::Ok();
}

#if B200SD_TUNING
extern "C" int b200sd_debug_read_skinny_timing(unsigned long long* out, int count) {
  cudaDeviceSynchronize();
  return int(cudaMemcpyFromSymbol(out, g_skinny_timing, sizeof(unsigned long long) * size_t(count)));
}
#endif

size_t SkinnyWorkspaceBytes(int64_t m, int64_t n, int64_t k) {
  if (m <= 0 || m > 128 || m % 16 != 0 || n <= 0 || k <= 0) return 0;
  return kFlagBytes + size_t(kMaxCtas) * size_t(kMaxSub) * size_t(m <= 64 ? m : m / 2) * kTileN * sizeof(float);
}

Status LaunchSkinny(const GemmProblem& g, cudaStream_t stream, LaunchStats* stats) {
  int device = 0;
  cudaGetDevice(&device);
  Status st = InitDevice(device);
  if (!st.ok()) return st;
  if (g.int8 || g.a_mn_major || !g.b_mn_major || g.m > 128 || g.m % 16 != 0)
    return Status::Error(kInvalidArgument, "split-K kernel: unsupported operand arrangement");
  // store_out() writes bf16, f16 or f32 and applies no output scale: anything else would be
  // stored with the wrong element size.
  if (!(g.d_dtype == kBF16 || g.d_dtype == kF16 || g.d_dtype == kF32) || g.d_scale != nullptr || g.c != nullptr ||
      g.bias != nullptr || g.activation != kActNone || g.amax != nullptr)
    return Status::Error(kInvalidArgument, "split-K kernel: computes the plain scaled dot with a bf16, f16 or f32 result only");
  const size_t need = SkinnyWorkspaceBytes(g.m, g.n, g.k);
  if (g.workspace == nullptr || g.workspace_bytes < need)
    return Status::Error(kInvalidArgument, "split-K kernel: workspace too small");
  if ((reinterpret_cast<uintptr_t>(g.workspace) & 15) != 0)
    return Status::Error(kInvalidArgument, "split-K kernel: workspace must be 16-byte aligned");

  static const int env_promo = TuningEnvInt("B200SD_SKINNY_PROMO", 3);
  static const int env_stages = TuningEnvInt("B200SD_SKINNY_STAGES", 0);
  CUtensorMap tmap_w, tmap_a;
  st = MakeByteMatrixMap(&tmap_w, g.b, g.k, g.n, kTileN, kBK, env_promo);  // W [k, n]: box 128(n) x 128(k)
  if (!st.ok()) return st;
  st = MakeByteMatrixMap(&tmap_a, g.a, g.m, g.k, kBK, uint32_t(g.m));     // A [m, k]: box 128(k) x m
  if (!st.ok()) return st;

  SkinnyArgs p{};
  p.m = int32_t(g.m); p.n = g.n; p.k = g.k;
  p.n_sub = StripTiles(g.m);
  p.a_stage_bytes = int32_t((g.m * kBK + 1023) / 1024 * 1024);
  const size_t stage_bytes = size_t(p.n_sub) * kWBoxBytes + p.a_stage_bytes;
  int stages = int((kSmemBudget - 1024 - sizeof(SkinnyAux)) / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  if (env_stages >= 2 && env_stages < stages) stages = env_stages;
  if (stages < 2) return Status::Error(kInternal, "split-K kernel: not enough shared memory for two stages");
  p.stages = stages;
  static const int env_group = TuningEnvInt("B200SD_SKINNY_GROUP", 2);
  p.group = (env_group == 1 || env_group == 2 || env_group == 4) ? env_group : 2;
  const int64_t strip_cols = int64_t(p.n_sub) * p.group * kTileN;
  p.num_strips = int32_t((g.n + strip_cols - 1) / strip_cols);
  p.num_k_blocks = int32_t((g.k + kBK - 1) / kBK);
  p.total_units = int64_t(p.num_strips) * p.num_k_blocks;
  // D^T = W^T . A^T: the 128-row operand is W (MN-major), the N operand is A (K-major), N = m.
  p.idesc = make_idesc(1u, g.b_dtype == kF8E5M2 ? 1u : 0u, g.a_dtype == kF8E5M2 ? 1u : 0u, true, false, 128,
                       uint32_t(g.m));
  p.a_scale = g.a_scale; p.b_scale = g.b_scale; p.alpha = g.alpha;
  p.d = g.d; p.d_dtype = g.d_dtype;
  p.flags = static_cast<uint64_t*>(g.workspace);
  p.epoch = NextEpoch();
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(g.workspace) + kFlagBytes);
  p.status = StatusWordPtr();
  p.timing = nullptr;
#if B200SD_TUNING
  static const bool timing_on = TuningEnvInt("B200SD_TIMING", 0) == 1;
  if (timing_on) {
    cudaGetSymbolAddress(reinterpret_cast<void**>(&p.timing), g_skinny_timing);
    cudaMemsetAsync(p.timing, 0, sizeof(g_skinny_timing), stream);
  }
#endif

  int64_t grid = DeviceSmCount();
  if (grid > kMaxCtas) grid = kMaxCtas;
  if (grid > p.total_units * p.group) grid = p.total_units * p.group;
  grid -= grid % p.group;
  if (StreamIsCapturing(stream)) {
    // Every replay of the recorded launch carries this same epoch: the flags the previous replay
    // raised must read "not raised" again, so a memset node goes in front of the kernel.
    cudaError_t me = cudaMemsetAsync(p.flags, 0, kFlagBytes, stream);
    if (me != cudaSuccess) return Status::Error(kInternal, std::string("cudaMemsetAsync(split-K flags): ") + cudaGetErrorString(me));
  }
  const size_t smem_bytes = 1024 + size_t(stages) * stage_bytes + sizeof(SkinnyAux);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(grid), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // see griddep_wait() in the kernel
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, skinny_gemm_kernel, tmap_w, tmap_a, p);
  if (e != cudaSuccess) return Status::Error(kInternal, std::string("skinny_gemm_kernel launch: ") + cudaGetErrorString(e));
  if (stats) {
    stats->kernel = kKernelSkinny;
    stats->grid = int32_t(grid);
    stats->launches = 1;
  }
  return Status::Ok();
}


// ----------------------------------------------------------------------------- no-allocation variant
// The split-K kernel needs scratch: per-CTA f32 partial tiles and the flags that publish them.
// The regular entry point takes that scratch from the caller.  Some callers have none to give
// and may not create any: an XLA executable runs on a memory plan fixed at compile time, its
// allocator usually already owns almost all of HBM, and a handler that promises to be recordable
// into a command buffer must not allocate while it executes.  When such a call site carries no
// workspace result, the variant below still works: its scratch is a fixed array that is part of
// the library image, so every GPU that loads the library holds these bytes until the process exits.
// The array bounds what the variant accepts (m <= 128 with single-tile strips on at most
// kMaxCtas CTAs).
constexpr size_t kStaticPartialBytes = size_t(kMaxCtas) * 128 * kTileN * sizeof(float);   // 10 MiB
constexpr size_t kStaticScratchBytes = kFlagBytes + kStaticPartialBytes;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {

struct StaticScratchState {
  std::once_flag once;
  cudaError_t error = cudaSuccess;
  unsigned char* device_ptr = nullptr;   // address of g_static_scratch on this device
};
StaticScratchState g_static_state[64];

// `g_static_scratch` named in host code is only a handle for the runtime, not a device address;
// the address on the current device has to be asked for, once per device.
Status StaticScratchPtr(int device, unsigned char** ptr) {
  if (device < 0 || device >= 64) return Status::Error(kInvalidArgument, "device ordinal out of range");
  StaticScratchState& st = g_static_state[device];
  std::call_once(st.once, [&] {
    void* p = nullptr;
    st.error = cudaGetSymbolAddress(&p, g_static_scratch);
    st.device_ptr = static_cast<unsigned char*>(p);
  });
  if (st.error != cudaSuccess || st.device_ptr == nullptr)
    return Status::Error(kInternal, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(st.error));
  *ptr = st.device_ptr;
  return Status::Ok();
}

}  // namespace

Status ValidateF8(const B200SD_ScaledDotF8& a, GemmProblem* g, bool check_pointers);

}  // namespace b200sd

extern "C" size_t b200sd_noalloc_scratch_bytes(void) { return b200sd::kStaticScratchBytes; }

extern "C" int b200sd_scaled_dot_f8_decode_noalloc(const B200SD_ScaledDotF8* args, void* cuda_stream, char* err,
                                                   size_t err_len) {
  using namespace b200sd;
  auto fail = [&](int code, const std::string& msg) {
    if (err != nullptr && err_len > 0) {
      const size_t n = msg.size() < err_len - 1 ? msg.size() : err_len - 1;
      std::memcpy(err, msg.data(), n);
      err[n] = '\0';
    }
    return code;
  };
  if (args == nullptr) return fail(kInvalidArgument, "args is null");
  GemmProblem g;
  Status st = ValidateF8(*args, &g, /*check_pointers=*/true);
  if (!st.ok()) return fail(st.code, st.message);
  if (g.batch > 1) return fail(kInvalidArgument, "the no-allocation decode entry point does not take batched dots");
  if (g.m > 128)
    return fail(kInvalidArgument, "the no-allocation decode entry point accepts at most 128 rows of A (m = " +
                                      std::to_string(g.m) + "): its built-in scratch holds one 128 x 128 f32 partial per CTA");
  if (g.a_mn_major || !g.b_mn_major || g.a_dtype != kF8E4M3FN || g.b_dtype != kF8E4M3FN || g.c != nullptr ||
      g.bias != nullptr || g.activation != kActNone || g.amax != nullptr || g.d_scale != nullptr ||
      !(g.d_dtype == kBF16 || g.d_dtype == kF16 || g.d_dtype == kF32))
    return fail(kInvalidArgument, "the no-allocation decode entry point computes the plain scaled dot only: e4m3 A[m,k] and "
                                  "B[k,n] row-major, per-tensor scales, bf16/f16/f32 output, no bias, activation, amax or d_scale");
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail(kInternal, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  st = InitDevice(device);
  if (!st.ok()) return fail(st.code, st.message);
  unsigned char* scratch = nullptr;
  st = StaticScratchPtr(device, &scratch);
  if (!st.ok()) return fail(st.code, st.message);

  CUtensorMap tmap_w, tmap_a;
  st = MakeByteMatrixMap(&tmap_w, g.b, g.k, g.n, kTileN, kBK);
  if (!st.ok()) return fail(st.code, st.message);
  st = MakeByteMatrixMap(&tmap_a, g.a, g.m, g.k, kBK, uint32_t(g.m));
  if (!st.ok()) return fail(st.code, st.message);

  SkinnyArgs p{};
  p.m = int32_t(g.m); p.n = g.n; p.k = g.k;
  p.n_sub = 1;                                        // one 128-column tile per strip keeps a partial at m * 128 floats
  p.group = 1;
  p.a_stage_bytes = int32_t((g.m * kBK + 1023) / 1024 * 1024);
  const size_t stage_bytes = size_t(kWBoxBytes) + p.a_stage_bytes;
  int stages = int((kSmemBudget - 1024 - sizeof(SkinnyAux)) / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  p.stages = stages;
  p.num_strips = int32_t((g.n + kTileN - 1) / kTileN);
  p.num_k_blocks = int32_t((g.k + kBK - 1) / kBK);
  p.total_units = int64_t(p.num_strips) * p.num_k_blocks;
  p.idesc = make_idesc(1u, 0u, 0u, true, false, 128, uint32_t(g.m));
  p.a_scale = g.a_scale; p.b_scale = g.b_scale; p.alpha = g.alpha;
  p.d = g.d; p.d_dtype = g.d_dtype;
  p.flags = reinterpret_cast<uint64_t*>(scratch);
  p.epoch = NextEpoch();
  p.partials = reinterpret_cast<float*>(scratch + kFlagBytes);
  p.status = StatusWordPtr();

  int64_t grid = DeviceSmCount();
  if (grid > kMaxCtas) grid = kMaxCtas;
  if (grid > p.total_units) grid = p.total_units;
  if (size_t(grid) * size_t(g.m) * kTileN * sizeof(float) > kStaticPartialBytes)
    return fail(kInvalidArgument, "problem does not fit the built-in scratch");
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // The array still holds the previous call's flags: they carry that call's epoch value, which no CTA of this
  // call takes for its own, so nothing has to be cleared first.
  const size_t smem_bytes = 1024 + size_t(stages) * stage_bytes + sizeof(SkinnyAux);
  skinny_gemm_kernel<<<int(grid), kThreads, smem_bytes, stream>>>(tmap_w, tmap_a, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(kInternal, std::string("skinny_gemm_kernel launch: ") + cudaGetErrorString(e));
  if (err != nullptr && err_len > 0) err[0] = '\0';
  return kOk;
}
