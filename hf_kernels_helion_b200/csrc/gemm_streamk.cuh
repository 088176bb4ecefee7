// Decode-shape (M <= 256 tokens) block-FP8 GEMM for sm_100a: swap-AB + stream-K.
//
// With few tokens the op is a stream over the weight B[N,K] and is HBM-bound, so
//   * the 128 weight rows of a tile sit on the UMMA M axis and the (padded) tokens on
//     the UMMA N axis (MP = 16..256), i.e. the kernel computes C^T tiles [128 n x MP m];
//   * the work is cut into (weight tile, 128-wide K block) units and every CTA gets
//     one contiguous, equally long range of units, so all SMs stream the same share
//     of B whatever N/128 is. A range may begin or end in the middle of a tile; such
//     partial sums go to an fp32 workspace and streamk_fixup_kernel adds the (at most
//     a few) pieces of each split tile in a fixed order - no atomics, no inter-CTA
//     waits, bit-reproducible.
// Token scales are needed per accumulator COLUMN here; streamk_prep_kernel first writes
// them K-block-major (AsT[kb][m]) so that the producer can fetch the MP scales of a unit
// with one bulk copy riding the same pipeline as the tiles.
#pragma once

#include <cuda_bf16.h>

#include "gemm_tile.cuh"
#include "ptx.cuh"

namespace b200fp8 {

struct StreamKArgs {
  const float* Bs;
  const float* AsT;    // [num_kb][MP] fp32, zero for m >= M (workspace)
  float* partial;      // [2 * grid][MP][128] fp32 (workspace)
  void* C;
  int64_t M, N, K;
  int64_t ld_bs, ldc;
  int out_fp32;
  uint32_t* status_word;
};

template <int MP_>
struct StreamKCfg {
  static constexpr int MP = MP_;
  static constexpr int BN = 128;  // weight rows per tile
  static constexpr int BK = 128;
  static constexpr int W_BYTES = BN * BK;
  static constexpr int X_BYTES = MP_ * BK;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int STAGES_RAW = (200 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 12 ? 12 : STAGES_RAW;
  static constexpr int TMEM_STAGES_RAW = 512 / MP_;
  static constexpr int TMEM_STAGES = TMEM_STAGES_RAW > 8 ? 8 : TMEM_STAGES_RAW;  // accumulator stages in TMEM
  static constexpr int SC_RING = STAGES + TMEM_STAGES + 2;  // see the note at the epilogue's TMEM release
  static constexpr int SC_BYTES = MP_ * 4;
  static constexpr int PRODUCER_BATCH = STAGES >= 8 ? 4 : (STAGES >= 4 ? 2 : 1);
  static constexpr int EPI_WARPS = MP_ >= 128 ? 8 : 4;
  static constexpr int EPI_COLS = MP_ / (EPI_WARPS / 4);
  static constexpr int THREADS = 128 + 32 * EPI_WARPS;
  static constexpr bool REBALANCE_REGS = (EPI_COLS > 64);
  // setmaxnreg.inc blocks until the registers exist: what the epilogue warpgroups take must
  // fit in what the launch allocated (168 per thread at 384 threads) minus what the control
  // warpgroup keeps.
  static constexpr int REGS_CONTROL = 56;
  static constexpr int REGS_EPILOGUE = 224;
  static_assert(!REBALANCE_REGS || 128 * REGS_CONTROL + 32 * EPI_WARPS * REGS_EPILOGUE <= 168 * THREADS,
                "setmaxnreg.inc would wait for registers that never become free");
  static constexpr int TMEM_COLS = TMEM_STAGES * MP_;  // 128, 256 or 512: a power of two >= 32
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SC_RING * SC_BYTES + BAR_BYTES + 1024;
};

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// AsT[kb][m] = As[m][kb] for m < M, 0 for M <= m < MP.
__global__ void streamk_prep_kernel(const float* __restrict__ As, float* __restrict__ AsT, int64_t M, int num_kb,
                                    int64_t ld_as, int MP) {
  const int total = num_kb * MP;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int kb = i / MP, m = i - kb * MP;
    AsT[i] = m < M ? __ldg(As + static_cast<int64_t>(m) * ld_as + kb) : 0.f;
  }
}

template <int MP>
__global__ void __launch_bounds__(StreamKCfg<MP>::THREADS, 1)
gemm_streamk_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                    const StreamKArgs args) {
  using Cfg = StreamKCfg<MP>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int SC_RING = Cfg::SC_RING;
  constexpr uint32_t TS = Cfg::TMEM_STAGES;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sc_ring = reinterpret_cast<float*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES + SC_RING * Cfg::SC_BYTES);
  uint64_t* full = bars;                            // [STAGES]
  uint64_t* empty = bars + STAGES;                  // [STAGES]
  uint64_t* sc_full = bars + 2 * STAGES;            // [SC_RING]
  uint64_t* tfull = bars + 2 * STAGES + SC_RING;    // [TS]
  uint64_t* tempty = tfull + TS;                    // [TS]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + TS);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  static_assert((2 * STAGES + SC_RING + 2 * TS) * 8 + 8 <= Cfg::BAR_BYTES, "barrier area too small");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < SC_RING; ++s) mbar_init(&sc_full[s], 1);
    for (uint32_t s = 0; s < TS; ++s) {
      mbar_init(&tfull[s], 1);
      mbar_init(&tempty[s], Cfg::EPI_WARPS);
    }
    *abort_flag = 0u;
    fence_barrier_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int64_t M = args.M, N = args.N, K = args.K;
  const int num_kb = static_cast<int>((K + Cfg::BK - 1) / Cfg::BK);
  const int64_t num_tiles = (N + Cfg::BN - 1) / Cfg::BN;
  const int64_t total_units = num_tiles * num_kb;
  const int64_t u0 = streamk_first_unit(blockIdx.x, total_units, gridDim.x);
  const int64_t u1 = streamk_first_unit(blockIdx.x + 1, total_units, gridDim.x);
  uint32_t* status_word = args.status_word;

  if (warp < 4) {
    if constexpr (Cfg::REBALANCE_REGS) setmaxnreg_dec<Cfg::REGS_CONTROL>();
  }
  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      prefetch_tmap(&tmap_w);
      prefetch_tmap(&tmap_x);
      const uint64_t pol_stream = policy_evict_first();  // weights are read exactly once
      const uint64_t pol_keep = policy_evict_last();     // the few activation rows are re-read by every CTA
      uint32_t it = 0;
      bool ok = true;
      // Units are issued in batches of up to kBatch consecutive K blocks: the batch's loads
      // go out back to back, so that DRAM sees kBatch * 128 contiguous bytes of each weight
      // row within one burst of requests instead of 128-byte pieces spread over time.
      constexpr int kBatch = Cfg::PRODUCER_BATCH;
      for (int64_t u = u0; ok && u < u1;) {
        const int64_t left = u1 - u;
        const int nb = left < kBatch ? static_cast<int>(left) : kBatch;
        for (int i = 0; i < nb; ++i) {
          const uint32_t j = it + i;
          if (!mbar_wait(&empty[j % STAGES], ((j / STAGES) & 1u) ^ 1u, abort_flag, status_word)) { ok = false; break; }
        }
        if (!ok) break;
        for (int i = 0; i < nb; ++i) {
          const uint32_t j = it + i;
          const int64_t tile = (u + i) / num_kb;
          const int kb = static_cast<int>((u + i) - tile * num_kb);
          const uint32_t s = j % STAGES;
          uint8_t* w_dst = smem + s * Cfg::STAGE_BYTES;
          mbar_arrive_expect_tx(&full[s], Cfg::STAGE_BYTES);
          tma_load_2d_hint(w_dst, &tmap_w, &full[s], kb * Cfg::BK, static_cast<int32_t>(tile * Cfg::BN), pol_stream);
        }
        for (int i = 0; i < nb; ++i) {
          const uint32_t j = it + i;
          const int64_t tile = (u + i) / num_kb;
          const int kb = static_cast<int>((u + i) - tile * num_kb);
          const uint32_t s = j % STAGES;
          uint8_t* x_dst = smem + s * Cfg::STAGE_BYTES + Cfg::W_BYTES;
          tma_load_2d_hint(x_dst, &tmap_x, &full[s], kb * Cfg::BK, 0, pol_keep);
          const uint32_t r = j % SC_RING;
          mbar_arrive_expect_tx(&sc_full[r], Cfg::SC_BYTES);
          bulk_load_1d(sc_ring + r * MP, args.AsT + static_cast<int64_t>(kb) * MP, Cfg::SC_BYTES, &sc_full[r]);
        }
        it += nb;
        u += nb;
      }
      if (!ok) {
        const uint32_t first = it > static_cast<uint32_t>(STAGES) ? it - STAGES : 0u;
        for (uint32_t j = first; j < it; ++j) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&full[j % STAGES], (j / STAGES) & 1u) ||
                 !mbar_try_wait(&sc_full[j % SC_RING], (j / SC_RING) & 1u)) {
            if (globaltimer_ns() - t0 > kWaitLimitNs) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_e4m3_f32(128, MP);
      uint32_t it = 0;
      bool ok = true;
      for (int64_t u = u0; u < u1; ++u, ++it) {
        const uint32_t s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1u;
        const uint32_t ts = it % TS;
        const uint32_t tph = (it / TS) & 1u;
        if (!mbar_wait(&tempty[ts], tph ^ 1u, abort_flag, status_word)) { ok = false; break; }
        if (!mbar_wait(&full[s], ph, abort_flag, status_word)) { ok = false; break; }
        tc_fence_after();
        const uint32_t w_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
        const uint64_t w_desc = make_smem_desc_sw128(w_addr);
        const uint64_t x_desc = make_smem_desc_sw128(w_addr + Cfg::W_BYTES);
        const uint32_t d_tmem = tmem_base + ts * MP;
#pragma unroll
        for (int k = 0; k < Cfg::BK / 32; ++k) umma_f8(d_tmem, w_desc + 2u * k, x_desc + 2u * k, idesc, k > 0 ? 1u : 0u);
        tc_commit(&empty[s]);
        tc_commit(&tfull[ts]);
      }
      if (!ok && it > 0) {
        const uint32_t j = it - 1;
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(&tfull[j % TS], (j / TS) & 1u)) {
          if (globaltimer_ns() - t0 > kWaitLimitNs) break;
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ promotion + epilogue
    if constexpr (Cfg::REBALANCE_REGS) setmaxnreg_inc<Cfg::REGS_EPILOGUE>();
    constexpr int EC = Cfg::EPI_COLS;
    const int e = warp - 4;
    const int q = warp & 3;
    const int col0 = (e >> 2) * EC;          // first token column of this warp
    const int n_local = q * 32 + lane;       // weight row inside the tile = TMEM lane
    uint32_t it = 0;
    bool ok = true;
    float acc[EC];
    int seg_first_kb = 0;
    bool seg_is_first = true;
    float sb_next = 0.f;
    if (u0 < u1) sb_next = __ldg(args.Bs + (u0 / num_kb) * args.ld_bs + (u0 % num_kb));
    for (int64_t u = u0; u < u1; ++u, ++it) {
      const int64_t tile = u / num_kb;
      const int kb = static_cast<int>(u - tile * num_kb);
      if (u == u0 || kb == 0) {
#pragma unroll
        for (int j = 0; j < EC; ++j) acc[j] = 0.f;
        seg_first_kb = kb;
        seg_is_first = (u == u0);
      }
      const float sb = sb_next;  // weight-block scale of this unit, fetched one unit ahead
      if (u + 1 < u1) sb_next = __ldg(args.Bs + ((u + 1) / num_kb) * args.ld_bs + ((u + 1) % num_kb));
      const uint32_t ts = it % TS;
      const uint32_t tph = (it / TS) & 1u;
      const uint32_t r = it % SC_RING;
      ok = __all_sync(0xffffffffu, mbar_wait(&tfull[ts], tph, abort_flag, status_word) &&
                                       mbar_wait(&sc_full[r], (it / SC_RING) & 1u, abort_flag, status_word));
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ts * MP + col0;
      const float* sc = sc_ring + r * MP + col0;
      if constexpr (EC == 16) {
        uint32_t p[16];
        tmem_ld_32x16(taddr, p);
        tmem_ld_wait_16(p);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[ts]);
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          const float4 s4 = *reinterpret_cast<const float4*>(sc + j);
          acc[j + 0] = fmaf(__uint_as_float(p[j + 0]), s4.x * sb, acc[j + 0]);
          acc[j + 1] = fmaf(__uint_as_float(p[j + 1]), s4.y * sb, acc[j + 1]);
          acc[j + 2] = fmaf(__uint_as_float(p[j + 2]), s4.z * sb, acc[j + 2]);
          acc[j + 3] = fmaf(__uint_as_float(p[j + 3]), s4.w * sb, acc[j + 3]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < EC; c += 32) {
          uint32_t p[32];
          tmem_ld_32x32(taddr + c, p);
          tmem_ld_wait_32(p);
          if (c + 32 == EC) {
            // The TMEM stage is handed back before the scale reads below. The MMA warp
            // can then run at most TS units ahead of this warp and the producer at most
            // STAGES units ahead of the MMA warp, so a scale slot is rewritten no earlier
            // than STAGES + TS + 1 units later: SC_RING = STAGES + TS + 2 slots suffice.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[ts]);
          }
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 s4 = *reinterpret_cast<const float4*>(sc + c + j);
            acc[c + j + 0] = fmaf(__uint_as_float(p[j + 0]), s4.x * sb, acc[c + j + 0]);
            acc[c + j + 1] = fmaf(__uint_as_float(p[j + 1]), s4.y * sb, acc[c + j + 1]);
            acc[c + j + 2] = fmaf(__uint_as_float(p[j + 2]), s4.z * sb, acc[c + j + 2]);
            acc[c + j + 3] = fmaf(__uint_as_float(p[j + 3]), s4.w * sb, acc[c + j + 3]);
          }
        }
      }

      if (kb == num_kb - 1 || u == u1 - 1) {
        // end of this CTA's segment of the tile
        const int64_t n = tile * Cfg::BN + n_local;
        if (seg_first_kb == 0 && kb == num_kb - 1) {
          // the whole K range was ours: write C[m, n] directly (lanes = consecutive n)
          if (n < N) {
            if (args.out_fp32) {
              float* c = reinterpret_cast<float*>(args.C) + n;
#pragma unroll
              for (int j = 0; j < EC; ++j)
                if (col0 + j < M) c[static_cast<int64_t>(col0 + j) * args.ldc] = acc[j];
            } else {
              __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(args.C) + n;
#pragma unroll
              for (int j = 0; j < EC; ++j)
                if (col0 + j < M) c[static_cast<int64_t>(col0 + j) * args.ldc] = __float2bfloat16_rn(acc[j]);
            }
          }
        } else {
          const int64_t slot = 2 * static_cast<int64_t>(blockIdx.x) + (seg_is_first ? 0 : 1);
          float* dst = args.partial + slot * (static_cast<int64_t>(MP) * Cfg::BN) + n_local;
#pragma unroll
          for (int j = 0; j < EC; ++j)
            if (col0 + j < M) dst[static_cast<int64_t>(col0 + j) * Cfg::BN] = acc[j];
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// Adds the pieces of every split tile. Grid = (weight tiles, ceil(M / 8)); a CTA of 128
// threads (one per weight row of the tile) sums 8 token rows, pieces in ascending CTA order.
// Tiles that a single CTA of the stream-K kernel covered completely were already written
// and are skipped.
constexpr int kFixupRows = 8;

__global__ void __launch_bounds__(128)
streamk_fixup_kernel(const float* __restrict__ partial, void* C, int64_t M, int64_t N, int num_kb, int64_t ldc,
                     int out_fp32, int MP, int64_t sk_grid) {
  const int64_t tile = blockIdx.x;
  const int64_t num_tiles = gridDim.x;
  const int64_t total = num_tiles * num_kb;
  const int64_t c_first = streamk_owner(tile * num_kb, total, sk_grid);
  const int64_t c_last = streamk_owner(tile * num_kb + num_kb - 1, total, sk_grid);
  if (c_first == c_last) return;
  const int64_t n = tile * 128 + threadIdx.x;
  if (n >= N) return;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kFixupRows;
  const int64_t slot_elems = static_cast<int64_t>(MP) * 128;
  float sum[kFixupRows];
#pragma unroll
  for (int i = 0; i < kFixupRows; ++i) sum[i] = 0.f;
  for (int64_t c = c_first; c <= c_last; ++c) {
    const int64_t first_tile_of_c = streamk_first_unit(c, total, sk_grid) / num_kb;
    const int64_t slot = 2 * c + (first_tile_of_c == tile ? 0 : 1);
    const float* src = partial + slot * slot_elems + m0 * 128 + threadIdx.x;
#pragma unroll
    for (int i = 0; i < kFixupRows; ++i)
      if (m0 + i < M) sum[i] += __ldg(src + i * 128);
  }
#pragma unroll
  for (int i = 0; i < kFixupRows; ++i) {
    if (m0 + i < M) {
      if (out_fp32)
        reinterpret_cast<float*>(C)[(m0 + i) * ldc + n] = sum[i];
      else
        reinterpret_cast<__nv_bfloat16*>(C)[(m0 + i) * ldc + n] = __float2bfloat16_rn(sum[i]);
    }
  }
}

}  // namespace b200fp8
