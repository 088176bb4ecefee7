// Persistent, warp-specialised block-FP8 GEMM for sm_100a:  C[M,N] = A[M,K] . B[N,K]^T
// with fp32 scales As[M, K/128] (per token, per 128-wide K group) and
// Bs[N/128, K/128] (per 128x128 weight block).
//
// Roles inside one CTA (one CTA per SM, tiles handed out round-robin):
//   warp 0      TMA producer: A tile [128 x 128 B] and B tile [BN x 128 B] per K block
//               into a STAGES-deep shared-memory ring (SWIZZLE_128B, no multicast)
//   warps 1, 3  MMA issuers, alternating K blocks: 4 x tcgen05.mma kind::f8f6f4 (K = 32 each) per
//               K block into one of the TMEM accumulator stages, then tcgen05.commit to release
//               the smem slot and to publish the TMEM stage
//   warp 2      TMEM allocation / deallocation
//   warps 4..   promotion + epilogue: tcgen05.ld the fp32 partial of one K block,
//               acc += partial * (As[row, kb] * Bs[nb, kb]) in registers (the block
//               scales are arbitrary fp32, so partial sums cannot stay in TMEM across
//               K blocks), and after the last K block convert and store the tile.
// Several TMEM accumulator stages (512 / BN) let the MMAs of later K blocks overlap the
// promotion of block k.
// Forms of the same body (template parameters of gemm_tile_body): 128- or 256-wide tiles; a
// multi-destination epilogue (TMA stores or multimem stores of every finished box into several
// [M, N] buffers: the N-sharded multi-GPU exchange); tail split-K; row-scaled B; decode forms
// with 16- or 64-row A slots; and CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles per pair).
#pragma once

#include <cuda_bf16.h>

#include "ptx.cuh"
#include "quant.cuh"

namespace b200fp8 {

// Even split of `total` work units over `grid` owners in contiguous ranges: owner c has
// units [streamk_first_unit(c), streamk_first_unit(c + 1)).
__host__ __device__ __forceinline__ int64_t streamk_first_unit(int64_t c, int64_t total, int64_t grid) {
  return (c * total) / grid;
}
__host__ __device__ __forceinline__ int64_t streamk_owner(int64_t u, int64_t total, int64_t grid) {
  return ((u + 1) * grid - 1) / total;
}

struct GemmArgs {
  // Tail split-K (kernels instantiated with SK = true): tiles [0, sk_full) are handed out
  // round-robin as whole tiles; the remaining R < grid tiles - the last, partly empty wave -
  // are each cut into sk_split K ranges of sk_kb_per K blocks, one range per CTA, so that the
  // tail takes 1 / sk_split of a tile time. CTA c < R * sk_split works on tile sk_full + c /
  // sk_split, range c % sk_split, and leaves its fp32 partial sums in slot c of `partial` (layout:
  // sk_partial_ptr); tile_sk_fixup_kernel adds the ranges of each tail tile in a fixed order.
  int sk_full, sk_split, sk_kb_per;
  float* partial;
  // Destinations of the result: dst[0] is C itself; dst[1..n_dst-1] are further buffers that
  // receive the same [M, N] block (other GPUs' output buffers mapped into this process, for
  // the N-sharded multi-GPU case). staged_store = 1 when every destination meets the TMA
  // rules (pointer and row pitch multiples of 16 bytes): the multi-destination kernel then
  // stages the tile in shared memory and sends it with asynchronous TMA stores.
  // mc_store = 1: dst[0] is a multimem address of a buffer replicated on every GPU of a multicast
  // group; the multi-destination kernel then re-reads each staged box row-wise and writes it
  // with multimem.st, once, and the NVSwitch delivers it to all GPUs (this one included).
  int a_from_prep;   // 1: A was re-laid by tile_prep_kernel (M <= 16: 16-row copy), the producer must wait for it
  int n_dst;
  int staged_store;
  int mc_store;
  void* dst[8];
  int64_t dst_ld[8];
  const float* AsT;   // [ceil(K/128)][m_pad] token scales, K-block-major (written by tile_prep_kernel)
  int64_t m_pad;      // M rounded up to 128
  // Row-scaled B (kernels instantiated with ROWB = true): one scale per row of B and K block,
  // given as Bs [N, ceil(K/128)] and re-laid K-block-major by tile_prep_kernel as BsT[kb][n_pad]
  // (n_pad = N rounded up to 128, padding zero); Bs / ld_bs are then unused by the GEMM kernel.
  const float* BsT;
  int64_t n_pad;
  // 1: the row-scaled kernel keeps the B scales of the current tile ([K blocks][128 columns]) in shared
  // memory, loaded by the producer with one TMA box per tile (K <= kRowbTableKb * 128); 0: it reads them
  // from BsT in global memory on every K block.
  int rowb_table;
  const float* As;
  const float* Bs;
  void* C;
  int64_t M, N, K;
  int64_t ld_as, ld_bs, ldc;
  int out_fp32;
  uint32_t* status_word;
};

// A_ROWS_: rows of A that the TMA actually brings in per K block (128; 16 or 64 for decode shapes
// with M <= 16 / M <= 64). The MMA always reads 128 rows from the A slot; with a short slot
// (2 or 8 KiB) the remaining rows alias the B tile that follows it in the same stage - garbage
// that lands in accumulator rows which are never stored - and the bytes saved buy one or two
// more pipeline stages (weight streaming is bound by the bytes in flight per SM).
// PAIR_: 0 = one CTA per tile. 1, 2 = CTA pairs (clusters of two, tcgen05 cta_group::2): a pair owns
// a 256 x BN tile, each CTA accumulates its 128 rows in its own TMEM and holds its 128 rows of A and
// HALF of the B rows of the tile in shared memory (the MMA reads B from both CTAs), so a K block costs
// each SM 32 KiB of shared-memory fill and read instead of 48. PAIR_ = 2 additionally issues every K
// block as two 128-column halves with a TMEM-full / TMEM-empty barrier pair each: the promotion of
// columns 0..127 starts when the first half of the MMAs has retired and its TMEM columns are handed
// back a half block earlier, which shortens the accumulator round trip that bounds the kernel.
template <int BN_, bool MULTI_ = false, int A_ROWS_ = 128, int PAIR_ = 0>
struct TileCfg {
  static constexpr int BM = 128;                          // rows per CTA
  static constexpr int PAIR = PAIR_;
  static constexpr int TILE_M = PAIR_ ? 256 : 128;        // rows per worker (CTA or CTA pair)
  static constexpr int BN = BN_;
  static constexpr int BK = 128;  // fp8 elements = bytes = one 128-byte swizzle span
  static constexpr int A_ROWS = A_ROWS_;
  static constexpr int HALVES = PAIR_ == 2 ? 2 : 1;       // separately signalled column halves of a K block
  static constexpr int B_ROWS = PAIR_ ? BN_ / 2 : BN_;    // rows of B per CTA and K block
  // (pair kernels: 32-KiB stages; the multi-destination pair kernel gives one stage up for a second set of
  // output staging buffers)
  static constexpr int STAGES = PAIR_ ? (MULTI_ ? 5 : 6) : (A_ROWS_ == 16) ? 6 : (A_ROWS_ == 64) ? 5 : (BN_ == 128) ? 6 : 4;
  static_assert(PAIR_ == 0 || (BN_ == 256 && A_ROWS_ == 128), "pair kernels: 256-wide tiles, full A slots");
  static constexpr int EPI_WARPS = 8;               // two warps per TMEM lane quarter
  static constexpr int EPI_COLS = BN_ / 2;          // accumulator columns (registers) per epilogue thread
  static constexpr int THREADS = 128 + 32 * EPI_WARPS;
  // 128 accumulators + 64 staging registers per epilogue thread do not fit the 168
  // registers a 384-thread CTA gets by default: the BN = 256 kernel moves registers
  // from the producer/MMA warpgroup to the two epilogue warpgroups with setmaxnreg.
  // The BN = 128 kernel takes the same re-balancing (measured a few per cent faster with it).
  // Starting the TMEM load of K block i + 1 before the FMAs of block i (a second staging set)
  // was measured 15-20 % SLOWER for both tile widths: FMAs issued behind an outstanding
  // tcgen05.ld of the same warp do not overlap it, so each warp simply loads, waits, multiplies,
  // and the overlap comes from the other warp of the scheduler.
  static constexpr bool REBALANCE_REGS = true;
  // setmaxnreg budget: the CTA is launched with 168 registers per thread (65536 / 384 rounded
  // down to a multiple of 8); the control warpgroup gives registers back, the two epilogue
  // warpgroups take them. setmaxnreg.inc BLOCKS until the registers exist, so the sum must
  // not exceed what the launch allocated.
  static constexpr int REGS_LAUNCH = 168;
  static constexpr int REGS_CONTROL = 56;
  static constexpr int REGS_EPILOGUE = 224;
  static_assert(128 * REGS_CONTROL + 32 * EPI_WARPS * REGS_EPILOGUE <= REGS_LAUNCH * THREADS,
                "setmaxnreg.inc would wait for registers that never become free");
  static constexpr int A_BYTES = A_ROWS_ * BK;
  static_assert(A_ROWS_ == 128 || ((A_ROWS_ == 16 || A_ROWS_ == 64) && BN_ == 256 && !MULTI_),
                "short A slots exist for the decode case only");
  static_assert(A_ROWS_ * BK % 1024 == 0, "stage slots must stay 1 KiB aligned for the 128-byte swizzle");
  static constexpr int B_BYTES = B_ROWS * BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int ISSUERS = 2;                 // MMA issuer warps; issuer p takes the K blocks with index = p (mod 2)
  static constexpr int TMEM_STAGES = 512 / BN_;     // accumulator stages in TMEM (all 512 columns are used)
  static constexpr int TMEM_COLS = TMEM_STAGES * BN_;
  static constexpr int BAR_BYTES = 256;
  // output staging: each epilogue warp owns OUT_BUFS boxes of 32 rows x 128 bytes (128-byte-swizzled).
  // With ONE box a warp cannot stage the next 128-byte column group before the TMA has read the
  // previous one out, i.e. before it has left over NVLink: the link idles during the next tile's K
  // loop and the warp idles while the link drains. Two boxes (pair kernels, whose smaller pipeline
  // stages leave the room) let a whole bf16 tile queue up behind the K loop of the next one. Measured,
  // 8192 x 18432 x 7168 N-sharded: 2 GPUs 590 vs 611 us for the single-CTA form with one box; 4 GPUs 538 vs 540.
  static constexpr int OUT_BUFS = (MULTI_ && PAIR_) ? 2 : 1;
  static constexpr int OUT_BOX_BYTES = 32 * 128;
  static constexpr int OUT_STAGE_BYTES_PER_WARP = OUT_BOX_BYTES * OUT_BUFS;
  // (MULTI_ instantiations stage their output; the host takes them for several destinations and,
  // for the 256-wide tile, also for one destination whose rows are 16-byte aligned: the staged tile
  // leaves by TMA while the next K loop runs, where register stores of row pieces - 32 sectors per
  // warp instruction - keep the promotion warps away from TMEM at the end of every tile. The other
  // instantiations store straight from registers.)
  static constexpr bool MULTI = MULTI_;
  static constexpr int OUT_STAGE_BYTES = MULTI_ ? EPI_WARPS * OUT_STAGE_BYTES_PER_WARP : 0;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_STAGE_BYTES + BAR_BYTES + 1024;  // +1024: alignment slack
};

// Tile order: panels of kRasterGroup M-blocks; inside a panel the M index runs fastest, then
// N. The 148 tiles in flight at any time then cover a roughly square patch of C, so the
// A rows and B rows they share are fetched from DRAM once and hit in L2 afterwards.
constexpr int kRasterGroup = 32;

// Row-scaled kernel: K blocks of per-column B scales held in shared memory per tile (128 floats each).
constexpr int kRowbTableKb = 64;
constexpr int kRowbTableBytes = kRowbTableKb * 128 * 4;

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_blk, int& n_blk,
                                            int group = kRasterGroup) {
  const int per_panel = group * num_n;
  const int panel = tile / per_panel;
  const int rem = tile - panel * per_panel;
  const int m_first = panel * group;
  const int gm = (num_m - m_first) < group ? (num_m - m_first) : group;
  n_blk = rem / gm;
  m_blk = m_first + (rem - n_blk * gm);
}

// Partial tiles in the workspace (split-K forms): per slot a [BN / 4][128] array of float4, i.e.
// groups of four columns outermost and the tile's rows innermost, so that the 32 lanes of a warp -
// which own consecutive rows - write and read 512 contiguous bytes per instruction (a row-major
// tile costs 32 separate 16-byte transactions per instruction and was measured at ~8 us per 128 KiB
// tile and direction).
template <int BN>
__device__ __forceinline__ float4* sk_partial_ptr(float* partial, int slot, int col4, int row) {
  return reinterpret_cast<float4*>(partial) + (static_cast<int64_t>(slot) * (BN / 4) + col4) * 128 + row;
}

// One CTA's work as a sequence of segments = (output tile, K-block range).
struct Segment {
  int m_blk, n_blk, kb_begin, kb_end;
  int tile;     // index of the tile in raster order
  bool first;   // first segment of this CTA
};

// A worker is one CTA, or one CTA pair in the pair kernels (both CTAs of a pair walk the same list).
struct SegCursor {
  int tile;          // next whole tile of the round-robin part
  int worker, nworkers;
  int group;         // row blocks per panel of the tile order
  bool tail_done;    // the tail range of this worker (SK kernels) has been handed out
  bool started;
};

template <int SK>
__device__ __forceinline__ SegCursor seg_begin(int worker, int nworkers) {
  SegCursor c;
  c.tile = worker;
  c.worker = worker;
  c.nworkers = nworkers;
  c.group = kRasterGroup;
  c.tail_done = false;
  c.started = false;
  return c;
}

// The tail range of this CTA: false if it has none.
__device__ __forceinline__ bool seg_tail(const GemmArgs& a, int worker, int num_m, int num_n, int num_kb, int num_tiles,
                                         Segment& s, int group = kRasterGroup) {
  const int u = worker;
  const int tail_tiles = num_tiles - a.sk_full;
  if (u >= tail_tiles * a.sk_split) return false;
  const int t = a.sk_full + u / a.sk_split;
  const int piece = u - (u / a.sk_split) * a.sk_split;
  tile_coords(t, num_m, num_n, s.m_blk, s.n_blk, group);
  s.kb_begin = piece * a.sk_kb_per;
  s.kb_end = s.kb_begin + a.sk_kb_per < num_kb ? s.kb_begin + a.sk_kb_per : num_kb;
  return s.kb_begin < s.kb_end;
}

// Number of K blocks this CTA processes in total.
template <int SK>
__device__ __forceinline__ uint32_t seg_total_kblocks(const GemmArgs& a, int worker, int nworkers, int num_m, int num_n,
                                                      int num_kb, int num_tiles) {
  const int whole_end = SK ? a.sk_full : num_tiles;
  int mine = 0;
  if (worker < whole_end) mine = (whole_end - worker + nworkers - 1) / nworkers;
  uint32_t total = static_cast<uint32_t>(mine) * static_cast<uint32_t>(num_kb);
  if constexpr (SK == 1) {
    Segment s;
    if (seg_tail(a, worker, num_m, num_n, num_kb, num_tiles, s)) total += static_cast<uint32_t>(s.kb_end - s.kb_begin);
  }
  return total;
}

template <int SK>
__device__ __forceinline__ bool seg_next(SegCursor& c, const GemmArgs& a, int num_m, int num_n, int num_kb, int num_tiles,
                                         Segment& s) {
  s.first = !c.started;
  const int whole_end = SK ? a.sk_full : num_tiles;
  c.started = true;
  if (c.tile < whole_end) {
    s.tile = c.tile;
    tile_coords(c.tile, num_m, num_n, s.m_blk, s.n_blk, c.group);
    s.kb_begin = 0;
    s.kb_end = num_kb;
    c.tile += c.nworkers;
    return true;
  }
  if constexpr (SK == 1) {
    if (!c.tail_done) {
      c.tail_done = true;
      return seg_tail(a, c.worker, num_m, num_n, num_kb, num_tiles, s, c.group);
    }
  }
  return false;
}

// Tensor maps of the destinations of the multi-destination kernel: byte matrices
// [M rows, N * element size] with box 32 rows x 128 bytes, SWIZZLE_128B.
struct DstMaps {
  CUtensorMap m[8];
};

// MULTI: the result leaves through the shared-memory staging area; MC (with MULTI): by
// multimem.st to a multicast address, otherwise by TMA stores to up to eight destinations.
// ROWB: B carries one scale per ROW and K block (the deep-gemm layout) instead of one per
// 128 x 128 block: the promotion multiplies every accumulator column by its own scale.
template <int BN, bool MULTI, int SK, bool MC = false, bool ROWB = false, int A_ROWS = 128, int PAIR = 0>
__device__ __forceinline__ void gemm_tile_body(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b,
                                               const GemmArgs& args, const CUtensorMap* dmaps,
                                               const CUtensorMap* tmap_bst = nullptr) {
  using Cfg = TileCfg<BN, MULTI, A_ROWS, PAIR>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr uint32_t TS = Cfg::TMEM_STAGES;
  constexpr uint32_t H = Cfg::HALVES;
  static_assert(!(PAIR && (MC || ROWB)), "pair kernels: block scales, plain or TMA-store output");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_stage = smem + STAGES * Cfg::STAGE_BYTES;
  static_assert(!(ROWB && MULTI), "the row-scaled kernel has one destination");
  float* rowb_table = reinterpret_cast<float*>(out_stage);   // ROWB: [kRowbTableKb][128] B scales of the current tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + (ROWB ? kRowbTableBytes : Cfg::OUT_STAGE_BYTES));
  uint64_t* full = bars;                  // [STAGES]  TMA bytes landed
  uint64_t* empty = bars + STAGES;        // [STAGES]  MMA finished reading the slot
  uint64_t* tfull = bars + 2 * STAGES;    // [TS * H]  TMEM stage (half) holds a finished K-block partial
  uint64_t* tempty = bars + 2 * STAGES + TS * H;  // [TS * H]  every epilogue warp has read the TMEM stage (half)
  uint64_t* sfull = bars + 2 * STAGES + 2 * TS * H;     // ROWB: the tile's scale table has landed
  uint64_t* sempty = sfull + 1;                           // ROWB: every promotion warp is done with the table
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * TS * H + 2);
  static_assert((2 * STAGES + 2 * TS * H + 2) * 8 + 8 <= Cfg::BAR_BYTES, "barrier area too small");
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Pair kernels: CTA 0 of the pair (the leader) issues the MMAs for both; its `full` barriers
  // collect the bytes of both CTAs' loads and its `tempty` barriers the arrivals of both CTAs'
  // promotion warps. `empty` and `tfull` exist in both CTAs and the leader signals each copy.
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0u;
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int nworkers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  // With a single block of rows and fewer than 97 of them (decode shapes) the upper TMEM lane
  // quarters hold rows that do not exist: the promotion warps of those quarters have nothing to
  // do and sit the kernel out (fewer instructions issued, and fewer arrivals per TMEM stage).
  const int live_quarters = (!PAIR && args.M <= 96) ? static_cast<int>((args.M + 31) / 32) : 4;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (uint32_t s = 0; s < TS * H; ++s) {
      mbar_init(&tfull[s], 1);
      mbar_init(&tempty[s], PAIR ? 2 * (Cfg::EPI_WARPS / H) : (Cfg::EPI_WARPS / 4) * live_quarters);
    }
    mbar_init(sfull, 1);
    mbar_init(sempty, (Cfg::EPI_WARPS / 4) * live_quarters);
    *abort_flag = 0u;
    fence_barrier_init();
  }
  if (warp == 2) {
    if constexpr (PAIR) {
      tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if constexpr (PAIR) {
    cluster_sync_all();   // the peer's barriers are initialised before anything arrives on them
  } else {
    __syncthreads();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int64_t M = args.M, N = args.N, K = args.K;
  const int num_m = static_cast<int>((M + Cfg::TILE_M - 1) / Cfg::TILE_M);
  const int num_n = static_cast<int>((N + BN - 1) / BN);
  const int num_kb = static_cast<int>((K + Cfg::BK - 1) / Cfg::BK);
  const int num_tiles = num_m * num_n;
  uint32_t* status_word = args.status_word;

  if (warp < 4) {
    if constexpr (Cfg::REBALANCE_REGS) setmaxnreg_dec<Cfg::REGS_CONTROL>();
  }
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tmap_a);
      prefetch_tmap(&tmap_b);
      // When A comes from the prep kernel of the same call (which may still be running: programmatic
      // dependent launch), the weight loads of the first K blocks do not wait for it: they are issued
      // at once, the A loads of those stages follow after griddepcontrol.wait.
      bool a_pending = args.a_from_prep != 0;
      if constexpr (PAIR) {
        // (pair kernels are not the decode path: they simply wait before their first load)
        if (a_pending) asm volatile("griddepcontrol.wait;" ::: "memory");
        a_pending = false;
      }
      uint32_t tile_no = 0;
      (void)tile_no;
      uint32_t pend_from = 0;
      int pend_kb0 = 0, pend_m0 = 0;
      const uint64_t pol_stream = policy_evict_first();
      const uint64_t pol_keep = policy_evict_last();
      uint32_t it = 0;
      bool ok = true;
      SegCursor cur = seg_begin<SK>(worker, nworkers);
      if constexpr (PAIR) cur.group = kRasterGroup / 2;   // 256-row tiles: the same 4096 rows per panel
      Segment seg;
      const uint32_t full_leader = PAIR ? mapa_shared(smem_u32(full), 0u) : 0u;
      while (ok && seg_next<SK>(cur, args, num_m, num_n, num_kb, num_tiles, seg)) {
        const int m0 = seg.m_blk * Cfg::TILE_M + static_cast<int>(cta_rank) * Cfg::BM;
        const int n0 = seg.n_blk * BN;
        if constexpr (ROWB) {
          if (args.rowb_table) {
            // the B scales of this tile: one box [K blocks x 128 columns] of the K-block-major copy, once
            // the promotion warps have let go of the previous tile's table
            if (!mbar_wait(sempty, (tile_no & 1u) ^ 1u, abort_flag, status_word)) { ok = false; break; }
            if (tile_no == 0) asm volatile("griddepcontrol.wait;" ::: "memory");   // the copy is written by the prep launch
            mbar_arrive_expect_tx(sfull, static_cast<uint32_t>(num_kb) * 512u);
            tma_load_2d(rowb_table, tmap_bst, sfull, n0, 0);
            ++tile_no;
          }
        }
        for (int kb = seg.kb_begin; kb < seg.kb_end; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, status_word)) { ok = false; break; }
          uint8_t* a_dst = smem + s * Cfg::STAGE_BYTES;
          uint8_t* b_dst = a_dst + Cfg::A_BYTES;
          if constexpr (PAIR) {
            // the leader's barrier counts the bytes of both CTAs' copies of this stage
            if (leader) mbar_arrive_expect_tx(&full[s], 2 * Cfg::STAGE_BYTES);
            const uint32_t fb = full_leader + s * 8u;
            tma_load_2d_pair(a_dst, &tmap_a, fb, kb * Cfg::BK, m0);
            if constexpr (PAIR == 1) {
              // B rows of the whole 256-column MMA: this CTA's half
              tma_load_2d_pair(b_dst, &tmap_b, fb, kb * Cfg::BK, n0 + static_cast<int>(cta_rank) * 128);
            } else {
              // two 128-column MMAs per K block: this CTA's 64 rows of each
#pragma unroll
              for (int h = 0; h < 2; ++h)
                tma_load_2d_pair(b_dst + h * 64 * Cfg::BK, &tmap_b, fb, kb * Cfg::BK,
                                 n0 + h * 128 + static_cast<int>(cta_rank) * 64);
            }
            continue;
          }
          mbar_arrive_expect_tx(&full[s], Cfg::STAGE_BYTES);
          // one M block: the weight is read exactly once, the few activation rows by every CTA
          const bool hinted = A_ROWS < 128 || num_m == 1;
          auto load_a = [&](uint32_t stage, int kb_a, int m0_a) {
            uint8_t* dst = smem + stage * Cfg::STAGE_BYTES;
            if (hinted) tma_load_2d_hint(dst, &tmap_a, &full[stage], kb_a * Cfg::BK, m0_a, pol_keep);
            else tma_load_2d(dst, &tmap_a, &full[stage], kb_a * Cfg::BK, m0_a);
          };
          if (hinted) tma_load_2d_hint(b_dst, &tmap_b, &full[s], kb * Cfg::BK, n0, pol_stream);
          else tma_load_2d(b_dst, &tmap_b, &full[s], kb * Cfg::BK, n0);
          if (!a_pending) {
            load_a(s, kb, m0);
          } else {
            if (it == pend_from) {
              pend_kb0 = kb;
              pend_m0 = m0;
            }
            if (it + 1 - pend_from == static_cast<uint32_t>(STAGES) || kb + 1 == seg.kb_end) {
              asm volatile("griddepcontrol.wait;" ::: "memory");
              a_pending = false;
              for (uint32_t j = pend_from; j <= it; ++j) load_a(j % STAGES, pend_kb0 + static_cast<int>(j - pend_from), pend_m0);
            }
          }
        }
      }
      if (!ok && leader) {
        // Abort path: let this CTA's own copies in flight land before shared memory is released
        // (pair kernels: the peer's copies are covered by the cluster barrier at the end).
        const uint32_t first = it > static_cast<uint32_t>(STAGES) ? it - STAGES : 0u;
        for (uint32_t j = first; j < it; ++j) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&full[j % STAGES], (j / STAGES) & 1u)) {
            if (globaltimer_ns() - t0 > kWaitLimitNs) break;
          }
        }
      }
    }
  } else if ((warp == 1 || warp == 3) && leader) {
    // ------------------------------------------------------------------ MMA issuers
    // Issuing the four tcgen05.mma of a K block, the two commits and the two barrier waits
    // costs an issuer some 650 clocks, while the tensor pipe needs 512 (BN = 256) or 256
    // (BN = 128) for that block. Two issuer warps therefore alternate: issuer p takes the
    // K blocks whose running index is p (mod 2). Consecutive K blocks use different smem
    // slots and different TMEM stages, so the two instruction streams are independent.
    // The whole warp runs the loop (addresses stay warp-uniform) and one elected lane issues.
    // Pair kernels: only the leader CTA issues; every commit is sent twice, once to each CTA's
    // copy of the barrier.
    const uint32_t p = (warp == 1) ? 0u : 1u;
    constexpr uint32_t idesc = make_idesc_e4m3_f32(Cfg::TILE_M, BN / H);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t empty_own = PAIR ? mapa_shared(smem_u32(empty), 0u) : 0u;
    const uint32_t empty_peer = PAIR ? mapa_shared(smem_u32(empty), 1u) : 0u;
    const uint32_t tfull_own = PAIR ? mapa_shared(smem_u32(tfull), 0u) : 0u;
    const uint32_t tfull_peer = PAIR ? mapa_shared(smem_u32(tfull), 1u) : 0u;
    uint32_t it = 0;
    uint32_t last = 0xffffffffu;
    bool ok = true;
    const uint32_t total_it = seg_total_kblocks<SK>(args, worker, nworkers, num_m, num_n, num_kb, num_tiles);
    {
      for (; it < total_it; ++it) {
        if ((it & 1u) != p) continue;
        const uint32_t s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1u;
        const uint32_t ts = it % TS;
        const uint32_t tph = (it / TS) & 1u;
        // operands first (they land long before), then the TMEM stage: nothing but the issue
        // itself is left to do once the epilogue hands the stage back
        const uint32_t a_addr = smem_base + s * Cfg::STAGE_BYTES;
        const uint64_t a_desc = make_smem_desc_sw128(a_addr);
        const uint64_t b_desc = make_smem_desc_sw128(a_addr + Cfg::A_BYTES);
        const uint32_t d_tmem = tmem_base + ts * BN;
        ok = __all_sync(0xffffffffu, mbar_wait(&full[s], ph, abort_flag, status_word));
        if (!ok) break;
#pragma unroll
        for (uint32_t h = 0; h < H; ++h) {
          ok = __all_sync(0xffffffffu, mbar_wait(&tempty[ts * H + h], tph ^ 1u, abort_flag, status_word));
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            if constexpr (PAIR) {
              // half h: this CTA's 64 (or, H = 1, 128) B rows sit h * 8 KiB into the B slot
              const uint64_t bh = b_desc + ((h * 64u * Cfg::BK) >> 4);
#pragma unroll
              for (int k = 0; k < Cfg::BK / 32; ++k)
                umma_f8_pair(d_tmem + h * (BN / H), a_desc + 2u * k, bh + 2u * k, idesc, k > 0 ? 1u : 0u);
              if (h + 1 == H) {
                tc_commit_pair(empty_own + s * 8u);
                tc_commit_pair(empty_peer + s * 8u);
              }
              tc_commit_pair(tfull_own + (ts * H + h) * 8u);
              tc_commit_pair(tfull_peer + (ts * H + h) * 8u);
            } else {
#pragma unroll
              for (int k = 0; k < Cfg::BK / 32; ++k) {
                // +2 in the start-address field = +32 bytes = one K=32 slice of e4m3
                umma_f8(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, k > 0 ? 1u : 0u);
              }
              tc_commit(&empty[s]);
              tc_commit(&tfull[ts]);
            }
          }
          __syncwarp();
        }
        if (!ok) break;
        last = it;
      }
    }
    if (!ok && last != 0xffffffffu && lane == 0) {
      // Abort path: bounded wait for the MMAs this warp already issued.
      const uint64_t t0 = globaltimer_ns();
      while (!mbar_try_wait(&tfull[(last % TS) * H + H - 1], (last / TS) & 1u)) {
        if (globaltimer_ns() - t0 > kWaitLimitNs) break;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ promotion + epilogue
    // (setmaxnreg is a warpgroup-wide instruction: the warps that sit out execute it too)
    if constexpr (Cfg::REBALANCE_REGS) setmaxnreg_inc<Cfg::REGS_EPILOGUE>();
    const int e = warp - 4;
    const int q = warp & 3;           // TMEM lane quarter this warp may read
    const int cw = e >> 2;            // which EPI_COLS-wide column slice of the tile
    const int num_nb = static_cast<int>((N + 127) / 128);
    constexpr int CHUNKS = Cfg::EPI_COLS / 32;
    const uint32_t lane_col = (static_cast<uint32_t>(q * 32) << 16) + cw * Cfg::EPI_COLS;
    uint32_t it = 0;
    uint32_t out_pass = 0;     // boxes this warp has staged so far (picks the staging buffer)
    (void)out_pass;
    uint32_t rowb_tile = 0;
    (void)rowb_tile;
    bool ok = (warp & 3) < live_quarters;
    // the scale copy AsT is written by the preceding tile_prep_kernel; with programmatic
    // dependent launch this kernel may have started before that grid finished
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // TMEM-full / TMEM-empty barrier of this warp's columns inside TMEM stage ts: index ts * H + hb
    const uint32_t hb = (H == 2) ? static_cast<uint32_t>(cw) : 0u;
    const uint32_t tempty_leader = PAIR ? mapa_shared(smem_u32(tempty), 0u) : 0u;
    auto release_stage = [&](uint32_t bar_idx) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(tempty_leader + bar_idx * 8u);
        else mbar_arrive(&tempty[bar_idx]);
      }
    };
    SegCursor cur = seg_begin<SK>(worker, nworkers);
      if constexpr (PAIR) cur.group = kRasterGroup / 2;   // 256-row tiles: the same 4096 rows per panel
    Segment seg;
    while (ok && seg_next<SK>(cur, args, num_m, num_n, num_kb, num_tiles, seg)) {
      const int m0 = seg.m_blk * Cfg::TILE_M + static_cast<int>(cta_rank) * Cfg::BM;
      const int n0 = seg.n_blk * BN;
      const int64_t row = static_cast<int64_t>(m0) + q * 32 + lane;
      const int col0 = n0 + cw * Cfg::EPI_COLS;
      int nb = col0 / 128;
      nb = nb < num_nb ? nb : num_nb - 1;
      // lanes of a warp own consecutive rows: K-block-major scales make this one coalesced
      // 128-byte load per warp and K block (row-major As would be 32 separate sectors)
      const float* as_col = args.AsT + row;
      const float* bs_row = args.Bs + static_cast<int64_t>(nb) * args.ld_bs;

      // accumulators as 32-column groups of pairs: acc[g][j] = columns 32 g + 2 j, + 1
      float2 acc[CHUNKS][16];
#pragma unroll
      for (int g = 0; g < CHUNKS; ++g)
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[g][j] = make_float2(0.f, 0.f);

      // Row-scaled B, BN = 128: this thread's 64 columns have 64 different B scales per K
      // block, the same for all lanes of the warp. They are fetched (16 broadcast loads of 16
      // bytes from the K-block-major copy) before the wait for the MMA, so that they arrive
      // while the warp waits; then acc += p * (sa * sb[col]) costs a multiply and an FMA.
      auto promote_rowb = [&](float sa, const float* sbt, bool from_smem) -> bool {
        static_assert(!ROWB || CHUNKS == 2, "row-scaled B is built for the 128-wide tile only");
        float4 sv[16];
        if (from_smem) {
#pragma unroll
          for (int i = 0; i < 16; ++i) sv[i] = reinterpret_cast<const float4*>(sbt)[i];   // same address in all lanes: broadcast
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) sv[i] = __ldg(reinterpret_cast<const float4*>(sbt) + i);
        }
        const uint32_t ts = it % TS;
        const uint32_t tph = (it / TS) & 1u;
        ++it;
        if (!__all_sync(0xffffffffu, mbar_wait(&tfull[ts], tph, abort_flag, status_word))) return false;
        tc_fence_after();
        const uint32_t taddr = tmem_base + lane_col + ts * BN;
        uint32_t pa[32], pb[32];
        tmem_ld_32x32(taddr, pa);
        tmem_ld_32x32(taddr + 32, pb);
        tmem_ld_wait_32(pa);
        tmem_ld_wait_32(pb);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[ts]);
#pragma unroll
        for (int g = 0; g < 2; ++g) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int c = 32 * g + 2 * j;
            const float4 s4 = sv[c >> 2];
            const float s_lo = (c & 2) ? s4.z : s4.x;
            const float s_hi = (c & 2) ? s4.w : s4.y;
            // two columns at a time: (sa * s_lo, sa * s_hi) and the accumulation are one packed instruction each
            ffma2(acc[g & (CHUNKS - 1)][j], g ? pb[2 * j] : pa[2 * j], g ? pb[2 * j + 1] : pa[2 * j + 1],
                  fmul2_bcast(s_lo, s_hi, sa));
          }
        }
        return true;
      };

      // One K block: wait for its partial in TMEM, pull it into registers (256-wide tile: two
      // 64-column loads; 128-wide tile: two 32-column loads in flight), hand the TMEM stage
      // back as soon as the last load has landed (before its FMAs).
      auto promote = [&](float sc) -> bool {
        const uint32_t ts = it % TS;
        const uint32_t tph = (it / TS) & 1u;
        ++it;
        if (!__all_sync(0xffffffffu, mbar_wait(&tfull[ts * H + hb], tph, abort_flag, status_word))) return false;
        tc_fence_after();
        const uint32_t taddr = tmem_base + lane_col + ts * BN;
        if constexpr (CHUNKS == 4) {
          // 256-wide tile: two 64-column loads, each followed by its 64 FMAs; the stage goes back
          // when the second has landed. Half the tcgen05.ld instructions of the 32-column form.
          uint32_t p[64];
          tmem_ld_32x64(taddr, p);
          tmem_ld_wait_64(p);
          fma64_scalar(acc[0], acc[1], p, sc);
          tmem_ld_32x64(taddr + 64, p);
          tmem_ld_wait_64(p);
          release_stage(ts * H + hb);
          fma64_scalar(acc[2 % CHUNKS], acc[3 % CHUNKS], p, sc);
          return true;
        }
        uint32_t pa[32], pb[32];
        tmem_ld_32x32(taddr, pa);
        tmem_ld_32x32(taddr + 32, pb);
        tmem_ld_wait_32(pa);
        tmem_ld_wait_32(pb);
#pragma unroll
        for (int g = 0; g < CHUNKS; g += 2) {
          const bool more = g + 2 < CHUNKS;
          if (!more) release_stage(ts * H + hb);
          fma32_scalar(acc[g], pa, sc);
          if (more) tmem_ld_32x32(taddr + (g + 2) * 32, pa);
          fma32_scalar(acc[g + 1], pb, sc);
          if (more) {
            tmem_ld_32x32(taddr + (g + 3) * 32, pb);
            tmem_ld_wait_32(pa);
            tmem_ld_wait_32(pb);
          }
        }
        return true;
      };

      // The scales AsT[kb][row] and Bs[nb, kb] come from global memory (L2 latency of several
      // hundred clocks). They are fetched a whole group of PF K blocks ahead so that their
      // first use never stalls the promotion loop.
      if constexpr (ROWB) {
        if (args.rowb_table) {
          ok = __all_sync(0xffffffffu, mbar_wait(sfull, rowb_tile & 1u, abort_flag, status_word));
          if (!ok) break;
        }
      }
      constexpr int PF = (CHUNKS == 2) ? 2 : 4;
      float sa_c[PF], sb_c[PF], sa_n[PF], sb_n[PF];
      const int kb_last = seg.kb_end - 1;
#pragma unroll
      for (int j = 0; j < PF; ++j) {
        const int k = seg.kb_begin + j < seg.kb_end ? seg.kb_begin + j : kb_last;
        sa_c[j] = __ldg(as_col + k * args.m_pad);
        sb_c[j] = ROWB ? 1.f : __ldg(bs_row + k);
      }
      for (int kb0 = seg.kb_begin; ok && kb0 < seg.kb_end; kb0 += PF) {
#pragma unroll
        for (int j = 0; j < PF; ++j) {
          int k = kb0 + PF + j;
          k = k < seg.kb_end ? k : kb_last;
          sa_n[j] = __ldg(as_col + k * args.m_pad);
          sb_n[j] = ROWB ? 1.f : __ldg(bs_row + k);
        }
#pragma unroll
        for (int j = 0; j < PF; ++j) {
          if (ok && kb0 + j < seg.kb_end) {
            if constexpr (ROWB) {
              ok = args.rowb_table
                       ? promote_rowb(sa_c[j], rowb_table + (kb0 + j) * 128 + cw * Cfg::EPI_COLS, true)
                       : promote_rowb(sa_c[j], args.BsT + static_cast<int64_t>(kb0 + j) * args.n_pad + col0, false);
            } else {
              ok = promote(sa_c[j] * sb_c[j]);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < PF; ++j) {
          sa_c[j] = sa_n[j];
          sb_c[j] = sb_n[j];
        }
      }
      if (!ok) break;
      if constexpr (ROWB) {
        if (args.rowb_table) {
          // done with this tile's scale table: the producer may load the next one
          __syncwarp();
          if (lane == 0) mbar_arrive(sempty);
          ++rowb_tile;
        }
      }

#define ACC(i) (((i) & 1) ? acc[(i) >> 5][((i) & 31) >> 1].y : acc[(i) >> 5][((i) & 31) >> 1].x)
      if (SK && (seg.kb_begin != 0 || seg.kb_end != num_kb)) {
        // tail split-K: this CTA saw only part of the K range - leave the fp32 partial sums of the
        // rows that exist in the workspace; tile_sk_fixup_kernel adds the ranges of the tile
        if (row < M) {
          float4* pcol = sk_partial_ptr<BN>(args.partial, static_cast<int>(blockIdx.x), cw * (Cfg::EPI_COLS / 4), q * 32 + lane);
#pragma unroll
          for (int j = 0; j < Cfg::EPI_COLS; j += 4)
            pcol[(j / 4) * Cfg::BM] = make_float4(ACC(j), ACC(j + 1), ACC(j + 2), ACC(j + 3));
        }
      } else if (MULTI && (MC || args.staged_store)) {
        // Multi-destination and multicast forms: per pass, 128 bytes of each of this warp's 32 rows
        // go to the warp's staging area in the SWIZZLE_128B pattern (16-byte chunk index XOR
        // row % 8, conflict-free for the row-wise writes).
        uint8_t* stage_base = out_stage + (warp - 4) * Cfg::OUT_STAGE_BYTES_PER_WARP;
        uint8_t* stage_w = stage_base;
        const int esize = args.out_fp32 ? 4 : 2;
        const int passes = Cfg::EPI_COLS * esize / 128;
        auto stage_pass = [&](int p) {
          if (args.out_fp32) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
              const int j0 = c * 4;
              // the pass index is a run-time value, the accumulator index must not be: select
              // over the unrolled candidates
#pragma unroll
              for (int pp = 0; pp < Cfg::EPI_COLS / 32; ++pp)
                if (pp == p) v4 = make_float4(ACC(pp * 32 + j0), ACC(pp * 32 + j0 + 1), ACC(pp * 32 + j0 + 2), ACC(pp * 32 + j0 + 3));
              *reinterpret_cast<float4*>(stage_w + lane * 128 + ((c ^ (lane & 7)) << 4)) = v4;
            }
          } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              uint4 u = make_uint4(0u, 0u, 0u, 0u);
              const int j0 = c * 8;
#pragma unroll
              for (int pp = 0; pp < Cfg::EPI_COLS / 64; ++pp)
                if (pp == p) {
                  __nv_bfloat162 v0 = __floats2bfloat162_rn(ACC(pp * 64 + j0), ACC(pp * 64 + j0 + 1));
                  __nv_bfloat162 v1 = __floats2bfloat162_rn(ACC(pp * 64 + j0 + 2), ACC(pp * 64 + j0 + 3));
                  __nv_bfloat162 v2 = __floats2bfloat162_rn(ACC(pp * 64 + j0 + 4), ACC(pp * 64 + j0 + 5));
                  __nv_bfloat162 v3 = __floats2bfloat162_rn(ACC(pp * 64 + j0 + 6), ACC(pp * 64 + j0 + 7));
                  u.x = *reinterpret_cast<uint32_t*>(&v0);
                  u.y = *reinterpret_cast<uint32_t*>(&v1);
                  u.z = *reinterpret_cast<uint32_t*>(&v2);
                  u.w = *reinterpret_cast<uint32_t*>(&v3);
                }
              *reinterpret_cast<uint4*>(stage_w + lane * 128 + ((c ^ (lane & 7)) << 4)) = u;
            }
          }
        };
        if constexpr (MC) {
          // Multicast destination: eight lanes per row read the staged row back as 16-byte chunks, so
          // that every 128-byte row segment leaves as one contiguous multimem.st request.
          const int64_t n_bytes = N * esize;
          uint8_t* mc_base = reinterpret_cast<uint8_t*>(args.dst[0]);
          const int64_t ld_bytes = args.dst_ld[0] * esize;
          for (int p = 0; p < passes; ++p) {
            __syncwarp();                                // the previous pass has been read back
            stage_pass(p);
            __syncwarp();
            const int c = lane & 7;
            const int64_t col_byte = static_cast<int64_t>(col0) * esize + p * 128 + c * 16;
            int64_t grow = static_cast<int64_t>(m0) + q * 32 + (lane >> 3);
            uint8_t* gptr = mc_base + grow * ld_bytes + col_byte;
            const bool col_ok = col_byte < n_bytes;
#pragma unroll 2
            for (int r = lane >> 3; r < 32; r += 4, grow += 4, gptr += 4 * ld_bytes) {
              const uint4 v = *reinterpret_cast<const uint4*>(stage_w + r * 128 + ((c ^ (r & 7)) << 4));
              if (col_ok && grow < M) multimem_st_v4(gptr, v);
            }
          }
        } else {
          // One TMA store per destination ships the 32 x 128-byte box; rows and columns beyond
          // [M, N] are clipped by the TMA.
          for (int p = 0; p < passes; ++p) {
            // the box that last used this staging buffer has been read out by the TMA
            if (lane == 0) {
              if constexpr (Cfg::OUT_BUFS == 2) bulk_wait_group_read1();
              else bulk_wait_group_read0();
            }
            __syncwarp();
            stage_w = stage_base + (out_pass % Cfg::OUT_BUFS) * Cfg::OUT_BOX_BYTES;
            ++out_pass;
            stage_pass(p);
            // generic-proxy writes above -> visible to the async proxy, then one lane sends the
            // box to every destination; the copies run on while the warp goes back to the K loop
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const int32_t col_byte = col0 * esize + p * 128;
              const int32_t row0 = m0 + q * 32;
              // evict-first in L2: the output is not read again here, and left to the default policy its
              // 300 MB push the operand panels out of the cache (measured with the hint: 8192 x 8192 x 1024
              // 102-107 vs 112-114 us, 4096 x 4096 x 8192 160-164 vs 164-168 us, 8192 x 18432 x 7168 -1 %)
              const uint64_t pol_out = policy_evict_first();
              for (int d = 0; d < args.n_dst; ++d) tma_store_2d_hint(&dmaps[d], stage_w, col_byte, row0, pol_out);
              bulk_commit_group();
            }
          }
        }
      } else
      if (row < M && col0 < N) {
        if (args.out_fp32) {
          float* crow = reinterpret_cast<float*>(args.C) + row * args.ldc + col0;
          if (col0 + Cfg::EPI_COLS <= N && (reinterpret_cast<uintptr_t>(crow) & 15u) == 0) {
#pragma unroll
            for (int j = 0; j < Cfg::EPI_COLS; j += 4)
              *reinterpret_cast<float4*>(crow + j) = make_float4(ACC(j), ACC(j + 1), ACC(j + 2), ACC(j + 3));
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::EPI_COLS; ++j)
              if (col0 + j < N) crow[j] = ACC(j);
          }
        } else {
          __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(args.C) + row * args.ldc + col0;
          if (col0 + Cfg::EPI_COLS <= N && (reinterpret_cast<uintptr_t>(crow) & 15u) == 0) {
#pragma unroll
            for (int j = 0; j < Cfg::EPI_COLS; j += 8) {
              __nv_bfloat162 v0 = __floats2bfloat162_rn(ACC(j), ACC(j + 1));
              __nv_bfloat162 v1 = __floats2bfloat162_rn(ACC(j + 2), ACC(j + 3));
              __nv_bfloat162 v2 = __floats2bfloat162_rn(ACC(j + 4), ACC(j + 5));
              __nv_bfloat162 v3 = __floats2bfloat162_rn(ACC(j + 6), ACC(j + 7));
              uint4 u;
              u.x = *reinterpret_cast<uint32_t*>(&v0);
              u.y = *reinterpret_cast<uint32_t*>(&v1);
              u.z = *reinterpret_cast<uint32_t*>(&v2);
              u.w = *reinterpret_cast<uint32_t*>(&v3);
              *reinterpret_cast<uint4*>(crow + j) = u;
            }
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::EPI_COLS; ++j)
              if (col0 + j < N) crow[j] = __float2bfloat16_rn(ACC(j));
          }
        }
      }
    }
  }
#undef ACC

  // ------------------------------------------------------------------ teardown
  if constexpr (MULTI) {
    // the output copies of this warp must be complete (written) before the CTA exits
    if (!MC && warp >= 4 && lane == 0) bulk_wait_group0();
    if (MC && warp >= 4) __threadfence_system();   // multimem stores ordered before the kernel's end
  }
  __syncwarp();
  tc_fence_before();
  if constexpr (PAIR) {
    // neither CTA may leave (its shared memory and TMEM are read and signalled by the other) before both are done
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BN, int SK>
__global__ void __launch_bounds__(TileCfg<BN, false>::THREADS, 1)
gemm_tile_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmArgs args) {
  gemm_tile_body<BN, false, SK>(tmap_a, tmap_b, args, nullptr);
}

// CTA-pair forms (launch with cluster dimension 2 and an even grid): 256 x 256 tiles per pair.
// SPLIT = false: one 256-column MMA chain per K block; true: two 128-column halves.
template <bool SPLIT>
__global__ void __launch_bounds__(TileCfg<256, false>::THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmArgs args) {
  gemm_tile_body<256, false, 0, false, false, 128, SPLIT ? 2 : 1>(tmap_a, tmap_b, args, nullptr);
}

// The split pair form with the last, partly empty wave of tiles cut into K ranges, one per idle pair
// (variant pair256_split_sk): whole tiles leave through the staging area as in gemm_pair_multi_kernel,
// a K range leaves as two fp32 partial tiles (one per CTA) for tile_sk_fixup_kernel.
__global__ void __launch_bounds__(TileCfg<256, true>::THREADS, 1)
gemm_pair_multi_sk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const GemmArgs args, const __grid_constant__ DstMaps dmaps) {
  gemm_tile_body<256, true, 1, false, false, 128, 2>(tmap_a, tmap_b, args, dmaps.m);
}

template <bool SPLIT>
__global__ void __launch_bounds__(TileCfg<256, true>::THREADS, 1)
gemm_pair_multi_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const GemmArgs args, const __grid_constant__ DstMaps dmaps) {
  gemm_tile_body<256, true, 0, false, false, 128, SPLIT ? 2 : 1>(tmap_a, tmap_b, args, dmaps.m);
}

// Multi-destination form: the finished tile is staged in shared memory and sent to every
// destination (this GPU's and its peers' output buffers) by asynchronous TMA stores.
template <int BN>
__global__ void __launch_bounds__(TileCfg<BN, true>::THREADS, 1)
gemm_tile_multi_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const GemmArgs args, const __grid_constant__ DstMaps dmaps) {
  gemm_tile_body<BN, true, 0>(tmap_a, tmap_b, args, dmaps.m);
}

// Decode forms: 16-row A slots and six pipeline stages (M <= 16), 64-row slots and five (M <= 64).
template <int BN, int A_ROWS>
__global__ void __launch_bounds__(TileCfg<BN, false>::THREADS, 1)
gemm_tile_decode_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const GemmArgs args) {
  gemm_tile_body<BN, false, 0, false, false, A_ROWS>(tmap_a, tmap_b, args, nullptr);
}

// Row-scaled B (deep-gemm layout): single destination, 128-wide tiles.
template <int BN>
__global__ void __launch_bounds__(TileCfg<BN, false>::THREADS, 1)
gemm_tile_rowb_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_bst, const GemmArgs args) {
  gemm_tile_body<BN, false, 0, false, true>(tmap_a, tmap_b, args, nullptr, &tmap_bst);
}

// Multicast form: args.dst[0] is a multimem address; every 128-byte row segment of a finished
// tile is written once with multimem.st and replicated into all GPUs' buffers by the NVSwitch.
template <int BN>
__global__ void __launch_bounds__(TileCfg<BN, true>::THREADS, 1)
gemm_tile_mc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmArgs args) {
  gemm_tile_body<BN, true, 0, true>(tmap_a, tmap_b, args, nullptr);
}

// Prep kernel of b200fp8_linear: quantises the bf16 activations (same arithmetic as
// quant_act_contig_kernel, so the bytes and scales are identical to b200fp8_quant_act's) and
// writes them where the GEMM kernel wants them: e4m3 rows into `Aq` (row pitch ldq, at least 16
// rows, rows >= M zero) and the scales K-block-major into AsT[kb][m_pad] (rows >= M zero).
// K is a multiple of 128. Eight threads per 128-element group; groups = m_pad x K/128.
__global__ void __launch_bounds__(256)
tile_prep_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, uint8_t* __restrict__ Aq, int64_t ldq,
                       int64_t rows_q, float* __restrict__ AsT, int64_t M, int64_t m_pad, int num_kb) {
  asm volatile("griddepcontrol.launch_dependents;");
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  const int64_t g = t >> 3;
  const int sub = threadIdx.x & 7;
  const int64_t row = g / num_kb;                 // whole warps share a row quadruple: m_pad * num_kb is a multiple of 4
  const int kg = static_cast<int>(g - row * num_kb);
  if (row >= m_pad) return;
  uint4 v[2];
  v[0] = make_uint4(0u, 0u, 0u, 0u);
  v[1] = make_uint4(0u, 0u, 0u, 0u);
  if (row < M) {
    const uint4* src = reinterpret_cast<const uint4*>(x + row * ldx + kg * 128 + sub * 16);
    v[0] = __ldg(src);
    v[1] = __ldg(src + 1);
  }
  float amax = fmax_nan(amax8(v[0]), amax8(v[1]));
  amax = fmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  const float scale = scale_of_amax(amax);
  uint2 o[2];
  quant_vecs<2>(v, scale, o);
  if (row < rows_q)
    *reinterpret_cast<uint4*>(Aq + row * ldq + kg * 128 + sub * 16) = make_uint4(o[0].x, o[0].y, o[1].x, o[1].y);
  if (sub == 0) AsT[static_cast<int64_t>(kg) * m_pad + row] = scale;
}

// Tail split-K: adds the K ranges of every tail tile (ascending range order: fixed, hence
// bit-reproducible) and writes C. Grid = (tail tiles, chunks of 32 rows: 4, or 8 for pair tiles,
// 4 quarters of 64 columns); 256 threads. Phase 1: warp w sums the float4 column groups 2 w and
// 2 w + 1 of the quarter for the chunk's 32 rows (lane = row: 512 contiguous bytes per load in the
// partial-tile layout of sk_partial_ptr; the loads of all ranges are independent and go out
// together) and parks the sums in shared memory; phase 2: warp w writes rows w, w + 8, ... with
// lane l holding columns 2 l, 2 l + 1, so that C leaves in whole 128-byte (bf16) or 256-byte
// (fp32) row segments. Launched with programmatic stream serialisation: it may be scheduled
// while the GEMM drains, and waits for it here before it reads.
__global__ void __launch_bounds__(256)
tile_sk_fixup_kernel(const float* __restrict__ partial, void* C, int64_t M, int64_t N, int num_kb, int64_t ldc,
                     int out_fp32, int num_m, int num_n, int sk_full, int sk_split, int sk_kb_per, int pair) {
  // pair != 0: the tiles are 256 rows tall and each K range was left by the two CTAs of a pair, rows
  // 0..127 in slot 2 u and rows 128..255 in slot 2 u + 1 of range u (grid.y = 8 instead of 4)
  constexpr int BN = 256;
  constexpr int QN = 64;                        // columns per CTA
  constexpr int PITCH = QN + 1;                 // floats per staged row: column c of row r sits in bank (r + c) % 32
  __shared__ float stage[32 * PITCH];
  asm volatile("griddepcontrol.wait;" ::: "memory");
  int m_blk, n_blk;
  tile_coords(sk_full + static_cast<int>(blockIdx.x), num_m, num_n, m_blk, n_blk, pair ? kRasterGroup / 2 : kRasterGroup);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(blockIdx.y) >> 2;
  const int r0 = (blockIdx.y & 3) * 32;
  const int cq = static_cast<int>(blockIdx.z);   // column quarter
  const int64_t row0 = static_cast<int64_t>(m_blk) * (pair ? 256 : 128) + rank * 128 + r0;
  if (row0 >= M) return;
  float4 sum[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  if (row0 + lane < M) {
    for (int j = 0; j < sk_split; ++j) {
      if (j * sk_kb_per >= num_kb) break;   // empty range: nothing was written
      const int unit = static_cast<int>(blockIdx.x) * sk_split + j;
      const int slot = pair ? 2 * unit + rank : unit;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int c4 = cq * (QN / 4) + 2 * warp + i;
        const float4 v = __ldg(reinterpret_cast<const float4*>(partial) + (static_cast<int64_t>(slot) * (BN / 4) + c4) * 128 + r0 + lane);
        sum[i].x += v.x;
        sum[i].y += v.y;
        sum[i].z += v.z;
        sum[i].w += v.w;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float* dst = stage + lane * PITCH + (2 * warp + i) * 4;
    dst[0] = sum[i].x;
    dst[1] = sum[i].y;
    dst[2] = sum[i].z;
    dst[3] = sum[i].w;
  }
  __syncthreads();
  const int64_t col0 = static_cast<int64_t>(n_blk) * BN + cq * QN + lane * 2;
  for (int r = warp; r < 32; r += 8) {
    const int64_t row = row0 + r;
    if (row >= M) break;
    const float v0 = stage[r * PITCH + lane * 2], v1 = stage[r * PITCH + lane * 2 + 1];
    if (out_fp32) {
      float* crow = reinterpret_cast<float*>(C) + row * ldc + col0;
      if (col0 + 2 <= N && (reinterpret_cast<uintptr_t>(crow) & 7u) == 0) {
        *reinterpret_cast<float2*>(crow) = make_float2(v0, v1);
      } else {
        if (col0 < N) crow[0] = v0;
        if (col0 + 1 < N) crow[1] = v1;
      }
    } else {
      __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(C) + row * ldc + col0;
      if (col0 + 2 <= N && (reinterpret_cast<uintptr_t>(crow) & 3u) == 0) {
        *reinterpret_cast<__nv_bfloat162*>(crow) = __floats2bfloat162_rn(v0, v1);
      } else {
        if (col0 < N) crow[0] = __float2bfloat16_rn(v0);
        if (col0 + 1 < N) crow[1] = __float2bfloat16_rn(v1);
      }
    }
  }
}

// Barrier between the GPUs of a node after a multi-destination GEMM: one warp per GPU. Lane p
// (p < n) stores `epoch` into slot `rank` of GPU p's flag array (a release store at system scope
// over NVLink), then polls slot p of its own array until GPU p's store of the same epoch has
// arrived. Epochs only grow, so a late reader never misses one (comparison is wrap-safe).
// The wait is bounded by `limit_clocks` SM clocks (default ~10 s, generous because the ranks' hosts
// may be seconds apart at start-up); on expiry the status word gets B200FP8_DEV_WAIT_TIMEOUT and
// the kernel returns normally. The kernels of different GPUs wait on one another: never run two
// ranks on one GPU.
struct PeerFlags {
  uint32_t* p[8];
};

constexpr long long kPeerBarrierDefaultLimitClks = 20000000000ll;

__global__ void __launch_bounds__(32)
peer_barrier_kernel(PeerFlags flags, int n, int rank, uint32_t epoch, long long limit_clocks, uint32_t* status_word) {
  const int lane = threadIdx.x;
  if (lane >= n) return;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[lane] + rank), "r"(epoch) : "memory");
  const uint32_t* mine = flags.p[rank] + lane;
  const long long t0 = clock64();
  for (uint32_t polls = 0;; ++polls) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (static_cast<int32_t>(v - epoch) >= 0) break;
    if ((polls & 255u) == 255u && clock64() - t0 > limit_clocks) {
      if (status_word != nullptr) atomicOr(status_word, B200FP8_DEV_WAIT_TIMEOUT);
      break;
    }
  }
}

// Launch-side preparation of one GEMM call, grid = (m_pad / 32, ceil(num_kb / 32), 1 or 2):
//   z = 0  AsT[kb][m] = As[m][kb] for m < M, 0 for M <= m < m_pad: 32 x 32 tiles through
//          shared memory so that both the row-major reads and the K-block-major writes are
//          coalesced;
//   z = 1  (only when M <= 16) A_pad[16][lda_pad] = A with zero rows appended: TMA boxes over a
//          tensor of fewer than 16 rows measured ~20 % slower on B200 than over 16 rows.
__global__ void __launch_bounds__(256)
tile_prep_kernel(const float* __restrict__ As, float* __restrict__ AsT, int64_t M, int64_t m_pad, int num_kb,
                 int64_t ld_as, const uint8_t* __restrict__ A, uint8_t* __restrict__ A_pad, int64_t K, int64_t lda,
                 int64_t lda_pad) {
  // let the GEMM kernel that follows (launched with programmatic stream serialisation) start
  // its prologue now; the warps that read what this grid writes wait for it (griddepcontrol.wait)
  asm volatile("griddepcontrol.launch_dependents;");
  if (blockIdx.z == 1) {
    const int64_t chunks_per_row = lda_pad / 16;
    const int64_t total = 16 * chunks_per_row;
    const int64_t nthreads = static_cast<int64_t>(gridDim.x) * gridDim.y * blockDim.x;
    for (int64_t i = (static_cast<int64_t>(blockIdx.y) * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += nthreads) {
      const int64_t r = i / chunks_per_row, c = (i - r * chunks_per_row) * 16;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < M) {
        if (c + 16 <= K) {
          v = __ldg(reinterpret_cast<const uint4*>(A + r * lda + c));
        } else {
          uint8_t b[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) b[j] = (c + j < K) ? A[r * lda + c + j] : uint8_t(0);
          memcpy(&v, b, 16);
        }
      }
      *reinterpret_cast<uint4*>(A_pad + r * lda_pad + c) = v;
    }
    return;
  }
  __shared__ float t[32][33];
  const int64_t m0 = static_cast<int64_t>(blockIdx.x) * 32;
  const int kb0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    const int64_t m = m0 + ty + i;
    const int kb = kb0 + tx;
    t[ty + i][tx] = (m < M && kb < num_kb) ? __ldg(As + m * ld_as + kb) : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    const int kb = kb0 + ty + i;
    const int64_t m = m0 + tx;
    if (kb < num_kb && m < m_pad) AsT[static_cast<int64_t>(kb) * m_pad + m] = t[tx][ty + i];
  }
}

// C[M,N] = 0 for the degenerate K == 0 product.
__global__ void gemm_zero_fill_kernel(void* C, int64_t M, int64_t N, int64_t ldc, int out_fp32) {
  const int64_t total = M * N;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / N, c = i % N;
    if (out_fp32)
      reinterpret_cast<float*>(C)[r * ldc + c] = 0.f;
    else
      reinterpret_cast<__nv_bfloat16*>(C)[r * ldc + c] = __float2bfloat16_rn(0.f);
  }
}

}  // namespace b200fp8
