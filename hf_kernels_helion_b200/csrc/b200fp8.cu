// C ABI of the block-FP8 hot path (declarations and contracts: include/b200fp8.h).
// Host side only validates, builds TMA descriptors and launches; nothing here
// allocates, frees or synchronises.
#include "../../include/b200fp8.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstring>
#include <mutex>

#include "gemm_streamk.cuh"
#include "gemm_tile.cuh"
#include "quant.cuh"

namespace {

using namespace b200fp8;

constexpr int kMaxDevices = 64;

struct DeviceInfo {
  std::atomic<int> ready{0};
  int cc_major = 0;
  int sm_count = 0;
  int pair_clusters = 0;   // CTA pairs of the pair kernels that can be resident at once
};
DeviceInfo g_dev[kMaxDevices];
std::mutex g_mutex;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::atomic<EncodeTiledFn> g_encode{nullptr};

// Per-device facts, read once; also opts every kernel into its dynamic shared memory size.
int device_info(const DeviceInfo** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200FP8_ERR_ARCH;
  DeviceInfo& d = g_dev[dev];
  if (!d.ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!d.ready.load(std::memory_order_relaxed)) {
      if (cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
          cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return B200FP8_ERR_ARCH;
      if (d.cc_major != 10) return B200FP8_ERR_ARCH;
      bool ok = true;
      auto opt_in = [&ok](const void* fn, int bytes) {
        ok = ok && cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
      };
      // setmaxnreg.inc blocks until registers are free: refuse to run a kernel whose compiled
      // register count (what the launch allocates) cannot cover its own re-balancing plan
      auto regs_ok = [&ok](const void* fn, int threads, int regs_needed_total) {
        cudaFuncAttributes attr;
        ok = ok && cudaFuncGetAttributes(&attr, fn) == cudaSuccess && attr.numRegs * threads >= regs_needed_total;
      };
      regs_ok(reinterpret_cast<const void*>(&gemm_tile_kernel<256, 0>), TileCfg<256>::THREADS,
              128 * TileCfg<256>::REGS_CONTROL + 256 * TileCfg<256>::REGS_EPILOGUE);
      regs_ok(reinterpret_cast<const void*>(&gemm_tile_multi_kernel<256>), TileCfg<256>::THREADS,
              128 * TileCfg<256>::REGS_CONTROL + 256 * TileCfg<256>::REGS_EPILOGUE);
      regs_ok(reinterpret_cast<const void*>(&gemm_streamk_kernel<256>), StreamKCfg<256>::THREADS,
              128 * StreamKCfg<256>::REGS_CONTROL + 256 * StreamKCfg<256>::REGS_EPILOGUE);
      opt_in(reinterpret_cast<const void*>(&gemm_tile_kernel<128, 0>), TileCfg<128, false>::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_tile_kernel<256, 0>), TileCfg<256, false>::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_tile_multi_kernel<128>), TileCfg<128, true>::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_tile_multi_kernel<256>), TileCfg<256, true>::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_tile_rowb_kernel<128>), TileCfg<128, false>::SMEM_BYTES + kRowbTableBytes);
      regs_ok(reinterpret_cast<const void*>(&gemm_tile_rowb_kernel<128>), TileCfg<128>::THREADS,
              128 * TileCfg<128>::REGS_CONTROL + 256 * TileCfg<128>::REGS_EPILOGUE);
      regs_ok(reinterpret_cast<const void*>(&gemm_tile_kernel<128, 0>), TileCfg<128>::THREADS,
              128 * TileCfg<128>::REGS_CONTROL + 256 * TileCfg<128>::REGS_EPILOGUE);
      regs_ok(reinterpret_cast<const void*>(&gemm_tile_multi_kernel<128>), TileCfg<128>::THREADS,
              128 * TileCfg<128>::REGS_CONTROL + 256 * TileCfg<128>::REGS_EPILOGUE);
      regs_ok(reinterpret_cast<const void*>(&gemm_tile_mc_kernel<128>), TileCfg<128>::THREADS,
              128 * TileCfg<128>::REGS_CONTROL + 256 * TileCfg<128>::REGS_EPILOGUE);
      opt_in(reinterpret_cast<const void*>(&gemm_tile_mc_kernel<128>), TileCfg<128, true>::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_tile_mc_kernel<256>), TileCfg<256, true>::SMEM_BYTES);
      regs_ok(reinterpret_cast<const void*>(&gemm_tile_mc_kernel<256>), TileCfg<256>::THREADS,
              128 * TileCfg<256>::REGS_CONTROL + 256 * TileCfg<256>::REGS_EPILOGUE);
      opt_in(reinterpret_cast<const void*>(&gemm_tile_decode_kernel<256, 16>), TileCfg<256, false, 16>::SMEM_BYTES);
      regs_ok(reinterpret_cast<const void*>(&gemm_tile_decode_kernel<256, 16>), TileCfg<256>::THREADS,
              128 * TileCfg<256>::REGS_CONTROL + 256 * TileCfg<256>::REGS_EPILOGUE);
      opt_in(reinterpret_cast<const void*>(&gemm_tile_decode_kernel<256, 64>), TileCfg<256, false, 64>::SMEM_BYTES);
      regs_ok(reinterpret_cast<const void*>(&gemm_tile_decode_kernel<256, 64>), TileCfg<256>::THREADS,
              128 * TileCfg<256>::REGS_CONTROL + 256 * TileCfg<256>::REGS_EPILOGUE);
      opt_in(reinterpret_cast<const void*>(&gemm_tile_kernel<256, 1>), TileCfg<256, false>::SMEM_BYTES);
      regs_ok(reinterpret_cast<const void*>(&gemm_tile_kernel<256, 1>), TileCfg<256>::THREADS,
              128 * TileCfg<256>::REGS_CONTROL + 256 * TileCfg<256>::REGS_EPILOGUE);
      using PairCfg = TileCfg<256, false, 128, 1>;
      using PairMultiCfg = TileCfg<256, true, 128, 1>;
      opt_in(reinterpret_cast<const void*>(&gemm_pair_kernel<false>), PairCfg::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_pair_kernel<true>), PairCfg::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_pair_multi_kernel<false>), PairMultiCfg::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_pair_multi_kernel<true>), PairMultiCfg::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_pair_multi_sk_kernel), PairMultiCfg::SMEM_BYTES);
      regs_ok(reinterpret_cast<const void*>(&gemm_pair_kernel<false>), PairCfg::THREADS,
              128 * PairCfg::REGS_CONTROL + 256 * PairCfg::REGS_EPILOGUE);
      regs_ok(reinterpret_cast<const void*>(&gemm_pair_kernel<true>), PairCfg::THREADS,
              128 * PairCfg::REGS_CONTROL + 256 * PairCfg::REGS_EPILOGUE);
      regs_ok(reinterpret_cast<const void*>(&gemm_pair_multi_kernel<false>), PairCfg::THREADS,
              128 * PairCfg::REGS_CONTROL + 256 * PairCfg::REGS_EPILOGUE);
      regs_ok(reinterpret_cast<const void*>(&gemm_pair_multi_kernel<true>), PairCfg::THREADS,
              128 * PairCfg::REGS_CONTROL + 256 * PairCfg::REGS_EPILOGUE);
      regs_ok(reinterpret_cast<const void*>(&gemm_pair_multi_sk_kernel), PairCfg::THREADS,
              128 * PairCfg::REGS_CONTROL + 256 * PairCfg::REGS_EPILOGUE);
      if (ok) {
        // how many CTA pairs fit on the device at once (one CTA per SM; not every SM need be pairable)
        cudaLaunchAttribute cattr[1];
        cattr[0].id = cudaLaunchAttributeClusterDimension;
        cattr[0].val.clusterDim.x = 2;
        cattr[0].val.clusterDim.y = 1;
        cattr[0].val.clusterDim.z = 1;
        cudaLaunchConfig_t ccfg = {};
        ccfg.gridDim = dim3(static_cast<unsigned>(d.sm_count & ~1));
        ccfg.blockDim = dim3(PairCfg::THREADS);
        ccfg.dynamicSmemBytes = PairMultiCfg::SMEM_BYTES;
        ccfg.attrs = cattr;
        ccfg.numAttrs = 1;
        int n_clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&n_clusters, gemm_pair_multi_kernel<true>, &ccfg) != cudaSuccess) {
          cudaGetLastError();
          n_clusters = 0;
        }
        d.pair_clusters = n_clusters < d.sm_count / 2 ? n_clusters : d.sm_count / 2;
      }
      opt_in(reinterpret_cast<const void*>(&gemm_streamk_kernel<16>), StreamKCfg<16>::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_streamk_kernel<32>), StreamKCfg<32>::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_streamk_kernel<64>), StreamKCfg<64>::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_streamk_kernel<128>), StreamKCfg<128>::SMEM_BYTES);
      opt_in(reinterpret_cast<const void*>(&gemm_streamk_kernel<256>), StreamKCfg<256>::SMEM_BYTES);
      if (!ok) {
        cudaGetLastError();
        return B200FP8_ERR_LAUNCH;
      }
      d.ready.store(1, std::memory_order_release);
    }
  }
  *out = &d;
  return B200FP8_OK;
}

int sm_count_or_default() {
  const DeviceInfo* d = nullptr;
  if (device_info(&d) == B200FP8_OK) return d->sm_count;
  cudaGetLastError();
  return 148;  // B200
}

EncodeTiledFn encode_fn() {
  EncodeTiledFn fn = g_encode.load(std::memory_order_acquire);
  if (fn != nullptr) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || sym == nullptr) {
    cudaGetLastError();
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  g_encode.store(fn, std::memory_order_release);
  return fn;
}

// 2-D tensor map over a row-major byte matrix [rows, cols] with row stride ld (bytes),
// box = [box_rows x 128 bytes], 128-byte swizzle, zero fill outside the matrix.
// A tensor map is a pure function of (base, rows, cols, ld, box_rows): the last few are kept per
// host thread (no lock, no shared mutable state) so that a caller that repeats a shape - a decode
// loop, a captured graph being re-recorded - does not pay the driver's encoder on every call.
struct TmapKey {
  const void* base;
  int64_t rows, cols, ld;
  uint32_t box_rows;
  int kind;   // 0: byte matrix, 128-byte boxes, SWIZZLE_128B; 1: fp32 matrix, 128-element boxes, no swizzle
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && kind == o.kind;
  }
};
constexpr int kTmapCacheEntries = 16;
struct TmapCache {
  TmapKey key[kTmapCacheEntries];
  CUtensorMap map[kTmapCacheEntries];
  int used = 0, next = 0;
};
thread_local TmapCache t_tmap_cache;

// kind 0: byte matrix [rows, cols], ld in bytes; kind 1: fp32 matrix [rows, cols], ld in bytes, box = [box_rows x 128 floats]
int make_tmap(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, uint32_t box_rows, int kind) {
  const TmapKey k = {base, rows, cols, ld, box_rows, kind};
  TmapCache& c = t_tmap_cache;
  for (int i = 0; i < c.used; ++i)
    if (c.key[i] == k) {
      *map = c.map[i];
      return B200FP8_OK;
    }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return B200FP8_ERR_DRIVER;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld)};
  const cuuint32_t box[2] = {128u, box_rows};
  const cuuint32_t elem[2] = {1u, 1u};
  const CUresult r = fn(map, kind == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                        const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        kind == 1 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return B200FP8_ERR_DRIVER;
  const int slot = c.used < kTmapCacheEntries ? c.used++ : c.next;
  c.next = (slot + 1) % kTmapCacheEntries;
  c.key[slot] = k;
  c.map[slot] = *map;
  return B200FP8_OK;
}

int make_tmap_u8(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, uint32_t box_rows) {
  return make_tmap(map, base, rows, cols, ld, box_rows, 0);
}

int launch_status() { return cudaGetLastError() == cudaSuccess ? B200FP8_OK : B200FP8_ERR_LAUNCH; }

// Scratch of b200fp8_gemm_decode_static: lives in the module image of every device that
// loads the library, from load until process exit. In host code the NAME of a __device__
// array is only a host-side stand-in, not a device address; the address a kernel may use
// comes from cudaGetSymbolAddress, taken once per device with that device current.
constexpr size_t kStaticScratchBytes = B200FP8_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
std::atomic<void*> g_static_scratch_addr[kMaxDevices];

int static_scratch_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200FP8_ERR_ARCH;
  void* p = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return B200FP8_ERR_DRIVER;
    }
    g_static_scratch_addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return B200FP8_OK;
}

int streamk_mp(int64_t M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

struct StreamKPlan {
  int mp;
  int num_kb;
  int64_t num_tiles;
  int64_t grid;
  int64_t ast_bytes;      // AsT region (first)
  int64_t partial_bytes;  // partial-sum region (second)
};

StreamKPlan streamk_plan(int64_t M, int64_t N, int64_t K, int sm_count) {
  StreamKPlan p;
  p.mp = streamk_mp(M);
  p.num_kb = static_cast<int>((K + 127) / 128);
  p.num_tiles = (N + 127) / 128;
  const int64_t total = p.num_tiles * p.num_kb;
  p.grid = total < sm_count ? total : sm_count;
  if (p.grid < 1) p.grid = 1;
  p.ast_bytes = align_up(static_cast<int64_t>(p.num_kb) * p.mp * 4, 256);
  p.partial_bytes = 2 * p.grid * p.mp * 128 * 4;
  return p;
}

// tile variants: AsT [ceil(K/128)][M rounded up to 128] fp32
int64_t tile_ast_bytes(int64_t M, int64_t K) { return align_up(((K + 127) / 128) * align_up(M, 128) * 4, 256); }
// + a 16-row copy of A (zero-padded) when M <= 16
int64_t tile_workspace_bytes(int64_t M, int64_t K) {
  if (M == 0 || K == 0) return 0;
  return tile_ast_bytes(M, K) + (M <= 16 ? 16 * align_up(K, 16) : 0);
}

// b200fp8_linear: scales K-block-major + the quantised activations (at least 16 rows, 16-byte row pitch)
int64_t linear_prefix_bytes(int64_t M, int64_t K) {
  if (M == 0 || K == 0) return 0;
  return tile_ast_bytes(M, K) + align_up((M < 16 ? 16 : M) * align_up(K, 16), 256);
}

// 128x256 tiles with the last, partly empty wave split along K (B200FP8_VARIANT_TILE256_SK)
struct TileSkPlan {
  int num_m, num_n, num_kb;
  int full;      // tiles handed out whole, round-robin
  int tail;      // remaining tiles (< grid)
  int split;     // K ranges per tail tile; < 2 means the shape gains nothing and runs as plain tiles
  int kb_per;    // K blocks per range
  int64_t grid;
  int64_t ast_bytes, partial_bytes;
};

TileSkPlan tile_sk_plan(int64_t M, int64_t N, int64_t K, int sm_count) {
  TileSkPlan p;
  p.num_m = static_cast<int>((M + 127) / 128);
  p.num_n = static_cast<int>((N + 255) / 256);
  p.num_kb = static_cast<int>((K + 127) / 128);
  const int64_t tiles = static_cast<int64_t>(p.num_m) * p.num_n;
  p.grid = sm_count;
  p.full = static_cast<int>((tiles / sm_count) * sm_count);
  p.tail = static_cast<int>(tiles - p.full);
  p.split = p.tail > 0 ? sm_count / p.tail : 1;
  if (p.split > p.num_kb / 4) p.split = p.num_kb / 4;   // keep ranges of at least 4 K blocks
  if (p.split < 1) p.split = 1;
  p.kb_per = (p.num_kb + p.split - 1) / p.split;
  p.ast_bytes = tile_workspace_bytes(M, K);
  p.partial_bytes = p.split >= 2 ? static_cast<int64_t>(p.tail) * p.split * 128 * 256 * 4 : 0;
  return p;
}

// The same for 256 x 256 tiles on CTA pairs (B200FP8_VARIANT_PAIR256_SPLIT_SK): the workers are the pairs,
// and every K range leaves two partial tiles (one per CTA of the pair).
TileSkPlan pair_sk_plan(int64_t M, int64_t N, int64_t K, int pairs) {
  TileSkPlan p;
  p.num_m = static_cast<int>((M + 255) / 256);
  p.num_n = static_cast<int>((N + 255) / 256);
  p.num_kb = static_cast<int>((K + 127) / 128);
  const int64_t tiles = static_cast<int64_t>(p.num_m) * p.num_n;
  if (pairs < 1) pairs = 1;
  p.grid = 2 * static_cast<int64_t>(pairs);
  p.full = static_cast<int>((tiles / pairs) * pairs);
  p.tail = static_cast<int>(tiles - p.full);
  p.split = p.tail > 0 ? pairs / p.tail : 1;
  if (p.split > p.num_kb / 4) p.split = p.num_kb / 4;   // keep ranges of at least 4 K blocks
  if (p.split < 1) p.split = 1;
  p.kb_per = (p.num_kb + p.split - 1) / p.split;
  p.ast_bytes = tile_workspace_bytes(M, K);
  p.partial_bytes = p.split >= 2 ? static_cast<int64_t>(p.tail) * p.split * 2 * 128 * 256 * 4 : 0;
  return p;
}

double wave_efficiency(int64_t tiles, int sms) {
  if (tiles <= 0) return 1.0;
  const int64_t waves = (tiles + sms - 1) / sms;
  return static_cast<double>(tiles) / static_cast<double>(waves * sms);
}

int pick_variant(int64_t M, int64_t N, int64_t K, int sm_count, int pairs) {
  const bool pair_ok = pairs > 0;
  // Decode shapes (M <= 256) are weight-streaming and HBM-bound. Measured on B200 at N = 28672,
  // K = 8192: the plain 128x256 tile kernel (46 us at M = 16, 5.1 TB/s with 112 of 148 SMs busy)
  // beats the swap-AB stream-K kernel (65 us), so AUTO does not pick that one.
  // (two row blocks, M in 129..256, go to the CTA pairs below when the device runs them: 79.5 vs 84-86 us at M = 256)
  if (M <= 128 || (M <= 256 && (N <= 128 || !pair_ok)))
    return (N > 128) ? B200FP8_VARIANT_TILE256 : B200FP8_VARIANT_TILE128;
  const int64_t num_m = (M + 127) / 128;
  const double e128 = wave_efficiency(num_m * ((N + 127) / 128), sm_count);
  const double e256 = wave_efficiency(num_m * ((N + 255) / 256), sm_count);
  // the 128x256 tile moves 25 % fewer operand bytes per flop; prefer it unless the last wave is much emptier
  if (e256 * 1.15 < e128) return B200FP8_VARIANT_TILE128;
  // CTA pairs on 256 x 256 tiles with the output staged through shared memory and written by TMA
  // (two staging sets per warp): the same tile waves as the single-CTA form when the number of
  // M-blocks is even, and measured faster than it and than its tail split-K form (8192 x 18432 x 7168:
  // 1.034 vs 1.11 ms, 1790 vs 1674 TFLOP/s sustained over 2.4 s; 4096 x 4096 x 8192: 141.3 vs 145.3 us).
  // With the stores out of the way the form that issues each K block as two 128-column halves is the
  // faster of the two pair kernels (same shapes: 1.002 vs 1.016 ms, 1846 vs 1811 sustained; 136.2 vs 139.4 us).
  if (pair_ok && num_m % 2 == 0) {
    // a partly empty last wave of pair tiles is split along K. The pair form's whole-tile part is not slower
    // for it and the fix-up pass is a few microseconds, so the bar is low: the idle share of the last wave
    // at least a fiftieth of the run (8192 x 18432 x 7168, 10 tiles in the 32nd wave: 986-989 vs 999-1000 us)
    const TileSkPlan pp = pair_sk_plan(M, N, K, pairs);
    const int64_t pw = (static_cast<int64_t>(pp.num_m) * pp.num_n + pairs - 1) / pairs;
    const bool pworth = pp.split >= 2 && (1.0 - 1.0 / pp.split) >= 0.02 * static_cast<double>(pw);
    return pworth ? B200FP8_VARIANT_PAIR256_SPLIT_SK : B200FP8_VARIANT_PAIR256_SPLIT;
  }
  // A mostly empty last wave is worth splitting along K, but the split-K kernel runs its
  // whole-tile part about 5 % slower (measured) and adds a fix-up pass: only take it when the
  // idle share of the last wave is at least a tenth of the whole run.
  const TileSkPlan p = tile_sk_plan(M, N, K, sm_count);
  const int64_t waves = (static_cast<int64_t>(p.num_m) * p.num_n + sm_count - 1) / sm_count;
  const bool worth = p.split >= 2 && (1.0 - 1.0 / p.split) >= 0.10 * static_cast<double>(waves);
  return worth ? B200FP8_VARIANT_TILE256_SK : B200FP8_VARIANT_TILE256;
}

template <int BN>
int launch_tile(const void* A, const void* B, const GemmArgs& args, int64_t lda, int64_t ldb, int sm_count,
                cudaStream_t stream, int64_t sk_grid = 0) {
  CUtensorMap ta, tb;
  // Weight-streaming shapes: kernel forms with 16- or 64-row A slots and six or five pipeline stages
  // (measured 3-4 % faster than the 128-row form at N = 28672, K = 8192: 44.5-46 us at M <= 17).
  // The prep kernel's copy of A has at least 16 rows (M <= 16 goes through a 16-row copy: TMA over the
  // caller's own 16-row tensor measured 4 % slower than over the copy in the workspace).
  const bool decode = BN == 256 && args.M <= 64 && args.sk_split < 2 && args.n_dst == 1 && !args.mc_store &&
                      args.BsT == nullptr;
  const uint32_t a_rows = !decode ? 128u : args.M <= 16 ? 16u : 64u;
  int st = make_tmap_u8(&ta, A, (args.a_from_prep && args.M < 16) ? 16 : args.M, args.K, lda, a_rows);
  if (st != B200FP8_OK) return st;
  st = make_tmap_u8(&tb, B, args.N, args.K, ldb, BN);
  if (st != B200FP8_OK) return st;
  const int64_t tiles = ((args.M + 127) / 128) * ((args.N + BN - 1) / BN);
  const int grid = sk_grid > 0 ? static_cast<int>(sk_grid) : static_cast<int>(tiles < sm_count ? tiles : sm_count);
  // Programmatic dependent launch: the kernel may begin (barrier set-up, TMEM allocation,
  // operand loads) while the tile_prep_kernel enqueued just before it is still running.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(TileCfg<BN, false>::THREADS);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t err;
  if (decode && a_rows == 16u) {
    cfg.dynamicSmemBytes = TileCfg<256, false, 16>::SMEM_BYTES;
    err = cudaLaunchKernelEx(&cfg, gemm_tile_decode_kernel<256, 16>, ta, tb, args);
  } else if (decode) {
    cfg.dynamicSmemBytes = TileCfg<256, false, 64>::SMEM_BYTES;
    err = cudaLaunchKernelEx(&cfg, gemm_tile_decode_kernel<256, 64>, ta, tb, args);
  } else if (BN == 256 && args.sk_split >= 2) {
    cfg.dynamicSmemBytes = TileCfg<256, false>::SMEM_BYTES;
    err = cudaLaunchKernelEx(&cfg, gemm_tile_kernel<256, 1>, ta, tb, args);
  } else if (BN == 128 && args.BsT != nullptr) {
    // the K-block-major copy of the row scales as an fp32 matrix [K blocks, n_pad]: one box = the
    // table of one tile (used when it fits the shared-memory table)
    CUtensorMap tbst;
    const int64_t kblocks = (args.K + 127) / 128;
    st = make_tmap(&tbst, args.BsT, kblocks, args.n_pad, args.n_pad * 4,
                   static_cast<uint32_t>(kblocks < kRowbTableKb ? kblocks : kRowbTableKb), 1);
    if (st != B200FP8_OK) return st;
    cfg.dynamicSmemBytes = TileCfg<128, false>::SMEM_BYTES + kRowbTableBytes;
    err = cudaLaunchKernelEx(&cfg, gemm_tile_rowb_kernel<128>, ta, tb, tbst, args);
  } else if (args.mc_store) {
    cfg.dynamicSmemBytes = TileCfg<BN, true>::SMEM_BYTES;
    err = cudaLaunchKernelEx(&cfg, gemm_tile_mc_kernel<BN>, ta, tb, args);
  } else if (args.n_dst > 1 || (BN == 256 && args.staged_store)) {
    // Several destinations, and the 256-wide tile with one: the output leaves through shared memory
    // and TMA stores instead of 16-byte stores of row pieces from registers (32 sectors per warp
    // instruction), which shortens the stretch at the end of a tile in which nothing drains TMEM.
    // One byte-matrix tensor map per destination: [M rows, N * element size], 32 x 128-byte boxes
    DstMaps dm;
    const int64_t esize = args.out_fp32 ? 4 : 2;
    for (int d = 0; d < 8; ++d) {
      const int src = d < args.n_dst ? d : 0;
      st = make_tmap_u8(&dm.m[d], args.dst[src], args.M, args.N * esize, args.dst_ld[src] * esize, 32);
      if (st != B200FP8_OK) return st;
    }
    cfg.dynamicSmemBytes = TileCfg<BN, true>::SMEM_BYTES;
    err = cudaLaunchKernelEx(&cfg, gemm_tile_multi_kernel<BN>, ta, tb, args, dm);
  } else {
    cfg.dynamicSmemBytes = TileCfg<BN, false>::SMEM_BYTES;
    err = cudaLaunchKernelEx(&cfg, gemm_tile_kernel<BN, 0>, ta, tb, args);
  }
  if (err != cudaSuccess) {
    cudaGetLastError();
    return B200FP8_ERR_LAUNCH;
  }
  return launch_status();
}

// CTA-pair kernels: 256 x 256 tiles, one cluster of two CTAs per tile, persistent over the pairs that
// fit on the device. The B map's box is this CTA's share of the B rows of one MMA.
template <bool SPLIT>
int launch_pair(const void* A, const void* B, const GemmArgs& args, int64_t lda, int64_t ldb, int pair_clusters,
                cudaStream_t stream) {
  if (pair_clusters < 1) return B200FP8_ERR_LAUNCH;
  CUtensorMap ta, tb;
  int st = make_tmap_u8(&ta, A, args.M, args.K, lda, 128);
  if (st != B200FP8_OK) return st;
  st = make_tmap_u8(&tb, B, args.N, args.K, ldb, SPLIT ? 64 : 128);
  if (st != B200FP8_OK) return st;
  const int64_t tiles = ((args.M + 255) / 256) * ((args.N + 255) / 256);
  // (the split-K plan counts on every pair the device can hold)
  const int pairs = args.sk_split >= 2 ? pair_clusters : static_cast<int>(tiles < pair_clusters ? tiles : pair_clusters);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  cfg.blockDim = dim3(TileCfg<256, false>::THREADS);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t err;
  if (args.n_dst > 1 || args.staged_store) {
    DstMaps dm;
    const int64_t esize = args.out_fp32 ? 4 : 2;
    for (int d = 0; d < 8; ++d) {
      const int src = d < args.n_dst ? d : 0;
      st = make_tmap_u8(&dm.m[d], args.dst[src], args.M, args.N * esize, args.dst_ld[src] * esize, 32);
      if (st != B200FP8_OK) return st;
    }
    cfg.dynamicSmemBytes = TileCfg<256, true, 128, 1>::SMEM_BYTES;
    if (args.sk_split >= 2) err = cudaLaunchKernelEx(&cfg, gemm_pair_multi_sk_kernel, ta, tb, args, dm);   // (SPLIT form only)
    else err = cudaLaunchKernelEx(&cfg, gemm_pair_multi_kernel<SPLIT>, ta, tb, args, dm);
  } else {
    cfg.dynamicSmemBytes = TileCfg<256, false, 128, 1>::SMEM_BYTES;
    err = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<SPLIT>, ta, tb, args);
  }
  if (err != cudaSuccess) {
    cudaGetLastError();
    return B200FP8_ERR_LAUNCH;
  }
  return launch_status();
}

template <int MP>
int launch_streamk(const void* A, const void* B, const StreamKArgs& args, int64_t lda, int64_t ldb, int64_t grid,
                   cudaStream_t stream) {
  CUtensorMap tw, tx;
  int st = make_tmap_u8(&tw, B, args.N, args.K, ldb, 128);
  if (st != B200FP8_OK) return st;
  st = make_tmap_u8(&tx, A, args.M, args.K, lda, MP);
  if (st != B200FP8_OK) return st;
  gemm_streamk_kernel<MP><<<static_cast<int>(grid), StreamKCfg<MP>::THREADS, StreamKCfg<MP>::SMEM_BYTES, stream>>>(
      tw, tx, args);
  return launch_status();
}

}  // namespace

extern "C" {

int b200fp8_version(void) { return 100; }

const char* b200fp8_strerror(int status) {
  switch (status) {
    case B200FP8_OK: return "ok";
    case B200FP8_ERR_NULL: return "a required pointer is NULL";
    case B200FP8_ERR_SHAPE: return "bad shape or leading dimension";
    case B200FP8_ERR_ALIGN: return "pointer or leading dimension violates a 16-byte alignment rule";
    case B200FP8_ERR_DTYPE: return "unknown output dtype";
    case B200FP8_ERR_VARIANT: return "unknown kernel variant, or variant cannot run this shape";
    case B200FP8_ERR_WORKSPACE: return "workspace missing or too small";
    case B200FP8_ERR_ARCH: return "current CUDA device is not compute capability 10.x (B200)";
    case B200FP8_ERR_DRIVER: return "cuTensorMapEncodeTiled unavailable or rejected the tensor";
    case B200FP8_ERR_LAUNCH: return "CUDA runtime refused the kernel launch";
    case B200FP8_ERR_TOO_LARGE: return "request exceeds a fixed capacity of this entry point";
    default: return "unknown status";
  }
}

int b200fp8_quant_act(const void* x, void* q, float* s, int64_t M, int64_t K, int64_t ldx, int64_t ldq, int64_t lds,
                      void* stream) {
  if (M < 0 || K < 0) return B200FP8_ERR_SHAPE;
  if (M == 0 || K == 0) return B200FP8_OK;
  if (x == nullptr || q == nullptr || s == nullptr) return B200FP8_ERR_NULL;
  if (ldx < K || ldq < K || lds < (K + 127) / 128) return B200FP8_ERR_SHAPE;
  if (K % 8 != 0 || ldx % 8 != 0 || ldq % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(q) & 7u) != 0)
    return B200FP8_ERR_ALIGN;
  const DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != B200FP8_OK) return st;
  const int64_t groups = M * ((K + 127) / 128);
  if (K % 128 == 0 && (M == 1 || (ldx == K && ldq == K && lds == K / 128)) &&
      (reinterpret_cast<uintptr_t>(q) & 15u) == 0 && groups <= (int64_t{1} << 35)) {
    // one unbroken run of 128-element groups: no row / column arithmetic in the kernel
    const int64_t blocks = (groups + 31) / 32;
    quant_act_contig_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(x), static_cast<uint4*>(q), s, groups);
    return launch_status();
  }
  const int64_t blocks_needed = (groups * 8 + 255) / 256;
  const int64_t max_blocks = static_cast<int64_t>(dev->sm_count) * 32;
  const int grid = static_cast<int>(blocks_needed < max_blocks ? blocks_needed : max_blocks);
  quant_act_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), s, M, K, ldx, ldq, lds);
  return launch_status();
}

int b200fp8_quant_weight(const void* w, void* q, float* s, int64_t N, int64_t K, int64_t ldw, int64_t ldq, int64_t lds,
                         void* stream) {
  if (N < 0 || K < 0) return B200FP8_ERR_SHAPE;
  if (N == 0 || K == 0) return B200FP8_OK;
  if (w == nullptr || q == nullptr || s == nullptr) return B200FP8_ERR_NULL;
  if (ldw < K || ldq < K || lds < (K + 127) / 128) return B200FP8_ERR_SHAPE;
  if (K % 8 != 0 || ldw % 8 != 0 || ldq % 8 != 0 || (reinterpret_cast<uintptr_t>(w) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(q) & 7u) != 0)
    return B200FP8_ERR_ALIGN;
  const DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != B200FP8_OK) return st;
  const int64_t blocks = ((N + 127) / 128) * ((K + 127) / 128);
  if (blocks > 0x7FFFFFFF) return B200FP8_ERR_TOO_LARGE;
  quant_weight_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q), s, N, K, ldw, ldq, lds);
  return launch_status();
}

int64_t b200fp8_streamk_first_unit(int64_t cta, int64_t total, int64_t grid) {
  return streamk_first_unit(cta, total, grid);
}
int64_t b200fp8_streamk_owner(int64_t unit, int64_t total, int64_t grid) { return streamk_owner(unit, total, grid); }
int64_t b200fp8_streamk_grid(int64_t M, int64_t N, int64_t K) {
  return streamk_plan(M, N, K, sm_count_or_default()).grid;
}

int b200fp8_gemm_pair_clusters(void) {
  const DeviceInfo* d = nullptr;
  if (device_info(&d) != B200FP8_OK) {
    cudaGetLastError();
    return 0;
  }
  return d->pair_clusters;
}

int b200fp8_gemm_pick_variant(int64_t M, int64_t N, int64_t K) {
  return pick_variant(M, N, K, sm_count_or_default(), b200fp8_gemm_pair_clusters());
}

int64_t b200fp8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int variant) {
  if (M < 0 || N < 0 || K < 0) return -static_cast<int64_t>(B200FP8_ERR_SHAPE);
  const int sms = sm_count_or_default();
  if (M == 0 || N == 0 || K == 0) return (variant >= B200FP8_VARIANT_AUTO && variant <= B200FP8_VARIANT_PAIR256_SPLIT_SK) ? 0 : -static_cast<int64_t>(B200FP8_ERR_VARIANT);
  if (variant == B200FP8_VARIANT_AUTO) {
    // whatever AUTO may resolve to for this shape, with or without CTA pairs (a destination that cannot
    // take 16-byte rows falls back to the single-CTA choice)
    int64_t need = tile_workspace_bytes(M, K);
    const int v1 = pick_variant(M, N, K, sms, 0);
    if (v1 == B200FP8_VARIANT_TILE256_SK) need = tile_workspace_bytes(M, K) + tile_sk_plan(M, N, K, sms).partial_bytes;
    const int pairs = b200fp8_gemm_pair_clusters();
    if (pairs > 0 && pick_variant(M, N, K, sms, pairs) == B200FP8_VARIANT_PAIR256_SPLIT_SK) {
      const int64_t np = tile_workspace_bytes(M, K) + pair_sk_plan(M, N, K, pairs).partial_bytes;
      need = np > need ? np : need;
    }
    return need;
  }
  if (variant == B200FP8_VARIANT_TILE128 || variant == B200FP8_VARIANT_TILE256 ||
      variant == B200FP8_VARIANT_PAIR256 || variant == B200FP8_VARIANT_PAIR256_SPLIT)
    return tile_workspace_bytes(M, K);
  if (variant == B200FP8_VARIANT_TILE256_SK) {
    const TileSkPlan p = tile_sk_plan(M, N, K, sms);
    return p.ast_bytes + p.partial_bytes;
  }
  if (variant == B200FP8_VARIANT_PAIR256_SPLIT_SK) {
    const TileSkPlan p = pair_sk_plan(M, N, K, b200fp8_gemm_pair_clusters());
    return p.ast_bytes + p.partial_bytes;
  }
  if (variant != B200FP8_VARIANT_STREAMK) return -static_cast<int64_t>(B200FP8_ERR_VARIANT);
  if (M > 256) return -static_cast<int64_t>(B200FP8_ERR_VARIANT);
  if (M == 0 || N == 0 || K == 0) return 0;
  const StreamKPlan p = streamk_plan(M, N, K, sms);
  return p.ast_bytes + p.partial_bytes;
}

// Shared body of b200fp8_gemm (n_dst = 1), b200fp8_gemm_scatter (n_dst >= 1) and
// b200fp8_gemm_multicast (n_dst = 1, mc = true: dst[0] is a multimem address).
// x_bf16 != nullptr: the activations arrive unquantised (b200fp8_linear); A and As are then
// produced by tile_prep_quant_kernel in the workspace.
struct FusedQuant {
  const void* x_bf16 = nullptr;
  int64_t ldx = 0;
  // rowb: Bs is [N, ceil(K/128)], one scale per row of B (b200fp8_gemm_rowscale)
  bool rowb = false;
};

int64_t bst_bytes(int64_t N, int64_t K) { return align_up(((K + 127) / 128) * align_up(N, 128) * 4, 256); }

static int gemm_impl(bool mc, const void* A, const void* B, const float* As, const float* Bs, int n_dst, void* const* dst,
                     const int64_t* dst_ld, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ld_as,
                     int64_t ld_bs, int out_dtype, int variant, void* workspace, size_t workspace_bytes,
                     uint32_t* status_word, void* stream_, FusedQuant fq = FusedQuant()) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const bool fused_q = fq.x_bf16 != nullptr;
  if (n_dst < 1 || n_dst > 8 || dst == nullptr || dst_ld == nullptr) return B200FP8_ERR_SHAPE;
  void* C = dst[0];
  const int64_t ldc = dst_ld[0];
  if (M < 0 || N < 0 || K < 0) return B200FP8_ERR_SHAPE;
  if (out_dtype != B200FP8_OUT_BF16 && out_dtype != B200FP8_OUT_FP32) return B200FP8_ERR_DTYPE;
  if (variant < B200FP8_VARIANT_AUTO || variant > B200FP8_VARIANT_PAIR256_SPLIT_SK) return B200FP8_ERR_VARIANT;
  if (M == 0 || N == 0) return B200FP8_OK;
  for (int d = 0; d < n_dst; ++d) {
    if (dst[d] == nullptr) return B200FP8_ERR_NULL;
    if (dst_ld[d] < N) return B200FP8_ERR_SHAPE;
  }

  const DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != B200FP8_OK) return st;

  // 16-byte vector stores through the staging path need aligned destinations
  const int64_t esize = out_dtype == B200FP8_OUT_FP32 ? 4 : 2;
  bool staged = (N * esize) % 16 == 0;
  for (int d = 0; d < n_dst; ++d)
    staged = staged && (reinterpret_cast<uintptr_t>(dst[d]) & 15u) == 0 && (dst_ld[d] * esize) % 16 == 0;
  if ((n_dst > 1 || mc) && !staged) return B200FP8_ERR_ALIGN;
  if (mc && n_dst != 1) return B200FP8_ERR_SHAPE;
  auto fill_dst = [&](GemmArgs& a) {
    a.n_dst = n_dst;
    a.staged_store = staged ? 1 : 0;
    a.mc_store = mc ? 1 : 0;
    for (int d = 0; d < 8; ++d) {
      a.dst[d] = d < n_dst ? dst[d] : nullptr;
      a.dst_ld[d] = d < n_dst ? dst_ld[d] : 0;
    }
  };

  if (K == 0) {
    if (n_dst > 1 || mc) return B200FP8_ERR_SHAPE;
    gemm_zero_fill_kernel<<<dev->sm_count, 256, 0, stream>>>(C, M, N, ldc, out_dtype == B200FP8_OUT_FP32);
    return launch_status();
  }
  const int64_t kblocks = (K + 127) / 128;
  if (fused_q) {
    if (B == nullptr || Bs == nullptr) return B200FP8_ERR_NULL;
    if (K % 128 != 0 || fq.ldx < K || ldb < K || ld_bs < kblocks) return B200FP8_ERR_SHAPE;
    if (fq.ldx % 8 != 0 || ldb % 16 != 0 || (reinterpret_cast<uintptr_t>(fq.x_bf16) & 15u) != 0 ||
        (reinterpret_cast<uintptr_t>(B) & 15u) != 0)
      return B200FP8_ERR_ALIGN;
  } else {
    if (A == nullptr || B == nullptr || As == nullptr || Bs == nullptr) return B200FP8_ERR_NULL;
    if (lda < K || ldb < K || ld_as < kblocks || ld_bs < kblocks) return B200FP8_ERR_SHAPE;
    if (lda % 16 != 0 || ldb % 16 != 0 || (reinterpret_cast<uintptr_t>(A) & 15u) != 0 ||
        (reinterpret_cast<uintptr_t>(B) & 15u) != 0)
      return B200FP8_ERR_ALIGN;
  }
  if (M > 0x7FFFFF00 || N > 0x7FFFFF00 || K > 0x7FFFFF00) return B200FP8_ERR_TOO_LARGE;

  const bool auto_variant = variant == B200FP8_VARIANT_AUTO;
  // (the pair form only pays with the staged output: a destination that cannot take 16-byte rows gets the single-CTA choice)
  if (auto_variant) variant = pick_variant(M, N, K, dev->sm_count, (staged && !mc && !fq.rowb) ? dev->pair_clusters : 0);
  if (fq.rowb) variant = B200FP8_VARIANT_TILE128;   // the row-scaled promotion exists for the 128-wide tile only
  const bool multi = n_dst > 1 || mc;
  if (fq.rowb && (multi || fused_q)) return B200FP8_ERR_VARIANT;
  // Several destinations (the N-sharded exchange): the pair kernel's smaller pipeline stages leave room
  // for a second set of output staging buffers, which keeps NVLink busy through the next tile's K loop
  if (multi && variant == B200FP8_VARIANT_TILE256_SK) variant = B200FP8_VARIANT_TILE256;
  // the K ranges of the pair split-K form leave through the fix-up pass, which writes one destination,
  // and its whole tiles through the staging area
  if (variant == B200FP8_VARIANT_PAIR256_SPLIT_SK && (multi || !staged || dev->pair_clusters < 1))
    variant = B200FP8_VARIANT_PAIR256_SPLIT;
  if (auto_variant && n_dst > 1 && !mc && M > 128 && dev->pair_clusters > 0 && variant == B200FP8_VARIANT_TILE256)
    variant = B200FP8_VARIANT_PAIR256_SPLIT;   // (2 GPUs, 8192 x 18432 x 7168: 0.596 vs 0.608 ms for the unsplit form)
  const bool pair = variant == B200FP8_VARIANT_PAIR256 || variant == B200FP8_VARIANT_PAIR256_SPLIT ||
                    variant == B200FP8_VARIANT_PAIR256_SPLIT_SK;
  if (pair && (mc || fq.rowb)) return B200FP8_ERR_VARIANT;
  if (multi && !pair && variant != B200FP8_VARIANT_TILE128 && variant != B200FP8_VARIANT_TILE256)
    return B200FP8_ERR_VARIANT;

  TileSkPlan skp = {};
  if (variant == B200FP8_VARIANT_TILE256_SK) {
    skp = tile_sk_plan(M, N, K, dev->sm_count);
    if (skp.split < 2) variant = B200FP8_VARIANT_TILE256;   // nothing to split: same as the plain tile kernel
  }
  if (variant == B200FP8_VARIANT_PAIR256_SPLIT_SK) {
    skp = pair_sk_plan(M, N, K, dev->pair_clusters);
    if (skp.split < 2) variant = B200FP8_VARIANT_PAIR256_SPLIT;
  }

  if (variant == B200FP8_VARIANT_TILE128 || variant == B200FP8_VARIANT_TILE256 ||
      variant == B200FP8_VARIANT_TILE256_SK || pair) {
    const bool pair_sk = variant == B200FP8_VARIANT_PAIR256_SPLIT_SK;
    const bool sk = variant == B200FP8_VARIANT_TILE256_SK || pair_sk;
    const int64_t prefix = fused_q ? linear_prefix_bytes(M, K) : tile_workspace_bytes(M, K);
    const int64_t need = prefix + (sk ? skp.partial_bytes : 0) + (fq.rowb ? bst_bytes(N, K) : 0);
    if (workspace == nullptr || static_cast<int64_t>(workspace_bytes) < need) return B200FP8_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200FP8_ERR_ALIGN;
    GemmArgs args;
    fill_dst(args);
    // the copy of A the prep kernel writes: the quantised activations (b200fp8_linear), or A
    // copied (and zero-padded) to 16 rows when M <= 16
    uint8_t* a_pad = (fused_q || M <= 16) ? static_cast<uint8_t*>(workspace) + tile_ast_bytes(M, K) : nullptr;
    args.a_from_prep = a_pad != nullptr;
    args.sk_full = sk ? skp.full : 0;
    args.sk_split = sk ? skp.split : 0;
    args.sk_kb_per = sk ? skp.kb_per : 0;
    args.partial = sk ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + prefix) : nullptr;
    args.AsT = static_cast<const float*>(workspace);
    args.m_pad = align_up(M, 128);
    if (fused_q) {
      const int64_t rows_q = M < 16 ? 16 : M;
      const int64_t threads = args.m_pad * kblocks * 8;
      tile_prep_quant_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(fq.x_bf16), fq.ldx, a_pad, align_up(K, 16), rows_q,
          static_cast<float*>(workspace), M, args.m_pad, static_cast<int>(kblocks));
      st = launch_status();
      if (st != B200FP8_OK) return st;
    } else {
      const dim3 grid(static_cast<unsigned>(args.m_pad / 32), static_cast<unsigned>((kblocks + 31) / 32));
      tile_prep_kernel<<<dim3(grid.x, grid.y, a_pad != nullptr ? 2u : 1u), 256, 0, stream>>>(
          As, static_cast<float*>(workspace), M, args.m_pad, static_cast<int>(kblocks), ld_as,
          static_cast<const uint8_t*>(A), a_pad, K, lda, align_up(K, 16));
      st = launch_status();
      if (st != B200FP8_OK) return st;
    }
    args.BsT = nullptr;
    args.rowb_table = 0;
    args.n_pad = align_up(N, 128);
    if (fq.rowb) {
      // second transposition: the row scales of B, K-block-major (same kernel, B in the role of A)
      float* bst = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + prefix);
      const dim3 grid(static_cast<unsigned>(args.n_pad / 32), static_cast<unsigned>((kblocks + 31) / 32));
      tile_prep_kernel<<<grid, 256, 0, stream>>>(Bs, bst, N, args.n_pad, static_cast<int>(kblocks), ld_bs, nullptr,
                                                 nullptr, K, 0, 0);
      st = launch_status();
      if (st != B200FP8_OK) return st;
      args.BsT = bst;
      args.rowb_table = kblocks <= kRowbTableKb ? 1 : 0;
    }
    args.As = As;
    args.Bs = Bs;
    args.C = C;
    args.M = M;
    args.N = N;
    args.K = K;
    args.ld_as = ld_as;
    args.ld_bs = ld_bs;
    args.ldc = ldc;
    args.out_fp32 = out_dtype == B200FP8_OUT_FP32;
    args.status_word = status_word;
    const void* a_eff = a_pad ? static_cast<const void*>(a_pad) : A;
    const int64_t lda_eff = a_pad ? align_up(K, 16) : lda;
    if (sk) {
      st = pair_sk ? launch_pair<true>(a_eff, B, args, lda_eff, ldb, dev->pair_clusters, stream)
                   : launch_tile<256>(a_eff, B, args, lda_eff, ldb, dev->sm_count, stream, skp.grid);
      if (st != B200FP8_OK) return st;
      cudaLaunchAttribute fattr[1];
      fattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      fattr[0].val.programmaticStreamSerializationAllowed = 1;
      cudaLaunchConfig_t fcfg = {};
      fcfg.gridDim = dim3(static_cast<unsigned>(skp.tail), pair_sk ? 8u : 4u, 4u);
      fcfg.blockDim = dim3(256);
      fcfg.stream = stream;
      fcfg.attrs = fattr;
      fcfg.numAttrs = 1;
      if (cudaLaunchKernelEx(&fcfg, tile_sk_fixup_kernel, static_cast<const float*>(args.partial), C, M, N, skp.num_kb,
                             ldc, static_cast<int>(out_dtype == B200FP8_OUT_FP32), skp.num_m, skp.num_n, skp.full,
                             skp.split, skp.kb_per, pair_sk ? 1 : 0) != cudaSuccess) {
        cudaGetLastError();
        return B200FP8_ERR_LAUNCH;
      }
      return launch_status();
    }
    if (variant == B200FP8_VARIANT_PAIR256)
      return launch_pair<false>(a_eff, B, args, lda_eff, ldb, dev->pair_clusters, stream);
    if (variant == B200FP8_VARIANT_PAIR256_SPLIT)
      return launch_pair<true>(a_eff, B, args, lda_eff, ldb, dev->pair_clusters, stream);
    return variant == B200FP8_VARIANT_TILE128 ? launch_tile<128>(a_eff, B, args, lda_eff, ldb, dev->sm_count, stream)
                                              : launch_tile<256>(a_eff, B, args, lda_eff, ldb, dev->sm_count, stream);
  }

  // stream-K decode variant
  if (fused_q) return B200FP8_ERR_VARIANT;
  if (M > 256) return B200FP8_ERR_VARIANT;
  const StreamKPlan p = streamk_plan(M, N, K, dev->sm_count);
  if (workspace == nullptr || static_cast<int64_t>(workspace_bytes) < p.ast_bytes + p.partial_bytes)
    return B200FP8_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200FP8_ERR_ALIGN;
  float* ast = static_cast<float*>(workspace);
  float* partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + p.ast_bytes);

  {
    const int total = p.num_kb * p.mp;
    streamk_prep_kernel<<<(total + 255) / 256, 256, 0, stream>>>(As, ast, M, p.num_kb, ld_as, p.mp);
    st = launch_status();
    if (st != B200FP8_OK) return st;
  }
  StreamKArgs args;
  args.Bs = Bs;
  args.AsT = ast;
  args.partial = partial;
  args.C = C;
  args.M = M;
  args.N = N;
  args.K = K;
  args.ld_bs = ld_bs;
  args.ldc = ldc;
  args.out_fp32 = out_dtype == B200FP8_OUT_FP32;
  args.status_word = status_word;
  switch (p.mp) {
    case 16: st = launch_streamk<16>(A, B, args, lda, ldb, p.grid, stream); break;
    case 32: st = launch_streamk<32>(A, B, args, lda, ldb, p.grid, stream); break;
    case 64: st = launch_streamk<64>(A, B, args, lda, ldb, p.grid, stream); break;
    case 128: st = launch_streamk<128>(A, B, args, lda, ldb, p.grid, stream); break;
    default: st = launch_streamk<256>(A, B, args, lda, ldb, p.grid, stream); break;
  }
  if (st != B200FP8_OK) return st;
  const dim3 fix_grid(static_cast<unsigned>(p.num_tiles), static_cast<unsigned>((M + kFixupRows - 1) / kFixupRows));
  streamk_fixup_kernel<<<fix_grid, 128, 0, stream>>>(
      partial, C, M, N, p.num_kb, ldc, out_dtype == B200FP8_OUT_FP32, p.mp, p.grid);
  return launch_status();
}

int b200fp8_gemm(const void* A, const void* B, const float* As, const float* Bs, void* C, int64_t M, int64_t N,
                 int64_t K, int64_t lda, int64_t ldb, int64_t ld_as, int64_t ld_bs, int64_t ldc, int out_dtype,
                 int variant, void* workspace, size_t workspace_bytes, uint32_t* status_word, void* stream) {
  void* dst[1] = {C};
  const int64_t ld[1] = {ldc};
  return gemm_impl(false, A, B, As, Bs, 1, dst, ld, M, N, K, lda, ldb, ld_as, ld_bs, out_dtype, variant, workspace,
                   workspace_bytes, status_word, stream);
}

int b200fp8_gemm_rowscale(const void* A, const void* B, const float* As, const float* Bs_row, void* C, int64_t M,
                          int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ld_as, int64_t ld_bs, int64_t ldc,
                          int out_dtype, void* workspace, size_t workspace_bytes, uint32_t* status_word,
                          void* stream) {
  void* dst[1] = {C};
  const int64_t ld[1] = {ldc};
  FusedQuant fq;
  fq.rowb = true;
  return gemm_impl(false, A, B, As, Bs_row, 1, dst, ld, M, N, K, lda, ldb, ld_as, ld_bs, out_dtype,
                   B200FP8_VARIANT_TILE128, workspace, workspace_bytes, status_word, stream, fq);
}

int64_t b200fp8_gemm_rowscale_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M < 0 || N < 0 || K < 0) return -static_cast<int64_t>(B200FP8_ERR_SHAPE);
  if (M == 0 || N == 0 || K == 0) return 0;
  return tile_workspace_bytes(M, K) + bst_bytes(N, K);
}

int b200fp8_linear(const void* x_bf16, const void* B, const float* Bs, void* C, int64_t M, int64_t N, int64_t K,
                   int64_t ldx, int64_t ldb, int64_t ld_bs, int64_t ldc, int out_dtype, int variant, void* workspace,
                   size_t workspace_bytes, uint32_t* status_word, void* stream) {
  if (x_bf16 == nullptr && M > 0 && K > 0) return B200FP8_ERR_NULL;
  void* dst[1] = {C};
  const int64_t ld[1] = {ldc};
  FusedQuant fq;
  fq.x_bf16 = x_bf16;
  fq.ldx = ldx;
  return gemm_impl(false, nullptr, B, nullptr, Bs, 1, dst, ld, M, N, K, 0, ldb, 0, ld_bs, out_dtype, variant, workspace,
                   workspace_bytes, status_word, stream, fq);
}

int64_t b200fp8_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int variant) {
  if (M < 0 || N < 0 || K < 0) return -static_cast<int64_t>(B200FP8_ERR_SHAPE);
  if (M == 0 || N == 0 || K == 0) return 0;
  const int sms = sm_count_or_default();
  if (variant == B200FP8_VARIANT_AUTO) {
    int64_t extra = 0;
    if (pick_variant(M, N, K, sms, 0) == B200FP8_VARIANT_TILE256_SK) extra = tile_sk_plan(M, N, K, sms).partial_bytes;
    const int pairs = b200fp8_gemm_pair_clusters();
    if (pairs > 0 && pick_variant(M, N, K, sms, pairs) == B200FP8_VARIANT_PAIR256_SPLIT_SK) {
      const int64_t ep = pair_sk_plan(M, N, K, pairs).partial_bytes;
      extra = ep > extra ? ep : extra;
    }
    return linear_prefix_bytes(M, K) + extra;
  }
  if (variant == B200FP8_VARIANT_TILE128 || variant == B200FP8_VARIANT_TILE256 ||
      variant == B200FP8_VARIANT_PAIR256 || variant == B200FP8_VARIANT_PAIR256_SPLIT)
    return linear_prefix_bytes(M, K);
  if (variant == B200FP8_VARIANT_TILE256_SK) return linear_prefix_bytes(M, K) + tile_sk_plan(M, N, K, sms).partial_bytes;
  if (variant == B200FP8_VARIANT_PAIR256_SPLIT_SK)
    return linear_prefix_bytes(M, K) + pair_sk_plan(M, N, K, b200fp8_gemm_pair_clusters()).partial_bytes;
  return -static_cast<int64_t>(B200FP8_ERR_VARIANT);
}

int b200fp8_gemm_multicast(const void* A, const void* B, const float* As, const float* Bs, void* C_multimem,
                           int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ld_as, int64_t ld_bs,
                           int64_t ldc, int out_dtype, int variant, void* workspace, size_t workspace_bytes,
                           uint32_t* status_word, void* stream) {
  void* dst[1] = {C_multimem};
  const int64_t ld[1] = {ldc};
  return gemm_impl(true, A, B, As, Bs, 1, dst, ld, M, N, K, lda, ldb, ld_as, ld_bs, out_dtype, variant, workspace,
                   workspace_bytes, status_word, stream);
}

int b200fp8_gemm_scatter(const void* A, const void* B, const float* As, const float* Bs, int n_dst, void* const* C_dst,
                         const int64_t* ldc_dst, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                         int64_t ld_as, int64_t ld_bs, int out_dtype, int variant, void* workspace,
                         size_t workspace_bytes, uint32_t* status_word, void* stream) {
  return gemm_impl(false, A, B, As, Bs, n_dst, C_dst, ldc_dst, M, N, K, lda, ldb, ld_as, ld_bs, out_dtype, variant,
                   workspace, workspace_bytes, status_word, stream);
}

int b200fp8_ipc_export(const void* ptr, void* handle_out_64, int64_t* offset_out) {
  if (ptr == nullptr || handle_out_64 == nullptr || offset_out == nullptr) return B200FP8_ERR_NULL;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  // the handle names the whole allocation; the offset of ptr inside it comes from the driver
  using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || sym == nullptr) {
    cudaGetLastError();
    return B200FP8_ERR_DRIVER;
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  if (reinterpret_cast<RangeFn>(sym)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS)
    return B200FP8_ERR_DRIVER;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) != cudaSuccess) {
    cudaGetLastError();
    return B200FP8_ERR_DRIVER;
  }
  memcpy(handle_out_64, &h, 64);
  *offset_out = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return B200FP8_OK;
}

int b200fp8_ipc_open(const void* handle_64, void** base_out) {
  if (handle_64 == nullptr || base_out == nullptr) return B200FP8_ERR_NULL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess || p == nullptr) {
    cudaGetLastError();
    return B200FP8_ERR_DRIVER;
  }
  *base_out = p;
  return B200FP8_OK;
}

int b200fp8_ipc_close(void* base) {
  if (base == nullptr) return B200FP8_ERR_NULL;
  if (cudaIpcCloseMemHandle(base) != cudaSuccess) {
    cudaGetLastError();
    return B200FP8_ERR_DRIVER;
  }
  return B200FP8_OK;
}

int b200fp8_peer_barrier_limited(uint32_t* const* flag_arrays, int n, int rank, uint32_t epoch, int64_t limit_clocks,
                                 uint32_t* status_word, void* stream) {
  if (flag_arrays == nullptr) return B200FP8_ERR_NULL;
  if (n < 1 || n > 8 || rank < 0 || rank >= n || limit_clocks < 1) return B200FP8_ERR_SHAPE;
  PeerFlags f;
  for (int i = 0; i < 8; ++i) {
    f.p[i] = i < n ? flag_arrays[i] : nullptr;
    if (i < n && (f.p[i] == nullptr || (reinterpret_cast<uintptr_t>(f.p[i]) & 3u) != 0)) return B200FP8_ERR_NULL;
  }
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, n, rank, epoch,
                                                                       static_cast<long long>(limit_clocks), status_word);
  return launch_status();
}

int b200fp8_peer_barrier(uint32_t* const* flag_arrays, int n, int rank, uint32_t epoch, uint32_t* status_word,
                         void* stream) {
  return b200fp8_peer_barrier_limited(flag_arrays, n, rank, epoch, kPeerBarrierDefaultLimitClks, status_word, stream);
}

int b200fp8_gemm_decode_static(const void* A, const void* B, const float* As, const float* Bs, void* C, int64_t M,
                               int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ld_as, int64_t ld_bs,
                               int64_t ldc, int out_dtype, uint32_t* status_word, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0 || N < 0 || K < 0) return B200FP8_ERR_SHAPE;
  if (out_dtype != B200FP8_OUT_BF16 && out_dtype != B200FP8_OUT_FP32) return B200FP8_ERR_DTYPE;
  if (M == 0 || N == 0) return B200FP8_OK;
  if (M > 256) return B200FP8_ERR_TOO_LARGE;
  if (A == nullptr || B == nullptr || As == nullptr || Bs == nullptr || C == nullptr) return B200FP8_ERR_NULL;
  if (K == 0) return B200FP8_ERR_SHAPE;
  const int64_t kblocks = (K + 127) / 128;
  if (ldc < N || lda < K || ldb < K || ld_as < kblocks || ld_bs < kblocks) return B200FP8_ERR_SHAPE;
  if (lda % 16 != 0 || ldb % 16 != 0 || (reinterpret_cast<uintptr_t>(A) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(B) & 15u) != 0)
    return B200FP8_ERR_ALIGN;
  if (N > 0x7FFFFF00 || K > 0x7FFFFF00) return B200FP8_ERR_TOO_LARGE;

  const DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != B200FP8_OK) return st;
  const StreamKPlan p = streamk_plan(M, N, K, dev->sm_count);
  if (static_cast<size_t>(p.ast_bytes + p.partial_bytes) > kStaticScratchBytes) return B200FP8_ERR_TOO_LARGE;
  void* scratch = nullptr;
  st = static_scratch_address(&scratch);   // first call on a device: cudaGetSymbolAddress
  if (st != B200FP8_OK) return st;
  float* ast = static_cast<float*>(scratch);
  float* partial = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + p.ast_bytes);

  // Nothing in the scratch has to start at zero: the prep kernel rewrites the whole AsT
  // region (padding included) and every partial slot the fix-up kernel reads is written by
  // the stream-K kernel of the same call first.
  const int total = p.num_kb * p.mp;
  streamk_prep_kernel<<<(total + 255) / 256, 256, 0, stream>>>(As, ast, M, p.num_kb, ld_as, p.mp);
  st = launch_status();
  if (st != B200FP8_OK) return st;
  StreamKArgs args;
  args.Bs = Bs;
  args.AsT = ast;
  args.partial = partial;
  args.C = C;
  args.M = M;
  args.N = N;
  args.K = K;
  args.ld_bs = ld_bs;
  args.ldc = ldc;
  args.out_fp32 = out_dtype == B200FP8_OUT_FP32;
  args.status_word = status_word;
  switch (p.mp) {
    case 16: st = launch_streamk<16>(A, B, args, lda, ldb, p.grid, stream); break;
    case 32: st = launch_streamk<32>(A, B, args, lda, ldb, p.grid, stream); break;
    case 64: st = launch_streamk<64>(A, B, args, lda, ldb, p.grid, stream); break;
    case 128: st = launch_streamk<128>(A, B, args, lda, ldb, p.grid, stream); break;
    default: st = launch_streamk<256>(A, B, args, lda, ldb, p.grid, stream); break;
  }
  if (st != B200FP8_OK) return st;
  const dim3 fix_grid(static_cast<unsigned>(p.num_tiles), static_cast<unsigned>((M + kFixupRows - 1) / kFixupRows));
  streamk_fixup_kernel<<<fix_grid, 128, 0, stream>>>(
      partial, C, M, N, p.num_kb, ldc, out_dtype == B200FP8_OUT_FP32, p.mp, p.grid);
  return launch_status();
}

}  // extern "C"
