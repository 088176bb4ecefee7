// bf16 -> e4m3 quantisers with fp32 scales = amax / 448.
//   quant_act_kernel     one scale per row and 128-wide K group   (activations)
//   quant_weight_kernel  one scale per 128x128 block              (weights)
// Both are single-pass and HBM-bound: every input byte is read once, every output
// byte written once. The arithmetic is the literal formula in IEEE fp32 (true
// division, round-to-nearest-even e4m3 cast) so that bytes and scales can be
// compared bit for bit with a CPU evaluation of the same formula.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace b200fp8 {

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// two fp32 -> two e4m3 bytes (low byte = first value), round-to-nearest-even, saturating
__device__ __forceinline__ uint32_t cvt_e4m3x2(float a, float b) {
  return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3));
}

// max |x| over 8 bf16 (one uint4), as fp32; packed bf16x2 abs / max, exact.
__device__ __forceinline__ float amax8(const uint4& v) {
  const uint32_t m = 0x7FFF7FFFu;
  uint32_t a = v.x & m, b = v.y & m, c = v.z & m, d = v.w & m;
  __nv_bfloat162 ab = __hmax2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  __nv_bfloat162 cd = __hmax2(*reinterpret_cast<__nv_bfloat162*>(&c), *reinterpret_cast<__nv_bfloat162*>(&d));
  ab = __hmax2(ab, cd);
  const uint32_t w = *reinterpret_cast<uint32_t*>(&ab);
  return fmaxf(bf16_lo(w), bf16_hi(w));
}

// e4m3(x / scale) without a division per element, bit-identical to the division.
// q = x * rcp (rcp = 1 / scale, correctly rounded) is within 2 ulp of the IEEE quotient, so
// the e4m3 cast of the two can differ only if an e4m3 rounding boundary lies between them:
//   - q within a few ulp of a tie of the normal e4m3 range, i.e. the 20 fp32 mantissa bits
//     below the three kept ones are about 0x80000;
//   - 0 < |q| < 2^-6 (the e4m3 subnormal range has its ties elsewhere).
// Both conditions are folded into two running unsigned minima over the elements a thread
// converts; if either fires (rare), the thread redoes its elements with the true division.
// (|q| cannot leave the range upwards since |x| <= amax; a scale so small that 1 / scale
// overflows is sent to the division path as a whole.)
struct ExactnessProbe {
  uint32_t tie_min = 0xFFFFFFFFu;   // min over elements of (bits & 0xFFFFF) - (0x80000 - 8); <= 16 means "near a tie"
  uint32_t low_min = 0xFFFFFFFFu;   // min over elements of |q| bits - 1; < 0x3C800000 - 1 means "0 < |q| < 2^-6"
  __device__ __forceinline__ float mul(float x, float rcp) {
    const float q = x * rcp;
    const uint32_t bits = __float_as_uint(q);
    tie_min = min(tie_min, (bits & 0xFFFFFu) - (0x80000u - 8u));
    low_min = min(low_min, (bits & 0x7FFFFFFFu) - 1u);
    return q;
  }
  __device__ __forceinline__ bool inexact() const { return tie_min <= 16u || low_min < 0x3C800000u - 1u; }
};

__device__ __forceinline__ uint2 quant8_fast(const uint4& v, float rcp, ExactnessProbe& pr) {
  uint2 o;
  o.x = cvt_e4m3x2(pr.mul(bf16_lo(v.x), rcp), pr.mul(bf16_hi(v.x), rcp)) |
        (cvt_e4m3x2(pr.mul(bf16_lo(v.y), rcp), pr.mul(bf16_hi(v.y), rcp)) << 16);
  o.y = cvt_e4m3x2(pr.mul(bf16_lo(v.z), rcp), pr.mul(bf16_hi(v.z), rcp)) |
        (cvt_e4m3x2(pr.mul(bf16_lo(v.w), rcp), pr.mul(bf16_hi(v.w), rcp)) << 16);
  return o;
}

__device__ __forceinline__ uint2 quant8_div(const uint4& v, float scale) {
  uint2 o;
  o.x = cvt_e4m3x2(__fdiv_rn(bf16_lo(v.x), scale), __fdiv_rn(bf16_hi(v.x), scale)) |
        (cvt_e4m3x2(__fdiv_rn(bf16_lo(v.y), scale), __fdiv_rn(bf16_hi(v.y), scale)) << 16);
  o.y = cvt_e4m3x2(__fdiv_rn(bf16_lo(v.z), scale), __fdiv_rn(bf16_hi(v.z), scale)) |
        (cvt_e4m3x2(__fdiv_rn(bf16_lo(v.w), scale), __fdiv_rn(bf16_hi(v.w), scale)) << 16);
  return o;
}

// N x 8 bf16 (N uint4) divided by `scale` and packed into N x 8 e4m3 bytes (N uint2).
// scale == 0 (all-zero group) yields zero bytes instead of the 0/0 NaN of the formula.
template <int NV>
__device__ __forceinline__ void quant_vecs(const uint4 (&v)[NV], float scale, uint2 (&o)[NV]) {
  if (scale == 0.f) {
#pragma unroll
    for (int i = 0; i < NV; ++i) o[i] = make_uint2(0u, 0u);
    return;
  }
  bool exact_path = scale < 1.0e-30f;   // 1 / scale would overflow or lose bits: divide
  if (!exact_path) {
    const float rcp = __frcp_rn(scale);
    ExactnessProbe pr;
#pragma unroll
    for (int i = 0; i < NV; ++i) o[i] = quant8_fast(v[i], rcp, pr);
    exact_path = pr.inexact();
  }
  if (exact_path) {
#pragma unroll
    for (int i = 0; i < NV; ++i) o[i] = quant8_div(v[i], scale);
  }
}

// Eight consecutive threads own one 128-element group: each loads two 16-byte
// vectors (16 bf16), the group amax is an 8-lane xor-shuffle reduction, each thread
// stores 16 e4m3 bytes. A warp therefore reads 1 KiB and writes 512 B contiguously.
__global__ void __launch_bounds__(256)
quant_act_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ s, int64_t M,
                 int64_t K, int64_t ldx, int64_t ldq, int64_t lds) {
  const int64_t groups_per_row = (K + 127) / 128;
  const int64_t total_groups = M * groups_per_row;
  const int sub = threadIdx.x & 7;
  const int64_t groups_per_pass = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 3;
  // total_groups rounded up to a multiple of 4 keeps all 32 lanes of a warp inside the shuffle
  const int64_t padded_groups = (total_groups + 3) & ~int64_t(3);

  // reduced, and the two dependent chains (shuffles, division, reciprocal) interleave.
  constexpr int U = 1;
  for (int64_t g0 = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 3; g0 < padded_groups;
       g0 += U * groups_per_pass) {
    uint4 v[U][2];
    int64_t row[U], kg[U], col[U];
    bool live[U], has0[U], has1[U], in_loop[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t g = g0 + u * groups_per_pass;
      in_loop[u] = g < padded_groups;          // warp-uniform: whole warps share a group quadruple
      live[u] = g < total_groups;
      row[u] = live[u] ? g / groups_per_row : 0;
      kg[u] = live[u] ? g - row[u] * groups_per_row : 0;
      col[u] = kg[u] * 128 + sub * 16;
      has0[u] = live[u] && (col[u] + 8 <= K);
      has1[u] = live[u] && (col[u] + 16 <= K);
      v[u][0] = make_uint4(0u, 0u, 0u, 0u);
      v[u][1] = make_uint4(0u, 0u, 0u, 0u);
      const __nv_bfloat16* src = x + row[u] * ldx + col[u];
      if (has0[u]) v[u][0] = __ldg(reinterpret_cast<const uint4*>(src));
      if (has1[u]) v[u][1] = __ldg(reinterpret_cast<const uint4*>(src + 8));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!in_loop[u]) continue;
      float amax = fmaxf(amax8(v[u][0]), amax8(v[u][1]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      const float scale = __fdiv_rn(amax, 448.0f);
      uint8_t* dst = q + row[u] * ldq + col[u];
      if (has0[u]) {
        uint2 o[2];   // a missing second vector is zeros and is simply not stored
        quant_vecs<2>(v[u], scale, o);
        if (has1[u]) {
          if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(o[0].x, o[0].y, o[1].x, o[1].y);
          } else {
            *reinterpret_cast<uint2*>(dst) = o[0];
            *reinterpret_cast<uint2*>(dst + 8) = o[1];
          }
        } else {
          *reinterpret_cast<uint2*>(dst) = o[0];
        }
      }
      if (live[u] && sub == 0) s[row[u] * lds + kg[u]] = scale;
    }
  }
}

// One CTA of 256 threads per 128x128 block: thread t owns row t/2, columns
// (t%2)*64 .. +63 (eight 16-byte vectors held in registers between the two phases).
__global__ void __launch_bounds__(256)
quant_weight_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q, float* __restrict__ s, int64_t N,
                    int64_t K, int64_t ldw, int64_t ldq, int64_t lds) {
  __shared__ float warp_max[8];
  const int64_t kblocks = (K + 127) / 128;
  const int64_t nb = blockIdx.x / kblocks;
  const int64_t kb = blockIdx.x - nb * kblocks;
  const int64_t row = nb * 128 + (threadIdx.x >> 1);
  const int64_t col0 = kb * 128 + (threadIdx.x & 1) * 64;
  uint4 v[8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] = make_uint4(0u, 0u, 0u, 0u);
    if (row < N && col0 + i * 8 + 8 <= K) v[i] = __ldg(reinterpret_cast<const uint4*>(w + row * ldw + col0 + i * 8));
    amax = fmaxf(amax, amax8(v[i]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = warp_max[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, warp_max[i]);
  const float scale = __fdiv_rn(amax, 448.0f);
  uint2 o[8];
  quant_vecs<8>(v, scale, o);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (row < N && col0 + i * 8 + 8 <= K) *reinterpret_cast<uint2*>(q + row * ldq + col0 + i * 8) = o[i];
  }
  if (threadIdx.x == 0) s[nb * lds + kb] = scale;
}

}  // namespace b200fp8
