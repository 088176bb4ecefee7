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

__device__ __forceinline__ float amax8(const uint4& v) {
  float m = fmaxf(fabsf(bf16_lo(v.x)), fabsf(bf16_hi(v.x)));
  m = fmaxf(m, fmaxf(fabsf(bf16_lo(v.y)), fabsf(bf16_hi(v.y))));
  m = fmaxf(m, fmaxf(fabsf(bf16_lo(v.z)), fabsf(bf16_hi(v.z))));
  m = fmaxf(m, fmaxf(fabsf(bf16_lo(v.w)), fabsf(bf16_hi(v.w))));
  return m;
}

// x / scale for the e4m3 cast, bit-identical to e4m3_rne(__fdiv_rn(x, scale)) but without
// a division per element. q = x * rcp (rcp = 1 / scale, correctly rounded) is within
// 2 ulp of the IEEE quotient; the cast to e4m3 can only differ if a rounding boundary
// of e4m3 lies between the two, i.e. if q sits within a few ulp of a tie (fp32
// mantissa bits below the three kept ones equal to 0x80000). Those rare elements, the
// e4m3 subnormal range (different tie positions) and non-finite / out-of-range q take
// the exact division instead.
__device__ __forceinline__ float quotient_for_cast(float x, float scale, float rcp) {
  const float q = x * rcp;
  const uint32_t mag = __float_as_uint(q) & 0x7FFFFFFFu;
  const bool near_tie = ((mag & 0xFFFFFu) - (0x80000u - 8u)) <= 16u;
  const bool odd_range = mag >= 0x43E80000u /* 464, inf, NaN */ || mag < 0x3C800000u /* 2^-6 */;
  if ((near_tie || odd_range) && mag != 0u) return __fdiv_rn(x, scale);  // a zero product casts to the same zero
  return q;
}

// 8 bf16 (one uint4) divided by `scale` and packed into 8 e4m3 bytes (one uint2).
// scale == 0 (all-zero group) yields zero bytes instead of the 0/0 NaN of the formula.
__device__ __forceinline__ uint2 quant8(const uint4& v, float scale) {
  if (scale == 0.f) return make_uint2(0u, 0u);
  const float rcp = __frcp_rn(scale);
  uint2 o;
  o.x = cvt_e4m3x2(quotient_for_cast(bf16_lo(v.x), scale, rcp), quotient_for_cast(bf16_hi(v.x), scale, rcp)) |
        (cvt_e4m3x2(quotient_for_cast(bf16_lo(v.y), scale, rcp), quotient_for_cast(bf16_hi(v.y), scale, rcp)) << 16);
  o.y = cvt_e4m3x2(quotient_for_cast(bf16_lo(v.z), scale, rcp), quotient_for_cast(bf16_hi(v.z), scale, rcp)) |
        (cvt_e4m3x2(quotient_for_cast(bf16_lo(v.w), scale, rcp), quotient_for_cast(bf16_hi(v.w), scale, rcp)) << 16);
  return o;
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
  for (int64_t g = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 3; g < padded_groups;
       g += groups_per_pass) {
    const bool live = g < total_groups;
    const int64_t row = live ? g / groups_per_row : 0;
    const int64_t kg = live ? g - row * groups_per_row : 0;
    const int64_t col = kg * 128 + sub * 16;
    const bool has0 = live && (col + 8 <= K);
    const bool has1 = live && (col + 16 <= K);
    uint4 v0 = make_uint4(0u, 0u, 0u, 0u), v1 = make_uint4(0u, 0u, 0u, 0u);
    const __nv_bfloat16* src = x + row * ldx + col;
    if (has0) v0 = __ldg(reinterpret_cast<const uint4*>(src));
    if (has1) v1 = __ldg(reinterpret_cast<const uint4*>(src + 8));
    float amax = fmaxf(amax8(v0), amax8(v1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const float scale = __fdiv_rn(amax, 448.0f);
    uint8_t* dst = q + row * ldq + col;
    if (has1) {
      const uint2 a = quant8(v0, scale), b = quant8(v1, scale);
      if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(a.x, a.y, b.x, b.y);
      } else {
        *reinterpret_cast<uint2*>(dst) = a;
        *reinterpret_cast<uint2*>(dst + 8) = b;
      }
    } else if (has0) {
      *reinterpret_cast<uint2*>(dst) = quant8(v0, scale);
    }
    if (live && sub == 0) s[row * lds + kg] = scale;
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
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (row < N && col0 + i * 8 + 8 <= K)
      *reinterpret_cast<uint2*>(q + row * ldq + col0 + i * 8) = quant8(v[i], scale);
  }
  if (threadIdx.x == 0) s[nb * lds + kb] = scale;
}

}  // namespace b200fp8
