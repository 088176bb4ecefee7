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

// max(a, b) that returns NaN when either operand is NaN (fmaxf would drop it).
__device__ __forceinline__ float fmax_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// max |x| over 8 bf16 (one uint4), as fp32; packed bf16x2 abs / max, exact. A NaN among the
// eight comes out as NaN (like torch.amax), so that it reaches the group's scale.
__device__ __forceinline__ float amax8(const uint4& v) {
  const uint32_t m = 0x7FFF7FFFu;
  uint32_t a = v.x & m, b = v.y & m, c = v.z & m, d = v.w & m;
  __nv_bfloat162 ab = __hmax2_nan(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  __nv_bfloat162 cd = __hmax2_nan(*reinterpret_cast<__nv_bfloat162*>(&c), *reinterpret_cast<__nv_bfloat162*>(&d));
  ab = __hmax2_nan(ab, cd);
  const uint32_t w = *reinterpret_cast<uint32_t*>(&ab);
  return fmax_nan(bf16_lo(w), bf16_hi(w));
}

// e4m3(x / scale) without a division per element, bit-identical to the division.
// With y = RN(1 / scale) (one correctly rounded reciprocal per group):
//     q0 = x * y            within an ulp of the quotient
//     r  = fma(-scale, q0, x)   the exact remainder
//     q  = fma(r, y, q0)    = RN(x / scale)          (Markstein's correction step)
// as long as nothing leaves the normal fp32 range where it matters. bf16 inputs have 8-bit
// mantissas and scale = amax / 448 with amax one of them, so the claim involves only
// 128 x 128 mantissa pairs; the tests run every pair through the kernel against the division.
// Range: |q| <= 448 always (|x| <= amax). Quotients below 2^-10 become e4m3 zero whatever their
// low bits; for |q| >= 2^-11 the remainder's last bit is >= scale * 2^-57, normal when
// scale >= 2^-60. Smaller scales (and infinite / NaN ones) take the true division.
// The sign of x is copied onto the result so that -0 stays -0 (the remainder of an exact
// zero is +0 and would otherwise absorb the sign).
constexpr float kScaleMinFast = 8.6736174e-19f;   // 2^-60
constexpr float kScaleMaxFast = 1.0e37f;          // every finite bf16 amax / 448 is below this

__device__ __forceinline__ float div_by_scale(float x, float scale, float y) {
  const float q0 = x * y;
  const float r = __fmaf_rn(-scale, q0, x);
  const float q = __fmaf_rn(r, y, q0);
  return __uint_as_float((__float_as_uint(q) & 0x7FFFFFFFu) | (__float_as_uint(x) & 0x80000000u));
}

// amax / 448 by the same correction step with the constant y = RN(1 / 448); exact for every
// bf16 amax whose quotient is a normal number (checked over all of them by the tests), true
// division otherwise.
__device__ __forceinline__ float scale_of_amax(float amax) {
  if (amax >= 1.0e-30f && amax <= 3.4e38f) {
    constexpr float y448 = 1.0f / 448.0f;
    const float q0 = amax * y448;
    const float r = __fmaf_rn(-448.0f, q0, amax);
    return __fmaf_rn(r, y448, q0);
  }
  return __fdiv_rn(amax, 448.0f);
}

__device__ __forceinline__ uint2 quant8_fast(const uint4& v, float scale, float y) {
  uint2 o;
  o.x = cvt_e4m3x2(div_by_scale(bf16_lo(v.x), scale, y), div_by_scale(bf16_hi(v.x), scale, y)) |
        (cvt_e4m3x2(div_by_scale(bf16_lo(v.y), scale, y), div_by_scale(bf16_hi(v.y), scale, y)) << 16);
  o.y = cvt_e4m3x2(div_by_scale(bf16_lo(v.z), scale, y), div_by_scale(bf16_hi(v.z), scale, y)) |
        (cvt_e4m3x2(div_by_scale(bf16_lo(v.w), scale, y), div_by_scale(bf16_hi(v.w), scale, y)) << 16);
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
// A NaN scale (a NaN in the group) makes every byte of the group NaN, an infinite one (an Inf in
// the group) makes finite elements zero and infinite ones NaN: what the formula gives.
template <int NV>
__device__ __forceinline__ void quant_vecs(const uint4 (&v)[NV], float scale, uint2 (&o)[NV]) {
  if (scale >= kScaleMinFast && scale <= kScaleMaxFast) {
    const float y = __frcp_rn(scale);
#pragma unroll
    for (int i = 0; i < NV; ++i) o[i] = quant8_fast(v[i], scale, y);
  } else if (scale == 0.f) {
#pragma unroll
    for (int i = 0; i < NV; ++i) o[i] = make_uint2(0u, 0u);
  } else {
#pragma unroll
    for (int i = 0; i < NV; ++i) o[i] = quant8_div(v[i], scale);
  }
}

// Contiguous case (K a multiple of 128, rows packed back to back in x, q and s): the matrix
// is one run of 128-element groups, thread t owns elements [16 t, 16 t + 16) and needs no
// row / column arithmetic at all. Eight consecutive threads share a group; the host rounds the
// grid up so that whole warps are inside or outside (four groups per warp).
__global__ void __launch_bounds__(256)
quant_act_contig_kernel(const uint4* __restrict__ x, uint4* __restrict__ q, float* __restrict__ s,
                        int64_t total_groups) {
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  const int64_t g = t >> 3;
  const bool live = g < total_groups;
  uint4 v[2];
  v[0] = make_uint4(0u, 0u, 0u, 0u);
  v[1] = make_uint4(0u, 0u, 0u, 0u);
  if (live) {
    v[0] = __ldg(x + 2 * t);
    v[1] = __ldg(x + 2 * t + 1);
  }
  float amax = fmax_nan(amax8(v[0]), amax8(v[1]));
  amax = fmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  const float scale = scale_of_amax(amax);
  uint2 o[2];
  quant_vecs<2>(v, scale, o);
  if (live) {
    q[t] = make_uint4(o[0].x, o[0].y, o[1].x, o[1].y);
    if ((threadIdx.x & 7) == 0) s[g] = scale;
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
      float amax = fmax_nan(amax8(v[u][0]), amax8(v[u][1]));
      amax = fmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      const float scale = scale_of_amax(amax);
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
    amax = fmax_nan(amax, amax8(v[i]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = warp_max[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmax_nan(amax, warp_max[i]);
  const float scale = scale_of_amax(amax);
  uint2 o[8];
  quant_vecs<8>(v, scale, o);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (row < N && col0 + i * 8 + 8 <= K) *reinterpret_cast<uint2*>(q + row * ldq + col0 + i * 8) = o[i];
  }
  if (threadIdx.x == 0) s[nb * lds + kb] = scale;
}

}  // namespace b200fp8
