// Activation quantisers shared by the permute+quantise kernels, the stand-alone quantiser ops and the
// expert-parallel dispatch (which quantises on the sending rank): one definition, so that every
// caller produces the same bytes.
#pragma once

#include "common.cuh"

namespace b200moe {

// ------------------------------------------------------------------------------------------
// NVFP4 activation quantiser, exact ("direct division") variant of the reference oracle
// (b12x/moe/_shared/kernels/reference.py:269-300):
//   sf    = e4m3_rn(min(amax * gs / 6, 448))
//   code  = e2m1_rte(x / max(sf / gs, 1e-30))
// One lane owns one 16-element block at a time.  Codes go to act_q[pos][K/2]; scales go to the
// 512-byte atoms of the row's 128-row tile, which is the layout tcgen05 block-scaled MMA reads.
// ------------------------------------------------------------------------------------------
// Branch-free reciprocal and division for the epilogues (a call with a slow-path branch per
// element keeps the compiler from interleaving the 16 independent element chains of a chunk).
__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// 1/x for normal x: hardware approximation + one Newton step (error <= 0.5 ulp + 2^-46)
__device__ __forceinline__ float rcp_newton(float x) {
  const float r = rcp_approx(x);
  return __fmaf_rn(r, __fmaf_rn(-x, r, 1.0f), r);
}
// a / b, correctly rounded when the quotient is a normal number or zero; rb = RN(1 / b).
// Two residual corrections with exact fma residuals (Markstein).
__device__ __forceinline__ float div_rn_normal(float a, float b, float rb) {
  float q = __fmul_rn(a, rb);
  q = __fmaf_rn(__fmaf_rn(-b, q, a), rb, q);
  q = __fmaf_rn(__fmaf_rn(-b, q, a), rb, q);
  return q;
}

// The quotient x / denom is first approximated by x * rcp(denom) (error < 2 ulp); if the values 2^-21
// below and above it round to the same E2M1 code, the correctly rounded quotient does too.  Only a
// block with a value that close to a rounding boundary takes the IEEE division, so the codes are
// those of the direct division at a fraction of its cost (sixteen divisions per block made the
// stand-alone quantiser arithmetic-bound: 2.1 TB/s at the Mixtral shape).
// `rgs` = RN(1 / gs), computed once per row or tile.
__device__ __forceinline__ void quant_block16(const float (&v)[16], float gs, float rgs, uint32_t& lo,
                                              uint32_t& hi, uint8_t& sf_byte) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float raw = fminf(div_rn_normal(__fmul_rn(amax, gs), 6.0f, 0.16666667163372039794921875f), 448.0f);
  sf_byte = f32_to_e4m3_rn_sat(raw);
  const float sf = e4m3_to_f32(sf_byte);
  const float denom = fmaxf(div_rn_normal(sf, gs, rgs), 1e-30f);
  const float r = rcp_approx(denom);
  float a0[8], a1[8], b0[8], b1[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float q0 = __fmul_rn(v[i], r), q1 = __fmul_rn(v[8 + i], r);
    a0[i] = __fmul_rn(q0, 1.0f - 4.76837158e-7f);
    b0[i] = __fmul_rn(q0, 1.0f + 4.76837158e-7f);
    a1[i] = __fmul_rn(q1, 1.0f - 4.76837158e-7f);
    b1[i] = __fmul_rn(q1, 1.0f + 4.76837158e-7f);
  }
  lo = pack_e2m1x8(a0);
  hi = pack_e2m1x8(a1);
  if (lo != pack_e2m1x8(b0) || hi != pack_e2m1x8(b1)) {
    float q0[8], q1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      q0[i] = __fdiv_rn(v[i], denom);
      q1[i] = __fdiv_rn(v[8 + i], denom);
    }
    lo = pack_e2m1x8(q0);
    hi = pack_e2m1x8(q1);
  }
}

// ------------------------------------------------------------------------------------------
// MXFP8 activation quantiser (b12x/_lib/intrinsics.py:223-265): per 32 elements
//   byte  = exponent of pow2_ceil(amax * (1/448))   (mantissa != 0 -> exponent + 1; 0 -> byte 0)
//   code  = e4m3_rn_sat(x * 2^(127 - byte))
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint8_t ue8m0_ceil_byte(float s) {
  uint32_t bits = __float_as_uint(s);
  if (bits & 0x007fffffu) bits = (bits + 0x00800000u) & 0x7f800000u;
  return static_cast<uint8_t>((bits >> 23) & 0xffu);
}
__device__ __forceinline__ float ue8m0_inv_scale(uint8_t byte) {
  if (byte == 0) return 0.f;
  const int ex = 254 - static_cast<int>(byte);
  return __uint_as_float(static_cast<uint32_t>(ex < 0 ? 0 : ex) << 23);
}

// 32 floats -> 32 E4M3 bytes (8 words, element 0 in the low byte) and their E8M0 scale byte
__device__ __forceinline__ void quant_block32_mx(const float (&v)[32], uint32_t (&o)[8], uint8_t& sf_byte) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
  sf_byte = ue8m0_ceil_byte(__fmul_rn(amax, static_cast<float>(1.0 / 448.0)));
  const float inv = ue8m0_inv_scale(sf_byte);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint32_t acc = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float s = fminf(fmaxf(__fmul_rn(v[4 * j + k], inv), -448.f), 448.f);
      acc |= static_cast<uint32_t>(f32_to_e4m3_rn_sat(s)) << (8 * k);
    }
    o[j] = acc;
  }
}

// 8 bf16 values (one 16-byte load) -> floats
__device__ __forceinline__ void bf16x8_to_f32(const uint4& p, float* v) {
  const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(w[j] << 16);
    v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
  }
}

}  // namespace b200moe
