// Activation quantisers shared by the stand-alone norm/quantise kernel and by the matvec
// kernel's fused prologue.  A warp holds one 256-value chunk, 8 consecutive values per lane.
//
//   Q8_K (quantize_q8_k_blocks, src/inference.rs:23121-23152 in the Camelid tree): the first
//        largest |v| of the 256 keeps its sign; iscale = -127/max; q = min(127, rne(iscale*v));
//        d = 1/iscale; an all-zero chunk gives d = 0.
//   Q8_0 (quantize_q8_0_block, src/inference.rs:22510-22528): per 32 values d = amax/127 kept
//        as its f16 rounding; q = round-half-away(v * (1/d_unrounded)) clamped to [-128,127].
#pragma once

#include "common.cuh"
#include "expf_exact.cuh"

namespace cmld {

// All 32 lanes must call.  q: this lane's 8 codes; d: the chunk's scale (same in every lane).
__device__ __forceinline__ void q8k_quantise_chunk(const float (&v)[8], int lane, int (&q)[8], float &d) {
  float amax = 0.0f, mx = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (fabsf(v[i]) > amax) {
      amax = fabsf(v[i]);
      mx = v[i];
    }
  // the chunk's largest |v|, and among equals the first: |v| >= 0 compares like its bits, lanes hold the values in order
  const uint32_t ab = __float_as_uint(amax);
  const uint32_t wmax = __reduce_max_sync(0xffffffffu, ab);
  const int src = __ffs((int)__ballot_sync(0xffffffffu, ab == wmax)) - 1;
  mx = __shfl_sync(0xffffffffu, mx, src);
  amax = __uint_as_float(wmax);
  d = 0.0f;
  if (amax == 0.0f) {
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = 0;
  } else {
    const float iscale = __fdiv_rn(-127.0f, mx);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = min(127, __float2int_rn(__fmul_rn(iscale, v[i])));
    d = __fdiv_rn(1.0f, iscale);
  }
}

// All 32 lanes must call.  A 32-value block spans 4 lanes; scale is the f16-rounded block scale.
__device__ __forceinline__ void q80_quantise_chunk(const float (&v)[8], int (&q)[8], float &scale) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const float du = __fdiv_rn(amax, 127.0f);
  const float inv = du == 0.0f ? 0.0f : __fdiv_rn(1.0f, du);
#pragma unroll
  for (int i = 0; i < 8; ++i) q[i] = (int)fminf(fmaxf(roundf(__fmul_rn(v[i], inv)), -128.0f), 127.0f);
  scale = f16_bits_to_f32(f32_to_f16_bits(du));
}

// Eight codes (each within int8) as bytes, the first lowest.
__device__ __forceinline__ uint2 pack8(const int (&q)[8]) {
  uint2 p;
  uint32_t t;
  // cvt.pack d, a, b, c: d = (c << 16) | (byte(a) << 8) | byte(b)
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(t) : "r"(q[3]), "r"(q[2]), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(p.x) : "r"(q[1]), "r"(q[0]), "r"(t));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(t) : "r"(q[7]), "r"(q[6]), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(p.y) : "r"(q[5]), "r"(q[4]), "r"(t));
  return p;
}

// SwiGLU element (src/inference.rs:13231-13236): g / (1 + exp(-g)) * u.
__device__ __forceinline__ float swiglu(float g, float u) {
  return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf_exact(-g))), u);
}

}  // namespace cmld
