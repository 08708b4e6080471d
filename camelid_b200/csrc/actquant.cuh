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
  int idx = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (fabsf(v[i]) > amax) {
      amax = fabsf(v[i]);
      mx = v[i];
      idx = lane * 8 + i;
    }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
    const float om = __shfl_xor_sync(0xffffffffu, mx, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (oa > amax || (oa == amax && oi < idx)) {
      amax = oa;
      mx = om;
      idx = oi;
    }
  }
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

__device__ __forceinline__ uint2 pack8(const int (&q)[8]) {
  uint2 p;
  p.x = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((q[3] & 0xff) << 24);
  p.y = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((q[7] & 0xff) << 24);
  return p;
}

// SwiGLU element (src/inference.rs:13231-13236): g / (1 + exp(-g)) * u.
__device__ __forceinline__ float swiglu(float g, float u) {
  return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf_exact(-g))), u);
}

}  // namespace cmld
