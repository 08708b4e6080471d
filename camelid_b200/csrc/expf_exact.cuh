// expf that returns the same bits as the host C library's.
//
// Camelid's CPU path calls Rust's f32::exp, i.e. glibc's expf, in SwiGLU (src/inference.rs:13231)
// and in the attention softmax (src/inference.rs:30369).  CUDA's expf is within 2 ulp of it, which
// is enough to move an activation across an int8 rounding boundary now and then.  glibc's expf is
// a short double-precision algorithm (scaled exp2 with a 32-entry table and a cubic; published as
// part of ARM's optimized-routines): restated here with separately rounded double operations it
// reproduces glibc 2.39's results bit for bit (checked on 4e7 inputs and on a dense sweep of the
// softmax / SwiGLU range by tests/test_oracle_pins.py through the C twin in the CPU checker).
#pragma once

#include <cstdint>

namespace cmld {

// T[i] = bits(2^(i/32)) - (i << 47).  In global memory and read through the read-only cache: as a
// function-local array it would be rebuilt on the stack by every call (256 bytes of local stores).
static __device__ const uint64_t kExpfTable[32] = {
      0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
      0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
      0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
      0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
      0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
      0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
      0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
      0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull};

__device__ __forceinline__ float expf_exact(float x) {
  if (x != x) return x;
  if (x > 0x1.62e42ep6f) return __int_as_float(0x7f800000);  // overflow
  if (x < -0x1.9fe368p6f) return 0.0f;                       // underflow
  const double xd = (double)x;
  const double z = __dmul_rn(0x1.71547652b82fep+0 * 32.0, xd);
  double kd = __dadd_rn(z, 0x1.8p+52);
  const uint64_t ki = (uint64_t)__double_as_longlong(kd);
  kd = __dadd_rn(kd, -0x1.8p+52);
  const double r = __dadd_rn(z, -kd);
  const uint64_t t = __ldg(&kExpfTable[ki & 31]) + (ki << 47);
  const double s = __longlong_as_double((long long)t);
  const double zz = __dadd_rn(__dmul_rn(0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0, r), 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0);
  const double r2 = __dmul_rn(r, r);
  double y = __dadd_rn(__dmul_rn(0x1.62e42ff0c52d6p-1 / 32.0, r), 1.0);
  y = __dadd_rn(__dmul_rn(zz, r2), y);
  y = __dmul_rn(y, s);
  return (float)y;
}

}  // namespace cmld
