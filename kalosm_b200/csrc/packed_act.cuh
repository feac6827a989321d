// Activation rows handed from one kernel to the next in the operand form of the single-row
// product (int8 limbs + per-16 scales and sums), so that the consumer needs no packing pass.
#pragma once

#include "common.cuh"

// An activation row in the form the single-row product consumes directly (all device pointers;
// K padded to a multiple of 256 with zero limbs).
struct fb200_packed_act {
  uint8_t* limbs = nullptr;  // [Kp/8][32]: per 8 elements limb 0, limb 2, limb 1, limb 3 (8 bytes each)
  float* xsc = nullptr;      // [Kp/16] power-of-two scale of each 16-element block
  float* xss = nullptr;      // [Kp/16] sum of the 16 activations
  float* sumsq = nullptr;    // [Kp/16] sums of squares of the un-weighted values (RMSNorm consumers)
};


// ---- packed activations between kernels ---------------------------------------------------------
// A producer kernel can hand its output row to the next product already in MMA-operand form:
// limbs [K/8][32] (the shared-memory layout of the consumer), per-16 power-of-two scales and
// per-16 sums, optionally multiplied by the consumer's RMSNorm weight, plus per-unit partial
// sums of squares (the consumer adds them in index order and applies 1/rms as one final factor).
// Sixteen consecutive lanes call this with sixteen consecutive elements.
__device__ __forceinline__ void emit_packed16(const fb200_packed_act& pk, int n, float value,
                                              float norm_value, bool valid, uint32_t mask) {
  // value: what the consumer multiplies (after the optional norm weight); norm_value: what
  // enters the sum of squares
  float amax = valid ? fabsf(value) : 0.f;
  float sq = valid ? norm_value * norm_value : 0.f;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(mask, amax, o, 16));
    sq += __shfl_xor_sync(mask, sq, o, 16);
  }
  // amax = f * 2^ex with f in [0.5, 1) for normal numbers, read off the exponent field (zero,
  // denormal and non-finite maxima take ex = 0); powers of two are built from their exponent
  int ex = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 126;
  if (ex <= -126 || ex > 127) ex = 0;
  if (ex < -100) ex = -100;  // keeps 2^(27 - ex) and 2^(ex - 13) inside the normal range
  const float qscale = __uint_as_float((uint32_t)(27 - ex + 127) << 23);  // 64 * 2^21 / 2^ex
  const int q = valid ? __float2int_rn(value * qscale) : 0;
  float qsum = (float)q;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) qsum += __shfl_xor_sync(mask, qsum, o, 16);
  uint8_t* blk = pk.limbs + (size_t)(n >> 3) * 32 + (n & 7);
  blk[0] = (uint8_t)(q >> 21);           // limb 0 (signed)
  blk[8] = (uint8_t)((q >> 7) & 0x7F);   // limb 2
  blk[16] = (uint8_t)((q >> 14) & 0x7F); // limb 1
  blk[24] = (uint8_t)(q & 0x7F);         // limb 3
  if ((n & 15) == 0) {
    const float sc = __uint_as_float((uint32_t)(ex - 13 + 127) << 23);  // 2^(ex - 13)
    pk.xsc[n >> 4] = sc;
    pk.xss[n >> 4] = qsum * (1.0f / 16384.0f) * sc;
    if (pk.sumsq) pk.sumsq[n >> 4] = sq;
  }
}
