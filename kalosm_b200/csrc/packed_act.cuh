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

// ---- flagged rows: activations that travel between the phases of the persistent decode kernel
// WITHOUT a grid barrier ------------------------------------------------------------------------
// Every 4-byte word of payload is stored together with a 4-byte epoch as ONE 8-byte store (a
// "granule"); a reader polls the granule until the epoch is the one it expects, so data and
// "data is ready" arrive in the same atomic unit: no fence before a flag, no barrier, no second
// trip to L2 for the payload. (The same idea as the low-latency protocol of collective
// libraries: 50 % payload, latency of one store + one load.) Epochs only grow (one per phase of
// the kernel's program, continued from launch to launch), and every buffer is rewritten by the
// same phase of the next layer only after all readers of the previous contents have produced
// output that the rewriting CTAs depend on, so a single buffer per activation is enough.
//
// A packed activation row in this form: per 16 elements one block of 12 granules (96 bytes)
//   0..7   limbs: granule 4h + 2l + f = limb l (0: q >> 7 signed, 1: q & 127) of elements
//          8h + 4f .. 8h + 4f + 3 of the block, q = rint(v * 2^(14 - ex)) clamped to +-16383
//   8      xsc: 2^(ex - 14), the power-of-two scale of the block (f32 bits)
//   9      xss: sum of the 16 quantised activations times xsc (f32 bits)
//   10     sumsq: sum of squares of the un-weighted values (RMSNorm of the consumer)
//   11     unused
// Two limbs of 7 bits + sign resolve 2^-14 of the block maximum (about 3e-5 relative to a
// Gaussian block's spread): far inside the 2e-3 contract, at half the bytes and half the tensor
// core work of the four-limb form above.
struct fb200_ll_act {
  uint2* g = nullptr;  // [Kp / 16][12]
};

constexpr int FB200_LL_GRANULES = 12;  // per 16-element block
constexpr int FB200_LL_LINES = 6;      // 16-byte lines per block

__device__ __forceinline__ void st_ll(uint2* p, uint32_t data, uint32_t epoch) {
  const unsigned long long v = ((unsigned long long)epoch << 32) | (unsigned long long)data;
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_ll_line(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_ll_granule(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

constexpr int FB200_LL_POLL_LIMIT = 1 << 21;  // polls of one granule before the wait gives up (seconds)

// One f32 that another CTA publishes as a granule. Bounded: after the poll limit (or once another
// wait has already failed) the time-out is recorded and the stale value is returned.
__device__ __forceinline__ float ld_ll_f32(const uint2* p, uint32_t epoch, int* status) {
  uint2 v = ld_ll_granule(p);
  int polls = 0;
  while (v.y != epoch) {
    if (++polls > FB200_LL_POLL_LIMIT || ((polls & 63) == 0 && __ldcg(status) != 0)) {
      atomicExch(status, FB200_ERR_TIMEOUT);
      break;
    }
    v = ld_ll_granule(p);
  }
  return __uint_as_float(v.x);
}

// Sixteen consecutive lanes publish sixteen consecutive elements of a packed row (see above).
__device__ __forceinline__ void emit_ll16(const fb200_ll_act& pk, int n, float value, float norm_value, bool valid,
                                          uint32_t mask, uint32_t epoch) {
  float amax = valid ? fabsf(value) : 0.f;
  float sq = valid ? norm_value * norm_value : 0.f;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(mask, amax, o, 16));
    sq += __shfl_xor_sync(mask, sq, o, 16);
  }
  int ex = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 126;  // amax = f * 2^ex, f in [0.5, 1)
  if (ex <= -126 || ex > 127) ex = 0;
  if (ex < -100) ex = -100;
  const float qscale = __uint_as_float((uint32_t)(14 - ex + 127) << 23);  // 2^(14 - ex)
  int q = valid ? __float2int_rn(value * qscale) : 0;
  q = max(-16383, min(16383, q));
  float qsum = (float)q;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) qsum += __shfl_xor_sync(mask, qsum, o, 16);
  // gather the limb bytes of four consecutive elements into the lanes with (n & 3) == 0
  const uint32_t x = ((uint32_t)(q >> 7) & 0xFFu) | (((uint32_t)q & 0x7Fu) << 16);
  const uint32_t y = x | (__shfl_xor_sync(mask, x, 1, 16) << 8);
  const uint32_t y2 = __shfl_xor_sync(mask, y, 2, 16);
  const int l16 = n & 15;
  uint2* blk = pk.g + (size_t)(n >> 4) * FB200_LL_GRANULES;
  if ((l16 & 3) == 0) {
    const int h = l16 >> 3, f = (l16 >> 2) & 1;
    st_ll(blk + 4 * h + f, (y & 0xFFFFu) | (y2 << 16), epoch);          // limb 0 of elements l16 .. l16 + 3
    st_ll(blk + 4 * h + 2 + f, (y >> 16) | (y2 & 0xFFFF0000u), epoch);  // limb 1
  } else if (l16 == 1) {
    st_ll(blk + 8, (uint32_t)(ex - 14 + 127) << 23, epoch);
  } else if (l16 == 2) {
    st_ll(blk + 9, __float_as_uint(qsum * __uint_as_float((uint32_t)(ex - 14 + 127) << 23)), epoch);
  } else if (l16 == 3) {
    st_ll(blk + 10, __float_as_uint(sq), epoch);
  }
}
