// Byte maps between raw GGUF blocks and the tile-interleaved device storage, and the
// bit-exact per-element dequantisation from that storage.
//
// Tile-group layouts (16 rows x one K group). "plane" = 512 bytes = 32 lanes x 16 bytes; lane
// (g = lane / 4, t = lane % 4) of plane h holds bytes of row g + 8h. A 32-bit word inside a
// lane's 16 bytes holds the four quant bytes [4t .. 4t+3] of one 16-element chunk, i.e. what
// that lane contributes to one mma.m16n8k16 A fragment.
//
//  Q4_0  (group = 4 blocks, 1152 B): planes h=0,1: word w = block w, bytes qs[4t..4t+3]
//        (low nibbles = elements 4t+b, high nibbles = elements 16+4t+b); then f16 d[row][block].
//  Q8_0  (group = 4 blocks, 2176 B): planes (part p, h): word w = block 2p + w/2, half w%2,
//        bytes qs[16*(w%2) + 4t ..]; then f16 d[row][block].
//  Q4_K  (group = 1 super-block, 2304 B): planes (jj, h): word w = byte pair group j = 2jj + w/2,
//        half w%2: bytes qs[32j + 16*(w%2) + 4t ..] (low nibbles -> sub-block 2j, high -> 2j+1);
//        then the 16-byte header {d, dmin, scales[12]} per row.
//  Q6_K  (group = 1 super-block, 3360 B): planes qlA(h), qlB(h), qh(h): word w = (c = w/2,
//        u = w%2): qlA = ql[64c + 16u + 4t ..], qlB = ql[64c + 32 + 16u + 4t ..],
//        qh = qh[32c + 16u + 4t ..]; then scales[16] per row; then f16 d per row.
#pragma once

#include "common.cuh"

namespace fb {

// For destination byte `o` of a tile-group: row inside the tile and source byte offset inside
// that row's bytes of the same K group (group_elems / block_elems consecutive blocks).
__host__ __device__ inline void tile_src(uint32_t type, int o, int* row, int* src) {
  int within = o & 511;
  int lane = within >> 4, w = (within >> 2) & 3, b = within & 3;
  int g = lane >> 2, t = lane & 3;
  int plane = o >> 9;
  switch (type) {
    case FB200_Q4_0:
      if (o < 1024) {
        *row = g + 8 * plane;
        *src = w * 18 + 2 + 4 * t + b;
      } else {
        int p = o - 1024;
        *row = p >> 3;
        *src = ((p & 7) >> 1) * 18 + (p & 1);
      }
      break;
    case FB200_Q8_0:
      if (o < 2048) {
        int part = plane >> 1, h = plane & 1;
        *row = g + 8 * h;
        *src = (2 * part + (w >> 1)) * 34 + 2 + 16 * (w & 1) + 4 * t + b;
      } else {
        int p = o - 2048;
        *row = p >> 3;
        *src = ((p & 7) >> 1) * 34 + (p & 1);
      }
      break;
    case FB200_Q4_K:
      if (o < 2048) {
        int jj = plane >> 1, h = plane & 1;
        int j = 2 * jj + (w >> 1);
        *row = g + 8 * h;
        *src = 16 + 32 * j + 16 * (w & 1) + 4 * t + b;
      } else {
        int p = o - 2048;
        *row = p >> 4;
        *src = p & 15;
      }
      break;
    default:  // FB200_Q6_K
      if (o < 3072) {
        int which = plane >> 1, h = plane & 1;
        int c = w >> 1, u = w & 1;
        *row = g + 8 * h;
        if (which == 0) *src = 64 * c + 16 * u + 4 * t + b;
        else if (which == 1) *src = 64 * c + 32 + 16 * u + 4 * t + b;
        else *src = 128 + 32 * c + 16 * u + 4 * t + b;
      } else if (o < 3328) {
        int p = o - 3072;
        *row = p >> 4;
        *src = 192 + (p & 15);
      } else {
        int p = o - 3328;
        *row = p >> 1;
        *src = 208 + (p & 1);
      }
      break;
  }
}

__device__ inline float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

__device__ inline uint16_t ld_u16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// Element i (0 .. group_elems) of row r (0..15) of the tile-group at `tg`, with exactly the
// roundings of GgufBlock::dequantize (fusor-ml/gguf/src/lib.rs:828-846, 1284-1288, 1526-1556,
// 2034-2085): products and differences are separate IEEE operations, never fused.
__device__ inline float tile_dequant(uint32_t type, const uint8_t* tg, int r, int i) {
  int g = r & 7, h = r >> 3;
  switch (type) {
    case FB200_Q4_0: {
      int blk = i >> 5, e = i & 31, hf = e >> 4, p = e & 15, t = p >> 2, b = p & 3;
      uint8_t byte = tg[h * 512 + (g * 4 + t) * 16 + blk * 4 + b];
      int q = (hf ? (byte >> 4) : (byte & 0xF)) - 8;
      float d = half_bits_to_float(ld_u16(tg + 1024 + (r * 4 + blk) * 2));
      return __fmul_rn((float)q, d);
    }
    case FB200_Q8_0: {
      int blk = i >> 5, e = i & 31, hf = e >> 4, p = e & 15, t = p >> 2, b = p & 3;
      int plane = (blk >> 1) * 2 + h, w = (blk & 1) * 2 + hf;
      int8_t q = (int8_t)tg[plane * 512 + (g * 4 + t) * 16 + w * 4 + b];
      float d = half_bits_to_float(ld_u16(tg + 2048 + (r * 4 + blk) * 2));
      return __fmul_rn((float)q, d);
    }
    case FB200_Q4_K: {
      int sb = i >> 5, e = i & 31, hf = e >> 4, p = e & 15, t = p >> 2, b = p & 3;
      int j = sb >> 1, hi = sb & 1;
      int plane = (j >> 1) * 2 + h, w = (j & 1) * 2 + hf;
      uint8_t byte = tg[plane * 512 + (g * 4 + t) * 16 + w * 4 + b];
      int q = hi ? (byte >> 4) : (byte & 0xF);
      const uint8_t* hd = tg + 2048 + r * 16;
      float d = half_bits_to_float(ld_u16(hd));
      float dmin = half_bits_to_float(ld_u16(hd + 2));
      const uint8_t* s = hd + 4;
      int sc, mn;
      if (sb < 4) {
        sc = s[sb] & 63;
        mn = s[sb + 4] & 63;
      } else {
        sc = ((s[sb - 4] >> 6) << 4) | (s[sb + 4] & 0xF);
        mn = ((s[sb] >> 6) << 4) | (s[sb + 4] >> 4);
      }
      float scale = __fmul_rn((float)sc, d);
      float off = __fmul_rn((float)mn, dmin);
      return __fsub_rn(__fmul_rn(scale, (float)q), off);
    }
    default: {  // FB200_Q6_K
      int c = i >> 7, rem = i & 127, qsel = rem >> 5, l = rem & 31, u = l >> 4, p = l & 15;
      int t = p >> 2, b = p & 3, w = c * 2 + u;
      int off = h * 512 + (g * 4 + t) * 16 + w * 4 + b;
      uint8_t wa = tg[off], wb = tg[1024 + off], wh = tg[2048 + off];
      int nibble = qsel == 0 ? (wa & 0xF) : qsel == 1 ? (wb & 0xF) : qsel == 2 ? (wa >> 4) : (wb >> 4);
      int q = ((((wh >> (2 * qsel)) & 3) << 4) | nibble) - 32;
      int sc = (int8_t)tg[3072 + r * 16 + 8 * c + 2 * qsel + u];
      float d = half_bits_to_float(ld_u16(tg + 3328 + r * 2));
      return __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
    }
  }
}

// ---- types kept in raw row-major form ---------------------------------------------------------

// BlockQ5_0::dequantize, fusor-ml/gguf/src/lib.rs:1046-1073
__device__ inline float deq_q5_0(const uint8_t* b, int i) {
  float d = half_bits_to_float(ld_u16(b));
  uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
  int p = i & 15;
  uint8_t byte = b[6 + p];
  int q;
  if (i < 16) q = (byte & 0xF) | (((qh >> p) << 4) & 0x10);
  else q = (byte >> 4) | ((qh >> (p + 12)) & 0x10);
  return __fmul_rn((float)(q - 16), d);
}

// BlockQ5K::dequantize, fusor-ml/gguf/src/lib.rs:1819-1861
__device__ inline float deq_q5k(const uint8_t* b, int i) {
  float d = half_bits_to_float(ld_u16(b));
  float dmin = half_bits_to_float(ld_u16(b + 2));
  const uint8_t* s = b + 4;
  int sb = i >> 5, l = i & 31, chunk = sb >> 1, hi = sb & 1;
  int sc, mn;
  if (sb < 4) {
    sc = s[sb] & 63;
    mn = s[sb + 4] & 63;
  } else {
    sc = ((s[sb - 4] >> 6) << 4) | (s[sb + 4] & 0xF);
    mn = ((s[sb] >> 6) << 4) | (s[sb + 4] >> 4);
  }
  uint8_t ql = b[48 + 32 * chunk + l];
  uint8_t qh = b[16 + l];
  int q = (hi ? (ql >> 4) : (ql & 0xF)) + (((qh >> (2 * chunk + hi)) & 1) ? 16 : 0);
  return __fsub_rn(__fmul_rn(__fmul_rn((float)sc, d), (float)q), __fmul_rn((float)mn, dmin));
}

__device__ inline float raw_elem(uint32_t type, const uint8_t* raw, uint64_t idx) {
  switch (type) {
    case FB200_F32: return ((const float*)raw)[idx];
    case FB200_F16: return __half2float(((const __half*)raw)[idx]);
    case FB200_Q5_0: return deq_q5_0(raw + (idx >> 5) * 22, (int)(idx & 31));
    default: return deq_q5k(raw + (idx >> 8) * 176, (int)(idx & 255));
  }
}


}  // namespace fb
