// Byte maps between raw GGUF blocks and the tile-interleaved device storage, and the
// bit-exact per-element dequantisation from that storage.
//
// A tile is 16 consecutive rows of W, a tile-group the bytes of those rows for one K group
// (4 blocks of 32 for Q4_0/Q8_0, one 256-element super-block for Q4_K/Q6_K). Inside a
// tile-group the quant bytes are a byte permutation of the GGUF blocks, ordered so that a warp
// executing int8 mma.m16n8k32 reads its A operands with 16-byte shared-memory loads and no
// shuffles. MMA lane (g = lane / 4, t = lane % 4) works on rows g and g + 8 ("h" = 0 / 1 below)
// and, in the single-row kernel, on ONE scale group per chain of MMAs (group index t), so the
// bytes of a scale group are kept contiguous per row:
//
//  Q4_0 (1152 B): planes h = 0,1 of 512 B: [g][block b = 0..3][qs 16 B]; then f16 d[row][block].
//  Q8_0 (2176 B): planes (h, half) of 512 B: [g][block b][qs 16*half .. +16]; then f16 d[row][block].
//  Q4_K (2304 B): planes (ch, h, half) of 256 B, ch = chain of 4 sub-blocks:
//                 [g][ps = 0,1][qs 32*(2ch + ps) + 16*half .. +16]  (low nibbles = sub-block
//                 4ch + 2ps, high nibbles = 4ch + 2ps + 1); then the 16-byte header
//                 {d, dmin, scales[12]} per row.
//  Q6_K (3360 B): ql planes (c, u, h) of 256 B: [g][sl = 0,1][ql 64c + 32sl + 16u .. +16];
//                 qh planes (c, u, h) of 128 B: [g][qh 32c + 16u .. +16]; then scales[16] per
//                 row; then f16 d per row. (c, u) names the chain of the four 16-element scale
//                 groups 8c + 2q + u, q = 0..3: group q takes nibble q/2 of ql plane slot q%2
//                 and bits 2q, 2q+1 of qh.
#pragma once

#include "common.cuh"

namespace fb {

// For destination byte `o` of a tile-group: row inside the tile and source byte offset inside
// that row's bytes of the same K group (group_elems / block_elems consecutive blocks).
__host__ __device__ inline void tile_src(uint32_t type, int o, int* row, int* src) {
  switch (type) {
    case FB200_Q4_0:
      if (o < 1024) {
        int h = o >> 9, w = o & 511, g = w >> 6, b = (w >> 4) & 3, i = w & 15;
        *row = g + 8 * h;
        *src = b * 18 + 2 + i;
      } else {
        int p = o - 1024;
        *row = p >> 3;
        *src = ((p & 7) >> 1) * 18 + (p & 1);
      }
      break;
    case FB200_Q8_0:
      if (o < 2048) {
        int plane = o >> 9, h = plane >> 1, half = plane & 1;
        int w = o & 511, g = w >> 6, b = (w >> 4) & 3, i = w & 15;
        *row = g + 8 * h;
        *src = b * 34 + 2 + 16 * half + i;
      } else {
        int p = o - 2048;
        *row = p >> 3;
        *src = ((p & 7) >> 1) * 34 + (p & 1);
      }
      break;
    case FB200_Q4_K:
      if (o < 2048) {
        int plane = o >> 8, ch = plane >> 2, h = (plane >> 1) & 1, half = plane & 1;
        int w = o & 255, g = w >> 5, ps = (w >> 4) & 1, i = w & 15;
        *row = g + 8 * h;
        *src = 16 + 32 * (2 * ch + ps) + 16 * half + i;
      } else {
        int p = o - 2048;
        *row = p >> 4;
        *src = p & 15;
      }
      break;
    default:  // FB200_Q6_K
      if (o < 2048) {
        int plane = o >> 8, c = plane >> 2, u = (plane >> 1) & 1, h = plane & 1;
        int w = o & 255, g = w >> 5, sl = (w >> 4) & 1, i = w & 15;
        *row = g + 8 * h;
        *src = 64 * c + 32 * sl + 16 * u + i;
      } else if (o < 3072) {
        int q = o - 2048;
        int plane = q >> 7, c = plane >> 2, u = (plane >> 1) & 1, h = plane & 1;
        int w = q & 127, g = w >> 4, i = w & 15;
        *row = g + 8 * h;
        *src = 128 + 32 * c + 16 * u + i;
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

// Inverse direction for one quant byte: offset inside the tile-group of source byte `src`
// (offset inside the row's group bytes) of tile row r. Only the quant planes are covered;
// scales and headers have fixed places.
__host__ __device__ inline int tile_qs_offset(uint32_t type, int r, int qs_index) {
  const int g = r & 7, h = r >> 3;
  switch (type) {
    case FB200_Q4_0: {  // qs_index = block * 16 + i
      int b = qs_index >> 4, i = qs_index & 15;
      return h * 512 + g * 64 + b * 16 + i;
    }
    case FB200_Q8_0: {  // qs_index = block * 32 + i
      int b = qs_index >> 5, i = qs_index & 31;
      return (h * 2 + (i >> 4)) * 512 + g * 64 + b * 16 + (i & 15);
    }
    case FB200_Q4_K: {  // qs_index = byte of qs[128]
      int pair = qs_index >> 5, i = qs_index & 31;
      int ch = pair >> 1, ps = pair & 1, half = i >> 4;
      return ((ch * 2 + h) * 2 + half) * 256 + g * 32 + ps * 16 + (i & 15);
    }
    default: {  // Q6_K: qs_index < 128 -> ql byte, else qh byte (qs_index - 128)
      if (qs_index < 128) {
        int c = qs_index >> 6, rem = qs_index & 63, sl = rem >> 5, u = (rem >> 4) & 1, i = rem & 15;
        return ((c * 2 + u) * 2 + h) * 256 + g * 32 + sl * 16 + i;
      }
      int q = qs_index - 128;
      int c = q >> 5, u = (q >> 4) & 1, i = q & 15;
      return 2048 + ((c * 2 + u) * 2 + h) * 128 + g * 16 + i;
    }
  }
}

__device__ inline float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

__device__ inline uint16_t ld_u16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// Element i (0 .. group_elems) of row r (0..15) of the tile-group at `tg`, with exactly the
// roundings of GgufBlock::dequantize (fusor-ml/gguf/src/lib.rs:828-846, 1284-1288, 1526-1556,
// 2034-2085): products and differences are separate IEEE operations, never fused.
__device__ inline float tile_dequant(uint32_t type, const uint8_t* tg, int r, int i) {
  switch (type) {
    case FB200_Q4_0: {
      int blk = i >> 5, e = i & 31;
      uint8_t byte = tg[tile_qs_offset(type, r, blk * 16 + (e & 15))];
      int q = ((e >> 4) ? (byte >> 4) : (byte & 0xF)) - 8;
      float d = half_bits_to_float(ld_u16(tg + 1024 + (r * 4 + blk) * 2));
      return __fmul_rn((float)q, d);
    }
    case FB200_Q8_0: {
      int blk = i >> 5;
      int8_t q = (int8_t)tg[tile_qs_offset(type, r, i)];
      float d = half_bits_to_float(ld_u16(tg + 2048 + (r * 4 + blk) * 2));
      return __fmul_rn((float)q, d);
    }
    case FB200_Q4_K: {
      int sb = i >> 5, l = i & 31;
      uint8_t byte = tg[tile_qs_offset(type, r, 32 * (sb >> 1) + l)];
      int q = (sb & 1) ? (byte >> 4) : (byte & 0xF);
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
      int c = i >> 7, rem = i & 127, qsel = rem >> 5, l = rem & 31;
      uint8_t wl = tg[tile_qs_offset(type, r, 64 * c + 32 * (qsel & 1) + l)];
      uint8_t wh = tg[tile_qs_offset(type, r, 128 + 32 * c + l)];
      int nibble = (qsel >> 1) ? (wl >> 4) : (wl & 0xF);
      int q = ((((wh >> (2 * qsel)) & 3) << 4) | nibble) - 32;
      int sc = (int8_t)tg[3072 + r * 16 + 8 * c + 2 * qsel + (l >> 4)];
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
