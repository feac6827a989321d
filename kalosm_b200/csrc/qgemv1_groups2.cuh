// Per-tile-group inner products against TWO-limb activations (the form that travels between the
// phases of the persistent decode kernel as flagged rows, packed_act.cuh): one warp, one
// tile-group (16 rows of W x one K group) against the limbs in shared memory.
//
// Same mapping as the four-limb functions of qgemv1_groups.cuh ("scale group per lane": MMA lane
// (g = lane / 4, t = lane % 4) feeds, per mma.m16n8k32, 8 elements of ONE scale group of rows g
// and g + 8; the B operand carries the limbs of group t' only in columns 2t', 2t' + 1 and only
// in the k-slots of lane t'), with limb 0 in column 2t' and limb 1 in column 2t' + 1, so ONE MMA
// per 8-element step yields both integer dot products of a lane's own group:
//   c[0], c[1] = row g x (limb 0, limb 1);  c[2], c[3] = row g + 8.
// The activation of element e is (128 * limb0 + limb1) * xsc[block of 16], limb0 = q >> 7
// signed, limb1 = q & 127.
//
// Shared-memory placement: 16 bytes per 8 elements, [limb 0 x 8][limb 1 x 8]; the block of
// 8-element group B sits at byte 16 B + 16 (B >> 3): one 16-byte pad after every 8 blocks. The
// eight lanes that feed B in one load (t = 0..3, limb j = g & 1) then touch 64 bytes in 16
// distinct banks (one wavefront), and a lane's four steps are a single base pointer plus the
// compile-time offsets 0, 16, 32, 48. Per 16-element block the scale and the sum sit side by
// side (float2), so one 16-byte load brings both 16-blocks of a lane's scale group.
//
// Pointer arguments are already advanced to the K group kg (256 elements = 576 bytes of limbs;
// 128-element groups of the 32-element block types = 288 bytes):
//   xq  = limbs + limb2_off(4t) + (g & 1) * 8 + kg * (blocks16 * 36);  step o at xq + 16 o,
//         the second chain of a 256-element group at + 288
//   xsp = scale_sum + kg * blocks16 + 2 t   (float2 {xsc, xss} per 16-element block)
#pragma once

#include "qgemv1_groups.cuh"

namespace {

// Byte offset of the 16-byte block of 8-element group B.
__device__ __forceinline__ int limb2_off(int B) { return 16 * B + 16 * (B >> 3); }
constexpr int LIMB2_CHAIN = 288;  // bytes from chain 0 to chain 1 of a 256-element group (16 blocks + 2 pads)

// 8 limb bytes of a lane that feeds B, zero otherwise.
__device__ __forceinline__ uint2 ldb2(const Lane& L, const uint8_t* p) {
  uint2 v = make_uint2(0u, 0u);
  if (L.feeds) v = *reinterpret_cast<const uint2*>(p);
  return v;
}

__device__ __forceinline__ float4 lds_f4(const float2* p) { return *reinterpret_cast<const float4*>(p); }

template <bool SIGNED_A>
__device__ __forceinline__ void step2(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, const uint2& v) {
  mma_i8_k32<SIGNED_A>(c, a0, a1, a2, a3, v.x, v.y);
}

// Integer dot products of one chain -> f32 in units of xsc.
__device__ __forceinline__ float limbs2_to_float(int c_l0, int c_l1) { return (float)(c_l0 * 128 + c_l1); }

__device__ __forceinline__ void group2_q4_0(const uint8_t* xq, const float2* xsp,
                                            const uint8_t* tg, const Lane& L, float& acc_g, float& acc_g8) {
  const uint4 qa = lds16(tg + L.g * 64 + L.t * 16);
  const uint4 qb = lds16(tg + 512 + L.g * 64 + L.t * 16);
  const float d_g = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 1024 + (L.g * 4 + L.t) * 2));
  const float d_g8 = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 1024 + ((L.g + 8) * 4 + L.t) * 2));
  const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w};
  const uint32_t wb[4] = {qb.x, qb.y, qb.z, qb.w};
  const float4 ss4 = lds_f4(xsp);  // {xsc, xss} of the lane's two 16-blocks
  const float2 xs2 = make_float2(ss4.x, ss4.z), sx2 = make_float2(ss4.y, ss4.w);
  float f_g = 0.f, f_g8 = 0.f;
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {  // elements 0..15 = low nibbles, 16..31 = high nibbles
    int c[4] = {0, 0, 0, 0};
#pragma unroll
    for (int sw = 0; sw < 2; ++sw) {
      const uint2 v = ldb2(L, xq + 16 * (hf * 2 + sw));
      const int w0 = sw * 2;
      if (hf == 0)
        step2<false>(c, wa[w0] & 0x0F0F0F0Fu, wb[w0] & 0x0F0F0F0Fu, wa[w0 + 1] & 0x0F0F0F0Fu, wb[w0 + 1] & 0x0F0F0F0Fu, v);
      else
        step2<false>(c, (wa[w0] >> 4) & 0x0F0F0F0Fu, (wb[w0] >> 4) & 0x0F0F0F0Fu, (wa[w0 + 1] >> 4) & 0x0F0F0F0Fu,
                     (wb[w0 + 1] >> 4) & 0x0F0F0F0Fu, v);
    }
    const float xs = hf ? xs2.y : xs2.x;
    f_g = fmaf(limbs2_to_float(c[0], c[1]), xs, f_g);
    f_g8 = fmaf(limbs2_to_float(c[2], c[3]), xs, f_g8);
  }
  const float sx8 = 8.0f * (sx2.x + sx2.y);  // (q - 8): centre folded into the sum
  acc_g = fmaf(d_g, f_g - sx8, acc_g);
  acc_g8 = fmaf(d_g8, f_g8 - sx8, acc_g8);
}

__device__ __forceinline__ void group2_q8_0(const uint8_t* xq, const float2* xsp, const uint8_t* tg,
                                            const Lane& L, float& acc_g, float& acc_g8) {
  uint4 q[2][2];  // [h][half]
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int half = 0; half < 2; ++half) q[h][half] = lds16(tg + (h * 2 + half) * 512 + L.g * 64 + L.t * 16);
  const float d_g = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 2048 + (L.g * 4 + L.t) * 2));
  const float d_g8 = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 2048 + ((L.g + 8) * 4 + L.t) * 2));
  const float4 ss4 = lds_f4(xsp);
  const float2 xs2 = make_float2(ss4.x, ss4.z);
  float f_g = 0.f, f_g8 = 0.f;
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    int c[4] = {0, 0, 0, 0};
    const uint4 a = q[0][hf], b = q[1][hf];
    step2<true>(c, a.x, b.x, a.y, b.y, ldb2(L, xq + 16 * (hf * 2)));
    step2<true>(c, a.z, b.z, a.w, b.w, ldb2(L, xq + 16 * (hf * 2 + 1)));
    const float xs = hf ? xs2.y : xs2.x;
    f_g = fmaf(limbs2_to_float(c[0], c[1]), xs, f_g);
    f_g8 = fmaf(limbs2_to_float(c[2], c[3]), xs, f_g8);
  }
  acc_g = fmaf(d_g, f_g, acc_g);
  acc_g8 = fmaf(d_g8, f_g8, acc_g8);
}

// Q4_K: chain ch covers sub-blocks 4ch .. 4ch+3; lane t owns sub-block 4ch + t (low or high
// nibbles of qs bytes 32 * (2ch + t/2) .. +32; high nibbles are used in place as 16 * q with the
// factor folded into the scale).
__device__ __forceinline__ void group2_q4k(const uint8_t* xq, const float2* xsp,
                                           const uint8_t* tg, const Lane& L, float& acc_g, float& acc_g8) {
  const uint32_t mask = (L.t & 1) ? 0xF0F0F0F0u : 0x0F0F0F0Fu;
  const float nib_scale = (L.t & 1) ? 0.0625f : 1.0f;
  const uint32_t sel = 0x4440u + (uint32_t)L.t;  // byte t of a word, zero-extended
  float sc_f[2][2], mn_f[2][2];  // [row half][chain]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint4 hd = lds16(tg + 2048 + (L.g + 8 * h) * 16);
    const float d = fb::half_bits_to_float((uint16_t)(hd.x & 0xFFFF)) * nib_scale;
    const float dmin = fb::half_bits_to_float((uint16_t)(hd.x >> 16));
    // 6-bit scales and mins of sub-blocks t and 4 + t (get_scale_min_k4 of the GGUF block)
    const uint32_t b0 = __byte_perm(hd.y, 0u, sel), b1 = __byte_perm(hd.z, 0u, sel), b2 = __byte_perm(hd.w, 0u, sel);
    sc_f[h][0] = d * (float)(b0 & 63u);
    mn_f[h][0] = dmin * (float)(b1 & 63u);
    sc_f[h][1] = d * (float)((b2 & 15u) | ((b0 >> 2) & 0x30u));
    mn_f[h][1] = dmin * (float)((b2 >> 4) | ((b1 >> 2) & 0x30u));
  }
  const int slot = L.g * 32 + (L.t >> 1) * 16;
#pragma unroll
  for (int ch = 0; ch < 2; ++ch) {
    const float4 ss4 = lds_f4(xsp + ch * 8);
    const float2 xs2 = make_float2(ss4.x, ss4.z), sx2 = make_float2(ss4.y, ss4.w);
    float f_g = 0.f, f_g8 = 0.f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {  // elements 0..15 and 16..31 of the sub-block
      int c[4] = {0, 0, 0, 0};
      const uint4 qa = lds16(tg + ((ch * 2 + 0) * 2 + half) * 256 + slot);
      const uint4 qb = lds16(tg + ((ch * 2 + 1) * 2 + half) * 256 + slot);
      const uint2 v0 = ldb2(L, xq + 16 * (half * 2) + ch * LIMB2_CHAIN);
      const uint2 v1 = ldb2(L, xq + 16 * (half * 2 + 1) + ch * LIMB2_CHAIN);
      step2<false>(c, qa.x & mask, qb.x & mask, qa.y & mask, qb.y & mask, v0);
      step2<false>(c, qa.z & mask, qb.z & mask, qa.w & mask, qb.w & mask, v1);
      const float xs = half ? xs2.y : xs2.x;
      f_g = fmaf(limbs2_to_float(c[0], c[1]), xs, f_g);
      f_g8 = fmaf(limbs2_to_float(c[2], c[3]), xs, f_g8);
    }
    const float sx = sx2.x + sx2.y;
    acc_g = fmaf(sc_f[0][ch], f_g, fmaf(-mn_f[0][ch], sx, acc_g));
    acc_g8 = fmaf(sc_f[1][ch], f_g8, fmaf(-mn_f[1][ch], sx, acc_g8));
  }
}

// Q6_K: chain (c, u) covers the 16-element groups 8c + 2q + u, q = 0..3; lane t owns q = t:
// nibble t/2 of ql plane slot t%2 and bits 2t, 2t+1 of qh, merged per byte into a u8 in 0..63.
__device__ __forceinline__ void group2_q6k(const uint8_t* xq, const float2* xsp,
                                           const uint8_t* tg, const Lane& L, float& acc_g, float& acc_g8) {
  const int sh4 = 4 * (L.t >> 1);
  const int rot = (4 - 2 * L.t) & 31;  // rotate-left that brings bits 2t, 2t+1 of each byte to 4, 5
  const uint4 sc_g = lds16(tg + 3072 + L.g * 16);
  const uint4 sc_g8 = lds16(tg + 3072 + (L.g + 8) * 16);
  const float d_g = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 3328 + L.g * 2));
  const float d_g8 = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 3328 + (L.g + 8) * 2));
  auto merge = [&](uint32_t wl, uint32_t wh) -> uint32_t {
    return ((wl >> sh4) & 0x0F0F0F0Fu) | (__funnelshift_l(wh, wh, rot) & 0x30303030u);
  };
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const float4 ss4 = lds_f4(xsp + 8 * c);
    const float2 xs2 = make_float2(ss4.x, ss4.z), sx2 = make_float2(ss4.y, ss4.w);
    // int8 scale bytes of this lane's groups 8c + 2t + u: word 2c + t/2, bytes 2(t%2) + u
    const uint32_t wg = (L.t >> 1) ? (c ? sc_g.w : sc_g.y) : (c ? sc_g.z : sc_g.x);
    const uint32_t wg8 = (L.t >> 1) ? (c ? sc_g8.w : sc_g8.y) : (c ? sc_g8.z : sc_g8.x);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int cu = 2 * c + u;
      const uint4 la = lds16(tg + (cu * 2 + 0) * 256 + L.g * 32 + (L.t & 1) * 16);
      const uint4 lb = lds16(tg + (cu * 2 + 1) * 256 + L.g * 32 + (L.t & 1) * 16);
      const uint4 ha = lds16(tg + 2048 + (cu * 2 + 0) * 128 + L.g * 16);
      const uint4 hb = lds16(tg + 2048 + (cu * 2 + 1) * 128 + L.g * 16);
      // this lane's scale group in the super-block is 8c + 2t + u: steps o = 2u, 2u + 1
      const uint2 v0 = ldb2(L, xq + 16 * (2 * u) + c * LIMB2_CHAIN);
      const uint2 v1 = ldb2(L, xq + 16 * (2 * u + 1) + c * LIMB2_CHAIN);
      int cc[4] = {0, 0, 0, 0};
      step2<false>(cc, merge(la.x, ha.x), merge(lb.x, hb.x), merge(la.y, ha.y), merge(lb.y, hb.y), v0);
      step2<false>(cc, merge(la.z, ha.z), merge(lb.z, hb.z), merge(la.w, ha.w), merge(lb.w, hb.w), v1);
      const int bsh = 8 * (2 * (L.t & 1) + u);
      const float s_g = d_g * (float)(int)(int8_t)((wg >> bsh) & 0xFF);
      const float s_g8 = d_g8 * (float)(int)(int8_t)((wg8 >> bsh) & 0xFF);
      const float xs = u ? xs2.y : xs2.x;
      const float sx32 = 32.0f * (u ? sx2.y : sx2.x);  // (q - 32): centre folded into the sum
      acc_g = fmaf(s_g, fmaf(limbs2_to_float(cc[0], cc[1]), xs, -sx32), acc_g);
      acc_g8 = fmaf(s_g8, fmaf(limbs2_to_float(cc[2], cc[3]), xs, -sx32), acc_g8);
    }
  }
}

// Pointers of a lane for K group kg. blocks16 = 16-element blocks per K group (8 or 16).
struct Group2Ptrs {
  const uint8_t* xq;
  const float2* xsp;
};
__device__ __forceinline__ Group2Ptrs group2_ptrs(const Lane& L, const uint8_t* xl, const float2* xsp, int kg, int blocks16) {
  Group2Ptrs G;
  G.xq = xl + limb2_off(4 * L.t) + (L.g & 1) * 8 + kg * blocks16 * 36;
  G.xsp = xsp + kg * blocks16 + 2 * L.t;
  return G;
}
__device__ __forceinline__ void group2_ptrs_next(Group2Ptrs& G, int blocks16) {
  G.xq += blocks16 * 36;
  G.xsp += blocks16;
}

}  // namespace
