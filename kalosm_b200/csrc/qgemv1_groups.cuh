// Per-tile-group inner products of the single-row quantised product: one warp, one tile-group
// (16 rows of W x one K group) against the activation limbs in shared memory.
//
// Mapping ("scale group per lane"): MMA lane (g = lane / 4, t = lane % 4) feeds, per
// mma.m16n8k32, 8 elements of ONE scale group of rows g and g + 8 (group index t of the chain);
// the B operand carries the activation limbs of group t' only in columns 2t', 2t'+1 and only in
// the k-slots of lane t' (lanes with g / 2 == t load their 16 limb bytes, all other lanes read
// 16 zero bytes), so lane t's accumulators hold the integer dot products of its own group with
// limb pairs (0, 1) and (2, 3). One scale decode per lane per chain, no shuffles until the end.
//
// Activation limbs: per 8 elements 32 bytes [limb 0 x8][limb 2 x8][limb 1 x8][limb 3 x8];
// q = rint(v / s * 2^27) as bit fields: l0 = q >> 21 (signed), then three 7-bit fields.
// xsc[b] = power-of-two scale of 16-element block b folded so that f * xsc[b] is the true
// partial dot product; xss[b] = true sum of the 16 activations (quant centres and offsets).
//
// Shared-memory placement of the limbs: the 32-byte block of 8-element group kb sits at block
// index kb ^ ((kb >> 2) & 3) (limb_block()), i.e. byte bits 5-6 are XOR-ed with bits 7-8. The
// lanes that feed B in one load differ exactly in bits 7-8 (their scale group t), so the swizzle
// spreads them over all 32 banks and a B load is a single conflict-free wavefront. Lanes that do
// not feed B skip the load (their operand is zero).
//
// Pointer arguments are already advanced to the K group `kg`:
//   xq[o] = limbs + (g & 1) * 16 + t * 128 + ((o ^ t) << 5) + kg * 4 * group_elems, o = 0..3
//           (o = the 8-element step inside a scale group; further offsets are multiples of 512)
//   xscp  = xsc + kg * (group_elems / 16) + 2 * t,  xssp likewise
// so every load below has a compile-time offset.
#pragma once

#include "qgemv_common.cuh"

namespace {

// Per-lane constants of the scale-group-per-lane mapping.
struct Lane {
  int g, t;
  bool feeds;  // this lane's k-slots carry the limbs of its scale group in the B operand
};

__device__ __forceinline__ Lane make_lane(int lane) {
  Lane L;
  L.g = lane >> 2; L.t = lane & 3;
  L.feeds = (L.g >> 1) == L.t;
  return L;
}

// Block index in shared memory of the limbs of 8-element group kb.
__device__ __forceinline__ int limb_block(int kb) { return kb ^ ((kb >> 2) & 3); }

// The four limb pointers of a lane for K group 0.
__device__ __forceinline__ void lane_limb_ptrs(const Lane& L, const uint8_t* xl, const uint8_t* (&xq)[4]) {
#pragma unroll
  for (int o = 0; o < 4; ++o) xq[o] = xl + (L.g & 1) * 16 + L.t * 128 + ((o ^ L.t) << 5);
}

// 16 limb bytes of a lane that feeds B, zero otherwise.
__device__ __forceinline__ uint4 ldb(const Lane& L, const uint8_t* p) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (L.feeds) v = *reinterpret_cast<const uint4*>(p);
  return v;
}

__device__ __forceinline__ uint4 lds16(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }

// Both limb pairs of one 8-element step.
template <bool SIGNED_A>
__device__ __forceinline__ void step(int (&c1)[4], int (&c2)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                     uint32_t a3, const uint4& v) {
  mma_i8_k32<SIGNED_A>(c1, a0, a1, a2, a3, v.x, v.y);
  mma_i8_k32<SIGNED_A>(c2, a0, a1, a2, a3, v.z, v.w);
}

// Integer dot products of one chain -> fp32 in units of 2^-13 * (w . x/scale):
// (C0 * 128 + C1) + (C2 * 128 + C3) / 2^14.
__device__ __forceinline__ float limbs_to_float(int c_l0, int c_l1, int c_l2, int c_l3) {
  return fmaf((float)(c_l2 * 128 + c_l3), 1.0f / 16384.0f, (float)(c_l0 * 128 + c_l1));
}

__device__ __forceinline__ float2 lds_f2(const float* p) { return *reinterpret_cast<const float2*>(p); }

__device__ __forceinline__ void group1_q4_0(const uint8_t* const (&xq)[4], const float* xscp, const float* xssp,
                                            const uint8_t* tg, const Lane& L, float& acc_g, float& acc_g8) {
  const uint4 qa = lds16(tg + L.g * 64 + L.t * 16);
  const uint4 qb = lds16(tg + 512 + L.g * 64 + L.t * 16);
  const float d_g = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 1024 + (L.g * 4 + L.t) * 2));
  const float d_g8 = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 1024 + ((L.g + 8) * 4 + L.t) * 2));
  const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w};
  const uint32_t wb[4] = {qb.x, qb.y, qb.z, qb.w};
  const float2 xs2 = lds_f2(xscp), sx2 = lds_f2(xssp);
  float f_g = 0.f, f_g8 = 0.f;
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {  // elements 0..15 = low nibbles, 16..31 = high nibbles
    int c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0};
#pragma unroll
    for (int sw = 0; sw < 2; ++sw) {
      const uint4 v = ldb(L, xq[hf * 2 + sw]);
      const int w0 = sw * 2;
      if (hf == 0)
        step<false>(c1, c2, wa[w0] & 0x0F0F0F0Fu, wb[w0] & 0x0F0F0F0Fu, wa[w0 + 1] & 0x0F0F0F0Fu,
                    wb[w0 + 1] & 0x0F0F0F0Fu, v);
      else
        step<false>(c1, c2, (wa[w0] >> 4) & 0x0F0F0F0Fu, (wb[w0] >> 4) & 0x0F0F0F0Fu,
                    (wa[w0 + 1] >> 4) & 0x0F0F0F0Fu, (wb[w0 + 1] >> 4) & 0x0F0F0F0Fu, v);
    }
    const float xs = hf ? xs2.y : xs2.x;
    f_g = fmaf(limbs_to_float(c1[0], c1[1], c2[0], c2[1]), xs, f_g);
    f_g8 = fmaf(limbs_to_float(c1[2], c1[3], c2[2], c2[3]), xs, f_g8);
  }
  const float sx8 = 8.0f * (sx2.x + sx2.y);  // (q - 8): centre folded into the sum
  acc_g = fmaf(d_g, f_g - sx8, acc_g);
  acc_g8 = fmaf(d_g8, f_g8 - sx8, acc_g8);
}

__device__ __forceinline__ void group1_q8_0(const uint8_t* const (&xq)[4], const float* xscp, const uint8_t* tg,
                                            const Lane& L, float& acc_g, float& acc_g8) {
  uint4 q[2][2];  // [h][half]
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int half = 0; half < 2; ++half) q[h][half] = lds16(tg + (h * 2 + half) * 512 + L.g * 64 + L.t * 16);
  const float d_g = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 2048 + (L.g * 4 + L.t) * 2));
  const float d_g8 = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 2048 + ((L.g + 8) * 4 + L.t) * 2));
  const float2 xs2 = lds_f2(xscp);
  float f_g = 0.f, f_g8 = 0.f;
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    int c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0};
    const uint4 a = q[0][hf], b = q[1][hf];
    step<true>(c1, c2, a.x, b.x, a.y, b.y, ldb(L, xq[hf * 2]));
    step<true>(c1, c2, a.z, b.z, a.w, b.w, ldb(L, xq[hf * 2 + 1]));
    const float xs = hf ? xs2.y : xs2.x;
    f_g = fmaf(limbs_to_float(c1[0], c1[1], c2[0], c2[1]), xs, f_g);
    f_g8 = fmaf(limbs_to_float(c1[2], c1[3], c2[2], c2[3]), xs, f_g8);
  }
  acc_g = fmaf(d_g, f_g, acc_g);
  acc_g8 = fmaf(d_g8, f_g8, acc_g8);
}

// Q4_K: chain ch covers sub-blocks 4ch .. 4ch+3; lane t owns sub-block 4ch + t, whose quants
// are the low (t even) or high (t odd) nibbles of qs bytes 32 * (2ch + t/2) .. +32. High
// nibbles are used in place as 16 * q and the factor goes into the scale.
__device__ __forceinline__ void group1_q4k(const uint8_t* const (&xq)[4], const float* xscp, const float* xssp,
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
    const float2 xs2 = lds_f2(xscp + ch * 8), sx2 = lds_f2(xssp + ch * 8);
    float f_g = 0.f, f_g8 = 0.f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {  // elements 0..15 and 16..31 of the sub-block
      int c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0};
      const uint4 qa = lds16(tg + ((ch * 2 + 0) * 2 + half) * 256 + slot);
      const uint4 qb = lds16(tg + ((ch * 2 + 1) * 2 + half) * 256 + slot);
      const uint4 v0 = ldb(L, xq[half * 2] + ch * 512);
      const uint4 v1 = ldb(L, xq[half * 2 + 1] + ch * 512);
      step<false>(c1, c2, qa.x & mask, qb.x & mask, qa.y & mask, qb.y & mask, v0);
      step<false>(c1, c2, qa.z & mask, qb.z & mask, qa.w & mask, qb.w & mask, v1);
      const float xs = half ? xs2.y : xs2.x;
      f_g = fmaf(limbs_to_float(c1[0], c1[1], c2[0], c2[1]), xs, f_g);
      f_g8 = fmaf(limbs_to_float(c1[2], c1[3], c2[2], c2[3]), xs, f_g8);
    }
    const float sx = sx2.x + sx2.y;
    acc_g = fmaf(sc_f[0][ch], f_g, fmaf(-mn_f[0][ch], sx, acc_g));
    acc_g8 = fmaf(sc_f[1][ch], f_g8, fmaf(-mn_f[1][ch], sx, acc_g8));
  }
}

// Q6_K: chain (c, u) covers the 16-element groups 8c + 2q + u, q = 0..3; lane t owns q = t:
// nibble t/2 of ql plane slot t%2 and bits 2t, 2t+1 of qh, merged per byte into a u8 in 0..63.
__device__ __forceinline__ void group1_q6k(const uint8_t* const (&xq)[4], const float* xscp, const float* xssp,
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
    const float2 xs2 = lds_f2(xscp + 8 * c), sx2 = lds_f2(xssp + 8 * c);
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
      const uint4 v0 = ldb(L, xq[2 * u] + c * 512);
      const uint4 v1 = ldb(L, xq[2 * u + 1] + c * 512);
      int c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0};
      step<false>(c1, c2, merge(la.x, ha.x), merge(lb.x, hb.x), merge(la.y, ha.y), merge(lb.y, hb.y), v0);
      step<false>(c1, c2, merge(la.z, ha.z), merge(lb.z, hb.z), merge(la.w, ha.w), merge(lb.w, hb.w), v1);
      const int bsh = 8 * (2 * (L.t & 1) + u);
      const float s_g = d_g * (float)(int)(int8_t)((wg >> bsh) & 0xFF);
      const float s_g8 = d_g8 * (float)(int)(int8_t)((wg8 >> bsh) & 0xFF);
      const float xs = u ? xs2.y : xs2.x;
      const float sx32 = 32.0f * (u ? sx2.y : sx2.x);  // (q - 32): centre folded into the sum
      acc_g = fmaf(s_g, fmaf(limbs_to_float(c1[0], c1[1], c2[0], c2[1]), xs, -sx32), acc_g);
      acc_g8 = fmaf(s_g8, fmaf(limbs_to_float(c1[2], c1[3], c2[2], c2[3]), xs, -sx32), acc_g8);
    }
  }
}

// Pointers of a lane for K group kg. group_elems = 128 (Q4_0, Q8_0) or 256 (Q4_K, Q6_K).
struct GroupPtrs {
  const uint8_t* xq[4];
  const float* xscp;
  const float* xssp;
};
__device__ __forceinline__ GroupPtrs group_ptrs(const Lane& L, const uint8_t* xl, const float* xsc,
                                                const float* xss, int kg, int blocks16) {
  GroupPtrs G;
  lane_limb_ptrs(L, xl, G.xq);
#pragma unroll
  for (int o = 0; o < 4; ++o) G.xq[o] += kg * blocks16 * 64;
  G.xscp = xsc + kg * blocks16 + 2 * L.t;
  G.xssp = xss + kg * blocks16 + 2 * L.t;
  return G;
}
__device__ __forceinline__ void group_ptrs_next(GroupPtrs& G, int blocks16) {
#pragma unroll
  for (int o = 0; o < 4; ++o) G.xq[o] += blocks16 * 64;
  G.xscp += blocks16;
  G.xssp += blocks16;
}

// One tile-group of any tiled type.
__device__ __forceinline__ void group1_any(int type, const GroupPtrs& G, const uint8_t* tg, const Lane& L,
                                           float& acc_g, float& acc_g8) {
  if (type == FB200_Q4_K) group1_q4k(G.xq, G.xscp, G.xssp, tg, L, acc_g, acc_g8);
  else if (type == FB200_Q6_K) group1_q6k(G.xq, G.xscp, G.xssp, tg, L, acc_g, acc_g8);
  else if (type == FB200_Q8_0) group1_q8_0(G.xq, G.xscp, tg, L, acc_g, acc_g8);
  else group1_q4_0(G.xq, G.xscp, G.xssp, tg, L, acc_g, acc_g8);
}

// Orderable key of (finite value, index): larger value wins, equal values -> larger index
// (the tie rule of Tensor::top_k_pairs, fusor-ml/fusor/src/lib.rs:432-443). 0 = nothing yet.
__device__ __forceinline__ unsigned long long argmax_key_of(float v, uint32_t idx) {
  if (!isfinite(v)) return 0ull;
  uint32_t b = __float_as_uint(v);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return ((unsigned long long)b << 32) | (unsigned long long)idx;
}

}  // namespace
