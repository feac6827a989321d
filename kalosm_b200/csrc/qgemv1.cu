// Decode GEMV: y[N] = W[N, K] . x[K] for ONE activation row, the shape of batch-1 decoding.
//
// Bound: HBM (algorithmic bytes = the raw GGUF bytes of W). Structure:
//  * persistent CTAs (SM count x CTAs per SM) walk the 16-row tiles of W; the warps of a CTA
//    split a tile's K groups; partial sums meet in shared memory in a fixed order;
//  * every warp owns a ring of shared-memory stages filled by 1-D TMA bulk copies
//    (cp.async.bulk + mbarrier complete_tx), one contiguous tile-group per stage, so tens of KB
//    per SM are in flight without holding registers; the first copies are issued before
//    griddepcontrol.wait, i.e. under programmatic dependent launch the weights stream in
//    while the kernel that produces x is still running;
//  * one launch may carry up to three matrices that share the activation row (the q, k and v
//    projections), of different quant types;
//  * the prologue turns x into int8 MMA B operands in shared memory once per CTA: optional
//    residual add and RMSNorm (so the norm needs no kernel of its own), a power-of-two row
//    scale, then FOUR 7-bit limbs per element, the bit fields of q = rint(x/scale * 2^27)
//    (x/scale = (l0 + u1/2^7 + u2/2^14 + u3/2^21) / 64 to 2^-28, l0 signed, u 0..127), plus the
//    per-16 sums the offsets of Q4_K/Q4_0/Q6_K need;
//  * quants stay in the byte domain: one logic op turns four packed nibbles into four u8
//    operands of mma.sync.m16n8k32 (u8 x s8 -> s32, exact), so the ALU pipe that limits an
//    fp16 expansion is nearly idle;
//  * "scale group per lane": in every MMA lane t of a quad feeds eight elements of scale group
//    t (for rows g and g+8), and the B operand carries the limbs of group t' only in columns
//    2t', 2t'+1. The accumulator of lane t then holds exactly its own group's integer dot
//    products, so each lane decodes and applies ONE scale per chain of MMAs and no data is
//    exchanged between lanes until the final sum;
//  * integer dot products are exact; they are scaled and accumulated in fp32.
//
// Replaces the reference's qgemv kernels (fusor-ml/tile-ir-kernels/src/kernels/qgemv.rs:356-678,
// qgemv_q6k.rs:84-385), their SwiGLU and residual epilogues
// (fusor-ml/core/src/quantized/matmul/mod.rs:435-439, 666-722) and the fused RMSNorm cluster
// (fusor-ml/core/src/composite/rms_norm_fused.rs:10-54) in front of a projection.
#include "packed_act.cuh"
#include "qgemv_common.cuh"

namespace {

// One weight matrix of a launch. A launch may carry up to three matrices that share the
// activation row (q, k and v projections), possibly of different quant types.
struct Seg {
  const uint8_t* w;
  float* y;
  int type;      // ggml type id
  int tg;        // bytes per tile-group
  int units;     // tiles (or gate/up tile pairs) of this matrix
  int n_out;
};

struct Gemv1Args {
  Seg seg[3];
  int nseg;
  const float* x;       // [K]
  const float* xres;    // optional [K]: v = x + xres
  const float* norm_w;  // optional [K]: activation = v / sqrt(mean(v^2) + eps) * norm_w
  float eps;
  int K, Kp;            // logical and padded (ngroups * group_elems) inner size
  const float* r1;
  const float* r2;
  unsigned long long* argmax_key;  // optional: running (value, index) maximum of seg[0]'s outputs
  fb200_packed_act xp;   // optional (xp.limbs != null): the activation row, already packed
  int xp_norm;           // ... to be divided by its RMS (weights already applied by the producer)
  fb200_packed_act yp;   // optional: also emit seg[0]'s output row in packed form
  const float* yp_norm_w;
  const float* yp_add;
  int ngroups, nunits, pair_tile_offset, stages, stride;
  int* status;
};

// Per-lane constants of the scale-group-per-lane mapping.
struct Lane {
  int g, t;
  // B data: lanes with g / 2 == t supply the limbs of group t in column g (limb pair g % 2:
  // 0 -> limbs 0 and 2, 1 -> limbs 1 and 3); every other lane reads 16 zero bytes. Encoded as a
  // base pointer and a stride so the load needs no branch: address = xb + block * xstep.
  const uint8_t* xb;
  int xstep;
};

__device__ __forceinline__ uint4 lds16(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }

// Limbs of 8-element block kb: 32 bytes = [e = 0: limb0 x8, limb2 x8][e = 1: limb1 x8, limb3 x8].
__device__ __forceinline__ uint4 load_limbs(const uint8_t* /*xl*/, int kb, const Lane& L) {
  return lds16(L.xb + kb * L.xstep);
}

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

// The four group functions below take, besides the limbs `xl`, two per-16-element arrays:
// xsc[b] = power-of-two scale of x-block b (true x = limb value * xsc[b] * 2^13 / 128 ...,
// folded so that f * xsc[b] is the true partial dot product) and xss[b] = true sum of the 16
// activations (for the quant centres and offsets).
__device__ __forceinline__ void group1_q4_0(const uint8_t* xl, const float* xsc, const float* xss,
                                            const uint8_t* tg, int kg, const Lane& L, float& acc_g,
                                            float& acc_g8) {
  const uint4 qa = lds16(tg + L.g * 64 + L.t * 16);
  const uint4 qb = lds16(tg + 512 + L.g * 64 + L.t * 16);
  const float d_g = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 1024 + (L.g * 4 + L.t) * 2));
  const float d_g8 = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 1024 + ((L.g + 8) * 4 + L.t) * 2));
  const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w};
  const uint32_t wb[4] = {qb.x, qb.y, qb.z, qb.w};
  const int blk = kg * 4 + L.t;
  float f_g = 0.f, f_g8 = 0.f;
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {  // elements 0..15 = low nibbles, 16..31 = high nibbles
    int c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0};
#pragma unroll
    for (int sw = 0; sw < 2; ++sw) {
      const uint4 v = load_limbs(xl, blk * 4 + hf * 2 + sw, L);
      const int w0 = sw * 2;
      if (hf == 0)
        step<false>(c1, c2, wa[w0] & 0x0F0F0F0Fu, wb[w0] & 0x0F0F0F0Fu, wa[w0 + 1] & 0x0F0F0F0Fu,
                    wb[w0 + 1] & 0x0F0F0F0Fu, v);
      else
        step<false>(c1, c2, (wa[w0] >> 4) & 0x0F0F0F0Fu, (wb[w0] >> 4) & 0x0F0F0F0Fu,
                    (wa[w0 + 1] >> 4) & 0x0F0F0F0Fu, (wb[w0 + 1] >> 4) & 0x0F0F0F0Fu, v);
    }
    const float xs = xsc[blk * 2 + hf];
    f_g = fmaf(limbs_to_float(c1[0], c1[1], c2[0], c2[1]), xs, f_g);
    f_g8 = fmaf(limbs_to_float(c1[2], c1[3], c2[2], c2[3]), xs, f_g8);
  }
  const float sx8 = 8.0f * (xss[blk * 2] + xss[blk * 2 + 1]);  // (q - 8): centre folded into the sum
  acc_g = fmaf(d_g, f_g - sx8, acc_g);
  acc_g8 = fmaf(d_g8, f_g8 - sx8, acc_g8);
}

__device__ __forceinline__ void group1_q8_0(const uint8_t* xl, const float* xsc, const uint8_t* tg,
                                            int kg, const Lane& L, float& acc_g, float& acc_g8) {
  uint4 q[2][2];  // [h][half]
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int half = 0; half < 2; ++half) q[h][half] = lds16(tg + (h * 2 + half) * 512 + L.g * 64 + L.t * 16);
  const float d_g = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 2048 + (L.g * 4 + L.t) * 2));
  const float d_g8 = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 2048 + ((L.g + 8) * 4 + L.t) * 2));
  const int blk = kg * 4 + L.t;
  float f_g = 0.f, f_g8 = 0.f;
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    int c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0};
    const uint4 a = q[0][hf], b = q[1][hf];
    step<true>(c1, c2, a.x, b.x, a.y, b.y, load_limbs(xl, blk * 4 + hf * 2, L));
    step<true>(c1, c2, a.z, b.z, a.w, b.w, load_limbs(xl, blk * 4 + hf * 2 + 1, L));
    const float xs = xsc[blk * 2 + hf];
    f_g = fmaf(limbs_to_float(c1[0], c1[1], c2[0], c2[1]), xs, f_g);
    f_g8 = fmaf(limbs_to_float(c1[2], c1[3], c2[2], c2[3]), xs, f_g8);
  }
  acc_g = fmaf(d_g, f_g, acc_g);
  acc_g8 = fmaf(d_g8, f_g8, acc_g8);
}

// Q4_K: chain ch covers sub-blocks 4ch .. 4ch+3; lane t owns sub-block 4ch + t, whose quants
// are the low (t even) or high (t odd) nibbles of qs bytes 32 * (2ch + t/2) .. +32. High
// nibbles are used in place as 16 * q and the factor goes into the scale.
__device__ __forceinline__ void group1_q4k(const uint8_t* xl, const float* xsc, const float* xss,
                                           const uint8_t* tg, int kg, const Lane& L, float& acc_g,
                                           float& acc_g8) {
  const uint32_t mask = (L.t & 1) ? 0xF0F0F0F0u : 0x0F0F0F0Fu;
  const float nib_scale = (L.t & 1) ? 0.0625f : 1.0f;
  float sc_f[2][2], mn_f[2][2];  // [row half][chain]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint4 hd = lds16(tg + 2048 + (L.g + 8 * h) * 16);
    const float d = fb::half_bits_to_float((uint16_t)(hd.x & 0xFFFF)) * nib_scale;
    const float dmin = fb::half_bits_to_float((uint16_t)(hd.x >> 16));
    const uint32_t s0 = hd.y, s1 = hd.z, s2 = hd.w;
    const uint32_t scB = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
    const uint32_t mnB = ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u);
    const int sh = 8 * L.t;
    sc_f[h][0] = d * (float)((s0 >> sh) & 0x3F);
    mn_f[h][0] = dmin * (float)((s1 >> sh) & 0x3F);
    sc_f[h][1] = d * (float)((scB >> sh) & 0xFF);
    mn_f[h][1] = dmin * (float)((mnB >> sh) & 0xFF);
  }
  const int slot = L.g * 32 + (L.t >> 1) * 16;
#pragma unroll
  for (int ch = 0; ch < 2; ++ch) {
    const int sb = kg * 8 + ch * 4 + L.t;
    float f_g = 0.f, f_g8 = 0.f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {  // elements 0..15 and 16..31 of the sub-block
      int c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0};
      const uint4 qa = lds16(tg + ((ch * 2 + 0) * 2 + half) * 256 + slot);
      const uint4 qb = lds16(tg + ((ch * 2 + 1) * 2 + half) * 256 + slot);
      const uint4 v0 = load_limbs(xl, sb * 4 + half * 2, L);
      const uint4 v1 = load_limbs(xl, sb * 4 + half * 2 + 1, L);
      step<false>(c1, c2, qa.x & mask, qb.x & mask, qa.y & mask, qb.y & mask, v0);
      step<false>(c1, c2, qa.z & mask, qb.z & mask, qa.w & mask, qb.w & mask, v1);
      const float xs = xsc[sb * 2 + half];
      f_g = fmaf(limbs_to_float(c1[0], c1[1], c2[0], c2[1]), xs, f_g);
      f_g8 = fmaf(limbs_to_float(c1[2], c1[3], c2[2], c2[3]), xs, f_g8);
    }
    const float sx = xss[sb * 2] + xss[sb * 2 + 1];
    acc_g = fmaf(sc_f[0][ch], f_g, fmaf(-mn_f[0][ch], sx, acc_g));
    acc_g8 = fmaf(sc_f[1][ch], f_g8, fmaf(-mn_f[1][ch], sx, acc_g8));
  }
}

// Q6_K: chain (c, u) covers the 16-element groups 8c + 2q + u, q = 0..3; lane t owns q = t:
// nibble t/2 of ql plane slot t%2 and bits 2t, 2t+1 of qh, merged per byte into a u8 in 0..63.
__device__ __forceinline__ void group1_q6k(const uint8_t* xl, const float* xsc, const float* xss,
                                           const uint8_t* tg, int kg, const Lane& L, float& acc_g,
                                           float& acc_g8) {
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
  for (int cu = 0; cu < 4; ++cu) {  // cu = 2c + u
    const int c = cu >> 1, u = cu & 1;
    const uint4 la = lds16(tg + (cu * 2 + 0) * 256 + L.g * 32 + (L.t & 1) * 16);
    const uint4 lb = lds16(tg + (cu * 2 + 1) * 256 + L.g * 32 + (L.t & 1) * 16);
    const uint4 ha = lds16(tg + 2048 + (cu * 2 + 0) * 128 + L.g * 16);
    const uint4 hb = lds16(tg + 2048 + (cu * 2 + 1) * 128 + L.g * 16);
    const int grp = 8 * c + 2 * L.t + u;           // this lane's scale group in the super-block
    const int kb = (kg * 16 + grp) * 2;
    const uint4 v0 = load_limbs(xl, kb, L);
    const uint4 v1 = load_limbs(xl, kb + 1, L);
    int c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0};
    step<false>(c1, c2, merge(la.x, ha.x), merge(lb.x, hb.x), merge(la.y, ha.y), merge(lb.y, hb.y), v0);
    step<false>(c1, c2, merge(la.z, ha.z), merge(lb.z, hb.z), merge(la.w, ha.w), merge(lb.w, hb.w), v1);
    // int8 scale byte `grp` of rows g and g+8: word grp/4 = 2c + t/2, byte grp%4 = 2(t%2) + u
    const uint32_t wg = (L.t >> 1) ? (c ? sc_g.w : sc_g.y) : (c ? sc_g.z : sc_g.x);
    const uint32_t wg8 = (L.t >> 1) ? (c ? sc_g8.w : sc_g8.y) : (c ? sc_g8.z : sc_g8.x);
    const int bsh = 8 * (2 * (L.t & 1) + u);
    const float s_g = d_g * (float)(int)(int8_t)((wg >> bsh) & 0xFF);
    const float s_g8 = d_g8 * (float)(int)(int8_t)((wg8 >> bsh) & 0xFF);
    const float xs = xsc[kg * 16 + grp];
    const float sx32 = 32.0f * xss[kg * 16 + grp];  // (q - 32): centre folded into the sum
    acc_g = fmaf(s_g, fmaf(limbs_to_float(c1[0], c1[1], c2[0], c2[1]), xs, -sx32), acc_g);
    acc_g8 = fmaf(s_g8, fmaf(limbs_to_float(c1[2], c1[3], c2[2], c2[3]), xs, -sx32), acc_g8);
  }
}

// Orderable key of (finite value, index): larger value wins, equal values -> larger index
// (the tie rule of Tensor::top_k_pairs, fusor-ml/fusor/src/lib.rs:432-443). 0 = nothing yet.
__device__ __forceinline__ unsigned long long argmax_key_of(float v, uint32_t idx) {
  if (!isfinite(v)) return 0ull;
  uint32_t b = __float_as_uint(v);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return ((unsigned long long)b << 32) | (unsigned long long)idx;
}

// TYPE: ggml type of the (single) matrix, or 0 = several matrices whose types are read at run
// time. EPI: 0 none, 1 residual(s), 2 SwiGLU pair. W = warps per CTA, MINB = CTAs per SM.
template <int TYPE, int EPI, int W, int MINB>
__global__ void __launch_bounds__(W * 32, MINB)
qgemv1_kernel(const Gemv1Args a) {
  constexpr int NP = EPI == 2 ? 2 : 1;
  constexpr int THREADS = W * 32;
  extern __shared__ __align__(128) uint8_t smem[];
  const int S = a.stages;
  uint8_t* ring = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + W * S * a.stride);
  uint8_t* xl = smem + W * S * a.stride + W * S * 8;  // first raw f32 x, then limbs (4 B / element)
  float* xf = reinterpret_cast<float*>(xl);
  float* xsc = reinterpret_cast<float*>(xl + (size_t)a.Kp * 4);  // per-16 scale of the limbs
  float* xss = xsc + a.Kp / 16;    // per-16 sum of the activations
  float* red = xss + a.Kp / 16;    // [NP][W][16]
  float* tmp = red + NP * W * 16;  // [2 W] block reductions
  uint8_t* zero16 = reinterpret_cast<uint8_t*>(tmp + 2 * W);  // 16 zero bytes (W is a multiple of 8)
  uint64_t* xbar = reinterpret_cast<uint64_t*>(zero16 + 16);  // arrival of a packed activation row

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Lane L;
  L.g = lane >> 2; L.t = lane & 3;
  {
    const bool mine = (L.g >> 1) == L.t;
    L.xb = mine ? xl + (L.g & 1) * 16 : zero16;
    L.xstep = mine ? 32 : 0;
  }
  if (threadIdx.x < 4) reinterpret_cast<uint32_t*>(zero16)[threadIdx.x] = 0u;
  uint8_t* my_ring = ring + warp * S * a.stride;
  const uint32_t my_bar = smem_u32(bars + warp * S);

  pdl_launch_dependents();
  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(my_bar + 8 * s, 1);
    if (warp == 0) mbar_init(smem_u32(xbar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // this warp's items in issue order: for each unit of the CTA, for each pass (gate / up), the
  // K groups warp, warp + W, ...
  const int gw = a.ngroups > warp ? (a.ngroups - warp + W - 1) / W : 0;
  const int my_units = a.nunits > (int)blockIdx.x ? (a.nunits - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int n_items = my_units * NP * gw;
  // unit -> (matrix, tile inside it)
  auto locate = [&](int unit, int& sidx, int& tile) {
    sidx = 0; tile = unit;
    if (TYPE == 0) {
      if (a.nseg > 1 && tile >= a.seg[0].units) { tile -= a.seg[0].units; sidx = 1; }
      if (a.nseg > 2 && sidx == 1 && tile >= a.seg[1].units) { tile -= a.seg[1].units; sidx = 2; }
    }
  };
  int is_unit = blockIdx.x, is_p = 0, is_kk = 0, issued = 0;  // issue-side cursor (lane 0)
  auto issue_next = [&](int st) {
    int sidx, tile;
    locate(is_unit, sidx, tile);
    const uint8_t* wbase = a.seg[0].w;
    int tgb = a.seg[0].tg;
    if (TYPE == 0 && sidx == 1) { wbase = a.seg[1].w; tgb = a.seg[1].tg; }
    if (TYPE == 0 && sidx == 2) { wbase = a.seg[2].w; tgb = a.seg[2].tg; }
    const uint8_t* src = wbase + ((size_t)(tile + is_p * a.pair_tile_offset) * a.ngroups + (warp + W * is_kk)) * tgb;
    mbar_expect_tx(my_bar + 8 * st, tgb);
    bulk_g2s(smem_u32(my_ring + st * a.stride), src, tgb, my_bar + 8 * st);
    ++issued;
    if (++is_kk == gw) {
      is_kk = 0;
      if (++is_p == NP) { is_p = 0; is_unit += gridDim.x; }
    }
  };
  if (lane == 0) {
    const int pre = n_items < S ? n_items : S;
    for (int i = 0; i < pre; ++i) issue_next(i);
  }
  // only weights were touched so far; x comes from the kernel before this one
  pdl_wait();

  // ---- activation prologue ------------------------------------------------------------------
  float final_scale = 1.0f;
  if (a.xp.limbs) {
    // The producer already packed the row: three bulk copies bring limbs, scales and sums into
    // shared memory; for an RMSNorm consumer the per-16 sums of squares are added in index
    // order and 1/rms becomes the final factor.
    __syncthreads();  // xbar initialised
    if (threadIdx.x == 0) {
      const uint32_t nb = (uint32_t)a.Kp * 4u, ns = (uint32_t)(a.Kp / 16) * 4u;
      mbar_expect_tx(smem_u32(xbar), nb + 2u * ns);
      bulk_g2s(smem_u32(xl), a.xp.limbs, nb, smem_u32(xbar));
      bulk_g2s(smem_u32(xsc), a.xp.xsc, ns, smem_u32(xbar));
      bulk_g2s(smem_u32(xss), a.xp.xss, ns, smem_u32(xbar));
    }
    if (a.xp_norm) {
      float ss = 0.f;
      for (int i = threadIdx.x; i < (a.K + 15) / 16; i += THREADS) ss += a.xp.sumsq[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
      if (lane == 0) tmp[warp] = ss;
      __syncthreads();
      ss = 0.f;
      for (int i = 0; i < W; ++i) ss += tmp[i];
      final_scale = 1.0f / sqrtf(ss / (float)a.K + a.eps);
    }
    mbar_wait(smem_u32(xbar), 0u, a.status);
  } else {
  // pass 1: v = x (+ residual) -> shared memory as f32;
    //         sum of squares and max |v * norm_w| in one block reduction
    float ss = 0.f, amax = 0.f;
    {
      for (int k = threadIdx.x; k < a.Kp; k += THREADS) {
        float v = 0.f;
        if (k < a.K) {
          v = a.x[k];
          if (a.xres) v += a.xres[k];
          ss = fmaf(v, v, ss);
          amax = fmaxf(amax, fabsf(a.norm_w ? v * a.norm_w[k] : v));
        }
        xf[k] = v;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
      amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    }
    if (lane == 0) { tmp[warp] = ss; tmp[W + warp] = amax; }
    __syncthreads();
    ss = 0.f; amax = 0.f;
    for (int i = 0; i < W; ++i) { ss += tmp[i]; amax = fmaxf(amax, tmp[W + i]); }
    float rms = 1.f;
    if (a.norm_w) {
      // rms_norm_fused_cpu_impl, fusor-ml/fusor/src/composite/normalization.rs:404-461
      rms = sqrtf(ss / (float)a.K + a.eps);
      amax = amax / rms * 1.0000005f;  // bound of |(v / rms) * w| with rounding slack
    }
    int ex = 0;
    if (amax > 0.f && amax < 3.0e38f) frexpf(amax, &ex);  // amax = f * 2^ex, f in [0.5, 1)
    const float inv64 = ldexpf(64.0f, -ex);               // x * inv64 in (-64, 64)
    const float out_scale = ldexpf(1.0f, ex - 13);        // 2^ex / (64 * 128)
    // pass 2: each thread turns whole 8-element blocks, in place, into four int8 limbs per element:
    // q = rint(v * 2^21) (|q| <= 2^27), l0 = q >> 21 (signed), u1, u2, u3 = the next three 7-bit
    // fields (0..127), so v = (l0 + u1/2^7 + u2/2^14 + u3/2^21) up to 2^-22.
    const float qscale = inv64 * 2097152.0f;
    const float inv_rms = 1.0f / rms;  // v * (1/rms) instead of v / rms: within 1.5 ulp of the division
    const int nblk = a.Kp >> 3;
    for (int b0 = 0; b0 < nblk; b0 += THREADS) {
      const int kb = b0 + threadIdx.x;
      float sum = 0.f;
      uint32_t wl[2][4];  // [half of the block][limb 3, 2, 1, 0] four elements per word
      if (kb < nblk) {
        const float4 va = *reinterpret_cast<const float4*>(xf + kb * 8);
        const float4 vb = *reinterpret_cast<const float4*>(xf + kb * 8 + 4);
        const float vin[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
        uint32_t r[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int k = kb * 8 + i;
          float v = vin[i];
          if (a.norm_w && k < a.K) v = (v * inv_rms) * a.norm_w[k];
          const int q = __float2int_rn(v * qscale);
          sum += (float)q;
          // fields at bits 0, 7, 14, 21 -> bytes 0..3 (byte 3 = bits 21..28 = l0 as s8)
          r[i] = ((uint32_t)q & 0x7Fu) | (((uint32_t)q << 1) & 0x7F00u) | (((uint32_t)q << 2) & 0x7F0000u) |
                 (((uint32_t)q << 3) & 0xFF000000u);
        }
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          // 4 x 4 byte transpose: word j = byte j of the four elements
          const uint32_t t01l = __byte_perm(r[4 * hb], r[4 * hb + 1], 0x5140), t23l = __byte_perm(r[4 * hb + 2], r[4 * hb + 3], 0x5140);
          const uint32_t t01h = __byte_perm(r[4 * hb], r[4 * hb + 1], 0x7362), t23h = __byte_perm(r[4 * hb + 2], r[4 * hb + 3], 0x7362);
          wl[hb][0] = __byte_perm(t01l, t23l, 0x5410);  // u3
          wl[hb][1] = __byte_perm(t01l, t23l, 0x7632);  // u2
          wl[hb][2] = __byte_perm(t01h, t23h, 0x5410);  // u1
          wl[hb][3] = __byte_perm(t01h, t23h, 0x7632);  // l0
        }
      }
      // per-16 sums in the units of the integer dot products (128 * sum(v) = sum(q) / 2^14)
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
      if (kb < nblk) {
        uint4* dst = reinterpret_cast<uint4*>(xl + (size_t)kb * 32);
        dst[0] = make_uint4(wl[0][3], wl[1][3], wl[0][1], wl[1][1]);  // limb 0, limb 2
        dst[1] = make_uint4(wl[0][2], wl[1][2], wl[0][0], wl[1][0]);  // limb 1, limb 3
        if ((threadIdx.x & 1) == 0) {
          xsc[kb >> 1] = out_scale;
          xss[kb >> 1] = sum * (1.0f / 16384.0f) * out_scale;
        }
      }
    }
    __syncthreads();
  }
  __syncthreads();

  int item = 0, st = 0;
  uint32_t phase = 0;
  unsigned long long best_key = 0ull;
  for (int j = 0; j < my_units; ++j) {
    const int unit = (int)blockIdx.x + j * (int)gridDim.x;
    int sidx, tile;
    locate(unit, sidx, tile);
    int type = TYPE ? TYPE : a.seg[0].type, n_out = a.seg[0].n_out;
    float* yout = a.seg[0].y;
    if (TYPE == 0 && sidx == 1) { type = a.seg[1].type; n_out = a.seg[1].n_out; yout = a.seg[1].y; }
    if (TYPE == 0 && sidx == 2) { type = a.seg[2].type; n_out = a.seg[2].n_out; yout = a.seg[2].y; }
    if (j > 0) __syncthreads();  // the previous unit's reduction has read `red`
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      float acc_g = 0.f, acc_g8 = 0.f;
      for (int kk = 0; kk < gw; ++kk, ++item) {
        mbar_wait(my_bar + 8 * st, phase, a.status);
        const uint8_t* tg = my_ring + st * a.stride;
        const int kg = warp + W * kk;
        if (type == FB200_Q4_K) group1_q4k(xl, xsc, xss, tg, kg, L, acc_g, acc_g8);
        else if (type == FB200_Q6_K) group1_q6k(xl, xsc, xss, tg, kg, L, acc_g, acc_g8);
        else if (type == FB200_Q8_0) group1_q8_0(xl, xsc, tg, kg, L, acc_g, acc_g8);
        else group1_q4_0(xl, xsc, xss, tg, kg, L, acc_g, acc_g8);
        // Every lane has read the stage (its loads precede this barrier in program order and
        // shared loads complete long before a refill from global memory can land).
        __syncwarp();
        if (lane == 0 && issued < n_items) issue_next(st);
        if (++st == S) { st = 0; phase ^= 1u; }
      }
      // lane t accumulated the scale groups it owns: sum over the quad
      acc_g += __shfl_xor_sync(0xFFFFFFFFu, acc_g, 1);
      acc_g += __shfl_xor_sync(0xFFFFFFFFu, acc_g, 2);
      acc_g8 += __shfl_xor_sync(0xFFFFFFFFu, acc_g8, 1);
      acc_g8 += __shfl_xor_sync(0xFFFFFFFFu, acc_g8, 2);
      if (L.t == 0) {
        red[(p * W + warp) * 16 + L.g] = acc_g;
        red[(p * W + warp) * 16 + L.g + 8] = acc_g8;
      }
    }
    __syncthreads();
    if (threadIdx.x < 16) {
      const int r = threadIdx.x;
      const int n = tile * 16 + r;
      const bool valid = n < n_out;
      float v[NP];
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        float s = 0.f;
        for (int w = 0; w < W; ++w) s += red[(p * W + w) * 16 + r];
        v[p] = s * final_scale;
      }
      float out = 0.f;
      if (valid) {
        if (EPI == 2) {
          // silu(gate) * up, fusor-ml/fusor/src/composite/activations.rs:47-64
          const float gate = v[0];
          out = (gate / (1.0f + expf(-gate))) * v[NP - 1];
        } else if (EPI == 1) {
          out = v[0] + a.r1[n];
          if (a.r2) out += a.r2[n];
        } else {
          out = v[0];
        }
        if (yout) yout[n] = out;
        if (a.argmax_key && sidx == 0) {
          const unsigned long long key = argmax_key_of(out, (uint32_t)n);
          if (key > best_key) best_key = key;
        }
      }
      if (a.yp.limbs && sidx == 0) {
        float pv = out;
        if (valid && a.yp_add) pv += a.yp_add[n];
        const float nv = pv;
        if (valid && a.yp_norm_w) pv *= a.yp_norm_w[n];
        emit_packed16(a.yp, n, pv, nv, valid, 0x0000FFFFu);
      }
    }
  }
  if (a.argmax_key && threadIdx.x < 32) {
    // threads 0..15 carry the maxima of the rows they wrote; one atomic per CTA
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, best_key, o);
      if (other > best_key) best_key = other;
    }
    if (threadIdx.x == 0 && best_key) atomicMax(a.argmax_key, best_key);
  }
}

constexpr int SMEM_LIMIT = 227 * 1024;

template <int EPI, int W>
size_t gemv1_smem(int stages, int stride, int kp) {
  constexpr int NP = EPI == 2 ? 2 : 1;
  return (size_t)W * stages * stride + (size_t)W * stages * 8 + (size_t)kp * 4 + (size_t)kp / 16 * 4 +
         (size_t)kp / 16 * 4 + (size_t)NP * W * 16 * 4 + (size_t)2 * W * 4 + 16 + 8 + 64;
}

template <int TYPE, int EPI, int W, int MINB>
int launch_w(fb200_device* dev, Gemv1Args& a) {
  auto kern = qgemv1_kernel<TYPE, EPI, W, MINB>;
  static bool configured[64] = {false};
  if (!configured[dev->ordinal & 63]) {
    FB_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
    configured[dev->ordinal & 63] = true;
  }
  int grid = dev->sm_count * MINB;
  if (grid > a.nunits) grid = a.nunits;
  // same number of units for every CTA where the unit count allows it
  const int rounds = (a.nunits + grid - 1) / grid;
  grid = (a.nunits + rounds - 1) / rounds;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(W * 32);
  cfg.dynamicSmemBytes = gemv1_smem<EPI, W>(a.stages, a.stride, a.Kp);
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dev->pdl ? 1 : 0;
  FB_CUDA(dev, cudaLaunchKernelEx(&cfg, kern, a));
  dev->launches++;
  return FB200_OK;
}

// Shared memory per SM is split between the activation limbs (4 B per element of K, one copy
// per CTA, built by every CTA in its prologue) and the weight rings. More, smaller CTAs give
// deeper rings per warp and more independent tiles in flight; larger K forces fewer CTAs.
template <int TYPE, int EPI>
int launch_cfg(fb200_device* dev, Gemv1Args& a) {
  const int per_sm = SMEM_LIMIT - 2048;
  auto fits = [&](size_t need, int ctas) { return (need + 1024) * ctas <= (size_t)per_sm; };
  for (int s = 3; s >= 2; --s)
    if (fits(gemv1_smem<EPI, 8>(s, a.stride, a.Kp), 4)) { a.stages = s; return launch_w<TYPE, EPI, 8, 4>(dev, a); }
  for (int s = 3; s >= 2; --s)
    if (fits(gemv1_smem<EPI, 8>(s, a.stride, a.Kp), 3)) { a.stages = s; return launch_w<TYPE, EPI, 8, 3>(dev, a); }
  for (int s = 3; s >= 2; --s)
    if (fits(gemv1_smem<EPI, 16>(s, a.stride, a.Kp), 2)) { a.stages = s; return launch_w<TYPE, EPI, 16, 2>(dev, a); }
  for (int s = 2; s >= 1; --s)
    if (fits(gemv1_smem<EPI, 32>(s, a.stride, a.Kp), 1)) { a.stages = s; return launch_w<TYPE, EPI, 32, 1>(dev, a); }
  return fb200_fail(dev, FB200_ERR_CAPACITY, "qgemv1: K = %d does not fit in shared memory", a.K);
}

template <int TYPE>
int launch_typed(fb200_device* dev, Gemv1Args& a, int epi) {
  if (epi == FB200_EPI_SWIGLU) return launch_cfg<TYPE, 2>(dev, a);
  if (epi == FB200_EPI_RESIDUAL) return launch_cfg<TYPE, 1>(dev, a);
  return launch_cfg<TYPE, 0>(dev, a);
}

}  // namespace

// Largest K the single-row kernel takes (activation limbs live in shared memory).
bool fb200_qgemv1_fits(const fb200_qmatrix* w) {
  TileGeom geo;
  if (!tile_geom(w->type, &geo)) return false;
  const uint64_t kp = (uint64_t)w->ngroups * geo.group_elems;
  return kp * 4 + kp / 4 + 16 * 3456 + 8192 <= (uint64_t)SMEM_LIMIT - 2048;
}

// ys[i][n_i] = epilogue(W_i . act(x)) for up to three matrices that share K and the group size;
// act = optional residual add + RMSNorm (norm_w != null). Epilogues apply to one matrix only.
int fb200_qgemv1_multi(fb200_device* dev, const fb200_qmatrix* const* ws, float* const* ys, int nw,
                       const float* x, const float* xres, const float* norm_w, float eps, int epi,
                       const float* r1, const float* r2, const fb200_gemv1_extra* extra) {
  if (nw < 1 || nw > 3 || (epi != FB200_EPI_NONE && nw != 1))
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "qgemv1: %d matrices with epilogue %d", nw, epi);
  Gemv1Args a = {};
  TileGeom geo0;
  tile_geom(ws[0]->type, &geo0);
  a.nseg = nw;
  a.stride = 0;
  a.nunits = 0;
  for (int i = 0; i < nw; ++i) {
    TileGeom geo;
    if (!tile_geom(ws[i]->type, &geo) || geo.group_elems != geo0.group_elems || ws[i]->k != ws[0]->k)
      return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "qgemv1: matrices of one launch must share K and the group size");
    a.seg[i].w = ws[i]->data; a.seg[i].y = ys[i]; a.seg[i].type = (int)ws[i]->type; a.seg[i].tg = geo.tg_bytes;
    a.seg[i].units = ws[i]->ntiles; a.seg[i].n_out = (int)ws[i]->n;
    a.nunits += ws[i]->ntiles;
    const int st = (geo.tg_bytes + 127) / 128 * 128;
    if (st > a.stride) a.stride = st;
  }
  a.x = x; a.xres = xres; a.norm_w = norm_w; a.eps = eps;
  a.K = (int)ws[0]->k; a.Kp = ws[0]->ngroups * geo0.group_elems;
  a.r1 = r1; a.r2 = r2;
  a.ngroups = ws[0]->ngroups; a.pair_tile_offset = 0;
  a.stages = 2; a.status = dev->status;
  if (extra) {
    a.argmax_key = extra->argmax_key;
    if (extra->x_packed) { a.xp = *extra->x_packed; a.xp_norm = extra->x_packed_norm ? 1 : 0; }
    if (extra->y_packed) { a.yp = *extra->y_packed; a.yp_norm_w = extra->y_packed_norm_w; a.yp_add = extra->y_packed_add; }
  }
  if (epi == FB200_EPI_SWIGLU) {
    a.seg[0].units = ws[0]->ntiles / 2;
    a.nunits = a.seg[0].units;
    a.seg[0].n_out = (int)(ws[0]->n / 2);
    a.pair_tile_offset = ws[0]->ntiles / 2;
  }
  if (nw > 1) return launch_cfg<0, 0>(dev, a);
  switch (ws[0]->type) {
    case FB200_Q4_K: return launch_typed<FB200_Q4_K>(dev, a, epi);
    case FB200_Q6_K: return launch_typed<FB200_Q6_K>(dev, a, epi);
    case FB200_Q8_0: return launch_typed<FB200_Q8_0>(dev, a, epi);
    default: return launch_typed<FB200_Q4_0>(dev, a, epi);
  }
}

int fb200_qgemv1(fb200_device* dev, const fb200_qmatrix* w, const float* x, const float* xres,
                 const float* norm_w, float eps, float* y, int epi, const float* r1,
                 const float* r2) {
  return fb200_qgemv1_multi(dev, &w, &y, 1, x, xres, norm_w, eps, epi, r1, r2, nullptr);
}
