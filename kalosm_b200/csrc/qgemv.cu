// Quantised matrix x small-batch activation product (decode GEMV and M <= 32 "skinny" GEMM).
//
// Bound: HBM. Persistent CTAs (a multiple of the SM count) walk the 16-row tiles of W; inside a
// CTA the 8 warps take the K groups of a tile round robin. Every warp owns a private ring of
// shared-memory stages that it fills with 1-D TMA bulk copies (cp.async.bulk + mbarrier
// complete_tx), one tile-group (1.1 - 3.4 KB, contiguous in the tiled storage) per stage, several
// stages ahead of the math, so tens of KB per SM are in flight without holding registers. The
// first copies are issued before griddepcontrol.wait: under programmatic dependent launch the
// weights of this product stream in while the producer of the activations is still running.
// Each lane reads the quant bytes of its MMA A fragments from the stage with 4-byte shared
// loads (conflict free in the tile-interleaved storage) and keeps them in the byte domain: one
// logic op turns four packed nibbles into four u8 operands of mma.sync.m16n8k32
// (u8 x s8 -> s32, exact). Activations are packed once per call into signed 7-bit limbs
// (x/scale = (l0 + l1/2^7 [+ l2/2^14 [+ l3/2^21]]) / 64: four limbs, 2^-27, for up to 8 rows;
// three, 2^-20, for 9..16 rows; two, 2^-13, for 17..32 rows), pre-scaled per row by a power of two. Integer dot products
// are exact; block scales are applied to them in fp32 per 16- or 32-element group.
// The batch occupies the N = 8 columns of the MMA, which makes M <= 8 cost the same weight
// traffic and nearly the same instruction count as M = 1.
//
// Replaces the reference's qgemv kernels (fusor-ml/tile-ir-kernels/src/kernels/qgemv.rs:356-678,
// qgemv_q6k.rs:84-385) and their SwiGLU / residual epilogues
// (fusor-ml/core/src/quantized/matmul/mod.rs:435-439, 666-722).
#include <atomic>
#include <cstdlib>

#include "qgemv_common.cuh"

namespace {

constexpr int GEMV_WARPS = 8;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;

struct GemvArgs {
  const uint8_t* w;     // tiled weights
  const uint8_t* xq;    // packed activation limbs [Kp/32][NL][Mp][32]
  const float* xs16;    // [Kp/16][Mp] sums of the scaled activations (centres and offsets)
  const float* xscale;  // [Mp] power-of-two output scales
  float* y;             // [M, Nout]
  const float* r1;      // residual rows [M, Nout], or one bias row [Nout] when r1_stride is 0
  const float* r2;
  int r1_stride;        // elements between consecutive rows of r1
  int M, Mp;
  int n_out;    // logical output columns (N, or N/2 for SwiGLU)
  int ngroups;  // K groups per tile
  int pair_tile_offset;  // SwiGLU: tile index distance between the gate and the up tile
  int nunits;            // work units: tiles, or (gate, up) tile pairs
  int* status;           // device status word (bounded waits that ran out are recorded here)
  // several matrices that share the activation rows in one launch (qgemm16s_multi_kernel): the
  // units of matrix 0 come first, then those of matrix 1, ...
  int nseg;
  struct Seg {
    const uint8_t* w;
    float* y;
    int n_out, units, type;
  } seg[3];
};

__device__ __forceinline__ uint32_t lds4(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ uint4 lds16(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }

// What a lane needs from the packed activations for one 32-element chunk kc: limb bytes
// {elements 4t..4t+3, elements 16+4t..16+4t+3} of batch row 8 nt + g (one uint2 per limb) and the
// sums of the two 16-element halves for batch columns 8 nt + 2t, 2t + 1. They come from L2; the
// group functions below request chunk k + 1 before they compute chunk k, and the first chunk of
// the next tile-group before the last chunk of this one, so the latency is covered by the math.
template <int NT, int NL>
struct ChunkIn {
  uint2 b[NT][NL];
  float2 sa[NT], sb[NT];
};

template <int NT, int NL, bool SUMS>
__device__ __forceinline__ void load_chunk(const GemvArgs& a, int kc, int g, int t, ChunkIn<NT, NL>& c) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int m = 8 * nt + g;
#pragma unroll
    for (int l = 0; l < NL; ++l) {
      c.b[nt][l] = make_uint2(0u, 0u);
      if (m < a.M)
        c.b[nt][l] = __ldg(reinterpret_cast<const uint2*>(a.xq + (((size_t)kc * NL + l) * a.Mp + m) * 32 + t * 8));
    }
    c.sa[nt] = make_float2(0.f, 0.f);
    c.sb[nt] = make_float2(0.f, 0.f);
    if (SUMS) {
      c.sa[nt] = __ldg(reinterpret_cast<const float2*>(a.xs16 + (size_t)(2 * kc) * a.Mp + 8 * nt + 2 * t));
      c.sb[nt] = __ldg(reinterpret_cast<const float2*>(a.xs16 + (size_t)(2 * kc + 1) * a.Mp + 8 * nt + 2 * t));
    }
  }
}

template <int NT, int NL>
__device__ __forceinline__ void zero_c(int (&c)[NT][NL][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int l = 0; l < NL; ++l)
#pragma unroll
      for (int i = 0; i < 4; ++i) c[nt][l][i] = 0;
}

template <bool SIGNED_A, int NT, int NL>
__device__ __forceinline__ void mma_all(int (&c)[NT][NL][4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, const uint2 (&b)[NT][NL]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int l = 0; l < NL; ++l) mma_i8_k32<SIGNED_A>(c[nt][l], a0, a1, a2, a3, b[nt][l].x, b[nt][l].y);
}

// Integer dot products -> fp32 in units of 2^-13 * (w . x/scale).
template <int NL>
__device__ __forceinline__ float limbs_f(const int (&c)[NL][4], int i) {
  float f = (float)(c[0][i] * 128 + c[1][i]);
  if (NL == 4) f = fmaf((float)(c[2][i] * 128 + c[3][i]), 1.0f / 16384.0f, f);
  if (NL == 3) f = fmaf((float)c[2][i], 1.0f / 128.0f, f);
  return f;
}

// acc += s * (f - centre * xs) - o * xs for the four accumulator slots of every n-tile;
// xs = sum of the scaled activations over the scale group, per batch column (BOTH: both halves
// of the chunk, else sx as given).
template <int NT, int NL>
__device__ __forceinline__ void apply(float (&acc)[NT][4], const int (&c)[NT][NL][4], float s_g,
                                      float s_g8, float o_g, float o_g8, float centre,
                                      const float2 (&sx)[NT]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    acc[nt][0] = fmaf(s_g, limbs_f<NL>(c[nt], 0) - centre * sx[nt].x, fmaf(-o_g, sx[nt].x, acc[nt][0]));
    acc[nt][1] = fmaf(s_g, limbs_f<NL>(c[nt], 1) - centre * sx[nt].y, fmaf(-o_g, sx[nt].y, acc[nt][1]));
    acc[nt][2] = fmaf(s_g8, limbs_f<NL>(c[nt], 2) - centre * sx[nt].x, fmaf(-o_g8, sx[nt].x, acc[nt][2]));
    acc[nt][3] = fmaf(s_g8, limbs_f<NL>(c[nt], 3) - centre * sx[nt].y, fmaf(-o_g8, sx[nt].y, acc[nt][3]));
  }
}

template <int NT, int NL>
__device__ __forceinline__ void both_halves(const ChunkIn<NT, NL>& c, float2 (&sx)[NT]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) sx[nt] = make_float2(c.sa[nt].x + c.sb[nt].x, c.sa[nt].y + c.sb[nt].y);
}

// ---- per-format processing of one tile-group by one warp --------------------------------------
// Standard MMA mapping: one m16n8k32 covers the 32 elements of one scale group (two 16-element
// groups for Q6_K, done as m16n8k16), the 8 columns are batch rows.

// `cur` holds the inputs of the group's first chunk on entry and, on exit, those of chunk
// `next_first` (the first chunk of the warp's next tile-group; -1: none).
template <int NT, int NL>
__device__ __forceinline__ void group_q4_0(const GemvArgs& a, const uint8_t* tg, int kg, int lane,
                                           float (&acc)[NT][4], ChunkIn<NT, NL>& cur, int next_first) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int blk = 0; blk < 4; ++blk) {
    const int kc = kg * 4 + blk;
    ChunkIn<NT, NL> nxt = cur;
    const int kn = blk < 3 ? kc + 1 : next_first;
    if (kn >= 0) load_chunk<NT, NL, true>(a, kn, g, t, nxt);
    const uint32_t w0 = lds4(tg + g * 64 + blk * 16 + 4 * t);
    const uint32_t w1 = lds4(tg + 512 + g * 64 + blk * 16 + 4 * t);
    int c[NT][NL][4];
    zero_c<NT, NL>(c);
    mma_all<false, NT, NL>(c, w0 & 0x0F0F0F0Fu, w1 & 0x0F0F0F0Fu, (w0 >> 4) & 0x0F0F0F0Fu,
                           (w1 >> 4) & 0x0F0F0F0Fu, cur.b);
    const float d_g = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 1024 + (g * 4 + blk) * 2));
    const float d_g8 = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 1024 + ((g + 8) * 4 + blk) * 2));
    float2 sx[NT];
    both_halves<NT, NL>(cur, sx);
    apply<NT, NL>(acc, c, d_g, d_g8, 0.f, 0.f, 8.0f, sx);
    cur = nxt;
  }
}

template <int NT, int NL>
__device__ __forceinline__ void group_q8_0(const GemvArgs& a, const uint8_t* tg, int kg, int lane,
                                           float (&acc)[NT][4], ChunkIn<NT, NL>& cur, int next_first) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int blk = 0; blk < 4; ++blk) {
    const int kc = kg * 4 + blk;
    ChunkIn<NT, NL> nxt = cur;
    const int kn = blk < 3 ? kc + 1 : next_first;
    if (kn >= 0) load_chunk<NT, NL, false>(a, kn, g, t, nxt);
    const int off = g * 64 + blk * 16 + 4 * t;
    const uint32_t a0 = lds4(tg + off), a2 = lds4(tg + 512 + off);
    const uint32_t a1 = lds4(tg + 1024 + off), a3 = lds4(tg + 1536 + off);
    int c[NT][NL][4];
    zero_c<NT, NL>(c);
    mma_all<true, NT, NL>(c, a0, a1, a2, a3, cur.b);
    const float d_g = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 2048 + (g * 4 + blk) * 2));
    const float d_g8 = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 2048 + ((g + 8) * 4 + blk) * 2));
    float2 sx[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) sx[nt] = make_float2(0.f, 0.f);
    apply<NT, NL>(acc, c, d_g, d_g8, 0.f, 0.f, 0.f, sx);
    cur = nxt;
  }
}

// Q4_K: lane t of each quad decodes the 6-bit (scale, offset) of sub-blocks t and t + 4 for its
// two rows; the quad shares them by shuffle.
template <int NT, int NL>
__device__ __forceinline__ void group_q4k(const GemvArgs& a, const uint8_t* tg, int kg, int lane,
                                          float (&acc)[NT][4], ChunkIn<NT, NL>& cur, int next_first) {
  const int g = lane >> 2, t = lane & 3;
  float sc_f[2][2], mn_f[2][2];  // [row half][sub-block t + 4 i]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint4 hd = lds16(tg + 2048 + (g + 8 * h) * 16);
    const float d = fb::half_bits_to_float((uint16_t)(hd.x & 0xFFFF));
    const float dmin = fb::half_bits_to_float((uint16_t)(hd.x >> 16));
    const uint32_t s0 = hd.y, s1 = hd.z, s2 = hd.w;
    const uint32_t scB = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
    const uint32_t mnB = ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u);
    const int sh = 8 * t;
    sc_f[h][0] = d * (float)((s0 >> sh) & 0x3F);
    mn_f[h][0] = dmin * (float)((s1 >> sh) & 0x3F);
    sc_f[h][1] = d * (float)((scB >> sh) & 0xFF);
    mn_f[h][1] = dmin * (float)((mnB >> sh) & 0xFF);
  }
#pragma unroll
  for (int pair = 0; pair < 4; ++pair) {
    const int ch = pair >> 1, ps = pair & 1;
    const int off = g * 32 + ps * 16 + 4 * t;
    const uint32_t w00 = lds4(tg + ((ch * 2 + 0) * 2 + 0) * 256 + off);  // row g,   elements 4t..
    const uint32_t w01 = lds4(tg + ((ch * 2 + 0) * 2 + 1) * 256 + off);  // row g,   elements 16+4t..
    const uint32_t w10 = lds4(tg + ((ch * 2 + 1) * 2 + 0) * 256 + off);  // row g+8
    const uint32_t w11 = lds4(tg + ((ch * 2 + 1) * 2 + 1) * 256 + off);
#pragma unroll
    for (int hi = 0; hi < 2; ++hi) {
      const int sb = 2 * pair + hi;
      const uint32_t mask = hi ? 0xF0F0F0F0u : 0x0F0F0F0Fu;
      const int kc = kg * 8 + sb;
      ChunkIn<NT, NL> nxt = cur;
      const int kn = sb < 7 ? kc + 1 : next_first;
      if (kn >= 0) load_chunk<NT, NL, true>(a, kn, g, t, nxt);
      int c[NT][NL][4];
      zero_c<NT, NL>(c);
      mma_all<false, NT, NL>(c, w00 & mask, w10 & mask, w01 & mask, w11 & mask, cur.b);
      const int src = (lane & ~3) | (sb & 3);
      float s_g = __shfl_sync(0xFFFFFFFFu, sc_f[0][sb >> 2], src);
      float s_g8 = __shfl_sync(0xFFFFFFFFu, sc_f[1][sb >> 2], src);
      const float o_g = __shfl_sync(0xFFFFFFFFu, mn_f[0][sb >> 2], src);
      const float o_g8 = __shfl_sync(0xFFFFFFFFu, mn_f[1][sb >> 2], src);
      if (hi) { s_g *= 0.0625f; s_g8 *= 0.0625f; }  // high nibbles were used in place as 16 q
      float2 sx[NT];
      both_halves<NT, NL>(cur, sx);
      apply<NT, NL>(acc, c, s_g, s_g8, o_g, o_g8, 0.f, sx);
      cur = nxt;
    }
  }
}

// Q6_K: sixteen 16-element scale groups per super-block, one m16n8k16 per group and limb.
template <int NT, int NL>
__device__ __forceinline__ void group_q6k(const GemvArgs& a, const uint8_t* tg, int kg, int lane,
                                          float (&acc)[NT][4], ChunkIn<NT, NL>& cur, int next_first) {
  const int g = lane >> 2, t = lane & 3;
  const uint4 sc_g = lds16(tg + 3072 + g * 16);
  const uint4 sc_g8 = lds16(tg + 3072 + (g + 8) * 16);
  const float d_g = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 3328 + g * 2));
  const float d_g8 = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 3328 + (g + 8) * 2));
  const uint32_t scw_g[4] = {sc_g.x, sc_g.y, sc_g.z, sc_g.w};
  const uint32_t scw_g8[4] = {sc_g8.x, sc_g8.y, sc_g8.z, sc_g8.w};
#pragma unroll
  for (int c2 = 0; c2 < 2; ++c2)
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      // groups 8c + 2q + u, u = 0, 1, are the two halves of 32-element chunk 4c + q
      const int kc = kg * 8 + c2 * 4 + q;
      ChunkIn<NT, NL> nxt = cur;
      const int kn = (c2 * 4 + q) < 7 ? kc + 1 : next_first;
      if (kn >= 0) load_chunk<NT, NL, true>(a, kn, g, t, nxt);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int cu = c2 * 2 + u, grp = 8 * c2 + 2 * q + u;
        uint32_t af[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t wl = lds4(tg + (cu * 2 + h) * 256 + g * 32 + (q & 1) * 16 + 4 * t);
          const uint32_t wh = lds4(tg + 2048 + (cu * 2 + h) * 128 + g * 16 + 4 * t);
          const uint32_t hb = q == 0 ? (wh << 4) : q == 1 ? (wh << 2) : q == 2 ? wh : (wh >> 2);
          af[h] = (((q >> 1) ? (wl >> 4) : wl) & 0x0F0F0F0Fu) | (hb & 0x30303030u);
        }
        int c[NT][NL][4];
        zero_c<NT, NL>(c);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int l = 0; l < NL; ++l) mma_u8_k16(c[nt][l], af[0], af[1], u ? cur.b[nt][l].y : cur.b[nt][l].x);
        const float s_g = d_g * (float)(int)(int8_t)((scw_g[grp >> 2] >> (8 * (grp & 3))) & 0xFF);
        const float s_g8 = d_g8 * (float)(int)(int8_t)((scw_g8[grp >> 2] >> (8 * (grp & 3))) & 0xFF);
        float2 sx[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) sx[nt] = u ? cur.sb[nt] : cur.sa[nt];
        apply<NT, NL>(acc, c, s_g, s_g8, 0.f, 0.f, 32.0f, sx);
      }
      cur = nxt;
    }
}

template <int TYPE>
struct Ring {
  static constexpr int TG = TYPE == FB200_Q4_0 ? 1152 : TYPE == FB200_Q8_0 ? 2176 : TYPE == FB200_Q4_K ? 2304 : 3360;
  static constexpr int STRIDE = (TG + 127) / 128 * 128;  // stage stride, keeps 128-byte alignment
  static constexpr int STAGES = TYPE == FB200_Q4_0 ? 8 : TYPE == FB200_Q6_K ? 3 : 4;
  static constexpr int RING_BYTES = GEMV_WARPS * STAGES * STRIDE;
  static constexpr int BAR_BYTES = GEMV_WARPS * STAGES * 8;
};

template <int NT>
struct Limbs { static constexpr int N = NT == 1 ? 4 : NT == 2 ? 3 : 2; };

template <int TYPE, int NT, int EPI>
constexpr int gemv_smem_bytes() {
  return Ring<TYPE>::RING_BYTES + Ring<TYPE>::BAR_BYTES +
         (EPI == 2 ? 2 : 1) * GEMV_WARPS * NT * 8 * 16 * (int)sizeof(float);
}

// EPI: 0 none, 1 residual(s), 2 SwiGLU pair
template <int TYPE, int NT, int EPI>
__global__ void __launch_bounds__(GEMV_THREADS)
qgemv_kernel(const GemvArgs a) {
  using R = Ring<TYPE>;
  constexpr int NP = EPI == 2 ? 2 : 1;
  constexpr int S = R::STAGES;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + R::RING_BYTES);
  float (*red)[GEMV_WARPS][NT * 8][16] =
      reinterpret_cast<float (*)[GEMV_WARPS][NT * 8][16]>(smem + R::RING_BYTES + R::BAR_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* my_ring = ring + warp * S * R::STRIDE;
  const uint32_t my_bar = smem_u32(bars + warp * S);

  pdl_launch_dependents();
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < S; ++s) mbar_init(my_bar + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // this warp's items: for each of the CTA's units, for each pass (gate / up), its K groups
  const int gw = a.ngroups > warp ? (a.ngroups - warp + GEMV_WARPS - 1) / GEMV_WARPS : 0;
  const int my_units = a.nunits > (int)blockIdx.x ? (a.nunits - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int per_unit = NP * gw;
  const int n_items = my_units * per_unit;
  auto issue = [&](int i) {
    const int j = i / per_unit, rem = i - j * per_unit;
    const int p = rem / gw, kk = rem - p * gw;
    const int tile = (int)blockIdx.x + j * (int)gridDim.x + p * a.pair_tile_offset;
    const int kg = warp + GEMV_WARPS * kk;
    const int st = i % S;
    const uint8_t* src = a.w + ((size_t)tile * a.ngroups + kg) * R::TG;
    mbar_expect_tx(my_bar + 8 * st, R::TG);
    bulk_g2s(smem_u32(my_ring + st * R::STRIDE), src, R::TG, my_bar + 8 * st);
  };
  if (lane == 0) {
    const int pre = n_items < S ? n_items : S;
    for (int i = 0; i < pre; ++i) issue(i);
  }
  // everything above touches only the weights; the activations come from the previous kernel
  pdl_wait();

  constexpr int NL = Limbs<NT>::N;
  constexpr int CHUNKS = (TYPE == FB200_Q4_0 || TYPE == FB200_Q8_0) ? 4 : 8;  // 32-element chunks per K group
  constexpr bool SUMS = TYPE != FB200_Q8_0;
  ChunkIn<NT, NL> cur;  // inputs of the first chunk of the warp's next tile-group
  if (n_items > 0) load_chunk<NT, NL, SUMS>(a, warp * CHUNKS, g, t, cur);
  int item = 0;
  for (int j = 0; j < my_units; ++j) {
    const int unit = (int)blockIdx.x + j * (int)gridDim.x;
    if (j > 0) __syncthreads();  // the previous unit's reduction has read `red`
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      float acc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
      for (int kk = 0; kk < gw; ++kk, ++item) {
        const int st = item % S;
        mbar_wait(my_bar + 8 * st, (uint32_t)((item / S) & 1), a.status);
        const uint8_t* tg = my_ring + st * R::STRIDE;
        const int kg = warp + GEMV_WARPS * kk;
        // first chunk of the warp's next tile-group: the next K group of this pass, or K group
        // `warp` again when another pass or unit follows
        const int next_first = kk + 1 < gw ? (kg + GEMV_WARPS) * CHUNKS : (item + 1 < n_items ? warp * CHUNKS : -1);
        if (TYPE == FB200_Q4_0) group_q4_0<NT, NL>(a, tg, kg, lane, acc, cur, next_first);
        else if (TYPE == FB200_Q8_0) group_q8_0<NT, NL>(a, tg, kg, lane, acc, cur, next_first);
        else if (TYPE == FB200_Q4_K) group_q4k<NT, NL>(a, tg, kg, lane, acc, cur, next_first);
        else group_q6k<NT, NL>(a, tg, kg, lane, acc, cur, next_first);
        __syncwarp();  // every lane has consumed the stage before it is refilled
        if (lane == 0 && item + S < n_items) issue(item + S);
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        red[p][warp][8 * nt + 2 * t][g] = acc[nt][0];
        red[p][warp][8 * nt + 2 * t + 1][g] = acc[nt][1];
        red[p][warp][8 * nt + 2 * t][g + 8] = acc[nt][2];
        red[p][warp][8 * nt + 2 * t + 1][g + 8] = acc[nt][3];
      }
    }
    __syncthreads();
    for (int o = threadIdx.x; o < NT * 8 * 16; o += GEMV_THREADS) {
      const int m = o >> 4, r = o & 15;
      const int n = unit * 16 + r;
      if (m >= a.M || n >= a.n_out) continue;
      float v[NP];
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_WARPS; ++w) s += red[p][w][m][r];
        v[p] = s * a.xscale[m];
      }
      const size_t idx = (size_t)m * a.n_out + n;
      float out;
      if (EPI == 2) {
        // silu(gate) * up, fusor-ml/fusor/src/composite/activations.rs:47-64: x / (1 + exp(-x))
        float gate = v[0];
        out = (gate / (1.0f + expf(-gate))) * v[NP - 1];
      } else if (EPI == 1) {
        out = v[0] + a.r1[(size_t)m * a.r1_stride + n];
        if (a.r2) out += a.r2[idx];
      } else {
        out = v[0];
      }
      a.y[idx] = out;
    }
  }
}

// x[M, K] f32 -> int8 limb planes [Kp/32][NL][Mp][32] (inside a 32-element chunk lane t's eight
// bytes are elements 4t..4t+3 then 16+4t..16+4t+3), per-16 sums of the scaled values and the
// power-of-two output scale of each row. One CTA per (padded) row.
template <int NL>
__global__ void __launch_bounds__(256)
pack_x_kernel(const float* __restrict__ x, int M, int K, int Kp, int Mp, uint8_t* __restrict__ xq,
              float* __restrict__ xs16, float* __restrict__ xscale) {
  const int m = blockIdx.x;
  __shared__ float wmax[8];
  pdl_launch_dependents();
  pdl_wait();
  float inv64 = 0.f;
  if (m < M) {
    float amax = 0.f;
    for (int k = threadIdx.x; k < K; k += 256) amax = fmaxf(amax, fabsf(x[(size_t)m * K + k]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = wmax[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, wmax[i]);
    int e = 0;
    if (amax > 0.f && amax < 3.0e38f) frexpf(amax, &e);
    inv64 = ldexpf(64.0f, -e);
    if (threadIdx.x == 0) xscale[m] = ldexpf(1.0f, e - 13);
  } else if (threadIdx.x == 0) {
    xscale[m] = 1.0f;
  }
  const int quads = Kp >> 2;  // a multiple of 32
  for (int q0 = 0; q0 < quads; q0 += 256) {
    const int q = q0 + threadIdx.x;
    const int k = q * 4;
    uint32_t lw[4] = {0u, 0u, 0u, 0u};
    float sum = 0.f;
    if (q < quads && m < M) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = (k + i < K) ? x[(size_t)m * K + k + i] * inv64 : 0.f;
        sum += v;
        float l0 = rintf(v), r = (v - l0) * 128.0f;
        float l1 = rintf(r); r = (r - l1) * 128.0f;
        float l2 = rintf(r); r = (r - l2) * 128.0f;
        float l3 = rintf(r);
        lw[0] |= ((uint32_t)(int)l0 & 0xFFu) << (8 * i);
        lw[1] |= ((uint32_t)(int)l1 & 0xFFu) << (8 * i);
        lw[2] |= ((uint32_t)(int)l2 & 0xFFu) << (8 * i);
        lw[3] |= ((uint32_t)(int)l3 & 0xFFu) << (8 * i);
      }
    }
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    if (q < quads) {
      const int kc = k >> 5, e = k & 31;  // e is a multiple of 4
      const int pos = e < 16 ? (e >> 2) * 8 : ((e - 16) >> 2) * 8 + 4;
#pragma unroll
      for (int l = 0; l < NL; ++l)
        *reinterpret_cast<uint32_t*>(xq + (((size_t)kc * NL + l) * Mp + m) * 32 + pos) = lw[l];
      if ((threadIdx.x & 3) == 0) xs16[(size_t)(k >> 4) * Mp + m] = sum * 128.0f;
    }
  }
}

// ================================================================================================
// 2 .. 32 activation rows: weights dequantised to fp16 in registers, fp16 tensor-core MMAs.
//
// With several rows the limb scheme pays per 32-element chunk for every (row, batch column) pair:
// integer sums to float, scale, offset. Here a chunk of weights is turned into fp16 once per lane
// (byte -> 1024 + byte by a byte permute, exact subtraction, one fused multiply-add with the
// block scale and offset) and fed to mma.m16n8k16.f16 with fp32 accumulation over the whole K:
// the work per tile-group no longer depends on the scale structure and grows by two MMAs per
// 8 more batch rows. Precision: weights and activations carry 11 bits (about 4e-4 relative L2 on
// the products, inside the 2e-3 contract); the limb kernels above serve a single row (in the
// single-row file) and, on request, 2 .. 8 rows.
//
// k-slots of an MMA and elements of a 32-element chunk: lane t holds elements 4t .. 4t+3 (first
// step) and 16+4t .. 16+4t+3 (second step) of its rows, the same bytes the int8 mapping reads;
// within a step, slots (2t, 2t+1) are elements (4t, 4t+1) and slots (2t+8, 2t+9) are (4t+2, 4t+3).
// The activation rows are packed accordingly: per chunk and row 64 bytes, lane t's eight halves
// at byte 16 t.

__device__ __forceinline__ void mma_f16_k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Four unsigned bytes -> two half2 (1024 + byte each), then (v - centre) * scale - offset.
// centre includes the 1024; scale and offset are per row.
// HIGH: the bytes hold a nibble in their upper half (byte = 16 n, taken from the packed word with a
// mask alone, no shift); under the exponent of 64 a byte counts sixteenths, so the half is 64 + n
// and the centre includes the 64.
template <bool HIGH = false>
__device__ __forceinline__ void deq4(uint32_t w, __half2 centre, __half2 scale, __half2 offset, uint32_t& h01,
                                     uint32_t& h23) {
  constexpr uint32_t MAGIC = HIGH ? 0x54545454u : 0x64646464u;
  const __half2 v01 = __hsub2(bits_h2(__byte_perm(w, MAGIC, 0x4140)), centre);
  const __half2 v23 = __hsub2(bits_h2(__byte_perm(w, MAGIC, 0x4342)), centre);
  h01 = h2_bits(__hfma2(v01, scale, offset));
  h23 = h2_bits(__hfma2(v23, scale, offset));
}

// ---- block scales in half precision ------------------------------------------------------------
// The fp16 kernels multiply every weight by its block scale in half precision. The scales are small
// integers times an fp16 block factor, so they are built with half arithmetic alone (integer n as
// the half 1024 + n minus 1024, then one rounded product: the same bits as the fp32 product
// rounded to half) instead of int -> float -> half conversions, which share one slow pipe.

// Q4_K header of rows g (h = 0) and g + 8 (h = 1): sm[h][j] = half2 {d * scale, -dmin * min} of
// sub-block t + 4 j (get_scale_min_k4 of the GGUF block).
__device__ __forceinline__ void q4k_scales_h2(const uint8_t* tg, int g, int t, uint32_t (&sm)[2][2]) {
  const __half2 c1024 = __float2half2_rn(1024.0f);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint4 hd = lds16(tg + 2048 + (g + 8 * h) * 16);
    const __half2 dd = bits_h2(hd.x ^ 0x80000000u);  // {d, -dmin}
    const uint32_t s0 = hd.y, s1 = hd.z, s2 = hd.w;
    const uint32_t scB = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
    const uint32_t mnB = ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u);
    const int sh = 8 * t;
    const uint32_t p0 = ((s0 >> sh) & 0x3Fu) | (((s1 >> sh) & 0x3Fu) << 16);
    const uint32_t p1 = ((scB >> sh) & 0xFFu) | (((mnB >> sh) & 0xFFu) << 16);
    sm[h][0] = h2_bits(__hmul2(__hsub2(bits_h2(p0 | 0x64006400u), c1024), dd));
    sm[h][1] = h2_bits(__hmul2(__hsub2(bits_h2(p1 | 0x64006400u), c1024), dd));
  }
}
// Scales and (negated) offsets of sub-block sb for this lane's rows, from the lane of the quad that
// decoded them.
__device__ __forceinline__ void q4k_chunk_scales(const uint32_t (&sm)[2][2], int lane, int sb, __half2& s_g, __half2& s_g8,
                                                 __half2& o_g, __half2& o_g8) {
  const int src = (lane & ~3) | (sb & 3);
  const uint32_t v0 = __shfl_sync(0xFFFFFFFFu, sm[0][sb >> 2], src);
  const uint32_t v1 = __shfl_sync(0xFFFFFFFFu, sm[1][sb >> 2], src);
  s_g = bits_h2(__byte_perm(v0, v0, 0x1010));
  o_g = bits_h2(__byte_perm(v0, v0, 0x3232));
  s_g8 = bits_h2(__byte_perm(v1, v1, 0x1010));
  o_g8 = bits_h2(__byte_perm(v1, v1, 0x3232));
}
// Q6_K: the int8 scales of the two 16-element groups of chunk (c2, q) of one row, times d, each
// duplicated into a half2. xw = the row's 16 scale bytes with the sign bit flipped (v + 128).
__device__ __forceinline__ void q6k_chunk_scales(const uint32_t (&xw)[4], __half2 d2, int c2, int q, __half2& s_u0,
                                                 __half2& s_u1) {
  const uint32_t w = xw[2 * c2 + (q >> 1)];
  const uint32_t pair = (q & 1) ? __byte_perm(w, 0x64646464u, 0x4342) : __byte_perm(w, 0x64646464u, 0x4140);
  const uint32_t sv = h2_bits(__hmul2(__hsub2(bits_h2(pair), __float2half2_rn(1152.0f)), d2));
  s_u0 = bits_h2(__byte_perm(sv, sv, 0x1010));
  s_u1 = bits_h2(__byte_perm(sv, sv, 0x3232));
}

template <int NT>
struct Chunk16 { uint4 b[NT]; };

template <int NT>
__device__ __forceinline__ void load_chunk16(const GemvArgs& a, int kc, int g, int t, Chunk16<NT>& c) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int m = 8 * nt + g;
    c.b[nt] = make_uint4(0u, 0u, 0u, 0u);
    if (m < a.M) c.b[nt] = __ldg(reinterpret_cast<const uint4*>(a.xq + ((size_t)kc * a.Mp + m) * 64 + t * 16));
  }
}

// One 32-element chunk: unsigned bytes of rows g / g+8, elements 4t.. (lo) and 16+4t.. (hi).
template <int NT, bool HIGH = false>
__device__ __forceinline__ void chunk16(float (&acc)[NT][4], const Chunk16<NT>& x, uint32_t lo_g, uint32_t lo_g8,
                                        uint32_t hi_g, uint32_t hi_g8, __half2 centre, __half2 s_lo_g,
                                        __half2 s_lo_g8, __half2 s_hi_g, __half2 s_hi_g8, __half2 o_g,
                                        __half2 o_g8) {
  uint32_t a0, a1, a2, a3;
  deq4<HIGH>(lo_g, centre, s_lo_g, o_g, a0, a2);
  deq4<HIGH>(lo_g8, centre, s_lo_g8, o_g8, a1, a3);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) mma_f16_k16(acc[nt], a0, a1, a2, a3, x.b[nt].x, x.b[nt].y);
  deq4<HIGH>(hi_g, centre, s_hi_g, o_g, a0, a2);
  deq4<HIGH>(hi_g8, centre, s_hi_g8, o_g8, a1, a3);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) mma_f16_k16(acc[nt], a0, a1, a2, a3, x.b[nt].z, x.b[nt].w);
}

// `cur` holds the activations of the group's first chunk on entry and, on exit, those of chunk
// `next_first` (the first chunk of the warp's next tile-group; -1: none).
template <int TYPE, int NT>
__device__ __forceinline__ void group16(const GemvArgs& a, const uint8_t* tg, int kg, int lane, float (&acc)[NT][4],
                                        Chunk16<NT>& cur, int next_first) {
  const int g = lane >> 2, t = lane & 3;
  const __half2 zero2 = __float2half2_rn(0.f);
  if constexpr (TYPE == FB200_Q4_0 || TYPE == FB200_Q8_0) {
#pragma unroll
    for (int blk = 0; blk < 4; ++blk) {
      const int kc = kg * 4 + blk;
      Chunk16<NT> nxt = cur;
      const int kn = blk < 3 ? kc + 1 : next_first;
      if (kn >= 0) load_chunk16<NT>(a, kn, g, t, nxt);
      const int dofs = TYPE == FB200_Q4_0 ? 1024 : 2048;
      const __half2 d_g = __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(tg + dofs + (g * 4 + blk) * 2)));
      const __half2 d_g8 = __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(tg + dofs + ((g + 8) * 4 + blk) * 2)));
      if constexpr (TYPE == FB200_Q4_0) {
        const uint32_t w0 = lds4(tg + g * 64 + blk * 16 + 4 * t);
        const uint32_t w1 = lds4(tg + 512 + g * 64 + blk * 16 + 4 * t);
        chunk16<NT>(acc, cur, w0 & 0x0F0F0F0Fu, w1 & 0x0F0F0F0Fu, (w0 >> 4) & 0x0F0F0F0Fu, (w1 >> 4) & 0x0F0F0F0Fu,
                    __float2half2_rn(1032.0f), d_g, d_g8, d_g, d_g8, zero2, zero2);  // (q - 8) d
      } else {
        const int off = g * 64 + blk * 16 + 4 * t;
        const uint32_t a0 = lds4(tg + off) ^ 0x80808080u, a2 = lds4(tg + 512 + off) ^ 0x80808080u;
        const uint32_t a1 = lds4(tg + 1024 + off) ^ 0x80808080u, a3 = lds4(tg + 1536 + off) ^ 0x80808080u;
        chunk16<NT>(acc, cur, a0, a1, a2, a3, __float2half2_rn(1152.0f), d_g, d_g8, d_g, d_g8, zero2, zero2);  // q d
      }
      cur = nxt;
    }
  } else if constexpr (TYPE == FB200_Q4_K) {
    // lane t of each quad decodes the 6-bit (scale, offset) of sub-blocks t and t + 4 for its two
    // rows; the quad shares them by shuffle
    uint32_t sm[2][2];
    q4k_scales_h2(tg, g, t, sm);
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) {
      const int ch = pair >> 1, ps = pair & 1;
      const int off = g * 32 + ps * 16 + 4 * t;
      const uint32_t w00 = lds4(tg + ((ch * 2 + 0) * 2 + 0) * 256 + off);  // row g,   elements 4t..
      const uint32_t w01 = lds4(tg + ((ch * 2 + 0) * 2 + 1) * 256 + off);  // row g,   elements 16+4t..
      const uint32_t w10 = lds4(tg + ((ch * 2 + 1) * 2 + 0) * 256 + off);  // row g+8
      const uint32_t w11 = lds4(tg + ((ch * 2 + 1) * 2 + 1) * 256 + off);
#pragma unroll
      for (int hi = 0; hi < 2; ++hi) {
        const int sb = 2 * pair + hi;
        const int kc = kg * 8 + sb;
        Chunk16<NT> nxt = cur;
        const int kn = sb < 7 ? kc + 1 : next_first;
        if (kn >= 0) load_chunk16<NT>(a, kn, g, t, nxt);
        __half2 hs_g, hs_g8, ho_g, ho_g8;
        q4k_chunk_scales(sm, lane, sb, hs_g, hs_g8, ho_g, ho_g8);
        if (hi == 0)
          chunk16<NT, false>(acc, cur, w00 & 0x0F0F0F0Fu, w10 & 0x0F0F0F0Fu, w01 & 0x0F0F0F0Fu, w11 & 0x0F0F0F0Fu,
                             __float2half2_rn(1024.0f), hs_g, hs_g8, hs_g, hs_g8, ho_g, ho_g8);
        else
          chunk16<NT, true>(acc, cur, w00 & 0xF0F0F0F0u, w10 & 0xF0F0F0F0u, w01 & 0xF0F0F0F0u, w11 & 0xF0F0F0F0u,
                            __float2half2_rn(64.0f), hs_g, hs_g8, hs_g, hs_g8, ho_g, ho_g8);
        cur = nxt;
      }
    }
  } else {  // Q6_K: the two 16-element halves of a chunk are two scale groups
    const uint4 sc_g = lds16(tg + 3072 + g * 16);
    const uint4 sc_g8 = lds16(tg + 3072 + (g + 8) * 16);
    const __half2 d_g = __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(tg + 3328 + g * 2)));
    const __half2 d_g8 = __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(tg + 3328 + (g + 8) * 2)));
    const uint32_t scw_g[4] = {sc_g.x ^ 0x80808080u, sc_g.y ^ 0x80808080u, sc_g.z ^ 0x80808080u, sc_g.w ^ 0x80808080u};
    const uint32_t scw_g8[4] = {sc_g8.x ^ 0x80808080u, sc_g8.y ^ 0x80808080u, sc_g8.z ^ 0x80808080u, sc_g8.w ^ 0x80808080u};
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int kc = kg * 8 + c2 * 4 + q;
        Chunk16<NT> nxt = cur;
        const int kn = (c2 * 4 + q) < 7 ? kc + 1 : next_first;
        if (kn >= 0) load_chunk16<NT>(a, kn, g, t, nxt);
        uint32_t af[2][2];  // [u][row half]
        __half2 hs[2][2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int cu = c2 * 2 + u;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t wl = lds4(tg + (cu * 2 + h) * 256 + g * 32 + (q & 1) * 16 + 4 * t);
            const uint32_t wh = lds4(tg + 2048 + (cu * 2 + h) * 128 + g * 16 + 4 * t);
            const uint32_t hb = q == 0 ? (wh << 4) : q == 1 ? (wh << 2) : q == 2 ? wh : (wh >> 2);
            af[u][h] = (((q >> 1) ? (wl >> 4) : wl) & 0x0F0F0F0Fu) | (hb & 0x30303030u);
          }
        }
        q6k_chunk_scales(scw_g, d_g, c2, q, hs[0][0], hs[1][0]);
        q6k_chunk_scales(scw_g8, d_g8, c2, q, hs[0][1], hs[1][1]);
        chunk16<NT>(acc, cur, af[0][0], af[0][1], af[1][0], af[1][1], __float2half2_rn(1056.0f), hs[0][0], hs[0][1],
                    hs[1][0], hs[1][1], zero2, zero2);  // (q - 32) d scale
        cur = nxt;
      }
  }
}

// Same persistent ring structure as qgemv_kernel; EPI: 0 none, 1 residual(s), 2 SwiGLU pair.
template <int TYPE, int NT, int EPI>
__global__ void __launch_bounds__(GEMV_THREADS)
qgemm16_kernel(const GemvArgs a) {
  using R = Ring<TYPE>;
  constexpr int NP = EPI == 2 ? 2 : 1;
  constexpr int S = R::STAGES;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + R::RING_BYTES);
  float (*red)[GEMV_WARPS][NT * 8][16] =
      reinterpret_cast<float (*)[GEMV_WARPS][NT * 8][16]>(smem + R::RING_BYTES + R::BAR_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* my_ring = ring + warp * S * R::STRIDE;
  const uint32_t my_bar = smem_u32(bars + warp * S);

  pdl_launch_dependents();
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < S; ++s) mbar_init(my_bar + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  const int gw = a.ngroups > warp ? (a.ngroups - warp + GEMV_WARPS - 1) / GEMV_WARPS : 0;
  const int my_units = a.nunits > (int)blockIdx.x ? (a.nunits - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int per_unit = NP * gw;
  const int n_items = my_units * per_unit;
  auto issue = [&](int i) {
    const int j = i / per_unit, rem = i - j * per_unit;
    const int p = rem / gw, kk = rem - p * gw;
    const int tile = (int)blockIdx.x + j * (int)gridDim.x + p * a.pair_tile_offset;
    const int kg = warp + GEMV_WARPS * kk;
    const int st = i % S;
    const uint8_t* src = a.w + ((size_t)tile * a.ngroups + kg) * R::TG;
    mbar_expect_tx(my_bar + 8 * st, R::TG);
    bulk_g2s(smem_u32(my_ring + st * R::STRIDE), src, R::TG, my_bar + 8 * st);
  };
  if (lane == 0) {
    const int pre = n_items < S ? n_items : S;
    for (int i = 0; i < pre; ++i) issue(i);
  }
  pdl_wait();  // the packed activations come from the kernel before this one

  constexpr int CHUNKS = (TYPE == FB200_Q4_0 || TYPE == FB200_Q8_0) ? 4 : 8;
  Chunk16<NT> cur;
  if (n_items > 0) load_chunk16<NT>(a, warp * CHUNKS, g, t, cur);
  int item = 0;
  for (int j = 0; j < my_units; ++j) {
    const int unit = (int)blockIdx.x + j * (int)gridDim.x;
    if (j > 0) __syncthreads();  // the previous unit's reduction has read `red`
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      float acc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
      for (int kk = 0; kk < gw; ++kk, ++item) {
        const int st = item % S;
        mbar_wait(my_bar + 8 * st, (uint32_t)((item / S) & 1), a.status);
        const uint8_t* tg = my_ring + st * R::STRIDE;
        const int kg = warp + GEMV_WARPS * kk;
        const int next_first = kk + 1 < gw ? (kg + GEMV_WARPS) * CHUNKS : (item + 1 < n_items ? warp * CHUNKS : -1);
        group16<TYPE, NT>(a, tg, kg, lane, acc, cur, next_first);
        __syncwarp();  // every lane has consumed the stage before it is refilled
        if (lane == 0 && item + S < n_items) issue(item + S);
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        red[p][warp][8 * nt + 2 * t][g] = acc[nt][0];
        red[p][warp][8 * nt + 2 * t + 1][g] = acc[nt][1];
        red[p][warp][8 * nt + 2 * t][g + 8] = acc[nt][2];
        red[p][warp][8 * nt + 2 * t + 1][g + 8] = acc[nt][3];
      }
    }
    __syncthreads();
    for (int o = threadIdx.x; o < NT * 8 * 16; o += GEMV_THREADS) {
      const int m = o >> 4, r = o & 15;
      const int n = unit * 16 + r;
      if (m >= a.M || n >= a.n_out) continue;
      float v[NP];
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_WARPS; ++w) s += red[p][w][m][r];
        v[p] = s * a.xscale[m];
      }
      const size_t idx = (size_t)m * a.n_out + n;
      float out;
      if (EPI == 2) {
        // silu(gate) * up, fusor-ml/fusor/src/composite/activations.rs:47-64
        const float gate = v[0];
        out = (gate / (1.0f + expf(-gate))) * v[NP - 1];
      } else if (EPI == 1) {
        out = v[0] + a.r1[(size_t)m * a.r1_stride + n];
        if (a.r2) out += a.r2[idx];
      } else {
        out = v[0];
      }
      a.y[idx] = out;
    }
  }
}

// ---- K-stationary form of the fp16 kernel ------------------------------------------------------
// With 2..32 activation rows a tile-group of W (1.1 - 3.4 KB) meets 4 - 16 KB of activations.
// Here every warp of a CTA owns ONE K group and keeps the MMA B fragments of all activation
// rows for that group in registers; the CTA walks an equal contiguous share of the 16-row tiles of
// W, warp w multiplying tile-group (tile, w), and the warps' partial tiles meet in shared memory
// once per tile (summed in warp order). Activations are read from L2 once per CTA instead of once
// per tile-group. Serves matrices of at most W K groups (K <= 4096 for the 256-element block types
// with 16 warps); longer rows take the streamed kernel above.
// Partial tiles of the warps meet in shared memory in the order of the MMA fragments: warp w, slot
// 4 nt + i, lane -- conflict-free for the writers (consecutive lanes) and for the readers. The warp
// stride is padded by two floats so that two threads that add different halves of the warps for
// the same output read different banks.
template <int NT>
struct Red16 {
  static constexpr int OUTS = NT * 8 * 16;   // outputs of one unit and pass
  static constexpr int WSTRIDE = OUTS + 2;   // floats between the partial tiles of two warps
  // fragment slot 4 nt + i of lane (g, t) -> activation row m and row r of the 16-row tile
  __device__ static void where(int v, int& m, int& r) {
    const int idx = v >> 5, ln = v & 31;
    m = 8 * (idx >> 2) + 2 * (ln & 3) + (idx & 1);
    r = (ln >> 2) + 8 * ((idx >> 1) & 1);
  }
};

template <int TYPE, int W, int BUDGET_KB = 168>
struct RingS {
  static constexpr int TG = Ring<TYPE>::TG;
  static constexpr int STRIDE = Ring<TYPE>::STRIDE;
  static constexpr int FIT = (BUDGET_KB * 1024) / (W * STRIDE);
  static constexpr int STAGES = FIT > 6 ? 6 : FIT;
  static constexpr int RING_BYTES = W * STAGES * STRIDE;
  static constexpr int BAR_BYTES = W * STAGES * 8;
};

// Shared memory of qgemm16s_kernel: ring, barriers, and the partial tiles of two consecutive units
// (NP passes each), so that one CTA barrier per unit is enough.
template <int NP>
constexpr int gemm16s_budget_kb() { return NP == 2 ? 150 : 168; }
template <int TYPE, int NT, int W, int NP>
constexpr int gemm16s_smem_bytes() {
  using R = RingS<TYPE, W, gemm16s_budget_kb<NP>()>;
  return R::RING_BYTES + R::BAR_BYTES + 2 * NP * W * Red16<NT>::WSTRIDE * (int)sizeof(float);
}

// group16 with the activations of the K group already in registers (x[chunk]).
template <int TYPE, int NT, int CHUNKS>
__device__ __forceinline__ void group16r(const uint8_t* tg, int lane, float (&acc)[NT][4],
                                         const Chunk16<NT> (&x)[CHUNKS]) {
  const int g = lane >> 2, t = lane & 3;
  const __half2 zero2 = __float2half2_rn(0.f);
  if constexpr (TYPE == FB200_Q4_0 || TYPE == FB200_Q8_0) {
#pragma unroll
    for (int blk = 0; blk < 4; ++blk) {
      const int dofs = TYPE == FB200_Q4_0 ? 1024 : 2048;
      const __half2 d_g = __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(tg + dofs + (g * 4 + blk) * 2)));
      const __half2 d_g8 = __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(tg + dofs + ((g + 8) * 4 + blk) * 2)));
      if constexpr (TYPE == FB200_Q4_0) {
        const uint32_t w0 = lds4(tg + g * 64 + blk * 16 + 4 * t);
        const uint32_t w1 = lds4(tg + 512 + g * 64 + blk * 16 + 4 * t);
        chunk16<NT>(acc, x[blk], w0 & 0x0F0F0F0Fu, w1 & 0x0F0F0F0Fu, (w0 >> 4) & 0x0F0F0F0Fu, (w1 >> 4) & 0x0F0F0F0Fu,
                    __float2half2_rn(1032.0f), d_g, d_g8, d_g, d_g8, zero2, zero2);  // (q - 8) d
      } else {
        const int off = g * 64 + blk * 16 + 4 * t;
        const uint32_t a0 = lds4(tg + off) ^ 0x80808080u, a2 = lds4(tg + 512 + off) ^ 0x80808080u;
        const uint32_t a1 = lds4(tg + 1024 + off) ^ 0x80808080u, a3 = lds4(tg + 1536 + off) ^ 0x80808080u;
        chunk16<NT>(acc, x[blk], a0, a1, a2, a3, __float2half2_rn(1152.0f), d_g, d_g8, d_g, d_g8, zero2, zero2);  // q d
      }
    }
  } else if constexpr (TYPE == FB200_Q4_K) {
    uint32_t sm[2][2];
    q4k_scales_h2(tg, g, t, sm);
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) {
      const int ch = pair >> 1, ps = pair & 1;
      const int off = g * 32 + ps * 16 + 4 * t;
      const uint32_t w00 = lds4(tg + ((ch * 2 + 0) * 2 + 0) * 256 + off);
      const uint32_t w01 = lds4(tg + ((ch * 2 + 0) * 2 + 1) * 256 + off);
      const uint32_t w10 = lds4(tg + ((ch * 2 + 1) * 2 + 0) * 256 + off);
      const uint32_t w11 = lds4(tg + ((ch * 2 + 1) * 2 + 1) * 256 + off);
#pragma unroll
      for (int hi = 0; hi < 2; ++hi) {
        const int sb = 2 * pair + hi;
        __half2 hs_g, hs_g8, ho_g, ho_g8;
        q4k_chunk_scales(sm, lane, sb, hs_g, hs_g8, ho_g, ho_g8);
        if (hi == 0)
          chunk16<NT, false>(acc, x[sb], w00 & 0x0F0F0F0Fu, w10 & 0x0F0F0F0Fu, w01 & 0x0F0F0F0Fu, w11 & 0x0F0F0F0Fu,
                             __float2half2_rn(1024.0f), hs_g, hs_g8, hs_g, hs_g8, ho_g, ho_g8);
        else
          chunk16<NT, true>(acc, x[sb], w00 & 0xF0F0F0F0u, w10 & 0xF0F0F0F0u, w01 & 0xF0F0F0F0u, w11 & 0xF0F0F0F0u,
                            __float2half2_rn(64.0f), hs_g, hs_g8, hs_g, hs_g8, ho_g, ho_g8);
      }
    }
  } else {  // Q6_K
    const uint4 sc_g = lds16(tg + 3072 + g * 16);
    const uint4 sc_g8 = lds16(tg + 3072 + (g + 8) * 16);
    const __half2 d_g = __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(tg + 3328 + g * 2)));
    const __half2 d_g8 = __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(tg + 3328 + (g + 8) * 2)));
    const uint32_t scw_g[4] = {sc_g.x ^ 0x80808080u, sc_g.y ^ 0x80808080u, sc_g.z ^ 0x80808080u, sc_g.w ^ 0x80808080u};
    const uint32_t scw_g8[4] = {sc_g8.x ^ 0x80808080u, sc_g8.y ^ 0x80808080u, sc_g8.z ^ 0x80808080u, sc_g8.w ^ 0x80808080u};
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t af[2][2];  // [u][row half]
        __half2 hs[2][2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int cu = c2 * 2 + u;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t wl = lds4(tg + (cu * 2 + h) * 256 + g * 32 + (q & 1) * 16 + 4 * t);
            const uint32_t wh = lds4(tg + 2048 + (cu * 2 + h) * 128 + g * 16 + 4 * t);
            const uint32_t hb = q == 0 ? (wh << 4) : q == 1 ? (wh << 2) : q == 2 ? wh : (wh >> 2);
            af[u][h] = (((q >> 1) ? (wl >> 4) : wl) & 0x0F0F0F0Fu) | (hb & 0x30303030u);
          }
        }
        q6k_chunk_scales(scw_g, d_g, c2, q, hs[0][0], hs[1][0]);
        q6k_chunk_scales(scw_g8, d_g8, c2, q, hs[0][1], hs[1][1]);
        chunk16<NT>(acc, x[c2 * 4 + q], af[0][0], af[0][1], af[1][0], af[1][1], __float2half2_rn(1056.0f), hs[0][0],
                    hs[0][1], hs[1][0], hs[1][1], zero2, zero2);  // (q - 32) d scale
      }
  }
}

template <int TYPE, int NT, int EPI, int W>
__global__ void __launch_bounds__(W * 32, 1)
qgemm16s_kernel(const GemvArgs a) {
  constexpr int NP = EPI == 2 ? 2 : 1;
  using R = RingS<TYPE, W, gemm16s_budget_kb<NP>()>;
  using RD = Red16<NT>;
  constexpr int S = R::STAGES;
  constexpr int CHUNKS = (TYPE == FB200_Q4_0 || TYPE == FB200_Q8_0) ? 4 : 8;
  constexpr int OUTS = RD::OUTS;
  constexpr int THREADS = W * 32;
  // threads that share one output (each adds the partial tiles of W / SPLIT warps, then a shuffle tree)
  constexpr int SPLIT = THREADS > OUTS ? THREADS / OUTS : 1;
  constexpr int PER = W / SPLIT;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + R::RING_BYTES);
  // [unit parity][pass][warp][fragment slot x lane (+ pad)]
  float (*red)[NP][W][RD::WSTRIDE] = reinterpret_cast<float (*)[NP][W][RD::WSTRIDE]>(smem + R::RING_BYTES + R::BAR_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* my_ring = ring + warp * S * R::STRIDE;
  const uint32_t my_bar = smem_u32(bars + warp * S);

  pdl_launch_dependents();
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < S; ++s) mbar_init(my_bar + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // this CTA's share of the units; warp w owns K group w
  const int base = a.nunits / (int)gridDim.x, rem = a.nunits - base * (int)gridDim.x;
  const int q0 = (int)blockIdx.x * base + min((int)blockIdx.x, rem), q1 = q0 + base + ((int)blockIdx.x < rem ? 1 : 0);
  const bool active = warp < a.ngroups;
  const int n_items = active ? (q1 - q0) * NP : 0;
  auto issue = [&](int i) {
    const int u = q0 + i / NP, p = i - (i / NP) * NP;
    const int tile = u + p * a.pair_tile_offset;
    const int st = i % S;
    const uint8_t* src = a.w + ((size_t)tile * a.ngroups + warp) * R::TG;
    mbar_expect_tx(my_bar + 8 * st, R::TG);
    bulk_g2s(smem_u32(my_ring + st * R::STRIDE), src, R::TG, my_bar + 8 * st);
  };
  if (lane == 0) {
    const int pre = n_items < S ? n_items : S;
    for (int i = 0; i < pre; ++i) issue(i);
  }
  pdl_wait();  // the packed activations come from the kernel before this one

  Chunk16<NT> xr[CHUNKS];
  if (n_items > 0) {
#pragma unroll
    for (int ch = 0; ch < CHUNKS; ++ch) load_chunk16<NT>(a, warp * CHUNKS + ch, g, t, xr[ch]);
  }
  const int nw = min(W, a.ngroups);  // warps that contribute to a tile
  int item = 0;
  for (int u = q0; u < q1; ++u) {
    const int par = (u - q0) & 1;
    if (active) {
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
        const int st = item % S;
        mbar_wait(my_bar + 8 * st, (uint32_t)((item / S) & 1), a.status);
        group16r<TYPE, NT, CHUNKS>(my_ring + st * R::STRIDE, lane, acc, xr);
        __syncwarp();  // every lane has consumed the stage before it is refilled
        if (lane == 0 && item + S < n_items) issue(item + S);
        ++item;
        float* rw = red[par][p][warp];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) rw[(nt * 4 + i) * 32 + lane] = acc[nt][i];
      }
    }
    // One barrier per unit: the buffers of this parity are next written two units from now, behind
    // the barrier of the unit in between, which every reader of this unit reaches only after reading.
    __syncthreads();
    // ---- the warps' partial tiles, summed in a fixed order: PER consecutive warps (= K groups) per
    // thread, then the SPLIT threads of an output
    for (int v = threadIdx.x / SPLIT; v < OUTS; v += THREADS / SPLIT) {
      const int part = threadIdx.x % SPLIT;
      float val[NP];
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
          const int w = part * PER + i;
          if (w < nw) sum += red[par][p][w][v];
        }
#pragma unroll
        for (int o = 1; o < SPLIT; o <<= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
        val[p] = sum;
      }
      int m, r;
      RD::where(v, m, r);
      const int n = u * 16 + r;
      if (part != 0 || m >= a.M || n >= a.n_out) continue;
      const float xs = a.xscale[m];
      const size_t idx = (size_t)m * a.n_out + n;
      float out;
      if (EPI == 2) {
        // silu(gate) * up, fusor-ml/fusor/src/composite/activations.rs:47-64
        const float gate = val[0] * xs;
        out = (gate / (1.0f + expf(-gate))) * (val[NP - 1] * xs);
      } else if (EPI == 1) {
        out = val[0] * xs + a.r1[(size_t)m * a.r1_stride + n];
        if (a.r2) out += a.r2[idx];
      } else {
        out = val[0] * xs;
      }
      a.y[idx] = out;
    }
  }
}

// x[M, K] f32 -> fp16 rows scaled by a power of two into (-64, 64), laid out [Kp/32][Mp][32]
// with lane t's eight halves of a chunk (elements 4t..4t+3, 16+4t..16+4t+3) at byte 16 t.
// One CTA per (padded) row.
__global__ void __launch_bounds__(256)
pack_x16_kernel(const float* __restrict__ x, int M, int K, int Kp, int Mp, __half* __restrict__ xh,
                float* __restrict__ xscale) {
  __shared__ float sh[8];
  const int m = blockIdx.x;
  const float* xr = x + (size_t)m * K;
  float amax = 0.f;
  if (m < M)
    for (int k = threadIdx.x; k < K; k += 256) amax = fmaxf(amax, fabsf(xr[k]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, sh[i]);
  int ex = 0;
  if (amax > 0.f && amax < 3.0e38f) frexpf(amax, &ex);
  const float inv = ldexpf(64.0f, -ex);  // x * inv in (-64, 64)
  if (threadIdx.x == 0) xscale[m] = ldexpf(1.0f, ex - 6);
  for (int k = threadIdx.x; k < Kp; k += 256) {
    const float v = (m < M && k < K) ? xr[k] * inv : 0.f;
    const int kc = k >> 5, e = k & 31;
    const int pos = ((e & 15) >> 2) * 8 + (e >> 4) * 4 + (e & 3);
    xh[((size_t)kc * Mp + m) * 32 + pos] = __float2half_rn(v);
  }
}

// RMS norm (optionally of x + res) and the packing of pack_x16_kernel in one pass over the row:
// y = ((x [+ res]) / rms) * w exactly as rms_norm_kernel computes it, then the row's power-of-two
// scale and the fp16 fragments. One CTA per (padded) row; rows of x are x_stride elements apart,
// rows of res are contiguous. EPT = elements a thread keeps in registers (K <= 256 * EPT).
template <int EPT>
__global__ void __launch_bounds__(256)
norm_pack_x16_kernel(const float* __restrict__ x, size_t x_stride, const float* __restrict__ res,
                     const float* __restrict__ w, float eps, int M, int K, int Kp, int Mp, __half* __restrict__ xh,
                     float* __restrict__ xscale) {
  __shared__ float sh[8];
  __shared__ float bc;
  const int m = blockIdx.x;
  const float* xr = x + (size_t)m * x_stride;
  const float* rr = res ? res + (size_t)m * K : nullptr;
  float v[EPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int k = threadIdx.x + 256 * i;
    v[i] = 0.f;
    if (m < M && k < K) v[i] = rr ? xr[k] + rr[k] : xr[k];
    ss = fmaf(v[i], v[i], ss);
  }
  // sum of squares in the order of rms_norm_kernel: per thread over k = tid, tid + 256, ..; lanes; warps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += sh[i];
    bc = t;
  }
  __syncthreads();
  const float rms = sqrtf(bc / (float)K + eps);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int k = threadIdx.x + 256 * i;
    if (m < M && k < K) v[i] = (v[i] / rms) * w[k];
    amax = fmaxf(amax, fabsf(v[i]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, sh[i]);
  int ex = 0;
  if (amax > 0.f && amax < 3.0e38f) frexpf(amax, &ex);
  const float inv = ldexpf(64.0f, -ex);  // y * inv in (-64, 64)
  if (threadIdx.x == 0) xscale[m] = ldexpf(1.0f, ex - 6);
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int k = threadIdx.x + 256 * i;
    if (k >= Kp) continue;
    const int kc = k >> 5, e = k & 31;
    const int pos = ((e & 15) >> 2) * 8 + (e >> 4) * 4 + (e & 3);
    xh[((size_t)kc * Mp + m) * 32 + pos] = __float2half_rn(v[i] * inv);
  }
}

// The two kernels above read their rows with dependent scalar loads (a few microseconds of pure
// latency per launch). These forms issue every load of a row (x, the residual row, the norm
// weights) as independent 16-byte loads before the first use, keep the row in registers, and
// store four packed halves at a time. They need 16-byte aligned rows and K a multiple of 4;
// V4 = float4 per thread (K <= 1024 * V4). NORM: rms_norm(x [+ res]) * w first, else x as it is.
template <int V4, bool NORM>
__global__ void __launch_bounds__(256)
pack_x16v_kernel(const float* __restrict__ x, size_t x_stride, const float* __restrict__ res,
                 const float* __restrict__ w, float eps, int M, int K, int Kp, int Mp, __half* __restrict__ xh,
                 float* __restrict__ xscale) {
  __shared__ float sh[8];
  __shared__ float bc;
  const int m = blockIdx.x;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 v[V4], r4[V4], w4[V4];
  pdl_launch_dependents();  // the product that follows may start fetching its weights
  pdl_wait();               // the rows come from the kernel before this one
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)m * x_stride);
  const float4* rr = reinterpret_cast<const float4*>(res ? res + (size_t)m * K : nullptr);
  const float4* wr = reinterpret_cast<const float4*>(w);
  const bool row = m < M;
#pragma unroll
  for (int i = 0; i < V4; ++i) {
    const int k4 = threadIdx.x + 256 * i;
    const bool in = row && 4 * k4 < K;
    v[i] = in ? __ldg(xr + k4) : zero4;
    r4[i] = (NORM && in && rr) ? __ldg(rr + k4) : zero4;
    w4[i] = (NORM && in) ? __ldg(wr + k4) : zero4;
  }
  if (NORM) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < V4; ++i) {
      if (rr) { v[i].x += r4[i].x; v[i].y += r4[i].y; v[i].z += r4[i].z; v[i].w += r4[i].w; }
      ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
      ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int i = 0; i < 8; ++i) t += sh[i];
      bc = t;
    }
    __syncthreads();
    // mean of squares, + eps, sqrt, divide, * weight (fusor-ml/fusor/src/composite/normalization.rs:404-461)
    const float rms = sqrtf(bc / (float)K + eps);
#pragma unroll
    for (int i = 0; i < V4; ++i) {
      v[i].x = (v[i].x / rms) * w4[i].x; v[i].y = (v[i].y / rms) * w4[i].y;
      v[i].z = (v[i].z / rms) * w4[i].z; v[i].w = (v[i].w / rms) * w4[i].w;
    }
    __syncthreads();  // sh is reused below
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < V4; ++i)
    amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v[i].x), fabsf(v[i].y))), fmaxf(fabsf(v[i].z), fabsf(v[i].w)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, sh[i]);
  int ex = 0;
  if (amax > 0.f && amax < 3.0e38f) frexpf(amax, &ex);
  const float inv = ldexpf(64.0f, -ex);  // row * inv in (-64, 64)
  if (threadIdx.x == 0) xscale[m] = ldexpf(1.0f, ex - 6);
#pragma unroll
  for (int i = 0; i < V4; ++i) {
    const int k = 4 * (threadIdx.x + 256 * i);
    if (k >= Kp) continue;
    const int kc = k >> 5, e = k & 31;
    const int pos = ((e & 15) >> 2) * 8 + (e >> 4) * 4;  // e is a multiple of 4: four consecutive slots
    const __half2 lo = __floats2half2_rn(v[i].x * inv, v[i].y * inv), hi = __floats2half2_rn(v[i].z * inv, v[i].w * inv);
    *reinterpret_cast<uint2*>(xh + ((size_t)kc * Mp + m) * 32 + pos) =
        make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
  }
}

template <bool NORM>
bool launch_pack_x16v(fb200_device* dev, const float* x, size_t x_stride, const float* res, const float* w, float eps,
                      int mc, uint64_t k, uint64_t kp, int mp, __half* h, float* sc) {
  const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(res) | reinterpret_cast<uintptr_t>(w);
  if ((bits & 15u) || (x_stride & 3u) || (k & 3u) || kp > 1024u * 16u) return false;
  const int K = (int)k, Kp = (int)kp;
  // launched with programmatic stream serialization: the kernel starts while its predecessor drains
  // and waits (griddepcontrol.wait) before it reads the rows
  if (kp <= 1024u * 4u)
    fb200_launch(dev, pack_x16v_kernel<4, NORM>, dim3(mp), dim3(256), 0, true, x, x_stride, res, w, eps, mc, K, Kp, mp, h, sc);
  else if (kp <= 1024u * 8u)
    fb200_launch(dev, pack_x16v_kernel<8, NORM>, dim3(mp), dim3(256), 0, true, x, x_stride, res, w, eps, mc, K, Kp, mp, h, sc);
  else
    fb200_launch(dev, pack_x16v_kernel<16, NORM>, dim3(mp), dim3(256), 0, true, x, x_stride, res, w, eps, mc, K, Kp, mp, h, sc);
  dev->launches--;  // counted by the caller's product, as the plain packing launch is
  return true;
}

template <int TYPE, int NT, int EPI>
int launch_one16(fb200_device* dev, GemvArgs& a) {
  constexpr int SMEM = gemv_smem_bytes<TYPE, NT, EPI>();
  static int occ[64] = {0};  // per device ordinal
  auto kern = qgemm16_kernel<TYPE, NT, EPI>;
  int& o = occ[dev->ordinal & 63];
  if (o == 0) {
    FB_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    int nb = 0;
    FB_CUDA(dev, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kern, GEMV_THREADS, SMEM));
    o = nb > 0 ? nb : 1;
  }
  int grid = dev->sm_count * o;
  if (grid > a.nunits) grid = a.nunits;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(GEMV_THREADS);
  cfg.dynamicSmemBytes = SMEM;
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

template <int TYPE, int NT>
int launch_epi16(fb200_device* dev, GemvArgs& a, int epi) {
  if (epi == FB200_EPI_SWIGLU) return launch_one16<TYPE, NT, 2>(dev, a);
  if (epi == FB200_EPI_RESIDUAL) return launch_one16<TYPE, NT, 1>(dev, a);
  return launch_one16<TYPE, NT, 0>(dev, a);
}

template <int TYPE>
int launch_nt16(fb200_device* dev, GemvArgs& a, int nt, int epi) {
  if (nt == 1) return launch_epi16<TYPE, 1>(dev, a, epi);
  if (nt == 2) return launch_epi16<TYPE, 2>(dev, a, epi);
  return launch_epi16<TYPE, 4>(dev, a, epi);
}

// The K-stationary kernel over up to three K-quant matrices (Q4_K / Q6_K, mixed) that share the
// activation rows, e.g. the q, k and v projections of a layer: one launch, one read of the
// activations, and the tiles of all matrices form one list that is cut into equal shares.
template <int NT, int W>
struct RingM {
  static constexpr int STRIDE = Ring<FB200_Q6_K>::STRIDE;  // the larger of the two tile-groups
  static constexpr int FIT = (168 * 1024) / (W * STRIDE);
  static constexpr int STAGES = FIT > 6 ? 6 : FIT;
  static constexpr int RING_BYTES = W * STAGES * STRIDE;
  static constexpr int BAR_BYTES = W * STAGES * 8;
  static constexpr int SMEM = RING_BYTES + BAR_BYTES + 2 * W * Red16<NT>::WSTRIDE * (int)sizeof(float);
};

template <int NT, int W>
__global__ void __launch_bounds__(W * 32, 1)
qgemm16s_multi_kernel(const GemvArgs a) {
  using R = RingM<NT, W>;
  constexpr int S = R::STAGES;
  constexpr int CHUNKS = 8;
  using RD = Red16<NT>;
  constexpr int OUTS = RD::OUTS;
  constexpr int THREADS = W * 32;
  constexpr int SPLIT = THREADS > OUTS ? THREADS / OUTS : 1;  // threads that share one output
  constexpr int PER = W / SPLIT;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + R::RING_BYTES);
  // [unit parity][warp][fragment slot x lane (+ pad)]
  float (*red)[W][RD::WSTRIDE] = reinterpret_cast<float (*)[W][RD::WSTRIDE]>(smem + R::RING_BYTES + R::BAR_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* my_ring = ring + warp * S * R::STRIDE;
  const uint32_t my_bar = smem_u32(bars + warp * S);

  pdl_launch_dependents();
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < S; ++s) mbar_init(my_bar + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  const int base = a.nunits / (int)gridDim.x, rem = a.nunits - base * (int)gridDim.x;
  const int q0 = (int)blockIdx.x * base + min((int)blockIdx.x, rem), q1 = q0 + base + ((int)blockIdx.x < rem ? 1 : 0);
  const bool active = warp < a.ngroups;
  const int n_items = active ? q1 - q0 : 0;
  // unit -> (matrix, tile)
  auto locate = [&](int u, int& sidx, int& tile) {
    sidx = 0; tile = u;
    if (a.nseg > 1 && tile >= a.seg[0].units) { tile -= a.seg[0].units; sidx = 1; }
    if (a.nseg > 2 && sidx == 1 && tile >= a.seg[1].units) { tile -= a.seg[1].units; sidx = 2; }
  };
  auto issue = [&](int i) {
    int sidx, tile;
    locate(q0 + i, sidx, tile);
    const uint32_t tg = a.seg[sidx].type == FB200_Q4_K ? Ring<FB200_Q4_K>::TG : Ring<FB200_Q6_K>::TG;
    const int st = i % S;
    const uint8_t* src = a.seg[sidx].w + ((size_t)tile * a.ngroups + warp) * tg;
    mbar_expect_tx(my_bar + 8 * st, tg);
    bulk_g2s(smem_u32(my_ring + st * R::STRIDE), src, tg, my_bar + 8 * st);
  };
  if (lane == 0) {
    const int pre = n_items < S ? n_items : S;
    for (int i = 0; i < pre; ++i) issue(i);
  }
  pdl_wait();  // the packed activations come from the kernel before this one

  Chunk16<NT> xr[CHUNKS];
  if (n_items > 0) {
#pragma unroll
    for (int ch = 0; ch < CHUNKS; ++ch) load_chunk16<NT>(a, warp * CHUNKS + ch, g, t, xr[ch]);
  }
  const int nw = min(W, a.ngroups);
  for (int u = q0; u < q1; ++u) {
    const int item = u - q0, par = item & 1;
    int sidx, tile;
    locate(u, sidx, tile);
    if (active) {
      float acc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
      const int st = item % S;
      mbar_wait(my_bar + 8 * st, (uint32_t)((item / S) & 1), a.status);
      if (a.seg[sidx].type == FB200_Q4_K) group16r<FB200_Q4_K, NT, CHUNKS>(my_ring + st * R::STRIDE, lane, acc, xr);
      else group16r<FB200_Q6_K, NT, CHUNKS>(my_ring + st * R::STRIDE, lane, acc, xr);
      __syncwarp();
      if (lane == 0 && item + S < n_items) issue(item + S);
      float* rw = red[par][warp];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) rw[(nt * 4 + i) * 32 + lane] = acc[nt][i];
    }
    __syncthreads();
    // PER consecutive warps (= K groups) per thread, then the SPLIT threads of an output: a fixed order
    for (int v = threadIdx.x / SPLIT; v < OUTS; v += THREADS / SPLIT) {
      const int part = threadIdx.x % SPLIT;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int w = part * PER + i;
        if (w < nw) sum += red[par][w][v];
      }
#pragma unroll
      for (int o = 1; o < SPLIT; o <<= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
      int m, r;
      RD::where(v, m, r);
      const int n = tile * 16 + r;
      if (part != 0 || m >= a.M || n >= a.seg[sidx].n_out) continue;
      a.seg[sidx].y[(size_t)m * a.seg[sidx].n_out + n] = sum * a.xscale[m];
    }
  }
}

// Warps per CTA of the K-stationary kernel: 16 while the activation fragments of a K group fit
// beside everything else in 128 registers per thread (up to 16 rows), 8 for 17..32 rows.
constexpr int gemm16s_warps(int nt) { return nt == 4 ? 8 : 16; }

template <int TYPE, int NT, int EPI>
int launch_one16s(fb200_device* dev, GemvArgs& a) {
  constexpr int W = gemm16s_warps(NT);
  constexpr int SMEM = gemm16s_smem_bytes<TYPE, NT, W, EPI == 2 ? 2 : 1>();
  static bool configured[64] = {false};  // per device ordinal
  auto kern = qgemm16s_kernel<TYPE, NT, EPI, W>;
  if (!configured[dev->ordinal & 63]) {
    FB_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured[dev->ordinal & 63] = true;
  }
  int grid = dev->sm_count;
  if (grid > a.nunits) grid = a.nunits;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(W * 32);
  cfg.dynamicSmemBytes = SMEM;
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

template <int TYPE, int NT>
int launch_epi16s(fb200_device* dev, GemvArgs& a, int epi) {
  if (epi == FB200_EPI_SWIGLU) return launch_one16s<TYPE, NT, 2>(dev, a);
  if (epi == FB200_EPI_RESIDUAL) return launch_one16s<TYPE, NT, 1>(dev, a);
  return launch_one16s<TYPE, NT, 0>(dev, a);
}

template <int TYPE>
int launch_nt16s(fb200_device* dev, GemvArgs& a, int nt, int epi) {
  if (nt == 1) return launch_epi16s<TYPE, 1>(dev, a, epi);
  if (nt == 2) return launch_epi16s<TYPE, 2>(dev, a, epi);
  return launch_epi16s<TYPE, 4>(dev, a, epi);
}

template <int TYPE, int NT, int EPI>
int launch_one(fb200_device* dev, GemvArgs& a) {
  constexpr int SMEM = gemv_smem_bytes<TYPE, NT, EPI>();
  static int occ[64] = {0};  // per device ordinal
  auto kern = qgemv_kernel<TYPE, NT, EPI>;
  int& o = occ[dev->ordinal & 63];
  if (o == 0) {
    FB_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    int nb = 0;
    FB_CUDA(dev, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kern, GEMV_THREADS, SMEM));
    o = nb > 0 ? nb : 1;
  }
  int grid = dev->sm_count * o;
  if (grid > a.nunits) grid = a.nunits;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(GEMV_THREADS);
  cfg.dynamicSmemBytes = SMEM;
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

template <int TYPE, int NT>
int launch_epi(fb200_device* dev, GemvArgs& a, int epi) {
  if (epi == FB200_EPI_SWIGLU) return launch_one<TYPE, NT, 2>(dev, a);
  if (epi == FB200_EPI_RESIDUAL) return launch_one<TYPE, NT, 1>(dev, a);
  return launch_one<TYPE, NT, 0>(dev, a);
}

template <int TYPE>
int launch_nt(fb200_device* dev, GemvArgs& a, int nt, int epi) {
  if (nt == 1) return launch_epi<TYPE, 1>(dev, a, epi);
  if (nt == 2) return launch_epi<TYPE, 2>(dev, a, epi);
  return launch_epi<TYPE, 4>(dev, a, epi);
}

}  // namespace

// Bytes of packed-activation scratch needed for an [M<=32, K] product.
size_t fb200_xpack_bytes(int mp, uint64_t kp) {
  return (size_t)(kp / 32) * 4 * mp * 32 + (size_t)(kp / 16) * mp * sizeof(float) +
         (size_t)mp * sizeof(float) + 256;
}

// Product of at most 32 activation rows that are already packed (fb200_pack_x16: fp16 fragments
// [Kp/32][Mp][32] and the rows' power-of-two scales).
int fb200_qgemm16_packed(fb200_device* dev, const fb200_qmatrix* w, const void* xh, const float* xscale16, int mc, int mp,
                         float* y, int epi, const float* r1, const float* r2, bool r1_is_bias) {
  const int nt = mp / 8;
  GemvArgs a16 = {};
  a16.w = w->data; a16.xq = reinterpret_cast<const uint8_t*>(xh); a16.xs16 = nullptr; a16.xscale = xscale16;
  a16.y = y; a16.r1 = r1; a16.r2 = r2;
  a16.r1_stride = r1_is_bias ? 0 : (int)(epi == FB200_EPI_SWIGLU ? w->n / 2 : w->n);
  a16.M = mc; a16.Mp = mp; a16.ngroups = w->ngroups;
  a16.nunits = w->ntiles;
  a16.n_out = (int)w->n;
  a16.pair_tile_offset = 0;
  a16.status = dev->status;
  if (epi == FB200_EPI_SWIGLU) {
    a16.nunits = w->ntiles / 2;
    a16.n_out = (int)(w->n / 2);
    a16.pair_tile_offset = w->ntiles / 2;
  }
  // FB200_GEMM16_STREAMED=1 keeps every shape on the streamed kernel (for comparisons)
  static const bool streamed_only = getenv("FB200_GEMM16_STREAMED") && getenv("FB200_GEMM16_STREAMED")[0] == '1';
  if (w->ngroups <= gemm16s_warps(nt) && !streamed_only) {
    switch (w->type) {
      case FB200_Q4_0: return launch_nt16s<FB200_Q4_0>(dev, a16, nt, epi);
      case FB200_Q8_0: return launch_nt16s<FB200_Q8_0>(dev, a16, nt, epi);
      case FB200_Q4_K: return launch_nt16s<FB200_Q4_K>(dev, a16, nt, epi);
      default: return launch_nt16s<FB200_Q6_K>(dev, a16, nt, epi);
    }
  }
  switch (w->type) {
    case FB200_Q4_0: return launch_nt16<FB200_Q4_0>(dev, a16, nt, epi);
    case FB200_Q8_0: return launch_nt16<FB200_Q8_0>(dev, a16, nt, epi);
    case FB200_Q4_K: return launch_nt16<FB200_Q4_K>(dev, a16, nt, epi);
    default: return launch_nt16<FB200_Q6_K>(dev, a16, nt, epi);
  }
}

// Padded inner size of a tiled matrix (what the packed activations must cover).
uint64_t fb200_qmatrix_kp(const fb200_qmatrix* w) {
  TileGeom geo;
  if (!w->tiled || !tile_geom(w->type, &geo)) return 0;
  return (uint64_t)w->ngroups * geo.group_elems;
}

// Up to three products over the same packed rows in one launch (no epilogue). Covers Q4_K / Q6_K
// matrices of at most 16 K groups and up to 16 rows; returns 1 otherwise (the caller then launches
// the products one by one).
int fb200_qgemm16_packed_multi(fb200_device* dev, const fb200_qmatrix* const* ws, float* const* ys, int nw, const void* xh,
                               const float* xscale16, int mc, int mp) {
  const int nt = mp / 8;
  if (nw < 1 || nw > 3 || nt > 2) return 1;
  GemvArgs a = {};
  a.xq = reinterpret_cast<const uint8_t*>(xh); a.xscale = xscale16;
  a.M = mc; a.Mp = mp; a.ngroups = ws[0]->ngroups; a.status = dev->status;
  a.nseg = nw;
  for (int i = 0; i < nw; ++i) {
    if (!ws[i]->tiled || (ws[i]->type != FB200_Q4_K && ws[i]->type != FB200_Q6_K) || ws[i]->ngroups != a.ngroups ||
        ws[i]->k != ws[0]->k)
      return 1;
    a.seg[i].w = ws[i]->data; a.seg[i].y = ys[i]; a.seg[i].n_out = (int)ws[i]->n; a.seg[i].units = ws[i]->ntiles;
    a.seg[i].type = (int)ws[i]->type;
    a.nunits += ws[i]->ntiles;
  }
  if (a.ngroups > 16 || a.nunits < 1) return 1;
  static const bool streamed_only = getenv("FB200_GEMM16_STREAMED") && getenv("FB200_GEMM16_STREAMED")[0] == '1';
  if (streamed_only) return 1;
  int grid = dev->sm_count < a.nunits ? dev->sm_count : a.nunits;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(16 * 32);
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dev->pdl ? 1 : 0;
  static bool configured[64][2] = {};
  if (nt == 1) {
    auto kern = qgemm16s_multi_kernel<1, 16>;
    if (!configured[dev->ordinal & 63][0]) {
      FB_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, RingM<1, 16>::SMEM));
      configured[dev->ordinal & 63][0] = true;
    }
    cfg.dynamicSmemBytes = RingM<1, 16>::SMEM;
    FB_CUDA(dev, cudaLaunchKernelEx(&cfg, kern, a));
  } else {
    auto kern = qgemm16s_multi_kernel<2, 16>;
    if (!configured[dev->ordinal & 63][1]) {
      FB_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, RingM<2, 16>::SMEM));
      configured[dev->ordinal & 63][1] = true;
    }
    cfg.dynamicSmemBytes = RingM<2, 16>::SMEM;
    FB_CUDA(dev, cudaLaunchKernelEx(&cfg, kern, a));
  }
  dev->launches++;
  return FB200_OK;
}

// Rows per packed batch: 8, 16 or 32.
int fb200_pack16_rows(int mc) { return mc <= 8 ? 8 : mc <= 16 ? 16 : 32; }

// x[mc, K] f32 -> the packed form of fb200_qgemm16_packed in `scratch` (fb200_xpack_bytes(mp, kp) bytes).
int fb200_pack_x16(fb200_device* dev, const float* x, int mc, uint64_t k, uint64_t kp, void* scratch, const void** xh,
                   const float** xscale) {
  const int mp = fb200_pack16_rows(mc);
  __half* h = reinterpret_cast<__half*>(scratch);
  float* sc = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + (size_t)kp * mp * 2);
  if (!launch_pack_x16v<false>(dev, x, (size_t)k, nullptr, nullptr, 0.f, mc, k, kp, mp, h, sc))
    pack_x16_kernel<<<mp, 256, 0, dev->stream>>>(x, mc, (int)k, (int)kp, mp, h, sc);
  FB_LAUNCH_CHECK(dev);
  *xh = h;
  *xscale = sc;
  return FB200_OK;
}

// rms_norm(x [+ res]) * w of mc rows, packed like fb200_pack_x16. Returns 1 when K is beyond what
// the fused kernel keeps in registers (the caller then normalises and packs in two steps).
int fb200_norm_pack_x16(fb200_device* dev, const float* x, size_t x_stride, const float* res, const float* w, float eps,
                        int mc, uint64_t k, uint64_t kp, void* scratch, const void** xh, const float** xscale) {
  const int mp = fb200_pack16_rows(mc);
  __half* h = reinterpret_cast<__half*>(scratch);
  float* sc = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + (size_t)kp * mp * 2);
  if (launch_pack_x16v<true>(dev, x, x_stride, res, w, eps, mc, k, kp, mp, h, sc)) {
  } else if (kp <= 256 * 8)
    norm_pack_x16_kernel<8><<<mp, 256, 0, dev->stream>>>(x, x_stride, res, w, eps, mc, (int)k, (int)kp, mp, h, sc);
  else if (kp <= 256 * 16)
    norm_pack_x16_kernel<16><<<mp, 256, 0, dev->stream>>>(x, x_stride, res, w, eps, mc, (int)k, (int)kp, mp, h, sc);
  else if (kp <= 256 * 32)
    norm_pack_x16_kernel<32><<<mp, 256, 0, dev->stream>>>(x, x_stride, res, w, eps, mc, (int)k, (int)kp, mp, h, sc);
  else
    return 1;
  FB_LAUNCH_CHECK(dev);
  *xh = h;
  *xscale = sc;
  return FB200_OK;
}

// y[m0 .. m0+mc) = x . W^T for a chunk of at most 32 activation rows, using `scratch`.
int fb200_qgemv_chunk(fb200_device* dev, const fb200_qmatrix* w, const float* x, int mc, float* y,
                      int epi, const float* r1, const float* r2, void* scratch, bool r1_is_bias) {
  TileGeom geo;
  tile_geom(w->type, &geo);
  const int nt = mc <= 8 ? 1 : mc <= 16 ? 2 : 4;
  const int mp = nt * 8;
  const uint64_t kp = (uint64_t)w->ngroups * geo.group_elems;
  const int nl = nt == 1 ? 4 : nt == 2 ? 3 : 2;
  // FB200_EXACT_SMALL_BATCH=1 keeps 2 .. 8 rows on the int8 limb kernel (2^-27 activations, about
  // 1.6 times slower); by default every batch of 2 .. 32 rows takes the fp16 kernel
  static const bool exact_small = getenv("FB200_EXACT_SMALL_BATCH") && getenv("FB200_EXACT_SMALL_BATCH")[0] == '1';
  if (nt > 1 || !exact_small) {
    const void* xh;
    const float* xscale16;
    int rc = fb200_pack_x16(dev, x, mc, w->k, kp, scratch, &xh, &xscale16);
    if (rc) return rc;
    return fb200_qgemm16_packed(dev, w, xh, xscale16, mc, mp, y, epi, r1, r2, r1_is_bias);
  }
  uint8_t* xq = reinterpret_cast<uint8_t*>(scratch);
  size_t off = (size_t)(kp / 32) * nl * mp * 32;
  float* xs16 = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + off);
  off += (size_t)(kp / 16) * mp * sizeof(float);
  float* xscale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + off);
  if (nl == 4) pack_x_kernel<4><<<mp, 256, 0, dev->stream>>>(x, mc, (int)w->k, (int)kp, mp, xq, xs16, xscale);
  else if (nl == 3) pack_x_kernel<3><<<mp, 256, 0, dev->stream>>>(x, mc, (int)w->k, (int)kp, mp, xq, xs16, xscale);
  else pack_x_kernel<2><<<mp, 256, 0, dev->stream>>>(x, mc, (int)w->k, (int)kp, mp, xq, xs16, xscale);
  FB_LAUNCH_CHECK(dev);
  GemvArgs a;
  a.w = w->data; a.xq = xq; a.xs16 = xs16; a.xscale = xscale; a.y = y; a.r1 = r1; a.r2 = r2;
  a.r1_stride = r1_is_bias ? 0 : (int)(epi == FB200_EPI_SWIGLU ? w->n / 2 : w->n);
  a.M = mc; a.Mp = mp; a.ngroups = w->ngroups;
  a.nunits = w->ntiles;
  a.n_out = (int)w->n;
  a.pair_tile_offset = 0;
  a.status = dev->status;
  if (epi == FB200_EPI_SWIGLU) {
    a.nunits = w->ntiles / 2;
    a.n_out = (int)(w->n / 2);
    a.pair_tile_offset = w->ntiles / 2;
  }
  switch (w->type) {
    case FB200_Q4_0: return launch_nt<FB200_Q4_0>(dev, a, nt, epi);
    case FB200_Q8_0: return launch_nt<FB200_Q8_0>(dev, a, nt, epi);
    case FB200_Q4_K: return launch_nt<FB200_Q4_K>(dev, a, nt, epi);
    default: return launch_nt<FB200_Q6_K>(dev, a, nt, epi);
  }
}

// ---- product without any allocation ------------------------------------------------------------
// Some hosts may not allocate device memory at the moment they need a product: code that runs
// inside a region where the CUDA allocator must not be entered (a latency-critical serving
// loop that has pinned its memory budget, a callback on a thread that holds locks the
// allocator also takes, a plug-in sandbox that forbids cudaMalloc after start-up). The regular
// entry point grows a scratch buffer for the packed activation limbs on demand; this variant
// keeps that scratch in a fixed array that is part of the library image instead.
//
// FB200_STATIC_SCRATCH_BYTES of device memory per GPU that loads the library, held until exit.
constexpr size_t FB200_STATIC_SCRATCH_BYTES = 4u << 20;
static __device__ __align__(256) uint8_t g_static_xpack[FB200_STATIC_SCRATCH_BYTES];

namespace {
// Device address of g_static_xpack per device ordinal. In host code the array's name is only a
// handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress, asked
// once per device with that device current. Atomic because two handles of one device may be
// driven by two host threads (both would store the same address).
std::atomic<void*> g_static_xpack_addr[64];
}  // namespace

extern "C" int fb200_q_mat_mul_noalloc(fb200_device* dev, const float* x_dev, size_t m,
                                       const fb200_qmatrix* w, float* y_dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!w || !x_dev || !y_dev)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "q_mat_mul_noalloc: null argument");
  if (w->dev != dev)
    return fb200_fail(dev, FB200_ERR_DEVICE_MISMATCH, "q_mat_mul_noalloc: weight lives on another device handle");
  if (!w->tiled)
    return fb200_fail(dev, FB200_ERR_UNSUPPORTED_DTYPE,
                      "q_mat_mul_noalloc: only Q4_0, Q5_0, Q8_0, Q4_K and Q6_K weights are supported");
  if (m == 0 || w->n == 0) return FB200_OK;
  if (m > 32)
    return fb200_fail(dev, FB200_ERR_CAPACITY, "q_mat_mul_noalloc: %zu activation rows, at most 32 per call", m);
  if (dev->ordinal < 0 || dev->ordinal >= 64)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "q_mat_mul_noalloc: device ordinal %d out of range", dev->ordinal);
  TileGeom geo;
  tile_geom(w->type, &geo);
  const uint64_t kp = (uint64_t)w->ngroups * geo.group_elems;
  const int mp = m <= 8 ? 8 : m <= 16 ? 16 : 32;
  const size_t need = fb200_xpack_bytes(mp, kp);
  if (need > FB200_STATIC_SCRATCH_BYTES)
    return fb200_fail(dev, FB200_ERR_CAPACITY,
                      "q_mat_mul_noalloc: %zu rows x K = %llu need %zu bytes of packed activations, the "
                      "built-in scratch holds %zu",
                      m, (unsigned long long)w->k, need, (size_t)FB200_STATIC_SCRATCH_BYTES);
  void* scratch = g_static_xpack_addr[dev->ordinal].load(std::memory_order_acquire);
  if (!scratch) {
    // first call on this device: resolve the array's device address (device is current)
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_xpack);
    if (e != cudaSuccess || !p)
      return fb200_fail(dev, FB200_ERR_CUDA, "q_mat_mul_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    scratch = p;
    g_static_xpack_addr[dev->ordinal].store(p, std::memory_order_release);
  }
  // Nothing in the scratch has to start at zero: the pack kernel rewrites every byte the
  // product kernel reads (limbs of padded rows are never loaded, their sums are written as 0).
  return fb200_qgemv_chunk(dev, w, x_dev, (int)m, y_dev, FB200_EPI_NONE, nullptr, nullptr, scratch, false);
}
