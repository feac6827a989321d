// Quantised matrix x small-batch activation product (decode GEMV and M <= 32 "skinny" GEMM).
//
// Bound: HBM. One CTA owns a 16-row tile of W and all of K; its 8 warps take K groups round
// robin, so a 4096 x 4096 matrix gives 256 CTAs x 8 warps of independent 16-byte loads.
// Each lane reads its mma.m16n8k16 A-fragment bytes straight from the tile-interleaved
// storage with coalesced 128-bit loads (a warp load covers 512 contiguous bytes), expands the
// 4/6/8-bit quants to exact fp16 integers in registers with logic ops (no int->float
// conversions), and lets the tensor cores form the integer-weight x activation dot products
// in fp32. Block scales are applied to the fp32 partial sums per 16- or 32-element group, so
// the only rounding beyond the reference's f32 path is that of the activations, which are
// carried as a hi + lo pair of fp16 values (about 22 mantissa bits; two MMAs per fragment),
// pre-scaled per row by a power of two so their range is never an issue.
// The batch occupies the N = 8 columns of the MMA, which makes M <= 8 cost the same weight
// traffic and nearly the same instruction count as M = 1.
//
// Replaces the reference's qgemv kernels (fusor-ml/tile-ir-kernels/src/kernels/qgemv.rs:356-678,
// qgemv_q6k.rs:84-385) and their SwiGLU / residual epilogues
// (fusor-ml/core/src/quantized/matmul/mod.rs:435-439, 666-722).
#include "formats.cuh"

namespace {

constexpr int GEMV_WARPS = 8;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;

struct GemvArgs {
  const uint8_t* w;     // tiled weights
  const __half* xt;     // packed activations [K/16][Mp][32] (hi/lo fp16 fragments)
  const float* xsum;    // [K/32][Mp] sums of the scaled activations (Q4_K offsets)
  const float* xscale;  // [Mp] power-of-two row scales
  float* y;             // [M, Nout]
  const float* r1;
  const float* r2;
  int M, Mp;
  int n_out;    // logical output columns (N, or N/2 for SwiGLU)
  int ngroups;  // K groups per tile
  int pair_tile_offset;  // SwiGLU: tile index distance between the gate and the up tile
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Nibbles of bytes (0, 2) / (1, 3) of a word as a pair of fp16 values with a bias:
// low nibbles land in the mantissa of 1024.0 (0x6400), high nibbles in that of 64.0 (0x5400).
__device__ __forceinline__ uint32_t lo02(uint32_t w) { return (w & 0x000F000Fu) | 0x64006400u; }
__device__ __forceinline__ uint32_t hi02(uint32_t w) { return (w & 0x00F000F0u) | 0x54005400u; }

__device__ __forceinline__ uint4 ldg16(const uint8_t* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// B fragments of one 16-element K chunk: {hi.b0, hi.b1, lo.b0, lo.b1} per 8-column tile.
// The activation is carried as hi + lo fp16 (lo = fp16(x - hi)), which keeps ~22 mantissa bits.
template <int NT>
__device__ __forceinline__ void load_b(const GemvArgs& a, int kk, int g, int t,
                                       uint32_t (&b)[NT][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    int m = 8 * nt + g;
    if (m < a.M) {
      uint4 v = __ldg(reinterpret_cast<const uint4*>(a.xt + ((size_t)kk * a.Mp + m) * 32 + 8 * t));
      b[nt][0] = v.x; b[nt][1] = v.y; b[nt][2] = v.z; b[nt][3] = v.w;
    } else {
      b[nt][0] = 0u; b[nt][1] = 0u; b[nt][2] = 0u; b[nt][3] = 0u;
    }
  }
}

template <int NT>
__device__ __forceinline__ void mma_hilo(float (&c)[NT][4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, const uint32_t (&b)[NT][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    mma16816(c[nt], a0, a1, a2, a3, b[nt][0], b[nt][1]);
    mma16816(c[nt], a0, a1, a2, a3, b[nt][2], b[nt][3]);
  }
}

template <int NT>
__device__ __forceinline__ void zero_c(float (&c)[NT][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) c[nt][i] = 0.f;
}

template <int NT>
__device__ __forceinline__ void scale_add(float (&acc)[NT][4], const float (&c)[NT][4], float s_g,
                                          float s_g8) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    acc[nt][0] = fmaf(s_g, c[nt][0], acc[nt][0]);
    acc[nt][1] = fmaf(s_g, c[nt][1], acc[nt][1]);
    acc[nt][2] = fmaf(s_g8, c[nt][2], acc[nt][2]);
    acc[nt][3] = fmaf(s_g8, c[nt][3], acc[nt][3]);
  }
}

// ---- per-format processing of one tile-group by one warp --------------------------------------

template <int NT>
__device__ __forceinline__ void group_q4_0(const GemvArgs& a, const uint8_t* tg, int kg, int lane,
                                           float (&acc)[NT][4]) {
  const int g = lane >> 2, t = lane & 3;
  uint4 qa = ldg16(tg + lane * 16);
  uint4 qb = ldg16(tg + 512 + lane * 16);
  uint2 dg = __ldg(reinterpret_cast<const uint2*>(tg + 1024 + g * 8));
  uint2 dg8 = __ldg(reinterpret_cast<const uint2*>(tg + 1024 + (g + 8) * 8));
  const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w};
  const uint32_t wb[4] = {qb.x, qb.y, qb.z, qb.w};
  const uint32_t sa[2] = {dg.x, dg.y};
  const uint32_t sb[2] = {dg8.x, dg8.y};
#pragma unroll
  for (int blk = 0; blk < 4; ++blk) {
    float c[NT][4];
    zero_c<NT>(c);
    uint32_t b[NT][4];
    const int kk = (kg * 4 + blk) * 2;
    // low nibbles: elements 0..15 of the block, centred by 8 (bias 1024 + 8)
    load_b<NT>(a, kk, g, t, b);
    {
      uint32_t a0 = hsub2(lo02(wa[blk]), 0x64086408u), a1 = hsub2(lo02(wb[blk]), 0x64086408u);
      uint32_t a2 = hsub2(lo02(wa[blk] >> 8), 0x64086408u), a3 = hsub2(lo02(wb[blk] >> 8), 0x64086408u);
      mma_hilo<NT>(c, a0, a1, a2, a3, b);
    }
    // high nibbles: elements 16..31 (bias 64 + 8)
    load_b<NT>(a, kk + 1, g, t, b);
    {
      uint32_t a0 = hsub2(hi02(wa[blk]), 0x54805480u), a1 = hsub2(hi02(wb[blk]), 0x54805480u);
      uint32_t a2 = hsub2(hi02(wa[blk] >> 8), 0x54805480u), a3 = hsub2(hi02(wb[blk] >> 8), 0x54805480u);
      mma_hilo<NT>(c, a0, a1, a2, a3, b);
    }
    uint16_t hg = (uint16_t)(sa[blk >> 1] >> (16 * (blk & 1)));
    uint16_t hg8 = (uint16_t)(sb[blk >> 1] >> (16 * (blk & 1)));
    scale_add<NT>(acc, c, fb::half_bits_to_float(hg), fb::half_bits_to_float(hg8));
  }
}

template <int NT>
__device__ __forceinline__ void group_q8_0(const GemvArgs& a, const uint8_t* tg, int kg, int lane,
                                           float (&acc)[NT][4]) {
  const int g = lane >> 2, t = lane & 3;
  uint4 q[2][2];
#pragma unroll
  for (int p = 0; p < 2; ++p)
#pragma unroll
    for (int h = 0; h < 2; ++h) q[p][h] = ldg16(tg + (p * 2 + h) * 512 + lane * 16);
  uint2 dg = __ldg(reinterpret_cast<const uint2*>(tg + 2048 + g * 8));
  uint2 dg8 = __ldg(reinterpret_cast<const uint2*>(tg + 2048 + (g + 8) * 8));
  const uint32_t sa[2] = {dg.x, dg.y};
  const uint32_t sb[2] = {dg8.x, dg8.y};
#pragma unroll
  for (int blk = 0; blk < 4; ++blk) {
    float c[NT][4];
    zero_c<NT>(c);
    const int p = blk >> 1;
    const uint32_t wa[4] = {q[p][0].x, q[p][0].y, q[p][0].z, q[p][0].w};
    const uint32_t wb[4] = {q[p][1].x, q[p][1].y, q[p][1].z, q[p][1].w};
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      uint32_t b[NT][4];
      load_b<NT>(a, (kg * 4 + blk) * 2 + hf, g, t, b);
      // signed byte + 128 sits in the mantissa of 1024.0; subtract 1152 to recover the value
      uint32_t xa = wa[(blk & 1) * 2 + hf] ^ 0x80808080u;
      uint32_t xb = wb[(blk & 1) * 2 + hf] ^ 0x80808080u;
      uint32_t a0 = hsub2(__byte_perm(xa, 0x64646464u, 0x4240), 0x64806480u);
      uint32_t a1 = hsub2(__byte_perm(xb, 0x64646464u, 0x4240), 0x64806480u);
      uint32_t a2 = hsub2(__byte_perm(xa, 0x64646464u, 0x4341), 0x64806480u);
      uint32_t a3 = hsub2(__byte_perm(xb, 0x64646464u, 0x4341), 0x64806480u);
      mma_hilo<NT>(c, a0, a1, a2, a3, b);
    }
    uint16_t hg = (uint16_t)(sa[blk >> 1] >> (16 * (blk & 1)));
    uint16_t hg8 = (uint16_t)(sb[blk >> 1] >> (16 * (blk & 1)));
    scale_add<NT>(acc, c, fb::half_bits_to_float(hg), fb::half_bits_to_float(hg8));
  }
}

// Q4_K: w = (d * sc) * q - (dmin * m). The q.x part runs on the tensor cores per 32-element
// sub-block; the offset part needs sum(x) over the sub-block, precomputed by the pack kernel.
// Lane t of each quad decodes the 6-bit (sc, m) of sub-blocks 2t and 2t+1 for its two rows
// and the quad shares them by shuffle.
template <int NT>
__device__ __forceinline__ void group_q4k(const GemvArgs& a, const uint8_t* tg, int kg, int lane,
                                          float (&acc)[NT][4]) {
  const int g = lane >> 2, t = lane & 3;
  uint4 q[2][2];
#pragma unroll
  for (int jj = 0; jj < 2; ++jj)
#pragma unroll
    for (int h = 0; h < 2; ++h) q[jj][h] = ldg16(tg + (jj * 2 + h) * 512 + lane * 16);
  float sc_f[2][2], mn_f[2][2];  // [row half][sub-block 2t + i]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint4 hd = ldg16(tg + 2048 + (g + 8 * h) * 16);
    float d = fb::half_bits_to_float((uint16_t)(hd.x & 0xFFFF));
    float dmin = fb::half_bits_to_float((uint16_t)(hd.x >> 16));
    uint32_t s0 = hd.y, s1 = hd.z, s2 = hd.w;
    uint32_t scA = s0 & 0x3F3F3F3Fu, mnA = s1 & 0x3F3F3F3Fu;
    uint32_t scB = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
    uint32_t mnB = ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u);
    uint32_t scw = (t < 2) ? scA : scB, mnw = (t < 2) ? mnA : mnB;
    int sh = (t & 1) * 16;
    sc_f[h][0] = d * (float)((scw >> sh) & 0xFF);
    sc_f[h][1] = d * (float)((scw >> (sh + 8)) & 0xFF);
    mn_f[h][0] = dmin * (float)((mnw >> sh) & 0xFF);
    mn_f[h][1] = dmin * (float)((mnw >> (sh + 8)) & 0xFF);
  }
#pragma unroll
  for (int sb = 0; sb < 8; ++sb) {
    const int j = sb >> 1, hi = sb & 1, jj = j >> 1;
    const uint32_t wa[4] = {q[jj][0].x, q[jj][0].y, q[jj][0].z, q[jj][0].w};
    const uint32_t wb[4] = {q[jj][1].x, q[jj][1].y, q[jj][1].z, q[jj][1].w};
    float c[NT][4];
    zero_c<NT>(c);
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      uint32_t b[NT][4];
      load_b<NT>(a, kg * 16 + sb * 2 + hf, g, t, b);
      uint32_t ua = wa[(j & 1) * 2 + hf], ub = wb[(j & 1) * 2 + hf];
      uint32_t a0, a1, a2, a3;
      if (hi == 0) {
        a0 = hsub2(lo02(ua), 0x64006400u); a1 = hsub2(lo02(ub), 0x64006400u);
        a2 = hsub2(lo02(ua >> 8), 0x64006400u); a3 = hsub2(lo02(ub >> 8), 0x64006400u);
      } else {
        a0 = hsub2(hi02(ua), 0x54005400u); a1 = hsub2(hi02(ub), 0x54005400u);
        a2 = hsub2(hi02(ua >> 8), 0x54005400u); a3 = hsub2(hi02(ub >> 8), 0x54005400u);
      }
      mma_hilo<NT>(c, a0, a1, a2, a3, b);
    }
    const int src = (lane & ~3) | (sb >> 1);
    float s_g = __shfl_sync(0xFFFFFFFFu, sc_f[0][sb & 1], src);
    float s_g8 = __shfl_sync(0xFFFFFFFFu, sc_f[1][sb & 1], src);
    float o_g = __shfl_sync(0xFFFFFFFFu, mn_f[0][sb & 1], src);
    float o_g8 = __shfl_sync(0xFFFFFFFFu, mn_f[1][sb & 1], src);
    const float* xs = a.xsum + (size_t)(kg * 8 + sb) * a.Mp;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float2 sx = __ldg(reinterpret_cast<const float2*>(xs + 8 * nt + 2 * t));
      acc[nt][0] = fmaf(s_g, c[nt][0], fmaf(-o_g, sx.x, acc[nt][0]));
      acc[nt][1] = fmaf(s_g, c[nt][1], fmaf(-o_g, sx.y, acc[nt][1]));
      acc[nt][2] = fmaf(s_g8, c[nt][2], fmaf(-o_g8, sx.x, acc[nt][2]));
      acc[nt][3] = fmaf(s_g8, c[nt][3], fmaf(-o_g8, sx.y, acc[nt][3]));
    }
  }
}

// Q6_K: sixteen 16-element scale groups per super-block, one MMA each.
template <int NT>
__device__ __forceinline__ void group_q6k(const GemvArgs& a, const uint8_t* tg, int kg, int lane,
                                          float (&acc)[NT][4]) {
  const int g = lane >> 2, t = lane & 3;
  uint4 qla[2], qlb[2], qhh[2];
  uint4 sc4[2];
  float d[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    qla[h] = ldg16(tg + h * 512 + lane * 16);
    qlb[h] = ldg16(tg + 1024 + h * 512 + lane * 16);
    qhh[h] = ldg16(tg + 2048 + h * 512 + lane * 16);
    sc4[h] = ldg16(tg + 3072 + (g + 8 * h) * 16);
    d[h] = fb::half_bits_to_float(__ldg(reinterpret_cast<const uint16_t*>(tg + 3328 + (g + 8 * h) * 2)));
  }
#pragma unroll
  for (int w = 0; w < 4; ++w) {  // (c = w / 2, u = w % 2)
    const uint32_t la[2] = {w == 0 ? qla[0].x : w == 1 ? qla[0].y : w == 2 ? qla[0].z : qla[0].w,
                            w == 0 ? qla[1].x : w == 1 ? qla[1].y : w == 2 ? qla[1].z : qla[1].w};
    const uint32_t lb[2] = {w == 0 ? qlb[0].x : w == 1 ? qlb[0].y : w == 2 ? qlb[0].z : qlb[0].w,
                            w == 0 ? qlb[1].x : w == 1 ? qlb[1].y : w == 2 ? qlb[1].z : qlb[1].w};
    const uint32_t hh[2] = {w == 0 ? qhh[0].x : w == 1 ? qhh[0].y : w == 2 ? qhh[0].z : qhh[0].w,
                            w == 0 ? qhh[1].x : w == 1 ? qhh[1].y : w == 2 ? qhh[1].z : qhh[1].w};
#pragma unroll
    for (int qsel = 0; qsel < 4; ++qsel) {
      const int grp = 8 * (w >> 1) + 2 * qsel + (w & 1);  // scale group inside the super-block
      uint32_t b[NT][4];
      load_b<NT>(a, kg * 16 + grp, g, t, b);
      uint32_t af[4];  // a0 (row g, bytes 0,2), a1 (row g+8), a2 (row g, bytes 1,3), a3
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t lw = (qsel & 1) ? lb[h] : la[h];
        if (qsel >= 2) lw >>= 4;
        uint32_t hw = hh[h];
        // two high bits of bytes (0,2): bits 2*qsel of each byte moved to bit 4
        uint32_t h02 = (qsel == 0 ? (hw << 4) : qsel == 1 ? (hw << 2) : qsel == 2 ? hw : (hw >> 2)) & 0x00300030u;
        uint32_t h13 = (qsel == 0 ? (hw >> 4) : qsel == 1 ? (hw >> 6) : qsel == 2 ? (hw >> 8) : (hw >> 10)) & 0x00300030u;
        uint32_t v02 = (lw & 0x000F000Fu) | h02 | 0x64006400u;
        uint32_t v13 = ((lw >> 8) & 0x000F000Fu) | h13 | 0x64006400u;
        af[h] = hsub2(v02, 0x64206420u);      // - (1024 + 32)
        af[2 + h] = hsub2(v13, 0x64206420u);
      }
      float c[NT][4];
      zero_c<NT>(c);
      mma_hilo<NT>(c, af[0], af[1], af[2], af[3], b);
      float s[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t word = (grp >> 2) == 0 ? sc4[h].x : (grp >> 2) == 1 ? sc4[h].y : (grp >> 2) == 2 ? sc4[h].z : sc4[h].w;
        int sv = (int)(int8_t)((word >> (8 * (grp & 3))) & 0xFF);
        s[h] = d[h] * (float)sv;
      }
      scale_add<NT>(acc, c, s[0], s[1]);
    }
  }
}

template <int TYPE, int NT>
__device__ __forceinline__ void process_tile(const GemvArgs& a, int tile, int warp, int lane,
                                             float (&acc)[NT][4]) {
  constexpr int TG = TYPE == FB200_Q4_0 ? 1152 : TYPE == FB200_Q8_0 ? 2176 : TYPE == FB200_Q4_K ? 2304 : 3360;
  const uint8_t* base = a.w + (size_t)tile * a.ngroups * TG;
  for (int kg = warp; kg < a.ngroups; kg += GEMV_WARPS) {
    const uint8_t* tg = base + (size_t)kg * TG;
    if (TYPE == FB200_Q4_0) group_q4_0<NT>(a, tg, kg, lane, acc);
    else if (TYPE == FB200_Q8_0) group_q8_0<NT>(a, tg, kg, lane, acc);
    else if (TYPE == FB200_Q4_K) group_q4k<NT>(a, tg, kg, lane, acc);
    else group_q6k<NT>(a, tg, kg, lane, acc);
  }
}

// EPI: 0 none, 1 residual(s), 2 SwiGLU pair
template <int TYPE, int NT, int EPI>
__global__ void __launch_bounds__(GEMV_THREADS)
qgemv_kernel(const GemvArgs a) {
  constexpr int NP = EPI == 2 ? 2 : 1;
  __shared__ float red[NP][GEMV_WARPS][NT * 8][16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int tile = blockIdx.x;
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    float acc[NT][4];
    zero_c<NT>(acc);
    process_tile<TYPE, NT>(a, tile + p * a.pair_tile_offset, warp, lane, acc);
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
    const int n = tile * 16 + r;
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
      out = v[0] + a.r1[idx];
      if (a.r2) out += a.r2[idx];
    } else {
      out = v[0];
    }
    a.y[idx] = out;
  }
}

// x[M, K] f32 -> fp16 MMA B-fragments [Kp/16][Mp][4 lanes t][hi x0 x2 x1 x3 | lo x0 x2 x1 x3],
// per-32 sums of the scaled values, and the power-of-two row scale.
__global__ void __launch_bounds__(256)
pack_x_kernel(const float* __restrict__ x, int M, int K, int Kp, int Mp, __half* __restrict__ xt,
              float* __restrict__ xsum, float* __restrict__ xscale) {
  const int m = blockIdx.x;
  __shared__ float wmax[8];
  float inv = 1.0f;
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
    inv = ldexpf(1.0f, -e);
    if (threadIdx.x == 0) xscale[m] = ldexpf(1.0f, e);
  } else if (threadIdx.x == 0) {
    xscale[m] = 1.0f;
  }
  const int quads = Kp >> 2;
  for (int q0 = 0; q0 < quads; q0 += 256) {
    const int q = q0 + threadIdx.x;
    float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
    const int k = q * 4;
    if (q < quads && m < M) {
      const float* xr = x + (size_t)m * K;
      if (k + 3 < K) {
        v0 = xr[k] * inv; v1 = xr[k + 1] * inv; v2 = xr[k + 2] * inv; v3 = xr[k + 3] * inv;
      } else {
        if (k < K) v0 = xr[k] * inv;
        if (k + 1 < K) v1 = xr[k + 1] * inv;
        if (k + 2 < K) v2 = xr[k + 2] * inv;
      }
    }
    float s = (v0 + v1) + (v2 + v3);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 4);
    if (q < quads) {
      __half2 h01 = __floats2half2_rn(v0, v2);
      __half2 h23 = __floats2half2_rn(v1, v3);
      float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
      __half2 l01 = __floats2half2_rn(v0 - f01.x, v2 - f01.y);
      __half2 l23 = __floats2half2_rn(v1 - f23.x, v3 - f23.y);
      uint4 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&h01);
      pk.y = *reinterpret_cast<uint32_t*>(&h23);
      pk.z = *reinterpret_cast<uint32_t*>(&l01);
      pk.w = *reinterpret_cast<uint32_t*>(&l23);
      const int kk = k >> 4, p = k & 15;
      *reinterpret_cast<uint4*>(xt + ((size_t)kk * Mp + m) * 32 + 2 * p) = pk;
      if ((threadIdx.x & 7) == 0) xsum[(size_t)(k >> 5) * Mp + m] = s;
    }
  }
}

template <int TYPE, int NT>
void launch_epi(const GemvArgs& a, int epi, int grid, cudaStream_t st) {
  if (epi == FB200_EPI_SWIGLU) qgemv_kernel<TYPE, NT, 2><<<grid, GEMV_THREADS, 0, st>>>(a);
  else if (epi == FB200_EPI_RESIDUAL) qgemv_kernel<TYPE, NT, 1><<<grid, GEMV_THREADS, 0, st>>>(a);
  else qgemv_kernel<TYPE, NT, 0><<<grid, GEMV_THREADS, 0, st>>>(a);
}

template <int TYPE>
void launch_nt(const GemvArgs& a, int nt, int epi, int grid, cudaStream_t st) {
  if (nt == 1) launch_epi<TYPE, 1>(a, epi, grid, st);
  else if (nt == 2) launch_epi<TYPE, 2>(a, epi, grid, st);
  else launch_epi<TYPE, 4>(a, epi, grid, st);
}

}  // namespace

// Bytes of packed-activation scratch needed for an [M<=32, K] product.
size_t fb200_xpack_bytes(int mp, uint64_t kp) {
  return (size_t)(kp / 16) * mp * 32 * sizeof(__half) + (size_t)(kp / 32) * mp * sizeof(float) +
         (size_t)mp * sizeof(float) + 256;
}

// y[m0 .. m0+mc) = x . W^T for a chunk of at most 32 activation rows, using `scratch`.
int fb200_qgemv_chunk(fb200_device* dev, const fb200_qmatrix* w, const float* x, int mc, float* y,
                      int epi, const float* r1, const float* r2, void* scratch) {
  TileGeom geo;
  tile_geom(w->type, &geo);
  const int nt = mc <= 8 ? 1 : mc <= 16 ? 2 : 4;
  const int mp = nt * 8;
  const uint64_t kp = (uint64_t)w->ngroups * geo.group_elems;
  __half* xt = reinterpret_cast<__half*>(scratch);
  size_t off = (size_t)(kp / 16) * mp * 32 * sizeof(__half);
  float* xsum = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + off);
  off += (size_t)(kp / 32) * mp * sizeof(float);
  float* xscale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + off);
  pack_x_kernel<<<mp, 256, 0, dev->stream>>>(x, mc, (int)w->k, (int)kp, mp, xt, xsum, xscale);
  FB_LAUNCH_CHECK(dev);
  GemvArgs a;
  a.w = w->data; a.xt = xt; a.xsum = xsum; a.xscale = xscale; a.y = y; a.r1 = r1; a.r2 = r2;
  a.M = mc; a.Mp = mp; a.ngroups = w->ngroups;
  int grid = w->ntiles;
  a.n_out = (int)w->n;
  a.pair_tile_offset = 0;
  if (epi == FB200_EPI_SWIGLU) {
    grid = w->ntiles / 2;
    a.n_out = (int)(w->n / 2);
    a.pair_tile_offset = w->ntiles / 2;
  }
  switch (w->type) {
    case FB200_Q4_0: launch_nt<FB200_Q4_0>(a, nt, epi, grid, dev->stream); break;
    case FB200_Q8_0: launch_nt<FB200_Q8_0>(a, nt, epi, grid, dev->stream); break;
    case FB200_Q4_K: launch_nt<FB200_Q4_K>(a, nt, epi, grid, dev->stream); break;
    default: launch_nt<FB200_Q6_K>(a, nt, epi, grid, dev->stream); break;
  }
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}
