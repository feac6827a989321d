// Device helpers shared by the quantised product kernels: PTX wrappers (mma.sync, mbarrier,
// cp.async.bulk, griddepcontrol) and the per-format expansion of one tile-group into
// mma.m16n8k16 A fragments.
#pragma once

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
  int nunits;            // work units: tiles, or (gate, up) tile pairs
  int* status;           // device status word (bounded waits that ran out are recorded here)
};

// ---- PTX wrappers: mbarrier, bulk copy, programmatic dependent launch -------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Bounded wait: gives up after ~2^22 polls, records it in the status word and lets the kernel
// run to its end (results are then invalid, the host sees a non-zero status).
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int* status) {
  for (int it = 0; it < (1 << 22); ++it) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return;
  }
  if (status) atomicExch(status, FB200_ERR_TIMEOUT);
}
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }


__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
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

// 16-byte load from a shared-memory stage
__device__ __forceinline__ uint4 ldg16(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
  return v;
}
__device__ __forceinline__ uint2 lds8(const uint8_t* p) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(smem_u32(p)));
  return v;
}
__device__ __forceinline__ uint16_t lds2(const uint8_t* p) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(smem_u32(p)));
  return v;
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
  uint2 dg = lds8(tg + 1024 + g * 8);
  uint2 dg8 = lds8(tg + 1024 + (g + 8) * 8);
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
  uint2 dg = lds8(tg + 2048 + g * 8);
  uint2 dg8 = lds8(tg + 2048 + (g + 8) * 8);
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
    d[h] = fb::half_bits_to_float(lds2(tg + 3328 + (g + 8 * h) * 2));
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

}  // namespace
