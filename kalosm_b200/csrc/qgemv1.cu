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
//  * the prologue turns x into MMA B fragments in shared memory once per CTA: optional
//    residual add and RMSNorm (so the norm needs no kernel of its own), a power-of-two row
//    scale, then a hi + lo pair of fp16 values per element (about 22 mantissa bits) and the
//    per-32 sums Q4_K's offsets need;
//  * quants are expanded to exact fp16 integers with logic ops and multiplied on the tensor
//    cores (mma.sync.m16n8k16, fp32 accumulate). With one activation row the 8 MMA columns are
//    otherwise idle, so hi sits in column 0 and lo in column 1 and one MMA covers both;
//  * block scales are applied to the fp32 partial sums per 16/32-element group.
//
// Replaces the reference's qgemv kernels (fusor-ml/tile-ir-kernels/src/kernels/qgemv.rs:356-678,
// qgemv_q6k.rs:84-385), their SwiGLU and residual epilogues
// (fusor-ml/core/src/quantized/matmul/mod.rs:435-439, 666-722) and the fused RMSNorm cluster
// (fusor-ml/core/src/composite/rms_norm_fused.rs:10-54) in front of a projection.
#include "qgemv_common.cuh"

namespace {

struct Gemv1Args {
  const uint8_t* w;
  const float* x;       // [K]
  const float* xres;    // optional [K]: v = x + xres
  const float* norm_w;  // optional [K]: activation = v / sqrt(mean(v^2) + eps) * norm_w
  float eps;
  int K, Kp;            // logical and padded (ngroups * group_elems) inner size
  float* y;             // [n_out]
  const float* r1;
  const float* r2;
  int n_out, ngroups, nunits, pair_tile_offset, stages;
  int* status;
};

template <int TYPE>
struct G1 {
  static constexpr int TG = TYPE == FB200_Q4_0 ? 1152 : TYPE == FB200_Q8_0 ? 2176 : TYPE == FB200_Q4_K ? 2304 : 3360;
  static constexpr int STRIDE = (TG + 127) / 128 * 128;
};

// ---- one activation row on an 8-column MMA -----------------------------------------------------
// Four consecutive scale groups (j = 0..3) of a tile-group form a chain of MMAs into one
// accumulator: the B operand of the MMAs of group j is non-zero only in columns 2j (hi half of
// x) and 2j+1 (lo half), so after the chain lane t of every quad holds, for rows g and g+8,
// the integer-weight dot product of scale group t. Each lane therefore decodes and applies the
// scale of ONE group per chain (a quarter of the scale work per lane), and each lane loads B
// data for one group only: lane (g, t) supplies group g/2, half g%2.
__device__ __forceinline__ uint2 load_bx(const uint8_t* xh, int kk, int g, int t) {
  return *reinterpret_cast<const uint2*>(xh + kk * 64 + t * 16 + (g & 1) * 8);
}

__device__ __forceinline__ uint4 lds16(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }

__device__ __forceinline__ void mma1(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                     uint2 v, bool mine) {
  mma16816(c, a0, a1, a2, a3, mine ? v.x : 0u, mine ? v.y : 0u);
}

__device__ __forceinline__ void group1_q4_0(const uint8_t* xh, const uint8_t* tg, int kg, int lane,
                                            float& acc_g, float& acc_g8) {
  const int g = lane >> 2, t = lane & 3, jb = g >> 1;
  const uint4 qa = lds16(tg + lane * 16);
  const uint4 qb = lds16(tg + 512 + lane * 16);
  const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w};
  const uint32_t wb[4] = {qb.x, qb.y, qb.z, qb.w};
  // this lane's block is t: its scales for rows g and g+8
  const float d_g = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 1024 + g * 8 + t * 2));
  const float d_g8 = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 1024 + (g + 8) * 8 + t * 2));
  const uint2 v0 = load_bx(xh, (kg * 4 + jb) * 2, g, t);
  const uint2 v1 = load_bx(xh, (kg * 4 + jb) * 2 + 1, g, t);
  float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int blk = 0; blk < 4; ++blk) {
    const bool mine = jb == blk;
    mma1(c, hsub2(lo02(wa[blk]), 0x64086408u), hsub2(lo02(wb[blk]), 0x64086408u),
         hsub2(lo02(wa[blk] >> 8), 0x64086408u), hsub2(lo02(wb[blk] >> 8), 0x64086408u), v0, mine);
    mma1(c, hsub2(hi02(wa[blk]), 0x54805480u), hsub2(hi02(wb[blk]), 0x54805480u),
         hsub2(hi02(wa[blk] >> 8), 0x54805480u), hsub2(hi02(wb[blk] >> 8), 0x54805480u), v1, mine);
  }
  acc_g = fmaf(d_g, c[0] + c[1], acc_g);
  acc_g8 = fmaf(d_g8, c[2] + c[3], acc_g8);
}

__device__ __forceinline__ void group1_q8_0(const uint8_t* xh, const uint8_t* tg, int kg, int lane,
                                            float& acc_g, float& acc_g8) {
  const int g = lane >> 2, t = lane & 3, jb = g >> 1;
  uint4 q[2][2];
#pragma unroll
  for (int p = 0; p < 2; ++p)
#pragma unroll
    for (int h = 0; h < 2; ++h) q[p][h] = lds16(tg + (p * 2 + h) * 512 + lane * 16);
  const float d_g = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 2048 + g * 8 + t * 2));
  const float d_g8 = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 2048 + (g + 8) * 8 + t * 2));
  const uint2 v0 = load_bx(xh, (kg * 4 + jb) * 2, g, t);
  const uint2 v1 = load_bx(xh, (kg * 4 + jb) * 2 + 1, g, t);
  float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int blk = 0; blk < 4; ++blk) {
    const bool mine = jb == blk;
    const int p = blk >> 1;
    const uint32_t wa[4] = {q[p][0].x, q[p][0].y, q[p][0].z, q[p][0].w};
    const uint32_t wb[4] = {q[p][1].x, q[p][1].y, q[p][1].z, q[p][1].w};
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const uint32_t xa = wa[(blk & 1) * 2 + hf] ^ 0x80808080u;
      const uint32_t xb = wb[(blk & 1) * 2 + hf] ^ 0x80808080u;
      mma1(c, hsub2(__byte_perm(xa, 0x64646464u, 0x4240), 0x64806480u),
           hsub2(__byte_perm(xb, 0x64646464u, 0x4240), 0x64806480u),
           hsub2(__byte_perm(xa, 0x64646464u, 0x4341), 0x64806480u),
           hsub2(__byte_perm(xb, 0x64646464u, 0x4341), 0x64806480u), hf ? v1 : v0, mine);
    }
  }
  acc_g = fmaf(d_g, c[0] + c[1], acc_g);
  acc_g8 = fmaf(d_g8, c[2] + c[3], acc_g8);
}

// Q4_K: chain ch covers sub-blocks 4ch .. 4ch+3 (pairs of sub-blocks share the qs bytes: even
// ones are the low nibbles, odd ones the high nibbles). Lane t owns sub-block 4ch + t.
__device__ __forceinline__ void group1_q4k(const uint8_t* xh, const float* xsum, const uint8_t* tg,
                                           int kg, int lane, float& acc_g, float& acc_g8) {
  const int g = lane >> 2, t = lane & 3, jb = g >> 1;
  // 6-bit scales / offsets of both chains' sub-blocks t and 4 + t, rows g and g+8
  float sc_f[2][2], mn_f[2][2];  // [row half][chain]
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
  for (int ch = 0; ch < 2; ++ch) {
    const uint4 qa = lds16(tg + (ch * 2) * 512 + lane * 16);
    const uint4 qb = lds16(tg + (ch * 2 + 1) * 512 + lane * 16);
    const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w};
    const uint32_t wb[4] = {qb.x, qb.y, qb.z, qb.w};
    const int kk0 = kg * 16 + (ch * 4 + jb) * 2;
    const uint2 v0 = load_bx(xh, kk0, g, t);
    const uint2 v1 = load_bx(xh, kk0 + 1, g, t);
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool mine = jb == j;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const uint32_t ua = wa[(j >> 1) * 2 + hf], ub = wb[(j >> 1) * 2 + hf];
        if ((j & 1) == 0)
          mma1(c, hsub2(lo02(ua), 0x64006400u), hsub2(lo02(ub), 0x64006400u),
               hsub2(lo02(ua >> 8), 0x64006400u), hsub2(lo02(ub >> 8), 0x64006400u), hf ? v1 : v0, mine);
        else
          mma1(c, hsub2(hi02(ua), 0x54005400u), hsub2(hi02(ub), 0x54005400u),
               hsub2(hi02(ua >> 8), 0x54005400u), hsub2(hi02(ub >> 8), 0x54005400u), hf ? v1 : v0, mine);
      }
    }
    const float sx = xsum[kg * 8 + ch * 4 + t];
    acc_g = fmaf(sc_f[0][ch], c[0] + c[1], fmaf(-mn_f[0][ch], sx, acc_g));
    acc_g8 = fmaf(sc_f[1][ch], c[2] + c[3], fmaf(-mn_f[1][ch], sx, acc_g8));
  }
}

// Q6_K: chain w = (c = w/2, u = w%2) covers the four groups 8c + 2*qsel + u, qsel = 0..3;
// lane t owns qsel = t.
__device__ __forceinline__ void group1_q6k(const uint8_t* xh, const uint8_t* tg, int kg, int lane,
                                           float& acc_g, float& acc_g8) {
  const int g = lane >> 2, t = lane & 3, jb = g >> 1;
  uint4 qla[2], qlb[2], qhh[2], sc4[2];
  float d[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    qla[h] = lds16(tg + h * 512 + lane * 16);
    qlb[h] = lds16(tg + 1024 + h * 512 + lane * 16);
    qhh[h] = lds16(tg + 2048 + h * 512 + lane * 16);
    sc4[h] = lds16(tg + 3072 + (g + 8 * h) * 16);
    d[h] = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 3328 + (g + 8 * h) * 2));
  }
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const uint32_t la[2] = {w == 0 ? qla[0].x : w == 1 ? qla[0].y : w == 2 ? qla[0].z : qla[0].w,
                            w == 0 ? qla[1].x : w == 1 ? qla[1].y : w == 2 ? qla[1].z : qla[1].w};
    const uint32_t lb[2] = {w == 0 ? qlb[0].x : w == 1 ? qlb[0].y : w == 2 ? qlb[0].z : qlb[0].w,
                            w == 0 ? qlb[1].x : w == 1 ? qlb[1].y : w == 2 ? qlb[1].z : qlb[1].w};
    const uint32_t hh[2] = {w == 0 ? qhh[0].x : w == 1 ? qhh[0].y : w == 2 ? qhh[0].z : qhh[0].w,
                            w == 0 ? qhh[1].x : w == 1 ? qhh[1].y : w == 2 ? qhh[1].z : qhh[1].w};
    const uint2 v = load_bx(xh, kg * 16 + 8 * (w >> 1) + 2 * jb + (w & 1), g, t);
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int qsel = 0; qsel < 4; ++qsel) {
      uint32_t af[4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t lw = (qsel & 1) ? lb[h] : la[h];
        if (qsel >= 2) lw >>= 4;
        const uint32_t hw = hh[h];
        const uint32_t h02 = (qsel == 0 ? (hw << 4) : qsel == 1 ? (hw << 2) : qsel == 2 ? hw : (hw >> 2)) & 0x00300030u;
        const uint32_t h13 = (qsel == 0 ? (hw >> 4) : qsel == 1 ? (hw >> 6) : qsel == 2 ? (hw >> 8) : (hw >> 10)) & 0x00300030u;
        af[h] = hsub2((lw & 0x000F000Fu) | h02 | 0x64006400u, 0x64206420u);
        af[2 + h] = hsub2(((lw >> 8) & 0x000F000Fu) | h13 | 0x64006400u, 0x64206420u);
      }
      mma1(c, af[0], af[1], af[2], af[3], v, jb == qsel);
    }
    // scale byte 8c + 2t + u of this lane's group, rows g and g+8
    float s[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t wlo = (w >> 1) ? sc4[h].z : sc4[h].x, whi = (w >> 1) ? sc4[h].w : sc4[h].y;
      const uint32_t word = (t >> 1) ? whi : wlo;
      const int sv = (int)(int8_t)((word >> (8 * (2 * (t & 1) + (w & 1)))) & 0xFF);
      s[h] = d[h] * (float)sv;
    }
    acc_g = fmaf(s[0], c[0] + c[1], acc_g);
    acc_g8 = fmaf(s[1], c[2] + c[3], acc_g8);
  }
}

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sh, int nwarps) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float u = __shfl_xor_sync(0xFFFFFFFFu, v, o);
    v = is_max ? fmaxf(v, u) : v + u;
  }
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sh[0];
  for (int i = 1; i < nwarps; ++i) r = is_max ? fmaxf(r, sh[i]) : r + sh[i];
  __syncthreads();
  return r;
}

// EPI: 0 none, 1 residual(s), 2 SwiGLU pair. W = warps per CTA.
template <int TYPE, int EPI, int W>
__global__ void __launch_bounds__(W * 32)
qgemv1_kernel(const Gemv1Args a) {
  using R = G1<TYPE>;
  constexpr int NP = EPI == 2 ? 2 : 1;
  constexpr int THREADS = W * 32;
  extern __shared__ __align__(128) uint8_t smem[];
  const int S = a.stages;
  uint8_t* ring = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + W * S * R::STRIDE);
  uint8_t* xh = smem + W * S * R::STRIDE + W * S * 8;  // multiple of 64 bytes
  float* xsum = reinterpret_cast<float*>(xh + (size_t)a.Kp * 4);
  float* red = xsum + a.Kp / 32;   // [NP][W][16]
  float* tmp = red + NP * W * 16;  // [W] block reductions

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* my_ring = ring + warp * S * R::STRIDE;
  const uint32_t my_bar = smem_u32(bars + warp * S);

  pdl_launch_dependents();
  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(my_bar + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  const int gw = a.ngroups > warp ? (a.ngroups - warp + W - 1) / W : 0;
  const int my_units = a.nunits > (int)blockIdx.x ? (a.nunits - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int per_unit = NP * gw;
  const int n_items = my_units * per_unit;
  auto issue = [&](int i, int st) {
    const int j = i / per_unit, rem = i - j * per_unit;
    const int p = rem / gw, kk = rem - p * gw;
    const int tile = (int)blockIdx.x + j * (int)gridDim.x + p * a.pair_tile_offset;
    const int kg = warp + W * kk;
    const uint8_t* src = a.w + ((size_t)tile * a.ngroups + kg) * R::TG;
    mbar_expect_tx(my_bar + 8 * st, R::TG);
    bulk_g2s(smem_u32(my_ring + st * R::STRIDE), src, R::TG, my_bar + 8 * st);
  };
  if (lane == 0) {
    const int pre = n_items < S ? n_items : S;
    for (int i = 0; i < pre; ++i) issue(i, i);
  }
  // only weights were touched so far; x comes from the kernel before this one
  pdl_wait();

  // ---- activation prologue: (residual) -> (RMSNorm) -> power-of-two scale -> hi/lo fragments
  float ss = 0.f, amax = 0.f;
  for (int k = threadIdx.x; k < a.K; k += THREADS) {
    float v = a.x[k];
    if (a.xres) v += a.xres[k];
    ss = fmaf(v, v, ss);
    if (!a.norm_w) amax = fmaxf(amax, fabsf(v));
  }
  float rms = 1.f;
  if (a.norm_w) {
    // rms_norm_fused_cpu_impl, fusor-ml/fusor/src/composite/normalization.rs:404-461
    ss = block_reduce(ss, false, tmp, W);
    rms = sqrtf(ss / (float)a.K + a.eps);
    for (int k = threadIdx.x; k < a.K; k += THREADS) {
      float v = a.x[k];
      if (a.xres) v += a.xres[k];
      amax = fmaxf(amax, fabsf((v / rms) * a.norm_w[k]));
    }
  }
  amax = block_reduce(amax, true, tmp, W);
  int e = 0;
  if (amax > 0.f && amax < 3.0e38f) frexpf(amax, &e);
  const float inv = ldexpf(1.0f, -e), xscale = ldexpf(1.0f, e);
  for (int q0 = 0; q0 < (a.Kp >> 2); q0 += THREADS) {
    const int q = q0 + threadIdx.x;  // Kp / 4 is a multiple of 32, so whole warps stay together
    const int k = q * 4;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (q < (a.Kp >> 2)) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (k + i < a.K) {
          float u = a.x[k + i];
          if (a.xres) u += a.xres[k + i];
          if (a.norm_w) u = (u / rms) * a.norm_w[k + i];
          v[i] = u * inv;
        }
    }
    float s = (v[0] + v[1]) + (v[2] + v[3]);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 4);
    if (q < (a.Kp >> 2)) {
      __half2 h01 = __floats2half2_rn(v[0], v[2]);
      __half2 h23 = __floats2half2_rn(v[1], v[3]);
      float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
      __half2 l01 = __floats2half2_rn(v[0] - f01.x, v[2] - f01.y);
      __half2 l23 = __floats2half2_rn(v[1] - f23.x, v[3] - f23.y);
      uint4 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&h01);
      pk.y = *reinterpret_cast<uint32_t*>(&h23);
      pk.z = *reinterpret_cast<uint32_t*>(&l01);
      pk.w = *reinterpret_cast<uint32_t*>(&l23);
      *reinterpret_cast<uint4*>(xh + (size_t)k * 4) = pk;  // chunk k/16 at 64 B, quad (k%16)/4 at 16 B
      if ((threadIdx.x & 7) == 0) xsum[k >> 5] = s;
    }
  }
  __syncthreads();

  int item = 0, st = 0;
  uint32_t phase = 0;
  for (int j = 0; j < my_units; ++j) {
    const int unit = (int)blockIdx.x + j * (int)gridDim.x;
    if (j > 0) __syncthreads();  // the previous unit's reduction has read `red`
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      float acc_g = 0.f, acc_g8 = 0.f;
      for (int kk = 0; kk < gw; ++kk, ++item) {
        mbar_wait(my_bar + 8 * st, phase, a.status);
        const uint8_t* tg = my_ring + st * R::STRIDE;
        const int kg = warp + W * kk;
        if (TYPE == FB200_Q4_0) group1_q4_0(xh, tg, kg, lane, acc_g, acc_g8);
        else if (TYPE == FB200_Q8_0) group1_q8_0(xh, tg, kg, lane, acc_g, acc_g8);
        else if (TYPE == FB200_Q4_K) group1_q4k(xh, xsum, tg, kg, lane, acc_g, acc_g8);
        else group1_q6k(xh, tg, kg, lane, acc_g, acc_g8);
        __syncwarp();  // every lane has consumed the stage before it is refilled
        if (lane == 0 && item + S < n_items) issue(item + S, st);
        if (++st == S) { st = 0; phase ^= 1u; }
      }
      // lane t accumulated the scale groups it owns: sum over the quad
      acc_g += __shfl_xor_sync(0xFFFFFFFFu, acc_g, 1);
      acc_g += __shfl_xor_sync(0xFFFFFFFFu, acc_g, 2);
      acc_g8 += __shfl_xor_sync(0xFFFFFFFFu, acc_g8, 1);
      acc_g8 += __shfl_xor_sync(0xFFFFFFFFu, acc_g8, 2);
      if (t == 0) {
        red[(p * W + warp) * 16 + g] = acc_g;
        red[(p * W + warp) * 16 + g + 8] = acc_g8;
      }
    }
    __syncthreads();
    if (threadIdx.x < 16) {
      const int r = threadIdx.x;
      const int n = unit * 16 + r;
      if (n < a.n_out) {
        float v[NP];
#pragma unroll
        for (int p = 0; p < NP; ++p) {
          float s = 0.f;
          for (int w = 0; w < W; ++w) s += red[(p * W + w) * 16 + r];
          v[p] = s * xscale;
        }
        float out;
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
        a.y[n] = out;
      }
    }
  }
}

constexpr int SMEM_LIMIT = 227 * 1024;

template <int TYPE, int EPI, int W>
size_t gemv1_smem(int stages, int kp) {
  constexpr int NP = EPI == 2 ? 2 : 1;
  return (size_t)W * stages * G1<TYPE>::STRIDE + (size_t)W * stages * 8 + (size_t)kp * 4 +
         (size_t)kp / 32 * 4 + (size_t)NP * W * 16 * 4 + (size_t)W * 4 + 64;
}

template <int TYPE, int EPI, int W>
int launch_w(fb200_device* dev, Gemv1Args& a, int ctas_per_sm) {
  auto kern = qgemv1_kernel<TYPE, EPI, W>;
  static bool configured[64] = {false};
  if (!configured[dev->ordinal & 63]) {
    FB_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
    configured[dev->ordinal & 63] = true;
  }
  int grid = dev->sm_count * ctas_per_sm;
  if (grid > a.nunits) grid = a.nunits;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(W * 32);
  cfg.dynamicSmemBytes = gemv1_smem<TYPE, EPI, W>(a.stages, a.Kp);
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

// Two 8-warp CTAs per SM when their rings and the activation fragments fit twice in shared
// memory, otherwise one 16-warp CTA; the ring depth takes what is left, up to 6 stages.
template <int TYPE, int EPI>
int launch_cfg(fb200_device* dev, Gemv1Args& a) {
  const int budget2 = (SMEM_LIMIT - 2048) / 2;
  for (int s = 6; s >= 2; --s)
    if ((int)gemv1_smem<TYPE, EPI, 8>(s, a.Kp) <= budget2) {
      a.stages = s;
      return launch_w<TYPE, EPI, 8>(dev, a, 2);
    }
  for (int s = 6; s >= 1; --s)
    if ((int)gemv1_smem<TYPE, EPI, 16>(s, a.Kp) <= SMEM_LIMIT - 1024) {
      a.stages = s;
      return launch_w<TYPE, EPI, 16>(dev, a, 1);
    }
  return fb200_fail(dev, FB200_ERR_CAPACITY, "qgemv1: K = %d does not fit in shared memory", a.K);
}

template <int TYPE>
int launch_epi1(fb200_device* dev, Gemv1Args& a, int epi) {
  if (epi == FB200_EPI_SWIGLU) return launch_cfg<TYPE, 2>(dev, a);
  if (epi == FB200_EPI_RESIDUAL) return launch_cfg<TYPE, 1>(dev, a);
  return launch_cfg<TYPE, 0>(dev, a);
}

}  // namespace

// Largest K the single-row kernel takes (activation fragments live in shared memory).
bool fb200_qgemv1_fits(const fb200_qmatrix* w) {
  TileGeom geo;
  if (!tile_geom(w->type, &geo)) return false;
  const uint64_t kp = (uint64_t)w->ngroups * geo.group_elems;
  return kp * 4 + kp / 8 + 16 * 3456 + 4096 <= (uint64_t)SMEM_LIMIT;
}

// y[n_out] = epilogue(W . act(x)); act = optional residual add + RMSNorm (norm_w != null).
int fb200_qgemv1(fb200_device* dev, const fb200_qmatrix* w, const float* x, const float* xres,
                 const float* norm_w, float eps, float* y, int epi, const float* r1,
                 const float* r2) {
  TileGeom geo;
  tile_geom(w->type, &geo);
  Gemv1Args a;
  a.w = w->data; a.x = x; a.xres = xres; a.norm_w = norm_w; a.eps = eps;
  a.K = (int)w->k; a.Kp = w->ngroups * geo.group_elems;
  a.y = y; a.r1 = r1; a.r2 = r2;
  a.ngroups = w->ngroups; a.nunits = w->ntiles; a.n_out = (int)w->n; a.pair_tile_offset = 0;
  a.stages = 2; a.status = dev->status;
  if (epi == FB200_EPI_SWIGLU) {
    a.nunits = w->ntiles / 2;
    a.n_out = (int)(w->n / 2);
    a.pair_tile_offset = w->ntiles / 2;
  }
  switch (w->type) {
    case FB200_Q4_0: return launch_epi1<FB200_Q4_0>(dev, a, epi);
    case FB200_Q8_0: return launch_epi1<FB200_Q8_0>(dev, a, epi);
    case FB200_Q4_K: return launch_epi1<FB200_Q4_K>(dev, a, epi);
    default: return launch_epi1<FB200_Q6_K>(dev, a, epi);
  }
}
