// Prefill product (M > 32 activation rows) on the 5th-generation tensor cores: tcgen05.mma with
// the accumulator in tensor memory (TMEM).
//
// Bound: tensor cores (2 M N K flops). Replaces the reference's tiled quantised matmul
// (fusor-ml/tile-ir-kernels/src/kernels/qmatmul.rs:237-349) for large M, where the small-batch
// kernels would re-read W once per 32 rows.
//
// One CTA computes a 128 (weight rows) x 128 or 256 (activation rows) tile of Y^T = W . X^T:
//  * W stays quantised in HBM. The raw tile-groups of the CTA's 8 row-tiles for one K group are
//    brought to shared memory by 1-D TMA bulk copies (double-buffered, one K group ahead);
//    warp w dequantises row-tile w to fp16 in registers (byte -> 1024 + byte by a byte permute,
//    exact subtraction, one fused multiply-add with block scale and offset) and stores it into
//    the A operand buffer in the canonical K-major core-matrix layout of the MMA (8 rows x 16
//    bytes per core matrix, no swizzle).
//  * X is converted once per call to fp16 rows scaled by a power of two; its 128/256 x 64 tile goes
//    to the B operand buffer with 16-byte cp.async copies in the same layout.
//  * A single thread issues four tcgen05.mma (M = 128, N = 128 or 256, K = 16, kind::f16, fp32
//    accumulate) per 64-wide K block; tcgen05.commit signals an mbarrier when the block's MMAs
//    have read their operands, which frees the buffer for the block after next, so conversion
//    and tensor-core work overlap (two operand stages).
//  * Epilogue: tcgen05.ld brings the fp32 accumulator out of TMEM (each warp its 32
//    lanes), rows are scaled back and written, optionally with the residual adds.
// Every wait is bounded (2^22 polls): on a time-out the status word is set and the CTA goes on
// to release its TMEM columns and exit.
#include <cstdlib>

#include "qgemv_common.cuh"

int fb200_ensure(fb200_device* dev, void** buf, size_t* cur, size_t bytes);

namespace {

constexpr int TC_THREADS = 256;
constexpr int BN = 128;  // weight rows per CTA tile  (M of the MMA)
// activation rows per CTA tile (N of the MMA): template parameter BM = 128 or 256
constexpr int BK = 64;   // K elements per operand stage (four K = 16 MMAs)
constexpr int A_BYTES = BN * BK * 2;              // one A stage
constexpr int CORE_LBO = 128;                     // bytes between core matrices adjacent in K
constexpr int CORE_SBO = (BK / 8) * 128;          // bytes between 8-row groups
constexpr int RAW_STRIDE = 3456;                  // largest tile-group, rounded up to 128
constexpr int RAW_BYTES = 8 * RAW_STRIDE;
constexpr int TC_STAGES = 3;                      // operand stages: convert / copy ahead of the MMAs
template <int BM>
struct Tc {
  static constexpr int B_BYTES = BM * BK * 2;               // one B stage
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int SMEM = TC_STAGES * STAGE + 2 * RAW_BYTES + 128;
  static constexpr int TMEM_COLS = BM;                      // fp32 accumulator columns
  // instruction descriptor: fp32 accumulator, fp16 A and B, both K-major, N = BM, M = BN
  static constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BM >> 3) << 17) | ((uint32_t)(BN >> 4) << 24);
};

struct TcArgs {
  const uint8_t* w;      // tiled weights
  const __half* xh;      // [Mp, K] fp16 activations (rows >= M are zero)
  const float* xscale;   // [Mp] power-of-two scale of each row
  float* y;              // [M, N]
  const float* r1;       // optional residuals [M, N]
  const float* r2;
  int M, N, K;
  int ngroups, ntiles, type, tgb, group_elems;
  int* status;
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ uint32_t h2u(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u2h(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t lds4(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ uint4 lds16(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }

// Four unsigned bytes -> four fp16 values ((1024 + byte) - centre) * scale + offset, as two half2.
__device__ __forceinline__ uint2 deq4(uint32_t w, __half2 centre, __half2 scale, __half2 offset) {
  const __half2 v01 = __hsub2(u2h(__byte_perm(w, 0x64646464u, 0x4140)), centre);
  const __half2 v23 = __hsub2(u2h(__byte_perm(w, 0x64646464u, 0x4342)), centre);
  return make_uint2(h2u(__hfma2(v01, scale, offset)), h2u(__hfma2(v23, scale, offset)));
}

// Shared-memory matrix descriptor of a K-major operand without swizzle: start address, leading
// (K direction) and stride (row-group direction) byte offsets in 16-byte units, descriptor
// version 1.
__device__ __forceinline__ uint64_t operand_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(CORE_LBO >> 4) << 16) |
         ((uint64_t)(CORE_SBO >> 4) << 32) | (1ull << 46);
}

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Row-tile `tile` of one K group: the four registers of 32-element chunk c for lane (g, t) --
// bytes of rows g / g + 8, elements 4t.. and 16 + 4t.. -- dequantised and stored into operand
// stage `abuf` at rows 16 * wrow + g (+ 8), K offset 32 * cib (chunk inside the 64-wide block).
struct RowScales {
  float sc[2][2], mn[2][2];  // Q4_K: [row half][sub-block t + 4 i]
  uint4 q6[2];               // Q6_K: scale bytes of rows g, g + 8
  float d[2];                // Q6_K: super-block scale
};

__device__ __forceinline__ void store_chunk(uint8_t* abuf, int wrow, int g, int t, int cib, uint2 lo_g, uint2 lo_g8,
                                            uint2 hi_g, uint2 hi_g8) {
  uint8_t* base = abuf + (2 * wrow) * CORE_SBO + g * 16 + (t & 1) * 8;
  const int klo = (4 * cib + (t >> 1)) * CORE_LBO, khi = (4 * cib + 2 + (t >> 1)) * CORE_LBO;
  *reinterpret_cast<uint2*>(base + klo) = lo_g;
  *reinterpret_cast<uint2*>(base + CORE_SBO + klo) = lo_g8;
  *reinterpret_cast<uint2*>(base + khi) = hi_g;
  *reinterpret_cast<uint2*>(base + CORE_SBO + khi) = hi_g8;
}

__device__ __forceinline__ void prepare_scales(int type, const uint8_t* tg, int g, int t, RowScales& S) {
  if (type == FB200_Q4_K) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint4 hd = lds16(tg + 2048 + (g + 8 * h) * 16);
      const float d = fb::half_bits_to_float((uint16_t)(hd.x & 0xFFFF));
      const float dmin = fb::half_bits_to_float((uint16_t)(hd.x >> 16));
      const uint32_t s0 = hd.y, s1 = hd.z, s2 = hd.w;
      const uint32_t scB = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
      const uint32_t mnB = ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u);
      const int sh = 8 * t;
      S.sc[h][0] = d * (float)((s0 >> sh) & 0x3F);
      S.mn[h][0] = dmin * (float)((s1 >> sh) & 0x3F);
      S.sc[h][1] = d * (float)((scB >> sh) & 0xFF);
      S.mn[h][1] = dmin * (float)((mnB >> sh) & 0xFF);
    }
  } else if (type == FB200_Q6_K) {
    S.q6[0] = lds16(tg + 3072 + g * 16);
    S.q6[1] = lds16(tg + 3072 + (g + 8) * 16);
    S.d[0] = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 3328 + g * 2));
    S.d[1] = fb::half_bits_to_float(*reinterpret_cast<const uint16_t*>(tg + 3328 + (g + 8) * 2));
  }
}

// chunk c of the tile-group (32 elements: c < 4 for Q4_0 / Q8_0, c < 8 for the K-quants)
__device__ __forceinline__ void dequant_chunk(int type, const uint8_t* tg, int c, int lane, const RowScales& S,
                                              uint8_t* abuf, int wrow, int cib) {
  const int g = lane >> 2, t = lane & 3;
  const __half2 zero2 = __float2half2_rn(0.f);
  if (type == FB200_Q4_K) {
    const int pair = c >> 1, hi = c & 1, ch = pair >> 1, ps = pair & 1;
    const int off = g * 32 + ps * 16 + 4 * t;
    const uint32_t sh4 = hi ? 4u : 0u;
    const uint32_t w00 = (lds4(tg + ((ch * 2 + 0) * 2 + 0) * 256 + off) >> sh4) & 0x0F0F0F0Fu;  // row g, lo
    const uint32_t w01 = (lds4(tg + ((ch * 2 + 0) * 2 + 1) * 256 + off) >> sh4) & 0x0F0F0F0Fu;  // row g, hi
    const uint32_t w10 = (lds4(tg + ((ch * 2 + 1) * 2 + 0) * 256 + off) >> sh4) & 0x0F0F0F0Fu;  // row g + 8
    const uint32_t w11 = (lds4(tg + ((ch * 2 + 1) * 2 + 1) * 256 + off) >> sh4) & 0x0F0F0F0Fu;
    const int src = (lane & ~3) | (c & 3);
    const __half2 s_g = __float2half2_rn(__shfl_sync(0xFFFFFFFFu, S.sc[0][c >> 2], src));
    const __half2 s_g8 = __float2half2_rn(__shfl_sync(0xFFFFFFFFu, S.sc[1][c >> 2], src));
    const __half2 o_g = __float2half2_rn(-__shfl_sync(0xFFFFFFFFu, S.mn[0][c >> 2], src));
    const __half2 o_g8 = __float2half2_rn(-__shfl_sync(0xFFFFFFFFu, S.mn[1][c >> 2], src));
    const __half2 ctr = __float2half2_rn(1024.0f);
    store_chunk(abuf, wrow, g, t, cib, deq4(w00, ctr, s_g, o_g), deq4(w10, ctr, s_g8, o_g8), deq4(w01, ctr, s_g, o_g),
                deq4(w11, ctr, s_g8, o_g8));
  } else if (type == FB200_Q6_K) {
    const int c2 = c >> 2, q = c & 3;
    uint2 out[2][2];  // [u][row half]
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int cu = c2 * 2 + u, grp = 8 * c2 + 2 * q + u;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t wl = lds4(tg + (cu * 2 + h) * 256 + g * 32 + (q & 1) * 16 + 4 * t);
        const uint32_t wh = lds4(tg + 2048 + (cu * 2 + h) * 128 + g * 16 + 4 * t);
        const uint32_t hb = q == 0 ? (wh << 4) : q == 1 ? (wh << 2) : q == 2 ? wh : (wh >> 2);
        const uint32_t bytes = (((q >> 1) ? (wl >> 4) : wl) & 0x0F0F0F0Fu) | (hb & 0x30303030u);
        const uint32_t scw = grp >> 2 == 0 ? S.q6[h].x : grp >> 2 == 1 ? S.q6[h].y : grp >> 2 == 2 ? S.q6[h].z : S.q6[h].w;
        const float s = S.d[h] * (float)(int)(int8_t)((scw >> (8 * (grp & 3))) & 0xFF);
        out[u][h] = deq4(bytes, __float2half2_rn(1056.0f), __float2half2_rn(s), zero2);  // (q - 32) d scale
      }
    }
    store_chunk(abuf, wrow, g, t, cib, out[0][0], out[0][1], out[1][0], out[1][1]);
  } else {
    const int dofs = type == FB200_Q4_0 ? 1024 : 2048;
    const __half2 d_g = __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(tg + dofs + (g * 4 + c) * 2)));
    const __half2 d_g8 = __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(tg + dofs + ((g + 8) * 4 + c) * 2)));
    if (type == FB200_Q4_0) {
      const uint32_t w0 = lds4(tg + g * 64 + c * 16 + 4 * t);
      const uint32_t w1 = lds4(tg + 512 + g * 64 + c * 16 + 4 * t);
      const __half2 ctr = __float2half2_rn(1032.0f);  // (q - 8) d
      store_chunk(abuf, wrow, g, t, cib, deq4(w0 & 0x0F0F0F0Fu, ctr, d_g, zero2), deq4(w1 & 0x0F0F0F0Fu, ctr, d_g8, zero2),
                  deq4((w0 >> 4) & 0x0F0F0F0Fu, ctr, d_g, zero2), deq4((w1 >> 4) & 0x0F0F0F0Fu, ctr, d_g8, zero2));
    } else {
      const int off = g * 64 + c * 16 + 4 * t;
      const __half2 ctr = __float2half2_rn(1152.0f);  // signed byte b as (b ^ 0x80) - 128
      store_chunk(abuf, wrow, g, t, cib, deq4(lds4(tg + off) ^ 0x80808080u, ctr, d_g, zero2),
                  deq4(lds4(tg + 1024 + off) ^ 0x80808080u, ctr, d_g8, zero2),
                  deq4(lds4(tg + 512 + off) ^ 0x80808080u, ctr, d_g, zero2),
                  deq4(lds4(tg + 1536 + off) ^ 0x80808080u, ctr, d_g8, zero2));
    }
  }
}

template <int BM>
__global__ void __launch_bounds__(TC_THREADS, 1)
qgemm_tc_kernel(const TcArgs a) {
  using T = Tc<BM>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* opnd = smem;                                   // [stage][A | B]
  uint8_t* raw = smem + TC_STAGES * T::STAGE;             // [2][8 tile-groups]
  uint64_t* bars = reinterpret_cast<uint64_t*>(raw + 2 * RAW_BYTES);  // raw_full[2], stage_free[TC_STAGES], done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 + TC_STAGES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
  const uint32_t bar_raw = smem_u32(bars), bar_free = smem_u32(bars + 2), bar_done = smem_u32(bars + 2 + TC_STAGES);

  if (tid == 0) {
    for (int i = 0; i < 3 + TC_STAGES; ++i) mbar_init(bar_raw + 8 * i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(T::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = *tmem_slot;

  const int tile0 = n0 / 16;
  const int my_tile = tile0 + warp;
  const int ntile_here = min(8, a.ntiles - tile0);
  auto issue_raw = [&](int kg, int rb) {  // thread 0
    mbar_expect_tx(bar_raw + 8 * rb, (uint32_t)(ntile_here * a.tgb));
    for (int i = 0; i < ntile_here; ++i)
      bulk_g2s(smem_u32(raw + rb * RAW_BYTES + i * RAW_STRIDE), a.w + ((size_t)(tile0 + i) * a.ngroups + kg) * a.tgb,
               (uint32_t)a.tgb, bar_raw + 8 * rb);
  };
  if (tid == 0) issue_raw(0, 0);

  const int blocks_per_group = a.group_elems / BK;  // 4 (K-quants) or 2
  const int nblocks = a.ngroups * blocks_per_group;
  // B tile of K block `blk` -> stage blk % TC_STAGES (one cp.async group per block); the stage
  // is free once the MMAs of block blk - TC_STAGES have read it
  auto copy_b = [&](int blk) {
    const int s = blk % TC_STAGES;
    if (blk >= TC_STAGES) mbar_wait(bar_free + 8 * s, (uint32_t)((blk / TC_STAGES - 1) & 1), a.status);
    uint8_t* bbuf = opnd + s * T::STAGE + A_BYTES;
    const int k0 = blk * BK;
#pragma unroll
    for (int i = 0; i < BM * 8 / TC_THREADS; ++i) {
      const int q = tid + TC_THREADS * i, r = q >> 3, kc8 = q & 7;
      cp_async16(bbuf + (r >> 3) * CORE_SBO + kc8 * CORE_LBO + (r & 7) * 16, a.xh + (size_t)(m0 + r) * a.K + k0 + kc8 * 8);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  copy_b(0);
  int it = 0;
  for (int kg = 0; kg < a.ngroups; ++kg) {
    const int rb = kg & 1;
    if (tid == 0 && kg + 1 < a.ngroups) issue_raw(kg + 1, rb ^ 1);  // its buffer was drained one group ago
    mbar_wait(bar_raw + 8 * rb, (uint32_t)((kg >> 1) & 1), a.status);
    const uint8_t* tg = raw + rb * RAW_BYTES + warp * RAW_STRIDE;
    RowScales S;
    if (my_tile < a.ntiles) prepare_scales(a.type, tg, lane >> 2, lane & 3, S);
    for (int b = 0; b < blocks_per_group; ++b, ++it) {
      const int s = it % TC_STAGES;
      uint8_t* abuf = opnd + s * T::STAGE;
      uint8_t* bbuf = abuf + A_BYTES;
      // the next block's activations start their trip now (also waits for that stage to be free;
      // stage s itself was freed before its own B copy was issued one iteration ago)
      if (it + 1 < nblocks) copy_b(it + 1);
      else asm volatile("cp.async.commit_group;" ::: "memory");
      // A: this warp's row-tile, two 32-element chunks
      if (my_tile < a.ntiles) {
        dequant_chunk(a.type, tg, 2 * b, lane, S, abuf, warp, 0);
        dequant_chunk(a.type, tg, 2 * b + 1, lane, S, abuf, warp, 1);
      }
      asm volatile("cp.async.wait_group 1;" ::: "memory");  // block `it`'s activations have landed
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> tensor-core reads
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncthreads();
      if (tid == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = smem_u32(abuf), sb = smem_u32(bbuf);
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks)
          tc_mma(tmem_d, operand_desc(sa + ks * 2 * CORE_LBO), operand_desc(sb + ks * 2 * CORE_LBO), T::IDESC,
                 (it | ks) ? 1u : 0u);
        tc_commit(bar_free + 8 * s);
      }
    }
  }
  if (tid == 0) tc_commit(bar_done);
  mbar_wait(bar_done, 0u, a.status);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  // ---- epilogue: warp w reads TMEM lanes 32 (w % 4) .. +31 (weight rows) and one half of the columns
  {
    const int n = n0 + 32 * (warp & 3) + lane;
    const int cbase = (BM / 2) * (warp >> 2);
#pragma unroll
    for (int half = 0; half < BM / 64; ++half) {
      uint32_t v[32];
      const uint32_t taddr = tmem_d + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(cbase + 32 * half);
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
          "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
            "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
            "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
            "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
          : "r"(taddr) : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int m = m0 + cbase + 32 * half + j;
        if (m < a.M && n < a.N) {
          const size_t idx = (size_t)m * a.N + n;
          float out = __uint_as_float(v[j]) * a.xscale[m];
          if (a.r1) out += a.r1[idx];
          if (a.r2) out += a.r2[idx];
          a.y[idx] = out;
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "n"(T::TMEM_COLS) : "memory");
}

// x[M, K] f32 -> fp16 rows [Mp, K] scaled by a power of two into (-64, 64); rows >= M are zero.
__global__ void __launch_bounds__(256)
pack_rows16_kernel(const float* __restrict__ x, int M, int K, __half* __restrict__ xh, float* __restrict__ xscale) {
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
  const float inv = ldexpf(64.0f, -ex);
  if (threadIdx.x == 0) xscale[m] = ldexpf(1.0f, ex - 6);
  for (int k = threadIdx.x; k < K; k += 256) xh[(size_t)m * K + k] = __float2half_rn(m < M ? xr[k] * inv : 0.f);
}

}  // namespace

// y[M, N] = x[M, K] . W^T (+ r1 + r2) for M > 32. Returns 1 when the shape is not covered (the
// caller falls back to the small-batch kernel in chunks of 32 rows).
int fb200_qgemm(fb200_device* dev, const fb200_qmatrix* w, const float* x, size_t m, float* y, const float* r1,
                const float* r2) {
  static const bool enabled = !(getenv("FB200_TCGEN05") && getenv("FB200_TCGEN05")[0] == '0');
  TileGeom geo;
  if (!enabled || !w->tiled || !tile_geom(w->type, &geo)) return 1;
  const size_t kp = (size_t)w->ngroups * geo.group_elems;
  if (kp != w->k || m > (1u << 20)) return 1;  // K is a whole number of K groups
  // 256 activation rows per tile when that still gives every SM a tile
  const int bm = (size_t)((w->n + BN - 1) / BN) * ((m + 255) / 256) >= (size_t)dev->sm_count ? 256 : 128;
  const int mp = (int)((m + bm - 1) / bm) * bm;
  const size_t xbytes = (size_t)mp * w->k * 2, need = xbytes + (size_t)mp * sizeof(float);
  int rc = fb200_ensure(dev, &dev->xpack, &dev->xpack_bytes, need);
  if (rc) return rc;
  __half* xh = reinterpret_cast<__half*>(dev->xpack);
  float* xscale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(dev->xpack) + xbytes);
  pack_rows16_kernel<<<mp, 256, 0, dev->stream>>>(x, (int)m, (int)w->k, xh, xscale);
  FB_LAUNCH_CHECK(dev);
  TcArgs a;
  a.w = w->data; a.xh = xh; a.xscale = xscale; a.y = y; a.r1 = r1; a.r2 = r2;
  a.M = (int)m; a.N = (int)w->n; a.K = (int)w->k;
  a.ngroups = w->ngroups; a.ntiles = w->ntiles; a.type = (int)w->type; a.tgb = geo.tg_bytes;
  a.group_elems = geo.group_elems; a.status = dev->status;
  static bool configured[64] = {false};
  if (!configured[dev->ordinal & 63]) {
    FB_CUDA(dev, cudaFuncSetAttribute(qgemm_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Tc<128>::SMEM));
    FB_CUDA(dev, cudaFuncSetAttribute(qgemm_tc_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, Tc<256>::SMEM));
    configured[dev->ordinal & 63] = true;
  }
  const dim3 grid((unsigned)((w->n + BN - 1) / BN), (unsigned)(mp / bm));
  if (bm == 256) return fb200_launch(dev, qgemm_tc_kernel<256>, grid, dim3(TC_THREADS), (size_t)Tc<256>::SMEM, false, a);
  return fb200_launch(dev, qgemm_tc_kernel<128>, grid, dim3(TC_THREADS), (size_t)Tc<128>::SMEM, false, a);
}
