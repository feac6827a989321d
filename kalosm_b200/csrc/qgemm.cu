// Prefill product (M > 32 activation rows) on the 5th-generation tensor cores: tcgen05.mma with
// the accumulator in tensor memory (TMEM).
//
// Bound: tensor cores (2 M N K flops). Replaces the reference's tiled quantised matmul
// (fusor-ml/tile-ir-kernels/src/kernels/qmatmul.rs:237-349) for large M, where the small-batch
// kernels would re-read W once per 32 rows.
//
// One CTA computes a tile of NH x 128 weight rows by BM = 128 or 256 activation rows of
// Y^T = W . X^T; the fp32 accumulators (NH x BM columns of 128 lanes) live in TMEM. The roles
// are coupled only by mbarriers, there is no CTA-wide barrier in the main loop:
//  * weight loader (one thread): W stays quantised in HBM; the raw tile-groups of the CTA's
//    8 NH row-tiles for one K group come by 1-D TMA bulk copies, two K groups in flight.
//  * conversion warps (8 NH, one per row-tile): dequantise to fp16 in registers (byte -> 1024 +
//    byte by a byte permute, exact subtraction, one fused multiply-add with block scale and
//    offset) and store into the A operand stage in the canonical K-major core-matrix layout of
//    the MMA (8 rows x 16 bytes per core matrix, no swizzle); a proxy fence, then one arrive per
//    warp on the stage's "A full" barrier.
//  * activation loader (one thread): X is converted once per call to fp16 rows scaled by a power
//    of two and stored tile by tile in the same operand layout, so a B stage is one contiguous
//    bulk copy.
//  * MMA issuer (one thread): waits for "A full" and "B full", issues 4 NH tcgen05.mma (M = 128,
//    N = BM, K = 16, kind::f16, fp32 accumulate) per 64-wide K block; tcgen05.commit on the
//    stage's "free" barrier hands the stage back to both producers (2..4 stages, as many as fit
//    beside the raw buffers).
//  * Epilogue: tcgen05.ld brings the accumulator out of TMEM (each warp its 32 lanes), rows are
//    scaled back and written, with the residual adds or SwiGLU (gate and up rows are the two
//    halves of one CTA, so both values of an output sit in the same TMEM lane).
// Every wait is bounded (2^22 polls): on a time-out the status word and a give-up flag in shared
// memory are set, the other roles leave at their next poll, and the CTA releases its TMEM
// columns and exits. FB200_TCGEN05=0 switches the kernel off (32-row kernel in chunks);
// FB200_TC_TILE="BM,NH" forces a tile shape (tests, tuning).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "qgemv_common.cuh"

int fb200_ensure(fb200_device* dev, void** buf, size_t* cur, size_t bytes);

namespace {

constexpr int BN = 128;  // weight rows per MMA (M of the MMA); a CTA tile holds NH such halves
// activation rows per CTA tile (N of the MMA): template parameter BM = 128 or 256
constexpr int BK = 64;   // K elements per operand stage (four K = 16 MMAs)
constexpr int A_SBO = (BK / 8) * 128 + 64;        // A operand: bytes between 8-row groups, padded by half a
                                                  // core matrix so that rows g and g + 8 fall into different banks
constexpr int A_HALF = (BN / 8) * A_SBO;          // one 128-row half of an A stage
constexpr int CORE_LBO = 128;                     // bytes between core matrices adjacent in K
constexpr int CORE_SBO = (BK / 8) * 128;          // B operand: bytes between 8-row groups
constexpr int MAX_STAGES = 4;
constexpr int TAIL_BYTES = 256;                   // barriers, TMEM slot, give-up flag
constexpr int SMEM_BUDGET = 227 * 1024;
template <int BM, int NH>
struct Tc {
  static constexpr int A_BYTES = NH * A_HALF;               // one A stage
  static constexpr int B_BYTES = BM * BK * 2;               // one B stage
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = NH * BM;                 // fp32 accumulator columns
  static constexpr int DQ_WARPS = 8 * NH;                   // one warp per 16-row tile
  static constexpr int THREADS = (DQ_WARPS + 3) * 32;       // + weight loader, activation loader, MMA issuer
  // instruction descriptor: fp32 accumulator, fp16 A and B, both K-major, N = BM, M = BN
  static constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BM >> 3) << 17) | ((uint32_t)(BN >> 4) << 24);
};

struct TcArgs {
  const uint8_t* w;      // tiled weights
  const __half* xh;      // fp16 activations, [Mp / BM][K / 64] tiles already in the operand layout
  const float* xscale;   // [Mp] power-of-two scale of each row
  float* y;              // [M, N]
  const float* r1;       // optional residuals [M, N], or one bias row [N] when r1_stride is 0
  const float* r2;
  int r1_stride;
  int M, N, K;
  int ngroups, ntiles, type, tgb, group_elems;
  int stages, raw_stride;  // operand stages that fit beside the raw buffers; bytes per raw tile-group slot
  int pair_tiles;          // SwiGLU (NH = 2): half 0 = gate rows, half 1 = up rows pair_tiles row-tiles further;
                           // y[M, N / 2] = silu(gate) * up. 0 = plain product
  int kg_per;              // K groups per split (grid.z splits; = ngroups without split-K). Split z covers the
                           // K groups z kg_per .. and writes its partial product to y + z M N (no residuals)
  int* status;
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait of the pipeline roles: gives up after 2^22 polls, or as soon as another thread
// of the CTA has given up (so a broken pipeline drains in one time-out, not one per wait).
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int* dead, int* status) {
  for (int it = 0; it < (1 << 22); ++it) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((it & 255) == 255 && *dead) return false;
  }
  *dead = 1;
  if (status) atomicExch(status, FB200_ERR_TIMEOUT);
  return false;
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
__device__ __forceinline__ uint64_t operand_desc(uint32_t saddr, uint32_t sbo) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(CORE_LBO >> 4) << 16) |
         ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
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

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr) : "memory");
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
  // In one store instruction the lanes with t < 2 write row g and the others row g + 8 (then the
  // other way round): with the padded row-group stride the 16 lanes of a half-warp cover all 32
  // banks once, where "every lane its row g" would put K chunks t / 2 = 0 and 1 on the same banks.
  const bool odd = (t & 2) != 0;
  uint8_t* base = abuf + (2 * wrow) * A_SBO + g * 16 + (t & 1) * 8 + (4 * cib + (t >> 1)) * CORE_LBO;
  uint8_t* p1 = base + (odd ? A_SBO : 0);
  uint8_t* p2 = base + (odd ? 0 : A_SBO);
  *reinterpret_cast<uint2*>(p1) = odd ? lo_g8 : lo_g;
  *reinterpret_cast<uint2*>(p2) = odd ? lo_g : lo_g8;
  *reinterpret_cast<uint2*>(p1 + 2 * CORE_LBO) = odd ? hi_g8 : hi_g;
  *reinterpret_cast<uint2*>(p2 + 2 * CORE_LBO) = odd ? hi_g : hi_g8;
}

template <int type>
__device__ __forceinline__ void prepare_scales(const uint8_t* tg, int g, int t, RowScales& S) {
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
template <int type>
__device__ __forceinline__ void dequant_chunk(const uint8_t* tg, int c, int lane, const RowScales& S,
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
    const __half2 s_g = __float2half2_rn(__shfl_sync(0xFFFFFFFFu, ((c >> 2) ? S.sc[0][1] : S.sc[0][0]), src));
    const __half2 s_g8 = __float2half2_rn(__shfl_sync(0xFFFFFFFFu, ((c >> 2) ? S.sc[1][1] : S.sc[1][0]), src));
    const __half2 o_g = __float2half2_rn(-__shfl_sync(0xFFFFFFFFu, ((c >> 2) ? S.mn[0][1] : S.mn[0][0]), src));
    const __half2 o_g8 = __float2half2_rn(-__shfl_sync(0xFFFFFFFFu, ((c >> 2) ? S.mn[1][1] : S.mn[1][0]), src));
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

template <int BM, int NH, int TYPE>
__global__ void __launch_bounds__(Tc<BM, NH>::THREADS, 1)
qgemm_tc_kernel(const TcArgs a) {
  using T = Tc<BM, NH>;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int raw_bytes = T::DQ_WARPS * a.raw_stride;
  uint8_t* opnd = smem;                                   // [stage][A halves | B]
  uint8_t* raw = smem + a.stages * T::STAGE;              // [2][DQ_WARPS tile-groups]
  uint64_t* bars = reinterpret_cast<uint64_t*>(raw + 2 * raw_bytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * (a.pair_tiles ? BN : BN * NH), m0 = blockIdx.y * BM;
  const uint32_t bar_raw_full = smem_u32(bars), bar_raw_free = smem_u32(bars + 2), bar_a_full = smem_u32(bars + 4),
                 bar_b_full = smem_u32(bars + 4 + MAX_STAGES), bar_free = smem_u32(bars + 4 + 2 * MAX_STAGES),
                 bar_done = smem_u32(bars + 4 + 3 * MAX_STAGES);

  if (tid == 0) {
    *dead = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_raw_full + 8 * i, 1);
      mbar_init(bar_raw_free + 8 * i, T::DQ_WARPS);
    }
    for (int i = 0; i < MAX_STAGES; ++i) {
      mbar_init(bar_a_full + 8 * i, T::DQ_WARPS);
      mbar_init(bar_b_full + 8 * i, 1);
      mbar_init(bar_free + 8 * i, 1);
    }
    mbar_init(bar_done, 1);
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
  // row-tile converted by warp i, and whether the matrix has it
  auto tile_of = [&](int i) { return a.pair_tiles ? tile0 + (i & 7) + (i >> 3) * a.pair_tiles : tile0 + i; };
  auto has_tile = [&](int i) { return a.pair_tiles ? tile0 + (i & 7) < a.pair_tiles : tile0 + i < a.ntiles; };
  constexpr int blocks_per_group = (TYPE == FB200_Q4_K || TYPE == FB200_Q6_K ? 256 : 128) / BK;
  // this CTA's K groups: kg0 .. kg0 + ngr - 1 (all of them without split-K); the loops below count
  // from 0 (barrier phases), only addresses use kg0
  const int kg0 = (int)blockIdx.z * a.kg_per;
  const int ngr = min(a.kg_per, a.ngroups - kg0);
  const int nblocks = ngr * blocks_per_group;

  if (warp < T::DQ_WARPS) {
    // ---- conversion: warp w turns row-tile w of each K block into fp16 operand rows
    const bool mine = has_tile(warp);
    uint8_t* const a_rows = opnd + (warp >> 3) * A_HALF;
    int s = 0, round = 0;
    bool alive = true;
    for (int kg = 0; kg < ngr && alive; ++kg) {
      const int rb = kg & 1;
      alive = tc_wait(bar_raw_full + 8 * rb, (uint32_t)((kg >> 1) & 1), dead, a.status);
      if (!alive) break;
      const uint8_t* tg = raw + rb * raw_bytes + warp * a.raw_stride;
      RowScales S;
      if (mine) prepare_scales<TYPE>(tg, lane >> 2, lane & 3, S);
#pragma unroll
      for (int b = 0; b < blocks_per_group; ++b) {
        // the stage is free once the MMAs of its previous use have read it
        if (round > 0) alive = tc_wait(bar_free + 8 * s, (uint32_t)((round - 1) & 1), dead, a.status);
        if (!alive) break;
        uint8_t* abuf = a_rows + s * T::STAGE;
        if (mine) {
          dequant_chunk<TYPE>(tg, 2 * b, lane, S, abuf, warp & 7, 0);
          dequant_chunk<TYPE>(tg, 2 * b + 1, lane, S, abuf, warp & 7, 1);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> tensor-core reads
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_a_full + 8 * s);
        if (++s == a.stages) { s = 0; ++round; }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_raw_free + 8 * rb);
    }
  } else if (warp == T::DQ_WARPS) {
    // ---- weight loader: raw tile-groups of one K group, two groups in flight
    if (lane == 0) {
      int ntile_here = 0;
      for (int i = 0; i < T::DQ_WARPS; ++i) ntile_here += has_tile(i) ? 1 : 0;
      for (int kg = 0; kg < ngr; ++kg) {
        const int rb = kg & 1;
        if (kg >= 2 && !tc_wait(bar_raw_free + 8 * rb, (uint32_t)(((kg >> 1) - 1) & 1), dead, a.status)) break;
        mbar_expect_tx(bar_raw_full + 8 * rb, (uint32_t)(ntile_here * a.tgb));
        for (int i = 0; i < T::DQ_WARPS; ++i)
          if (has_tile(i))
            bulk_g2s(smem_u32(raw + rb * raw_bytes + i * a.raw_stride),
                     a.w + ((size_t)tile_of(i) * a.ngroups + kg0 + kg) * a.tgb, (uint32_t)a.tgb, bar_raw_full + 8 * rb);
      }
    }
  } else if (warp == T::DQ_WARPS + 1) {
    // ---- activation loader: one bulk copy per K block (the tile is stored in operand layout)
    if (lane == 0) {
      const __half* src = a.xh + ((size_t)blockIdx.y * a.ngroups + kg0) * blocks_per_group * (BM * BK);
      int s = 0, round = 0;
      for (int blk = 0; blk < nblocks; ++blk) {
        if (round > 0 && !tc_wait(bar_free + 8 * s, (uint32_t)((round - 1) & 1), dead, a.status)) break;
        mbar_expect_tx(bar_b_full + 8 * s, (uint32_t)T::B_BYTES);
        bulk_g2s(smem_u32(opnd + s * T::STAGE + T::A_BYTES), src + (size_t)blk * (BM * BK), (uint32_t)T::B_BYTES,
                 bar_b_full + 8 * s);
        if (++s == a.stages) { s = 0; ++round; }
      }
    }
  } else {
    // ---- MMA issuer: 4 NH instructions per K block; the commit frees the stage
    if (lane == 0) {
      int s = 0, round = 0;
      bool alive = true;
      for (int blk = 0; blk < nblocks; ++blk) {
        alive = tc_wait(bar_a_full + 8 * s, (uint32_t)(round & 1), dead, a.status) &&
                tc_wait(bar_b_full + 8 * s, (uint32_t)(round & 1), dead, a.status);
        if (!alive) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = smem_u32(opnd + s * T::STAGE), sb = sa + T::A_BYTES;
#pragma unroll
        for (int h = 0; h < NH; ++h)
#pragma unroll
          for (int ks = 0; ks < BK / 16; ++ks)
            tc_mma(tmem_d + (uint32_t)(h * BM), operand_desc(sa + h * A_HALF + ks * 2 * CORE_LBO, A_SBO),
                   operand_desc(sb + ks * 2 * CORE_LBO, CORE_SBO), T::IDESC, (blk | ks) ? 1u : 0u);
        tc_commit(bar_free + 8 * s);
        if (++s == a.stages) { s = 0; ++round; }
      }
      if (alive) tc_commit(bar_done);
    }
  }

  // ---- epilogue: warp w reads TMEM lanes 32 (w % 4) .. +31 (weight rows) of one half and one
  // half of that half's columns
  if (NH == 2 && a.pair_tiles) {
    // SwiGLU: the gate and the up value of an output sit in the same TMEM lane, BM columns apart
    if (warp < T::DQ_WARPS && tc_wait(bar_done, 0u, dead, a.status)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int n = n0 + 32 * (warp & 3) + lane, n_out = a.pair_tiles * 16;
      const int cbase = (BM / 4) * (warp >> 2);
#pragma unroll
      for (int i = 0; i < BM / 64; ++i) {
        uint32_t g[16], u[16];
        const uint32_t taddr = tmem_d + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(cbase + 16 * i);
        tmem_ld16(taddr, g);
        tmem_ld16(taddr + BM, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m0 + cbase + 16 * i + j;
          if (m < a.M && n < n_out) {
            // silu(gate) * up, fusor-ml/fusor/src/composite/activations.rs:47-64: x / (1 + exp(-x))
            const float sc = a.xscale[m], gate = __uint_as_float(g[j]) * sc;
            a.y[(size_t)m * n_out + n] = (gate / (1.0f + expf(-gate))) * (__uint_as_float(u[j]) * sc);
          }
        }
      }
    }
  } else if (warp < T::DQ_WARPS && tc_wait(bar_done, 0u, dead, a.status)) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int part = warp >> 2, h = part >> 1;
    const int n = n0 + h * BN + 32 * (warp & 3) + lane;
    const int cbase = (BM / 2) * (part & 1);
#pragma unroll
    for (int i = 0; i < BM / 64; ++i) {
      uint32_t v[32];
      const uint32_t taddr = tmem_d + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(h * BM + cbase + 32 * i);
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
        const int m = m0 + cbase + 32 * i + j;
        if (m < a.M && n < a.N) {
          const size_t idx = (size_t)m * a.N + n;
          float out = __uint_as_float(v[j]) * a.xscale[m];
          if (a.r1) out += a.r1[(size_t)m * a.r1_stride + n];
          if (a.r2) out += a.r2[idx];
          a.y[(size_t)blockIdx.z * a.M * a.N + idx] = out;
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "n"(T::TMEM_COLS) : "memory");
}

// x[M, K] f32 -> fp16 scaled by a power of two per row into (-64, 64), stored as [Mp / bm][K / 64]
// tiles of bm rows x 64 values in the operand layout of the MMA (8 rows x 16 bytes per core
// matrix, core matrices adjacent in K 128 bytes apart, 8-row groups 1024 bytes apart), so that a
// tile is one contiguous bulk copy. One CTA per PACK_ROWS rows (512 rows give 128 CTAs); two warps
// find the maximum of a row with independent 16-byte loads; rows >= M are zero.
constexpr int PACK_ROWS = 4;
__global__ void __launch_bounds__(256)
pack_rows16_kernel(const float* __restrict__ x, int M, int K, int bm, __half* __restrict__ xh, float* __restrict__ xscale) {
  __shared__ float part[8];
  __shared__ float inv_s[PACK_ROWS];
  const int m0 = blockIdx.x * PACK_ROWS, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    const int row = warp % PACK_ROWS, half = warp / PACK_ROWS;  // 8 warps: two per row, half of K each
    const int m = m0 + row;
    float amax = 0.f;
    if (m < M) {
      const float4* xr = reinterpret_cast<const float4*>(x + (size_t)m * K) + (size_t)half * (K / 8);
      const int n4 = K / 8;  // float4 per half row (K is a multiple of 64)
#pragma unroll 8
      for (int i = lane; i < n4; i += 32) {
        const float4 v = __ldg(xr + i);
        amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if (lane == 0) part[warp] = amax;
  }
  __syncthreads();
  if (threadIdx.x < PACK_ROWS) {
    const float amax = fmaxf(part[threadIdx.x], part[threadIdx.x + PACK_ROWS]);
    int ex = 0;
    if (amax > 0.f && amax < 3.0e38f) frexpf(amax, &ex);
    inv_s[threadIdx.x] = ldexpf(64.0f, -ex);
    xscale[m0 + threadIdx.x] = ldexpf(1.0f, ex - 6);
  }
  __syncthreads();
  const int nkb = K / BK;
  uint8_t* tile_row = reinterpret_cast<uint8_t*>(xh) + (size_t)(m0 / bm) * nkb * ((size_t)bm * BK * 2) +
                      ((m0 % bm) >> 3) * CORE_SBO + (m0 & 7) * 16;
  for (int q = threadIdx.x; q < K / 8 * PACK_ROWS; q += 256) {  // K / 8 chunks of 8 values x PACK_ROWS rows
    const int r = q % PACK_ROWS, kc = q / PACK_ROWS, m = m0 + r;
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (m < M) {
      const float4* src = reinterpret_cast<const float4*>(x + (size_t)m * K + 8 * kc);
      const float4 lo = __ldg(src), hi = __ldg(src + 1);
      const float inv = inv_s[r];
      out.x = h2u(__floats2half2_rn(lo.x * inv, lo.y * inv));
      out.y = h2u(__floats2half2_rn(lo.z * inv, lo.w * inv));
      out.z = h2u(__floats2half2_rn(hi.x * inv, hi.y * inv));
      out.w = h2u(__floats2half2_rn(hi.z * inv, hi.w * inv));
    }
    *reinterpret_cast<uint4*>(tile_row + (size_t)(kc >> 3) * ((size_t)bm * BK * 2) + (kc & 7) * CORE_LBO + r * 16) = out;
  }
}

template <int BM, int NH, int TYPE>
int launch_tc_type(fb200_device* dev, const TcArgs& a, unsigned grid_n, unsigned grid_m, unsigned grid_z, int smem) {
  using T = Tc<BM, NH>;
  static bool configured[64] = {false};
  if (!configured[dev->ordinal & 63]) {
    FB_CUDA(dev, cudaFuncSetAttribute(qgemm_tc_kernel<BM, NH, TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET));
    configured[dev->ordinal & 63] = true;
  }
  return fb200_launch(dev, qgemm_tc_kernel<BM, NH, TYPE>, dim3(grid_n, grid_m, grid_z), dim3(T::THREADS), (size_t)smem, false, a);
}

template <int BM, int NH>
int launch_tc(fb200_device* dev, const TcArgs& a, unsigned grid_n, unsigned grid_m, unsigned grid_z, int smem) {
  switch (a.type) {
    case FB200_Q4_0: return launch_tc_type<BM, NH, FB200_Q4_0>(dev, a, grid_n, grid_m, grid_z, smem);
    case FB200_Q8_0: return launch_tc_type<BM, NH, FB200_Q8_0>(dev, a, grid_n, grid_m, grid_z, smem);
    case FB200_Q4_K: return launch_tc_type<BM, NH, FB200_Q4_K>(dev, a, grid_n, grid_m, grid_z, smem);
    case FB200_Q6_K: return launch_tc_type<BM, NH, FB200_Q6_K>(dev, a, grid_n, grid_m, grid_z, smem);
  }
  return 1;
}

// Tile shape of one product: NH x 128 weight rows by bm activation rows, and the operand stages that
// fit. Returns false when no shape fits.
struct TcShape { int bm = 0, nh = 0, stages = 0, split = 1; size_t ctas = 0, cost = 0; };

// measured time per unit of tile area relative to the 256 x 256 tile, in 1/64ths
static const int kRelCost[2][2] = {{134, 87}, {96, 64}};  // [nh - 1][bm == 256]

bool tc_shape(const fb200_qmatrix* w, const TileGeom& geo, size_t m, int swiglu, int bm, int nh, TcShape* out) {
  const int raw_stride = (geo.tg_bytes + 127) & ~127;
  const int stage = nh * A_HALF + bm * BK * 2;
  const int stages = std::min(MAX_STAGES, (SMEM_BUDGET - TAIL_BYTES - 2 * 8 * nh * raw_stride) / stage);
  if (stages < 2) return false;
  const size_t n_rows = swiglu ? w->n / 2 : w->n;  // weight rows along the grid
  const size_t rows_per_cta = swiglu ? BN : BN * nh;
  out->bm = bm; out->nh = nh; out->stages = stages;
  out->ctas = ((n_rows + rows_per_cta - 1) / rows_per_cta) * ((m + bm - 1) / bm);
  out->cost = (size_t)(nh * bm) * kRelCost[nh - 1][bm == 256];  // time of one CTA
  return true;
}

bool tc_covers(const fb200_qmatrix* w, const float* x, size_t m, TileGeom* geo) {
  static const bool enabled = !(getenv("FB200_TCGEN05") && getenv("FB200_TCGEN05")[0] == '0');
  if (!enabled || !w->tiled || !tile_geom(w->type, geo)) return false;
  const size_t kp = (size_t)w->ngroups * geo->group_elems;
  if (kp != w->k || m > (1u << 20)) return false;  // K is a whole number of K groups
  return (reinterpret_cast<uintptr_t>(x) & 15) == 0;
}

// y = p[0] + p[1] + .. (+ r1 + r2): the partial products of a split-K launch, added in split order.
__global__ void __launch_bounds__(256)
splitk_add_kernel(const float4* __restrict__ parts, int nsplit, size_t n4, int ncols4, const float* __restrict__ r1,
                  int r1_stride, const float* __restrict__ r2, float4* __restrict__ y) {
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n4) return;
  float4 acc = __ldg(parts + i);
  for (int s = 1; s < nsplit; ++s) {
    const float4 v = __ldg(parts + (size_t)s * n4 + i);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  if (r1) {
    const size_t m = i / (size_t)ncols4, c = i - m * (size_t)ncols4;
    const float4 v = __ldg(reinterpret_cast<const float4*>(r1 + m * (size_t)r1_stride) + c);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  if (r2) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(r2) + i);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  y[i] = acc;
}

// Launches the product of packed rows (xh, xscale: pack_rows16_kernel with this bm) on dev->stream.
// With sh.split > 1 the K groups are cut into sh.split ranges (grid.z), every range writes its
// partial product into the handle's split-K scratch and a second kernel adds them (+ residuals).
int tc_launch(fb200_device* dev, const fb200_qmatrix* w, const TileGeom& geo, const TcShape& sh, const __half* xh,
              const float* xscale, size_t m, float* y, bool r1_is_bias, const float* r1, const float* r2, int swiglu) {
  const int bm = sh.bm, nh = sh.nh;
  const int raw_stride = (geo.tg_bytes + 127) & ~127;
  const int mp = (int)((m + bm - 1) / bm) * bm;
  const int split = swiglu ? 1 : sh.split;
  float* parts = nullptr;
  if (split > 1) {
    int rc = fb200_ensure(dev, &dev->splitk, &dev->splitk_bytes, (size_t)split * m * w->n * sizeof(float));
    if (rc) return rc;
    parts = reinterpret_cast<float*>(dev->splitk);
  }
  TcArgs a;
  a.w = w->data; a.xh = xh; a.xscale = xscale;
  a.y = split > 1 ? parts : y;
  a.r1 = split > 1 ? nullptr : r1;
  a.r2 = split > 1 ? nullptr : r2;
  a.r1_stride = r1_is_bias ? 0 : (int)w->n;
  a.M = (int)m; a.N = (int)w->n; a.K = (int)w->k;
  a.ngroups = w->ngroups; a.ntiles = w->ntiles; a.type = (int)w->type; a.tgb = geo.tg_bytes;
  a.group_elems = geo.group_elems; a.status = dev->status;
  a.stages = sh.stages; a.raw_stride = raw_stride;
  a.pair_tiles = swiglu ? w->ntiles / 2 : 0;
  a.kg_per = (w->ngroups + split - 1) / split;
  const unsigned gz = (unsigned)((w->ngroups + a.kg_per - 1) / a.kg_per);  // every range holds at least one K group
  const int smem = sh.stages * (nh * A_HALF + bm * BK * 2) + 2 * 8 * nh * raw_stride + TAIL_BYTES;
  const size_t n_rows = swiglu ? w->n / 2 : w->n;
  const size_t rows_per_cta = swiglu ? BN : BN * nh;
  const unsigned gn = (unsigned)((n_rows + rows_per_cta - 1) / rows_per_cta), gm = (unsigned)(mp / bm);
  int rc;
  if (nh == 2) rc = bm == 256 ? launch_tc<256, 2>(dev, a, gn, gm, gz, smem) : launch_tc<128, 2>(dev, a, gn, gm, gz, smem);
  else rc = bm == 256 ? launch_tc<256, 1>(dev, a, gn, gm, gz, smem) : launch_tc<128, 1>(dev, a, gn, gm, gz, smem);
  if (rc || split == 1) return rc;
  const size_t n4 = m * w->n / 4;
  splitk_add_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, dev->stream>>>(
      reinterpret_cast<const float4*>(parts), (int)gz, n4, (int)(w->n / 4), r1, r1_is_bias ? 0 : (int)w->n, r2,
      reinterpret_cast<float4*>(y));
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}

}  // namespace

// y[M, N] = x[M, K] . W^T (+ r1 + r2) for M > 32; with `swiglu`, W stacks gate rows over up rows
// and y[M, N / 2] = silu(gate) * up. Returns 1 when the shape is not covered (the
// caller falls back to the small-batch kernel in chunks of 32 rows).
int fb200_qgemm(fb200_device* dev, const fb200_qmatrix* w, const float* x, size_t m, float* y, bool r1_is_bias, const float* r1,
                const float* r2, int swiglu) {
  TileGeom geo;
  if (!tc_covers(w, x, m, &geo)) return 1;
  // CTA tile: cost model waves x time of one CTA; among equals the larger tile (fewer re-reads of
  // the activations through L2).
  int force_bm = 0, force_nh = 0;
  if (const char* cfg = getenv("FB200_TC_TILE")) sscanf(cfg, "%d,%d", &force_bm, &force_nh);
  TcShape best;
  size_t best_cost = ~(size_t)0;
  for (int nh = 2; nh >= (swiglu ? 2 : 1); --nh)
    for (int bm = 256; bm >= 128; bm -= 128) {
      if ((force_bm && bm != force_bm) || (force_nh && nh != force_nh && !swiglu)) continue;
      TcShape sh;
      if (!tc_shape(w, geo, m, swiglu, bm, nh, &sh)) continue;
      const size_t cost = ((sh.ctas + dev->sm_count - 1) / dev->sm_count) * sh.cost;
      if (cost < best_cost) { best_cost = cost; best = sh; }
    }
  if (!best.bm) return 1;
  // Split-K (plain and residual epilogues, 16-byte aligned outputs, at least 2048 values of K per range):
  // the K groups in 2 or 4 ranges side by side (grid.z) when that lets a larger, more efficient tile
  // fill the SMs. Times in ns, from measurements at 512 rows: a 256 x 256 tile takes 4 us per 256 values
  // of K (the other shapes in proportion to the table above), a CTA costs 8 us beside its K loop, the
  // ranges write split x the output at about 3 TB/s and the adding kernel takes 2 us + (split + 1)
  // passes over the output at 7 TB/s.
  static const bool no_split = getenv("FB200_TC_SPLITK") && getenv("FB200_TC_SPLITK")[0] == '0';
  const bool may_split = !no_split && !swiglu && !force_bm && !force_nh && w->n % 4 == 0 &&
                         ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(r1) | reinterpret_cast<uintptr_t>(r2)) & 15) == 0;
  if (may_split) {
    const double unit_ns = 4000.0 * ((double)w->k / 256.0) / 32768.0, out_bytes = (double)m * (double)w->n * 4.0;
    auto total_ns = [&](const TcShape& sh, int split) {
      const double waves = (double)((sh.ctas * split + dev->sm_count - 1) / dev->sm_count);
      double t = waves * ((double)sh.cost * unit_ns / split + 8000.0);
      if (split > 1) t += split * out_bytes / 3000.0 + 2000.0 + (split + 1) * out_bytes / 7000.0;
      return t;
    };
    double best_ns = 0.9 * total_ns(best, 1);  // a split has to promise a tenth less
    for (int split = 2; split <= 4; split *= 2) {
      if (w->k / split < 2048 || w->ngroups < 2 * split) break;
      for (int nh = 2; nh >= 1; --nh)
        for (int bm = 256; bm >= 128; bm -= 128) {
          TcShape sh;
          if (!tc_shape(w, geo, m, 0, bm, nh, &sh)) continue;
          const double t = total_ns(sh, split);
          if (t < best_ns) { best_ns = t; best = sh; best.split = split; }
        }
    }
  }
  const int mp = (int)((m + best.bm - 1) / best.bm) * best.bm;
  const size_t xbytes = (size_t)mp * w->k * 2, need = xbytes + (size_t)mp * sizeof(float);
  int rc = fb200_ensure(dev, &dev->xpack, &dev->xpack_bytes, need);
  if (rc) return rc;
  __half* xh = reinterpret_cast<__half*>(dev->xpack);
  float* xscale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(dev->xpack) + xbytes);
  pack_rows16_kernel<<<mp / PACK_ROWS, 256, 0, dev->stream>>>(x, (int)m, (int)w->k, best.bm, xh, xscale);
  FB_LAUNCH_CHECK(dev);
  return tc_launch(dev, w, geo, best, xh, xscale, m, y, r1_is_bias, r1, r2, swiglu);
}

// Up to three products of the same rows (the q, k and v projections of a prompt pass):
// ys[i][M, N_i] = x[M, K] . W_i^T. One of them alone leaves most SMs idle (a 1024-row matrix at
// 512 rows is 16..32 CTA tiles, each walking the whole K), so the rows are packed once and the
// products run side by side: the first on the handle's stream, the others on side streams forked
// behind the packing kernel and joined again before the call returns to the stream. Returns 1 when
// the shapes are not covered (the caller issues the products one after the other).
int fb200_qgemm_group(fb200_device* dev, const fb200_qmatrix* const* ws, float* const* ys, int n, const float* x, size_t m) {
  static const bool off = getenv("FB200_TC_GROUP") && getenv("FB200_TC_GROUP")[0] == '0';
  if (off || n < 2 || n > 3 || m <= 32 || getenv("FB200_TC_TILE")) return 1;
  TileGeom geo[3];
  for (int i = 0; i < n; ++i)
    if (!ws[i] || !tc_covers(ws[i], x, m, &geo[i]) || ws[i]->k != ws[0]->k) return 1;
  // one bm for all (they share the packed rows), nh per matrix; cost = waves of all CTAs together x
  // the time of the slowest CTA
  TcShape best[3];
  size_t best_cost = ~(size_t)0;
  for (int bm = 256; bm >= 128; bm -= 128)
    for (int mask = 0; mask < (1 << n); ++mask) {
      TcShape sh[3];
      size_t ctas = 0, slowest = 0;
      bool ok = true;
      for (int i = 0; i < n && ok; ++i) {
        ok = tc_shape(ws[i], geo[i], m, 0, bm, (mask >> i) & 1 ? 2 : 1, &sh[i]);
        if (ok) { ctas += sh[i].ctas; slowest = std::max(slowest, sh[i].cost); }
      }
      if (!ok) continue;
      const size_t cost = ((ctas + dev->sm_count - 1) / dev->sm_count) * slowest;
      if (cost < best_cost) { best_cost = cost; for (int i = 0; i < n; ++i) best[i] = sh[i]; }
    }
  if (best_cost == ~(size_t)0) return 1;
  for (int i = 0; i < n - 1; ++i) {
    if (!dev->side_stream[i]) FB_CUDA(dev, cudaStreamCreateWithFlags(&dev->side_stream[i], cudaStreamNonBlocking));
    if (!dev->join_ev[i]) FB_CUDA(dev, cudaEventCreateWithFlags(&dev->join_ev[i], cudaEventDisableTiming));
  }
  if (!dev->fork_ev) FB_CUDA(dev, cudaEventCreateWithFlags(&dev->fork_ev, cudaEventDisableTiming));
  const int bm = best[0].bm;
  const int mp = (int)((m + bm - 1) / bm) * bm;
  const size_t xbytes = (size_t)mp * ws[0]->k * 2, need = xbytes + (size_t)mp * sizeof(float);
  int rc = fb200_ensure(dev, &dev->xpack, &dev->xpack_bytes, need);
  if (rc) return rc;
  __half* xh = reinterpret_cast<__half*>(dev->xpack);
  float* xscale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(dev->xpack) + xbytes);
  pack_rows16_kernel<<<mp / PACK_ROWS, 256, 0, dev->stream>>>(x, (int)m, (int)ws[0]->k, bm, xh, xscale);
  FB_LAUNCH_CHECK(dev);
  FB_CUDA(dev, cudaEventRecord(dev->fork_ev, dev->stream));
  cudaStream_t main_stream = dev->stream;
  // the largest product stays on the handle's stream
  int first = 0;
  for (int i = 1; i < n; ++i) if (best[i].ctas > best[first].ctas) first = i;
  int side = 0;
  for (int i = 0; i < n && !rc; ++i) {
    if (i == first) continue;
    cudaStream_t st = dev->side_stream[side];
    FB_CUDA(dev, cudaStreamWaitEvent(st, dev->fork_ev, 0));
    dev->stream = st;  // the launch helpers take the handle's stream
    rc = tc_launch(dev, ws[i], geo[i], best[i], xh, xscale, m, ys[i], false, nullptr, nullptr, 0);
    dev->stream = main_stream;
    if (!rc) {
      FB_CUDA(dev, cudaEventRecord(dev->join_ev[side], st));
      ++side;
    }
  }
  if (!rc) rc = tc_launch(dev, ws[first], geo[first], best[first], xh, xscale, m, ys[first], false, nullptr, nullptr, 0);
  // join whatever was forked, also after a failed launch: the stream must not run ahead of its side streams
  for (int j = 0; j < side; ++j) FB_CUDA(dev, cudaStreamWaitEvent(main_stream, dev->join_ev[j], 0));
  return rc;
}
