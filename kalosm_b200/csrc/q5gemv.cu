// Products with Q5_K weights, read in the byte order of the GGUF file.
// (Q5_0 needs no kernel of its own: it is widened to Q8_0 tiles when the matrix is built.)
//
// The reference's Tensor::q_mat_mul dequantises such a matrix and multiplies densely
// (fusor-ml/fusor/src/lib.rs:1184-1215; block layout fusor-ml/gguf/src/lib.rs:1819-1861). Here the
// blocks are expanded in registers and fed to mma.m16n8k16.f16:
//
//  * One persistent CTA of 16 warps per SM walks over tiles of 16 consecutive rows of W. The warps
//    take the 176-byte blocks of those rows in turn (warp w: blocks w, w + 16, ..) and their
//    partial sums are added in a fixed order in shared memory. Every warp keeps a ring of stages
//    in shared memory, each stage the same block of the 16 rows, fetched as one box of a 2-D
//    tensor map over W (cp.async.bulk.tensor.2d; 16 separate 176-byte row copies per stage run
//    into the request rate of the copy engine); the fetches stay several stages ahead of the
//    arithmetic, across tile boundaries.
//  * Lane (g = lane / 4, t = lane % 4) expands rows g and g + 8. Of every 32-element sub-block it
//    takes elements 4t .. 4t+3 and 16+4t .. 16+4t+3: two words 16 bytes apart of the quant field,
//    whose fifth bits sit at the same bit of four bytes of the high-bit field (one shift).
//  * A quant byte q becomes the half 1024 + q with one byte permute. Per sub-block the tensor cores
//    form sum((1024 + q) x) and, with an A operand of ones, sum(x), both with fp32 accumulation;
//    the sub-block's scale and offset are applied to those sums in fp32:
//    scale * sum((1024 + q) x) - (1024 scale + offset) * sum(x). The only rounding beyond fp32 is
//    the activations' (11 bits).
//  * The activation rows arrive packed (fb200_pack_x16): per chunk and row 64 bytes with lane t's
//    eight halves at byte 16 t, each row scaled by a power of two into (-64, 64).
//
// Bytes read per launch = the bytes of W + the packed activations (from L2 after the first CTA).
// The kernel is bound by instruction issue (the integer pipe that unpacks the quants), not by HBM.
#include <cstdlib>
#include <cstring>

#include <cuda.h>
#include <cuda_fp16.h>

#include "qgemv_common.cuh"

namespace {

constexpr int Q5K_WARPS = 16;
constexpr int Q5K_STAGE = 16 * 176;  // one block of each of the 16 rows

struct Q5Args {
  const uint8_t* w;     // raw row-major blocks
  const uint8_t* xh;    // packed activations: [K / 32][Mp][64 bytes]
  const float* xscale;  // [Mp] power-of-two scale of each packed row
  float* y;             // [M][N]
  const float* r1;      // optional rows added to y: r1_stride = N (a residual) or 0 (one bias row)
  const float* r2;      // optional second residual [M][N]
  int r1_stride;
  int M, Mp, N;
  int nblk;             // blocks per row
  int ntiles;           // ceil(N / 16)
  uint64_t row_bytes;
  int* status;          // device status word: a wait that gave up is recorded there
};

__device__ __forceinline__ void mma16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                      uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT>
struct XChunk { uint4 b[NT]; };

// Chunk kc of the packed rows 8 nt + g (rows M .. Mp - 1 are packed as zeros, so every lane loads);
// xl = xh + g * 64 + t * 16, the lane's place inside a chunk.
template <int NT>
__device__ __forceinline__ void load_x(const uint8_t* xl, int chunk_bytes, int kc, XChunk<NT>& x) {
  const uint8_t* p = xl + (size_t)kc * chunk_bytes;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) x.b[nt] = __ldg(reinterpret_cast<const uint4*>(p + nt * 512));
}
// D = A B with a zero C operand
__device__ __forceinline__ void mma16z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Adds the warps' partial sums in warp order and writes the tile's outputs.
// Accumulator i of lane (g, t) of n-tile nt: row g + 8 (i / 2), activation row 8 nt + 2t + i % 2.
template <int NT, int WARPS>
__device__ __forceinline__ void reduce_store(const Q5Args& a, const float (*red)[NT * 4][32], int row0) {
  for (int v = threadIdx.x; v < NT * 4 * 32; v += WARPS * 32) {
    const int idx = v >> 5, ln = v & 31;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) s += red[w][idx][ln];
    const int nt = idx >> 2, i = idx & 3;
    const int row = row0 + (ln >> 2) + 8 * (i >> 1);
    const int m = 8 * nt + 2 * (ln & 3) + (i & 1);
    if (row < a.N && m < a.M) {
      float out = s * a.xscale[m];
      if (a.r1) out += a.r1[(size_t)m * a.r1_stride + row];
      if (a.r2) out += a.r2[(size_t)m * a.N + row];
      a.y[(size_t)m * a.N + row] = out;
    }
  }
}

// ---- Q5_K: block = {f16 d, f16 dmin, scales[12], qh[32], qs[128]} (176 bytes) -------------------
// Sub-block j = 2c + hi (32 elements): nibble hi of qs[32c + l], bit j of qh[l], l = 0..31.
struct Raw5K {
  uint4 hd;           // d | dmin << 16, scales[12]
  uint32_t qh[2];     // qh words t and t + 4
  uint32_t qs[4][2];  // qs words 8c + t and 8c + t + 4
};

// `blk` = the block of one row in shared memory. Rows are 176 bytes apart: the 4-byte loads of
// lanes (g, t) fall into 32 different banks.
__device__ __forceinline__ void lds_q5k(const uint8_t* blk, int t, Raw5K& r) {
  r.hd = *reinterpret_cast<const uint4*>(blk);
  r.qh[0] = *reinterpret_cast<const uint32_t*>(blk + 16 + 4 * t);
  r.qh[1] = *reinterpret_cast<const uint32_t*>(blk + 32 + 4 * t);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    r.qs[c][0] = *reinterpret_cast<const uint32_t*>(blk + 48 + 32 * c + 4 * t);
    r.qs[c][1] = *reinterpret_cast<const uint32_t*>(blk + 64 + 32 * c + 4 * t);
  }
}

// Activation chunks are fetched XPF chunks ahead of their use (they come from L2: the ring leaves
// little L1), across the boundary between two super-blocks.
template <int NT>
struct XPipe {
  static constexpr int PF = NT == 1 ? 3 : 1;  // 8 % (PF + 1) == 0: the slots line up again after a super-block
  XChunk<NT> slot[PF + 1];
};

// One super-block (8 chunks) of rows g / g + 8; kc0 = index of its first chunk, whose first PF
// chunks are in xp on entry; on exit xp holds the first PF chunks of the super-block that starts
// at chunk next_kc0 (-1: none follows).
template <int NT>
__device__ __forceinline__ void step_q5k(const uint8_t* xl, int chunk_bytes, const Raw5K (&r)[2], int kc0, int next_kc0,
                                         XPipe<NT>& xp, float (&acc)[NT][4]) {
  constexpr int PF = XPipe<NT>::PF;
  const uint32_t ones = 0x3C003C00u;
  float sc[2][8], off[2][8];  // d * scale and 1024 d scale + dmin min of the eight sub-blocks
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t s0 = r[h].hd.y, s1 = r[h].hd.z, s2 = r[h].hd.w;
    // get_scale_min_k4 on four sub-blocks at a time: one byte per sub-block
    const uint32_t sc_w[2] = {s0 & 0x3F3F3F3Fu, (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u)};
    const uint32_t mn_w[2] = {s1 & 0x3F3F3F3Fu, ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u)};
    const float d = __half2float(__ushort_as_half((unsigned short)(r[h].hd.x & 0xFFFFu)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(r[h].hd.x >> 16)));
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      sc[h][j] = d * (float)((sc_w[j >> 2] >> (8 * (j & 3))) & 0xFFu);
      off[h][j] = fmaf(1024.f, sc[h][j], dmin * (float)((mn_w[j >> 2] >> (8 * (j & 3))) & 0xFFu));
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = j >> 1, hi = j & 1;
    // chunk j + PF: of this super-block, or of the next one
    if (j + PF < 8) load_x<NT>(xl, chunk_bytes, kc0 + j + PF, xp.slot[(j + PF) % (PF + 1)]);
    else if (next_kc0 >= 0) load_x<NT>(xl, chunk_bytes, next_kc0 + j + PF - 8, xp.slot[(j + PF) % (PF + 1)]);
    const XChunk<NT>& x = xp.slot[j % (PF + 1)];
    uint32_t av[2][2][2];  // [part][row half][k pair]: halves 1024 + q
#pragma unroll
    for (int part = 0; part < 2; ++part)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t w = r[h].qs[c][part];
        const uint32_t nib = (hi ? (w >> 4) : w) & 0x0F0F0F0Fu;
        const int sh = 4 - j;  // bit j of every byte -> bit 4
        const uint32_t hb = sh >= 0 ? (r[h].qh[part] << (sh & 31)) : (r[h].qh[part] >> ((-sh) & 31));
        const uint32_t v = nib | (hb & 0x10101010u);
        av[part][h][0] = __byte_perm(v, 0x64646464u, 0x4140u);
        av[part][h][1] = __byte_perm(v, 0x64646464u, 0x4342u);
      }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float qx[4], sx[4];
      mma16z(qx, av[0][0][0], av[0][1][0], av[0][0][1], av[0][1][1], x.b[nt].x, x.b[nt].y);
      mma16(qx, av[1][0][0], av[1][1][0], av[1][0][1], av[1][1][1], x.b[nt].z, x.b[nt].w);
      mma16z(sx, ones, ones, ones, ones, x.b[nt].x, x.b[nt].y);
      mma16(sx, ones, ones, ones, ones, x.b[nt].z, x.b[nt].w);
      acc[nt][0] = fmaf(sc[0][j], qx[0], fmaf(-off[0][j], sx[0], acc[nt][0]));
      acc[nt][1] = fmaf(sc[0][j], qx[1], fmaf(-off[0][j], sx[1], acc[nt][1]));
      acc[nt][2] = fmaf(sc[1][j], qx[2], fmaf(-off[1][j], sx[2], acc[nt][2]));
      acc[nt][3] = fmaf(sc[1][j], qx[3], fmaf(-off[1][j], sx[3], acc[nt][3]));
    }
  }
}

template <int NT>
struct Q5KSmem {
  static constexpr int STAGES = NT == 4 ? 3 : 4;
  static constexpr int RING = Q5K_WARPS * STAGES * Q5K_STAGE;
  static constexpr int BARS = Q5K_WARPS * STAGES * 8;
  static constexpr int RED = 2 * Q5K_WARPS * NT * 4 * 32 * (int)sizeof(float);  // two buffers: one barrier per tile
  static constexpr int BYTES = RING + BARS + RED;
};

// y[m, n] = xscale[m] * sum_k xh[m, k] * W[n, k] (+ r1 + r2) for M <= 8 NT activation rows.
// TENSOR: a stage arrives as one box of a 2-D tensor map over W ([N rows] x [row bytes as 32-bit
// words], box = 44 words x 16 rows; rows beyond N arrive as zeros) instead of 16 row copies: the
// copy engine takes one request per 2816 bytes instead of one per 176, which is what bounds the
// kernel otherwise.
template <int NT, bool TENSOR>
__global__ void __launch_bounds__(Q5K_WARPS * 32, 1) q5k_gemv_kernel(const Q5Args a, const __grid_constant__ CUtensorMap wmap) {
  using SM = Q5KSmem<NT>;
  constexpr int S = SM::STAGES;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::RING);
  float (*red)[Q5K_WARPS][NT * 4][32] = reinterpret_cast<float (*)[Q5K_WARPS][NT * 4][32]>(smem + SM::RING + SM::BARS);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* my_ring = smem + warp * S * Q5K_STAGE;
  const uint32_t my_bar = smem_u32(bars + warp * S);
  pdl_launch_dependents();
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < S; ++s) mbar_init(my_bar + 8 * s, TENSOR ? 1 : 16);  // one arrival per copying lane
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // this warp's items: for each of the CTA's tiles, the blocks warp, warp + 16, ..
  const int bw = a.nblk > warp ? (a.nblk - warp + Q5K_WARPS - 1) / Q5K_WARPS : 0;
  const int my_tiles = a.ntiles > (int)blockIdx.x ? (a.ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int n_items = my_tiles * bw;
  const uint64_t pol = l2_evict_first_policy();
  auto issue = [&](int i) {  // TENSOR: lane 0; else lanes 0..15, lane = row of the tile (rows beyond N repeat the last row)
    const int j = i / bw, kk = i - j * bw;
    const int tile = (int)blockIdx.x + j * (int)gridDim.x;
    const int st = i % S;
    if constexpr (TENSOR) {
      mbar_expect_tx(my_bar + 8 * st, Q5K_STAGE);
      asm volatile(
          "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
          ::"r"(smem_u32(my_ring + st * Q5K_STAGE)), "l"(&wmap), "r"((warp + Q5K_WARPS * kk) * 44), "r"(tile * 16),
            "r"(my_bar + 8 * st), "l"(pol) : "memory");
    } else {
      const uint8_t* src =
          a.w + (uint64_t)min(tile * 16 + lane, a.N - 1) * a.row_bytes + (size_t)(warp + Q5K_WARPS * kk) * 176;
      mbar_expect_tx(my_bar + 8 * st, 176);
      bulk_g2s_stream(smem_u32(my_ring + st * Q5K_STAGE + lane * 176), src, 176, my_bar + 8 * st, pol);
    }
  };
  const bool copier = TENSOR ? lane == 0 : lane < 16;
  if (copier) {
    const int pre = n_items < S ? n_items : S;
    for (int i = 0; i < pre; ++i) issue(i);
  }
  // everything above touches only the weights; the packed activations come from the kernel before
  // this one (launched with programmatic stream serialization: it may still be running)
  pdl_wait();
  const uint8_t* xl = a.xh + g * 64 + t * 16;
  const int chunk_bytes = a.Mp * 64;
  XPipe<NT> xp;
  if (n_items > 0) {
#pragma unroll
    for (int i = 0; i < XPipe<NT>::PF; ++i) load_x<NT>(xl, chunk_bytes, warp * 8 + i, xp.slot[i]);
  }
  int item = 0;
  for (int j = 0; j < my_tiles; ++j) {
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
    for (int kk = 0; kk < bw; ++kk, ++item) {
      const int st = item % S;
      mbar_wait(my_bar + 8 * st, (uint32_t)((item / S) & 1), a.status);
      const uint8_t* stage = my_ring + st * Q5K_STAGE;
      Raw5K r[2];
      lds_q5k(stage + g * 176, t, r[0]);
      lds_q5k(stage + (g + 8) * 176, t, r[1]);
      // the warp's next super-block: its next block of this tile, or block `warp` of the next tile
      const int next_kc0 = kk + 1 < bw ? (warp + Q5K_WARPS * (kk + 1)) * 8 : (item + 1 < n_items ? warp * 8 : -1);
      step_q5k<NT>(xl, chunk_bytes, r, (warp + Q5K_WARPS * kk) * 8, next_kc0, xp, acc);
      __syncwarp();  // every lane has read the stage before it is refilled
      if (copier && item + S < n_items) issue(item + S);
    }
    float (*rb)[NT * 4][32] = red[j & 1];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) rb[warp][nt * 4 + i][lane] = acc[nt][i];
    __syncthreads();
    reduce_store<NT, Q5K_WARPS>(a, rb, ((int)blockIdx.x + j * (int)gridDim.x) * 16);
  }
}

typedef CUresult (*q5_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
q5_encode_fn q5_encoder() {
  static q5_encode_fn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<q5_encode_fn>(p);
  }();
  return fn;
}

// W as [N][row_bytes / 4] 32-bit words, boxes of 44 words (one block) x 16 rows.
bool q5_make_map(CUtensorMap* map, const Q5Args& a) {
  q5_encode_fn enc = q5_encoder();
  if (!enc) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)(a.row_bytes / 4), (cuuint64_t)a.N};
  const cuuint64_t strides[1] = {(cuuint64_t)a.row_bytes};
  const cuuint32_t box[2] = {44, 16};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(a.w), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NT, bool TENSOR>
int launch_q5k_form(fb200_device* dev, const Q5Args& a, const CUtensorMap& map) {
  static bool attr_set[64] = {};
  if (dev->ordinal < 0 || dev->ordinal >= 64 || !attr_set[dev->ordinal]) {
    FB_CUDA(dev, cudaFuncSetAttribute(q5k_gemv_kernel<NT, TENSOR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Q5KSmem<NT>::BYTES));
    if (dev->ordinal >= 0 && dev->ordinal < 64) attr_set[dev->ordinal] = true;
  }
  const int grid = a.ntiles < dev->sm_count ? a.ntiles : dev->sm_count;
  return fb200_launch(dev, q5k_gemv_kernel<NT, TENSOR>, dim3(grid), dim3(Q5K_WARPS * 32), (size_t)Q5KSmem<NT>::BYTES, true,
                      a, map);
}

// FB200_Q5K_TENSOR_TMA=0 keeps the per-row copies (also taken when the driver offers no tensor-map encoder).
template <int NT>
int launch_q5k(fb200_device* dev, const Q5Args& a) {
  static const bool rows_only = getenv("FB200_Q5K_TENSOR_TMA") && getenv("FB200_Q5K_TENSOR_TMA")[0] == '0';
  CUtensorMap map;
  if (!rows_only && q5_make_map(&map, a)) return launch_q5k_form<NT, true>(dev, a, map);
  memset(&map, 0, sizeof(map));
  return launch_q5k_form<NT, false>(dev, a, map);
}

int launch_q5(fb200_device* dev, const Q5Args& a, int nt) {
  return nt == 1 ? launch_q5k<1>(dev, a) : nt == 2 ? launch_q5k<2>(dev, a) : launch_q5k<4>(dev, a);
}

}  // namespace

size_t fb200_xpack_bytes(int mp, uint64_t kp);
int fb200_pack16_rows(int mc);
int fb200_pack_x16(fb200_device* dev, const float* x, int mc, uint64_t k, uint64_t kp, void* scratch, const void** xh,
                   const float** xscale);

bool fb200_q5_covers(const fb200_qmatrix* w) {
  return !w->tiled && w->type == FB200_Q5_K && w->n < (1ull << 31) && w->k > 0 && w->k < (1ull << 31) &&
         w->data && (reinterpret_cast<uintptr_t>(w->data) & 15u) == 0;
}

// y = x . W^T (+ r1 + r2) for a Q5_K matrix (kept in raw form); any number of rows, 32 at a
// time (each pass reads W once). r1_is_bias: r1 is one row shared by all activation rows.
int fb200_q5_mat_mul(fb200_device* dev, const fb200_qmatrix* w, const float* x, size_t m, float* y, const float* r1,
                     const float* r2, bool r1_is_bias) {
  const int be = 256, bb = 176;
  int rc = fb200_ensure(dev, &dev->xpack, &dev->xpack_bytes, fb200_xpack_bytes(32, w->k));
  if (rc) return rc;
  for (size_t m0 = 0; m0 < m; m0 += 32) {
    const int mc = (int)((m - m0) < 32 ? (m - m0) : 32);
    const void* xh;
    const float* xs;
    rc = fb200_pack_x16(dev, x + m0 * w->k, mc, w->k, w->k, dev->xpack, &xh, &xs);
    if (rc) return rc;
    Q5Args a;
    a.w = w->data;
    a.xh = reinterpret_cast<const uint8_t*>(xh);
    a.xscale = xs;
    a.y = y + m0 * w->n;
    a.r1 = r1 ? r1 + (r1_is_bias ? 0 : m0 * w->n) : nullptr;
    a.r2 = r2 ? r2 + m0 * w->n : nullptr;
    a.r1_stride = r1_is_bias ? 0 : (int)w->n;
    a.M = mc;
    a.Mp = fb200_pack16_rows(mc);
    a.N = (int)w->n;
    a.nblk = (int)(w->k / be);
    a.ntiles = (a.N + 15) / 16;
    a.row_bytes = (uint64_t)a.nblk * bb;
    a.status = dev->status;
    rc = launch_q5(dev, a, a.Mp / 8);
    if (rc) return rc;
  }
  return FB200_OK;
}
