// Prefill attention (many query positions, no mask or causal) on fp16 tensor cores.
//
// Bound: tensor cores; causal-effective flops 2 Sq (Sq + 1 + 2 (Skv - Sq)) D H per sequence.
// Replaces the reference's flash attention row program for Sq > 1
// (fusor-ml/tile-ir-kernels/src/kernels/row_program.rs:1210-1382; the math is
// fusor-ml/fusor/src/composite/flash_attention.rs:113-236: softmax(q k^T scale + mask) v with
// each KV head shared by `groups` query heads).
//
// One CTA = 64 query rows of one head (4 warps x 16 rows). Keys and values (fp16 cache rows)
// stream through a double-buffered shared-memory tile of 64 keys filled with 16-byte cp.async
// (rows past the valid length are zero-filled, so masked probabilities never meet garbage).
// S = Q K^T and O += P V run on mma.sync.m16n8k16 with fp32 accumulation; operands come out of
// XOR-swizzled shared memory with ldmatrix (transposed for V); the softmax is the online form in
// the exp2 domain, probabilities are rounded to fp16 for the second product. Tiles strictly
// below the diagonal skip the mask arithmetic; CTAs with the longest key range are scheduled
// first. The key count may come from device memory (graph replay).
#include "attn_mma.cuh"

namespace {

constexpr int PF_BQ = 64, PF_BKV = 64, PF_THREADS = 128;
static_assert(PF_BQ == PF_BKV, "the Q tile borrows the K half of the second buffer");

struct PrefillArgs {
  const float* q;      // [B, H, Sq, D] or [B, Sq, H, D]
  const __half* k;     // [B, Hkv, cap, D]
  const __half* v;
  float* out;          // same layout as q
  const int* skv_dev;  // if not null: valid keys = *skv_dev + sq
  int b, h, hkv, sq, skv, cap, groups, bshd, causal;
  float scale_log2;    // scale * log2(e)
};

template <int D>
__global__ void __launch_bounds__(PF_THREADS, 3)
attn_prefill_kernel(const PrefillArgs a) {
  constexpr int CH = D / 8;                    // 16-byte chunks per row
  constexpr int TILE = PF_BKV * D * 2;         // bytes of one K or V tile
  extern __shared__ __align__(128) uint8_t sm[];
  uint8_t* KV = sm;                            // [2 buffers][K | V]
  uint8_t* Qs = sm + 2 * TILE;                 // [64][D] fp16, in the K half of buffer 1: only needed
                                               // until the Q fragments sit in registers
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int qt = gridDim.x - 1 - blockIdx.x;   // longest key ranges first
  const int head = blockIdx.y, bi = blockIdx.z, kvh = head / a.groups;
  const int skv = a.skv_dev ? (*a.skv_dev + a.sq) : a.skv;
  const int off = skv - a.sq;                  // query i sees keys j <= i + off
  const int q0 = qt * PF_BQ;
  const int kmax = max(0, a.causal ? min(skv, q0 + PF_BQ + off) : skv);
  const int ntiles = (kmax + PF_BKV - 1) / PF_BKV;

  const size_t q_row = a.bshd ? (size_t)a.h * D : (size_t)D;
  const size_t q_base = (size_t)bi * a.h * a.sq * D + (a.bshd ? (size_t)head * D : (size_t)head * a.sq * D);
  const __half* kb = a.k + ((size_t)bi * a.hkv + kvh) * (size_t)a.cap * D;
  const __half* vb = a.v + ((size_t)bi * a.hkv + kvh) * (size_t)a.cap * D;

  auto load_tile = [&](int tile, int buf) {
    const int kt = tile * PF_BKV;
    const uint32_t kdst = pf_smem(KV + buf * 2 * TILE), vdst = kdst + TILE;
#pragma unroll
    for (int i = 0; i < PF_BKV * CH / PF_THREADS; ++i) {
      const int idx = tid + PF_THREADS * i, row = idx / CH, c = idx % CH;
      const bool valid = kt + row < skv;
      const size_t src = (size_t)(valid ? kt + row : 0) * D + c * 8;
      pf_cp16(kdst + pf_off<D>(row, c), kb + src, valid);
      pf_cp16(vdst + pf_off<D>(row, c), vb + src, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (ntiles > 0) load_tile(0, 0);

  // Q tile: f32 -> fp16 into swizzled shared memory (rows past Sq are zero)
  for (int idx = tid; idx < PF_BQ * D / 4; idx += PF_THREADS) {
    const int row = idx / (D / 4), c4 = idx % (D / 4);
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (q0 + row < a.sq) x = *reinterpret_cast<const float4*>(a.q + q_base + (size_t)(q0 + row) * q_row + c4 * 4);
    *reinterpret_cast<uint2*>(Qs + pf_off<D>(row, c4 >> 1) + (c4 & 1) * 8) = make_uint2(pf_pack(x.x, x.y), pf_pack(x.z, x.w));
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
  {
    const int j = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      pf_ldsm4(pf_smem(Qs) + pf_off<D>(warp * 16 + (j & 1) * 8 + r, 2 * ks + (j >> 1)), qf[ks]);
  }
  __syncthreads();  // buffer 1 may now be overwritten by the second K/V tile

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row_lo = q0 + warp * 16 + g;  // this thread's rows: row_lo and row_lo + 8

  for (int tile = 0; tile < ntiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < ntiles) {
      load_tile(tile + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const uint32_t ks_base = pf_smem(KV + buf * 2 * TILE), vs_base = ks_base + TILE;

    // ---- S = Q K^T: 8 column tiles of 8 keys
    float s[PF_BKV / 8][4];
#pragma unroll
    for (int nt = 0; nt < PF_BKV / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
    // K steps outermost: consecutive MMAs go to different accumulators
#pragma unroll
    for (int k2 = 0; k2 < D / 32; ++k2) {
#pragma unroll
      for (int nt = 0; nt < PF_BKV / 8; ++nt) {
        uint32_t b[4];  // keys nt*8.., K elements 32 k2 .. +31 as (b0, b1) of two k-steps
        pf_ldsm4(ks_base + pf_off<D>(nt * 8 + (lane & 7), 4 * k2 + (lane >> 3)), b);
        pf_mma(s[nt], qf[2 * k2], b[0], b[1]);
        pf_mma(s[nt], qf[2 * k2 + 1], b[2], b[3]);
      }
    }

    // ---- scale, mask (only on tiles that touch the diagonal or the end of the keys)
    const int kt = tile * PF_BKV;
    const bool need_mask = kt + PF_BKV > skv || (a.causal && kt + PF_BKV - 1 > q0 + warp * 16 + off);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < PF_BKV / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x = s[nt][e];  // raw score: the (positive) scale is folded into the exponent below
        if (need_mask) {
          const int col = kt + nt * 8 + 2 * t + (e & 1), row = row_lo + (e >> 1) * 8;
          if (col >= skv || (a.causal && col > row + off)) x = -INFINITY;
        }
        s[nt][e] = x;
        mx[e >> 1] = fmaxf(mx[e >> 1], x);
      }
    float alpha[2], msafe[2];
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
      mx[hrow] = fmaxf(mx[hrow], __shfl_xor_sync(0xFFFFFFFFu, mx[hrow], 1));
      mx[hrow] = fmaxf(mx[hrow], __shfl_xor_sync(0xFFFFFFFFu, mx[hrow], 2));
      const float mnew = fmaxf(m_run[hrow], mx[hrow] * a.scale_log2);
      msafe[hrow] = mnew == -INFINITY ? 0.f : mnew;  // a row that has seen no key yet
      alpha[hrow] = exp2f(m_run[hrow] - msafe[hrow]);
      m_run[hrow] = mnew;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < PF_BKV / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f(fmaf(s[nt][e], a.scale_log2, -msafe[e >> 1]));
        s[nt][e] = p;
        psum[e >> 1] += p;
      }
    l_run[0] = l_run[0] * alpha[0] + psum[0];
    l_run[1] = l_run[1] * alpha[1] + psum[1];
    // the running maximum settles after the first tiles: skip the rescale when no row of the warp moved
    if (__any_sync(0xFFFFFFFFu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
        o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
      }
    }

    // ---- O += P V: P (fp16) as the A operand, V through transposing ldmatrix
#pragma unroll
    for (int kk = 0; kk < PF_BKV / 16; ++kk) {
      uint32_t pa[4];
      pa[0] = pf_pack(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pf_pack(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pf_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pf_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      const int j = lane >> 3, r = lane & 7;
#pragma unroll
      for (int d2 = 0; d2 < D / 16; ++d2) {
        uint32_t b[4];  // keys kk*16.., dims 16 d2 .. +15 as (b0, b1) of two column tiles
        pf_ldsm4_t(vs_base + pf_off<D>(kk * 16 + (j & 1) * 8 + r, 2 * d2 + (j >> 1)), b);
        pf_mma(o[2 * d2], pa, b[0], b[1]);
        pf_mma(o[2 * d2 + 1], pa, b[2], b[3]);
      }
    }
    __syncthreads();  // every warp is done with this buffer before the tile after next lands in it
  }

  // ---- normalise and store
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    l_run[hrow] += __shfl_xor_sync(0xFFFFFFFFu, l_run[hrow], 1);
    l_run[hrow] += __shfl_xor_sync(0xFFFFFFFFu, l_run[hrow], 2);
  }
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    const int row = row_lo + 8 * hrow;
    if (row >= a.sq) continue;
    const float inv = l_run[hrow] > 0.f ? 1.0f / l_run[hrow] : 0.f;
    float* dst = a.out + q_base + (size_t)row * q_row + 2 * t;
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
      *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2 * hrow] * inv, o[i][2 * hrow + 1] * inv);
  }
}

}  // namespace

// Covers: no mask or causal, head size 64 / 128. Returns 1 when the shape is not covered (the
// caller then runs the general row kernel).
int fb200_launch_attention_prefill(fb200_device* dev, const float* q, const __half* k, const __half* v, int b, int h,
                                   int hkv, int sq, int skv, const int* skv_dev, int cap, int d, float scale,
                                   int causal, float* out, int bshd) {
  if ((d != 64 && d != 128) || h % hkv || b > 65535 || h > 65535 || !(scale > 0.f)) return 1;
  PrefillArgs a = {};
  a.q = q; a.k = k; a.v = v; a.out = out; a.skv_dev = skv_dev;
  a.b = b; a.h = h; a.hkv = hkv; a.sq = sq; a.skv = skv; a.cap = cap; a.groups = h / hkv; a.bshd = bshd;
  a.causal = causal; a.scale_log2 = scale * 1.4426950408889634f;
  const dim3 grid((unsigned)((sq + PF_BQ - 1) / PF_BQ), (unsigned)h, (unsigned)b);
  const size_t smem = (size_t)(4 * PF_BKV) * d * 2;
  static bool configured[64] = {false};
  if (!configured[dev->ordinal & 63]) {
    FB_CUDA(dev, cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * PF_BKV * 128 * 2));
    FB_CUDA(dev, cudaFuncSetAttribute(attn_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * PF_BKV * 64 * 2));
    configured[dev->ordinal & 63] = true;
  }
  if (d == 128) return fb200_launch(dev, attn_prefill_kernel<128>, grid, dim3(PF_THREADS), smem, false, a);
  return fb200_launch(dev, attn_prefill_kernel<64>, grid, dim3(PF_THREADS), smem, false, a);
}
