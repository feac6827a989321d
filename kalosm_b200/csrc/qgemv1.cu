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
#include "qgemv1_groups.cuh"

namespace {

struct Gemv1Args {
  const uint8_t* w;     // tiled weight bytes
  float* y;             // [n_out]
  int tg;               // bytes per tile-group
  int n_out;
  const float* x;       // [K]
  const float* xres;    // optional [K]: v = x + xres
  const float* norm_w;  // optional [K]: activation = v / sqrt(mean(v^2) + eps) * norm_w
  float eps;
  int K, Kp;            // logical and padded (ngroups * group_elems) inner size
  const float* r1;
  const float* r2;
  int ngroups, nunits, pair_tile_offset, stages, stride;
  int* status;
};

// TYPE: ggml type of the matrix. EPI: 0 none, 1 residual(s), 2 SwiGLU pair. W = warps per CTA,
// MINB = CTAs per SM.
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

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Lane L = make_lane(lane);
  uint8_t* my_ring = ring + warp * S * a.stride;
  const uint32_t my_bar = smem_u32(bars + warp * S);

  pdl_launch_dependents();
  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(my_bar + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // this warp's items in issue order: for each unit of the CTA, for each pass (gate / up), the
  // K groups warp, warp + W, ...
  const int gw = a.ngroups > warp ? (a.ngroups - warp + W - 1) / W : 0;
  const int my_units = a.nunits > (int)blockIdx.x ? (a.nunits - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int n_items = my_units * NP * gw;
  int is_unit = blockIdx.x, is_p = 0, is_kk = 0, issued = 0;  // issue-side cursor (lane 0)
  auto issue_next = [&](int st) {
    const uint8_t* src = a.w + ((size_t)(is_unit + is_p * a.pair_tile_offset) * a.ngroups + (warp + W * is_kk)) * a.tg;
    mbar_expect_tx(my_bar + 8 * st, a.tg);
    bulk_g2s(smem_u32(my_ring + st * a.stride), src, a.tg, my_bar + 8 * st);
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
  const float final_scale = 1.0f;  // the scale of the limbs travels in xsc
  {
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
      // per-16 sums in the units of the integer dot products (128 * sum(v) = sum(q) / 2^14);
      // the shuffle also orders the reads above before the writes below: a block's limbs go to
      // the place of another block of the same aligned group of four (limb_block)
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
      __syncwarp();
      if (kb < nblk) {
        uint4* dst = reinterpret_cast<uint4*>(xl + (size_t)limb_block(kb) * 32);
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
  constexpr int BLOCKS16 = (TYPE == FB200_Q4_K || TYPE == FB200_Q6_K) ? 16 : 8;  // 16-element blocks per K group
  for (int j = 0; j < my_units; ++j) {
    const int tile = (int)blockIdx.x + j * (int)gridDim.x;
    if (j > 0) __syncthreads();  // the previous unit's reduction has read `red`
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      float acc_g = 0.f, acc_g8 = 0.f;
      GroupPtrs G = group_ptrs(L, xl, xsc, xss, warp, BLOCKS16);
      for (int kk = 0; kk < gw; ++kk, ++item) {
        mbar_wait(my_bar + 8 * st, phase, a.status);
        const uint8_t* tg = my_ring + st * a.stride;
        group1_any(TYPE, G, tg, L, acc_g, acc_g8);
        // Every lane has read the stage (its loads precede this barrier in program order and
        // shared loads complete long before a refill from global memory can land).
        __syncwarp();
        if (lane == 0 && issued < n_items) issue_next(st);
        if (++st == S) { st = 0; phase ^= 1u; }
        group_ptrs_next(G, BLOCKS16 * W);  // K group warp + W * (kk + 1)
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
      float v[NP];
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        float s = 0.f;
        for (int w = 0; w < W; ++w) s += red[(p * W + w) * 16 + r];
        v[p] = s * final_scale;
      }
      if (n < a.n_out) {
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

template <int EPI, int W>
size_t gemv1_smem(int stages, int stride, int kp) {
  constexpr int NP = EPI == 2 ? 2 : 1;
  return (size_t)W * stages * stride + (size_t)W * stages * 8 + (size_t)kp * 4 + (size_t)kp / 16 * 4 +
         (size_t)kp / 16 * 4 + (size_t)NP * W * 16 * 4 + (size_t)2 * W * 4 + 64;
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

// y[n] = epilogue(W . act(x)) for one activation row; act = optional residual add + RMSNorm
// (norm_w != null).
int fb200_qgemv1(fb200_device* dev, const fb200_qmatrix* w, const float* x, const float* xres,
                 const float* norm_w, float eps, float* y, int epi, const float* r1,
                 const float* r2) {
  TileGeom geo;
  if (!w->tiled || !tile_geom(w->type, &geo))
    return fb200_fail(dev, FB200_ERR_UNSUPPORTED_DTYPE, "qgemv1: type %u has no tiled storage", w->type);
  Gemv1Args a = {};
  a.w = w->data; a.y = y; a.tg = geo.tg_bytes; a.n_out = (int)w->n;
  a.nunits = w->ntiles;
  a.stride = (geo.tg_bytes + 127) / 128 * 128;
  a.x = x; a.xres = xres; a.norm_w = norm_w; a.eps = eps;
  a.K = (int)w->k; a.Kp = w->ngroups * geo.group_elems;
  a.r1 = r1; a.r2 = r2;
  a.ngroups = w->ngroups; a.pair_tile_offset = 0;
  a.stages = 2; a.status = dev->status;
  if (epi == FB200_EPI_SWIGLU) {
    a.nunits = w->ntiles / 2;
    a.n_out = (int)(w->n / 2);
    a.pair_tile_offset = w->ntiles / 2;
  }
  switch (w->type) {
    case FB200_Q4_K: return launch_typed<FB200_Q4_K>(dev, a, epi);
    case FB200_Q6_K: return launch_typed<FB200_Q6_K>(dev, a, epi);
    case FB200_Q8_0: return launch_typed<FB200_Q8_0>(dev, a, epi);
    default: return launch_typed<FB200_Q4_0>(dev, a, epi);
  }
}
