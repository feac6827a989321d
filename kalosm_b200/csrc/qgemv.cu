// Quantised matrix x small-batch activation product (decode GEMV and M <= 32 "skinny" GEMM).
//
// Bound: HBM. Persistent CTAs (a multiple of the SM count) walk the 16-row tiles of W; inside a
// CTA the 8 warps take the K groups of a tile round robin. Every warp owns a private ring of
// shared-memory stages that it fills with 1-D TMA bulk copies (cp.async.bulk + mbarrier
// complete_tx), one tile-group (1.1 - 3.4 KB, contiguous in the tiled storage) per stage, several
// stages ahead of the math, so tens of KB per SM are in flight without holding registers. The
// first copies are issued before griddepcontrol.wait: under programmatic dependent launch the
// weights of this product stream in while the producer of the activations is still running.
// Each lane then reads its mma.m16n8k16 A-fragment bytes from the stage with conflict-free
// 128-bit shared loads (the tile-interleaved storage is already in fragment order), expands the
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
#include "qgemv_common.cuh"

namespace {

template <int TYPE>
struct Ring {
  static constexpr int TG = TYPE == FB200_Q4_0 ? 1152 : TYPE == FB200_Q8_0 ? 2176 : TYPE == FB200_Q4_K ? 2304 : 3360;
  static constexpr int STRIDE = (TG + 127) / 128 * 128;  // stage stride, keeps 128-byte alignment
  static constexpr int STAGES = TYPE == FB200_Q4_0 ? 8 : TYPE == FB200_Q6_K ? 3 : 4;
  static constexpr int RING_BYTES = GEMV_WARPS * STAGES * STRIDE;
  static constexpr int BAR_BYTES = GEMV_WARPS * STAGES * 8;
};

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

  int item = 0;
  for (int j = 0; j < my_units; ++j) {
    const int unit = (int)blockIdx.x + j * (int)gridDim.x;
    if (j > 0) __syncthreads();  // the previous unit's reduction has read `red`
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      float acc[NT][4];
      zero_c<NT>(acc);
      for (int kk = 0; kk < gw; ++kk, ++item) {
        const int st = item % S;
        mbar_wait(my_bar + 8 * st, (uint32_t)((item / S) & 1), a.status);
        const uint8_t* tg = my_ring + st * R::STRIDE;
        const int kg = warp + GEMV_WARPS * kk;
        if (TYPE == FB200_Q4_0) group_q4_0<NT>(a, tg, kg, lane, acc);
        else if (TYPE == FB200_Q8_0) group_q8_0<NT>(a, tg, kg, lane, acc);
        else if (TYPE == FB200_Q4_K) group_q4k<NT>(a, tg, kg, lane, acc);
        else group_q6k<NT>(a, tg, kg, lane, acc);
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
        out = v[0] + a.r1[idx];
        if (a.r2) out += a.r2[idx];
      } else {
        out = v[0];
      }
      a.y[idx] = out;
    }
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
