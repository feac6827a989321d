// Elementwise and row-wise ops of the decoder: RMSNorm (+residual), SiLU-gate, RoPE, embedding
// lookup, argmax. All are HBM/L2-bound single-pass kernels.
#include <cmath>
#include <vector>

#include "formats.cuh"

namespace {

__device__ __forceinline__ float block_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float s = 0.f;
  for (int i = 0; i < nw; ++i) s += sh[i];
  __syncthreads();
  return s;
}

// rms_norm_fused_cpu_impl, fusor-ml/fusor/src/composite/normalization.rs:404-461:
// mean of squares, + eps, sqrt, divide, * weight (+ bias). Residual form adds first (:392-395).
__global__ void __launch_bounds__(256)
rms_norm_kernel(const float* __restrict__ x, size_t x_stride, const float* __restrict__ res,
                const float* __restrict__ w, const float* __restrict__ b, float eps, int n,
                float* __restrict__ y) {
  __shared__ float sh[8];
  const size_t row = blockIdx.x;
  const float* xr = x + row * x_stride;
  const float* rr = res ? res + row * n : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) {
    float v = rr ? xr[i] + rr[i] : xr[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, sh);
  const float rms = sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += 256) {
    float v = rr ? xr[i] + rr[i] : xr[i];
    float o = (v / rms) * w[i];
    y[row * n + i] = b ? o + b[i] : o;
  }
}

// silu(gate) * up, fusor-ml/fusor/src/composite/activations.rs:47-64
__global__ void silu_mul_kernel(const float* __restrict__ g, const float* __restrict__ u, size_t n,
                                float* __restrict__ out) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    float x = g[i];
    out[i] = (x / (1.0f + expf(-x))) * u[i];
  }
}

// rope_interleaved / rope, fusor-ml/fusor/src/composite/rope.rs:46-108. One thread per pair.
__global__ void rope_kernel(float* __restrict__ x, int heads, int s, int d,
                            const float* __restrict__ cs, const float* __restrict__ sn,
                            int start_pos, int interleaved, size_t pairs) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs) return;
  const int half = d >> 1;
  const int p = (int)(i % half);
  const size_t vec = i / half;  // (b * heads + h) * s + si
  const int si = (int)(vec % s);
  float* v = x + vec * d;
  const float c = cs[(size_t)(start_pos + si) * half + p];
  const float sv = sn[(size_t)(start_pos + si) * half + p];
  if (interleaved) {
    float x0 = v[2 * p], x1 = v[2 * p + 1];
    v[2 * p] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sv));
    v[2 * p + 1] = __fadd_rn(__fmul_rn(x0, sv), __fmul_rn(x1, c));
  } else {
    float x0 = v[p], x1 = v[p + half];
    v[p] = __fadd_rn(__fmul_rn(x0, c), __fmul_rn(-x1, sv));
    v[p + half] = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, sv));
  }
  (void)heads;
}

// Tensor::top_k_pairs with k = 1, fusor-ml/fusor/src/lib.rs:416-453: highest finite logit,
// ties -> higher token id. One block per row.
__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, size_t n, uint32_t* __restrict__ ids,
              float* __restrict__ vals) {
  __shared__ float sv[32];
  __shared__ uint32_t si[32];
  const float* row = logits + (size_t)blockIdx.x * n;
  float best = -INFINITY;
  uint32_t bi = 0xFFFFFFFFu;
  for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
    float v = row[i];
    if (!isfinite(v)) continue;
    if (bi == 0xFFFFFFFFu || v > best || (v == best && (uint32_t)i > bi)) { best = v; bi = (uint32_t)i; }
  }
  auto better = [](float v, uint32_t i, float bv, uint32_t b) {
    if (i == 0xFFFFFFFFu) return false;
    if (b == 0xFFFFFFFFu) return true;
    return v > bv || (v == bv && i > b);
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
    uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
    if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0xFFFFFFFFu;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
      if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
      ids[blockIdx.x] = bi;
      if (vals) vals[blockIdx.x] = best;
    }
  }
}

}  // namespace

// Host-side table build, models/kalosm-llama/src/raw/rope.rs:9-85 (f32 arithmetic as there).
// `freq_weight` (optional, head_dim / 2 values): the rope_freqs.weight tensor of a checkpoint, which
// the reference multiplies into the inverse frequencies after the scaling (rope.rs:40-49).
void fb200_rope_tables_host(int head_dim, int ctx, float theta, float factor, float low_ff,
                            float high_ff, int original_ctx, const float* freq_weight,
                            std::vector<float>& cs, std::vector<float>& sn) {
  const int half = head_dim / 2;
  std::vector<float> inv(half);
  for (int i = 0; i < half; ++i) inv[i] = 1.0f / powf(theta, (float)(2 * i) / (float)head_dim);
  if (factor > 0.f) {
    const float PI = 3.14159265358979323846f;
    const float low_wavelen = (float)original_ctx / low_ff;
    const float high_wavelen = (float)original_ctx / high_ff;
    for (auto& f : inv) {
      float wavelen = 2.0f * PI / f;
      if (wavelen > low_wavelen) {
        f /= factor;
      } else if (wavelen == high_wavelen) {
        float smooth = ((float)original_ctx / wavelen - low_ff) / (high_ff - low_ff);
        f = (1.0f - smooth) * f / factor + smooth * f;
      }
    }
  }
  if (freq_weight)
    for (int i = 0; i < half; ++i) inv[i] = inv[i] * freq_weight[i];
  cs.resize((size_t)ctx * half);
  sn.resize((size_t)ctx * half);
  for (int p = 0; p < ctx; ++p)
    for (int i = 0; i < half; ++i) {
      float a = (float)p * inv[i];
      cs[(size_t)p * half + i] = cosf(a);
      sn[(size_t)p * half + i] = sinf(a);
    }
}

int fb200_launch_rms_norm(fb200_device* dev, const float* x, const float* res, const float* w,
                          const float* b, float eps, size_t rows, size_t n, float* y) {
  if (rows == 0 || n == 0) return FB200_OK;
  rms_norm_kernel<<<(unsigned)rows, 256, 0, dev->stream>>>(x, n, res, w, b, eps, (int)n, y);
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}

// Rows of x are x_stride elements apart (used to normalise only the last position of each
// sequence); residual and output rows are contiguous.
int fb200_launch_rms_norm_strided(fb200_device* dev, const float* x, size_t x_stride,
                                  const float* res, const float* w, float eps, size_t rows,
                                  size_t n, float* y) {
  if (rows == 0 || n == 0) return FB200_OK;
  rms_norm_kernel<<<(unsigned)rows, 256, 0, dev->stream>>>(x, x_stride, res, w, nullptr, eps, (int)n, y);
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}

int fb200_launch_rope(fb200_device* dev, float* x, int b, int heads, int s, int d, const float* cs,
                      const float* sn, int start_pos, int interleaved) {
  size_t pairs = (size_t)b * heads * s * (d / 2);
  if (pairs == 0) return FB200_OK;
  rope_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, dev->stream>>>(x, heads, s, d, cs, sn,
                                                                        start_pos, interleaved, pairs);
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}

// Two steps for wide rows: ARGMAX_PARTS CTAs per row leave their best (value, index) as an ordered
// 64-bit key (value in the high half, mapped so that unsigned order = float order; index in the
// low half, so that equal values resolve to the higher index), then one thread per row takes the
// largest key. One CTA per row would read a 128 256-wide row at a fraction of the bandwidth.
constexpr int ARGMAX_PARTS = 16;

__global__ void __launch_bounds__(512)
argmax_parts_kernel(const float* __restrict__ logits, size_t n, unsigned long long* __restrict__ part) {
  __shared__ unsigned long long sk[16];
  const float* row = logits + (size_t)blockIdx.y * n;
  const size_t per = (n + ARGMAX_PARTS - 1) / ARGMAX_PARTS;
  const size_t i0 = (size_t)blockIdx.x * per, i1 = i0 + per < n ? i0 + per : n;
  unsigned long long best = 0ull;  // 0: no finite value seen
  for (size_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
    const float v = row[i];
    if (!isfinite(v)) continue;
    const uint32_t u = __float_as_uint(v);
    const uint32_t ordered = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    const unsigned long long key = ((unsigned long long)ordered << 32) | (uint32_t)i;
    if (key > best) best = key;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, best, o);
    if (other > best) best = other;
  }
  if ((threadIdx.x & 31) == 0) sk[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i)
      if (sk[i] > best) best = sk[i];
    part[(size_t)blockIdx.y * ARGMAX_PARTS + blockIdx.x] = best;
  }
}

__global__ void argmax_pick_kernel(const unsigned long long* __restrict__ part, int rows, uint32_t* __restrict__ ids,
                                   float* __restrict__ vals) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  unsigned long long best = 0ull;
  for (int i = 0; i < ARGMAX_PARTS; ++i) {
    const unsigned long long k = part[(size_t)r * ARGMAX_PARTS + i];
    if (k > best) best = k;
  }
  ids[r] = best ? (uint32_t)(best & 0xFFFFFFFFull) : 0xFFFFFFFFu;
  if (vals) {
    const uint32_t o = (uint32_t)(best >> 32);
    vals[r] = best ? __uint_as_float((o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o) : -INFINITY;
  }
}

int fb200_launch_argmax(fb200_device* dev, const float* logits, size_t rows, size_t n,
                        uint32_t* ids, float* vals) {
  if (rows == 0) return FB200_OK;
  if (n < 16384 || rows > 65535) {
    argmax_kernel<<<(unsigned)rows, 1024, 0, dev->stream>>>(logits, n, ids, vals);
    FB_LAUNCH_CHECK(dev);
    return FB200_OK;
  }
  int rc = fb200_ensure(dev, &dev->argmax_part, &dev->argmax_part_bytes, rows * ARGMAX_PARTS * sizeof(unsigned long long));
  if (rc) return rc;
  unsigned long long* part = reinterpret_cast<unsigned long long*>(dev->argmax_part);
  argmax_parts_kernel<<<dim3(ARGMAX_PARTS, (unsigned)rows), 512, 0, dev->stream>>>(logits, n, part);
  FB_LAUNCH_CHECK(dev);
  argmax_pick_kernel<<<(unsigned)((rows + 127) / 128), 128, 0, dev->stream>>>(part, (int)rows, ids, vals);
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}

extern "C" {

int fb200_rms_norm(fb200_device* dev, const float* x_dev, const float* residual_dev,
                   const float* weight_dev, const float* bias_dev, float eps, size_t rows, size_t n,
                   float* y_dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!x_dev || !weight_dev || !y_dev) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "rms_norm: null argument");
  fb200_op_trace scope(dev, "rms_norm", 8.0 * (double)rows * (double)n);
  return fb200_launch_rms_norm(dev, x_dev, residual_dev, weight_dev, bias_dev, eps, rows, n, y_dev);
}

int fb200_silu_mul(fb200_device* dev, const float* gate_dev, const float* up_dev, size_t n,
                   float* out_dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (n == 0) return FB200_OK;
  fb200_op_trace scope(dev, "silu_mul", 12.0 * (double)n);
  silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(gate_dev, up_dev, n, out_dev);
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}

int fb200_rope_tables(fb200_device* dev, int head_dim, int ctx, float theta, float factor,
                      float low_freq_factor, float high_freq_factor, int original_ctx,
                      float* cos_dev, float* sin_dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (head_dim <= 0 || head_dim % 2 || ctx <= 0)
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "rope_tables: head_dim %d ctx %d", head_dim, ctx);
  std::vector<float> cs, sn;
  fb200_rope_tables_host(head_dim, ctx, theta, factor, low_freq_factor, high_freq_factor,
                         original_ctx, nullptr, cs, sn);
  FB_CUDA(dev, cudaMemcpyAsync(cos_dev, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, dev->stream));
  FB_CUDA(dev, cudaMemcpyAsync(sin_dev, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice, dev->stream));
  FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  return FB200_OK;
}

int fb200_rope_pair(fb200_device* dev, float* q_dev, float* k_dev, int b, int h, int hkv, int s,
                    int d, const float* cos_dev, const float* sin_dev, int start_pos,
                    int interleaved) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (d % 2) return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "rope: odd head_dim %d", d);
  fb200_op_trace scope(dev, "rope", 8.0 * (double)b * (double)(h + hkv) * (double)s * (double)d);
  if (q_dev && (rc = fb200_launch_rope(dev, q_dev, b, h, s, d, cos_dev, sin_dev, start_pos, interleaved))) return rc;
  if (k_dev && (rc = fb200_launch_rope(dev, k_dev, b, hkv, s, d, cos_dev, sin_dev, start_pos, interleaved))) return rc;
  return FB200_OK;
}

int fb200_embedding_lookup(fb200_device* dev, const fb200_qmatrix* w, const uint32_t* ids_dev,
                           size_t n_ids, float* out_dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!w || w->dev != dev) return fb200_fail(dev, FB200_ERR_DEVICE_MISMATCH, "embedding: bad weight handle");
  fb200_op_trace scope(dev, "embedding", 4.0 * (double)n_ids * (double)w->k);
  return fb200_launch_dequantize_rows(dev, w, ids_dev, n_ids, out_dev);
}

int fb200_argmax(fb200_device* dev, const float* logits_dev, size_t rows, size_t n,
                 uint32_t* ids_dev, float* vals_dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  fb200_op_trace scope(dev, "argmax", 4.0 * (double)rows * (double)n);
  return fb200_launch_argmax(dev, logits_dev, rows, n, ids_dev, vals_dev);
}

}  // extern "C"
