// KV cache (fp16, [B, Hkv, capacity, D]) and attention over it.
//
// attn_rows_kernel: one CTA takes up to 8 query rows that share a KV head (the G heads of a GQA
// group x consecutive query positions) and a contiguous slice of the keys ("split"). K and V
// are streamed once per CTA in 128-key chunks with online softmax; the rows reuse every K/V
// load, which is what makes GQA decode HBM-bound on the cache rather than on re-reads.
// Several splits of one row are merged by attn_combine_kernel in a fixed order.
// Replaces the reference's attention row program (fusor-ml/core/src/row_program.rs:1210-1382)
// and follows the arithmetic of the CPU composite
// (fusor-ml/fusor/src/composite/flash_attention.rs:113-236): scores * scale + mask, softmax, . v.
#include <algorithm>

#include "common.cuh"
#include "packed_act.cuh"
#include "attn_decode.cuh"

struct fb200_kv_cache {
  fb200_device* dev = nullptr;
  int batch = 0, n_kv_head = 0, head_dim = 0, max_seq_len = 0;
  int len = 0, capacity = 0;
  __half* k = nullptr;
  __half* v = nullptr;
};

int fb200_launch_attention_prefill(fb200_device* dev, const float* q, const __half* k, const __half* v, int b, int h,
                                   int hkv, int sq, int skv, const int* skv_dev, int cap, int d, float scale,
                                   int causal, float* out, int bshd);

int fb200_launch_attention_decode_tc(fb200_device* dev, const fb200_dec_args& a, int d);
int fb200_launch_attention_prefill_tc(fb200_device* dev, const float* q, const __half* k, const __half* v, int b, int h,
                                      int hkv, int sq, int skv, const int* skv_dev, int cap, int d, float scale,
                                      int causal, float* out, int bshd);

namespace {

constexpr int PREFILL_MIN_ROWS = 32;  // from here on the tensor-core prefill kernel takes over
constexpr int ROWS = 8;      // query rows per CTA
constexpr int CHUNK = 128;   // keys per smem chunk
constexpr int ATT_THREADS = 256;

struct AttnArgs {
  const float* q;      // [B, H, Sq, D]
  const __half* k;     // [B, Hkv, cap, D]
  const __half* v;
  float* out;          // [B, H, Sq, D]
  float* part;         // [nsplit][B*H*Sq][D + 2] when nsplit > 1
  const float* mask;
  const int* skv_dev;  // if not null: number of valid keys is read from here
  int b, h, hkv, sq, skv, cap, groups;
  int bshd;            // 1: q and out are [B, Sq, H, D] instead of [B, H, Sq, D]
  int mask_kind;       // 0 none, 1 causal, 2 [Sq,Skv], 3 [B,Skv]
  int nsplit, row_tiles;  // row tiles per (b, kv head)
  float scale;
};

__device__ __forceinline__ void att_pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void att_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <int D>
__global__ void __launch_bounds__(ATT_THREADS)
attn_rows_kernel(const AttnArgs a) {
  constexpr int DL = D / 4;  // dims per lane in the score phase (4 lanes per key)
  constexpr int DV = D / 32; // dims per lane in the value phase
  __shared__ float qs[ROWS][D];
  __shared__ float sc[ROWS][CHUNK];
  __shared__ float alpha[ROWS];
  __shared__ float row_m[ROWS], row_l[ROWS];
  __shared__ float ored[ATT_THREADS / 32][ROWS][D];  // cross-warp reduction of o
  static_assert(D == 64 || D == 128, "head_dim 64 or 128");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  att_pdl_launch();
  att_pdl_wait();
  const int skv = a.skv_dev ? (*a.skv_dev + a.sq) : a.skv;
  int bid = blockIdx.x;
  const int split = bid % a.nsplit; bid /= a.nsplit;
  const int rt = bid % a.row_tiles; bid /= a.row_tiles;
  const int kvh = bid % a.hkv;
  const int bi = bid / a.hkv;
  const int rows_total = a.groups * a.sq;  // rows sharing this kv head
  const int r0 = rt * ROWS;
  const int nrows = min(ROWS, rows_total - r0);

  // row r -> (head, query position): rows are ordered head-major inside the group
  auto row_head = [&](int r) { return kvh * a.groups + (r0 + r) / a.sq; };
  auto row_qi = [&](int r) { return (r0 + r) % a.sq; };
  auto row_index = [&](int r) -> size_t {
    return a.bshd ? ((size_t)bi * a.sq + row_qi(r)) * a.h + row_head(r)
                  : ((size_t)bi * a.h + row_head(r)) * a.sq + row_qi(r);
  };

  for (int i = tid; i < ROWS * D; i += ATT_THREADS) {
    int r = i / D, e = i % D;
    float v = 0.f;
    if (r < nrows) {
      v = a.q[row_index(r) * D + e];
    }
    qs[r][e] = v;
  }
  if (tid < ROWS) { row_m[tid] = -INFINITY; row_l[tid] = 0.f; }

  // keys visible to any row of this CTA, then this split's slice of them
  int kmax = skv;
  if (a.mask_kind == 1) {
    int lim = 0;
    for (int r = 0; r < nrows; ++r) lim = max(lim, row_qi(r) + (skv - a.sq) + 1);
    kmax = min(skv, lim);
  }
  const int per = (kmax + a.nsplit - 1) / a.nsplit;
  const int kbeg = min(kmax, split * per), kend = min(kmax, kbeg + per);

  const __half* kb = a.k + ((size_t)bi * a.hkv + kvh) * (size_t)a.cap * D;
  const __half* vb = a.v + ((size_t)bi * a.hkv + kvh) * (size_t)a.cap * D;

  float o[ROWS][DV];
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int e = 0; e < DV; ++e) o[r][e] = 0.f;
  __syncthreads();

  for (int c0 = kbeg; c0 < kend; c0 += CHUNK) {
    const int cn = min(CHUNK, kend - c0);
    // ---- phase 1: scores. 4 lanes per key, 8 keys per warp pass, 64 keys per CTA pass
    for (int j0 = 0; j0 < cn; j0 += 64) {
      const int j = j0 + warp * 8 + (lane >> 2);
      const int sub = lane & 3;
      float acc[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
      if (j < cn) {
        const uint4* kp = reinterpret_cast<const uint4*>(kb + (size_t)(c0 + j) * D + sub * DL);
#pragma unroll
        for (int v8 = 0; v8 < DL / 8; ++v8) {
          uint4 raw = kp[v8];
          const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
          float kf[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(h2[i]);
            kf[2 * i] = f.x; kf[2 * i + 1] = f.y;
          }
#pragma unroll
          for (int r = 0; r < ROWS; ++r) {
            const float* qr = &qs[r][sub * DL + v8 * 8];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[r] = fmaf(qr[i], kf[i], acc[r]);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        acc[r] += __shfl_xor_sync(0xFFFFFFFFu, acc[r], 1);
        acc[r] += __shfl_xor_sync(0xFFFFFFFFu, acc[r], 2);
      }
      if (j < cn && sub == 0) {
        const int key = c0 + j;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          float s = acc[r] * a.scale;
          if (r < nrows) {
            const int qi = row_qi(r);
            if (a.mask_kind == 1) {
              if (key > qi + (skv - a.sq)) s = -INFINITY;
            } else if (a.mask_kind == 2) {
              s += a.mask[(size_t)qi * skv + key];
            } else if (a.mask_kind == 3) {
              s += a.mask[(size_t)bi * skv + key];
            }
          }
          sc[r][j] = s;
        }
      }
    }
    __syncthreads();
    // ---- phase 2: online softmax statistics, warp r owns row r
    {
      const int r = warp;
      float mx = -INFINITY;
      for (int j = lane; j < cn; j += 32) mx = fmaxf(mx, sc[r][j]);
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o2));
      const float m_old = row_m[r];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int j = lane; j < cn; j += 32) {
        float p = (m_new == -INFINITY) ? 0.f : __expf(sc[r][j] - m_new);
        sc[r][j] = p;
        sum += p;
      }
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o2);
      if (lane == 0) {
        float al = (m_old == -INFINITY) ? 0.f : __expf(m_old - m_new);
        alpha[r] = al;
        row_l[r] = row_l[r] * al + sum;
        row_m[r] = m_new;
      }
    }
    __syncthreads();
    // ---- phase 3: o = o * alpha + p . v; warp w takes keys w, w+8, ...; lane owns DV dims
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float al = alpha[r];
#pragma unroll
      for (int e = 0; e < DV; ++e) o[r][e] *= al;
    }
    for (int j = warp; j < cn; j += ATT_THREADS / 32) {
      float vf[DV];
      const __half* vp = vb + (size_t)(c0 + j) * D + lane * DV;
      if constexpr (DV == 4) {
        uint2 raw = *reinterpret_cast<const uint2*>(vp);
        const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
        float2 f0 = __half22float2(h2[0]), f1 = __half22float2(h2[1]);
        vf[0] = f0.x; vf[1] = f0.y; vf[2] = f1.x; vf[3] = f1.y;
      } else {
        float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(vp));
        vf[0] = f0.x; vf[1] = f0.y;
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const float p = sc[r][j];
#pragma unroll
        for (int e = 0; e < DV; ++e) o[r][e] = fmaf(p, vf[e], o[r][e]);
      }
    }
    __syncthreads();
  }

  // ---- cross-warp reduction of o (each warp saw a different subset of the keys)
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int e = 0; e < DV; ++e) ored[warp][r][lane * DV + e] = o[r][e];
  __syncthreads();
  for (int i = tid; i < ROWS * D; i += ATT_THREADS) {
    const int r = i / D, e = i % D;
    if (r >= nrows) continue;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_THREADS / 32; ++w) s += ored[w][r][e];
    const size_t grow = row_index(r);
    if (a.nsplit == 1) {
      const float l = row_l[r];
      a.out[grow * D + e] = l > 0.f ? s / l : 0.f;
    } else {
      float* pp = a.part + ((size_t)split * ((size_t)a.b * a.h * a.sq) + grow) * (D + 2);
      pp[e] = s;
      if (e == 0) { pp[D] = row_m[r]; pp[D + 1] = row_l[r]; }
    }
  }
}

template <int D>
__global__ void attn_combine_kernel(const float* __restrict__ part, int nsplit, size_t rows,
                                    float* __restrict__ out) {
  const size_t row = blockIdx.x;
  const int e = threadIdx.x;  // blockDim.x == D
  float mx = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mx = fmaxf(mx, part[((size_t)s * rows + row) * (D + 2) + D]);
  float l = 0.f, acc = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float* pp = part + ((size_t)s * rows + row) * (D + 2);
    const float m = pp[D];
    const float w = (m == -INFINITY) ? 0.f : __expf(m - mx);
    l = fmaf(pp[D + 1], w, l);
    acc = fmaf(pp[e], w, acc);
  }
  out[row * D + e] = l > 0.f ? acc / l : 0.f;
}

// k, v f32 [B, Hkv, S, D] -> fp16 cache rows [pos .. pos + S)
__global__ void kv_append_kernel(const float* __restrict__ k, const float* __restrict__ v,
                                 __half* __restrict__ kc, __half* __restrict__ vc, int s, int d,
                                 int cap, int pos, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int e = (int)(i % d);
  const size_t t = i / d;
  const int si = (int)(t % s);
  const size_t bh = t / s;
  const size_t dst = (bh * cap + pos + si) * d + e;
  kc[dst] = __float2half_rn(k[i]);
  vc[dst] = __float2half_rn(v[i]);
}

__global__ void kv_grow_kernel(const __half* __restrict__ src, __half* __restrict__ dst, int len,
                               int d, int old_cap, int new_cap, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t per = (size_t)len * d;
  const size_t bh = i / per, r = i % per;
  dst[bh * (size_t)new_cap * d + r] = src[bh * (size_t)old_cap * d + r];
}

// gpu_allocation_seq_len, fusor-ml/fusor/src/cache/tensor_cache.rs:304-312
int kv_capacity_rule(int required, int max_len) {
  int min_alloc = std::min(256, max_len);
  int p = 1;
  while (p < required) p <<= 1;
  return std::min(std::max(p, min_alloc), max_len);
}


// ---- one new position per sequence (decode) -----------------------------------------------------
// RoPE(q), RoPE(k) + fp16 append, split-KV attention and the merge of the splits in one kernel.
// CTA = (batch, kv head, split); the G <= 8 query heads of the kv head share every K/V load.
// Under programmatic dependent launch the CTA copies its slice of the KV cache (written in
// earlier decode steps, never by the kernels just before this one) into shared memory with
// cp.async BEFORE griddepcontrol.wait, so the cache streams in while the q/k/v projection is
// still running; only q and the new k, v rows are read after the wait.
// One query position per sequence against a cache that already holds every key (q already
// rotated): the decode form of fb200_flash_attention. One CTA per (batch, KV head, split).
constexpr int DEC_CH = 64;   // keys per shared-memory chunk
constexpr int DEC_NB = 2;    // two staging buffers: the next chunk is copied while this one is used

template <int D, int ROWS_T>
__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_kernel(const fb200_dec_args a0) {
  extern __shared__ __align__(128) uint8_t dsm[];
  // The launch provides nsplit splits per (batch, kv head) for the longest context; a short context
  // uses the first few of them (at least min_keys keys each) and the other CTAs have nothing to do.
  fb200_dec_args a = a0;
  const int skv = a.pos_dev ? __ldcg(a.pos_dev) + 1 : a.skv;
  const int mk = a.min_keys > 0 ? a.min_keys : 64;
  const int ns = max(1, min(a.nsplit, (skv + mk - 1) / mk));
  const int split = (int)blockIdx.x % a.nsplit, rest = (int)blockIdx.x / a.nsplit;
  if (split >= ns) return;
  if (a.pos_dev) a.pos_plus1 = skv;
  a.nsplit = ns;
  attn_decode_item<D, DEC_CH, ROWS_T, 0, false, false, DEC_NB>(a, rest * ns + split, dsm, (int)threadIdx.x);
}

}  // namespace

int fb200_attention_scratch_bytes(int b, int h, int sq, int d, int nsplit, size_t* out) {
  *out = nsplit > 1 ? (size_t)nsplit * b * h * sq * (d + 2) * sizeof(float) : 0;
  return FB200_OK;
}

int fb200_attention_nsplit(const fb200_device* dev, int b, int hkv, int groups, int sq, int skv) {
  const int row_tiles = (groups * sq + ROWS - 1) / ROWS;
  const long base = (long)b * hkv * row_tiles;
  int want = (int)((2L * dev->sm_count + base - 1) / base);
  int maxs = std::max(1, skv / 256);
  return std::max(1, std::min(std::min(want, maxs), 64));
}

// Launches attention with explicit scratch and split count (used by the model's captured graph).
int fb200_launch_attention(fb200_device* dev, const float* q, const __half* k, const __half* v,
                           int b, int h, int hkv, int sq, int skv, const int* skv_dev, int cap,
                           int d, float scale, const float* mask, int mask_kind, float* out,
                           float* part, int nsplit, int bshd) {
  if (h % hkv) return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "attention: %d heads not divisible by %d kv heads", h, hkv);
  if (d != 64 && d != 128) return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "attention: head_dim %d (64 or 128 supported)", d);
  if (sq >= PREFILL_MIN_ROWS && mask_kind <= 1) {
    // many query positions, no mask or causal: the tensor-core kernels (tcgen05 for head size 128
    // and at least half a 128-row tile of queries, mma.sync otherwise)
    int rc = 1;
    if (sq >= 64) rc = fb200_launch_attention_prefill_tc(dev, q, k, v, b, h, hkv, sq, skv, skv_dev, cap, d, scale, mask_kind, out, bshd);
    if (rc == 1) rc = fb200_launch_attention_prefill(dev, q, k, v, b, h, hkv, sq, skv, skv_dev, cap, d, scale, mask_kind, out, bshd);
    if (rc != 1) return rc;
  }
  AttnArgs a = {};
  a.q = q; a.k = k; a.v = v; a.out = out; a.part = part; a.mask = mask; a.skv_dev = skv_dev;
  a.b = b; a.h = h; a.hkv = hkv; a.sq = sq; a.skv = skv; a.cap = cap; a.groups = h / hkv;
  a.mask_kind = mask_kind; a.nsplit = nsplit; a.scale = scale; a.bshd = bshd;
  a.row_tiles = (a.groups * sq + ROWS - 1) / ROWS;
  const long grid = (long)b * hkv * a.row_tiles * nsplit;
  if (grid <= 0) return FB200_OK;
  if (grid >= (1L << 31)) return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "attention: grid too large");
  int rc;
  if (d == 128) rc = fb200_launch(dev, attn_rows_kernel<128>, dim3((unsigned)grid), dim3(ATT_THREADS), 0, false, a);
  else rc = fb200_launch(dev, attn_rows_kernel<64>, dim3((unsigned)grid), dim3(ATT_THREADS), 0, false, a);
  if (rc) return rc;
  if (nsplit > 1) {
    const size_t rows = (size_t)b * h * sq;
    if (d == 128) attn_combine_kernel<128><<<(unsigned)rows, 128, 0, dev->stream>>>(part, nsplit, rows, out);
    else attn_combine_kernel<64><<<(unsigned)rows, 64, 0, dev->stream>>>(part, nsplit, rows, out);
    FB_LAUNCH_CHECK(dev);
  }
  return FB200_OK;
}

// Launches the decode attention kernel for prepared arguments (a.done must point to b * hkv
// zeroed arrival counters; the kernel leaves them zero again).
int fb200_launch_attention_decode_args(fb200_device* dev, const fb200_dec_args& a, int d) {
  // the tensor-core kernel covers every layout of the models; FB200_ATTN_DECODE_TC=0 keeps the scalar kernel
  static const bool no_tc = getenv("FB200_ATTN_DECODE_TC") && getenv("FB200_ATTN_DECODE_TC")[0] == '0';
  if (!no_tc) {
    const int rc = fb200_launch_attention_decode_tc(dev, a, d);
    if (rc != 1) return rc;
  }
  if (a.h % a.hkv || a.groups > DEC_ROWS || (d != 64 && d != 128) || a.nsplit < 1 || a.nsplit > 32)
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "attention_decode: unsupported head layout");
  const unsigned grid = (unsigned)(a.b * a.hkv * a.nsplit);
  const size_t smem = dec_smem_bytes(d, DEC_CH, DEC_NB);
  static bool configured[64] = {false};
  if (!configured[dev->ordinal & 63]) {
    FB_CUDA(dev, cudaFuncSetAttribute(attn_decode_kernel<128, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024));
    FB_CUDA(dev, cudaFuncSetAttribute(attn_decode_kernel<128, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024));
    FB_CUDA(dev, cudaFuncSetAttribute(attn_decode_kernel<64, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024));
    configured[dev->ordinal & 63] = true;
  }
  if (d == 128 && a.groups <= 4)
    return fb200_launch(dev, attn_decode_kernel<128, 4>, dim3(grid), dim3(DEC_THREADS), smem, false, a);
  if (d == 128) return fb200_launch(dev, attn_decode_kernel<128, 8>, dim3(grid), dim3(DEC_THREADS), smem, false, a);
  return fb200_launch(dev, attn_decode_kernel<64, 8>, dim3(grid), dim3(DEC_THREADS), smem, false, a);
}

// Decode form of flash_attention: sq = 1, no mask, q already rotated, nothing appended. `part`
// holds nsplit * b * h * (d + 2) floats followed by b * hkv arrival counters.
int fb200_launch_attention_decode(fb200_device* dev, const float* q, const __half* k, const __half* v, int b,
                                  int h, int hkv, int skv, int cap, int d, float scale, float* out, float* part,
                                  int nsplit) {
  fb200_dec_args a = {};
  a.q = q; a.kc = const_cast<__half*>(k); a.vc = const_cast<__half*>(v);
  a.pos_dev = nullptr; a.skv = skv; a.part = part; a.out = out;
  a.done = reinterpret_cast<int*>(part + (size_t)nsplit * b * h * (d + 2));
  a.b = b; a.h = h; a.hkv = hkv; a.groups = h / hkv; a.cap = cap; a.nsplit = nsplit; a.scale = scale;
  FB_CUDA(dev, cudaMemsetAsync(a.done, 0, (size_t)b * hkv * sizeof(int), dev->stream));
  return fb200_launch_attention_decode_args(dev, a, d);
}

int fb200_launch_kv_append(fb200_device* dev, const float* k, const float* v, __half* kc, __half* vc,
                           int bh, int s, int d, int cap, int pos) {
  const size_t total = (size_t)bh * s * d;
  if (!total) return FB200_OK;
  kv_append_kernel<<<(unsigned)((total + 255) / 256), 256, 0, dev->stream>>>(k, v, kc, vc, s, d, cap, pos, total);
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}

extern "C" {

int fb200_kv_cache_create(fb200_device* dev, int batch, int n_kv_head, int head_dim,
                          int max_seq_len, fb200_kv_cache** out) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!out) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "out is null");
  *out = nullptr;
  if (batch <= 0 || n_kv_head <= 0 || head_dim <= 0 || max_seq_len <= 0)
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "kv_cache_create: non-positive dimension");
  fb200_kv_cache* c = new fb200_kv_cache();
  c->dev = dev; c->batch = batch; c->n_kv_head = n_kv_head; c->head_dim = head_dim;
  c->max_seq_len = max_seq_len;
  *out = c;
  return FB200_OK;
}

int fb200_kv_cache_free(fb200_kv_cache* c) {
  if (!c) return FB200_OK;
  int rc = fb200_bind(c->dev);
  if (rc) return rc;
  cudaStreamSynchronize(c->dev->stream);
  if (c->k) cudaFree(c->k);
  if (c->v) cudaFree(c->v);
  delete c;
  return FB200_OK;
}

int fb200_kv_cache_reset(fb200_kv_cache* c) {
  if (!c) return FB200_ERR_INVALID_ARGUMENT;
  c->len = 0;
  return FB200_OK;
}

int fb200_kv_cache_truncate(fb200_kv_cache* c, int len) {
  if (!c) return FB200_ERR_INVALID_ARGUMENT;
  if (len < 0 || len > c->len)
    return fb200_fail(c->dev, FB200_ERR_INVALID_ARGUMENT, "kv cache: cannot truncate %d positions to %d", c->len, len);
  c->len = len;  // rows past len stay allocated and are overwritten by the next append
  return FB200_OK;
}

int fb200_kv_cache_len(const fb200_kv_cache* c, int* len_out, int* capacity_out) {
  if (!c) return FB200_ERR_INVALID_ARGUMENT;
  if (len_out) *len_out = c->len;
  if (capacity_out) *capacity_out = c->capacity;
  return FB200_OK;
}

int fb200_kv_cache_append(fb200_kv_cache* c, const float* k_dev, const float* v_dev, int s) {
  if (!c) return FB200_ERR_INVALID_ARGUMENT;
  fb200_device* dev = c->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (s <= 0) return FB200_OK;
  const int need = c->len + s;
  if (need > c->max_seq_len)
    return fb200_fail(dev, FB200_ERR_CAPACITY, "kv cache: %d positions exceed max_seq_len %d", need, c->max_seq_len);
  const size_t bh = (size_t)c->batch * c->n_kv_head;
  if (need > c->capacity) {
    const int ncap = kv_capacity_rule(need, c->max_seq_len);
    __half *nk = nullptr, *nv = nullptr;
    const size_t bytes = bh * ncap * c->head_dim * sizeof(__half);
    FB_CUDA(dev, cudaMalloc(&nk, bytes));
    cudaError_t e = cudaMalloc(&nv, bytes);
    if (e != cudaSuccess) { cudaFree(nk); return fb200_fail(dev, FB200_ERR_CUDA, "kv cache grow: %s", cudaGetErrorString(e)); }
    cudaMemsetAsync(nk, 0, bytes, dev->stream);
    cudaMemsetAsync(nv, 0, bytes, dev->stream);
    if (c->len > 0) {
      const size_t total = bh * c->len * c->head_dim;
      kv_grow_kernel<<<(unsigned)((total + 255) / 256), 256, 0, dev->stream>>>(c->k, nk, c->len, c->head_dim, c->capacity, ncap, total);
      dev->launches++;
      kv_grow_kernel<<<(unsigned)((total + 255) / 256), 256, 0, dev->stream>>>(c->v, nv, c->len, c->head_dim, c->capacity, ncap, total);
      dev->launches++;
    }
    FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
    if (c->k) cudaFree(c->k);
    if (c->v) cudaFree(c->v);
    c->k = nk; c->v = nv; c->capacity = ncap;
  }
  rc = fb200_launch_kv_append(dev, k_dev, v_dev, c->k, c->v, (int)bh, s, c->head_dim, c->capacity, c->len);
  if (rc) return rc;
  c->len = need;
  return FB200_OK;
}

int fb200_kv_cache_buffers(const fb200_kv_cache* c, const void** k_dev, const void** v_dev) {
  if (!c) return FB200_ERR_INVALID_ARGUMENT;
  if (k_dev) *k_dev = c->k;
  if (v_dev) *v_dev = c->v;
  return FB200_OK;
}

int fb200_flash_attention(fb200_device* dev, const float* q_dev, const void* k_dev,
                          const void* v_dev, int b, int h, int hkv, int sq, int skv,
                          int kv_capacity, int d, float scale, const float* mask_dev,
                          int mask_kind, float* out_dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!q_dev || !k_dev || !v_dev || !out_dev) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "attention: null argument");
  if (b <= 0 || h <= 0 || hkv <= 0 || sq <= 0 || skv < 0 || kv_capacity < skv)
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "attention: bad shape");
  if (mask_kind < 0 || mask_kind > 3 || (mask_kind >= 2 && !mask_dev))
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "attention: mask kind %d", mask_kind);
  fb200_op_trace scope(dev, sq == 1 ? "attention (decode)" : "attention (prefill)",
                       4.0 * (double)b * hkv * (double)skv * d + 8.0 * (double)b * h * (double)sq * d);
  if (sq == 1 && skv > 0 && (mask_kind == 0 || !mask_dev) && h % hkv == 0 && h / hkv <= DEC_ROWS && (d == 64 || d == 128)) {
    // decode form: as many (batch, KV head, split) items as run side by side (two per SM), at least 64 keys each
    int ns = 2 * dev->sm_count / (b * hkv);
    ns = std::max(1, std::min(std::min(ns, 32), (skv + 63) / 64));
    const size_t need = ((size_t)ns * b * h * (d + 2)) * sizeof(float) + (size_t)b * hkv * sizeof(int);
    rc = fb200_ensure(dev, &dev->stage, &dev->stage_bytes, need);
    if (rc) return rc;
    return fb200_launch_attention_decode(dev, q_dev, (const __half*)k_dev, (const __half*)v_dev, b, h, hkv, skv,
                                         kv_capacity, d, scale, out_dev, (float*)dev->stage, ns);
  }
  const int nsplit = fb200_attention_nsplit(dev, b, hkv, h / hkv, sq, skv);
  size_t bytes;
  fb200_attention_scratch_bytes(b, h, sq, d, nsplit, &bytes);
  float* part = nullptr;
  if (bytes) {
    rc = fb200_ensure(dev, &dev->stage, &dev->stage_bytes, bytes);
    if (rc) return rc;
    part = (float*)dev->stage;
  }
  return fb200_launch_attention(dev, q_dev, (const __half*)k_dev, (const __half*)v_dev, b, h, hkv,
                                sq, skv, nullptr, kv_capacity, d, scale, mask_dev, mask_kind,
                                out_dev, part, nsplit, 0);
}

}  // extern "C"
