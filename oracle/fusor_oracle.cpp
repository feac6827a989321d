// CPU oracle for the Fusor quantized-inference path.
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. It restates, in plain C++, the CPU
// algorithms of floneum/kalosm's Fusor runtime so the CUDA kernels have something to be
// checked against, and so a CPU baseline can be timed. Only tests, the smoke check and the
// benchmark's CPU-baseline leg may load it; the CUDA library never links or calls it.
//
// Pinning: the reference is Rust and cannot be compiled where this is built, so the oracle is
// pinned by the reference's own known-answer tests (see tests/test_oracle_golden.py):
// Q4_0/Q5_0/Q8_0 GEMV -> [528, -528], Q5_K -> 32896, Q5_K literal blocks, RoPE table
// literals, KV capacity literals, and the conformance fixture byte generators.
//
// Every function cites the reference file:line it follows (paths inside floneum/kalosm).
// Floating point order: dequantisation is written so that each output needs exactly the
// reference's roundings (no FMA contraction: build this file with -ffp-contract=off).
// The dot product keeps the reference's structure: a vector accumulator of LANES partial
// sums fed by fused multiply-add (pulp's mul_add_f32s), reduced at the end. LANES is fixed
// at 8 (the AVX2 width pulp picks on x86-64-v3) so results do not depend on the host.

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

#define ORACLE_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int LANES = 8;

// ---- ggml type ids: fusor-ml/gguf/src/lib.rs:35-50 ------------------------------------
enum GgmlType : uint32_t {
  F32 = 0, F16 = 1, Q4_0 = 2, Q5_0 = 6, Q8_0 = 8, Q4K = 12, Q5K = 13, Q6K = 14,
};

// (elements, bytes) per block: fusor-ml/gguf/src/lib.rs:99-121
bool block_geometry(uint32_t ty, int* elems, int* bytes) {
  switch (ty) {
    case Q4_0: *elems = 32; *bytes = 18; return true;
    case Q5_0: *elems = 32; *bytes = 22; return true;
    case Q8_0: *elems = 32; *bytes = 34; return true;
    case Q4K: *elems = 256; *bytes = 144; return true;
    case Q5K: *elems = 256; *bytes = 176; return true;
    case Q6K: *elems = 256; *bytes = 210; return true;
    default: return false;
  }
}

// IEEE binary16 -> binary32, exact (what half::f16::to_f32 does).
inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
      man &= 0x3FFu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

// binary32 -> binary16, round to nearest even (half::f16::from_f32).
inline uint16_t f32_to_f16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t absx = x & 0x7FFFFFFFu;
  if (absx >= 0x7F800000u) {  // inf / nan
    return (uint16_t)(sign | 0x7C00u | (absx > 0x7F800000u ? 0x200u : 0));
  }
  if (absx >= 0x477FF000u) {  // rounds to >= 65520 -> inf
    return (uint16_t)(sign | 0x7C00u);
  }
  if (absx < 0x33000001u) {  // below half of the smallest subnormal
    return (uint16_t)sign;
  }
  int exp = (int)(absx >> 23) - 127;
  uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
  int shift;
  uint32_t base;
  if (exp < -14) {  // subnormal half
    shift = 13 + (-14 - exp);
    base = 0;
  } else {
    shift = 13;
    base = (uint32_t)(exp + 15) << 10;
    man &= 0x7FFFFFu;
  }
  uint32_t q = man >> shift;
  uint32_t rem = man & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  return (uint16_t)(sign | (base + q));
}

inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// ---- per-block dequantisation -----------------------------------------------------------

// BlockQ4_0::dequantize, fusor-ml/gguf/src/lib.rs:828-846
void deq_q4_0(const uint8_t* b, float* out) {
  float scale = f16_to_f32(rd16(b));
  const uint8_t* qs = b + 2;
  for (int i = 0; i < 16; ++i) {
    int lo = (int)(qs[i] & 0x0F) - 8;
    int hi = (int)(qs[i] >> 4) - 8;
    out[i] = (float)lo * scale;
    out[i + 16] = (float)hi * scale;
  }
}

// BlockQ5_0::dequantize, fusor-ml/gguf/src/lib.rs:1046-1073
void deq_q5_0(const uint8_t* b, float* out) {
  float scale = f16_to_f32(rd16(b));
  uint32_t high_bits = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) |
                       ((uint32_t)b[5] << 24);
  const uint8_t* qs = b + 6;
  for (int i = 0; i < 16; ++i) {
    uint8_t low = qs[i] & 0x0F;
    uint8_t high = qs[i] >> 4;
    uint8_t low_bit = (uint8_t)((high_bits >> i) << 4) & 0x10;
    uint8_t high_bit = (uint8_t)(high_bits >> (i + 12)) & 0x10;
    int lo = (int)(low | low_bit) - 16;
    int hi = (int)(high | high_bit) - 16;
    out[i] = (float)lo * scale;
    out[i + 16] = (float)hi * scale;
  }
}

// BlockQ8_0::dequantize, fusor-ml/gguf/src/lib.rs:1284-1288
void deq_q8_0(const uint8_t* b, float* out) {
  float scale = f16_to_f32(rd16(b));
  const int8_t* qs = (const int8_t*)(b + 2);
  for (int i = 0; i < 32; ++i) out[i] = (float)qs[i] * scale;
}

// unpack_k4_scales_offsets, fusor-ml/gguf/src/lib.rs:2138-2208: twelve packed bytes ->
// eight 6-bit scales and eight 6-bit offsets.
void unpack_k4(const uint8_t* p, uint8_t* sc, uint8_t* mn) {
  for (int j = 0; j < 4; ++j) {
    sc[j] = p[j] & 63;
    mn[j] = p[j + 4] & 63;
    sc[j + 4] = (uint8_t)(((p[j] >> 6) << 4) | (p[j + 8] & 0x0F));
    mn[j + 4] = (uint8_t)(((p[j + 4] >> 6) << 4) | (p[j + 8] >> 4));
  }
}

// BlockQ4K::dequantize, fusor-ml/gguf/src/lib.rs:1526-1556
void deq_q4k(const uint8_t* b, float* out) {
  float d = f16_to_f32(rd16(b));
  float dmin = f16_to_f32(rd16(b + 2));
  uint8_t sc[8], mn[8];
  unpack_k4(b + 4, sc, mn);
  const uint8_t* qs = b + 16;
  for (int j = 0; j < 4; ++j) {
    float low_scale = (float)sc[2 * j] * d;
    float low_off = (float)mn[2 * j] * dmin;
    float high_scale = (float)sc[2 * j + 1] * d;
    float high_off = (float)mn[2 * j + 1] * dmin;
    for (int l = 0; l < 32; ++l) {
      uint8_t w = qs[32 * j + l];
      float a = low_scale * (float)(w & 0xF);
      out[64 * j + l] = a - low_off;
      float c = high_scale * (float)(w >> 4);
      out[64 * j + 32 + l] = c - high_off;
    }
  }
}

// BlockQ5K::dequantize, fusor-ml/gguf/src/lib.rs:1819-1861
void deq_q5k(const uint8_t* b, float* out) {
  float d = f16_to_f32(rd16(b));
  float dmin = f16_to_f32(rd16(b + 2));
  uint8_t sc[8], mn[8];
  unpack_k4(b + 4, sc, mn);
  const uint8_t* qh = b + 16;
  const uint8_t* qs = b + 48;
  uint8_t u1 = 1, u2 = 2;
  for (int chunk = 0; chunk < 4; ++chunk) {
    float d1 = (float)sc[2 * chunk] * d;
    float m1 = (float)mn[2 * chunk] * dmin;
    float d2 = (float)sc[2 * chunk + 1] * d;
    float m2 = (float)mn[2 * chunk + 1] * dmin;
    for (int l = 0; l < 32; ++l) {
      uint8_t ql = qs[32 * chunk + l];
      int q_lo = (ql & 0xF) + ((qh[l] & u1) ? 16 : 0);
      float a = d1 * (float)q_lo;
      out[64 * chunk + l] = a - m1;
    }
    for (int l = 0; l < 32; ++l) {
      uint8_t ql = qs[32 * chunk + l];
      int q_hi = (ql >> 4) + ((qh[l] & u2) ? 16 : 0);
      float a = d2 * (float)q_hi;
      out[64 * chunk + 32 + l] = a - m2;
    }
    u1 = (uint8_t)(u1 << 2);
    u2 = (uint8_t)(u2 << 2);
  }
}

// BlockQ6K::dequantize, fusor-ml/gguf/src/lib.rs:2034-2085
void deq_q6k(const uint8_t* b, float* out) {
  const uint8_t* ql = b;
  const uint8_t* qh = b + 128;
  const int8_t* scales = (const int8_t*)(b + 192);
  float d = f16_to_f32(rd16(b + 208));
  for (int c = 0; c < 2; ++c) {
    for (int l = 0; l < 32; ++l) {
      int is = 8 * c + l / 16;
      uint8_t h = qh[32 * c + l];
      uint8_t l0 = ql[64 * c + l];
      uint8_t l1 = ql[64 * c + l + 32];
      int q1 = (int)(int8_t)(((h & 3) << 4) | (l0 & 0xF)) - 32;
      int q2 = (int)(int8_t)((((h >> 2) & 3) << 4) | (l1 & 0xF)) - 32;
      int q3 = (int)(int8_t)((((h >> 4) & 3) << 4) | (l0 >> 4)) - 32;
      int q4 = (int)(int8_t)((((h >> 6) & 3) << 4) | (l1 >> 4)) - 32;
      // `scale * scales[i] as f32 * q as f32` evaluates left to right.
      float s1 = d * (float)scales[is];
      float s2 = d * (float)scales[is + 2];
      float s3 = d * (float)scales[is + 4];
      float s4 = d * (float)scales[is + 6];
      out[128 * c + l] = s1 * (float)q1;
      out[128 * c + l + 32] = s2 * (float)q2;
      out[128 * c + l + 64] = s3 * (float)q3;
      out[128 * c + l + 96] = s4 * (float)q4;
    }
  }
}

typedef void (*deq_fn)(const uint8_t*, float*);

deq_fn deq_for(uint32_t ty) {
  switch (ty) {
    case Q4_0: return deq_q4_0;
    case Q5_0: return deq_q5_0;
    case Q8_0: return deq_q8_0;
    case Q4K: return deq_q4k;
    case Q5K: return deq_q5k;
    case Q6K: return deq_q6k;
    default: return nullptr;
  }
}

// ---- threading ----------------------------------------------------------------------------

// num_threads(), fusor-ml/cpu/src/parallel.rs:12-23 (available_parallelism); the caller may
// override it so tests are independent of the host.
std::atomic<int> g_threads{0};

int num_threads() {
  int t = g_threads.load();
  if (t > 0) return t;
  unsigned hc = std::thread::hardware_concurrency();
  return hc ? (int)hc : 1;
}

template <class F>
void run_threads(int n, F&& f) {
  if (n <= 1) { f(0); return; }
  std::vector<std::thread> th;
  th.reserve(n);
  for (int i = 0; i < n; ++i) th.emplace_back([&f, i] { f(i); });
  for (auto& t : th) t.join();
}

// ---- quantised dot / matmul ---------------------------------------------------------------

// Horizontal sum of the vector accumulator (SumOp::reduce_simd_vec): halves, quarters, pair.
inline float hsum(const float* a) {
  float b[4];
  for (int i = 0; i < 4; ++i) b[i] = a[i] + a[i + 4];
  float c0 = b[0] + b[2];
  float c1 = b[1] + b[3];
  return c0 + c1;
}

// compute_dot_product, fusor-ml/cpu/src/quantized.rs:641-675
float dot_row(deq_fn deq, int bs, int bbytes, const float* x, const uint8_t* w, size_t n_out,
              size_t blocks_per_row) {
  float acc[LANES] = {0, 0, 0, 0, 0, 0, 0, 0};
  float tmp[256];
  const uint8_t* row = w + n_out * blocks_per_row * (size_t)bbytes;
  for (size_t kb = 0; kb < blocks_per_row; ++kb) {
    deq(row + kb * bbytes, tmp);
    const float* xb = x + kb * bs;
    for (int i = 0; i < bs; i += LANES)
      for (int l = 0; l < LANES; ++l) acc[l] = std::fmaf(xb[i + l], tmp[i + l], acc[l]);
  }
  return hsum(acc) + 0.0f;  // + scalar tail accumulator, always empty for these block sizes
}

// process_row_simd_tiled, fusor-ml/cpu/src/quantized.rs:562-637 (four output columns share one
// pass over the activation row; each column still has its own vector accumulator, so the
// arithmetic per output equals dot_row's).
void row_tiled(deq_fn deq, int bs, int bbytes, const float* x, const uint8_t* w, float* out,
               size_t n, size_t blocks_per_row) {
  size_t n_tiles = n / 4;
  float tmp[4][256];
  for (size_t tile = 0; tile < n_tiles; ++tile) {
    size_t base = tile * 4;
    float acc[4][LANES];
    std::memset(acc, 0, sizeof(acc));
    for (size_t kb = 0; kb < blocks_per_row; ++kb) {
      for (int c = 0; c < 4; ++c)
        deq(w + ((base + c) * blocks_per_row + kb) * (size_t)bbytes, tmp[c]);
      const float* xb = x + kb * bs;
      for (int i = 0; i < bs; i += LANES)
        for (int c = 0; c < 4; ++c)
          for (int l = 0; l < LANES; ++l)
            acc[c][l] = std::fmaf(xb[i + l], tmp[c][i + l], acc[c][l]);
    }
    for (int c = 0; c < 4; ++c) out[base + c] = hsum(acc[c]) + 0.0f;
  }
  for (size_t i = n_tiles * 4; i < n; ++i)
    out[i] = dot_row(deq, bs, bbytes, x, w, i, blocks_per_row);
}

// QMatmulSimd::with_simd, fusor-ml/cpu/src/quantized.rs:381-538 — same partitioning:
// m == 1 and n >= 64: 32-column chunks dealt to threads; m >= 4: rows dealt to threads;
// m in {2,3}: sequential.
int q_mat_mul_impl(const float* x, size_t m, size_t k, const uint8_t* w, uint32_t ty, size_t n,
                   float* y) {
  int bs, bbytes;
  if (!block_geometry(ty, &bs, &bbytes)) return -2;
  if (k % (size_t)bs != 0) return -1;
  deq_fn deq = deq_for(ty);
  size_t bpr = k / bs;
  int nt = num_threads();
  if (m == 1) {
    if (n < 64 || nt == 1) {
      row_tiled(deq, bs, bbytes, x, w, y, n, bpr);
    } else {
      const size_t CHUNK = 32;
      size_t total_chunks = (n + CHUNK - 1) / CHUNK;
      size_t chunks_per_thread = (total_chunks + nt - 1) / nt;
      size_t per_thread = chunks_per_thread * CHUNK;
      run_threads(nt, [&](int t) {
        size_t start = (size_t)t * per_thread;
        if (start >= n) return;
        size_t end = (t == nt - 1) ? n : std::min(n, start + per_thread);
        for (size_t i = start; i < end; ++i) y[i] = dot_row(deq, bs, bbytes, x, w, i, bpr);
      });
    }
  } else if (m >= 4 && nt > 1) {
    size_t rows_per_thread = (m + nt - 1) / nt;
    run_threads(nt, [&](int t) {
      size_t r0 = (size_t)t * rows_per_thread;
      if (r0 >= m) return;
      size_t r1 = (t == nt - 1) ? m : std::min(m, r0 + rows_per_thread);
      for (size_t r = r0; r < r1; ++r) row_tiled(deq, bs, bbytes, x + r * k, w, y + r * n, n, bpr);
    });
  } else {
    for (size_t r = 0; r < m; ++r) row_tiled(deq, bs, bbytes, x + r * k, w, y + r * n, n, bpr);
  }
  return 0;
}

// ---- elementwise / composite ops ----------------------------------------------------------

// rms_norm_fused_cpu_impl, fusor-ml/fusor/src/composite/normalization.rs:404-461:
// x^2 -> mean -> +eps -> sqrt -> x / rms -> * w (-> + b). The residual form adds first
// (normalization.rs:392-395). Mean = sum in index order divided by the length.
void rms_norm_row(const float* x, const float* res, const float* w, const float* b, float eps,
                  size_t n, float* y) {
  float sum = 0.0f;
  for (size_t i = 0; i < n; ++i) {
    float v = res ? x[i] + res[i] : x[i];
    y[i] = v;
    sum += v * v;
  }
  float mean = sum / (float)n;
  float rms = std::sqrt(mean + eps);
  for (size_t i = 0; i < n; ++i) {
    float v = (y[i] / rms) * w[i];
    y[i] = b ? v + b[i] : v;
  }
}

// silu, fusor-ml/fusor/src/composite/activations.rs:47-64: x / (1 + exp(-x))
inline float silu(float x) { return x / (std::exp(-x) + 1.0f); }

// ---- Llama oracle state ---------------------------------------------------------------------

struct QMat {
  uint32_t ty = 0;
  size_t n = 0, k = 0;
  std::vector<uint8_t> bytes;
};

struct Layer {
  QMat wq, wk, wv, wo, gate, up, down;
  std::vector<float> attn_norm, ffn_norm;
};

struct Llama {
  int n_layer = 0, hidden = 0, ffn = 0, n_head = 0, n_kv_head = 0, head_dim = 0, vocab = 0;
  int ctx = 0;
  float eps = 1e-5f, theta = 10000.f;
  bool kv_f16 = false;  // round K/V to binary16 on append (the CUDA path keeps an fp16 cache)
  int batch = 1;
  QMat token_embd, output;
  std::vector<float> output_norm;
  std::vector<Layer> layers;
  std::vector<float> cos, sin;        // [ctx, head_dim/2]
  std::vector<float> kcache, vcache;  // [layer][batch][kv_head][ctx][head_dim]
  int pos = 0;
};

}  // namespace

// =================================================================================================
// C API (ctypes)
// =================================================================================================

ORACLE_API void oracle_set_threads(int n) { g_threads.store(n); }
ORACLE_API int oracle_num_threads() { return num_threads(); }

ORACLE_API int oracle_block_geometry(uint32_t ty, int* elems, int* bytes) {
  return block_geometry(ty, elems, bytes) ? 0 : -2;
}

ORACLE_API float oracle_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
ORACLE_API uint16_t oracle_f32_to_f16(float f) { return f32_to_f16(f); }

// QuantizedTensor::dequantize, fusor-ml/cpu/src/quantized.rs:130-146: block outputs concatenated.
ORACLE_API int oracle_dequantize(const uint8_t* bytes, uint32_t ty, size_t n_elems, float* out) {
  int bs, bbytes;
  if (!block_geometry(ty, &bs, &bbytes)) return -2;
  if (n_elems % (size_t)bs) return -1;
  deq_fn deq = deq_for(ty);
  size_t nb = n_elems / bs;
  int nt = nb > 4096 ? num_threads() : 1;
  run_threads(nt, [&](int t) {
    size_t b0 = nb * t / nt, b1 = nb * (t + 1) / nt;
    for (size_t b = b0; b < b1; ++b) deq(bytes + b * bbytes, out + b * bs);
  });
  return 0;
}

// ConcreteTensor::q_mat_mul, fusor-ml/cpu/src/quantized.rs:246-365 (contiguous x[M,K], W[N,K]).
ORACLE_API int oracle_q_mat_mul(const float* x, size_t m, size_t k, const uint8_t* w, uint32_t ty,
                                size_t n, float* y) {
  return q_mat_mul_impl(x, m, k, w, ty, n, y);
}

ORACLE_API void oracle_rms_norm(const float* x, const float* residual, const float* w,
                                const float* bias, float eps, size_t rows, size_t n, float* y) {
  for (size_t r = 0; r < rows; ++r)
    rms_norm_row(x + r * n, residual ? residual + r * n : nullptr, w, bias, eps, n, y + r * n);
}

ORACLE_API void oracle_silu_mul(const float* gate, const float* up, size_t n, float* out) {
  for (size_t i = 0; i < n; ++i) out[i] = silu(gate[i]) * up[i];
}

// RoPE tables: base_inverse_frequency (fusor-ml/fusor/src/composite/rope.rs:241-246) and the
// outer product with positions followed by sin/cos (models/kalosm-llama/src/raw/rope.rs:63-85).
// Llama-3 frequency scaling (kalosm-llama raw/rope.rs:21-38) applies when factor > 0.
// freq_weight (optional): rope_freqs.weight, multiplied into the inverse frequencies after the
// scaling (models/kalosm-llama/src/raw/rope.rs:40-49).
ORACLE_API void oracle_rope_tables_w(int head_dim, int ctx, float theta, float factor,
                                     float low_freq_factor, float high_freq_factor,
                                     int original_ctx, const float* freq_weight, float* cos_out, float* sin_out);

ORACLE_API void oracle_rope_tables(int head_dim, int ctx, float theta, float factor,
                                   float low_freq_factor, float high_freq_factor,
                                   int original_ctx, float* cos_out, float* sin_out) {
  oracle_rope_tables_w(head_dim, ctx, theta, factor, low_freq_factor, high_freq_factor, original_ctx, nullptr,
                       cos_out, sin_out);
}

ORACLE_API void oracle_rope_tables_w(int head_dim, int ctx, float theta, float factor,
                                     float low_freq_factor, float high_freq_factor,
                                     int original_ctx, const float* freq_weight, float* cos_out, float* sin_out) {
  int half = head_dim / 2;
  std::vector<float> inv(half);
  for (int i = 0; i < half; ++i)
    inv[i] = 1.0f / std::pow(theta, (float)(2 * i) / (float)head_dim);
  if (factor > 0.0f) {
    const float PI = 3.14159265358979323846f;
    float low_wavelen = (float)original_ctx / low_freq_factor;
    float high_wavelen = (float)original_ctx / high_freq_factor;
    for (auto& f : inv) {
      float wavelen = 2.0f * PI / f;
      if (wavelen > low_wavelen) {
        f /= factor;
      } else if (wavelen == high_wavelen) {
        float smooth = ((float)original_ctx / wavelen - low_freq_factor) /
                       (high_freq_factor - low_freq_factor);
        f = (1.0f - smooth) * f / factor + smooth * f;
      }
    }
  }
  if (freq_weight)
    for (int i = 0; i < half; ++i) inv[i] = inv[i] * freq_weight[i];
  for (int p = 0; p < ctx; ++p)
    for (int i = 0; i < half; ++i) {
      float a = (float)p * inv[i];
      cos_out[(size_t)p * half + i] = std::cos(a);
      sin_out[(size_t)p * half + i] = std::sin(a);
    }
}

// rope_interleaved (fusor-ml/fusor/src/composite/rope.rs:77-108): pairs (2p, 2p+1),
// y0 = x0*c - x1*s, y1 = x0*s + x1*c; half-split `rope` (rope.rs:46-68) pairs (p, p+D/2):
// y = x*cos + rotate_half(x)*sin. x is [B, H, S, D]; row s uses table row start_pos + s
// (RopeCache::forward_interleaved, rope.rs:309-329).
ORACLE_API void oracle_rope(float* x, int b, int h, int s, int d, const float* cos_t,
                            const float* sin_t, int start_pos, int interleaved) {
  int half = d / 2;
  for (int bi = 0; bi < b; ++bi)
    for (int hi = 0; hi < h; ++hi)
      for (int si = 0; si < s; ++si) {
        float* v = x + (((size_t)bi * h + hi) * s + si) * d;
        const float* c = cos_t + (size_t)(start_pos + si) * half;
        const float* sn = sin_t + (size_t)(start_pos + si) * half;
        if (interleaved) {
          for (int p = 0; p < half; ++p) {
            float x0 = v[2 * p], x1 = v[2 * p + 1];
            float ac = x0 * c[p], bs = x1 * sn[p];
            float as = x0 * sn[p], bc = x1 * c[p];
            v[2 * p] = ac - bs;
            v[2 * p + 1] = as + bc;
          }
        } else {
          for (int p = 0; p < half; ++p) {
            float x0 = v[p], x1 = v[p + half];
            float a0 = x0 * c[p], r0 = (-x1) * sn[p];
            float a1 = x1 * c[p], r1 = x0 * sn[p];
            v[p] = a0 + r0;
            v[p + half] = a1 + r1;
          }
        }
      }
}

// Attention as the CPU composite computes it, fusor-ml/fusor/src/composite/flash_attention.rs:113-236:
// scores = q.k^T; *scale; + mask; max; exp(s - max); sum; divide; .v — GQA by kv_head = head / groups.
// The dense matmuls go to the third-party `gemm` crate (0.19.0) in the reference; its summation
// order is not pinned, so sequential index order is used here (as the reference's scalar test
// reference does, fusor-ml/core/tests/attention.rs:25-81).
// q [B,H,Sq,D], k/v [B,Hkv,Skv,D] with row stride kv_stride (elements between consecutive heads'
// row 0 is kv_stride*D), mask: null, or [Sq,Skv] additive (mask_kind 0/2), or [B,Skv] (mask_kind 1).
// causal != 0 builds the strict causal mask of AttentionMask::causal (attention_mask.rs:45-65),
// left-padded with zeros for earlier cache positions (mask_cache.rs:74-85).
ORACLE_API void oracle_attention(const float* q, const float* k, const float* v, int b, int h,
                                 int hkv, int sq, int skv, int d, size_t kv_head_stride,
                                 float scale, const float* mask, int mask_kind, int causal,
                                 float* out) {
  int groups = h / hkv;
  int total = b * h;
  int nt = std::min(num_threads(), total);
  std::atomic<int> next{0};
  run_threads(nt, [&](int) {
    std::vector<float> s(skv);
    for (;;) {
      int idx = next.fetch_add(1);
      if (idx >= total) break;
      int bi = idx / h, hi = idx % h;
      int kvh = hi / groups;
      const float* kb = k + ((size_t)bi * hkv + kvh) * kv_head_stride;
      const float* vb = v + ((size_t)bi * hkv + kvh) * kv_head_stride;
      for (int qi = 0; qi < sq; ++qi) {
        const float* qr = q + (((size_t)bi * h + hi) * sq + qi) * d;
        float mx = -std::numeric_limits<float>::infinity();
        for (int j = 0; j < skv; ++j) {
          const float* kr = kb + (size_t)j * d;
          float acc = 0.0f;
          for (int e = 0; e < d; ++e) acc += qr[e] * kr[e];
          acc = acc * scale;
          if (mask) {
            acc += (mask_kind == 1) ? mask[(size_t)bi * skv + j] : mask[(size_t)qi * skv + j];
          }
          if (causal && j > qi + (skv - sq)) acc += -std::numeric_limits<float>::infinity();
          s[j] = acc;
          mx = std::max(mx, acc);
        }
        float sum = 0.0f;
        for (int j = 0; j < skv; ++j) {
          s[j] = std::exp(s[j] - mx);
          sum += s[j];
        }
        float* o = out + (((size_t)bi * h + hi) * sq + qi) * d;
        for (int e = 0; e < d; ++e) o[e] = 0.0f;
        for (int j = 0; j < skv; ++j) {
          float p = s[j] / sum;
          const float* vr = vb + (size_t)j * d;
          for (int e = 0; e < d; ++e) o[e] += p * vr[e];
        }
      }
    }
  });
}

// gpu_allocation_seq_len, fusor-ml/fusor/src/cache/tensor_cache.rs:304-312
ORACLE_API size_t oracle_kv_capacity(size_t required, size_t max_len) {
  size_t min_alloc = std::min<size_t>(256, max_len);
  size_t p = 1;
  while (p < required) p <<= 1;
  return std::min(std::max(p, min_alloc), max_len);
}

// Tensor::top_k_pairs, fusor-ml/fusor/src/lib.rs:416-453: descending logit, ties -> higher id
// first; non-finite logits skipped. Returns the number of pairs written.
ORACLE_API int oracle_top_k(const float* logits, size_t n, int k, uint32_t* ids, float* vals) {
  std::vector<std::pair<uint32_t, float>> top;
  if (k <= 0) return 0;
  for (size_t i = 0; i < n; ++i) {
    float l = logits[i];
    if (!std::isfinite(l)) continue;
    if ((int)top.size() == k) {
      auto last = top.back();
      if (l > last.second || (l == last.second && (uint32_t)i > last.first)) top.pop_back();
      else continue;
    }
    size_t ins = 0;
    while (ins < top.size() &&
           (top[ins].second > l || (top[ins].second == l && top[ins].first > (uint32_t)i)))
      ++ins;
    top.insert(top.begin() + ins, {(uint32_t)i, l});
  }
  for (size_t i = 0; i < top.size(); ++i) { ids[i] = top[i].first; vals[i] = top[i].second; }
  return (int)top.size();
}


// ---- samplers: models/kalosm-llama/src/sampler.rs ----------------------------------------------
// The uniform draw: the reference takes rand::StdRng (third-party); the CUDA path and this oracle
// use the same counter-based function instead (splitmix64 finaliser of seed, counter and row),
// top 24 bits as a float in [0, 1 - 2^-24] (the reference clamps to RANDOM_MAX = 0.99999994).
static float sampler_uniform(uint64_t seed, uint64_t counter, uint32_t row) {
  uint64_t z = seed + 0x9E3779B97F4A7C15ull * (counter * 65536ull + (uint64_t)row + 1ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

namespace {
struct SLogit { uint32_t id; float logit; };
struct WLogit { SLogit l; float w; };
const float S_EPSILON = 1.0e-20f;  // sampler.rs:6

float normalized_probability(float v, float dflt) {  // sampler.rs:305-311
  if (!std::isfinite(v)) return dflt;
  return std::min(std::max(v, 0.0f), 1.0f);
}

// process_logit (sampler.rs:262-295) over all logits, then sort_logits_desc (:252-259) and the
// top_k cut (:154-166)
std::vector<SLogit> processed_top(const float* logits, size_t n, float temperature, float rep_penalty, int range,
                                  int top_k, const uint32_t* prev, int prev_len) {
  // previous_tokens_for_config, sampler.rs:297-303
  int len = std::min(prev_len, range);
  if (len < 0) len = 0;
  const uint32_t* pv = prev ? prev + (prev_len - len) : nullptr;
  std::vector<SLogit> top;
  top.reserve(n);
  for (size_t i = 0; i < n; ++i) {
    float value = logits[i];
    if (!std::isfinite(value)) continue;
    if (rep_penalty > 1.0f && pv && std::find(pv, pv + len, (uint32_t)i) != pv + len) {
      if (value <= 0.0f) value *= rep_penalty;
      else value /= rep_penalty;
    }
    if (temperature != 0.0f) value /= temperature;
    if (!std::isfinite(value)) continue;
    top.push_back({(uint32_t)i, value});
  }
  // f32::total_cmp descending, then token id descending
  auto ord = [](float f) { uint32_t b; std::memcpy(&b, &f, 4); return (b & 0x80000000u) ? ~b : (b | 0x80000000u); };
  std::sort(top.begin(), top.end(), [&](const SLogit& a, const SLogit& b) {
    uint32_t oa = ord(a.logit), ob = ord(b.logit);
    if (oa != ob) return oa > ob;
    return a.id > b.id;
  });
  top_k = std::max(top_k, 1);
  if ((int)top.size() > top_k) top.resize(top_k);
  return top;
}
}  // namespace

// One draw of CpuStandardSampler (strategy 0, sampler.rs:135-241) or CpuMirostat2Sampler (strategy
// 1, :44-133). Returns the token id, or 0xFFFFFFFF when no logit survives. *margin (optional) is
// the distance, relative to the candidates' total weight, between the draw's threshold and the
// nearest cumulative sum: a tiny margin means one ulp of an exponential can change the token.
ORACLE_API uint32_t oracle_sample(const float* logits, size_t n, int strategy, float temperature, float rep_penalty,
                                  int range, int top_k, float top_p_in, float min_p_in, float tau, float eta, float* mu,
                                  const uint32_t* prev, int prev_len, uint64_t seed, uint64_t counter, uint32_t row,
                                  float* margin) {
  if (margin) *margin = 1.0f;
  std::vector<SLogit> top = processed_top(logits, n, temperature, rep_penalty, range, top_k, prev, prev_len);
  if (top.empty()) return 0xFFFFFFFFu;
  const float u = sampler_uniform(seed, counter, row);
  const float max = top[0].logit;
  auto note = [&](float cum, float thr, float total) {
    if (margin) *margin = std::min(*margin, std::fabs(cum - thr) / total);
  };
  if (strategy == 0) {
    if (temperature <= 0.0f) return top[0].id;
    std::vector<WLogit> cand;
    for (auto& l : top) cand.push_back({l, std::exp(l.logit - max)});
    float min_p = normalized_probability(min_p_in, 0.0f);
    if (min_p > 0.0f) {
      float thr = cand[0].w * min_p;
      std::vector<WLogit> kept;
      for (auto& c : cand) if (c.w >= thr) kept.push_back(c);
      cand.swap(kept);
    }
    float top_p = normalized_probability(top_p_in, 1.0f);
    if (top_p < 1.0f) {
      float total = 0.f;
      for (auto& c : cand) total += c.w;
      total = std::max(total, S_EPSILON);
      float thr = total * top_p, cum = 0.f;
      size_t cutoff = 0;
      for (size_t i = 0; i < cand.size(); ++i) {
        cum += cand[i].w;
        cutoff = i + 1;
        note(cum, thr, total);
        if (cum >= thr) break;
      }
      cand.resize(std::max<size_t>(cutoff, 1));
    }
    float total = 0.f;
    for (auto& c : cand) total += c.w;
    total = std::max(total, S_EPSILON);
    float thr = u * total, cum = 0.f;
    for (auto& c : cand) {
      cum += c.w;
      note(cum, thr, total);
      if (cum >= thr) return c.l.id;
    }
    return cand.back().l.id;
  }
  // Mirostat 2
  float total = 0.f;
  for (auto& l : top) total += std::exp(l.logit - max);
  total = std::max(total, S_EPSILON);
  size_t cutoff = top.size();
  for (size_t i = 0; i < top.size(); ++i) {
    float p = std::max(std::exp(top[i].logit - max) / total, S_EPSILON);
    if (-std::log2(p) > *mu) { cutoff = std::max<size_t>(i, 1); break; }
  }
  cutoff = std::min(cutoff, top.size());
  float csum = 0.f;
  for (size_t i = 0; i < cutoff; ++i) csum += std::exp(top[i].logit - max);
  csum = std::max(csum, S_EPSILON);
  float thr = u * csum, cum = 0.f;
  SLogit sel = top[0];
  float selw = std::exp(sel.logit - max);
  for (size_t i = 0; i < cutoff; ++i) {
    float w = std::exp(top[i].logit - max);
    cum += w;
    note(cum, thr, csum);
    if (cum >= thr) { sel = top[i]; selw = w; break; }
  }
  float psel = std::max(selw / csum, S_EPSILON);
  float next_mu = *mu - eta * (-std::log2(psel) - tau);
  if (std::isfinite(next_mu)) *mu = next_mu;
  return sel.id;
}

// ---- synthetic-weight quantisers ------------------------------------------------------------
// The reference only loads pre-quantised GGUF files; it has no f32 -> Q4_0/Q4_K/Q6_K encoder.
// These encoders are this project's own (simple min/max and absmax rounding). Their only duty
// is to emit structurally valid blocks with finite scales; parity is defined on the bytes.

namespace {

inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

void quant_q4_0(const float* x, uint8_t* b) {
  float amax = 0.f;
  for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(x[i]));
  uint16_t dh = f32_to_f16(amax / 7.0f);
  float d = f16_to_f32(dh);
  float id = d > 0.f ? 1.0f / d : 0.f;
  b[0] = dh & 0xFF; b[1] = dh >> 8;
  for (int i = 0; i < 16; ++i) {
    int lo = clampi((int)std::lrintf(x[i] * id) + 8, 0, 15);
    int hi = clampi((int)std::lrintf(x[i + 16] * id) + 8, 0, 15);
    b[2 + i] = (uint8_t)(lo | (hi << 4));
  }
}

void quant_q8_0(const float* x, uint8_t* b) {
  float amax = 0.f;
  for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(x[i]));
  uint16_t dh = f32_to_f16(amax / 127.0f);
  float d = f16_to_f32(dh);
  float id = d > 0.f ? 1.0f / d : 0.f;
  b[0] = dh & 0xFF; b[1] = dh >> 8;
  for (int i = 0; i < 32; ++i) b[2 + i] = (uint8_t)(int8_t)clampi((int)std::lrintf(x[i] * id), -127, 127);
}

void quant_q4k(const float* x, uint8_t* b) {
  float scale_sb[8], off_sb[8];
  float max_scale = 0.f, max_off = 0.f;
  for (int j = 0; j < 8; ++j) {
    float lo = x[32 * j], hi = x[32 * j];
    for (int l = 1; l < 32; ++l) { lo = std::min(lo, x[32 * j + l]); hi = std::max(hi, x[32 * j + l]); }
    float off = lo < 0.f ? -lo : 0.f;
    float sc = (hi + off) / 15.0f;
    scale_sb[j] = sc; off_sb[j] = off;
    max_scale = std::max(max_scale, sc);
    max_off = std::max(max_off, off);
  }
  uint16_t dh = f32_to_f16(max_scale / 63.0f), mh = f32_to_f16(max_off / 63.0f);
  float d = f16_to_f32(dh), dmin = f16_to_f32(mh);
  uint8_t sc[8], mn[8];
  for (int j = 0; j < 8; ++j) {
    sc[j] = (uint8_t)clampi(d > 0.f ? (int)std::lrintf(scale_sb[j] / d) : 0, 0, 63);
    mn[j] = (uint8_t)clampi(dmin > 0.f ? (int)std::lrintf(off_sb[j] / dmin) : 0, 0, 63);
  }
  b[0] = dh & 0xFF; b[1] = dh >> 8; b[2] = mh & 0xFF; b[3] = mh >> 8;
  uint8_t* p = b + 4;
  for (int j = 0; j < 4; ++j) {
    p[j] = (uint8_t)(sc[j] | ((sc[j + 4] >> 4) << 6));
    p[j + 4] = (uint8_t)(mn[j] | ((mn[j + 4] >> 4) << 6));
    p[j + 8] = (uint8_t)((sc[j + 4] & 0xF) | ((mn[j + 4] & 0xF) << 4));
  }
  uint8_t* qs = b + 16;
  for (int j = 0; j < 4; ++j) {
    float s0 = d * sc[2 * j], o0 = dmin * mn[2 * j];
    float s1 = d * sc[2 * j + 1], o1 = dmin * mn[2 * j + 1];
    float i0 = s0 > 0.f ? 1.0f / s0 : 0.f, i1 = s1 > 0.f ? 1.0f / s1 : 0.f;
    for (int l = 0; l < 32; ++l) {
      int q0 = clampi((int)std::lrintf((x[64 * j + l] + o0) * i0), 0, 15);
      int q1 = clampi((int)std::lrintf((x[64 * j + 32 + l] + o1) * i1), 0, 15);
      qs[32 * j + l] = (uint8_t)(q0 | (q1 << 4));
    }
  }
}

void quant_q6k(const float* x, uint8_t* b) {
  float gs[16];
  float max_gs = 0.f;
  for (int g = 0; g < 16; ++g) {
    float amax = 0.f;
    for (int l = 0; l < 16; ++l) amax = std::max(amax, std::fabs(x[16 * g + l]));
    gs[g] = amax / 31.0f;
    max_gs = std::max(max_gs, gs[g]);
  }
  uint16_t dh = f32_to_f16(max_gs / 127.0f);
  float d = f16_to_f32(dh);
  int8_t sc[16];
  uint8_t q[256];
  for (int g = 0; g < 16; ++g) {
    sc[g] = (int8_t)clampi(d > 0.f ? (int)std::lrintf(gs[g] / d) : 0, 0, 127);
    float s = d * (float)sc[g];
    float is = s > 0.f ? 1.0f / s : 0.f;
    for (int l = 0; l < 16; ++l)
      q[16 * g + l] = (uint8_t)clampi((int)std::lrintf(x[16 * g + l] * is) + 32, 0, 63);
  }
  uint8_t* ql = b;
  uint8_t* qh = b + 128;
  for (int c = 0; c < 2; ++c)
    for (int l = 0; l < 32; ++l) {
      uint8_t q1 = q[128 * c + l], q2 = q[128 * c + l + 32], q3 = q[128 * c + l + 64],
              q4 = q[128 * c + l + 96];
      ql[64 * c + l] = (uint8_t)((q1 & 0xF) | ((q3 & 0xF) << 4));
      ql[64 * c + l + 32] = (uint8_t)((q2 & 0xF) | ((q4 & 0xF) << 4));
      qh[32 * c + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
    }
  std::memcpy(b + 192, sc, 16);
  b[208] = dh & 0xFF; b[209] = dh >> 8;
}

// SplitMix64 -> two uniforms -> Box-Muller; counter based, so any block can be generated
// independently of the others (thread count does not change the bytes).
inline uint64_t splitmix(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

inline void normal_pair(uint64_t seed, uint64_t idx, float sigma, float* a, float* b) {
  uint64_t r = splitmix(seed ^ splitmix(idx));
  float u1 = ((float)(uint32_t)(r >> 40) + 1.0f) * (1.0f / 16777216.0f);  // (0,1]
  float u2 = (float)(uint32_t)((r >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);
  float rad = std::sqrt(-2.0f * std::log(u1)) * sigma;
  float ang = 6.28318530717958647692f * u2;
  *a = rad * std::cos(ang);
  *b = rad * std::sin(ang);
}

}  // namespace

ORACLE_API int oracle_quantize(const float* x, size_t n_elems, uint32_t ty, uint8_t* out) {
  int bs, bbytes;
  if (!block_geometry(ty, &bs, &bbytes)) return -2;
  if (n_elems % (size_t)bs) return -1;
  size_t nb = n_elems / bs;
  int nt = nb > 1024 ? num_threads() : 1;
  run_threads(nt, [&](int t) {
    size_t b0 = nb * t / nt, b1 = nb * (t + 1) / nt;
    for (size_t i = b0; i < b1; ++i) {
      const float* xb = x + i * bs;
      uint8_t* ob = out + i * bbytes;
      switch (ty) {
        case Q4_0: quant_q4_0(xb, ob); break;
        case Q8_0: quant_q8_0(xb, ob); break;
        case Q4K: quant_q4k(xb, ob); break;
        case Q6K: quant_q6k(xb, ob); break;
        default: break;
      }
    }
  });
  return (ty == Q4_0 || ty == Q8_0 || ty == Q4K || ty == Q6K) ? 0 : -2;
}

// Seeded N(0, sigma) f32 values (element i of stream `seed`).
ORACLE_API void oracle_normal(uint64_t seed, float sigma, size_t n, float* out) {
  size_t pairs = (n + 1) / 2;
  int nt = n > (1u << 16) ? num_threads() : 1;
  run_threads(nt, [&](int t) {
    size_t p0 = pairs * t / nt, p1 = pairs * (t + 1) / nt;
    for (size_t p = p0; p < p1; ++p) {
      float a, b;
      normal_pair(seed, p, sigma, &a, &b);
      out[2 * p] = a;
      if (2 * p + 1 < n) out[2 * p + 1] = b;
    }
  });
}

// Seeded N(0, sigma) weights quantised block by block without materialising the f32 matrix.
ORACLE_API int oracle_random_qweights(uint64_t seed, float sigma, size_t n_elems, uint32_t ty,
                                      uint8_t* out) {
  int bs, bbytes;
  if (!block_geometry(ty, &bs, &bbytes)) return -2;
  if (ty != Q4_0 && ty != Q8_0 && ty != Q4K && ty != Q6K) return -2;
  if (n_elems % (size_t)bs) return -1;
  size_t nb = n_elems / bs;
  int nt = nb > 1024 ? num_threads() : 1;
  run_threads(nt, [&](int t) {
    size_t b0 = nb * t / nt, b1 = nb * (t + 1) / nt;
    float xb[256];
    for (size_t i = b0; i < b1; ++i) {
      for (int p = 0; p < bs / 2; ++p)
        normal_pair(seed, i * (size_t)(bs / 2) + p, sigma, &xb[2 * p], &xb[2 * p + 1]);
      uint8_t* ob = out + i * bbytes;
      switch (ty) {
        case Q4_0: quant_q4_0(xb, ob); break;
        case Q8_0: quant_q8_0(xb, ob); break;
        case Q4K: quant_q4k(xb, ob); break;
        default: quant_q6k(xb, ob); break;
      }
    }
  });
  return 0;
}

// =================================================================================================
// Llama decoder oracle: the order of operations of Model::forward_last_hidden_from_embeddings
// (models/kalosm-llama/src/raw/mod.rs:925-1049), LlamaAttention::forward
// (raw/attention_layer.rs:514-573), SeparateAttention::forward (:281-427), the CPU FFN branch
// (:220-235, gate_up is None on CPU) and forward_attention_qkv_f32 (:659-694).
// =================================================================================================

ORACLE_API void* oracle_llama_create(int n_layer, int hidden, int ffn, int n_head, int n_kv_head,
                                     int head_dim, int vocab, int ctx, float eps, float theta,
                                     int batch, int kv_f16) {
  Llama* m = new Llama();
  m->n_layer = n_layer; m->hidden = hidden; m->ffn = ffn; m->n_head = n_head;
  m->n_kv_head = n_kv_head; m->head_dim = head_dim; m->vocab = vocab; m->ctx = ctx;
  m->eps = eps; m->theta = theta; m->batch = batch; m->kv_f16 = kv_f16 != 0;
  m->layers.resize(n_layer);
  m->cos.resize((size_t)ctx * head_dim / 2);
  m->sin.resize((size_t)ctx * head_dim / 2);
  oracle_rope_tables(head_dim, ctx, theta, 0.f, 1.f, 4.f, ctx, m->cos.data(), m->sin.data());
  size_t kv = (size_t)n_layer * batch * n_kv_head * ctx * head_dim;
  m->kcache.assign(kv, 0.f);
  m->vcache.assign(kv, 0.f);
  return m;
}

ORACLE_API void oracle_llama_free(void* h) { delete (Llama*)h; }

// RoPE scaling (an argument of Model::from_var_source, raw/mod.rs:271) and rope_freqs.weight
// (raw/mod.rs:417-421): rebuilds the tables.
ORACLE_API void oracle_llama_set_rope(void* h, float factor, float low_freq_factor, float high_freq_factor,
                                      int original_ctx, const float* freq_weight) {
  Llama* m = (Llama*)h;
  oracle_rope_tables_w(m->head_dim, m->ctx, m->theta, factor, low_freq_factor, high_freq_factor, original_ctx,
                       freq_weight, m->cos.data(), m->sin.data());
}

// which: 0 token_embd, 1 output, 2 wq, 3 wk, 4 wv, 5 wo, 6 gate, 7 up, 8 down (layer ignored for 0/1)
ORACLE_API int oracle_llama_set_qmatrix(void* h, int layer, int which, uint32_t ty, size_t n,
                                        size_t k, const uint8_t* bytes, size_t nbytes) {
  Llama* m = (Llama*)h;
  QMat* q = nullptr;
  if (which == 0) q = &m->token_embd;
  else if (which == 1) q = &m->output;
  else {
    if (layer < 0 || layer >= m->n_layer) return -1;
    Layer& L = m->layers[layer];
    QMat* tbl[] = {&L.wq, &L.wk, &L.wv, &L.wo, &L.gate, &L.up, &L.down};
    if (which < 2 || which > 8) return -1;
    q = tbl[which - 2];
  }
  int bs, bbytes;
  if (!block_geometry(ty, &bs, &bbytes)) return -2;
  if (k % bs || nbytes != n * (k / bs) * (size_t)bbytes) return -1;
  q->ty = ty; q->n = n; q->k = k;
  q->bytes.assign(bytes, bytes + nbytes);
  return 0;
}

// which: 0 attn_norm, 1 ffn_norm, 2 output_norm
ORACLE_API int oracle_llama_set_norm(void* h, int layer, int which, const float* w, size_t n) {
  Llama* m = (Llama*)h;
  if (which == 2) { m->output_norm.assign(w, w + n); return 0; }
  if (layer < 0 || layer >= m->n_layer) return -1;
  (which == 0 ? m->layers[layer].attn_norm : m->layers[layer].ffn_norm).assign(w, w + n);
  return 0;
}

ORACLE_API void oracle_llama_reset(void* h) {
  Llama* m = (Llama*)h;
  m->pos = 0;
  std::fill(m->kcache.begin(), m->kcache.end(), 0.f);
  std::fill(m->vcache.begin(), m->vcache.end(), 0.f);
}

ORACLE_API int oracle_llama_pos(void* h) { return ((Llama*)h)->pos; }

// Keeps the first `len` cached positions (the reference trims its caches to the common prefix of
// cached and new tokens and re-runs the rest, models/kalosm-llama/src/raw/mod.rs:769-793).
ORACLE_API int oracle_llama_truncate(void* h, int len) {
  Llama* m = (Llama*)h;
  if (len < 0 || len > m->pos) return -1;
  m->pos = len;
  return 0;
}

namespace {

void qmm(const QMat& w, const float* x, size_t m, float* y) {
  q_mat_mul_impl(x, m, w.k, w.bytes.data(), w.ty, w.n, y);
}

}  // namespace

// tokens [batch, seq]; writes logits of the LAST position, [batch, vocab]
// (raw/mod.rs:1046: only the last position reaches the output projection).
ORACLE_API int oracle_llama_forward(void* h, const uint32_t* tokens, int seq, float* logits) {
  Llama* m = (Llama*)h;
  const int B = m->batch, H = m->n_head, HK = m->n_kv_head, D = m->head_dim, E = m->hidden;
  const int start = m->pos;
  if (start + seq > m->ctx) return -3;
  const size_t rows = (size_t)B * seq;
  std::vector<float> x(rows * E), xn(rows * E), q(rows * H * D), k(rows * HK * D),
      v(rows * HK * D), qt(rows * H * D), att(rows * H * D), att_t(rows * H * D),
      attn_out(rows * E), g(rows * m->ffn), u(rows * m->ffn), dn(rows * E), tmp(256);

  // Embedding::forward (fusor-ml/fusor/src/layers/embedding.rs:43-107): dequantised rows.
  {
    int bs, bbytes;
    block_geometry(m->token_embd.ty, &bs, &bbytes);
    size_t row_bytes = (size_t)(E / bs) * bbytes;
    for (size_t r = 0; r < rows; ++r)
      oracle_dequantize(m->token_embd.bytes.data() + (size_t)tokens[r] * row_bytes,
                        m->token_embd.ty, E, x.data() + r * E);
  }
  const float scale = (float)(1.0 / std::sqrt((double)D));
  const int skv = start + seq;
  for (int li = 0; li < m->n_layer; ++li) {
    Layer& L = m->layers[li];
    oracle_rms_norm(x.data(), nullptr, L.attn_norm.data(), nullptr, m->eps, rows, E, xn.data());
    qmm(L.wq, xn.data(), rows, q.data());
    qmm(L.wk, xn.data(), rows, k.data());
    qmm(L.wv, xn.data(), rows, v.data());
    // [B,S,H,D] -> [B,H,S,D]
    for (int b = 0; b < B; ++b)
      for (int s = 0; s < seq; ++s)
        for (int hh = 0; hh < H; ++hh)
          std::memcpy(&qt[(((size_t)b * H + hh) * seq + s) * D],
                      &q[(((size_t)b * seq + s) * H + hh) * D], D * sizeof(float));
    oracle_rope(qt.data(), B, H, seq, D, m->cos.data(), m->sin.data(), start, 1);
    // K: rope then append; V: append. Cache layout [layer][B][HK][ctx][D].
    float* kc = m->kcache.data() + (size_t)li * B * HK * m->ctx * D;
    float* vc = m->vcache.data() + (size_t)li * B * HK * m->ctx * D;
    for (int b = 0; b < B; ++b)
      for (int hh = 0; hh < HK; ++hh)
        for (int s = 0; s < seq; ++s) {
          float kr[512];
          std::memcpy(kr, &k[(((size_t)b * seq + s) * HK + hh) * D], D * sizeof(float));
          oracle_rope(kr, 1, 1, 1, D, m->cos.data(), m->sin.data(), start + s, 1);
          float* kd = kc + (((size_t)b * HK + hh) * m->ctx + start + s) * D;
          float* vd = vc + (((size_t)b * HK + hh) * m->ctx + start + s) * D;
          const float* vs = &v[(((size_t)b * seq + s) * HK + hh) * D];
          for (int e = 0; e < D; ++e) {
            kd[e] = m->kv_f16 ? f16_to_f32(f32_to_f16(kr[e])) : kr[e];
            vd[e] = m->kv_f16 ? f16_to_f32(f32_to_f16(vs[e])) : vs[e];
          }
        }
    oracle_attention(qt.data(), kc, vc, B, H, HK, seq, skv, D, (size_t)m->ctx * D, scale, nullptr,
                     0, seq > 1 ? 1 : 0, att.data());
    // [B,H,S,D] -> [B,S,H*D]
    for (int b = 0; b < B; ++b)
      for (int hh = 0; hh < H; ++hh)
        for (int s = 0; s < seq; ++s)
          std::memcpy(&att_t[(((size_t)b * seq + s) * H + hh) * D],
                      &att[(((size_t)b * H + hh) * seq + s) * D], D * sizeof(float));
    qmm(L.wo, att_t.data(), rows, attn_out.data());
    // ffn_norm.forward_residual_f32(attn, residual): normalise (attn + residual)
    oracle_rms_norm(attn_out.data(), x.data(), L.ffn_norm.data(), nullptr, m->eps, rows, E,
                    xn.data());
    qmm(L.gate, xn.data(), rows, g.data());
    qmm(L.up, xn.data(), rows, u.data());
    oracle_silu_mul(g.data(), u.data(), rows * m->ffn, g.data());
    qmm(L.down, g.data(), rows, dn.data());
    // (projected + attn) + residual  (attention_layer.rs:170-172; raw/mod.rs:1036)
    for (size_t i = 0; i < rows * E; ++i) x[i] = (dn[i] + attn_out[i]) + x[i];
  }
  // final norm on the last position of every batch row, then the output projection
  std::vector<float> last((size_t)B * E), lastn((size_t)B * E);
  for (int b = 0; b < B; ++b)
    std::memcpy(&last[(size_t)b * E], &x[((size_t)b * seq + seq - 1) * E], E * sizeof(float));
  oracle_rms_norm(last.data(), nullptr, m->output_norm.data(), nullptr, m->eps, B, E, lastn.data());
  const QMat& out_w = m->output.bytes.empty() ? m->token_embd : m->output;  // tied fallback, raw/mod.rs:480-486
  // The reference projects each batch row as its own [1,K] product; M = B here takes the
  // m >= 4 branch for B >= 4, whose per-output arithmetic is the same.
  qmm(out_w, lastn.data(), B, logits);
  m->pos += seq;
  return 0;
}
