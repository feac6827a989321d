// On-device sampling: top-k selection and the token samplers that follow the output head, so
// that only token ids leave the GPU.
//
// Mirrors the reference's samplers operation for operation:
//   * Tensor::top_k_pairs (fusor-ml/fusor/src/lib.rs:416-453): the k highest finite logits,
//     descending, ties -> higher token id;
//   * CpuStandardSampler / CpuMirostat2Sampler (models/kalosm-llama/src/sampler.rs:44-241):
//     per-logit processing (drop non-finite, repetition penalty over the last
//     `repetition_penalty_range` tokens, divide by the temperature, :262-295), sort descending
//     with ties -> higher id (:252-259), keep top_k, then min-p, top-p and the cumulative walk
//     (standard, :144-240) or the surprise cut-off and mu update (Mirostat 2, :58-133).
// The reference draws its uniform number from rand's StdRng, which is a third-party stream cipher
// generator; here the draw is a counter-based function of (seed, counter, row) (the splitmix64
// finaliser), which the CPU restatement used by the tests repeats, so both sides see the same number.
//
// One CTA of 1024 threads per row. A (processed value, token id) pair is one 64-bit key whose
// unsigned order is exactly the reference's sort order, so "top k, sorted" = the k largest keys:
// an MSB-first radix select (11-bit digits, keys recomputed from the logits on every pass: no
// scratch in global memory) finds the k-th largest key, the keys at or above it are collected in
// shared memory and sorted by a bitonic network. The tail of the sampler (at most 1024
// candidates) runs in one thread in the reference's order of additions, so that the cumulative
// sums match the CPU's bit for bit given equal exponentials.
#include <cmath>

#include "common.cuh"

namespace {

constexpr int ST = 1024;               // threads per CTA
constexpr int MAX_K = FB200_SAMPLER_MAX_TOP_K;
constexpr int BINS = 2048;
constexpr float EPSILON = 1.0e-20f;    // sampler.rs:6

struct SampleArgs {
  const float* logits;   // [rows, n]
  size_t n;
  int k;
  // processing (sampler.rs:262-295); mode 0 = plain top-k of the raw logits
  int mode;              // 0 top-k, 1 standard sampler, 2 Mirostat 2
  float temperature, rep_penalty;
  const uint32_t* prev;  // [rows, prev_stride] previous tokens (window already cut), or null
  size_t prev_stride;
  int prev_len;
  float top_p, min_p;    // already normalised: top_p in [0, 1] (1 = off), min_p in [0, 1] (0 = off)
  float tau, eta;
  float* mu;             // [rows] Mirostat state
  unsigned long long seed, counter;
  // outputs
  uint32_t* ids;         // top-k: [rows, k]; samplers: [rows]
  float* vals;           // top-k only: [rows, k] or null
  uint32_t* also0;       // optional extra destinations of the sampled id: also0[row * stride0]
  size_t stride0;
  uint32_t* also1;
  size_t stride1;
};

__device__ __forceinline__ unsigned long long key_of(float v, uint32_t idx) {
  if (!isfinite(v)) return 0ull;
  uint32_t b = __float_as_uint(v);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return ((unsigned long long)b << 32) | (unsigned long long)idx;
}
__device__ __forceinline__ float value_of(unsigned long long key) {
  uint32_t b = (uint32_t)(key >> 32);
  b = (b & 0x80000000u) ? (b & 0x7FFFFFFFu) : ~b;
  return __uint_as_float(b);
}

// process_logit, sampler.rs:262-295
__device__ __forceinline__ unsigned long long processed_key(const SampleArgs& a, const uint32_t* bitmap, float logit,
                                                            uint32_t id) {
  float v = logit;
  if (!isfinite(v)) return 0ull;
  if (a.mode != 0) {
    if (bitmap && ((bitmap[id >> 5] >> (id & 31u)) & 1u)) {
      if (v <= 0.0f) v = __fmul_rn(v, a.rep_penalty);
      else v = __fdiv_rn(v, a.rep_penalty);
    }
    if (a.temperature != 0.0f) v = __fdiv_rn(v, a.temperature);
  }
  return key_of(v, id);
}

// uniform number in [0, 1 - 2^-24] from (seed, counter, row): splitmix64 finaliser, top 24 bits
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long counter, unsigned row) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (counter * 65536ull + (unsigned long long)row + 1ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(ST)
sample_kernel(const SampleArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  unsigned long long* cand = reinterpret_cast<unsigned long long*>(smem);       // [MAX_K]
  float* wgt = reinterpret_cast<float*>(cand + MAX_K);                          // [MAX_K]
  unsigned* hist = reinterpret_cast<unsigned*>(wgt + MAX_K);                    // [BINS]
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(hist + BINS);                  // [(n + 31) / 32] or unused
  __shared__ unsigned long long s_prefix;
  __shared__ unsigned s_remaining, s_count, s_done, s_valid;
  const int tid = threadIdx.x;
  const unsigned row = blockIdx.x;
  const float* lg = a.logits + (size_t)row * a.n;
  const bool penal = a.mode != 0 && a.rep_penalty > 1.0f && a.prev && a.prev_len > 0;
  if (penal) {
    const size_t words = (a.n + 31) / 32;
    for (size_t i = tid; i < words; i += ST) bitmap[i] = 0u;
    __syncthreads();
    const uint32_t* pv = a.prev + (size_t)row * a.prev_stride;
    for (int i = tid; i < a.prev_len; i += ST) {
      const uint32_t t = pv[i];
      if ((size_t)t < a.n) atomicOr(&bitmap[t >> 5], 1u << (t & 31u));
    }
  }
  if (tid == 0) { s_prefix = 0ull; s_remaining = (unsigned)a.k; s_done = 0u; s_valid = 0u; }
  __syncthreads();
  const uint32_t* bm = penal ? bitmap : nullptr;

  // ---- radix select of the k-th largest key (digits from the top: 9 bits, then 5 x 11)
  unsigned long long threshold = 0ull;  // keys >= threshold are the top k
  for (int pass = 0; pass < 6; ++pass) {
    const int shift = 55 - 11 * pass;
    const int bits = pass == 0 ? 9 : 11;
    for (int i = tid; i < BINS; i += ST) hist[i] = 0u;
    __syncthreads();
    const unsigned long long prefix = s_prefix;
    const int hshift = shift + bits;  // bits above this digit must equal the prefix
    unsigned valid_local = 0;
    for (size_t i = tid; i < a.n; i += ST) {
      const unsigned long long key = processed_key(a, bm, lg[i], (uint32_t)i);
      if (key == 0ull) continue;
      ++valid_local;
      if (hshift < 64 && (key >> hshift) != (prefix >> hshift)) continue;
      atomicAdd(&hist[(unsigned)(key >> shift) & ((1u << bits) - 1u)], 1u);
    }
    if (pass == 0 && valid_local) atomicAdd(&s_valid, valid_local);
    __syncthreads();
    if (tid == 0) {
      unsigned remaining = s_remaining;
      if (pass == 0 && s_valid < remaining) { remaining = s_valid; }
      if (remaining == 0) {
        s_done = 1u;  // nothing finite at all
        threshold = ~0ull;
      } else {
        unsigned cum = 0;
        int b = (1 << bits) - 1;
        for (; b > 0; --b) {
          if (cum + hist[b] >= remaining) break;
          cum += hist[b];
        }
        // bin b holds the k-th key; everything in higher bins is in
        remaining -= cum;
        s_prefix = prefix | ((unsigned long long)b << shift);
        if (hist[b] == remaining || shift == 0) s_done = 1u;  // the whole bin is in: cut below it
      }
      s_remaining = remaining;
    }
    __syncthreads();
    if (s_done) break;
  }
  threshold = s_remaining == 0 ? ~0ull : s_prefix;
  const unsigned k_eff = min((unsigned)a.k, s_valid);

  // ---- collect and sort the candidates (descending keys)
  if (tid == 0) s_count = 0u;
  int p2 = 1;
  while (p2 < (int)k_eff) p2 <<= 1;
  for (int i = tid; i < p2; i += ST) cand[i] = 0ull;
  __syncthreads();
  if (k_eff) {
    for (size_t i = tid; i < a.n; i += ST) {
      const unsigned long long key = processed_key(a, bm, lg[i], (uint32_t)i);
      if (key != 0ull && key >= threshold) {
        const unsigned slot = atomicAdd(&s_count, 1u);
        if (slot < (unsigned)MAX_K) cand[slot] = key;
      }
    }
  }
  __syncthreads();
  for (int size = 2; size <= p2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < p2; i += ST) {
        const int j = i ^ stride;
        if (j > i) {
          const unsigned long long x = cand[i], y = cand[j];
          const bool desc = (i & size) == 0;
          if (desc ? x < y : x > y) { cand[i] = y; cand[j] = x; }
        }
      }
      __syncthreads();
    }
  }

  if (a.mode == 0) {
    for (int i = tid; i < a.k; i += ST) {
      const bool have = i < (int)k_eff;
      a.ids[(size_t)row * a.k + i] = have ? (uint32_t)(cand[i] & 0xFFFFFFFFull) : 0xFFFFFFFFu;
      if (a.vals) a.vals[(size_t)row * a.k + i] = have ? value_of(cand[i]) : -INFINITY;
    }
    return;
  }

  // ---- sampler tail: weights in parallel, the walk in the reference's order in one thread
  const float vmax = k_eff ? value_of(cand[0]) : 0.f;
  for (int i = tid; i < (int)k_eff; i += ST) wgt[i] = expf(value_of(cand[i]) - vmax);
  __syncthreads();
  if (tid != 0) return;
  uint32_t chosen = 0xFFFFFFFFu;
  if (k_eff) {
    const float u = uniform01(a.seed, a.counter, row);
    int cnt = (int)k_eff;
    if (a.mode == 1) {
      if (a.temperature <= 0.0f) {
        chosen = (uint32_t)(cand[0] & 0xFFFFFFFFull);
      } else {
        if (a.min_p > 0.0f) {  // apply_min_p, sampler.rs:200-214 (weights are non-increasing: a prefix survives)
          const float thr = wgt[0] * a.min_p;
          int keep = 0;
          for (int i = 0; i < cnt; ++i)
            if (wgt[i] >= thr) { wgt[keep] = wgt[i]; cand[keep] = cand[i]; ++keep; }
          cnt = keep;
        }
        if (a.top_p < 1.0f) {  // apply_top_p, sampler.rs:216-240
          float total = 0.f;
          for (int i = 0; i < cnt; ++i) total += wgt[i];
          total = fmaxf(total, EPSILON);
          const float thr = total * a.top_p;
          float cum = 0.f;
          int cutoff = 0;
          for (int i = 0; i < cnt; ++i) {
            cum += wgt[i];
            cutoff = i + 1;
            if (cum >= thr) break;
          }
          cnt = max(cutoff, 1);
        }
        float total = 0.f;
        for (int i = 0; i < cnt; ++i) total += wgt[i];
        total = fmaxf(total, EPSILON);
        const float thr = u * total;
        float cum = 0.f;
        chosen = (uint32_t)(cand[cnt - 1] & 0xFFFFFFFFull);
        for (int i = 0; i < cnt; ++i) {
          cum += wgt[i];
          if (cum >= thr) { chosen = (uint32_t)(cand[i] & 0xFFFFFFFFull); break; }
        }
      }
    } else {
      // Mirostat 2, sampler.rs:58-133
      float mu = a.mu[row];
      float total = 0.f;
      for (int i = 0; i < cnt; ++i) total += wgt[i];
      total = fmaxf(total, EPSILON);
      int cutoff = cnt;
      for (int i = 0; i < cnt; ++i) {
        const float p = fmaxf(wgt[i] / total, EPSILON);
        if (-log2f(p) > mu) { cutoff = max(i, 1); break; }
      }
      cutoff = min(cutoff, cnt);
      float csum = 0.f;
      for (int i = 0; i < cutoff; ++i) csum += wgt[i];
      csum = fmaxf(csum, EPSILON);
      const float thr = u * csum;
      float cum = 0.f;
      int sel = 0;
      for (int i = 0; i < cutoff; ++i) {
        cum += wgt[i];
        if (cum >= thr) { sel = i; break; }
      }
      chosen = (uint32_t)(cand[sel] & 0xFFFFFFFFull);
      const float psel = fmaxf(wgt[sel] / csum, EPSILON);
      const float next_mu = mu - a.eta * (-log2f(psel) - a.tau);
      if (isfinite(next_mu)) a.mu[row] = next_mu;
    }
  }
  a.ids[row] = chosen;
  if (a.also0) a.also0[(size_t)row * a.stride0] = chosen;
  if (a.also1) a.also1[(size_t)row * a.stride1] = chosen;
}

size_t sample_smem(size_t n, bool penal) {
  return (size_t)MAX_K * 8 + (size_t)MAX_K * 4 + (size_t)BINS * 4 + (penal ? (n + 31) / 32 * 4 : 0);
}

float normalized_probability(float v, float dflt) {  // sampler.rs:305-311
  if (!std::isfinite(v)) return dflt;
  return v < 0.f ? 0.f : (v > 1.f ? 1.f : v);
}

int launch_sample(fb200_device* dev, const SampleArgs& a, size_t rows, bool penal) {
  if (rows == 0) return FB200_OK;
  const size_t smem = sample_smem(a.n, penal);
  if (smem > 200 * 1024)
    return fb200_fail(dev, FB200_ERR_CAPACITY, "sampling: a row of %zu logits with a repetition penalty does not fit "
                      "the shared-memory token bitmap", a.n);
  static bool configured[64] = {};
  if (!configured[dev->ordinal & 63]) {
    FB_CUDA(dev, cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured[dev->ordinal & 63] = true;
  }
  sample_kernel<<<(unsigned)rows, ST, smem, dev->stream>>>(a);
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}

}  // namespace

// Enqueues one sampling step over device logits [rows, n]. `prev` points at the first token of
// each row's penalty window. The sampled ids go to ids[row] and to the two optional extra
// destinations (the next step's input and the output history of a device-resident loop).
int fb200_launch_sampler(fb200_device* dev, const float* logits, size_t rows, size_t n, const fb200_sampler_config* c,
                         const uint32_t* prev, size_t prev_stride, int prev_len, unsigned long long counter, float* mu,
                         uint32_t* ids, uint32_t* also0, size_t stride0, uint32_t* also1, size_t stride1) {
  if (!c || !logits || !ids) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "sampler: null argument");
  if (c->top_k < 1 || c->top_k > MAX_K)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "sampler: top_k %d outside 1..%d", c->top_k, MAX_K);
  if (c->strategy != FB200_SAMPLER_STANDARD && c->strategy != FB200_SAMPLER_MIROSTAT2)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "sampler: strategy %d", c->strategy);
  if (c->strategy == FB200_SAMPLER_MIROSTAT2 && !mu)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "sampler: Mirostat 2 needs its mu state");
  if (n == 0 || n > (1ull << 31)) return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "sampler: %zu logits per row", n);
  SampleArgs a = {};
  a.logits = logits; a.n = n; a.k = c->top_k;
  a.mode = c->strategy == FB200_SAMPLER_MIROSTAT2 ? 2 : 1;
  a.temperature = c->temperature; a.rep_penalty = c->repetition_penalty;
  int len = prev_len;
  if (len > c->repetition_penalty_range) {  // previous_tokens_for_config, sampler.rs:297-303: the LAST `range` tokens
    prev += len - c->repetition_penalty_range;
    len = c->repetition_penalty_range;
  }
  a.prev = prev; a.prev_stride = prev_stride; a.prev_len = len < 0 ? 0 : len;
  a.top_p = normalized_probability(c->top_p, 1.0f);
  a.min_p = normalized_probability(c->min_p, 0.0f);
  a.tau = c->tau; a.eta = c->eta; a.mu = mu;
  a.seed = c->seed; a.counter = counter;
  a.ids = ids; a.also0 = also0; a.stride0 = stride0; a.also1 = also1; a.stride1 = stride1;
  const bool penal = a.rep_penalty > 1.0f && a.prev && a.prev_len > 0;
  return launch_sample(dev, a, rows, penal);
}

extern "C" {

int fb200_top_k(fb200_device* dev, const float* logits_dev, size_t rows, size_t n, int k, uint32_t* ids_dev,
                float* vals_dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!logits_dev || !ids_dev) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "top_k: null argument");
  if (k < 1 || k > MAX_K) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "top_k: k %d outside 1..%d", k, MAX_K);
  if (n == 0 || n > (1ull << 31)) return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "top_k: %zu logits per row", n);
  SampleArgs a = {};
  a.logits = logits_dev; a.n = n; a.k = k; a.mode = 0;
  a.ids = ids_dev; a.vals = vals_dev;
  fb200_op_trace scope(dev, "top_k", 4.0 * (double)rows * (double)n);
  return launch_sample(dev, a, rows, false);
}

int fb200_sample(fb200_device* dev, const float* logits_dev, size_t rows, size_t n, const fb200_sampler_config* cfg,
                 const uint32_t* prev_dev, size_t prev_stride, int prev_len, uint64_t counter, float* mu_dev,
                 uint32_t* ids_dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  fb200_op_trace scope(dev, "sample", 4.0 * (double)rows * (double)n);
  return fb200_launch_sampler(dev, logits_dev, rows, n, cfg, prev_dev, prev_stride, prev_len, counter, mu_dev, ids_dev,
                              nullptr, 0, nullptr, 0);
}

}  // extern "C"
