/*
 * fusor_b200 — C ABI of the B200 (sm_100a) backend for Fusor's quantized-inference path.
 *
 * Every entry point mirrors one operation of the `fusor` crate of floneum/kalosm (cited per
 * function as file:line inside that project). A Rust `extern "C"` block binding these symbols
 * is what `fusor::Device::Gpu`, `fusor::QMatrix::Gpu` and `fusor::Tensor::Gpu` would call.
 *
 * Conventions
 *  - Plain pointers and sizes only. Pointers named *_dev are device pointers (from
 *    fb200_malloc or any CUDA allocation on the handle's device); *_host are host pointers.
 *  - Every function returns an fb200_status (0 = OK, negative = error). The text of the last
 *    error of a device handle is available from fb200_last_error(). Nothing aborts, traps or
 *    unwinds across this boundary (the reference mixes Result and panics,
 *    fusor-ml/fusor/src/error.rs:4-15 and src/lib.rs:1133-1138; both become status codes).
 *  - Work is enqueued on the handle's CUDA stream and is asynchronous; fb200_download,
 *    fb200_device_synchronize and the *_host entry points block. One host thread drives a
 *    device handle at a time (the reference serialises a forward pass per session,
 *    models/kalosm-llama/src/model/inference.rs:47-50).
 *  - There is no CPU fallback: without a CUDA device every call fails with FB200_ERR_CUDA.
 */
#ifndef FUSOR_B200_H
#define FUSOR_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define FB200_API __attribute__((visibility("default")))
#else
#define FB200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum fb200_status {
  FB200_OK = 0,
  FB200_ERR_INVALID_SHAPE = -1,
  FB200_ERR_UNSUPPORTED_DTYPE = -2,
  FB200_ERR_CAPACITY = -3,
  FB200_ERR_CUDA = -4,
  FB200_ERR_INVALID_ARGUMENT = -5,
  FB200_ERR_TIMEOUT = -6,
  FB200_ERR_DEVICE_MISMATCH = -7,
  FB200_ERR_NCCL = -8
} fb200_status;

/* ggml type ids, fusor-ml/gguf/src/lib.rs:35-50 */
typedef enum fb200_ggml_type {
  FB200_F32 = 0, FB200_F16 = 1, FB200_Q4_0 = 2, FB200_Q5_0 = 6, FB200_Q8_0 = 8,
  FB200_Q4_K = 12, FB200_Q5_K = 13, FB200_Q6_K = 14
} fb200_ggml_type;

typedef struct fb200_device fb200_device;
typedef struct fb200_qmatrix fb200_qmatrix;
typedef struct fb200_kv_cache fb200_kv_cache;
typedef struct fb200_llama fb200_llama;

/* ---- device: fusor::Device::gpu(), fusor-ml/fusor/src/device.rs:29-40 -------------------------
 * One CUDA device + one stream per handle. `stream` may be an existing cudaStream_t (the
 * handle then enqueues on it and does not own it) or NULL (the handle creates its own). */
FB200_API int fb200_device_create(int ordinal, void* stream, fb200_device** out);
FB200_API int fb200_device_destroy(fb200_device* dev);
FB200_API int fb200_device_synchronize(fb200_device* dev);
FB200_API const char* fb200_last_error(const fb200_device* dev);
/* Number of kernels this library has launched through the handle since creation. */
FB200_API uint64_t fb200_launch_count(const fb200_device* dev);
/* Device-side status word: 0 unless a kernel recorded a fault it recovered from (bounded
 * wait ran out, bad index skipped). Reading it synchronises the stream. While the word is set,
 * every blocking entry point (fb200_device_synchronize, fb200_download, fb200_llama_forward,
 * fb200_llama_generate_greedy, fb200_llama_generate_sampled) returns FB200_ERR_TIMEOUT after its
 * synchronisation: the reference reports a failed dispatch when the result is read back
 * (Tensor::as_slice, fusor-ml/fusor/src/lib.rs:364-368), this is the same point. */
FB200_API int fb200_device_status(fb200_device* dev, int* status_out);
/* Resets the status word to 0 after the caller has dealt with the failure (results produced while
 * it was set are invalid; a tensor-parallel communicator that saw the time-out stays closed and
 * has to be made again). */
FB200_API int fb200_device_clear_status(fb200_device* dev);
/* Scratch buffers of the handle (packed activations, normalised rows, host staging) replace the
 * reference's BufferPool (fusor-ml/tile-ir-runtime/src/buffer_pool.rs:74-260). A budget of
 * `bytes` (0 = unlimited; also FB200_SCRATCH_LIMIT in the environment at creation) makes a call
 * that would grow them beyond it fail with FB200_ERR_CAPACITY instead of allocating. */
FB200_API int fb200_device_set_scratch_limit(fb200_device* dev, size_t bytes);
/* Poison mode (also FB200_POISON=1 at creation): freshly allocated scratch is filled with 0xFF
 * bytes (NaN as f32 / f16), the analogue of the pool's poison fill (buffer_pool.rs:198-207,
 * fusor/src/device.rs:113-118); a kernel that reads scratch nobody wrote then shows in its output. */
FB200_API int fb200_device_set_poison(fb200_device* dev, int enable);

/* ---- tensors: Tensor::from_slice / as_slice, fusor-ml/fusor/src/lib.rs:356-368 -----------------
 * Tensors are contiguous row-major device buffers; shapes travel as arguments. */
FB200_API int fb200_malloc(fb200_device* dev, size_t bytes, void** out_dev);
FB200_API int fb200_free(fb200_device* dev, void* ptr_dev);
FB200_API int fb200_upload(fb200_device* dev, void* dst_dev, const void* src_host, size_t bytes);
FB200_API int fb200_download(fb200_device* dev, void* dst_host, const void* src_dev, size_t bytes);
FB200_API int fb200_memset(fb200_device* dev, void* dst_dev, int value, size_t bytes);

/* ---- QMatrix: fusor-ml/fusor/src/quantized.rs:80-284 -------------------------------------------
 * from_raw_bytes (quantized.rs:183-231): `bytes` are raw GGUF blocks of the logical [N, K]
 * weight (row-major blocks along K, fusor-ml/cpu/src/quantized.rs:293-294), copied during the
 * call. K must be a multiple of the block size (else FB200_ERR_INVALID_SHAPE, where the
 * reference panics, cpu/src/quantized.rs:54-69); unknown types give
 * FB200_ERR_UNSUPPORTED_DTYPE (GgufReadError::UnsupportedDType). F32/F16 are accepted as dense.
 * On the device the blocks are stored in a tile-interleaved order (same bytes, permuted) so
 * that warps read them with coalesced 128-bit loads. Two types are stored otherwise: Q5_0 as Q8_0
 * tiles (the same scale, the 5-bit integer widened to 8 bits: the same values, 34 instead of 22
 * bytes per block of device memory) and Q5_K in the byte order of the file. The type and byte
 * count reported by fb200_qmatrix_ggml_type / fb200_qmatrix_nbytes are always the file's. */
FB200_API int fb200_qmatrix_from_raw_bytes(fb200_device* dev, const uint64_t* shape, int rank,
                                 const void* bytes_host, size_t nbytes, uint32_t ggml_type,
                                 fb200_qmatrix** out);
FB200_API int fb200_qmatrix_free(fb200_qmatrix* q);
/* quantized.rs:115-175 */
FB200_API int fb200_qmatrix_shape(const fb200_qmatrix* q, uint64_t* n_out, uint64_t* k_out);
FB200_API int fb200_qmatrix_ggml_type(const fb200_qmatrix* q, uint32_t* type_out);
/* Raw GGUF byte count of the matrix (the algorithmic bytes one product streams). */
FB200_API int fb200_qmatrix_nbytes(const fb200_qmatrix* q, uint64_t* nbytes_out);
/* QMatrix::dequantize, quantized.rs:233-284: f32 [N, K] into out_dev, bit-exact with
 * GgufBlock::dequantize (fusor-ml/gguf/src/lib.rs:828,1046,1284,1526,1819,2034). */
FB200_API int fb200_qmatrix_dequantize(const fb200_qmatrix* q, float* out_dev);
/* QMatrix::concat_rows, quantized.rs:102-112 / core/src/quantized/mod.rs:312-386: same type
 * and same K required; otherwise FB200_ERR_INVALID_SHAPE and *out = NULL (the reference
 * returns None). Every N but the last must be a multiple of 16. */
FB200_API int fb200_qmatrix_concat_rows(const fb200_qmatrix* const* ms, int n, fb200_qmatrix** out);

/* ---- q_mat_mul: Tensor::q_mat_mul, fusor-ml/fusor/src/lib.rs:1132-1223 --------------------------
 * y[M, N] = x[M, K] . W^T (+ epilogue), x and y f32 contiguous; rank-1 x is M = 1.
 * Epilogues mirror the fused forms the reference's GPU path recognises:
 *   FB200_EPI_RESIDUAL  y = (W.x + r1) + r2          (r2 may be NULL) — down/O projection with
 *                       residual adds, models/kalosm-llama/src/raw/attention_layer.rs:147-174
 *   FB200_EPI_SWIGLU    W is [gate; up] row-concatenated (2F rows); y[M, F] =
 *                       silu(gate.x) * (up.x) — attention_layer.rs:184-196
 *   FB200_EPI_BIAS      y = W.x + bias, bias = r1 of shape [N] shared by all rows — Linear with a
 *                       bias, fusor-ml/fusor/src/layers/linear.rs:93-121 (r2 must be NULL) */
typedef enum fb200_epilogue_kind {
  FB200_EPI_NONE = 0, FB200_EPI_RESIDUAL = 1, FB200_EPI_SWIGLU = 2, FB200_EPI_BIAS = 3
} fb200_epilogue_kind;

typedef struct fb200_epilogue {
  int kind;
  const float* r1_dev; /* [M, N]; FB200_EPI_BIAS: [N] */
  const float* r2_dev; /* [M, N] or NULL */
} fb200_epilogue;

FB200_API int fb200_q_mat_mul(fb200_device* dev, const float* x_dev, size_t m, const fb200_qmatrix* w,
                    float* y_dev, const fb200_epilogue* epilogue);
/* RMSNorm feeding a projection, as one call: y = epilogue(W . rms_norm(x (+ residual))).
 * The reference authors this as rms_norm_fused / rms_norm_residual_fused followed by q_mat_mul
 * (models/kalosm-llama/src/raw/mod.rs:964,1017 then attention_layer.rs:364-404, 220-235) and
 * its resolver fuses what it can (fusor-ml/core/src/composite/rms_norm_fused.rs:10-54). For
 * one activation row the norm runs in the prologue of the product kernel; other shapes
 * normalise into scratch first. norm_weight_dev is [K]; residual_dev [M, K] or NULL. */
FB200_API int fb200_rms_norm_q_mat_mul(fb200_device* dev, const float* x_dev,
                                       const float* residual_dev, const float* norm_weight_dev,
                                       float eps, size_t m, const fb200_qmatrix* w, float* y_dev,
                                       const fb200_epilogue* epilogue);
/* The same product for callers that must not allocate. This entry point has no counterpart in
 * the reference. fb200_q_mat_mul grows a device scratch buffer (for the activations repacked
 * as integer limbs) with cudaMalloc when a larger product arrives; hosts that cannot enter the
 * CUDA allocator at call time -- a serving loop whose memory budget is frozen after start-up,
 * a callback running on a thread that holds a lock the allocator needs, an embedding
 * application that forbids allocation after initialisation -- call this instead. The scratch is
 * a fixed 4 MiB array inside the library image (every GPU that loads the library carries it
 * until the process exits); neither this function nor anything it calls allocates or frees
 * device or host memory through the CUDA allocator or the C/C++ heap (refusals write their text
 * into fixed storage inside the handle).
 *   - y[M, N] = x[M, K] . W^T, 1 <= M <= 32, W of type Q4_0 / Q5_0 / Q8_0 / Q4_K / Q6_K, no epilogue.
 *   - Every row count, M = 1 included, runs the fp16 tensor-core kernel of the 2..32-row path
 *     (11-bit operands, about 5e-4 relative L2 against fp32; fb200_q_mat_mul sends a single row to
 *     its integer-limb kernel instead, which needs no scratch and is closer to fp32).
 *   - Warm-up: the first call per device looks up the array's device address, and the first call
 *     per (weight type, row bucket 1..8 / 9..16 / 17..32, K) sets that kernel variant's
 *     shared-memory attribute and, under CUDA's lazy loading, loads its code (K selects the
 *     variant: rows of at most 16 block groups take another product kernel than longer rows, and
 *     the packing kernel has variants for K up to 4096 / 8192 / 16384). Make one call of every
 *     combination you will use before entering the region that must not allocate, and before
 *     any stream capture.
 *   - FB200_ERR_CAPACITY when M > 32 or when the packed activations (about 136 bytes per
 *     element of K for 17..32 rows, 68 for 9..16, 34 for 1..8) exceed the 4 MiB array.
 *   - All calls share the one array and it keeps the previous call's contents; each call
 *     rewrites everything it reads, so nothing needs clearing, but two calls whose kernels
 *     overlap on the GPU (different streams or device handles) race on it. Keep calls on one
 *     stream, or otherwise ordered. */
FB200_API int fb200_q_mat_mul_noalloc(fb200_device* dev, const float* x_dev, size_t m,
                                      const fb200_qmatrix* w, float* y_dev);
/* Same product with host buffers: uploads x, runs, downloads y, synchronises. */
FB200_API int fb200_q_mat_mul_host(fb200_device* dev, const float* x_host, size_t m,
                         const fb200_qmatrix* w, float* y_host);

/* ---- elementwise / composite ops ---------------------------------------------------------------
 * rms_norm_fused / rms_norm_residual_fused, fusor-ml/fusor/src/composite/normalization.rs:287-402:
 * y = v / sqrt(mean(v^2) + eps) * w (+ bias), v = x (+ residual); f32; rows x n. */
FB200_API int fb200_rms_norm(fb200_device* dev, const float* x_dev, const float* residual_dev,
                   const float* weight_dev, const float* bias_dev, float eps, size_t rows,
                   size_t n, float* y_dev);
/* silu(gate) * up, fusor-ml/fusor/src/composite/activations.rs:47-64 */
FB200_API int fb200_silu_mul(fb200_device* dev, const float* gate_dev, const float* up_dev, size_t n,
                   float* out_dev);
/* RoPE tables [ctx, head_dim/2]: base_inverse_frequency (composite/rope.rs:241-246) and the
 * Llama-3 scaling of models/kalosm-llama/src/raw/rope.rs:21-38 (factor <= 0 disables it).
 * Computed on the host in f32 exactly as the reference does, then uploaded. */
FB200_API int fb200_rope_tables(fb200_device* dev, int head_dim, int ctx, float theta, float factor,
                      float low_freq_factor, float high_freq_factor, int original_ctx,
                      float* cos_dev, float* sin_dev);
/* RopeCache::forward / forward_interleaved, composite/rope.rs:284-329: q [B,H,S,D] and
 * k [B,Hkv,S,D] rotated in place with table rows start_pos .. start_pos + S. */
FB200_API int fb200_rope_pair(fb200_device* dev, float* q_dev, float* k_dev, int b, int h, int hkv, int s,
                    int d, const float* cos_dev, const float* sin_dev, int start_pos,
                    int interleaved);
/* Embedding::forward, fusor-ml/fusor/src/layers/embedding.rs:43-107: dequantised rows of W. */
FB200_API int fb200_embedding_lookup(fb200_device* dev, const fb200_qmatrix* w, const uint32_t* ids_dev,
                           size_t n_ids, float* out_dev);
/* Tensor::top_k_pairs, fusor-ml/fusor/src/lib.rs:416-453 with k = 1 per row: highest finite
 * logit, ties -> higher token id. ids_dev [rows] u32, vals_dev [rows] f32 (may be NULL). */
FB200_API int fb200_argmax(fb200_device* dev, const float* logits_dev, size_t rows, size_t n,
                 uint32_t* ids_dev, float* vals_dev);
/* Tensor::top_k_pairs(k), fusor-ml/fusor/src/lib.rs:416-453 (GPU form:
 * fusor-ml/core/src/mir/kernel_backend/sampling_topk.rs): per row the k highest finite logits in
 * descending order, ties -> higher token id. ids_dev [rows, k] u32, vals_dev [rows, k] f32 (may
 * be NULL); a row with fewer than k finite logits is padded with id 0xFFFFFFFF / value -inf.
 * 1 <= k <= FB200_SAMPLER_MAX_TOP_K. */
#define FB200_SAMPLER_MAX_TOP_K 1024
FB200_API int fb200_top_k(fb200_device* dev, const float* logits_dev, size_t rows, size_t n, int k,
                          uint32_t* ids_dev, float* vals_dev);

/* ---- on-device samplers: models/kalosm-llama/src/sampler.rs:44-311 (CPU) and
 * fusor-ml/core/src/sampling/{pipeline,row_kernels,processors}.rs (GPU) ------------------------
 * Field meanings are those of GpuSamplerConfig (models/kalosm-llama/src/lib.rs:477-488). Per
 * logit: non-finite values are dropped, tokens among the last repetition_penalty_range previous
 * tokens are penalised (repetition_penalty > 1: positive logits divided, others multiplied), the
 * result is divided by the temperature (if not 0). The top_k survivors, sorted descending (ties
 * -> higher id), then go through min-p, top-p and a cumulative walk against a uniform draw
 * (standard; temperature <= 0 returns the first), or through the surprise cut-off and mu update
 * of Mirostat 2. The uniform draw is a counter-based function of (seed, counter, row) instead of
 * the reference's rand::StdRng stream: equal inputs give equal tokens on every run. */
typedef enum fb200_sampler_strategy { FB200_SAMPLER_STANDARD = 0, FB200_SAMPLER_MIROSTAT2 = 1 } fb200_sampler_strategy;
typedef struct fb200_sampler_config {
  int strategy;
  float temperature;
  float repetition_penalty;
  int repetition_penalty_range;
  int top_k;      /* 1 .. FB200_SAMPLER_MAX_TOP_K */
  float top_p;    /* >= 1 or NaN: off */
  float min_p;    /* <= 0 or NaN: off */
  float tau, eta, mu; /* Mirostat 2: target surprise, learning rate, initial mu */
  uint64_t seed;
} fb200_sampler_config;
/* One sampling step over logits_dev [rows, n]. prev_dev [rows, prev_stride] u32 holds each row's
 * previous tokens, the first prev_len of them valid (NULL / 0: none). counter selects the draw.
 * mu_dev [rows] f32 is the Mirostat state (read and updated; NULL for the standard sampler).
 * ids_dev [rows] receives the sampled ids (0xFFFFFFFF for a row without a finite logit). */
FB200_API int fb200_sample(fb200_device* dev, const float* logits_dev, size_t rows, size_t n,
                           const fb200_sampler_config* cfg, const uint32_t* prev_dev, size_t prev_stride,
                           int prev_len, uint64_t counter, float* mu_dev, uint32_t* ids_dev);

/* ---- KV cache: KvCache / TensorCache, fusor-ml/fusor/src/cache/kv_cache.rs:12-68 ----------------
 * Layout [B, Hkv, capacity, D], fp16 on the device (the reference's cache is f32). Capacity
 * follows tensor_cache.rs:304-312 (next power of two, at least 256, at most max_seq_len) and
 * grows by reallocation + copy. Appending beyond max_seq_len returns FB200_ERR_CAPACITY (the
 * reference evicts the oldest entries, tensor_cache.rs:175-202). */
FB200_API int fb200_kv_cache_create(fb200_device* dev, int batch, int n_kv_head, int head_dim,
                          int max_seq_len, fb200_kv_cache** out);
FB200_API int fb200_kv_cache_free(fb200_kv_cache* c);
FB200_API int fb200_kv_cache_reset(fb200_kv_cache* c);
FB200_API int fb200_kv_cache_len(const fb200_kv_cache* c, int* len_out, int* capacity_out);
/* Drops the positions from `len` on (0 <= len <= current length): the tokens a session shares
 * with its cache stay, the rest is recomputed. The reference trims its cache this way before it
 * re-prefills (models/kalosm-llama/src/raw/mod.rs:769-793, TensorCache truncation in
 * fusor-ml/fusor/src/cache/tensor_cache.rs:175-202). */
FB200_API int fb200_kv_cache_truncate(fb200_kv_cache* c, int len);
/* k, v f32 [B, Hkv, S, D]; rounded to fp16 and stored at positions len .. len + S. */
FB200_API int fb200_kv_cache_append(fb200_kv_cache* c, const float* k_dev, const float* v_dev, int s);
/* Device pointers of the fp16 K and V buffers ([B, Hkv, capacity, D]). */
FB200_API int fb200_kv_cache_buffers(const fb200_kv_cache* c, const void** k_dev, const void** v_dev);

/* ---- attention: Tensor::flash_attention, fusor-ml/fusor/src/composite/flash_attention.rs:58-236 --
 * out = softmax(q.k^T * scale + mask).v, GQA by kv_head = head / (H / Hkv). q, out f32
 * [B,H,Sq,D]; k, v fp16 [B,Hkv,*,D] with kv_capacity rows allocated per head and the first
 * skv rows valid. mask_kind: 0 none, 1 causal (query row i sees keys 0 .. i + skv - sq;
 * AttentionMask::causal, cache/attention_mask.rs:45-65 with the left padding of
 * mask_cache.rs:74-85), 2 additive f32 [Sq, Skv], 3 additive f32 [B, Skv]. */
FB200_API int fb200_flash_attention(fb200_device* dev, const float* q_dev, const void* k_dev,
                          const void* v_dev, int b, int h, int hkv, int sq, int skv,
                          int kv_capacity, int d, float scale, const float* mask_dev,
                          int mask_kind, float* out_dev);

/* ---- whole model: Model::forward, models/kalosm-llama/src/raw/mod.rs:851-1049 -------------------
 * Llama-architecture decoder (separate q/k/v, SiLU-gated FFN, interleaved RoPE, raw/mod.rs:488-490).
 * The model owns its KV caches, activation buffers and the CUDA graph of a decode step. */
typedef struct fb200_llama_config {
  int n_layer, hidden, ffn, n_head, n_kv_head, head_dim, vocab;
  int max_seq_len; /* context_length */
  int max_batch;
  float rms_eps;    /* llama.attention.layer_norm_rms_epsilon, raw/mod.rs:383 */
  float rope_theta; /* llama.rope.freq_base */
  float rope_factor, rope_low_freq_factor, rope_high_freq_factor;
  int rope_original_ctx;
} fb200_llama_config;

typedef enum fb200_llama_tensor {
  FB200_T_TOKEN_EMBD = 0, FB200_T_OUTPUT = 1, FB200_T_ATTN_Q = 2, FB200_T_ATTN_K = 3,
  FB200_T_ATTN_V = 4, FB200_T_ATTN_OUTPUT = 5, FB200_T_FFN_GATE = 6, FB200_T_FFN_UP = 7,
  FB200_T_FFN_DOWN = 8, FB200_T_ATTN_NORM = 9, FB200_T_FFN_NORM = 10, FB200_T_OUTPUT_NORM = 11
} fb200_llama_tensor;

FB200_API int fb200_llama_create(fb200_device* dev, const fb200_llama_config* cfg, fb200_llama** out);
FB200_API int fb200_llama_free(fb200_llama* m);
/* Tensor names of raw/mod.rs:473-646: blk.{i}.attn_q.weight ... ; norms are f32 vectors
 * (ggml_type FB200_F32), everything else raw GGUF blocks of shape [N, K]. `layer` is ignored
 * for the three model-level tensors. Missing FB200_T_OUTPUT ties it to the embedding
 * (raw/mod.rs:480-486). */
FB200_API int fb200_llama_set_tensor(fb200_llama* m, int layer, int which, uint32_t ggml_type,
                           uint64_t n, uint64_t k, const void* bytes_host, size_t nbytes);
/* The rope_freqs.weight tensor of a checkpoint (head_dim / 2 f32 values): multiplied into the
 * inverse frequencies after the Llama-3 scaling, as create_inverse_frequency does
 * (models/kalosm-llama/src/raw/rope.rs:9-52; loaded at raw/mod.rs:417-421). Rebuilds the model's
 * RoPE tables; call before the first forward pass. */
FB200_API int fb200_llama_set_rope_freqs(fb200_llama* m, const float* weights_host, size_t n);
FB200_API int fb200_llama_reset(fb200_llama* m);
/* Rewinds the model's KV caches to the first `len` positions (0 <= len <= position): the next
 * forward pass continues from there (raw/mod.rs:769-793 keeps the common prefix of the cached
 * and the new tokens and re-runs the rest). */
FB200_API int fb200_llama_truncate(fb200_llama* m, int len);
FB200_API int fb200_llama_position(const fb200_llama* m, int* pos_out);
/* tokens_host [batch, seq] u32. Runs the forward pass over `seq` new positions and writes the
 * logits of the last position, f32 [batch, vocab], to logits_host if not NULL, and the greedy
 * token per batch row to next_host if not NULL (tie -> higher id). Blocks until done. */
FB200_API int fb200_llama_forward(fb200_llama* m, const uint32_t* tokens_host, int batch, int seq,
                        float* logits_host, uint32_t* next_host);
/* Greedy decode: feeds tokens_host [batch] and then its own argmax for `steps` steps entirely
 * on the device (replaying the captured CUDA graph); out_host [batch, steps] receives the
 * generated ids. Only the ids cross PCIe. */
FB200_API int fb200_llama_generate_greedy(fb200_llama* m, const uint32_t* tokens_host, int batch,
                                int steps, uint32_t* out_host);
/* Sampled decode: like fb200_llama_generate_greedy, but every step's token comes from the sampler
 * (fb200_sampler_config) run on the device over that step's logits; the penalty window is the
 * session's own token history (every token fed to or produced by the model since the last
 * reset), the draw counter is the token's position. All steps are enqueued without waiting for
 * any of them, the run-ahead of models/kalosm-llama/src/model/inference.rs:41-170; only the ids
 * come back. Not available on a tensor-parallel model (the logits are sharded). */
FB200_API int fb200_llama_generate_sampled(fb200_llama* m, const uint32_t* tokens_host, int batch, int steps,
                                           const fb200_sampler_config* cfg, uint32_t* out_host);
/* Device pointer of the last forward pass's logits, f32 [batch, vocab] (tensor parallel:
 * [batch, vocab / size], this rank's rows of the output head). */
FB200_API int fb200_llama_logits_dev(const fb200_llama* m, const float** logits_dev);

/* ---- tensor parallelism (no counterpart in the reference, which runs one device) ------------
 * One process and one device handle per GPU. Rank 0 makes an id (FB200_COMM_ID_BYTES bytes) and
 * hands it to the other ranks by any host channel; every rank then calls fb200_comm_create, which
 * blocks until all `size` ranks have joined (NCCL, loaded at run time: FB200_ERR_NCCL if absent).
 * A tensor-parallel model is created from the LOCAL configuration (n_head, n_kv_head and ffn
 * divided by size; hidden and vocab whole), attached to the communicator before any tensor is
 * set, and given this rank's shards: attn_q / attn_k / attn_v / ffn_gate / ffn_up rows
 * [rank * N / size, (rank + 1) * N / size), attn_output / ffn_down the matching K columns (whole
 * quantisation blocks), output rows [rank * vocab / size, ...); token_embd and the norms whole.
 * The partial sums of attn_output and ffn_down are added over the ranks (two all-reduces per
 * layer) and the greedy token is the best (value, id) pair over the ranks' shards of the output
 * head, so every rank returns the same ids. */
#define FB200_COMM_ID_BYTES 128
typedef struct fb200_comm fb200_comm;
FB200_API int fb200_comm_unique_id(uint8_t* id_out, size_t id_bytes);
FB200_API int fb200_comm_create(fb200_device* dev, int size, int rank, const uint8_t* id, size_t id_bytes,
                                fb200_comm** out);
FB200_API int fb200_comm_destroy(fb200_comm* c);
/* In-place sum of buf_dev[n] (f32) over the ranks, asynchronous on the device handle's stream. */
FB200_API int fb200_comm_all_reduce_sum(fb200_comm* c, float* buf_dev, size_t n);
/* Peer exchange of the single-sequence decode kernel (optional; without it the step uses the
 * NCCL sums above): every rank makes a buffer for rows of row_floats floats (the model's hidden
 * size) and gets an FB200_IPC_HANDLE_BYTES handle; the handles of all ranks, in rank order, go to
 * every rank's _attach, which maps the peers' buffers (CUDA IPC, ranks are processes of one node
 * with NVLink / P2P access). The decode kernel then writes its partial rows straight into the
 * peers' buffers and sums them itself: no library collective on the step's critical path. */
#define FB200_IPC_HANDLE_BYTES 64
FB200_API int fb200_comm_exchange_handle(fb200_comm* c, size_t row_floats, uint8_t* handle_out, size_t handle_bytes);
FB200_API int fb200_comm_exchange_attach(fb200_comm* c, const uint8_t* handles, size_t handle_bytes);
/* Diagnostic: runs the bounded arrival wait of the peer exchange on a word that nothing sets.
 * Returns FB200_ERR_TIMEOUT after poll_limit polls and leaves that code in the handle's status
 * word, exactly as a peer that never arrives would; the context stays usable. */
FB200_API int fb200_exchange_wait_check(fb200_device* dev, int poll_limit);
/* Must precede fb200_llama_set_tensor. The communicator must outlive the model. */
FB200_API int fb200_llama_set_tensor_parallel(fb200_llama* m, fb200_comm* comm);

#ifdef __cplusplus
}
#endif
#endif /* FUSOR_B200_H */
