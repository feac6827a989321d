// Whole-model host code: Llama-architecture decoder on one device.
//
// Order of operations follows Model::forward_last_hidden_from_embeddings
// (models/kalosm-llama/src/raw/mod.rs:925-1049): pre-norm -> attention -> residual + norm ->
// SiLU-gated FFN -> + attention output + residual; final norm; only the last position reaches
// the output projection (:1046). Attention block: LlamaAttention::forward
// (raw/attention_layer.rs:514-573) with separate q/k/v projections (:281-427), interleaved RoPE
// (raw/mod.rs:488-490) and a KV cache per layer (raw/cache.rs:14-46).
// The reference's lazy graph + resolver (fusor-ml/core/src/compute_graph/resolve/run.rs:29-135)
// is replaced by a fixed kernel sequence on one CUDA stream; a single-token step is captured
// into a CUDA graph whose kernels read the position from device memory, so it replays as is.
#include <cstring>
#include <memory>

#include "common.cuh"
#include "fused_step.cuh"
#include "packed_act.cuh"

void fb200_rope_tables_host(int head_dim, int ctx, float theta, float factor, float low_ff,
                            float high_ff, int original_ctx, const float* freq_weight,
                            std::vector<float>& cs, std::vector<float>& sn);
int fb200_launch_rms_norm_strided(fb200_device* dev, const float* x, size_t x_stride,
                                  const float* res, const float* w, float eps, size_t rows,
                                  size_t n, float* y);
int fb200_launch_argmax(fb200_device* dev, const float* logits, size_t rows, size_t n,
                        uint32_t* ids, float* vals);
int fb200_launch_attention(fb200_device* dev, const float* q, const __half* k, const __half* v,
                           int b, int h, int hkv, int sq, int skv, const int* skv_dev, int cap,
                           int d, float scale, const float* mask, int mask_kind, float* out,
                           float* part, int nsplit, int bshd);
size_t fb200_xpack_bytes(int mp, uint64_t kp);
int fb200_pack16_rows(int mc);
int fb200_qgemm_group(fb200_device* dev, const fb200_qmatrix* const* ws, float* const* ys, int n, const float* x, size_t m);
uint64_t fb200_qmatrix_kp(const fb200_qmatrix* w);
int fb200_pack_x16(fb200_device* dev, const float* x, int mc, uint64_t k, uint64_t kp, void* scratch, const void** xh,
                   const float** xscale);
int fb200_norm_pack_x16(fb200_device* dev, const float* x, size_t x_stride, const float* res, const float* w, float eps,
                        int mc, uint64_t k, uint64_t kp, void* scratch, const void** xh, const float** xscale);
int fb200_qgemm16_packed(fb200_device* dev, const fb200_qmatrix* w, const void* xh, const float* xscale16, int mc, int mp,
                         float* y, int epi, const float* r1, const float* r2, bool r1_is_bias);
int fb200_qgemm16_packed_multi(fb200_device* dev, const fb200_qmatrix* const* ws, float* const* ys, int nw, const void* xh,
                               const float* xscale16, int mc, int mp);
int fb200_attention_nsplit(const fb200_device* dev, int b, int hkv, int groups, int sq, int skv);
int fb200_launch_attention_decode_args(fb200_device* dev, const fb200_dec_args& a, int d);
bool fb200_qgemv1_fits(const fb200_qmatrix* w);
int fb200_attention_scratch_bytes(int b, int h, int sq, int d, int nsplit, size_t* out);
struct fb200_comm;
int fb200_comm_all_reduce(fb200_comm* c, float* buf, size_t n);
int fb200_comm_all_gather_bytes(fb200_comm* c, const void* in, void* out, size_t bytes);
int fb200_comm_rank(const fb200_comm* c);
int fb200_comm_size(const fb200_comm* c);
fb200_device* fb200_comm_device(const fb200_comm* c);
bool fb200_comm_take_exchange(fb200_comm* c, int row_floats, unsigned count, fb200_fused_xchg* out);
bool fb200_comm_exchange_ready(const fb200_comm* c, int row_floats);
void fb200_comm_mark_broken(fb200_comm* c);
int fb200_launch_sampler(fb200_device* dev, const float* logits, size_t rows, size_t n, const fb200_sampler_config* c,
                         const uint32_t* prev, size_t prev_stride, int prev_len, unsigned long long counter, float* mu,
                         uint32_t* ids, uint32_t* also0, size_t stride0, uint32_t* also1, size_t stride1);

namespace {

struct LayerW {
  fb200_qmatrix *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr;
  fb200_qmatrix *gate = nullptr, *up = nullptr, *down = nullptr, *gate_up = nullptr;
  float *attn_norm = nullptr, *ffn_norm = nullptr;
  __half *kc = nullptr, *vc = nullptr;  // [max_batch, Hkv, max_seq, D]
};

// q [rows, H*D] rotated in place; k rotated and v copied into the fp16 cache at position
// *pos + s. Row = b * S + s. RoPE pairs are interleaved (2p, 2p+1) as in
// fusor-ml/fusor/src/composite/rope.rs:77-108; append as KvCache::append
// (fusor-ml/fusor/src/cache/kv_cache.rs:50-62).
__global__ void rope_append_kernel(float* __restrict__ q, const float* __restrict__ k,
                                   const float* __restrict__ v, __half* __restrict__ kc,
                                   __half* __restrict__ vc, const float* __restrict__ cs,
                                   const float* __restrict__ sn, const int* __restrict__ pos_dev,
                                   int s_len, int h, int hkv, int d, int cap, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int half = d >> 1;
  const int per_row = (h + 2 * hkv) * half;
  const size_t row = i / per_row;
  int rem = (int)(i % per_row);
  const int b = (int)(row / s_len), s = (int)(row % s_len);
  const int pos = *pos_dev + s;
  if (rem < h * half) {
    const int head = rem / half, p = rem % half;
    float* x = q + (row * h + head) * d;
    const float c = cs[(size_t)pos * half + p], sv = sn[(size_t)pos * half + p];
    const float x0 = x[2 * p], x1 = x[2 * p + 1];
    x[2 * p] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sv));
    x[2 * p + 1] = __fadd_rn(__fmul_rn(x0, sv), __fmul_rn(x1, c));
    return;
  }
  rem -= h * half;
  const bool is_v = rem >= hkv * half;
  if (is_v) rem -= hkv * half;
  const int head = rem / half, p = rem % half;
  const size_t dst = (((size_t)b * hkv + head) * cap + pos) * d + 2 * p;
  if (is_v) {
    const float* x = v + (row * hkv + head) * d;
    *reinterpret_cast<__half2*>(vc + dst) = __floats2half2_rn(x[2 * p], x[2 * p + 1]);
  } else {
    const float* x = k + (row * hkv + head) * d;
    const float c = cs[(size_t)pos * half + p], sv = sn[(size_t)pos * half + p];
    const float x0 = x[2 * p], x1 = x[2 * p + 1];
    const float y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sv));
    const float y1 = __fadd_rn(__fmul_rn(x0, sv), __fmul_rn(x1, c));
    *reinterpret_cast<__half2*>(kc + dst) = __floats2half2_rn(y0, y1);
  }
}

// After a greedy step: record the new ids, feed them back, advance the position.
__global__ void advance_kernel(uint32_t* __restrict__ next, uint32_t* __restrict__ ids,
                               uint32_t* __restrict__ hist, int* pos_dev, int* step_dev, int batch,
                               int max_steps, int advance, unsigned long long* argmax_key) {
  const int b = threadIdx.x;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int step = *step_dev;
  if (argmax_key && b == 0) {
    // the output projection kept a running (value, index) maximum; 0 means no finite logit
    const unsigned long long key = *argmax_key;
    next[0] = key ? (uint32_t)(key & 0xFFFFFFFFull) : 0xFFFFFFFFu;
    *argmax_key = 0ull;
  }
  __syncthreads();
  if (b < batch) {
    ids[b] = next[b];
    if (hist && step < max_steps) hist[(size_t)b * max_steps + step] = next[b];
  }
  __syncthreads();
  if (b == 0) {
    *pos_dev += advance;
    *step_dev = step + 1;
  }
}

}  // namespace

struct fb200_llama {
  fb200_device* dev = nullptr;
  fb200_llama_config cfg{};
  fb200_qmatrix *token_embd = nullptr, *output = nullptr;
  float* output_norm = nullptr;
  std::vector<LayerW> layers;
  float *rope_cos = nullptr, *rope_sin = nullptr;
  bool finalized = false;
  int pos = 0;
  // activation buffers, sized for `rows_cap` rows
  size_t rows_cap = 0;
  float *x = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr,
        *attn_out = nullptr, *hbuf = nullptr, *gbuf = nullptr, *last = nullptr, *logits = nullptr;
  float* att_part = nullptr;
  size_t att_part_bytes = 0;
  uint32_t *ids = nullptr, *next = nullptr, *hist = nullptr;
  int hist_cap = 0;
  // every token fed to or produced by the model since the last reset, [max_batch, max_seq_len + 1]:
  // the penalty window of the samplers
  uint32_t* tok_hist = nullptr;
  float* mu_dev = nullptr;  // [max_batch] Mirostat 2 state of a sampled decode
  int *pos_dev = nullptr, *step_dev = nullptr;
  unsigned long long* argmax_key = nullptr;
  int* att_done = nullptr;  // arrival counters of the attention splits, one per (batch, kv head)
  // single-row step: activation rows travel between kernels in the products' operand form
  fb200_packed_act px, patt, pv, ph;  // residual stream, attention output, attn_out + x, SwiGLU output
  // the same rows (and q / k / v, the residual stream and the attention projection as f32) as flagged
  // rows for the barrier-free variants of the persistent kernel: one slab, zero at creation
  uint8_t* ll_slab = nullptr;
  fb200_ll_act px_ll, patt_ll, pv_ll, ph_ll;
  uint2 *q_ll = nullptr, *k_ll = nullptr, *v_ll = nullptr, *x_ll = nullptr, *attn_ll = nullptr;
  // FB200_FUSED_LL=1 selects the barrier-free variants. Off by default: they are correct (parity
  // tests run both forms) but measured slower so far (2.2 - 2.6 ms per step of the 8B-shaped model
  // against 2.03 ms with grid barriers): the trip a flagged row saves at each phase boundary is
  // outweighed by slower epilogues (8-byte flagged stores), the 86 KB polled row in front of the
  // down projection and a product loop that gets fewer registers.
  bool fused_flagged = false;
  bool fused_is_flagged = false;  // the current program uses the flagged rows
  bool used_key = false;  // the last forward pass left its greedy id in argmax_key, not in next
  // CUDA graph of a single-token step, per batch size
  cudaGraphExec_t graph_exec = nullptr;
  int graph_batch = 0;
  uint64_t graph_kernels = 0;  // kernels inside the captured step
  uint64_t graph_gen = 0;      // the handle's scratch generation the capture recorded addresses of
  // single-sequence step as one persistent kernel: its program (host and device copies)
  bool fused_enabled = true;   // FB200_FUSED=0 keeps the multi-kernel step
  bool fused_valid = false;    // the program matches the current buffers
  bool fused_usable = false;
  std::vector<fb200_fused_phase> prog_host;
  fb200_fused_phase* prog_dev = nullptr;
  // tensor parallelism: cfg holds the local head / ffn counts; the output head has vocab_local rows
  fb200_comm* comm = nullptr;
  int tp_rank = 0, tp_size = 1, vocab_local = 0;
  float* best_val = nullptr;            // [max_batch] value of the local greedy candidate
  unsigned long long* best_pair = nullptr;  // [(1 + size) * max_batch] (value, global id) pairs
};

namespace {

int alloc_f(fb200_device* dev, float** p, size_t n) {
  if (*p) { cudaFree(*p); *p = nullptr; }
  FB_CUDA(dev, cudaMalloc(p, (n ? n : 1) * sizeof(float)));
  return FB200_OK;
}

int ensure_rows(fb200_llama* m, size_t rows) {
  if (rows <= m->rows_cap) return FB200_OK;
  fb200_device* dev = m->dev;
  const auto& c = m->cfg;
  FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  if (m->graph_exec) { cudaGraphExecDestroy(m->graph_exec); m->graph_exec = nullptr; }
  m->fused_valid = false;  // the program holds pointers into these buffers
  int rc;
  if ((rc = alloc_f(dev, &m->x, rows * c.hidden))) return rc;
  if ((rc = alloc_f(dev, &m->xn, rows * c.hidden))) return rc;
  if ((rc = alloc_f(dev, &m->q, rows * c.n_head * c.head_dim))) return rc;
  if ((rc = alloc_f(dev, &m->k, rows * c.n_kv_head * c.head_dim))) return rc;
  if ((rc = alloc_f(dev, &m->v, rows * c.n_kv_head * c.head_dim))) return rc;
  if ((rc = alloc_f(dev, &m->att, rows * c.n_head * c.head_dim))) return rc;
  if ((rc = alloc_f(dev, &m->attn_out, rows * c.hidden))) return rc;
  if ((rc = alloc_f(dev, &m->hbuf, rows * c.ffn))) return rc;
  if ((rc = alloc_f(dev, &m->gbuf, rows * c.ffn))) return rc;
  if (m->ids) cudaFree(m->ids);
  FB_CUDA(dev, cudaMalloc(&m->ids, rows * sizeof(uint32_t)));
  m->rows_cap = rows;
  return FB200_OK;
}

int finalize(fb200_llama* m) {
  if (m->finalized) return FB200_OK;
  fb200_device* dev = m->dev;
  const auto& c = m->cfg;
  if (!m->token_embd || !m->output_norm)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama: token_embd / output_norm not set");
  if (m->tp_size > 1 && !m->output)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama: a tensor-parallel model needs its shard of the output head");
  for (int i = 0; i < c.n_layer; ++i) {
    LayerW& L = m->layers[i];
    if (!L.wq || !L.wk || !L.wv || !L.wo || !L.gate || !L.up || !L.down || !L.attn_norm || !L.ffn_norm)
      return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama: layer %d is missing a tensor", i);
    if (!L.gate_up) {
      // QMatrix::concat_rows (fusor-ml/fusor/src/quantized.rs:102-112): gate and up share one
      // launch with the SwiGLU epilogue when their types match.
      const fb200_qmatrix* pair[2] = {L.gate, L.up};
      fb200_qmatrix* gu = nullptr;
      if (L.gate->tiled && L.gate->type == L.up->type && L.gate->n == L.up->n && L.gate->n % 16 == 0 &&
          fb200_qmatrix_concat_rows(pair, 2, &gu) == FB200_OK) {
        L.gate_up = gu;
        fb200_qmatrix_free(L.gate);
        fb200_qmatrix_free(L.up);
        L.gate = L.up = nullptr;
      }
    }
  }
  m->finalized = true;
  return FB200_OK;
}

// Shapes the fused single-sequence step takes: gate and up concatenated, every matrix tiled and
// small enough for its activation row to sit in shared memory, q/k/v with one K group size,
// at most 8 query heads per KV head.
bool decode1_supported(const fb200_llama* m) {
  const auto& c = m->cfg;
  if (c.n_head / c.n_kv_head > 8) return false;
  for (const auto& L : m->layers) {
    if (!L.gate_up) return false;
    const fb200_qmatrix* qs[] = {L.wq, L.wk, L.wv, L.wo, L.gate_up, L.down};
    for (auto* q : qs) if (!q->tiled || !fb200_qgemv1_fits(q)) return false;
    TileGeom a, b, cc;
    tile_geom(L.wq->type, &a); tile_geom(L.wk->type, &b); tile_geom(L.wv->type, &cc);
    if (a.group_elems != b.group_elems || a.group_elems != cc.group_elems) return false;
  }
  const fb200_qmatrix* ow = m->output ? m->output : m->token_embd;
  return ow->tiled && fb200_qgemv1_fits(ow);
}

// One new position of one sequence as the program of the persistent fused kernel:
//   embedding -> packed row (times the first attention norm weight)
//   per layer: q/k/v product | RoPE + append + attention | output projection (packs attn_out + x
//   times the FFN norm weight) | gate/up product with SwiGLU | down product with both residuals
//   (packs the new residual stream times the next norm weight)
//   output head with running argmax key | greedy id, position + 1
int build_fused_program(fb200_llama* m) {
  if (m->fused_valid) return FB200_OK;
  fb200_device* dev = m->dev;
  const auto& c = m->cfg;
  m->fused_usable = false;
  m->fused_valid = true;
  if (!m->fused_enabled || !decode1_supported(m)) return FB200_OK;
  if (m->tp_size > 1 && !fb200_comm_exchange_ready(m->comm, m->cfg.hidden)) return FB200_OK;
  if (m->tp_size > 1)  // the exchange variants of the kernel exist for K-quant weights only
    for (const auto& L : m->layers)
      for (const fb200_qmatrix* q : {L.wq, L.wk, L.wv, L.wo, L.gate_up, L.down})
        if (q->type == FB200_Q4_0 || q->type == FB200_Q8_0) return FB200_OK;
  const int grid = fb200_fused_grid(dev);
  const int H = c.n_head, HK = c.n_kv_head, D = c.head_dim;
  std::vector<fb200_fused_phase> prog;
  auto blank = [] { fb200_fused_phase p; std::memset(&p, 0, sizeof(p)); p.next_gemv = -1; p.xs_index = -1; return p; };
  // tensor parallel: the partial rows of the o and down projections go to the peers' exchange
  // buffers and an XSUM phase adds them up (needs the peer exchange; otherwise the step runs as
  // separate kernels with NCCL sums)
  const bool tp = m->tp_size > 1;
  // the barrier-free variants: one GPU, K-quant weights (decided before the phases are laid out: their
  // weight ring is deeper)
  bool kquant = true;
  for (const auto& L : m->layers)
    for (const fb200_qmatrix* q : {L.wq, L.wk, L.wv, L.wo, L.gate_up, L.down})
      kquant = kquant && (q->type == FB200_Q4_K || q->type == FB200_Q6_K);
  {
    const fb200_qmatrix* ow = m->output ? m->output : m->token_embd;
    kquant = kquant && (ow->type == FB200_Q4_K || ow->type == FB200_Q6_K);
  }
  const bool flagged = m->fused_flagged && !tp && kquant;
  {
    fb200_fused_phase p = blank();
    p.kind = FB200_PH_EMBED;
    p.K = c.hidden;
    p.emb = m->token_embd->data;
    p.emb_type = (int)m->token_embd->type;
    p.emb_tiled = m->token_embd->tiled ? 1 : 0;
    p.emb_n = m->token_embd->n;
    if (m->token_embd->tiled) {
      TileGeom g;
      tile_geom(m->token_embd->type, &g);
      p.emb_ngroups = m->token_embd->ngroups; p.emb_ge = g.group_elems; p.emb_tgb = g.tg_bytes;
    }
    p.ids = m->ids;
    p.xout = m->x;
    p.yp = m->px;
    p.yp_norm_w = m->layers[0].attn_norm;
    p.xoutl = m->x_ll; p.yll = m->px_ll;
    if (flagged) p.xout = nullptr;
    prog.push_back(p);
  }
  int nsplit = grid / HK;
  if (nsplit > 32) nsplit = 32;
  if (nsplit < 1) nsplit = 1;
  if ((size_t)nsplit * H * (D + 2) * sizeof(float) > m->att_part_bytes) return FB200_OK;
  auto gemv = [&](const fb200_qmatrix* const* ws, float* const* ys, int nw, int epi, fb200_fused_phase& p) {
    p = blank();
    p.eps = c.rms_eps;
    return fb200_fused_gemv_phase(&p, ws, ys, nw, epi, grid, flagged);
  };
  for (int li = 0; li < c.n_layer; ++li) {
    LayerW& L = m->layers[li];
    fb200_fused_phase p;
    const fb200_qmatrix* qkv[3] = {L.wq, L.wk, L.wv};
    float* qkv_out[3] = {m->q, m->k, m->v};
    if (!gemv(qkv, qkv_out, 3, FB200_EPI_NONE, p)) return FB200_OK;
    p.xp = m->px; p.xp_norm = 1;
    p.xll = m->px_ll; p.seg[0].yl = m->q_ll; p.seg[1].yl = m->k_ll; p.seg[2].yl = m->v_ll;
    if (flagged) p.seg[0].y = p.seg[1].y = p.seg[2].y = nullptr;  // the flagged rows are the only copy
    prog.push_back(p);

    p = blank();
    p.kind = FB200_PH_ATTN;
    p.att_d = D;
    p.att.q = m->q; p.att.k_new = m->k; p.att.v_new = m->v; p.att.kc = L.kc; p.att.vc = L.vc;
    p.att.rope_cos = m->rope_cos; p.att.rope_sin = m->rope_sin; p.att.pos_dev = m->pos_dev;
    p.att.part = m->att_part; p.att.out = nullptr; p.att.done = m->att_done; p.att.out_packed = m->patt;
    p.att.b = 1; p.att.h = H; p.att.hkv = HK; p.att.groups = H / HK; p.att.cap = c.max_seq_len;
    p.att.nsplit = nsplit; p.att.scale = (float)(1.0 / sqrt((double)D));
    p.att.q_ll = m->q_ll; p.att.k_ll = m->k_ll; p.att.v_ll = m->v_ll; p.att.out_ll = m->patt_ll;
    prog.push_back(p);

    const fb200_qmatrix* wo = L.wo;
    float* wo_out = tp ? nullptr : m->attn_out;
    if (!gemv(&wo, &wo_out, 1, FB200_EPI_NONE, p)) return FB200_OK;
    p.xp = m->patt;
    // flagged rows: attn_out as granules; the packed row is (attn_out + x) times the FFN norm weight, x
    // published three phases earlier (the previous layer's down projection, or the embedding)
    p.xll = m->patt_ll; p.seg[0].yl = m->attn_ll; p.yll = m->pv_ll; p.addl = m->x_ll; p.add_back = 3;
    if (flagged) p.seg[0].y = nullptr;
    if (tp) {
      p.xs_index = 2 * li;
      prog.push_back(p);
      p = blank();
      p.kind = FB200_PH_XSUM; p.K = c.hidden; p.xs_index = 2 * li;
      p.out_sum = m->attn_out; p.src = m->x;            // attn_out = sum; packed row = (attn_out + x) w
    }
    p.yp = m->pv; p.yp_add = tp ? nullptr : m->x; p.yp_norm_w = L.ffn_norm;
    prog.push_back(p);

    const fb200_qmatrix* gu = L.gate_up;
    float* gu_out = nullptr;
    if (!gemv(&gu, &gu_out, 1, FB200_EPI_SWIGLU, p)) return FB200_OK;
    p.xp = m->pv; p.xp_norm = 1;
    p.yp = m->ph;
    p.xll = m->pv_ll; p.yll = m->ph_ll;
    prog.push_back(p);

    const fb200_qmatrix* dn = L.down;
    float* dn_out = tp ? nullptr : m->x;
    if (!gemv(&dn, &dn_out, 1, tp ? FB200_EPI_NONE : FB200_EPI_RESIDUAL, p)) return FB200_OK;
    p.xp = m->ph;
    // flagged rows: x = (down + attn_out) + x with attn_out from two phases back and x from five
    p.xll = m->ph_ll; p.seg[0].yl = m->x_ll; p.yll = m->px_ll;
    p.r1l = m->attn_ll; p.r1_back = 2; p.r2l = m->x_ll; p.r2_back = 5;
    if (flagged) p.seg[0].y = nullptr;
    if (tp) {
      p.xs_index = 2 * li + 1;
      prog.push_back(p);
      p = blank();
      p.kind = FB200_PH_XSUM; p.K = c.hidden; p.xs_index = 2 * li + 1;
      p.src = m->attn_out; p.src_add = m->x; p.xout = m->x;   // x = (sum + attn_out) + x
    } else {
      p.r1 = m->attn_out; p.r2 = m->x;
    }
    p.yp = m->px;
    p.yp_norm_w = li + 1 < c.n_layer ? m->layers[li + 1].attn_norm : m->output_norm;
    prog.push_back(p);
  }
  {
    fb200_fused_phase p;
    const fb200_qmatrix* ow = m->output ? m->output : m->token_embd;
    float* lg = m->logits;
    if (!gemv(&ow, &lg, 1, FB200_EPI_NONE, p)) return FB200_OK;
    p.xp = m->px; p.xp_norm = 1;
    p.xll = m->px_ll;
    p.argmax_key = m->argmax_key;
    prog.push_back(p);
    p = blank();
    p.kind = FB200_PH_ADVANCE;
    p.argmax_key = m->argmax_key;
    p.next = m->next; p.ids_w = m->ids; p.hist = m->hist; p.pos_dev = m->pos_dev; p.step_dev = m->step_dev;
    p.hist_cap = m->hist_cap;
    if (tp) p.xs_index = 2 * c.n_layer;  // the greedy key of the sharded output head is exchanged too
    prog.push_back(p);
  }
  // chain the product phases (the last one wraps to the first, used when several steps run in one launch)
  int first = -1, prev = -1;
  for (int i = 0; i < (int)prog.size(); ++i) {
    if (prog[i].kind != FB200_PH_GEMV) continue;
    if (first < 0) first = i;
    if (prev >= 0) prog[prev].next_gemv = i;
    prev = i;
  }
  if (prev >= 0) prog[prev].next_gemv = first;
  {
    // weights requested into L2 ahead of their phase; FB200_FUSED_L2_AHEAD_MB = 0 turns the plan off
    size_t ahead_mb = 0;
    if (const char* e = getenv("FB200_FUSED_L2_AHEAD_MB")) ahead_mb = (size_t)std::max(0, atoi(e));
    fb200_fused_plan_prefetch(prog.data(), (int)prog.size(), fb200_fused_grid(dev), ahead_mb << 20);
  }
  // the barrier-free variants: one GPU, K-quant weights
  m->fused_is_flagged = flagged && fb200_fused_flagged_available(prog.data(), (int)prog.size());
  if (flagged && !m->fused_is_flagged) return FB200_OK;  // laid out for a variant that does not exist
  if (!fb200_fused_smem_bytes(prog.data(), (int)prog.size(), m->fused_is_flagged)) return FB200_OK;
  FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  if (m->prog_dev) { cudaFree(m->prog_dev); m->prog_dev = nullptr; }
  FB_CUDA(dev, cudaMalloc(&m->prog_dev, prog.size() * sizeof(fb200_fused_phase)));
  FB_CUDA(dev, cudaMemcpy(m->prog_dev, prog.data(), prog.size() * sizeof(fb200_fused_phase), cudaMemcpyHostToDevice));
  m->prog_host = std::move(prog);
  m->fused_usable = true;
  return FB200_OK;
}

// `steps` greedy single-token steps of one sequence in fused launches; ids are already in m->ids.
int run_fused(fb200_llama* m, int steps, bool record) {
  fb200_device* dev = m->dev;
  FB_CUDA(dev, cudaMemsetAsync(m->argmax_key, 0, 8, dev->stream));
  int rc;
  for (int done = 0; done < steps;) {
    const int n = std::min(steps - done, 256);  // bounded kernel run time
    fb200_fused_xchg xs = {};
    if (m->tp_size > 1) {
      const int per_step = 2 * m->cfg.n_layer + 1;
      if (!fb200_comm_take_exchange(m->comm, m->cfg.hidden, (unsigned)(n * per_step), &xs))
        return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama: the peer exchange is not available (detached, or closed after a time-out)");
      xs.per_step = per_step;
      xs.id_base = (unsigned)(m->tp_rank * m->vocab_local);
    }
    if ((rc = fb200_fused_launch(dev, m->prog_dev, m->prog_host.data(), (int)m->prog_host.size(), n, record,
                                 m->tp_size > 1 ? &xs : nullptr, m->fused_is_flagged)))
      return rc;
    done += n;
  }
  return FB200_OK;
}

// One forward pass over `seq` new positions per batch row; ids are already in m->ids.
// Leaves logits [batch, vocab] in m->logits and the greedy ids in m->next.
// x = (down + attn) + x, the order of attention_layer.rs:170-172 / raw/mod.rs:1036
__global__ void add_residuals_kernel(const float* __restrict__ down, const float* __restrict__ attn,
                                     float* __restrict__ x, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = (down[i] + attn[i]) + x[i];
}

// Greedy candidates of the sharded output head as sortable 64-bit keys: the f32 value mapped to
// an order-preserving unsigned integer in the high half, the global token id in the low half, so
// that the largest key is the highest value and, among equals, the higher id. A shard without a
// finite logit gives key 0.
__global__ void pack_candidates_kernel(const float* __restrict__ val, const uint32_t* __restrict__ id, int batch,
                                       uint32_t id_base, unsigned long long* __restrict__ out) {
  const int b = threadIdx.x;
  if (b >= batch) return;
  unsigned long long key = 0;
  if (id[b] != 0xFFFFFFFFu) {
    const uint32_t u = __float_as_uint(val[b]);
    const uint32_t ordered = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    key = ((unsigned long long)ordered << 32) | (id[b] + id_base);
  }
  out[b] = key;
}

__global__ void pick_candidate_kernel(const unsigned long long* __restrict__ all, int batch, int stride, int ranks,
                                      uint32_t* __restrict__ next) {
  const int b = threadIdx.x;
  if (b >= batch) return;
  unsigned long long best = 0;
  for (int r = 0; r < ranks; ++r) best = max(best, all[(size_t)r * stride + b]);
  next[b] = best ? (uint32_t)(best & 0xFFFFFFFFu) : 0xFFFFFFFFu;
}

int run_forward(fb200_llama* m, int batch, int seq) {
  m->used_key = false;
  fb200_device* dev = m->dev;
  const auto& c = m->cfg;
  const size_t rows = (size_t)batch * seq;
  const int E = c.hidden, H = c.n_head, HK = c.n_kv_head, D = c.head_dim;
  int rc;
  if ((rc = fb200_embedding_lookup(dev, m->token_embd, m->ids, rows, m->x))) return rc;
  const float scale = (float)(1.0 / sqrt((double)D));  // attention_layer.rs:674
  const int nsplit = fb200_attention_nsplit(dev, batch, HK, H / HK, seq, seq > 1 ? seq : c.max_seq_len);
  size_t part_bytes;
  fb200_attention_scratch_bytes(batch, H, seq, D, nsplit, &part_bytes);
  if (part_bytes > m->att_part_bytes)
    return fb200_fail(dev, FB200_ERR_CAPACITY, "llama: attention scratch too small");
  // 2..32 sequences, one new position each: activations are packed once per distinct input row
  // set (the fused norm writes the packed form directly) and the products take the packed rows
  bool packed = seq == 1 && rows >= 2 && rows <= 32;
  uint64_t kp_e = 0, kp_o = 0, kp_d = 0;
  for (int li = 0; li < c.n_layer && packed; ++li) {
    const LayerW& L = m->layers[li];
    packed = L.gate_up && L.wq->tiled && L.wk->tiled && L.wv->tiled && L.wo->tiled && L.gate_up->tiled && L.down->tiled;
    if (!packed) break;
    const uint64_t e = fb200_qmatrix_kp(L.wq), o = fb200_qmatrix_kp(L.wo), d = fb200_qmatrix_kp(L.down);
    packed = fb200_qmatrix_kp(L.wk) == e && fb200_qmatrix_kp(L.wv) == e && fb200_qmatrix_kp(L.gate_up) == e &&
             (li == 0 || (e == kp_e && o == kp_o && d == kp_d)) && e <= 8192;
    kp_e = e; kp_o = o; kp_d = d;
  }
  const int mp = fb200_pack16_rows((int)rows);
  const void* xh = nullptr;
  const float* xs = nullptr;
  if (packed && (rc = fb200_ensure(dev, &dev->xpack, &dev->xpack_bytes, fb200_xpack_bytes(32, std::max(std::max(kp_e, kp_o), kp_d)))))
    return rc;
  for (int li = 0; li < c.n_layer; ++li) {
    LayerW& L = m->layers[li];
    if (rows == 1) {
      // one activation row: the norm runs in the prologue of each projection kernel
      if ((rc = fb200_rms_norm_q_mat_mul(dev, m->x, nullptr, L.attn_norm, c.rms_eps, 1, L.wq, m->q, nullptr))) return rc;
      if ((rc = fb200_rms_norm_q_mat_mul(dev, m->x, nullptr, L.attn_norm, c.rms_eps, 1, L.wk, m->k, nullptr))) return rc;
      if ((rc = fb200_rms_norm_q_mat_mul(dev, m->x, nullptr, L.attn_norm, c.rms_eps, 1, L.wv, m->v, nullptr))) return rc;
    } else if (packed) {
      // 2..32 sequences: the norm writes the packed fp16 fragments the three projections share
      if ((rc = fb200_norm_pack_x16(dev, m->x, E, nullptr, L.attn_norm, c.rms_eps, (int)rows, E, kp_e, dev->xpack, &xh, &xs))) return rc;
      const fb200_qmatrix* qkv_w[3] = {L.wq, L.wk, L.wv};
      float* qkv_y[3] = {m->q, m->k, m->v};
      rc = fb200_qgemm16_packed_multi(dev, qkv_w, qkv_y, 3, xh, xs, (int)rows, mp);
      if (rc == 1) {  // not covered by the joint launch: one product after the other
        for (int i = 0; i < 3; ++i)
          if ((rc = fb200_qgemm16_packed(dev, qkv_w[i], xh, xs, (int)rows, mp, qkv_y[i], FB200_EPI_NONE, nullptr, nullptr, false)))
            return rc;
      }
      if (rc) return rc;
    } else {
      if ((rc = fb200_launch_rms_norm_strided(dev, m->x, E, nullptr, L.attn_norm, c.rms_eps, rows, E, m->xn))) return rc;
      // a prompt pass: the three projections side by side (each alone fills a fraction of the SMs)
      const fb200_qmatrix* qkv_w[3] = {L.wq, L.wk, L.wv};
      float* qkv_y[3] = {m->q, m->k, m->v};
      rc = rows > 32 ? fb200_qgemm_group(dev, qkv_w, qkv_y, 3, m->xn, rows) : 1;
      if (rc == 1) {
        if ((rc = fb200_q_mat_mul(dev, m->xn, rows, L.wq, m->q, nullptr))) return rc;
        if ((rc = fb200_q_mat_mul(dev, m->xn, rows, L.wk, m->k, nullptr))) return rc;
        if ((rc = fb200_q_mat_mul(dev, m->xn, rows, L.wv, m->v, nullptr))) return rc;
      }
      if (rc) return rc;
    }
    if (seq == 1 && H / HK <= 8) {
      // one new position per sequence: RoPE(q, k) + fp16 append + split-KV attention in one kernel
      fb200_dec_args da = {};
      da.q = m->q; da.k_new = m->k; da.v_new = m->v; da.kc = L.kc; da.vc = L.vc;
      da.rope_cos = m->rope_cos; da.rope_sin = m->rope_sin; da.pos_dev = m->pos_dev;
      da.part = m->att_part; da.out = m->att; da.done = m->att_done;
      da.b = batch; da.h = H; da.hkv = HK; da.groups = H / HK; da.cap = c.max_seq_len; da.scale = scale;
      // many sequences: the (batch, kv head) pairs alone fill the GPU, so a context is cut only
      // when it is long. The launch provides the splits of the longest context the cache can hold;
      // the kernel uses those its actual context needs.
      da.min_keys = batch * HK >= dev->sm_count / 2 ? 1024 : 64;
      int ns = 2 * dev->sm_count / (batch * HK);  // two CTAs per SM: all splits run side by side
      ns = std::max(1, std::min(std::min(ns, 32), (c.max_seq_len + da.min_keys - 1) / da.min_keys));
      da.nsplit = ns;
      if ((size_t)ns * batch * H * (D + 2) * sizeof(float) > m->att_part_bytes)
        return fb200_fail(dev, FB200_ERR_CAPACITY, "llama: attention scratch too small");
      if ((rc = fb200_launch_attention_decode_args(dev, da, D))) return rc;
    } else {
      const size_t total = rows * (size_t)(H + 2 * HK) * (D / 2);
      rope_append_kernel<<<(unsigned)((total + 255) / 256), 256, 0, dev->stream>>>(
          m->q, m->k, m->v, L.kc, L.vc, m->rope_cos, m->rope_sin, m->pos_dev, seq, H, HK, D,
          c.max_seq_len, total);
      FB_LAUNCH_CHECK(dev);
      // mask only when seq_len > 1 (raw/mod.rs:969); strictly causal over the new positions
      // keys = position + seq: known on the host (the tcgen05 kernel needs it for its tensor maps) and
      // on the device (pos_dev, for kernels inside a captured graph)
      if ((rc = fb200_launch_attention(dev, m->q, L.kc, L.vc, batch, H, HK, seq, seq > 1 ? m->pos + seq : 0, m->pos_dev,
                                       c.max_seq_len, D, scale, nullptr, seq > 1 ? 1 : 0, m->att,
                                       m->att_part, nsplit, 1))) return rc;
    }
    if (packed) {
      if ((rc = fb200_pack_x16(dev, m->att, (int)rows, L.wo->k, kp_o, dev->xpack, &xh, &xs))) return rc;
      if ((rc = fb200_qgemm16_packed(dev, L.wo, xh, xs, (int)rows, mp, m->attn_out, FB200_EPI_NONE, nullptr, nullptr, false))) return rc;
    } else if ((rc = fb200_q_mat_mul(dev, m->att, rows, L.wo, m->attn_out, nullptr))) {
      return rc;
    }
    // tensor parallel: this rank's heads gave a partial sum over K of the output projection
    if (m->tp_size > 1 && (rc = fb200_comm_all_reduce(m->comm, m->attn_out, rows * (size_t)E))) return rc;
    // ffn_norm.forward_residual_f32(attn, residual) (raw/mod.rs:1017)
    if (rows == 1 && L.gate_up) {
      fb200_epilogue ep{FB200_EPI_SWIGLU, nullptr, nullptr};
      if ((rc = fb200_rms_norm_q_mat_mul(dev, m->attn_out, m->x, L.ffn_norm, c.rms_eps, 1, L.gate_up, m->hbuf, &ep))) return rc;
    } else if (packed) {
      if ((rc = fb200_norm_pack_x16(dev, m->attn_out, E, m->x, L.ffn_norm, c.rms_eps, (int)rows, E, kp_e, dev->xpack, &xh, &xs))) return rc;
      if ((rc = fb200_qgemm16_packed(dev, L.gate_up, xh, xs, (int)rows, mp, m->hbuf, FB200_EPI_SWIGLU, nullptr, nullptr, false))) return rc;
    } else if (L.gate_up) {
      if ((rc = fb200_launch_rms_norm_strided(dev, m->attn_out, E, m->x, L.ffn_norm, c.rms_eps, rows, E, m->xn))) return rc;
      fb200_epilogue ep{FB200_EPI_SWIGLU, nullptr, nullptr};
      if ((rc = fb200_q_mat_mul(dev, m->xn, rows, L.gate_up, m->hbuf, &ep))) return rc;
    } else {
      if ((rc = fb200_launch_rms_norm_strided(dev, m->attn_out, E, m->x, L.ffn_norm, c.rms_eps, rows, E, m->xn))) return rc;
      if ((rc = fb200_q_mat_mul(dev, m->xn, rows, L.gate, m->gbuf, nullptr))) return rc;
      if ((rc = fb200_q_mat_mul(dev, m->xn, rows, L.up, m->hbuf, nullptr))) return rc;
      if ((rc = fb200_silu_mul(dev, m->gbuf, m->hbuf, rows * (size_t)c.ffn, m->hbuf))) return rc;
    }
    // (down(h) + attn) + residual, written over the residual stream
    // (attention_layer.rs:170-172 for one position, raw/mod.rs:1036 otherwise)
    if (packed && (rc = fb200_pack_x16(dev, m->hbuf, (int)rows, L.down->k, kp_d, dev->xpack, &xh, &xs))) return rc;
    if (packed && m->tp_size == 1) {
      if ((rc = fb200_qgemm16_packed(dev, L.down, xh, xs, (int)rows, mp, m->x, FB200_EPI_RESIDUAL, m->attn_out, m->x, false))) return rc;
    } else if (m->tp_size > 1) {
      // partial sum over this rank's slice of the FFN width, summed over the ranks, then the residuals
      if (packed) rc = fb200_qgemm16_packed(dev, L.down, xh, xs, (int)rows, mp, m->xn, FB200_EPI_NONE, nullptr, nullptr, false);
      else rc = fb200_q_mat_mul(dev, m->hbuf, rows, L.down, m->xn, nullptr);
      if (rc) return rc;
      if ((rc = fb200_comm_all_reduce(m->comm, m->xn, rows * (size_t)E))) return rc;
      const size_t total = rows * (size_t)E;
      add_residuals_kernel<<<(unsigned)((total + 255) / 256), 256, 0, dev->stream>>>(m->xn, m->attn_out, m->x, total);
      FB_LAUNCH_CHECK(dev);
    } else {
      fb200_epilogue ep{FB200_EPI_RESIDUAL, m->attn_out, m->x};
      if ((rc = fb200_q_mat_mul(dev, m->hbuf, rows, L.down, m->x, &ep))) return rc;
    }
  }
  // final norm on the last position of every batch row, then the output projection
  fb200_qmatrix* ow = m->output ? m->output : m->token_embd;
  if (batch == 1) {
    if ((rc = fb200_rms_norm_q_mat_mul(dev, m->x + (size_t)(seq - 1) * E, nullptr, m->output_norm,
                                       c.rms_eps, 1, ow, m->logits, nullptr))) return rc;
  } else {
    if ((rc = fb200_launch_rms_norm_strided(dev, m->x + (size_t)(seq - 1) * E, (size_t)seq * E, nullptr,
                                            m->output_norm, c.rms_eps, batch, E, m->last))) return rc;
    if ((rc = fb200_q_mat_mul(dev, m->last, batch, ow, m->logits, nullptr))) return rc;
  }
  if (m->tp_size == 1) return fb200_launch_argmax(dev, m->logits, batch, c.vocab, m->next, nullptr);
  // sharded output head: the best (value, global id) pair of every rank, gathered; every rank then
  // picks the same winner (highest value, ties -> higher id, as Tensor::top_k_pairs does)
  if ((rc = fb200_launch_argmax(dev, m->logits, batch, m->vocab_local, m->next, m->best_val))) return rc;
  unsigned long long* mine = m->best_pair;
  unsigned long long* all = m->best_pair + c.max_batch;
  const unsigned threads = batch < 64 ? 64u : (unsigned)((batch + 31) / 32) * 32u;
  pack_candidates_kernel<<<1, threads, 0, dev->stream>>>(
      m->best_val, m->next, batch, (uint32_t)(m->tp_rank * m->vocab_local), mine);
  FB_LAUNCH_CHECK(dev);
  if ((rc = fb200_comm_all_gather_bytes(m->comm, mine, all, (size_t)c.max_batch * 8))) return rc;
  pick_candidate_kernel<<<1, threads, 0, dev->stream>>>(
      all, batch, c.max_batch, m->tp_size, m->next);
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}

int launch_advance(fb200_llama* m, int batch, int advance, bool record) {
  const unsigned threads = 64 > batch ? 64 : ((batch + 31) / 32) * 32;
  unsigned long long* key = m->used_key ? m->argmax_key : nullptr;
  return fb200_launch(m->dev, advance_kernel, dim3(1), dim3(threads), 0, m->used_key, m->next, m->ids,
                      record ? m->hist : nullptr, m->pos_dev, m->step_dev, batch, m->hist_cap, advance, key);
}

// Captures embed -> layers -> logits -> argmax -> advance for one token per batch row.
int ensure_graph(fb200_llama* m, int batch) {
  fb200_device* dev = m->dev;
  // The captured kernels hold the addresses of the handle's shared scratch buffers (packed
  // activations, normalised rows). Another model or a larger product on the same handle may have
  // moved them since: the generation counter tells, and the step is captured again.
  if (m->graph_exec && m->graph_batch == batch && m->graph_gen == dev->scratch_gen) return FB200_OK;
  if (m->graph_exec) { cudaGraphExecDestroy(m->graph_exec); m->graph_exec = nullptr; }
  // make sure every lazily grown scratch buffer already has its final size
  int rc = run_forward(m, batch, 1);
  if (rc) return rc;
  FB_CUDA(dev, cudaMemsetAsync(m->argmax_key, 0, 8, dev->stream));  // the warm-up pass left its maximum there
  FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  const uint64_t launches_before = dev->launches;
  cudaGraph_t graph = nullptr;
  FB_CUDA(dev, cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal));
  dev->capturing = true;  // no event timing inside a capture
  rc = run_forward(m, batch, 1);
  if (!rc) rc = launch_advance(m, batch, 1, true);
  dev->capturing = false;
  cudaError_t e = cudaStreamEndCapture(dev->stream, &graph);
  m->graph_kernels = dev->launches - launches_before;
  dev->launches = launches_before;  // capture enqueues nothing
  if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
  if (e != cudaSuccess) return fb200_fail(dev, FB200_ERR_CUDA, "graph capture: %s", cudaGetErrorString(e));
  e = cudaGraphInstantiate(&m->graph_exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return fb200_fail(dev, FB200_ERR_CUDA, "graph instantiate: %s", cudaGetErrorString(e));
  m->graph_batch = batch;
  m->graph_gen = dev->scratch_gen;
  return FB200_OK;
}

// After a blocking call's work is enqueued: synchronise and surface a recorded time-out. Under
// tensor parallelism a time-out leaves the ranks' exchange epochs out of step, so the
// communicator is closed for further use.
int finish_blocking(fb200_llama* m) {
  const int rc = fb200_sync_check(m->dev);
  if (rc == FB200_ERR_TIMEOUT && m->comm) fb200_comm_mark_broken(m->comm);
  return rc;
}

}  // namespace

int fb200_launch_rms_norm(fb200_device* dev, const float* x, const float* res, const float* w,
                          const float* b, float eps, size_t rows, size_t n, float* y);

extern "C" {

int fb200_llama_create(fb200_device* dev, const fb200_llama_config* cfg, fb200_llama** out) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!cfg || !out) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama_create: null argument");
  *out = nullptr;
  const auto& c = *cfg;
  if (c.n_layer <= 0 || c.hidden <= 0 || c.ffn <= 0 || c.n_head <= 0 || c.n_kv_head <= 0 ||
      c.head_dim <= 0 || c.vocab <= 0 || c.max_seq_len <= 0 || c.max_batch <= 0 ||
      c.n_head % c.n_kv_head != 0 || (c.head_dim != 64 && c.head_dim != 128))
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "llama_create: unsupported configuration");
  auto m = std::unique_ptr<fb200_llama>(new fb200_llama());
  m->dev = dev;
  m->cfg = c;
  m->layers.resize(c.n_layer);
  m->vocab_local = c.vocab;
  if (const char* e = getenv("FB200_FUSED")) m->fused_enabled = !(e[0] == '0' && e[1] == 0);
  std::vector<float> cs, sn;
  fb200_rope_tables_host(c.head_dim, c.max_seq_len, c.rope_theta, c.rope_factor,
                         c.rope_low_freq_factor, c.rope_high_freq_factor, c.rope_original_ctx, nullptr, cs, sn);
  FB_CUDA(dev, cudaMalloc(&m->rope_cos, cs.size() * 4));
  FB_CUDA(dev, cudaMalloc(&m->rope_sin, sn.size() * 4));
  FB_CUDA(dev, cudaMemcpy(m->rope_cos, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice));
  FB_CUDA(dev, cudaMemcpy(m->rope_sin, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice));
  const size_t kv = (size_t)c.max_batch * c.n_kv_head * c.max_seq_len * c.head_dim * sizeof(__half);
  for (auto& L : m->layers) {
    FB_CUDA(dev, cudaMalloc(&L.kc, kv));
    FB_CUDA(dev, cudaMalloc(&L.vc, kv));
    FB_CUDA(dev, cudaMemset(L.kc, 0, kv));
    FB_CUDA(dev, cudaMemset(L.vc, 0, kv));
  }
  FB_CUDA(dev, cudaMalloc(&m->last, (size_t)c.max_batch * c.hidden * 4));
  FB_CUDA(dev, cudaMalloc(&m->logits, (size_t)c.max_batch * c.vocab * 4));
  FB_CUDA(dev, cudaMalloc(&m->next, (size_t)c.max_batch * 4));
  FB_CUDA(dev, cudaMalloc(&m->pos_dev, 4));
  FB_CUDA(dev, cudaMalloc(&m->step_dev, 4));
  m->hist_cap = c.max_seq_len;
  FB_CUDA(dev, cudaMalloc(&m->hist, (size_t)c.max_batch * m->hist_cap * 4));
  FB_CUDA(dev, cudaMemset(m->pos_dev, 0, 4));
  FB_CUDA(dev, cudaMemset(m->step_dev, 0, 4));
  FB_CUDA(dev, cudaMalloc(&m->tok_hist, (size_t)c.max_batch * (c.max_seq_len + 1) * 4));
  FB_CUDA(dev, cudaMemset(m->tok_hist, 0, (size_t)c.max_batch * (c.max_seq_len + 1) * 4));
  FB_CUDA(dev, cudaMalloc(&m->mu_dev, (size_t)c.max_batch * 4));
  FB_CUDA(dev, cudaMalloc(&m->att_done, (size_t)c.max_batch * c.n_kv_head * sizeof(int)));
  FB_CUDA(dev, cudaMemset(m->att_done, 0, (size_t)c.max_batch * c.n_kv_head * sizeof(int)));
  FB_CUDA(dev, cudaMalloc(&m->argmax_key, 8));
  FB_CUDA(dev, cudaMemset(m->argmax_key, 0, 8));
  {
    // packed rows, zero beyond the logical length up to the next multiple of 256 (and one
    // 16-row tile of slack for the producers' last tile)
    auto packed = [&](fb200_packed_act* p, size_t n) -> int {
      const size_t np = (n + 255) / 256 * 256 + 256;
      FB_CUDA(dev, cudaMalloc(&p->limbs, np * 4));
      FB_CUDA(dev, cudaMemset(p->limbs, 0, np * 4));
      float** fs[3] = {&p->xsc, &p->xss, &p->sumsq};
      for (float** f : fs) {
        FB_CUDA(dev, cudaMalloc(f, np / 16 * 4));
        FB_CUDA(dev, cudaMemset(*f, 0, np / 16 * 4));
      }
      return FB200_OK;
    };
    int prc;
    if ((prc = packed(&m->px, c.hidden)) || (prc = packed(&m->pv, c.hidden)) ||
        (prc = packed(&m->patt, (size_t)c.n_head * c.head_dim)) || (prc = packed(&m->ph, c.ffn)))
      return prc;
  }
  {
    // flagged rows: packed rows take 96 bytes per 16 elements, f32 rows 8 bytes per element
    auto padded = [](size_t n) { return (n + 255) / 256 * 256 + 256; };
    const size_t qd = (size_t)c.n_head * c.head_dim, kvd = (size_t)c.n_kv_head * c.head_dim;
    const size_t packed_n[4] = {padded(c.hidden), padded(qd), padded(c.hidden), padded(c.ffn)};
    const size_t f32_n[5] = {padded(qd), padded(kvd), padded(kvd), padded(c.hidden), padded(c.hidden)};
    size_t bytes = 0;
    for (size_t n : packed_n) bytes += n / 16 * FB200_LL_GRANULES * sizeof(uint2);
    for (size_t n : f32_n) bytes += n * sizeof(uint2);
    FB_CUDA(dev, cudaMalloc(&m->ll_slab, bytes));
    FB_CUDA(dev, cudaMemset(m->ll_slab, 0, bytes));
    uint8_t* p = m->ll_slab;
    fb200_ll_act* rows[4] = {&m->px_ll, &m->patt_ll, &m->pv_ll, &m->ph_ll};
    for (int i = 0; i < 4; ++i) { rows[i]->g = reinterpret_cast<uint2*>(p); p += packed_n[i] / 16 * FB200_LL_GRANULES * sizeof(uint2); }
    uint2** f32s[5] = {&m->q_ll, &m->k_ll, &m->v_ll, &m->x_ll, &m->attn_ll};
    for (int i = 0; i < 5; ++i) { *f32s[i] = reinterpret_cast<uint2*>(p); p += f32_n[i] * sizeof(uint2); }
    if (const char* e = getenv("FB200_FUSED_LL")) m->fused_flagged = e[0] == '1' && e[1] == 0;
  }
  // attention split scratch: the largest a forward pass can ask for is bounded by 64 splits of
  // a single-token step or one split set of a whole-context prefill
  size_t a1, a2;
  fb200_attention_scratch_bytes(c.max_batch, c.n_head, 1, c.head_dim, 64, &a1);
  fb200_attention_scratch_bytes(c.max_batch, c.n_head, c.max_seq_len, c.head_dim, 2, &a2);
  m->att_part_bytes = a1 > a2 ? a1 : a2;
  FB_CUDA(dev, cudaMalloc(&m->att_part, m->att_part_bytes));
  *out = m.release();
  return FB200_OK;
}

int fb200_llama_free(fb200_llama* m) {
  if (!m) return FB200_OK;
  fb200_device* dev = m->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  cudaStreamSynchronize(dev->stream);
  if (m->graph_exec) cudaGraphExecDestroy(m->graph_exec);
  if (m->prog_dev) cudaFree(m->prog_dev);
  for (auto& L : m->layers) {
    fb200_qmatrix* qs[] = {L.wq, L.wk, L.wv, L.wo, L.gate, L.up, L.down, L.gate_up};
    for (auto* q : qs) if (q) fb200_qmatrix_free(q);
    float* fs[] = {L.attn_norm, L.ffn_norm};
    for (auto* f : fs) if (f) cudaFree(f);
    if (L.kc) cudaFree(L.kc);
    if (L.vc) cudaFree(L.vc);
  }
  if (m->token_embd) fb200_qmatrix_free(m->token_embd);
  if (m->output) fb200_qmatrix_free(m->output);
  void* bufs[] = {m->output_norm, m->rope_cos, m->rope_sin, m->x, m->xn, m->q, m->k, m->v, m->att,
                  m->attn_out, m->hbuf, m->gbuf, m->last, m->logits, m->att_part, m->ids, m->next,
                  m->hist, m->pos_dev, m->step_dev, m->argmax_key, m->att_done, m->best_val, m->best_pair,
                  m->tok_hist, m->mu_dev, m->ll_slab};
  for (void* b : bufs) if (b) cudaFree(b);
  for (fb200_packed_act* p : {&m->px, &m->patt, &m->pv, &m->ph}) {
    void* pb[] = {p->limbs, p->xsc, p->xss, p->sumsq};
    for (void* b : pb) if (b) cudaFree(b);
  }
  delete m;
  return FB200_OK;
}

int fb200_llama_set_tensor(fb200_llama* m, int layer, int which, uint32_t ggml_type, uint64_t n,
                           uint64_t k, const void* bytes_host, size_t nbytes) {
  if (!m) return FB200_ERR_INVALID_ARGUMENT;
  fb200_device* dev = m->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  const auto& c = m->cfg;
  if (m->finalized) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama: tensors are frozen after the first forward pass");
  if (which >= FB200_T_ATTN_NORM) {
    const uint64_t len = n * (k ? k : 1);
    if (ggml_type != FB200_F32 || len != (uint64_t)c.hidden || nbytes != len * 4)
      return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "llama: norm weights are f32 vectors of length hidden");
    float** dst;
    if (which == FB200_T_OUTPUT_NORM) dst = &m->output_norm;
    else {
      if (layer < 0 || layer >= c.n_layer) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama: layer %d", layer);
      dst = which == FB200_T_ATTN_NORM ? &m->layers[layer].attn_norm : &m->layers[layer].ffn_norm;
    }
    if (!*dst) FB_CUDA(dev, cudaMalloc(dst, len * 4));
    FB_CUDA(dev, cudaMemcpy(*dst, bytes_host, len * 4, cudaMemcpyHostToDevice));
    return FB200_OK;
  }
  uint64_t en = 0, ek = 0;
  fb200_qmatrix** slot = nullptr;
  const uint64_t qd = (uint64_t)c.n_head * c.head_dim, kvd = (uint64_t)c.n_kv_head * c.head_dim;
  if (which == FB200_T_TOKEN_EMBD) { slot = &m->token_embd; en = c.vocab; ek = c.hidden; }
  else if (which == FB200_T_OUTPUT) { slot = &m->output; en = m->vocab_local; ek = c.hidden; }
  else {
    if (layer < 0 || layer >= c.n_layer) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama: layer %d", layer);
    LayerW& L = m->layers[layer];
    switch (which) {
      case FB200_T_ATTN_Q: slot = &L.wq; en = qd; ek = c.hidden; break;
      case FB200_T_ATTN_K: slot = &L.wk; en = kvd; ek = c.hidden; break;
      case FB200_T_ATTN_V: slot = &L.wv; en = kvd; ek = c.hidden; break;
      case FB200_T_ATTN_OUTPUT: slot = &L.wo; en = c.hidden; ek = qd; break;
      case FB200_T_FFN_GATE: slot = &L.gate; en = c.ffn; ek = c.hidden; break;
      case FB200_T_FFN_UP: slot = &L.up; en = c.ffn; ek = c.hidden; break;
      case FB200_T_FFN_DOWN: slot = &L.down; en = c.hidden; ek = c.ffn; break;
      default: return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama: tensor id %d", which);
    }
  }
  if (n != en || k != ek)
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "llama: tensor %d has shape [%llu, %llu], expected [%llu, %llu]",
                      which, (unsigned long long)n, (unsigned long long)k, (unsigned long long)en, (unsigned long long)ek);
  if (*slot) { fb200_qmatrix_free(*slot); *slot = nullptr; }
  const uint64_t shape[2] = {n, k};
  return fb200_qmatrix_from_raw_bytes(dev, shape, 2, bytes_host, nbytes, ggml_type, slot);
}

int fb200_llama_set_rope_freqs(fb200_llama* m, const float* weights_host, size_t n) {
  if (!m) return FB200_ERR_INVALID_ARGUMENT;
  fb200_device* dev = m->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  const auto& c = m->cfg;
  if (m->finalized) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama: the RoPE tables are frozen after the first forward pass");
  if (!weights_host || n != (size_t)c.head_dim / 2)
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "llama: rope_freqs needs head_dim / 2 = %d values, got %zu", c.head_dim / 2, n);
  std::vector<float> cs, sn;
  fb200_rope_tables_host(c.head_dim, c.max_seq_len, c.rope_theta, c.rope_factor, c.rope_low_freq_factor,
                         c.rope_high_freq_factor, c.rope_original_ctx, weights_host, cs, sn);
  FB_CUDA(dev, cudaMemcpyAsync(m->rope_cos, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, dev->stream));
  FB_CUDA(dev, cudaMemcpyAsync(m->rope_sin, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice, dev->stream));
  FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  return FB200_OK;
}

int fb200_llama_reset(fb200_llama* m) {
  if (!m) return FB200_ERR_INVALID_ARGUMENT;
  fb200_device* dev = m->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  m->pos = 0;
  FB_CUDA(dev, cudaMemsetAsync(m->pos_dev, 0, 4, dev->stream));
  FB_CUDA(dev, cudaMemsetAsync(m->step_dev, 0, 4, dev->stream));
  return FB200_OK;
}

int fb200_llama_truncate(fb200_llama* m, int len) {
  if (!m) return FB200_ERR_INVALID_ARGUMENT;
  fb200_device* dev = m->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (len < 0 || len > m->pos)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama: cannot truncate %d positions to %d", m->pos, len);
  // the caches keep their rows; positions >= len are overwritten as the sequence grows again
  m->pos = len;
  FB_CUDA(dev, cudaMemcpyAsync(m->pos_dev, &m->pos, 4, cudaMemcpyHostToDevice, dev->stream));
  FB_CUDA(dev, cudaStreamSynchronize(dev->stream));  // the copy reads a member that may change right after
  return FB200_OK;
}

int fb200_llama_position(const fb200_llama* m, int* pos_out) {
  if (!m || !pos_out) return FB200_ERR_INVALID_ARGUMENT;
  *pos_out = m->pos;
  return FB200_OK;
}

int fb200_llama_forward(fb200_llama* m, const uint32_t* tokens_host, int batch, int seq,
                        float* logits_host, uint32_t* next_host) {
  if (!m) return FB200_ERR_INVALID_ARGUMENT;
  fb200_device* dev = m->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  const auto& c = m->cfg;
  if (!tokens_host || batch <= 0 || batch > c.max_batch || seq <= 0)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama_forward: batch %d seq %d", batch, seq);
  if (m->pos + seq > c.max_seq_len)
    return fb200_fail(dev, FB200_ERR_CAPACITY, "llama_forward: position %d + %d exceeds max_seq_len %d", m->pos, seq, c.max_seq_len);
  if ((rc = finalize(m))) return rc;
  const size_t rows = (size_t)batch * seq;
  if ((rc = ensure_rows(m, rows))) return rc;
  FB_CUDA(dev, cudaMemcpy2DAsync(m->tok_hist + m->pos, (size_t)(c.max_seq_len + 1) * 4, tokens_host, (size_t)seq * 4,
                                 (size_t)seq * 4, batch, cudaMemcpyHostToDevice, dev->stream));
  if (seq == 1 && batch == 1 && (rc = build_fused_program(m))) return rc;
  if (seq == 1 && batch == 1 && m->fused_usable) {
    FB_CUDA(dev, cudaMemcpyAsync(m->ids, tokens_host, 4, cudaMemcpyHostToDevice, dev->stream));
    if ((rc = run_fused(m, 1, false))) return rc;
  } else if (seq == 1) {
    // single-token step: replay the captured graph (capture leaves the position untouched)
    if (!m->graph_exec || m->graph_batch != batch || m->graph_gen != dev->scratch_gen) {
      FB_CUDA(dev, cudaMemcpyAsync(m->ids, tokens_host, rows * 4, cudaMemcpyHostToDevice, dev->stream));
      if ((rc = ensure_graph(m, batch))) return rc;
    }
    FB_CUDA(dev, cudaMemcpyAsync(m->ids, tokens_host, rows * 4, cudaMemcpyHostToDevice, dev->stream));
    FB_CUDA(dev, cudaGraphLaunch(m->graph_exec, dev->stream));
    dev->launches += m->graph_kernels;
  } else {
    FB_CUDA(dev, cudaMemcpyAsync(m->ids, tokens_host, rows * 4, cudaMemcpyHostToDevice, dev->stream));
    if ((rc = run_forward(m, batch, seq))) return rc;
    if ((rc = launch_advance(m, batch, seq, false))) return rc;
  }
  m->pos += seq;
  if (logits_host)
    FB_CUDA(dev, cudaMemcpyAsync(logits_host, m->logits, (size_t)batch * m->vocab_local * 4, cudaMemcpyDeviceToHost, dev->stream));
  if (next_host)
    FB_CUDA(dev, cudaMemcpyAsync(next_host, m->next, (size_t)batch * 4, cudaMemcpyDeviceToHost, dev->stream));
  return finish_blocking(m);
}

int fb200_llama_generate_greedy(fb200_llama* m, const uint32_t* tokens_host, int batch, int steps,
                                uint32_t* out_host) {
  if (!m) return FB200_ERR_INVALID_ARGUMENT;
  fb200_device* dev = m->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  const auto& c = m->cfg;
  if (!tokens_host || !out_host || batch <= 0 || batch > c.max_batch || steps <= 0)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "generate_greedy: batch %d steps %d", batch, steps);
  if (m->pos + steps > c.max_seq_len)
    return fb200_fail(dev, FB200_ERR_CAPACITY, "generate_greedy: position %d + %d exceeds max_seq_len %d", m->pos, steps, c.max_seq_len);
  if ((rc = finalize(m))) return rc;
  if ((rc = ensure_rows(m, batch))) return rc;
  if (m->hist_cap < steps || !m->hist) {
    FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
    if (m->hist) cudaFree(m->hist);
    m->hist = nullptr;
    FB_CUDA(dev, cudaMalloc(&m->hist, (size_t)c.max_batch * steps * 4));
    m->hist_cap = steps;
    if (m->graph_exec) { cudaGraphExecDestroy(m->graph_exec); m->graph_exec = nullptr; }
  }
  if (batch == 1) {
    m->fused_valid = m->fused_valid && !m->prog_host.empty() && m->prog_host.back().hist == m->hist &&
                     m->prog_host.back().hist_cap == m->hist_cap;
    if ((rc = build_fused_program(m))) return rc;
  }
  if (batch == 1 && m->fused_usable) {
    FB_CUDA(dev, cudaMemcpyAsync(m->ids, tokens_host, 4, cudaMemcpyHostToDevice, dev->stream));
    FB_CUDA(dev, cudaMemsetAsync(m->step_dev, 0, 4, dev->stream));
    if ((rc = run_fused(m, steps, true))) return rc;
  } else {
    FB_CUDA(dev, cudaMemcpyAsync(m->ids, tokens_host, (size_t)batch * 4, cudaMemcpyHostToDevice, dev->stream));
    if ((rc = ensure_graph(m, batch))) return rc;
    FB_CUDA(dev, cudaMemcpyAsync(m->ids, tokens_host, (size_t)batch * 4, cudaMemcpyHostToDevice, dev->stream));
    FB_CUDA(dev, cudaMemsetAsync(m->step_dev, 0, 4, dev->stream));
    for (int s = 0; s < steps; ++s) {
      FB_CUDA(dev, cudaGraphLaunch(m->graph_exec, dev->stream));
      dev->launches += m->graph_kernels;
    }
  }
  // the session's token history: the fed tokens at the old position, the generated ones after it
  FB_CUDA(dev, cudaMemcpy2DAsync(m->tok_hist + m->pos, (size_t)(c.max_seq_len + 1) * 4, tokens_host, 4, 4, batch,
                                 cudaMemcpyHostToDevice, dev->stream));
  FB_CUDA(dev, cudaMemcpy2DAsync(m->tok_hist + m->pos + 1, (size_t)(c.max_seq_len + 1) * 4, m->hist,
                                 (size_t)m->hist_cap * 4, (size_t)steps * 4, batch, cudaMemcpyDeviceToDevice, dev->stream));
  m->pos += steps;
  // hist is [batch, hist_cap]; gather the first `steps` columns
  std::vector<uint32_t> tmp((size_t)batch * m->hist_cap);
  FB_CUDA(dev, cudaMemcpyAsync(tmp.data(), m->hist, tmp.size() * 4, cudaMemcpyDeviceToHost, dev->stream));
  if ((rc = finish_blocking(m))) return rc;
  for (int b = 0; b < batch; ++b)
    std::memcpy(out_host + (size_t)b * steps, tmp.data() + (size_t)b * m->hist_cap, (size_t)steps * 4);
  return FB200_OK;
}

namespace {
__global__ void fill_f32_kernel(float* p, float v, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}
}  // namespace

int fb200_llama_generate_sampled(fb200_llama* m, const uint32_t* tokens_host, int batch, int steps,
                                 const fb200_sampler_config* cfg, uint32_t* out_host) {
  if (!m) return FB200_ERR_INVALID_ARGUMENT;
  fb200_device* dev = m->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  const auto& c = m->cfg;
  if (!tokens_host || !out_host || !cfg || batch <= 0 || batch > c.max_batch || steps <= 0)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "generate_sampled: batch %d steps %d", batch, steps);
  if (m->tp_size > 1)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "generate_sampled: a tensor-parallel model holds only a shard of the logits");
  if (m->pos + steps > c.max_seq_len)
    return fb200_fail(dev, FB200_ERR_CAPACITY, "generate_sampled: position %d + %d exceeds max_seq_len %d", m->pos, steps, c.max_seq_len);
  if ((rc = finalize(m))) return rc;
  if ((rc = ensure_rows(m, batch))) return rc;
  if (batch == 1 && (rc = build_fused_program(m))) return rc;
  const size_t hstride = (size_t)c.max_seq_len + 1;
  FB_CUDA(dev, cudaMemcpyAsync(m->ids, tokens_host, (size_t)batch * 4, cudaMemcpyHostToDevice, dev->stream));
  if (!(batch == 1 && m->fused_usable)) {
    if ((rc = ensure_graph(m, batch))) return rc;  // may run a warm-up pass over the ids
    FB_CUDA(dev, cudaMemcpyAsync(m->ids, tokens_host, (size_t)batch * 4, cudaMemcpyHostToDevice, dev->stream));
  }
  FB_CUDA(dev, cudaMemcpy2DAsync(m->tok_hist + m->pos, hstride * 4, tokens_host, 4, 4, batch, cudaMemcpyHostToDevice,
                                 dev->stream));
  if (cfg->strategy == FB200_SAMPLER_MIROSTAT2) {
    fill_f32_kernel<<<1, 256, 0, dev->stream>>>(m->mu_dev, cfg->mu, batch < 256 ? batch : 256);
    FB_LAUNCH_CHECK(dev);
    if (batch > 256) return fb200_fail(dev, FB200_ERR_CAPACITY, "generate_sampled: at most 256 sequences");
  }
  const int pos0 = m->pos;
  for (int s = 0; s < steps; ++s) {
    // one new position per sequence (leaves the logits in m->logits and advances the position) ...
    if (batch == 1 && m->fused_usable) {
      if ((rc = run_fused(m, 1, false))) return rc;
    } else {
      FB_CUDA(dev, cudaGraphLaunch(m->graph_exec, dev->stream));
      dev->launches += m->graph_kernels;
    }
    // ... then the sampler: its id replaces the greedy one as the next step's input and joins the history
    const int seen = pos0 + s + 1;  // tokens of the session so far, the one just consumed included
    if ((rc = fb200_launch_sampler(dev, m->logits, (size_t)batch, (size_t)c.vocab, cfg, m->tok_hist, hstride, seen,
                                   (unsigned long long)seen, m->mu_dev, m->next, m->ids, 1, m->tok_hist + seen, hstride)))
      return rc;
  }
  m->pos += steps;
  std::vector<uint32_t> tmp((size_t)batch * steps);
  FB_CUDA(dev, cudaMemcpy2DAsync(tmp.data(), (size_t)steps * 4, m->tok_hist + pos0 + 1, hstride * 4, (size_t)steps * 4,
                                 batch, cudaMemcpyDeviceToHost, dev->stream));
  if ((rc = finish_blocking(m))) return rc;
  std::memcpy(out_host, tmp.data(), tmp.size() * 4);
  return FB200_OK;
}

int fb200_llama_set_tensor_parallel(fb200_llama* m, fb200_comm* comm) {
  if (!m || !comm) return FB200_ERR_INVALID_ARGUMENT;
  fb200_device* dev = m->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (fb200_comm_device(comm) != dev)
    return fb200_fail(dev, FB200_ERR_DEVICE_MISMATCH, "llama: the communicator lives on another device handle");
  if (m->finalized || m->token_embd || m->output)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "llama: attach the communicator before any tensor is set");
  const int size = fb200_comm_size(comm);
  if (m->cfg.vocab % size)
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "llama: vocab %d is not divisible by %d ranks", m->cfg.vocab, size);
  m->comm = comm;
  m->tp_size = size;
  m->tp_rank = fb200_comm_rank(comm);
  m->vocab_local = m->cfg.vocab / size;
  if (size > 1) {
    FB_CUDA(dev, cudaMalloc(&m->best_val, (size_t)m->cfg.max_batch * 4));
    FB_CUDA(dev, cudaMalloc(&m->best_pair, (size_t)(1 + size) * m->cfg.max_batch * 8));
  }
  return FB200_OK;
}

int fb200_llama_logits_dev(const fb200_llama* m, const float** logits_dev) {
  if (!m || !logits_dev) return FB200_ERR_INVALID_ARGUMENT;
  *logits_dev = m->logits;
  return FB200_OK;
}

}  // extern "C"
