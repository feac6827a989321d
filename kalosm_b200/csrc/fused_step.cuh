// Program of the fused decode-step kernel: a list of phases that one persistent cooperative
// kernel (one CTA per SM) executes in order, with a grid-wide barrier between phases. The
// weight stream never leaves the TMA-fed shared-memory rings: at the end of a product phase
// every warp already fetches its first tile-groups of the next product phase, so HBM stays busy
// across the barrier, the attention phase and the activation reload.
#pragma once

#include "attn_decode.cuh"
#include "common.cuh"
#include "packed_act.cuh"

enum fb200_fused_kind {
  FB200_PH_GEMV = 0,     // single-row quantised product(s), stream-K over tile-groups
  FB200_PH_ATTN = 1,     // RoPE + KV append + split-KV attention for the new position
  FB200_PH_PACK = 2,     // float row (+ row) -> packed row (optionally times a norm weight)
  FB200_PH_EMBED = 3,    // embedding row of ids[0] -> float row + packed row
  FB200_PH_ADVANCE = 4,  // greedy id from the argmax key -> ids, history; position + 1
  FB200_PH_XSUM = 5,     // tensor parallel: signal the peers, wait for theirs, sum the ranks' partial rows in
                         // rank order (+ residual rows) -> float row(s) + packed row
};

// Tensor-parallel exchange over peer memory (NVLink): every rank owns one buffer
//   [2 parities][world][stride floats] partial rows | [2][world] greedy keys | [world] arrival epochs
// that all its peers have mapped. A product phase with xs_index >= 0 writes its output rows into
// slot [epoch & 1][this rank] of EVERY rank's buffer; the FB200_PH_XSUM phase after the grid barrier
// publishes "epoch" in every peer's arrival word for this rank (release at system scope), waits
// (bounded) for the peers' words to reach the epoch and sums the slots. epoch = epoch_base +
// step * per_step + xs_index is the same number on all ranks; a rank can run at most one
// exchange ahead of a peer, so two parities are enough.
struct fb200_fused_xchg {
  float* data[8];
  unsigned long long* keys[8];
  unsigned* flags[8];
  int world, me, stride;
  unsigned epoch_base;
  int per_step;
  unsigned id_base;  // first global token id of this rank's rows of the output head
  int poll_limit;    // polls of one arrival word before the wait gives up
};

constexpr int FB200_XCHG_POLL_LIMIT = 1 << 22;

#ifdef __CUDACC__
// Bounded wait for an arrival word (written by a peer with release at system scope) to reach
// `epoch`. Gives up after `poll_limit` polls, or at once when another wait has already set the
// status word; returns false then (the caller records FB200_ERR_TIMEOUT and carries on).
__device__ __forceinline__ bool fb200_wait_arrival(const unsigned* word, unsigned epoch, int poll_limit, const int* status) {
  for (int it = 0; it < poll_limit; ++it) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
    if ((int)(v - epoch) >= 0) return true;
    if ((it & 1023) == 1023 && __ldcg(status) != 0) return false;
    __nanosleep(64);
  }
  return false;
}
#endif

struct fb200_fused_seg {
  const uint8_t* w;  // tiled weight bytes
  float* y;          // optional float output row
  uint2* yl;         // optional output row as f32 granules {value, epoch} (flagged rows)
  int type;          // ggml type id
  int tg;            // bytes per tile-group
  int units;         // tiles (tile pairs for SwiGLU) of this matrix
  int n_out;         // logical outputs
};

struct alignas(16) fb200_fused_phase {  // 16-byte multiples: descriptors are copied with 16-byte asynchronous copies
  int kind;
  int next_gemv;  // index of the next product phase in execution order (may wrap to the next step), -1: none
  // ---- FB200_PH_GEMV: up to three matrices that share the activation row
  fb200_fused_seg seg[3];
  int nseg;
  int epi;          // FB200_EPI_*
  int K, Kp;        // logical and padded inner size
  int ngroups;      // K groups per tile
  int nunits;       // tiles (tile pairs) over all matrices
  int ipu;          // items (tile-groups) per unit = passes * ngroups
  int total;        // nunits * ipu
  int chunk;        // items per CTA
  int pair_off;     // SwiGLU: tile distance between a gate tile and its up tile
  int stride;       // ring slot bytes (largest tile-group of the phase, rounded up to 128)
  int stages;       // ring slots per warp in this phase
  float rcp_ipu, rcp_ng;  // 1 / ipu, 1 / ngroups (the kernel divides item indices by multiplication)
  fb200_packed_act xp;  // activation row
  int xp_norm;          // divide by its RMS (norm weights were applied by the producer)
  float eps;
  const float* r1;      // residual epilogue
  const float* r2;
  fb200_packed_act yp;  // optional packed output (also the output of PACK / EMBED)
  const float* yp_norm_w;
  const float* yp_add;
  unsigned long long* argmax_key;
  // ---- FB200_PH_ATTN
  fb200_dec_args att;
  int att_d;
  // ---- FB200_PH_PACK / FB200_PH_EMBED
  const float* src;
  const float* src_add;
  float* xout;         // optional float copy of the row
  const uint8_t* emb;  // embedding matrix bytes
  int emb_type, emb_tiled, emb_ngroups, emb_ge, emb_tgb;
  unsigned long long emb_n;
  const uint32_t* ids;
  // ---- FB200_PH_ADVANCE
  uint32_t* next;
  uint32_t* ids_w;
  uint32_t* hist;
  int* pos_dev;
  int* step_dev;
  int hist_cap;
  // ---- flagged rows (single-GPU kernel variants without grid barriers between phases): the same
  // operands as above, published by their producers as {data, epoch} granules (packed_act.cuh)
  // that the consumer polls. *_back = how many phases before this one the producer ran.
  fb200_ll_act xll;   // activation row (producer: the phase before)
  fb200_ll_act yll;   // packed output (also of EMBED)
  const uint2* r1l;   // residual epilogue operands as f32 granules
  const uint2* r2l;
  const uint2* addl;  // yp_add
  int r1_back, r2_back, add_back;
  uint2* xoutl;       // EMBED: the float row as granules
  // ---- tensor parallel: index of this phase's exchange within a step (-1: none). On a product
  // phase: rows go to the peers instead of seg[0].y; on FB200_PH_XSUM: out_sum = sum over ranks,
  // v = sum + src + src_add -> xout, packed into yp (times yp_norm_w); on FB200_PH_ADVANCE: the
  // greedy key is exchanged and the largest wins.
  int xs_index;
  float* out_sum;
  // ---- L2 plan of a product phase (fb200_fused_plan_prefetch): a warp that has consumed its share of
  // this phase asks L2 for its share of the product phases pf_off[j] phases further on (0: none),
  // from item pf_skip[j] of that share (the items before go to the ring) and at most pf_cap[j] items.
  int pf_off[2], pf_skip[2], pf_cap[2];
};

// Fills the derived fields of a product phase (units, items, chunk, ring geometry) from its
// matrices; `grid` = CTAs of the launch. Returns false if the matrices cannot share a phase.
bool fb200_fused_gemv_phase(fb200_fused_phase* p, const fb200_qmatrix* const* ws, float* const* ys, int nw,
                            int epi, int grid, bool flagged);
// Fills the L2 plan of every product phase of a complete program (next_gemv already chained):
// which later phases' weights a warp requests into L2 when its share of a phase ends, so that HBM
// keeps streaming through barriers, attention phases and activation reloads. `ahead_bytes` bounds
// the weight bytes requested but not yet consumed (they must fit in L2 beside everything else).
void fb200_fused_plan_prefetch(fb200_fused_phase* prog, int nphases, int grid, size_t ahead_bytes);
// Shared memory the program needs; 0 if it does not fit.
size_t fb200_fused_smem_bytes(const fb200_fused_phase* prog_host, int nphases, bool flagged = false);
// Number of CTAs of a launch on this device.
int fb200_fused_grid(const fb200_device* dev);
// Runs `nsteps` passes over the program (device copy `prog_dev` of `prog_host`).
// `flagged`: the program carries flagged rows; the launch takes the barrier-free kernel variant.
int fb200_fused_launch(fb200_device* dev, const fb200_fused_phase* prog_dev, const fb200_fused_phase* prog_host,
                       int nphases, int nsteps, bool record_history, const fb200_fused_xchg* xchg, bool flagged);
// True when a program of these matrix types and attention shape has a barrier-free variant.
bool fb200_fused_flagged_available(const fb200_fused_phase* prog_host, int nphases);
