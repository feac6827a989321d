// Fused decode step: one persistent cooperative kernel, one CTA per SM, runs a whole single-token
// forward pass (or several in a row) as a program of phases separated by grid-wide barriers.
//
// Replaces, for one new position of one sequence, the reference's per-operation graph execution
// (fusor-ml/core/src/compute_graph/resolve/run.rs:29-135) of the Llama decoder
// (models/kalosm-llama/src/raw/mod.rs:925-1049): embedding, per layer q/k/v projections,
// RoPE + KV append + attention, output projection, SwiGLU FFN with both residual adds, final
// norm + output head + greedy argmax.
//
// Product phases stream the quantised weights exactly once from HBM:
//  * stream-K: the tile-groups (16 rows x one K group) of all matrices of a phase form one
//    list; every CTA takes an equal contiguous share and every warp an equal contiguous share
//    of that, whatever the matrix shapes. A unit (16 output rows, or a gate/up pair of tiles)
//    that straddles warps is summed through shared memory in warp order; one that straddles
//    CTAs is summed in CTA order by the CTA that arrives last (arrival counter per unit), so
//    results do not depend on timing;
//  * each warp owns a ring of shared-memory slots filled by 1-D TMA bulk copies and mbarriers;
//    when a warp has consumed its share it immediately fetches the first slots of its share of
//    the NEXT product phase, so the weight stream continues across the grid barrier;
//  * activations arrive packed (int8 limbs, per-16 scales and sums) and are copied to shared
//    memory once per CTA; the per-tile-group math is that of the single-row kernel.
// Tensor parallel (variants with XS = true): the ranks' kernels run side by side, one per GPU;
// the o and down projections store their partial rows into every rank's exchange buffer (peer
// memory over NVLink), arrival words written with release at system scope tell the peers, and
// an XSUM phase adds the ranks' rows in rank order; the greedy key of the sharded output head
// is exchanged the same way (fused_step.cuh: fb200_fused_xchg).
// Single-GPU programs of K-quant weights run the variants with LL = true: no grid barrier inside a
// step. Every activation that crosses CTAs (packed rows, q / k / v, the residual stream, the
// attention output) travels as flagged rows (packed_act.cuh: payload word + epoch in one 8-byte
// store, polled by the reader), so a phase boundary costs one store and one load through L2
// instead of fence -> barrier -> reload, and CTAs without work in a phase run ahead to the next.
// Only the greedy-token hand-over at the end of a step (argmax key -> ids) keeps two barriers.
// Everything another CTA wrote during the kernel is read through L2 (ld.global.cg).
// All waits are bounded: a wait that gives up sets the device status word and the kernel runs to
// its end without waiting again.
#include <algorithm>
#include <cstdlib>
#include <vector>

#include "fused_step.cuh"
#include "qgemv1_groups2.cuh"

namespace {

constexpr int FW = 16;             // warps per CTA
constexpr int FT = FW * 32;        // threads per CTA
constexpr int RING_BYTES = 6912;   // ring bytes per warp: 3 x 2304 (Q4_K) or 2 x 3456 (Q6_K)
constexpr int MAX_STAGES = 2;  // ring slots per warp: a third slot measured slower, not faster
// Ring of the barrier-free variants: the same bytes per warp, Q4_K phases may use a third slot. A larger
// ring was measured and is far slower: shared memory beyond ~185 KB leaves the L1 too small for the
// kernel's register spills (local memory), and those then travel to L2.
constexpr int RING_BYTES_LL = 6912;
constexpr int MAX_STAGES_LL = 3;
constexpr int FUSED_DEC_CH = 64;
constexpr int FUSED_SPLIT_KEYS = 32;  // smallest share of the context an attention item takes   // keys per shared-memory chunk of the attention phase
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int STATIC_SMEM_RESERVE = 4096;  // static shared memory of the attention phase
constexpr int DESC_WORDS = (int)((sizeof(fb200_fused_phase) + 15) / 16 * 4);  // 32-bit words per descriptor slot
constexpr int DESC_SLOTS = 5;

struct FusedArgs {
  const fb200_fused_phase* prog;
  int nphases, nsteps, record, first_gemv;
  int xregion;     // bytes of the activation region (limbs, scales, sums; aliased by attention)
  unsigned* bar;   // grid barrier arrival counter, zero at launch
  float* gp;       // [grid][2][32] partial sums of units split across CTAs
  int* counters;   // arrival counters per unit, zero between uses
  int* status;
  unsigned long long* trace;  // optional [nphases][8] time stamps of CTA 0 in the last step (ns)
  fb200_fused_xchg x;         // tensor-parallel exchange (world <= 1: none)
  unsigned epoch_base;        // flagged rows: epoch of phase 0 of this launch
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Grid-wide barrier: every CTA adds one to a counter that only grows; generation n is complete
// when the counter reaches n * gridDim.x. Bounded: after ~2^24 polls (seconds) or as soon as
// another wait has given up, the CTA records the timeout and carries on.
__device__ __forceinline__ void grid_barrier(const FusedArgs& A, unsigned& target, unsigned long long* arrive_max) {
  __syncthreads();
  target += gridDim.x;
  if (threadIdx.x == 0) {
    if (arrive_max) atomicMax(arrive_max, global_ns());
    // arrival = one fire-and-forget reduction with release semantics (orders this CTA's writes,
    // made visible to thread 0 by the barrier above, before the count)
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(A.bar) : "memory");
    // polls are relaxed loads (no ordering work per poll); one acquire fence after the last one
    // orders everything this CTA reads next behind the arrivals it has seen
    unsigned polls = 0;
    while ((int)(ld_relaxed_u32(A.bar) - target) < 0) {
      ++polls;
      if ((polls & 1023u) == 0u && __ldcg(A.status) != 0) break;
      if (polls > (1u << 24)) { atomicExch(A.status, FB200_ERR_TIMEOUT); break; }
    }
    asm volatile("fence.acq_rel.gpu;" ::: "memory");
  }
  __syncthreads();
}

// floor(i / d) for 0 <= i < 2^21 with rcp = 1 / d rounded to float: (i + 0.5) / d is at least
// 0.5 / d away from every integer, far more than the rounding errors of the product.
__device__ __forceinline__ int fdiv(int i, float rcp) { return __float2int_rz(((float)i + 0.5f) * rcp); }

// The fields of a product phase the inner loops use, read once into registers.
struct PhaseLocal {
  int ng, npass, ipu, stride, stages, total, chunk, pair_off;
  float rcp_ipu, rcp_ng;
};
__device__ __forceinline__ PhaseLocal phase_local(const fb200_fused_phase& P) {
  PhaseLocal q;
  q.ng = P.ngroups; q.npass = P.epi == FB200_EPI_SWIGLU ? 2 : 1; q.ipu = P.ipu; q.stride = P.stride;
  q.stages = P.stages; q.total = P.total; q.chunk = P.chunk; q.pair_off = P.pair_off;
  q.rcp_ipu = P.rcp_ipu; q.rcp_ng = P.rcp_ng;
  return q;
}

// A CTA's and a warp's share of the items of a product phase.
struct Range {
  int c0, c1;  // CTA
  int per;     // items per warp (last warps may have fewer or none)
  int w0, w1;  // warp
};
__device__ __forceinline__ Range warp_range(int total, int chunk, int warp) {
  Range r;
  r.c0 = min((int)blockIdx.x * chunk, total);
  r.c1 = min(r.c0 + chunk, total);
  const int n = r.c1 - r.c0;
  r.per = n > 0 ? (n + FW - 1) / FW : 1;
  r.w0 = min(r.c0 + warp * r.per, r.c1);
  r.w1 = min(r.w0 + r.per, r.c1);
  return r;
}

// Position in the item list: item i = (unit u, pass p, K group kg), plus where its bytes are.
struct Cursor {
  int i, u, p, kg;
  int type, tgb;
  const uint8_t* src;
};
__device__ __forceinline__ void unit_locate(const fb200_fused_phase& P, int u, int& sidx, int& tile) {
  sidx = 0; tile = u;
  if (P.nseg > 1 && tile >= P.seg[0].units) { tile -= P.seg[0].units; sidx = 1; }
  if (P.nseg > 2 && sidx == 1 && tile >= P.seg[1].units) { tile -= P.seg[1].units; sidx = 2; }
}
__device__ __forceinline__ void cur_locate(const fb200_fused_phase& P, const PhaseLocal& q, Cursor& c) {
  int sidx, tile;
  unit_locate(P, c.u, sidx, tile);
  c.type = P.seg[sidx].type;
  c.tgb = P.seg[sidx].tg;
  c.src = P.seg[sidx].w + ((size_t)(tile + c.p * q.pair_off) * q.ng + c.kg) * (size_t)c.tgb;
}
__device__ __forceinline__ void cur_init(const fb200_fused_phase& P, const PhaseLocal& q, Cursor& c, int i) {
  c.i = i;
  c.u = fdiv(i, q.rcp_ipu);
  const int rem = i - c.u * q.ipu;
  c.p = fdiv(rem, q.rcp_ng);
  c.kg = rem - c.p * q.ng;
  cur_locate(P, q, c);
}
__device__ __forceinline__ void cur_next(const fb200_fused_phase& P, const PhaseLocal& q, Cursor& c) {
  ++c.i;
  c.src += c.tgb;
  if (++c.kg == q.ng) {
    c.kg = 0;
    if (++c.p == q.npass) { c.p = 0; ++c.u; }
    if (c.i < q.total) cur_locate(P, q, c);
  }
}

struct WarpRing {
  uint32_t base;   // shared address of this warp's ring
  uint32_t bar0;   // shared address of its first mbarrier
  uint32_t par;    // bit s = parity of the next completion of slot s
  uint8_t* ptr;    // generic pointer to the ring
  uint64_t policy; // L2 policy of the weight stream (evict first)
};

__device__ __forceinline__ void ring_issue(const WarpRing& R, int slot, int stride, const Cursor& c) {
  mbar_expect_tx(R.bar0 + 8 * slot, (uint32_t)c.tgb);
  bulk_g2s_stream(R.base + slot * stride, c.src, (uint32_t)c.tgb, R.bar0 + 8 * slot, R.policy);
}

// What a warp carries from the prefetch of a product phase into that phase. Invariant: when the
// phase starts, exactly the items cc.i .. cc.i + n - 1 are in flight in slots 0 .. n-1 and
// n = min(stages, items of the warp) (or n = 0 and nothing is in flight); the consumer refills
// the slot it has just read, so slots are always used round-robin.
struct Carry {
  Cursor cc;  // first item of the warp's share
  Cursor ic;  // next item to fetch
  int n;      // items already in flight, in slots 0 .. n-1 (0: nothing was prefetched)
};

// First slots of this warp's share of product phase P (weights only, nothing to wait for).
__device__ __forceinline__ void prefetch_phase(const fb200_fused_phase& P, const WarpRing& R, int warp, int lane,
                                               Carry& C) {
  const PhaseLocal q = phase_local(P);
  const Range r = warp_range(q.total, q.chunk, warp);
  C.n = 0;
  if (r.w0 >= r.w1) return;
  cur_init(P, q, C.cc, r.w0);
  C.ic = C.cc;
  const int n = min(q.stages, r.w1 - r.w0);
  for (int j = 0; j < n; ++j) {
    if (lane == 0) ring_issue(R, j, q.stride, C.ic);
    cur_next(P, q, C.ic);
  }
  C.n = n;
}

// Asks L2 for `bytes` (a multiple of 16) at p: no shared memory, no barrier, nothing to wait for.
__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// This warp's share of product phase P from item `skip` on, at most `cap` items, into L2: one
// request per run of consecutive tile-groups (the K groups of one tile are contiguous).
__device__ __noinline__ void l2_prefetch_share(const fb200_fused_phase& P, int warp, int lane, int skip, int cap) {
  const PhaseLocal q = phase_local(P);
  const Range r = warp_range(q.total, q.chunk, warp);
  int i = min(r.w0 + skip, r.w1);
  const int end = min(r.w1, i + cap);
  while (i < end) {
    Cursor c;
    cur_init(P, q, c, i);
    const int run = min(end - i, q.ng - c.kg);
    if (lane == 0) l2_prefetch(c.src, (uint32_t)(run * c.tgb));
    i += run;
  }
}

struct EpiCtx {
  float final_scale;
  unsigned long long best_key;
  const fb200_fused_xchg* xs;  // not null: rows of matrix 0 go to every rank's exchange buffer
  int xs_off;                  // float offset of this rank's slot for the current epoch
  unsigned ep;                 // flagged rows: epoch of the current phase
};

__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Tells every peer that this rank's contribution to exchange `epoch` is complete in its buffer
// (called by one thread after the grid barrier that followed the writes), then waits until every
// peer has said the same here. Bounded (fb200_wait_arrival): after poll_limit polls, or when
// another wait has already given up, the time-out is recorded and the kernel carries on with
// whatever is there.
__device__ __forceinline__ void xchg_signal_and_wait(const FusedArgs& A, unsigned epoch, bool signal) {
  const fb200_fused_xchg& X = A.x;
  if (signal) {
    __threadfence_system();
    for (int r = 0; r < X.world; ++r)
      if (r != X.me) st_release_sys_u32(X.flags[r] + X.me, epoch);
  }
  for (int r = 0; r < X.world; ++r) {
    if (r == X.me) continue;
    if (!fb200_wait_arrival(X.flags[X.me] + r, epoch, X.poll_limit, A.status)) {
      atomicExch(A.status, FB200_ERR_TIMEOUT);
      break;
    }
  }
}

// The operands of a unit's epilogue (row `lane` of the unit): residuals, the row added before
// packing, the norm weight folded into the packed row. Everything was produced before the phase
// began, so a warp may fetch them long before it needs them.
struct EpiOperands {
  int unit;  // -1: nothing fetched
  float res1, res2, padd, pw;
  // flagged rows: bit i set = operand i (res1, res2, padd) was read before its producer had
  // published it; it is polled where the value is used, so that fetching ahead never waits
  unsigned stale;
};
template <bool LL>
__device__ __forceinline__ EpiOperands epilogue_operands(const fb200_fused_phase& P, int unit, int lane, const EpiCtx& E) {
  int sidx, tile;
  unit_locate(P, unit, sidx, tile);
  const int n = tile * 16 + lane;
  const bool valid = n < P.seg[sidx].n_out;
  EpiOperands o;
  o.unit = unit;
  if constexpr (LL) {
    const bool pack = P.yll.g && sidx == 0;
    o.res1 = o.res2 = o.padd = 0.f;
    o.stale = 0u;
    if (valid && P.epi == FB200_EPI_RESIDUAL) {
      const uint2 g = ld_ll_granule(P.r1l + n);
      o.res1 = __uint_as_float(g.x);
      if (g.y != E.ep - (unsigned)P.r1_back) o.stale |= 1u;
    }
    if (valid && P.epi == FB200_EPI_RESIDUAL && P.r2l) {
      const uint2 g = ld_ll_granule(P.r2l + n);
      o.res2 = __uint_as_float(g.x);
      if (g.y != E.ep - (unsigned)P.r2_back) o.stale |= 2u;
    }
    if (valid && pack && P.addl) {
      const uint2 g = ld_ll_granule(P.addl + n);
      o.padd = __uint_as_float(g.x);
      if (g.y != E.ep - (unsigned)P.add_back) o.stale |= 4u;
    }
    o.pw = valid && pack && P.yp_norm_w ? P.yp_norm_w[n] : 1.0f;
  } else {
    const bool pack = P.yp.limbs && sidx == 0;
    o.stale = 0u;
    o.res1 = valid && P.epi == FB200_EPI_RESIDUAL ? __ldcg(P.r1 + n) : 0.f;
    o.res2 = valid && P.epi == FB200_EPI_RESIDUAL && P.r2 ? __ldcg(P.r2 + n) : 0.f;
    o.padd = valid && pack && P.yp_add ? __ldcg(P.yp_add + n) : 0.f;
    o.pw = valid && pack && P.yp_norm_w ? P.yp_norm_w[n] : 1.0f;
  }
  return o;
}

// Epilogue of one unit; lanes 0..15 call it with the sums of row `lane` (pass 0 / pass 1).
template <bool XS, bool LL>
__device__ __noinline__ void unit_epilogue(const fb200_fused_phase& P, int unit, float s0, float s1, int lane,
                                           EpiCtx& E, const EpiOperands& pre, int* A_status) {
  int sidx, tile;
  unit_locate(P, unit, sidx, tile);
  const int n = tile * 16 + lane;
  const bool valid = n < P.seg[sidx].n_out;
  float* yout = P.seg[sidx].y;
  const float v0 = s0 * E.final_scale, v1 = s1 * E.final_scale;
  const bool pack = (LL ? P.yll.g != nullptr : P.yp.limbs != nullptr) && sidx == 0;
  // operands fetched ahead by the caller, or all together now (one trip to L2 instead of a chain)
  EpiOperands op = pre.unit == unit ? pre : epilogue_operands<LL>(P, unit, lane, E);
  const bool has_r2 = LL ? P.r2l != nullptr : P.r2 != nullptr;
  if constexpr (LL) {
    if (op.stale & 1u) op.res1 = ld_ll_f32(P.r1l + n, E.ep - (unsigned)P.r1_back, A_status);
    if (op.stale & 2u) op.res2 = ld_ll_f32(P.r2l + n, E.ep - (unsigned)P.r2_back, A_status);
    if (op.stale & 4u) op.padd = ld_ll_f32(P.addl + n, E.ep - (unsigned)P.add_back, A_status);
  }
  float out = 0.f;
  if (valid) {
    if (P.epi == FB200_EPI_SWIGLU) {
      // silu(gate) * up, fusor-ml/fusor/src/composite/activations.rs:47-64
      out = (v0 / (1.0f + expf(-v0))) * v1;
    } else if (P.epi == FB200_EPI_RESIDUAL) {
      out = v0 + op.res1;
      if (has_r2) out += op.res2;
    } else {
      out = v0;
    }
    if (yout) yout[n] = out;
    if (LL && P.seg[sidx].yl) st_ll(P.seg[sidx].yl + n, __float_as_uint(out), E.ep);
    if (XS && E.xs && sidx == 0) {
      // partial row of a tensor-parallel projection: straight into every rank's buffer (P2P stores)
      for (int r = 0; r < E.xs->world; ++r) E.xs->data[r][E.xs_off + n] = out;
    }
    if (P.argmax_key && sidx == 0) {
      const unsigned long long key = argmax_key_of(out, (uint32_t)n);
      if (key > E.best_key) E.best_key = key;
    }
  }
  if (pack) {
    const float nv = out + op.padd;
    if constexpr (LL) emit_ll16(P.yll, n, nv * op.pw, nv, valid, 0x0000FFFFu, E.ep);
    else emit_packed16(P.yp, n, nv * op.pw, nv, valid, 0x0000FFFFu);
  }
}

// ---- flagged activation row -> shared memory -------------------------------------------------
// Every thread takes the 16-byte lines tid, tid + FT, ... of the row (6 lines per 16-element
// block: 4 of limbs, 1 of scale and sum, 1 of the sum of squares), keeps up to LL_BATCH of them
// in flight, and polls each until its epoch is the expected one. Returns this thread's share of
// the sum of squares (added in line order: the result does not depend on timing).
constexpr int LL_BATCH = 12;

// `with_sumsq` false: the consumer does not normalise, the sixth line of every block is not read.
__device__ __noinline__ float load_act_ll(const fb200_ll_act& row, int K, int Kp, uint8_t* xl, float2* xsp,
                                             unsigned epoch, int* status, bool with_sumsq) {
  const int tid = threadIdx.x;
  const int nblk = (K + 15) / 16;  // blocks the producers publish; the padding up to Kp is zero-filled here
  const int per = with_sumsq ? 6 : 5;  // lines read per block
  const float rcp_per = with_sumsq ? 1.0f / 6.0f : 0.2f;
  const int nlines = nblk * per;
  const uint4* src = reinterpret_cast<const uint4*>(row.g);
  float ss = 0.f;
  for (int l0 = tid; l0 < nlines; l0 += FT * LL_BATCH) {
    uint4 v[LL_BATCH];
    float sq[LL_BATCH];
    unsigned pending = 0u;
#pragma unroll
    for (int j = 0; j < LL_BATCH; ++j) {
      const int l = l0 + j * FT;
      sq[j] = 0.f;
      if (l < nlines) {
        const int b = fdiv(l, rcp_per);
        v[j] = ld_ll_line(src + b * FB200_LL_LINES + (l - per * b));
        pending |= 1u << j;
      }
    }
    int polls = 0;
    while (pending) {
#pragma unroll
      for (int j = 0; j < LL_BATCH; ++j) {
        if (!((pending >> j) & 1u)) continue;
        const int l = l0 + j * FT;
        const int b = fdiv(l, rcp_per), line = l - per * b;
        if (v[j].y == epoch && (line == 5 || v[j].w == epoch)) {
          if (line < 4) {
            const int B = 2 * b + (line >> 1);
            *reinterpret_cast<uint2*>(xl + limb2_off(B) + (line & 1) * 8) = make_uint2(v[j].x, v[j].z);
          } else if (line == 4) {
            xsp[b] = make_float2(__uint_as_float(v[j].x), __uint_as_float(v[j].z));  // {xsc, xss}
          } else {
            sq[j] = __uint_as_float(v[j].x);
          }
          pending &= ~(1u << j);
        } else {
          v[j] = ld_ll_line(src + b * FB200_LL_LINES + line);
        }
      }
      if (pending && (++polls > FB200_LL_POLL_LIMIT || ((polls & 63) == 0 && __ldcg(status) != 0))) {
        atomicExch(status, FB200_ERR_TIMEOUT);
        break;
      }
    }
#pragma unroll
    for (int j = 0; j < LL_BATCH; ++j) ss += sq[j];
  }
  for (int b = nblk + tid; b < Kp / 16; b += FT) {
    xsp[b] = make_float2(0.f, 0.f);
    *reinterpret_cast<uint4*>(xl + limb2_off(2 * b)) = make_uint4(0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(xl + limb2_off(2 * b + 1)) = make_uint4(0u, 0u, 0u, 0u);
  }
  return ss;
}

struct Smem {
  uint8_t* xl;
  float* xsc;
  float* xss;
  float* pieces;              // [FW][2][32]
  float* tmp;                 // [FW]
  unsigned long long* keys;   // [FW]
};

// (Inlined on purpose: as a separate function, with its state passed by reference or copied, the
// product loop measured 25 % slower.)
template <bool LEGACY, bool XS, bool LL>
__device__ __forceinline__ void gemv_phase(const FusedArgs& A, const fb200_fused_phase& P, const fb200_fused_phase* Pnext,
                           const fb200_fused_phase* Pf0, const fb200_fused_phase* Pf1, const Smem& S, WarpRing& R, Carry& C, unsigned long long* tr, unsigned epoch, unsigned lep) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K = P.K, Kp = P.Kp;
  const PhaseLocal q = phase_local(P);
  const Range r = warp_range(q.total, q.chunk, warp);
  const bool has_items = r.c0 < r.c1;  // the same for every thread of the CTA

  EpiCtx E;
  E.final_scale = 1.0f;
  E.best_key = 0ull;
  E.xs = XS && P.xs_index >= 0 && A.x.world > 1 ? &A.x : nullptr;
  E.xs_off = XS ? (int)((epoch & 1u) * (unsigned)A.x.world + (unsigned)A.x.me) * A.x.stride : 0;
  E.ep = lep;
  if constexpr (LL) {
    // ---- activation row: poll the producers' flagged row straight into shared memory. A CTA
    // without items in this phase needs no activations and goes on to the next phase.
    if (has_items) {
      float ss = load_act_ll(P.xll, K, Kp, S.xl, reinterpret_cast<float2*>(S.xsc), lep - 1u, A.status, P.xp_norm != 0);
      if (P.xp_norm) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
        if (lane == 0) S.tmp[warp] = ss;
        __syncthreads();
        ss = 0.f;
        for (int i = 0; i < FW; ++i) ss += S.tmp[i];
        E.final_scale = 1.0f / sqrtf(ss / (float)K + P.eps);
      }
      __syncthreads();
    }
  } else {
  // ---- activation row: limbs, scales, sums -> shared memory (asynchronous 16-byte copies through
  // L2, all in flight at once); 1/rms from the producer's sums of squares
  {
    const uint4* src = reinterpret_cast<const uint4*>(P.xp.limbs);
    uint4* dst = reinterpret_cast<uint4*>(S.xl);
    // 32-byte limb blocks are placed as limb_block() says: bits 1-2 of the 16-byte chunk index
    // are XOR-ed with bits 3-4
    for (int i = tid; i < Kp / 4; i += FT) cp_async16(dst + (i ^ (((i >> 3) & 3) << 1)), src + i);
    const uint4* s1 = reinterpret_cast<const uint4*>(P.xp.xsc);
    const uint4* s2 = reinterpret_cast<const uint4*>(P.xp.xss);
    uint4* d1 = reinterpret_cast<uint4*>(S.xsc);
    uint4* d2 = reinterpret_cast<uint4*>(S.xss);
    for (int i = tid; i < Kp / 64; i += FT) { cp_async16(d1 + i, s1 + i); cp_async16(d2 + i, s2 + i); }
  }
  if (P.xp_norm) {
    float ss = 0.f;
    for (int i = tid; i < (K + 15) / 16; i += FT) ss += __ldcg(P.xp.sumsq + i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if (lane == 0) S.tmp[warp] = ss;
    __syncthreads();
    ss = 0.f;
    for (int i = 0; i < FW; ++i) ss += S.tmp[i];
    E.final_scale = 1.0f / sqrtf(ss / (float)K + P.eps);
  }
  cp_async_wait_all();
  __syncthreads();
  }
  if (tr) tr[1] = global_ns();

  // ---- this warp's share: runs of items inside one (unit, pass), K group after K group
  const Lane L = make_lane(lane);
  // the first unit this warp will finish in the merge stage below: its epilogue operands are
  // requested now and arrive while the warp works
  EpiOperands pre;
  pre.unit = -1;
  const int ua = r.c0 < r.c1 ? fdiv(r.c0, q.rcp_ipu) : 0, ub = r.c0 < r.c1 ? fdiv(r.c1 - 1, q.rcp_ipu) : -1;
  if (ua + warp <= ub && lane < 16 && (P.epi == FB200_EPI_RESIDUAL || (LL ? P.addl != nullptr : P.yp_add != nullptr) || P.yp_norm_w))
    pre = epilogue_operands<LL>(P, ua + warp, lane, E);
  if (r.w0 < r.w1) {
    if (C.n == 0) prefetch_phase(P, R, warp, lane, C);  // nothing was fetched ahead
    Cursor cc = C.cc, ic = C.ic;
    const int u_first = cc.u;
    const int blocks16 = (cc.type == FB200_Q4_K || cc.type == FB200_Q6_K) ? 16 : 8;  // 16-element blocks per K group
    int i = r.w0, unit_first_item = r.w0, slot = 0;
    float pv0 = 0.f, pv1 = 0.f;
    while (i < r.w1) {
      const int kend = min(q.ng, cc.kg + (r.w1 - i));
      float acc_g = 0.f, acc_g8 = 0.f;
      auto refill = [&]() {
        __syncwarp();
        if (ic.i < r.w1) {  // refill the slot just consumed
          if (lane == 0) ring_issue(R, slot, q.stride, ic);
          cur_next(P, q, ic);
        }
        R.par ^= 1u << slot;
        slot = slot + 1 == q.stages ? 0 : slot + 1;
      };
      if constexpr (LL) {
        Group2Ptrs G = group2_ptrs(L, S.xl, reinterpret_cast<const float2*>(S.xsc), cc.kg, blocks16);
        auto run = [&](auto group_fn) {
          for (int kg = cc.kg; kg < kend; ++kg) {
            mbar_wait(R.bar0 + 8 * slot, (R.par >> slot) & 1u, A.status);
            group_fn(R.ptr + slot * q.stride, G);
            refill();
            group2_ptrs_next(G, blocks16);
          }
        };
        // the barrier-free variants exist for K-quant programs only
        if (cc.type == FB200_Q4_K) run([&](const uint8_t* tg, const Group2Ptrs& G2) { group2_q4k(G2.xq, G2.xsp, tg, L, acc_g, acc_g8); });
        else run([&](const uint8_t* tg, const Group2Ptrs& G2) { group2_q6k(G2.xq, G2.xsp, tg, L, acc_g, acc_g8); });
      } else {
      GroupPtrs G = group_ptrs(L, S.xl, S.xsc, S.xss, cc.kg, blocks16);
      auto run = [&](auto group_fn) {
        for (int kg = cc.kg; kg < kend; ++kg) {
          mbar_wait(R.bar0 + 8 * slot, (R.par >> slot) & 1u, A.status);
          group_fn(R.ptr + slot * q.stride);
          refill();
          group_ptrs_next(G, blocks16);
        }
      };
      // 32-element block types are compiled only into the kernel variants that serve them
      if (cc.type == FB200_Q4_K) {
        run([&](const uint8_t* tg) { group1_q4k(G.xq, G.xscp, G.xssp, tg, L, acc_g, acc_g8); });
      } else if (cc.type == FB200_Q6_K) {
        run([&](const uint8_t* tg) { group1_q6k(G.xq, G.xscp, G.xssp, tg, L, acc_g, acc_g8); });
      } else if (LEGACY) {
        if (cc.type == FB200_Q8_0) run([&](const uint8_t* tg) { group1_q8_0(G.xq, G.xscp, tg, L, acc_g, acc_g8); });
        else run([&](const uint8_t* tg) { group1_q4_0(G.xq, G.xscp, G.xssp, tg, L, acc_g, acc_g8); });
      }
      }
      i += kend - cc.kg;
      const int u_done = cc.u, p_done = cc.p;
      cc.kg = kend;
      if (kend == q.ng) {
        cc.kg = 0;
        if (++cc.p == q.npass) {
          cc.p = 0;
          ++cc.u;
          if (i < r.w1 && P.nseg > 1) {
            int sidx, tile;
            unit_locate(P, cc.u, sidx, tile);
            cc.type = P.seg[sidx].type;
          }
        }
      }
      // the pass, or this warp's share of it, ends here: rows 0..7 sit in acc_g of lanes 0, 4, ..,
      // rows 8..15 in acc_g8; lane (r & 15) takes row r
      acc_g += __shfl_xor_sync(0xFFFFFFFFu, acc_g, 1);
      acc_g += __shfl_xor_sync(0xFFFFFFFFu, acc_g, 2);
      acc_g8 += __shfl_xor_sync(0xFFFFFFFFu, acc_g8, 1);
      acc_g8 += __shfl_xor_sync(0xFFFFFFFFu, acc_g8, 2);
      const float lo = __shfl_sync(0xFFFFFFFFu, acc_g, (lane & 7) * 4);
      const float hi = __shfl_sync(0xFFFFFFFFu, acc_g8, (lane & 7) * 4);
      const float row = (lane & 8) ? hi : lo;
      if (p_done == 0) pv0 = row; else pv1 = row;
      if (cc.u != u_done || i == r.w1) {  // the unit, or this warp's share of it, ends here
        const bool complete = unit_first_item == u_done * q.ipu && i == (u_done + 1) * q.ipu;
        if (lane < 16) {
          if (complete) {
            unit_epilogue<XS, LL>(P, u_done, pv0, pv1, lane, E, pre, A.status);
          } else {
            float* pc = S.pieces + (warp * 2 + (u_done == u_first ? 0 : 1)) * 32;
            pc[lane] = pv0;
            pc[16 + lane] = pv1;
          }
        }
        __syncwarp();
        pv0 = 0.f; pv1 = 0.f;
        unit_first_item = i;
      }
    }
  }
  if (tr) tr[4] = global_ns();
  // ---- the ring is free: fetch the first slots of the next product phase
  C.n = 0;
  if (Pnext) prefetch_phase(*Pnext, R, warp, lane, C);
  // ... and ask L2 for the rest of it and for the phases the plan names: HBM keeps streaming while
  // the CTAs merge, meet, run attention and reload activations
  if (Pf0) l2_prefetch_share(*Pf0, warp, lane, P.pf_skip[0], P.pf_cap[0]);
  if (Pf1) l2_prefetch_share(*Pf1, warp, lane, P.pf_skip[1], P.pf_cap[1]);
  __syncthreads();
  if (tr) tr[2] = global_ns();

  // ---- units shared by several warps (summed in warp order) or several CTAs (in CTA order)
  if (r.c0 < r.c1) {
    const float rcp_per = 1.0f / (float)r.per, rcp_chunk = 1.0f / (float)q.chunk;
    for (int m = ua + warp; m <= ub; m += FW) {
      const int ib = max(m * q.ipu, r.c0), ie = min((m + 1) * q.ipu, r.c1);
      const int wlo = fdiv(ib - r.c0, rcp_per), whi = fdiv(ie - 1 - r.c0, rcp_per);
      const bool cta_whole = ib == m * q.ipu && ie == (m + 1) * q.ipu;
      if (wlo == whi && cta_whole) continue;  // one warp had the whole unit and finished it
      float s0 = 0.f, s1 = 0.f;
      if (lane < 16) {
        // warp wlo holds its piece of unit m in slot 0 if its share starts inside m, else in
        // slot 1; every later warp starts inside m
        int slot = r.c0 + wlo * r.per >= m * q.ipu ? 0 : 1;
        for (int w = wlo; w <= whi; ++w) {
          const float* pc = S.pieces + (w * 2 + slot) * 32;
          s0 += pc[lane];
          s1 += pc[16 + lane];
          slot = 0;
        }
      }
      if (tr && m == ua) tr[6] = global_ns();
      if (cta_whole) {
        if (lane < 16) unit_epilogue<XS, LL>(P, m, s0, s1, lane, E, pre, A.status);
        __syncwarp();
        if (tr && m == ua) tr[7] = global_ns();
        continue;
      }
      float* mine = A.gp + ((size_t)blockIdx.x * 2 + (m == ua ? 0 : 1)) * 32;
      if (lane < 16) { mine[lane] = s0; mine[16 + lane] = s1; }
      __threadfence();
      __syncwarp();
      const int clo = fdiv(m * q.ipu, rcp_chunk), chi = fdiv((m + 1) * q.ipu - 1, rcp_chunk);
      int last = 0;
      if (lane == 0) {
        const int old = atomicAdd(A.counters + m, 1);
        last = old == chi - clo;
        if (last) A.counters[m] = 0;
      }
      last = __shfl_sync(0xFFFFFFFFu, last, 0);
      if (!last) continue;
      __threadfence();
      if (lane < 16) {
        float t0 = 0.f, t1 = 0.f;
        for (int c = clo; c <= chi; ++c) {
          const int cfirst = fdiv(c * q.chunk, q.rcp_ipu);  // first unit of CTA c
          const float* pc = A.gp + ((size_t)c * 2 + (m == cfirst ? 0 : 1)) * 32;
          t0 += __ldcg(pc + lane);
          t1 += __ldcg(pc + 16 + lane);
        }
        unit_epilogue<XS, LL>(P, m, t0, t1, lane, E, pre, A.status);
      }
      __syncwarp();
    }
  }
  if (tr) tr[5] = global_ns();
  if (LL && A.trace && tid == 0) atomicMax(A.trace + (size_t)A.nphases * 8 + (int)(lep - A.epoch_base) % A.nphases, global_ns());
  if (P.argmax_key) {
    // one atomic per CTA: lanes -> warp -> CTA maximum of the running keys
    unsigned long long k = E.best_key;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, k, o);
      if (other > k) k = other;
    }
    if (lane == 0) S.keys[warp] = k;
    __syncthreads();
    if (tid == 0) {
      for (int i = 1; i < FW; ++i) if (S.keys[i] > k) k = S.keys[i];
      if (k) atomicMax(P.argmax_key, k);
    }
  }
}

// value of element n of the row a PACK / EMBED phase packs
__device__ __forceinline__ float pack_source(const fb200_fused_phase& P, uint32_t id, int n) {
  if (P.kind == FB200_PH_EMBED) {
    if ((unsigned long long)id >= P.emb_n) return 0.f;
    if (P.emb_tiled) {
      const int kg = n / P.emb_ge, i = n - kg * P.emb_ge;
      const uint8_t* tg = P.emb + ((size_t)(id >> 4) * P.emb_ngroups + kg) * (size_t)P.emb_tgb;
      return fb::tile_dequant((uint32_t)P.emb_type, tg, (int)(id & 15u), i);
    }
    return fb::raw_elem((uint32_t)P.emb_type, P.emb, (uint64_t)id * (uint64_t)P.K + n);
  }
  float v = __ldcg(P.src + n);
  if (P.src_add) v += __ldcg(P.src_add + n);
  return v;
}

template <bool LL>
__device__ __noinline__ void pack_phase(const fb200_fused_phase& P, unsigned lep) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (P.K + 31) / 32;
  const uint32_t id = P.kind == FB200_PH_EMBED ? __ldcg(P.ids) : 0u;
  for (int b = (int)blockIdx.x * FW + warp; b < nblk; b += (int)gridDim.x * FW) {
    const int n = b * 32 + lane;
    const bool valid = n < P.K;
    float v = valid ? pack_source(P, id, n) : 0.f;
    if (valid && P.xout) P.xout[n] = v;
    if (LL && valid && P.xoutl) st_ll(P.xoutl + n, __float_as_uint(v), lep);
    const float nv = v;
    if (valid && P.yp_norm_w) v *= P.yp_norm_w[n];
    if constexpr (LL) emit_ll16(P.yll, n, v, nv, valid, 0xFFFFFFFFu, lep);
    else emit_packed16(P.yp, n, v, nv, valid, 0xFFFFFFFFu);
  }
}

// Sum of the ranks' partial rows (rank order: the same bits on every rank), residual rows added
// in the order of the single-GPU epilogues, float copies and the packed row for the next product.
__device__ __noinline__ void xsum_phase(const FusedArgs& A, const fb200_fused_phase& P, unsigned epoch) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) xchg_signal_and_wait(A, epoch, blockIdx.x == 0);
  __syncthreads();
  const fb200_fused_xchg& X = A.x;
  const float* base = X.data[X.me] + (size_t)(epoch & 1u) * X.world * X.stride;
  const int nblk = (P.K + 31) / 32;
  for (int b = (int)blockIdx.x * FW + warp; b < nblk; b += (int)gridDim.x * FW) {
    const int n = b * 32 + lane;
    const bool valid = n < P.K;
    float v = 0.f;
    if (valid) {
      for (int r = 0; r < X.world; ++r) v += __ldcg(base + (size_t)r * X.stride + n);
      if (P.out_sum) P.out_sum[n] = v;
      if (P.src) v += __ldcg(P.src + n);
      if (P.src_add) v += __ldcg(P.src_add + n);
      if (P.xout) P.xout[n] = v;
    }
    const float nv = v;
    if (valid && P.yp_norm_w) v *= P.yp_norm_w[n];
    emit_packed16(P.yp, n, v, nv, valid, 0xFFFFFFFFu);
  }
}

template <bool XS>
__device__ __noinline__ void advance_phase(const FusedArgs& A, const fb200_fused_phase& P, unsigned epoch) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  // the output head kept a running (value, index) maximum; 0 means no finite logit
  unsigned long long key = __ldcg(P.argmax_key);
  if (XS && A.x.world > 1 && P.xs_index >= 0) {
    // sharded output head: every rank's best (value, global id); the largest key wins everywhere
    const fb200_fused_xchg& X = A.x;
    if (key) key += X.id_base;  // the id sits in the low half and stays below 2^32
    const int slot = (int)(epoch & 1u) * X.world;
    for (int r = 0; r < X.world; ++r) X.keys[r][slot + X.me] = key;
    xchg_signal_and_wait(A, epoch, true);
    for (int r = 0; r < X.world; ++r) {
      const unsigned long long k = __ldcg(X.keys[X.me] + slot + r);
      if (k > key) key = k;
    }
  }
  const uint32_t tok = key ? (uint32_t)(key & 0xFFFFFFFFull) : 0xFFFFFFFFu;
  *P.argmax_key = 0ull;
  P.next[0] = tok;
  P.ids_w[0] = tok;
  const int step = __ldcg(P.step_dev);
  if (A.record && P.hist && step < P.hist_cap) P.hist[step] = tok;
  *P.pos_dev = __ldcg(P.pos_dev) + 1;
  *P.step_dev = step + 1;
}

// The context is cut into at most att.nsplit splits of at least FUSED_SPLIT_KEYS keys: an item's
// run time is mostly fixed latencies, so many small items finish sooner than few large ones, and
// very short contexts run a single item per KV head with nothing to merge.
template <int D, int ROWS, bool LL>
__device__ __noinline__ void attn_phase(const fb200_fused_phase& P, uint8_t* dsm, unsigned lep, int* status) {
  const int tid = threadIdx.x;
  if (tid >= DEC_THREADS) return;
  fb200_dec_args a = P.att;
  a.pos_plus1 = __ldcg(a.pos_dev) + 1;
  const int skv = a.pos_plus1;
  a.nsplit = max(1, min(a.nsplit, (skv + FUSED_SPLIT_KEYS - 1) / FUSED_SPLIT_KEYS));
  a.ep_in = lep - 1u;
  a.ep_out = lep;
  a.status = status;
  const int nitems = a.b * a.hkv * a.nsplit;
  for (int item = (int)blockIdx.x; item < nitems; item += (int)gridDim.x) {
    attn_decode_item<D, FUSED_DEC_CH, ROWS, 1, false, LL>(a, item, dsm, tid);
    dec_sync<1>();
  }
}

// One kernel variant per attention shape (head size D, query rows per KV head ROWS) and per
// family of weight types (LEGACY = the 32-element block types too): a variant carries only the
// code it runs, which keeps the instruction footprint of a step small.
// LL: the phases of a step exchange flagged rows instead of meeting at grid barriers.
template <int D, int ROWS, bool LEGACY, bool XS, bool LL>
__global__ void __launch_bounds__(FT, 1)
fused_step_kernel(const FusedArgs A) {
  static_assert(!(LL && (XS || LEGACY)), "barrier-free variants: single GPU, K-quant weights");
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* ring = smem;
  constexpr int RB = LL ? RING_BYTES_LL : RING_BYTES;
  constexpr int MS = LL ? MAX_STAGES_LL : MAX_STAGES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FW * RB);
  uint8_t* xreg = smem + FW * RB + FW * MS * 8;
  Smem S;
  S.xl = xreg;
  S.pieces = reinterpret_cast<float*>(xreg + A.xregion);
  S.tmp = S.pieces + FW * 2 * 32;
  S.keys = reinterpret_cast<unsigned long long*>(S.tmp + 32);
  WarpRing R;
  R.ptr = ring + warp * RB;
  R.base = smem_u32(R.ptr);
  R.bar0 = smem_u32(bars + warp * MS);
  R.par = 0u;
  R.policy = l2_evict_first_policy();
  if (lane == 0) {
    for (int s = 0; s < MS; ++s) mbar_init(R.bar0 + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // Phase descriptors live in shared memory: a window of five consecutive phases (the current one,
  // the next three, which always include the next product phase, and the one being fetched). The
  // descriptor of phase g + 4 is copied asynchronously while phase g runs, so that its trip to L2
  // never sits between two phases.
  uint32_t* sdesc = reinterpret_cast<uint32_t*>(S.keys + 32);
  const int total_phases = A.nsteps * A.nphases;
  auto desc_of = [&](int g) { return reinterpret_cast<const fb200_fused_phase*>(sdesc + (g % DESC_SLOTS) * DESC_WORDS); };
  auto load_desc = [&](int g) {
    if (g >= total_phases) return;
    const uint4* src = reinterpret_cast<const uint4*>(A.prog + g % A.nphases);
    uint4* dst = reinterpret_cast<uint4*>(sdesc + (g % DESC_SLOTS) * DESC_WORDS);
    for (int i = tid; i < DESC_WORDS / 4; i += FT) cp_async16(dst + i, src + i);
  };
  for (int g = 0; g < DESC_SLOTS - 1; ++g) load_desc(g);
  cp_async_wait_all();
  __syncthreads();

  unsigned target = 0u;
  Carry C;
  C.n = 0;
  if (A.first_gemv >= 0 && A.first_gemv < DESC_SLOTS - 1) prefetch_phase(*desc_of(A.first_gemv), R, warp, lane, C);
  int g = 0;
  int prev_kind = -1;
  for (int step = 0; step < A.nsteps; ++step) {
    for (int ph = 0; ph < A.nphases; ++ph, ++g) {
      const fb200_fused_phase& P = *desc_of(g);
      if (g) {
        // Flagged rows carry their own readiness, so a barrier-free variant meets only where plain
        // memory changes hands: the greedy-token hand-over (argmax key -> ADVANCE -> next EMBED).
        const bool meet = !LL || P.kind == FB200_PH_ADVANCE || prev_kind == FB200_PH_ADVANCE;
        if (meet)
          grid_barrier(A, target, A.trace && step == A.nsteps - 1 ? A.trace + (size_t)A.nphases * 8 + ph : nullptr);
        else
          __syncthreads();  // every warp is done with the previous phase (descriptor slot, activation region)
      }
      load_desc(g + DESC_SLOTS - 1);  // into the slot of the phase that has just ended; waited for below
      prev_kind = P.kind;
      const unsigned epoch = XS ? A.x.epoch_base + (unsigned)(step * A.x.per_step + (P.xs_index >= 0 ? P.xs_index : 0)) : 0u;
      const unsigned lep = A.epoch_base + (unsigned)g;  // flagged rows: this phase's epoch
      unsigned long long* tr = A.trace && blockIdx.x == 0 && tid == 0 && step == A.nsteps - 1 ? A.trace + ph * 8 : nullptr;
      if (tr) tr[0] = global_ns();
      switch (P.kind) {
        case FB200_PH_GEMV: {
          S.xsc = reinterpret_cast<float*>(S.xl + (LL ? ((size_t)P.Kp / 8 * 18 + 63) / 64 * 64 : (size_t)P.Kp * 4));
          S.xss = S.xsc + P.Kp / 16;
          const int ahead = P.next_gemv < 0 ? -1 : (P.next_gemv > ph ? P.next_gemv - ph : P.next_gemv + A.nphases - ph);
          const bool has_next = ahead > 0 && ahead <= 3 && g + ahead < total_phases;
          auto planned = [&](int j) -> const fb200_fused_phase* {
            const int off = P.pf_off[j];
            return off > 0 && off < DESC_SLOTS - 1 && g + off < total_phases ? desc_of(g + off) : nullptr;
          };
          gemv_phase<LEGACY, XS, LL>(A, P, has_next ? desc_of(g + ahead) : nullptr, planned(0), planned(1), S, R, C, tr, epoch, lep);
          break;
        }
        case FB200_PH_ATTN:
          attn_phase<D, ROWS, LL>(P, xreg, lep, A.status);
          break;
        case FB200_PH_PACK:
        case FB200_PH_EMBED:
          pack_phase<LL>(P, lep);
          break;
        case FB200_PH_XSUM:
          if (XS) xsum_phase(A, P, epoch);
          break;
        default:
          advance_phase<XS>(A, P, epoch);
          break;
      }
      if (tr) tr[3] = global_ns();
      cp_async_wait_all();  // this thread's part of the descriptor fetched during the phase (the meeting above publishes it)
    }
  }
}

size_t x_region_need(const fb200_fused_phase* prog, int nphases, bool flagged) {
  size_t need = 0;
  for (int i = 0; i < nphases; ++i) {
    const auto& p = prog[i];
    if (p.kind == FB200_PH_GEMV) need = std::max(need, flagged ? (size_t)p.Kp / 8 * 18 + 64 + (size_t)p.Kp / 16 * 8 : (size_t)p.Kp * 4 + (size_t)p.Kp / 16 * 8);
    if (p.kind == FB200_PH_ATTN) need = std::max(need, dec_smem_bytes(p.att_d, FUSED_DEC_CH));
  }
  return (need + 127) / 128 * 128;
}

size_t smem_total(size_t xregion, bool flagged) {
  return (size_t)FW * (flagged ? RING_BYTES_LL : RING_BYTES) + (size_t)FW * (flagged ? MAX_STAGES_LL : MAX_STAGES) * 8 + xregion + (size_t)FW * 2 * 32 * 4 + 32 * 4 +
         32 * 8 + DESC_SLOTS * DESC_WORDS * 4;
}

}  // namespace

int fb200_fused_grid(const fb200_device* dev) { return dev->sm_count; }

bool fb200_fused_gemv_phase(fb200_fused_phase* p, const fb200_qmatrix* const* ws, float* const* ys, int nw,
                            int epi, int grid, bool flagged) {
  if (nw < 1 || nw > 3 || (epi != FB200_EPI_NONE && nw != 1)) return false;
  TileGeom geo0;
  if (!tile_geom(ws[0]->type, &geo0)) return false;
  p->kind = FB200_PH_GEMV;
  p->nseg = nw;
  p->epi = epi;
  p->stride = 0;
  p->nunits = 0;
  for (int i = 0; i < nw; ++i) {
    TileGeom geo;
    if (!ws[i]->tiled || !tile_geom(ws[i]->type, &geo) || geo.group_elems != geo0.group_elems ||
        ws[i]->k != ws[0]->k)
      return false;
    p->seg[i].w = ws[i]->data;
    p->seg[i].y = ys[i];
    p->seg[i].type = (int)ws[i]->type;
    p->seg[i].tg = geo.tg_bytes;
    p->seg[i].units = ws[i]->ntiles;
    p->seg[i].n_out = (int)ws[i]->n;
    p->nunits += ws[i]->ntiles;
    p->stride = std::max(p->stride, (geo.tg_bytes + 127) / 128 * 128);
  }
  p->K = (int)ws[0]->k;
  p->ngroups = ws[0]->ngroups;
  p->Kp = p->ngroups * geo0.group_elems;
  p->pair_off = 0;
  int npass = 1;
  if (epi == FB200_EPI_SWIGLU) {
    if (ws[0]->ntiles % 2) return false;
    npass = 2;
    p->seg[0].units = ws[0]->ntiles / 2;
    p->nunits = p->seg[0].units;
    p->seg[0].n_out = (int)(ws[0]->n / 2);
    p->pair_off = ws[0]->ntiles / 2;
  }
  p->ipu = npass * p->ngroups;
  const long long total = (long long)p->nunits * p->ipu;
  if (total <= 0 || total > (1ll << 21)) return false;  // bound of the reciprocal divisions in the kernel
  p->rcp_ipu = (float)(1.0 / (double)p->ipu);
  p->rcp_ng = (float)(1.0 / (double)p->ngroups);
  p->total = (int)total;
  p->chunk = (int)((total + grid - 1) / grid);
  // Whole units per CTA when that costs at most a fifth more items for the busiest CTA: no unit
  // is then shared between CTAs and nothing has to be merged through global memory.
  const long long aligned = (long long)((p->nunits + grid - 1) / grid) * p->ipu;
  if (aligned * 5 <= (long long)p->chunk * 6) p->chunk = (int)aligned;
  p->stages = flagged ? std::min(MAX_STAGES_LL, RING_BYTES_LL / p->stride) : std::min(MAX_STAGES, RING_BYTES / p->stride);
  if (const char* e = getenv("FB200_FUSED_STAGES")) p->stages = std::max(1, std::min(p->stages, atoi(e)));
  return p->stages >= 1;
}

void fb200_fused_plan_prefetch(fb200_fused_phase* prog, int nphases, int grid, size_t ahead_bytes) {
  std::vector<int> gv;
  for (int i = 0; i < nphases; ++i) {
    if (prog[i].kind != FB200_PH_GEMV) continue;
    gv.push_back(i);
    for (int j = 0; j < 2; ++j) prog[i].pf_off[j] = prog[i].pf_skip[j] = prog[i].pf_cap[j] = 0;
  }
  const int n = (int)gv.size();
  if (n < 2 || ahead_bytes == 0) return;
  const int warps = grid * FW;
  // weight bytes of a phase and the items per warp that fit the bound (a phase larger than the bound,
  // the output head, is requested in part)
  auto phase_bytes = [&](const fb200_fused_phase& p) {
    size_t b = 0;
    const int npass = p.epi == FB200_EPI_SWIGLU ? 2 : 1;
    for (int s = 0; s < p.nseg; ++s) b += (size_t)p.seg[s].units * npass * p.ngroups * p.seg[s].tg;
    return b;
  };
  // Walk the cyclic chain of product phases twice (the second lap is the steady state that is kept).
  // front = product phases after the current one whose shares have been requested already.
  int front = 0;
  for (int lap = 0; lap < 2; ++lap) {
    for (int s = 0; s < n; ++s) {
      fb200_fused_phase& p = prog[gv[s]];
      int slots = 0;
      for (int j = 0; j < 2; ++j) p.pf_off[j] = p.pf_skip[j] = p.pf_cap[j] = 0;
      for (int d = 1; d <= 2 && slots < 2; ++d) {
        const int t = gv[(s + d) % n];
        int off = t - gv[s];
        if (off <= 0) off += nphases;
        if (off >= DESC_SLOTS - 1) break;  // outside the descriptor window of the kernel
        size_t pending = 0;  // bytes requested and not yet consumed once phase d ahead is added
        for (int e = 1; e <= d; ++e) pending += std::min(phase_bytes(prog[gv[(s + e) % n]]), ahead_bytes);
        if (pending > ahead_bytes && d > 1) break;
        if (d <= front) continue;  // requested when an earlier phase ended
        const fb200_fused_phase& q = prog[t];
        p.pf_off[slots] = off;
        p.pf_skip[slots] = d == 1 ? q.stages : 0;  // the ring takes the first items of the next product phase
        p.pf_cap[slots] = 1 << 20;
        if (phase_bytes(q) > ahead_bytes)  // only d == 1 gets here: the first ahead_bytes of the phase
          p.pf_cap[slots] = (int)std::max<size_t>(1, ahead_bytes / ((size_t)warps * (size_t)q.stride));
        ++slots;
        front = d;
      }
      front = std::max(front - 1, 0);
    }
  }
}

size_t fb200_fused_smem_bytes(const fb200_fused_phase* prog_host, int nphases, bool flagged) {
  const size_t total = smem_total(x_region_need(prog_host, nphases, flagged), flagged);
  return total + STATIC_SMEM_RESERVE <= (size_t)SMEM_LIMIT ? total : 0;
}

namespace {
// attention shape and weight-type family of a program
void program_shape(const fb200_fused_phase* prog_host, int nphases, int* att_d, int* groups, bool* legacy) {
  *att_d = 128; *groups = 1; *legacy = false;
  for (int i = 0; i < nphases; ++i) {
    const auto& ph = prog_host[i];
    if (ph.kind == FB200_PH_ATTN) { *att_d = ph.att_d; *groups = std::max(*groups, ph.att.groups); }
    if (ph.kind == FB200_PH_GEMV)
      for (int j = 0; j < ph.nseg; ++j) *legacy = *legacy || ph.seg[j].type == FB200_Q4_0 || ph.seg[j].type == FB200_Q8_0;
  }
}
}  // namespace

bool fb200_fused_flagged_available(const fb200_fused_phase* prog_host, int nphases) {
  int att_d, groups;
  bool legacy;
  program_shape(prog_host, nphases, &att_d, &groups, &legacy);
  return !legacy && (att_d == 128 || att_d == 64);
}

int fb200_fused_launch(fb200_device* dev, const fb200_fused_phase* prog_dev, const fb200_fused_phase* prog_host,
                       int nphases, int nsteps, bool record_history, const fb200_fused_xchg* xchg, bool flagged) {
  if (nphases <= 0 || nsteps <= 0) return FB200_OK;
  const int grid = fb200_fused_grid(dev);
  const size_t xregion = x_region_need(prog_host, nphases, flagged);
  const size_t smem = fb200_fused_smem_bytes(prog_host, nphases, flagged);
  if (!smem) return fb200_fail(dev, FB200_ERR_CAPACITY, "fused step: the program does not fit in shared memory");
  int max_units = 1, first = -1;
  for (int i = 0; i < nphases; ++i)
    if (prog_host[i].kind == FB200_PH_GEMV) {
      max_units = std::max(max_units, prog_host[i].nunits);
      if (first < 0) first = i;
    }
  // scratch: [barrier word, padded to 256 B][gp: grid * 64 floats][counters: max_units ints]
  const size_t gp_off = 256, cnt_off = gp_off + (size_t)grid * 64 * 4;
  const size_t need = cnt_off + (size_t)max_units * 4;
  if (need > dev->fused_bytes) {
    FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
    if (dev->fused) cudaFree(dev->fused);
    dev->fused = nullptr;
    dev->fused_bytes = 0;
    const size_t cap = need + (64 << 10);
    FB_CUDA(dev, cudaMalloc(&dev->fused, cap));
    FB_CUDA(dev, cudaMemsetAsync(dev->fused, 0, cap, dev->stream));
    dev->fused_bytes = cap;
  }
  // kernel variant: attention shape and weight-type family of this program
  int att_d, groups;
  bool legacy;
  program_shape(prog_host, nphases, &att_d, &groups, &legacy);
  void (*kern)(const FusedArgs) = nullptr;
  int variant = 0;
  const bool xs = xchg && xchg->world > 1;  // the exchange code lives in variants of its own
  if (xs && legacy) return fb200_fail(dev, FB200_ERR_UNSUPPORTED_DTYPE, "fused step: tensor parallel needs K-quant weights");
  if (flagged && (xs || legacy)) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "fused step: no barrier-free variant for this program");
  if (flagged) {
    if (att_d == 128 && groups <= 4) { kern = fused_step_kernel<128, 4, false, false, true>; variant = 8; }
    else if (att_d == 128) { kern = fused_step_kernel<128, 8, false, false, true>; variant = 9; }
    else if (att_d == 64) { kern = fused_step_kernel<64, 8, false, false, true>; variant = 10; }
    else return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "fused step: head size %d", att_d);
  }
  else if (att_d == 128 && groups <= 4 && !legacy) { kern = xs ? fused_step_kernel<128, 4, false, true, false> : fused_step_kernel<128, 4, false, false, false>; variant = xs ? 5 : 0; }
  else if (att_d == 128 && !legacy) { kern = xs ? fused_step_kernel<128, 8, false, true, false> : fused_step_kernel<128, 8, false, false, false>; variant = xs ? 6 : 1; }
  else if (att_d == 128) { kern = fused_step_kernel<128, 8, true, false, false>; variant = 2; }
  else if (att_d == 64 && !legacy) { kern = xs ? fused_step_kernel<64, 8, false, true, false> : fused_step_kernel<64, 8, false, false, false>; variant = xs ? 7 : 3; }
  else if (att_d == 64) { kern = fused_step_kernel<64, 8, true, false, false>; variant = 4; }
  else return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "fused step: head size %d", att_d);
  static bool configured[64][12] = {};
  if (!configured[dev->ordinal & 63][variant]) {
    FB_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      SMEM_LIMIT - STATIC_SMEM_RESERVE));
    configured[dev->ordinal & 63][variant] = true;
  }
  FusedArgs a = {};
  a.prog = prog_dev;
  a.nphases = nphases;
  a.nsteps = nsteps;
  a.record = record_history ? 1 : 0;
  a.first_gemv = first;
  a.xregion = (int)xregion;
  a.bar = reinterpret_cast<unsigned*>(dev->fused);
  a.gp = reinterpret_cast<float*>((uint8_t*)dev->fused + gp_off);
  a.counters = reinterpret_cast<int*>((uint8_t*)dev->fused + cnt_off);
  a.status = dev->status;
  if (xchg) a.x = *xchg;
  if (flagged) {
    // one epoch per phase executed; 0 is the value of cleared buffers and is skipped when the
    // 32-bit counter wraps (readers compare for equality, so old epochs never match new ones)
    const uint32_t count = (uint32_t)nsteps * (uint32_t)nphases;
    if (dev->ll_epoch + count < dev->ll_epoch || dev->ll_epoch == 0) dev->ll_epoch = 1;
    a.epoch_base = dev->ll_epoch;
    dev->ll_epoch += count;
  }
  FB_CUDA(dev, cudaMemsetAsync(a.bar, 0, 4, dev->stream));
  // FB200_FUSED_TRACE=1: per-phase time stamps of CTA 0, printed to stderr after the launch
  static const bool want_trace = getenv("FB200_FUSED_TRACE") && getenv("FB200_FUSED_TRACE")[0] == '1';
  unsigned long long* trace_dev = nullptr;
  if (want_trace) {
    FB_CUDA(dev, cudaMalloc(&trace_dev, (size_t)nphases * 9 * 8));
    FB_CUDA(dev, cudaMemsetAsync(trace_dev, 0, (size_t)nphases * 9 * 8, dev->stream));
    a.trace = trace_dev;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(FT);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once, or the launch fails
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FB_CUDA(dev, cudaLaunchKernelEx(&cfg, kern, a));
  dev->launches++;
  if (trace_dev) {
    std::vector<unsigned long long> t((size_t)nphases * 9);
    FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
    FB_CUDA(dev, cudaMemcpy(t.data(), trace_dev, t.size() * 8, cudaMemcpyDeviceToHost));
    cudaFree(trace_dev);
    fprintf(stderr, "fused step trace (CTA 0, last of %d steps): phase kind start_us [last CTA arrived before] load_us work_us tail_us\n", nsteps);
    for (int i = 0; i < nphases; ++i) {
      const unsigned long long* q = t.data() + (size_t)i * 8;
      const double t0 = (double)(q[0] - t[0]) / 1e3;
      // barriers: phase start minus the last CTA's arrival; flagged rows: end of this CTA's activation
      // load minus the moment the last producer CTA of the previous phase finished its epilogues
      const double ta = !i ? 0.0 : flagged ? ((double)q[1] - (double)t[(size_t)nphases * 8 + i - 1]) / 1e3
                                           : ((double)q[0] - (double)t[(size_t)nphases * 8 + i]) / 1e3;
      if (prog_host[i].kind == FB200_PH_GEMV)
        fprintf(stderr, "  %3d gemv  %9.2f [%5.2f] %7.2f %7.2f %7.2f  (items %d, K %d; own loop %.2f, sync %.2f, merge %.2f = sum %.2f + epilogue %.2f + rest)\n",
                i, t0, ta, (double)(q[1] - q[0]) / 1e3, (double)(q[2] - q[1]) / 1e3, (double)(q[3] - q[2]) / 1e3,
                prog_host[i].total, prog_host[i].K, (double)(q[4] - q[1]) / 1e3, (double)(q[2] - q[4]) / 1e3,
                (double)(q[5] - q[2]) / 1e3, (double)(q[6] - q[2]) / 1e3, (double)(q[7] - q[6]) / 1e3);
      else
        fprintf(stderr, "  %3d kind%d %9.2f [%5.2f] %7.2f\n", i, prog_host[i].kind, t0, ta, (double)(q[3] - q[0]) / 1e3);
    }
  }
  return FB200_OK;
}
