// Decode-time attention for one new position per sequence, as a device function shared by the
// stand-alone kernel and the fused decode-step kernel: RoPE(q), RoPE(k) + fp16 append,
// split-KV online softmax over the cache, partials merged by the split that arrives last.
// Attention math as fusor-ml/fusor/src/composite/attention.rs (scaled q.k, softmax, .v) with
// interleaved RoPE (fusor-ml/fusor/src/composite/rope.rs:77-108) and the KV append of
// fusor-ml/fusor/src/cache/kv_cache.rs:50-62. Everything another CTA may have written during
// the same kernel is read through L2 (ld.global.cg / cp.async.cg).
#pragma once

#include "common.cuh"
#include "packed_act.cuh"

// Arguments of one decode-attention launch / phase (all device pointers).
struct fb200_dec_args {
  const float* q;       // [B, H, D]   (not yet rotated)
  const float* k_new;   // [B, Hkv, D] (not yet rotated)
  const float* v_new;   // [B, Hkv, D]
  __half* kc;           // [B, Hkv, cap, D]
  __half* vc;
  const float* rope_cos;  // [ctx, D/2]
  const float* rope_sin;
  const int* pos_dev;   // position of the new token = number of cached keys; null: the cache
                        // already holds all `skv` keys, q is already rotated, nothing is appended
  int skv;              // number of keys when pos_dev is null
  float* part;          // [nsplit][B * H][D + 2]
  float* out;           // [B, H * D]
  int* done;            // [B * Hkv] arrival counters, zero between launches
  fb200_packed_act out_packed;  // optional: the merged rows also in packed form (row of H * D)
  int b, h, hkv, groups, cap, nsplit;
  float scale;
  int pos_plus1;        // > 0: *pos_dev + 1, already read by the caller (saves a dependent load); 0: not known
  int min_keys;         // stand-alone kernel: a split takes at least this many keys (0: 64), so short
                        // contexts run fewer splits than the launch provided
  // flagged rows (persistent decode kernel without grid barriers between its phases): q, k_new
  // and v_new arrive as f32 granules {value, epoch} that the item polls, and the merged output
  // leaves as a flagged packed row
  const uint2* q_ll;
  const uint2* k_ll;
  const uint2* v_ll;
  fb200_ll_act out_ll;
  unsigned ep_in, ep_out;
  int* status;          // device status word for waits that give up
};

namespace {

using DecArgs = fb200_dec_args;

constexpr int DEC_ROWS = 8;       // query rows per KV head (H / Hkv <= 8)
constexpr int DEC_THREADS = 256;  // threads per item



__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's committed copy groups are still in flight.
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Bytes of dynamic shared memory one item needs (nb = staging buffers: 1, or 2 to copy the next
// chunk of keys while the current one is being used).
__host__ __device__ constexpr size_t dec_smem_bytes(int d, int dec_ch, int nb = 1) {
  return (size_t)nb * 2 * dec_ch * (d * 2 + 64) + (size_t)DEC_ROWS * d * 4 + (size_t)DEC_ROWS * dec_ch * 4;
}

// Barrier of the 256 threads that work on an item: the whole CTA (BAR = 0) or a named barrier
// when the CTA has more warps than the team.
template <int BAR>
__device__ __forceinline__ void dec_sync() {
  if (BAR == 0) __syncthreads();
  else asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(DEC_THREADS) : "memory");
}

// One (batch, kv head, split) item, executed by DEC_THREADS threads (tid = 0 .. DEC_THREADS - 1).
// DEC_CH = keys per shared-memory chunk; ROWS = query rows computed per KV head (>= H / Hkv). PDL: the caller is a kernel launched with programmatic
// stream serialization, whose predecessor produced q, k_new and v_new.
// Two neighbouring f32 granules (elements 2p, 2p + 1) of a flagged row, polled until both carry
// `epoch` (bounded, like every wait).
__device__ __forceinline__ float2 ld_ll_pair(const uint2* p, uint32_t epoch, int* status) {
  const uint4* line = reinterpret_cast<const uint4*>(p);
  uint4 v = ld_ll_line(line);
  int polls = 0;
  while (v.y != epoch || v.w != epoch) {
    if (++polls > FB200_LL_POLL_LIMIT || ((polls & 63) == 0 && __ldcg(status) != 0)) {
      atomicExch(status, FB200_ERR_TIMEOUT);
      break;
    }
    v = ld_ll_line(line);
  }
  return make_float2(__uint_as_float(v.x), __uint_as_float(v.z));
}

// LLIO: q / k_new / v_new come in and the merged row goes out as flagged rows (see DecArgs).
// NB = 2: two staging buffers; the copy of chunk i + 1 runs while chunk i is being used, so a long
// key range streams at the memory system's pace instead of paying its latency once per chunk.
template <int D, int DEC_CH, int ROWS, int BAR, bool PDL, bool LLIO = false, int NB = 1>
__device__ void attn_decode_item(const DecArgs& a, int item, uint8_t* dsm, int tid) {
  constexpr int ATT_THREADS = DEC_THREADS;
  constexpr int KSTR = D * 2 + 64;   // bytes per staged row: consecutive keys land 64 B apart mod 128
  constexpr int DV = D / 32;
  constexpr int NC = D / 8;          // 16-byte chunks per row
  uint8_t* kbuf = dsm;                                   // [DEC_CH][KSTR], buffer b at + b * BUFB
  uint8_t* vbuf = dsm + DEC_CH * KSTR;                   // [DEC_CH][KSTR]
  constexpr int BUFB = 2 * DEC_CH * KSTR;                // bytes of one staging buffer (keys + values)
  float (*qs)[D] = reinterpret_cast<float (*)[D]>(dsm + NB * BUFB);                  // [ROWS][D]
  float (*sc)[DEC_CH] = reinterpret_cast<float (*)[DEC_CH]>(qs + ROWS);              // [ROWS][DEC_CH]
  float (*ored)[ROWS][D] = reinterpret_cast<float (*)[ROWS][D]>(dsm);                // aliases kbuf/vbuf
  __shared__ float alpha[ROWS], row_m[ROWS], row_l[ROWS];
  __shared__ int is_last;
  static_assert((ATT_THREADS / 32) * ROWS * D * 4 <= 2 * DEC_CH * KSTR, "reduction buffer must fit the staging area");

  const int warp = tid >> 5, lane = tid & 31;
  int bid = item;
  const int split = bid % a.nsplit; bid /= a.nsplit;
  const int kvh = bid % a.hkv;
  const int bi = bid / a.hkv;
  const int nrows = a.groups;
  const int pos = a.pos_dev ? (a.pos_plus1 > 0 ? a.pos_plus1 - 1 : __ldcg(a.pos_dev)) : -1;
  const int skv = a.pos_dev ? pos + 1 : a.skv;
  const int per = (skv + a.nsplit - 1) / a.nsplit;
  const int kbeg = min(skv, split * per), kend = min(skv, kbeg + per);
  __half* kb = a.kc + ((size_t)bi * a.hkv + kvh) * (size_t)a.cap * D;
  __half* vb = a.vc + ((size_t)bi * a.hkv + kvh) * (size_t)a.cap * D;

  // stage chunk [c0, c0 + cn) of the cached rows (the new row `pos` is filled in separately)
  auto stage = [&](int c0, int cn, int buf) {
    for (int i = tid; i < cn * NC * 2; i += ATT_THREADS) {
      const int which = i / (cn * NC), rem = i - which * (cn * NC);
      const int j = rem / NC, c = rem - j * NC;
      if (c0 + j == pos) continue;
      const __half* src = (which ? vb : kb) + (size_t)(c0 + j) * D + c * 8;
      cp_async16((which ? vbuf : kbuf) + buf * BUFB + j * KSTR + c * 16, src);
    }
  };
  // the row of the new position, appended by this item a moment ago, goes into a staged chunk by hand
  auto patch_new_row = [&](int c0, int buf) {
    *reinterpret_cast<__half2*>(kbuf + buf * BUFB + (pos - c0) * KSTR + 4 * tid) =
        *reinterpret_cast<const __half2*>(kb + (size_t)pos * D + 2 * tid);
    *reinterpret_cast<__half2*>(vbuf + buf * BUFB + (pos - c0) * KSTR + 4 * tid) =
        *reinterpret_cast<const __half2*>(vb + (size_t)pos * D + 2 * tid);
  };
  const int cn0 = min(DEC_CH, kend - kbeg);
  if (cn0 > 0) stage(kbeg, cn0, 0);
  if (NB > 1) cp_async_commit();
  if (tid < ROWS) { row_m[tid] = -INFINITY; row_l[tid] = 0.f; }

  if (PDL) asm volatile("griddepcontrol.wait;" ::: "memory");  // q, k_new, v_new come from the kernel before this one

  for (int i = tid; i < ROWS * D; i += ATT_THREADS) {
    const int r = i / D, e = i % D;
    float v = 0.f;
    if (r < nrows) {
      const size_t qoff = ((size_t)bi * a.h + kvh * a.groups + r) * D;
      const float* qr = a.q + qoff;
      // interleaved RoPE at the new position (fusor-ml/fusor/src/composite/rope.rs:77-108)
      float self, other = 0.f;
      if constexpr (LLIO) {
        const float2 pr = ld_ll_pair(a.q_ll + qoff + (e & ~1), a.ep_in, a.status);
        self = (e & 1) ? pr.y : pr.x;
        other = (e & 1) ? pr.x : pr.y;
      } else {
        self = __ldcg(qr + e);
        if (pos >= 0) other = __ldcg(qr + (e ^ 1));
      }
      v = self;
      if (pos >= 0) {
        const float c = a.rope_cos[(size_t)pos * (D / 2) + (e >> 1)];
        const float sn = a.rope_sin[(size_t)pos * (D / 2) + (e >> 1)];
        v = (e & 1) ? __fadd_rn(__fmul_rn(other, sn), __fmul_rn(self, c))
                    : __fsub_rn(__fmul_rn(self, c), __fmul_rn(other, sn));
      }
    }
    qs[r][e] = v;
  }
  const bool has_new = kbeg <= pos && pos < kend;
  if (has_new && tid < D / 2) {
    // append the new position (KvCache::append, fusor-ml/fusor/src/cache/kv_cache.rs:50-62)
    const int p = tid;
    const float* kn = a.k_new + ((size_t)bi * a.hkv + kvh) * D;
    const float* vn = a.v_new + ((size_t)bi * a.hkv + kvh) * D;
    const float c = a.rope_cos[(size_t)pos * (D / 2) + p], sn = a.rope_sin[(size_t)pos * (D / 2) + p];
    float x0, x1, v0, v1;
    if constexpr (LLIO) {
      const size_t koff = ((size_t)bi * a.hkv + kvh) * D + 2 * p;
      const float2 kp = ld_ll_pair(a.k_ll + koff, a.ep_in, a.status);
      const float2 vp = ld_ll_pair(a.v_ll + koff, a.ep_in, a.status);
      x0 = kp.x; x1 = kp.y; v0 = vp.x; v1 = vp.y;
    } else {
      x0 = __ldcg(kn + 2 * p); x1 = __ldcg(kn + 2 * p + 1);
      v0 = __ldcg(vn + 2 * p); v1 = __ldcg(vn + 2 * p + 1);
    }
    const __half2 kh = __floats2half2_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn)),
                                         __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c)));
    const __half2 vh = __floats2half2_rn(v0, v1);
    *reinterpret_cast<__half2*>(kb + (size_t)pos * D + 2 * p) = kh;
    *reinterpret_cast<__half2*>(vb + (size_t)pos * D + 2 * p) = vh;
    if (pos - kbeg < DEC_CH) {
      *reinterpret_cast<__half2*>(kbuf + (pos - kbeg) * KSTR + 4 * p) = kh;
      *reinterpret_cast<__half2*>(vbuf + (pos - kbeg) * KSTR + 4 * p) = vh;
    }
  }

  float o[ROWS][DV];
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int e = 0; e < DV; ++e) o[r][e] = 0.f;

  int buf = 0;
  for (int c0 = kbeg; c0 < kend; c0 += DEC_CH) {
    const int cn = min(DEC_CH, kend - c0);
    if constexpr (NB > 1) {
      // copy the next chunk into the other buffer (everyone has finished with it: it held chunk
      // c0 - DEC_CH), then wait for this chunk only
      const int cnext = c0 + DEC_CH;
      if (c0 > kbeg) dec_sync<BAR>();
      if (cnext < kend) {
        const int cnn = min(DEC_CH, kend - cnext);
        stage(cnext, cnn, buf ^ 1);
        if (has_new && pos >= cnext && pos < cnext + cnn && tid < D / 2) patch_new_row(cnext, buf ^ 1);
        cp_async_commit();
        cp_async_wait_group<1>();
      } else {
        cp_async_wait_group<0>();
      }
    } else {
      if (c0 > kbeg) {
        dec_sync<BAR>();  // the previous chunk has been consumed
        stage(c0, cn, 0);
        if (has_new && pos >= c0 && pos < c0 + cn && tid < D / 2) patch_new_row(c0, 0);
      }
      cp_async_wait_all();
    }
    dec_sync<BAR>();
    const uint8_t* kcur = kbuf + buf * BUFB;
    const uint8_t* vcur = vbuf + buf * BUFB;
    // ---- scores: 4 lanes per key (16-byte chunks sub, sub + 4, ...), 64 keys per CTA pass
    for (int j0 = 0; j0 < cn; j0 += 64) {
      const int j = j0 + warp * 8 + (lane >> 2);
      const int sub = lane & 3;
      float acc[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
      if (j < cn) {
#pragma unroll
        for (int v8 = 0; v8 < NC / 4; ++v8) {
          const int c = v8 * 4 + sub;
          const uint4 raw = *reinterpret_cast<const uint4*>(kcur + j * KSTR + c * 16);
          const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
          float kf[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h2[i]);
            kf[2 * i] = f.x; kf[2 * i + 1] = f.y;
          }
#pragma unroll
          for (int r = 0; r < ROWS; ++r) {
            const float* qr = &qs[r][c * 8];
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
#pragma unroll
        for (int r = 0; r < ROWS; ++r) sc[r][j] = acc[r] * a.scale;
      }
    }
    dec_sync<BAR>();
    // ---- online softmax statistics, warp r owns row r
    if (warp < ROWS) {
      const int r = warp;
      float mx = -INFINITY;
      for (int j = lane; j < cn; j += 32) mx = fmaxf(mx, sc[r][j]);
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o2));
      const float m_old = row_m[r];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int j = lane; j < cn; j += 32) {
        const float p = (m_new == -INFINITY) ? 0.f : __expf(sc[r][j] - m_new);
        sc[r][j] = p;
        sum += p;
      }
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o2);
      if (lane == 0) {
        const float al = (m_old == -INFINITY) ? 0.f : __expf(m_old - m_new);
        alpha[r] = al;
        row_l[r] = row_l[r] * al + sum;
        row_m[r] = m_new;
      }
    }
    dec_sync<BAR>();
    // ---- o = o * alpha + p . v; warp w takes keys w, w + 8, ...; lane owns DV dims
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float al = alpha[r];
#pragma unroll
      for (int e = 0; e < DV; ++e) o[r][e] *= al;
    }
    for (int j = warp; j < cn; j += ATT_THREADS / 32) {
      float vf[DV];
      const uint8_t* vp = vcur + j * KSTR + lane * DV * 2;
      if constexpr (DV == 4) {
        const uint2 raw = *reinterpret_cast<const uint2*>(vp);
        const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
        const float2 f0 = __half22float2(h2[0]), f1 = __half22float2(h2[1]);
        vf[0] = f0.x; vf[1] = f0.y; vf[2] = f1.x; vf[3] = f1.y;
      } else {
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(vp));
        vf[0] = f0.x; vf[1] = f0.y;
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const float p = sc[r][j];
#pragma unroll
        for (int e = 0; e < DV; ++e) o[r][e] = fmaf(p, vf[e], o[r][e]);
      }
    }
    if (NB > 1) buf ^= 1;
  }
  dec_sync<BAR>();  // staging area is free: reuse it for the cross-warp reduction
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int e = 0; e < DV; ++e) ored[warp][r][lane * DV + e] = o[r][e];
  dec_sync<BAR>();
  const size_t rows_all = (size_t)a.b * a.h;
  if (a.nsplit == 1) {
    // a single split: nothing to merge, the normalised rows go straight out (the same arithmetic as
    // the merge below with one partial of weight 1)
    for (int i0 = 0; i0 < nrows * D; i0 += ATT_THREADS) {
      const int i = i0 + tid;
      const bool valid = i < nrows * D;
      const int r = valid ? i / D : 0, e = i % D;
      const size_t grow = (size_t)bi * a.h + kvh * a.groups + r;
      float acc = 0.f;
      if (valid) {
#pragma unroll
        for (int w = 0; w < ATT_THREADS / 32; ++w) acc += ored[w][r][e];
        const float l = row_l[r];
        acc *= l > 0.f ? 1.0f / l : 0.f;
        if (a.out) a.out[grow * D + e] = acc;
      }
      if constexpr (LLIO) {
        if (bi == 0 && valid) emit_ll16(a.out_ll, (int)(grow * D) + e, acc, acc, true, 0xFFFFFFFFu, a.ep_out);
      } else {
        if (a.out_packed.limbs && bi == 0 && valid)
          emit_packed16(a.out_packed, (int)(grow * D) + e, acc, acc, true, 0xFFFFFFFFu);
      }
    }
    return;
  }
  for (int i = tid; i < nrows * D; i += ATT_THREADS) {
    const int r = i / D, e = i % D;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_THREADS / 32; ++w) s += ored[w][r][e];
    const size_t grow = (size_t)bi * a.h + kvh * a.groups + r;
    float* pp = a.part + ((size_t)split * rows_all + grow) * (D + 2);
    pp[e] = s;
    if (e == 0) { pp[D] = row_m[r]; pp[D + 1] = row_l[r]; }
  }
  // ---- the split that arrives last merges all partials of this (batch, kv head) in split order
  __threadfence();
  dec_sync<BAR>();
  if (tid == 0) {
    const int old = atomicAdd(a.done + bi * a.hkv + kvh, 1);
    is_last = (old == a.nsplit - 1);
    if (is_last) a.done[bi * a.hkv + kvh] = 0;
  }
  dec_sync<BAR>();
  if (!is_last) return;
  __threadfence();
  // Merge in split order. Every thread owns one output element (r, e) per pass and needs, for its
  // row, all splits' maxima and normalisers and its own column of all partial rows: all of these
  // loads are issued before the first use, so the merge costs one trip to L2, not one per step.
  // Lane s of a warp holds split s's maximum and normaliser; the weights travel by shuffle.
  constexpr int MAXS = 32;
  for (int i0 = 0; i0 < nrows * D; i0 += ATT_THREADS) {
    const int i = i0 + tid;
    const bool valid = i < nrows * D;
    const int r = valid ? i / D : 0, e = i % D;
    const size_t grow = (size_t)bi * a.h + kvh * a.groups + r;
    float acc = 0.f;
    if (valid) {
      // (a warp's 32 consecutive elements share the row r: D is a multiple of 32)
      const float* base = a.part + grow * (D + 2);
      const size_t sstride = rows_all * (D + 2);
      const float pm = lane < a.nsplit ? __ldcg(base + lane * sstride + D) : -INFINITY;  // lane s: split s
      const float pl = lane < a.nsplit ? __ldcg(base + lane * sstride + D + 1) : 0.f;
      float pv[MAXS];
#pragma unroll
      for (int s0 = 0; s0 < MAXS; ++s0) pv[s0] = s0 < a.nsplit ? __ldcg(base + s0 * sstride + e) : 0.f;
      float mx = pm;
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o2));
      const float wgt = (pm == -INFINITY) ? 0.f : __expf(pm - mx);
      float l = pl * wgt;
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) l += __shfl_xor_sync(0xFFFFFFFFu, l, o2);
#pragma unroll
      for (int s0 = 0; s0 < MAXS; ++s0) acc = fmaf(pv[s0], __shfl_sync(0xFFFFFFFFu, wgt, s0), acc);
      acc *= l > 0.f ? 1.0f / l : 0.f;
      if (a.out) a.out[grow * D + e] = acc;
    }
    // packed rows are single-sequence; nrows * D is a multiple of 32, so `valid` is warp-uniform
    if constexpr (LLIO) {
      if (bi == 0 && valid) emit_ll16(a.out_ll, (int)(grow * D) + e, acc, acc, true, 0xFFFFFFFFu, a.ep_out);
    } else {
      if (a.out_packed.limbs && bi == 0 && valid)
        emit_packed16(a.out_packed, (int)(grow * D) + e, acc, acc, true, 0xFFFFFFFFu);
    }
  }
}

}  // namespace
