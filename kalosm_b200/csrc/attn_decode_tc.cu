// Decode attention (one new position per sequence) on fp16 tensor cores.
//
// Bound: HBM (the fp16 KV cache is read once). Replaces, for single-position queries, the
// reference's flash attention (fusor-ml/fusor/src/composite/flash_attention.rs:113-236: softmax(q k^T
// scale) v, each KV head shared by `groups` query heads) together with the interleaved RoPE of q
// and k (fusor-ml/fusor/src/composite/rope.rs:77-108) and the cache append
// (fusor-ml/fusor/src/cache/kv_cache.rs:50-62) that precede it in the decoder
// (models/kalosm-llama/src/raw/attention_layer.rs).
//
// One CTA (4 warps) = one (sequence, KV head, split of the context). The `groups` query heads that
// share the KV head are the rows of one m16 MMA tile (rows beyond `groups` are zero), so the cache
// is read once for all of them. Keys and values stream through a ring of three XOR-swizzled
// shared-memory tiles of 64 keys filled with 16-byte cp.async (two tiles in flight while one is
// used, two CTAs per SM); warp w owns keys 16 w .. 16 w + 15
// of every tile: S = Q K^T (2 column tiles x D / 16 steps of mma.sync.m16n8k16), online softmax in
// the exp2 domain on the accumulator fragments, O += P V with P rounded to fp16 and V through the
// transposing ldmatrix. The four warps' (max, sum, O) meet in shared memory at the end; with
// several splits the partial rows go to global memory and the split that arrives last merges them
// in split order (arrival counter per (sequence, KV head)), so results do not depend on timing.
// The split that holds the new position rotates and appends k / v and patches the row into its
// staged tile by hand (the cache row is not yet visible to the asynchronous copies).
#include "attn_decode.cuh"
#include "attn_mma.cuh"

namespace {

constexpr int TC_KEYS = 64;      // keys per staged tile
constexpr int TC_THREADS = 128;  // 4 warps x 16 keys
constexpr int TC_ROWS = 16;      // query rows of the MMA tile (groups <= 16)
constexpr int TC_MAXS = 32;      // splits merged by one pass of loads
constexpr int TC_STAGES = 3;     // staged tiles (two CTAs per SM: 2 x 96 KB of keys and values for head size 128)

template <int N>
__device__ __forceinline__ void tc_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// PDL: launched with programmatic stream serialization; everything that does not depend on the
// kernel before (the position, the cached keys and values of earlier positions) is requested
// before griddepcontrol.wait, q and the new k / v after it.
template <int D, bool PDL>
__global__ void __launch_bounds__(TC_THREADS, 2)
attn_decode_tc_kernel(const fb200_dec_args a0) {
  constexpr int CH = D / 8;             // 16-byte chunks per row
  constexpr int TILE = TC_KEYS * D * 2;  // bytes of one K or V tile
  extern __shared__ __align__(128) uint8_t sm[];
  uint8_t* KV = sm;                      // [TC_STAGES][K | V]
  uint8_t* Qs = sm + TC_STAGES * 2 * TILE;  // [16][D] fp16
  __shared__ float wm[4][TC_ROWS], wl[4][TC_ROWS];
  __shared__ int is_last;

  // The launch provides nsplit splits per (sequence, KV head) for the longest context; a short
  // context uses the first few of them (at least min_keys keys each), the other CTAs have nothing to do.
  fb200_dec_args a = a0;
  const int pos = a.pos_dev ? __ldcg(a.pos_dev) : -1;
  const int skv = a.pos_dev ? pos + 1 : a.skv;
  // CTAs are numbered split-major, so that the splits in use are the first CTAs to start.
  const int pairs = a.b * a.hkv;
  const int split = (int)blockIdx.x / pairs;
  {
    const int mk = a.min_keys > 0 ? a.min_keys : 64;
    const int ns = max(1, min(a.nsplit, (skv + mk - 1) / mk));
    if (split >= ns) return;
    a.nsplit = ns;
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int kvh = ((int)blockIdx.x % pairs) % a.hkv, bi = ((int)blockIdx.x % pairs) / a.hkv;
  const int per = (skv + a.nsplit - 1) / a.nsplit;
  const int kbeg = min(skv, split * per), kend = min(skv, kbeg + per);
  const int ntiles = (kend - kbeg + TC_KEYS - 1) / TC_KEYS;
  const bool has_new = pos >= 0 && kbeg <= pos && pos < kend;
  const int skip = has_new ? pos : -1;  // the cache row that this CTA writes itself
  __half* kb = a.kc + ((size_t)bi * a.hkv + kvh) * (size_t)a.cap * D;
  __half* vb = a.vc + ((size_t)bi * a.hkv + kvh) * (size_t)a.cap * D;
  const float scale_log2 = a.scale * 1.4426950408889634f;

  auto load_tile = [&](int tile, int buf) {
    const int kt = kbeg + tile * TC_KEYS;
    const uint32_t kdst = pf_smem(KV + buf * 2 * TILE), vdst = kdst + TILE;
#pragma unroll
    for (int i = 0; i < TC_KEYS * CH / TC_THREADS; ++i) {
      const int idx = tid + TC_THREADS * i, row = idx / CH, c = idx % CH;
      if (kt + row == skip) continue;
      const bool valid = kt + row < kend;
      const size_t src = (size_t)(valid ? kt + row : 0) * D + c * 8;
      pf_cp16(kdst + pf_off<D>(row, c), kb + src, valid);
      pf_cp16(vdst + pf_off<D>(row, c), vb + src, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // one commit group per tile slot, empty beyond the last tile, so that the group count is uniform
  auto fetch = [&](int tile) {
    if (tile < ntiles) load_tile(tile, tile % TC_STAGES);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int i = 0; i < TC_STAGES - 1; ++i) fetch(i);
  if (PDL) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }

  // ---- the new position: rotate k, append k and v (fp16), keep the pair for the staged tile
  uint32_t knew = 0u, vnew = 0u;
  if (has_new && tid < D / 2) {
    const int p = tid;
    const float* kn = a.k_new + ((size_t)bi * a.hkv + kvh) * D;
    const float* vn = a.v_new + ((size_t)bi * a.hkv + kvh) * D;
    const float2 kx = __ldcg(reinterpret_cast<const float2*>(kn) + p), vx = __ldcg(reinterpret_cast<const float2*>(vn) + p);
    const float c = a.rope_cos[(size_t)pos * (D / 2) + p], sn = a.rope_sin[(size_t)pos * (D / 2) + p];
    knew = pf_pack(__fsub_rn(__fmul_rn(kx.x, c), __fmul_rn(kx.y, sn)), __fadd_rn(__fmul_rn(kx.x, sn), __fmul_rn(kx.y, c)));
    vnew = pf_pack(vx.x, vx.y);
    *reinterpret_cast<uint32_t*>(kb + (size_t)pos * D + 2 * p) = knew;
    *reinterpret_cast<uint32_t*>(vb + (size_t)pos * D + 2 * p) = vnew;
  }
  // ---- q rows of the group: interleaved RoPE at the new position, fp16, swizzled rows (rows
  // beyond `groups` are zero); every load is issued before the first use
  {
    constexpr int NQ = TC_ROWS * (D / 2) / TC_THREADS;
    float2 qx[NQ], cs[NQ];
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
      const int idx = tid + TC_THREADS * i, r = idx / (D / 2), p = idx % (D / 2);
      qx[i] = make_float2(0.f, 0.f);
      cs[i] = make_float2(1.f, 0.f);
      if (r < a.groups) {
        qx[i] = __ldcg(reinterpret_cast<const float2*>(a.q + ((size_t)bi * a.h + kvh * a.groups + r) * D) + p);
        if (pos >= 0) cs[i] = make_float2(a.rope_cos[(size_t)pos * (D / 2) + p], a.rope_sin[(size_t)pos * (D / 2) + p]);
      }
    }
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
      const int idx = tid + TC_THREADS * i, r = idx / (D / 2), p = idx % (D / 2);
      float y0 = qx[i].x, y1 = qx[i].y;
      if (pos >= 0 && r < a.groups) {
        y0 = __fsub_rn(__fmul_rn(qx[i].x, cs[i].x), __fmul_rn(qx[i].y, cs[i].y));
        y1 = __fadd_rn(__fmul_rn(qx[i].x, cs[i].y), __fmul_rn(qx[i].y, cs[i].x));
      }
      *reinterpret_cast<uint32_t*>(Qs + pf_off<D>(r, p >> 2) + (p & 3) * 4) = pf_pack(y0, y1);
    }
  }
  auto patch_new_row = [&](int tile) {
    const int row = pos - (kbeg + tile * TC_KEYS);
    if (!has_new || row < 0 || row >= TC_KEYS || tid >= D / 2) return;
    uint8_t* kdst = KV + (tile % TC_STAGES) * 2 * TILE;
    *reinterpret_cast<uint32_t*>(kdst + pf_off<D>(row, tid >> 2) + (tid & 3) * 4) = knew;
    *reinterpret_cast<uint32_t*>(kdst + TILE + pf_off<D>(row, tid >> 2) + (tid & 3) * 4) = vnew;
  };
#pragma unroll
  for (int i = 0; i < TC_STAGES - 1; ++i) patch_new_row(i);
  __syncthreads();
  uint32_t qf[D / 16][4];
  {
    const int j = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) pf_ldsm4(pf_smem(Qs) + pf_off<D>((j & 1) * 8 + r, 2 * ks + (j >> 1)), qf[ks]);
  }

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  for (int tile = 0; tile < ntiles; ++tile) {
    const int buf = tile % TC_STAGES;
    // the slot of tile - 1 is free (every warp passed the barrier that ended it): the tile after the ones in flight goes there
    fetch(tile + TC_STAGES - 1);
    patch_new_row(tile + TC_STAGES - 1);
    tc_wait_group<TC_STAGES - 1>();  // this thread's part of tile `tile` has landed
    __syncthreads();
    const int k0 = kbeg + tile * TC_KEYS + warp * 16;  // first key of this warp in the tile
    if (k0 < kend) {
      const uint32_t ks_base = pf_smem(KV + buf * 2 * TILE), vs_base = ks_base + TILE;
      // ---- S = Q K^T for this warp's 16 keys
      float s[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int k2 = 0; k2 < D / 32; ++k2) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          uint32_t b[4];
          pf_ldsm4(ks_base + pf_off<D>(warp * 16 + nt * 8 + (lane & 7), 4 * k2 + (lane >> 3)), b);
          pf_mma(s[nt], qf[2 * k2], b[0], b[1]);
          pf_mma(s[nt], qf[2 * k2 + 1], b[2], b[3]);
        }
      }
      // ---- online softmax (exp2 domain; the positive scale is folded into the exponent)
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (k0 + nt * 8 + 2 * t + (e & 1) >= kend) s[nt][e] = -INFINITY;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
        }
      float alpha[2], msafe[2];
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        mx[hrow] = fmaxf(mx[hrow], __shfl_xor_sync(0xFFFFFFFFu, mx[hrow], 1));
        mx[hrow] = fmaxf(mx[hrow], __shfl_xor_sync(0xFFFFFFFFu, mx[hrow], 2));
        const float mnew = fmaxf(m_run[hrow], mx[hrow] * scale_log2);
        msafe[hrow] = mnew == -INFINITY ? 0.f : mnew;
        alpha[hrow] = exp2f(m_run[hrow] - msafe[hrow]);
        m_run[hrow] = mnew;
      }
      float psum[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = exp2f(fmaf(s[nt][e], scale_log2, -msafe[e >> 1]));
          s[nt][e] = p;
          psum[e >> 1] += p;
        }
      l_run[0] = l_run[0] * alpha[0] + psum[0];
      l_run[1] = l_run[1] * alpha[1] + psum[1];
      if (__any_sync(0xFFFFFFFFu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
          o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
      }
      // ---- O += P V: P (fp16) as the A operand of one k16 step, V through transposing ldmatrix
      uint32_t pa[4];
      pa[0] = pf_pack(s[0][0], s[0][1]);
      pa[1] = pf_pack(s[0][2], s[0][3]);
      pa[2] = pf_pack(s[1][0], s[1][1]);
      pa[3] = pf_pack(s[1][2], s[1][3]);
      const int j = lane >> 3, r = lane & 7;
#pragma unroll
      for (int d2 = 0; d2 < D / 16; ++d2) {
        uint32_t b[4];
        pf_ldsm4_t(vs_base + pf_off<D>(warp * 16 + (j & 1) * 8 + r, 2 * d2 + (j >> 1)), b);
        pf_mma(o[2 * d2], pa, b[0], b[1]);
        pf_mma(o[2 * d2 + 1], pa, b[2], b[3]);
      }
    }
    __syncthreads();  // every warp is done with this slot before a later tile lands in it
  }

  // ---- the four warps' (max, sum, O) meet in shared memory (the staging area is free now)
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    l_run[hrow] += __shfl_xor_sync(0xFFFFFFFFu, l_run[hrow], 1);
    l_run[hrow] += __shfl_xor_sync(0xFFFFFFFFu, l_run[hrow], 2);
  }
  float (*ow)[TC_ROWS][D] = reinterpret_cast<float (*)[TC_ROWS][D]>(sm);  // [4 warps][16][D]
  static_assert(4 * TC_ROWS * D * 4 <= TC_STAGES * 2 * TILE, "the warps' output rows must fit the staging area");
  if (t == 0) {
    wm[warp][g] = m_run[0]; wm[warp][g + 8] = m_run[1];
    wl[warp][g] = l_run[0]; wl[warp][g + 8] = l_run[1];
  }
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    *reinterpret_cast<float2*>(&ow[warp][g][i * 8 + 2 * t]) = make_float2(o[i][0], o[i][1]);
    *reinterpret_cast<float2*>(&ow[warp][g + 8][i * 8 + 2 * t]) = make_float2(o[i][2], o[i][3]);
  }
  __syncthreads();
  const size_t rows_all = (size_t)a.b * a.h;
  const float ln2 = 0.6931471805599453f;
  for (int idx = tid; idx < a.groups * D; idx += TC_THREADS) {
    const int r = idx / D, e = idx % D;
    float m = fmaxf(fmaxf(wm[0][r], wm[1][r]), fmaxf(wm[2][r], wm[3][r]));
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float wgt = wm[w][r] == -INFINITY ? 0.f : exp2f(wm[w][r] - m);
      l = fmaf(wl[w][r], wgt, l);
      acc = fmaf(ow[w][r][e], wgt, acc);
    }
    const size_t grow = (size_t)bi * a.h + kvh * a.groups + r;
    if (a.nsplit == 1) {
      a.out[grow * D + e] = acc * (l > 0.f ? 1.0f / l : 0.f);
    } else {
      // partial row of this split: unnormalised sum, maximum (natural-log domain) and normaliser
      float* pp = a.part + ((size_t)split * rows_all + grow) * (D + 2);
      pp[e] = acc;
      if (e == 0) { pp[D] = m == -INFINITY ? -INFINITY : m * ln2; pp[D + 1] = l; }
    }
  }
  if (a.nsplit == 1) return;
  // ---- the split that arrives last merges all partials of this (sequence, KV head) in split order
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(a.done + bi * a.hkv + kvh, 1);
    is_last = (old == a.nsplit - 1);
    if (is_last) a.done[bi * a.hkv + kvh] = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int idx = tid; idx < a.groups * D; idx += TC_THREADS) {
    const int r = idx / D, e = idx % D;
    const size_t grow = (size_t)bi * a.h + kvh * a.groups + r;
    const float* base = a.part + grow * (D + 2);
    const size_t sstride = rows_all * (D + 2);
    // (a warp's 32 consecutive elements share the row r: D is a multiple of 32.) Lane s holds split
    // s's maximum and normaliser, the weights travel by shuffle; all loads are issued before the
    // first use, so the merge costs one trip to L2.
    const float pm = lane < a.nsplit ? __ldcg(base + lane * sstride + D) : -INFINITY;
    const float pl = lane < a.nsplit ? __ldcg(base + lane * sstride + D + 1) : 0.f;
    float pv[TC_MAXS];
#pragma unroll
    for (int s0 = 0; s0 < TC_MAXS; ++s0) pv[s0] = s0 < a.nsplit ? __ldcg(base + s0 * sstride + e) : 0.f;
    float mx = pm;
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o2));
    const float wgt = pm == -INFINITY ? 0.f : __expf(pm - mx);
    float l = pl * wgt;
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) l += __shfl_xor_sync(0xFFFFFFFFu, l, o2);
    float acc = 0.f;
#pragma unroll
    for (int s0 = 0; s0 < TC_MAXS; ++s0) acc = fmaf(pv[s0], __shfl_sync(0xFFFFFFFFu, wgt, s0), acc);
    a.out[grow * D + e] = acc * (l > 0.f ? 1.0f / l : 0.f);
  }
}

}  // namespace

// Launches the tensor-core decode attention for prepared arguments (a.done must point to b * hkv
// zeroed arrival counters; the kernel leaves them zero again). Returns 1 when the head layout is
// not covered (the caller then runs the general decode kernel).
int fb200_launch_attention_decode_tc(fb200_device* dev, const fb200_dec_args& a, int d) {
  if (a.h % a.hkv || a.groups > TC_ROWS || (d != 64 && d != 128) || a.nsplit < 1 || a.nsplit > TC_MAXS || !a.out ||
      !(a.scale > 0.f))
    return 1;
  const unsigned grid = (unsigned)(a.b * a.hkv * a.nsplit);
  const size_t smem = (size_t)(TC_STAGES * 2 * TC_KEYS + TC_ROWS) * d * 2;
  static bool configured[64] = {false};
  // with a device-resident position the kernel is part of a decode step: its predecessor produced q, k, v
  const bool pdl = a.pos_dev != nullptr;
  if (!configured[dev->ordinal & 63]) {
    const int bytes128 = (TC_STAGES * 2 * TC_KEYS + TC_ROWS) * 128 * 2, bytes64 = (TC_STAGES * 2 * TC_KEYS + TC_ROWS) * 64 * 2;
    FB_CUDA(dev, cudaFuncSetAttribute(attn_decode_tc_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes128));
    FB_CUDA(dev, cudaFuncSetAttribute(attn_decode_tc_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes128));
    FB_CUDA(dev, cudaFuncSetAttribute(attn_decode_tc_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes64));
    FB_CUDA(dev, cudaFuncSetAttribute(attn_decode_tc_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes64));
    configured[dev->ordinal & 63] = true;
  }
  if (d == 128 && pdl) return fb200_launch(dev, attn_decode_tc_kernel<128, true>, dim3(grid), dim3(TC_THREADS), smem, true, a);
  if (d == 128) return fb200_launch(dev, attn_decode_tc_kernel<128, false>, dim3(grid), dim3(TC_THREADS), smem, false, a);
  if (pdl) return fb200_launch(dev, attn_decode_tc_kernel<64, true>, dim3(grid), dim3(TC_THREADS), smem, true, a);
  return fb200_launch(dev, attn_decode_tc_kernel<64, false>, dim3(grid), dim3(TC_THREADS), smem, false, a);
}
