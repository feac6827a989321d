// Prefill attention (many query positions, no mask or causal, head size 128) on the 5th-generation
// tensor cores: both products of the attention run as tcgen05.mma with their results in tensor
// memory (TMEM).
//
// Bound: tensor cores; causal-effective flops 2 Sq (Sq + 1 + 2 (Skv - Sq)) D H per sequence.
// Replaces the reference's flash attention row program for Sq > 1
// (fusor-ml/tile-ir-kernels/src/kernels/row_program.rs:1210-1382; the math is
// fusor-ml/fusor/src/composite/flash_attention.rs:113-236: softmax(q k^T scale + mask) v with
// each KV head shared by `groups` query heads).
//
// One CTA = 128 query rows of one head: 128 softmax threads (thread r owns query row r, which is
// also lane r of the CTA's TMEM columns, so the softmax statistics of a row never leave a thread)
// one warp whose first lane issues the MMAs and one whose first lane requests the K and V tiles
// (TMA). The roles meet only at mbarriers (tile landed: the copy's byte count; P written: 128
// arrivals; product done: tcgen05.commit); there is no CTA-wide barrier in the loop, and neither
// the issue latency of the MMAs nor the copies are on the softmax threads' path.
// Per tile t of 64 keys:
//   S_t = Q K_t^T   8 tcgen05.mma (M = 128 queries, N = 64 keys, K = 16 of the head size) into one of
//                   two S buffers in TMEM; it is issued one tile ahead, so it runs while the threads
//                   work on the softmax of tile t - 1,
//   softmax         every thread reads its row of S_t with tcgen05.ld, applies the mask, the
//                   running maximum and sum (exp2 domain, the scale folded into the exponent),
//                   writes P as fp16 pairs back into TMEM (tcgen05.st, over the S buffer it read),
//   O += P V_t      4 tcgen05.mma (M = 128, N = 128 dims, K = 16 keys; A = P from TMEM, V is read
//                   MN-major from shared memory, as it lies in the cache) accumulating in TMEM
//                   across the tiles.
// The exponentials use a reference maximum that follows the true running maximum lazily: O (in
// TMEM) and the running sum are rescaled only when the maximum has grown by more than 2^8 since
// the last rescale (a warp-uniform decision; tcgen05.ld, multiply, tcgen05.st), so P stays below
// 256 (exact range of fp16) and most tiles never touch O outside the MMA.
// Q sits in shared memory in the canonical core-matrix layout of the MMA without swizzle (8 rows x
// 16 bytes per core matrix, written by the softmax threads). K and V tiles come by tensor TMA
// (cp.async.bulk.tensor, two boxes of 64 keys x 64 dims per tile, 128-byte swizzle; rows past the
// valid length are outside the tensor map and arrive as zeros), two tiles ahead, and are read by
// the MMA through 128-byte-swizzle descriptors: K as a K-major operand, V as an MN-major one, as
// it lies in the cache. Two CTAs share an SM (112 KB of shared memory and 256 TMEM columns each). Tiles above the diagonal are never visited; CTAs with the longest key range
// start first.
// Every mbarrier wait is bounded: a wait that gives up sets the device status word and a flag in
// shared memory, every later wait of the CTA then returns at once, the CTA runs through its loop
// without waiting (results invalid, nothing stored), frees its TMEM columns and exits.
#include <cuda.h>

#include "attn_mma.cuh"
#include "qgemv_common.cuh"

namespace {

constexpr int XQ = 128, XK = 64, XD = 128, X_THREADS = 128;  // X_THREADS: the softmax threads (one per query row)
constexpr int X_BLOCK = X_THREADS + 64;                       // + the MMA issuer's warp + the copy requester's warp
constexpr int X_Q_BYTES = XQ * XD * 2;   // 32 KB
constexpr int X_KV_BYTES = XK * XD * 2;  // 16 KB per K or V tile
constexpr int X_TAIL = 256;              // barriers, TMEM slot, give-up flag
constexpr int X_KBUFS = 3, X_VBUFS = 2;   // K tiles are requested three tiles ahead, V tiles two
constexpr int X_SMEM = X_Q_BYTES + (X_KBUFS + X_VBUFS) * X_KV_BYTES + X_TAIL;
constexpr int X_TMEM_COLS = 256;         // S buffers: columns 0..63 and 64..127; O: columns 128..255
constexpr float X_RESCALE = 8.0f;        // log2 of the growth of a row maximum that triggers a rescale of O

struct XArgs {
  const float* q;      // [B, H, Sq, D] or [B, Sq, H, D]
  const __half* k;     // [B, Hkv, cap, D]
  const __half* v;
  float* out;          // same layout as q
  const int* skv_dev;  // if not null: valid keys = *skv_dev + sq
  int b, h, hkv, sq, skv, cap, groups, bshd, causal;
  float scale_log2;    // scale * log2(e)
  int k_lbo, v_lbo, v_sbo;  // descriptor strides (bytes) of the swizzled operands
  int* status;
};
// descriptor strides (bytes) of the swizzled operands, and the layout code of the 128-byte swizzle
constexpr uint32_t X_SW128 = 2;
constexpr uint32_t X_BOX_BYTES = XK * 64 * 2;  // one TMA box: 64 keys x 64 dims of fp16 = 8 KB

__device__ __forceinline__ bool x_wait(uint32_t bar, uint32_t parity, volatile int* dead, int* status) {
  for (int it = 0; it < (1 << 22); ++it) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((it & 255) == 255 && *dead) return false;
  }
  *dead = 1;
  if (status) atomicExch(status, FB200_ERR_TIMEOUT);
  return false;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Shared-memory matrix descriptor without swizzle: start address, leading and stride byte offsets
// in 16-byte units, descriptor version 1.
__device__ __forceinline__ uint64_t x_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout = 0) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46) |
         ((uint64_t)layout << 61);
}
// One box of a 3-D tensor map (dims, keys, sequence x KV head) into shared memory; completion is
// counted in bytes on the mbarrier.
__device__ __forceinline__ void x_tma_box(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
__device__ __forceinline__ void x_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the A operand in tensor memory (row i of A in lane i, two fp16 values per column)
__device__ __forceinline__ void x_mma_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void x_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void x_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void x_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
// 2^x, flushing denormals (2^-inf = 0)
__device__ __forceinline__ float x_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Byte offset of the 16-byte chunk `chunk` (8 K elements) of row `row` in a K-major operand whose K
// extent is `kchunks` chunks: core matrices of a row group side by side along K, row groups behind.
__device__ __forceinline__ uint32_t x_kmajor(int row, int chunk, int kchunks) {
  return (uint32_t)((row >> 3) * (kchunks * 128) + chunk * 128 + (row & 7) * 16);
}

__global__ void __launch_bounds__(X_BLOCK, 2)
attn_prefill_tc_kernel(const XArgs a, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
  extern __shared__ __align__(1024) uint8_t sm[];  // the swizzled tiles need 1024-byte alignment (checked below)
  uint8_t* Qs = sm;
  uint8_t* Ks = sm + X_Q_BYTES;                        // [X_KBUFS][2 boxes]
  uint8_t* Vs = Ks + X_KBUFS * X_KV_BYTES;             // [X_VBUFS][2 boxes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(Vs + X_VBUFS * X_KV_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // bar_s[2]: S_t complete (one per S buffer); bar_o: O += P V_t complete; bar_kfull[3], bar_vfull[2]: tile
  // landed (byte count of its two boxes); bar_pfull: P written (128 arrivals)
  const uint32_t bar_s = smem_u32(bars), bar_o = smem_u32(bars + 2), bar_kfull = smem_u32(bars + 3),
                 bar_vfull = smem_u32(bars + 6), bar_pfull = smem_u32(bars + 8);

  const int qt = gridDim.x - 1 - blockIdx.x;  // longest key ranges first
  const int head = blockIdx.y, bi = blockIdx.z, kvh = head / a.groups;
  const int skv = a.skv_dev ? (*a.skv_dev + a.sq) : a.skv;
  const int off = skv - a.sq;  // query i sees keys j <= i + off
  const int q0 = qt * XQ;
  const int kmax = max(0, a.causal ? min(skv, q0 + XQ + off) : skv);
  const int ntiles = (kmax + XK - 1) / XK;
  const size_t q_row = a.bshd ? (size_t)a.h * XD : (size_t)XD;
  const size_t q_base = (size_t)bi * a.h * a.sq * XD + (a.bshd ? (size_t)head * XD : (size_t)head * a.sq * XD);
  const int plane = bi * a.hkv + kvh;  // third coordinate of the tensor maps

  if (tid == 0) {
    *dead = 0;
    if (smem_u32(sm) & 1023u) {  // never seen; the MMA would read the tiles with the wrong swizzle phase
      *dead = 1;
      atomicExch(a.status, FB200_ERR_TIMEOUT);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 8, 1);
    mbar_init(bar_o, 1);
    for (int i = 0; i < X_KBUFS; ++i) mbar_init(bar_kfull + 8 * i, 1);
    for (int i = 0; i < X_VBUFS; ++i) mbar_init(bar_vfull + 8 * i, 1);
    mbar_init(bar_pfull, X_THREADS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(X_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // Q tile: f32 -> fp16 into the K-major operand layout (rows past Sq are zero), by the softmax threads
  if (warp < X_THREADS / 32) {
    for (int id = warp; id < (XQ / 8) * (XD / 32); id += X_THREADS / 32) {
      const int row = (id >> 2) * 8 + (lane & 7), c = (id & 3) * 4 + (lane >> 3);
      float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0;
      if (q0 + row < a.sq) {
        const float4* src = reinterpret_cast<const float4*>(a.q + q_base + (size_t)(q0 + row) * q_row + c * 8);
        x0 = src[0];
        x1 = src[1];
      }
      *reinterpret_cast<uint4*>(Qs + x_kmajor(row, c, XD / 8)) =
          make_uint4(pf_pack(x0.x, x0.y), pf_pack(x0.z, x0.w), pf_pack(x1.x, x1.y), pf_pack(x1.z, x1.w));
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these stores -> tensor-core reads
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();  // barriers initialised, TMEM columns allocated, Q staged
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  // instruction descriptors: fp32 accumulator, fp16 operands, M = 128; S: N = 64, both K-major; O: N = 128, B MN-major
  constexpr uint32_t IDESC_S = (1u << 4) | ((uint32_t)(XK >> 3) << 17) | ((uint32_t)(XQ >> 4) << 24);
  constexpr uint32_t IDESC_O = (1u << 4) | (1u << 16) | ((uint32_t)(XD >> 3) << 17) | ((uint32_t)(XQ >> 4) << 24);

  if (warp == X_THREADS / 32 + 1) {
    // ---- copy requester: K0..K2, V0, V1, then K(t+3) when S_t has completed and V(t+2) when
    // O += P V_t has. A tile is two boxes (dims 0..63 and 64..127) of 64 keys.
    if (lane == 0 && ntiles > 0) {
      auto fetch = [&](const CUtensorMap* map, int tile, uint32_t dst, uint32_t bar) {
        mbar_expect_tx(bar, 2 * X_BOX_BYTES);
        x_tma_box(dst, map, 0, tile * XK, plane, bar);
        x_tma_box(dst + X_BOX_BYTES, map, 64, tile * XK, plane, bar);
      };
      const uint32_t k0 = pf_smem(Ks), v0 = pf_smem(Vs);
      for (int t = 0; t < X_KBUFS && t < ntiles; ++t) fetch(&kmap, t, k0 + t * X_KV_BYTES, bar_kfull + 8 * t);
      for (int t = 0; t < X_VBUFS && t < ntiles; ++t) fetch(&vmap, t, v0 + t * X_KV_BYTES, bar_vfull + 8 * t);
      for (int tile = 0; tile + X_VBUFS < ntiles; ++tile) {
        x_wait(bar_s + 8 * (tile & 1), (uint32_t)((tile >> 1) & 1), dead, a.status);  // K buffer of tile t is free
        if (tile + X_KBUFS < ntiles)
          fetch(&kmap, tile + X_KBUFS, k0 + (tile % X_KBUFS) * X_KV_BYTES, bar_kfull + 8 * (tile % X_KBUFS));
        x_wait(bar_o, (uint32_t)(tile & 1), dead, a.status);  // V buffer of tile t is free
        fetch(&vmap, tile + X_VBUFS, v0 + (tile % X_VBUFS) * X_KV_BYTES, bar_vfull + 8 * (tile % X_VBUFS));
      }
    }
  } else if (warp == X_THREADS / 32) {
    // ---- MMA issuer: S_0, then per tile S_(t+1) (runs under the softmax of tile t) and O += P V_t
    if (lane == 0 && ntiles > 0) {
      auto issue_s = [&](int tile) {  // S buffer tile & 1 = Q . K_tile^T
        x_wait(bar_kfull + 8 * (tile % X_KBUFS), (uint32_t)((tile / X_KBUFS) & 1), dead, a.status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t ks = pf_smem(Ks + (tile % X_KBUFS) * X_KV_BYTES);
#pragma unroll
        for (int s = 0; s < XD / 16; ++s)  // k-step s: box s / 4, 32 bytes further inside the 128-byte rows per step
          x_mma(tmem + (uint32_t)((tile & 1) * XK), x_desc(pf_smem(Qs) + s * 256, 128, (XD / 8) * 128),
                x_desc(ks + (s >> 2) * X_BOX_BYTES + (s & 3) * 32, (uint32_t)a.k_lbo, 1024, X_SW128), IDESC_S, s ? 1u : 0u);
        x_commit(bar_s + 8 * (tile & 1));
      };
      issue_s(0);
      for (int tile = 0; tile < ntiles; ++tile) {
        if (tile + 1 < ntiles) issue_s(tile + 1);
        x_wait(bar_pfull, (uint32_t)(tile & 1), dead, a.status);
        x_wait(bar_vfull + 8 * (tile % X_VBUFS), (uint32_t)((tile / X_VBUFS) & 1), dead, a.status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t vs = pf_smem(Vs + (tile % X_VBUFS) * X_KV_BYTES);
#pragma unroll
        for (int s = 0; s < XK / 16; ++s)  // k-step s: 16 keys = 16 rows of 128 bytes further
          x_mma_ta(tmem + 2 * XK, tmem + (uint32_t)((tile & 1) * XK + s * 8),
                   x_desc(vs + s * 2048, (uint32_t)a.v_lbo, (uint32_t)a.v_sbo, X_SW128), IDESC_O, (tile | s) ? 1u : 0u);
        x_commit(bar_o);
      }
    }
  } else {
    // ---- softmax threads
    const uint32_t tmem_lane = tmem + ((uint32_t)(32 * warp) << 16);  // this warp's 32 lanes
    float m_ref = -INFINITY;  // the maximum the exponentials and O currently refer to (scaled, log2 domain)
    float l_run = 0.f;
    const int row = q0 + tid;

    for (int tile = 0; tile < ntiles; ++tile) {
      const int sb = tile & 1;
      x_wait(bar_s + 8 * sb, (uint32_t)((tile >> 1) & 1), dead, a.status);  // S_t is there
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

      // ---- this thread's row of S: mask, running maximum and sum
      const int kt = tile * XK;
      uint32_t sv[2][32];
      x_ld32(tmem_lane + (uint32_t)(sb * XK), sv[0]);
      x_ld32(tmem_lane + (uint32_t)(sb * XK + 32), sv[1]);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (kt + XK > skv || (a.causal && kt + XK - 1 > q0 + off)) {  // only tiles that touch the diagonal or the end
#pragma unroll
        for (int j = 0; j < XK; ++j) {
          const int col = kt + j;
          if (col >= skv || (a.causal && col > row + off)) sv[j >> 5][j & 31] = 0xFF800000u;  // -inf
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < XK; ++j) mx = fmaxf(mx, __uint_as_float(sv[j >> 5][j & 31]));
      const float m_new = fmaxf(m_ref, mx * a.scale_log2);
      // follow the maximum lazily: rescale when it has outgrown the reference by more than 2^X_RESCALE
      const bool grow = m_new > m_ref + X_RESCALE;  // also true for the first finite maximum (m_ref = -inf)
      const float alpha = grow ? x_ex2(m_ref - m_new) : 1.0f;  // 2^-inf = 0 for a row that had no key yet
      if (grow) m_ref = m_new;
      const float msafe = m_ref == -INFINITY ? 0.f : m_ref;
      float psum = 0.f;
      uint32_t pk[XK / 2];  // P as fp16 pairs: column j of the A operand holds keys 2 j, 2 j + 1
#pragma unroll
      for (int j = 0; j < XK / 2; ++j) {
        const float p0 = x_ex2(fmaf(__uint_as_float(sv[(2 * j) >> 5][(2 * j) & 31]), a.scale_log2, -msafe));
        const float p1 = x_ex2(fmaf(__uint_as_float(sv[(2 * j + 1) >> 5][(2 * j + 1) & 31]), a.scale_log2, -msafe));
        psum += p0 + p1;
        pk[j] = pf_pack(p0, p1);
      }
      l_run = l_run * alpha + psum;
      // P goes into the first half of the S buffer it came from (this thread's lane only; the next
      // product into that buffer, S_(t+2), is issued behind O += P V_t)
      x_st32(tmem_lane + (uint32_t)(sb * XK), pk);

      // ---- O is rescaled only after the previous tile's O += P V has completed
      if (tile > 0 && __any_sync(0xFFFFFFFFu, grow)) {
        x_wait(bar_o, (uint32_t)((tile - 1) & 1), dead, a.status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int c = 0; c < XD / 32; ++c) {
          uint32_t ov[32];
          x_ld32(tmem_lane + 2 * XK + 32 * c, ov);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          x_st32(tmem_lane + 2 * XK + 32 * c, ov);
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(bar_pfull);  // phase t
    }

    // ---- the last product, then normalise and store (nothing is stored after a wait has given up)
    if (ntiles > 0) {
      x_wait(bar_o, (uint32_t)((ntiles - 1) & 1), dead, a.status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    const bool store = row < a.sq && !*dead;
    const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
    float4* dst = reinterpret_cast<float4*>(a.out + q_base + (size_t)row * q_row);
#pragma unroll
    for (int c = 0; c < XD / 32; ++c) {
      uint32_t ov[32];
      if (ntiles > 0) {
        x_ld32(tmem_lane + 2 * XK + 32 * c, ov);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) ov[i] = 0u;
      }
      if (store) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          dst[8 * c + i] = make_float4(__uint_as_float(ov[4 * i]) * inv, __uint_as_float(ov[4 * i + 1]) * inv,
                                       __uint_as_float(ov[4 * i + 2]) * inv, __uint_as_float(ov[4 * i + 3]) * inv);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(X_TMEM_COLS) : "memory");
}

// cuTensorMapEncodeTiled of the driver, looked up once (the library does not link against libcuda)
typedef CUresult (*x_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
x_encode_fn x_encoder() {
  static x_encode_fn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<x_encode_fn>(p);
  }();
  return fn;
}
// fp16 cache [planes][cap][128] seen as (dims, keys, planes) with `rows` valid keys per plane; boxes
// of 64 dims x 64 keys, 128-byte swizzle, zeros outside.
bool x_make_map(CUtensorMap* map, const __half* base, int rows, int cap, int planes) {
  x_encode_fn enc = x_encoder();
  if (!enc) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)XD, (cuuint64_t)rows, (cuuint64_t)planes};
  const cuuint64_t strides[2] = {(cuuint64_t)XD * 2, (cuuint64_t)cap * XD * 2};
  const cuuint32_t box[3] = {64, (cuuint32_t)XK, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Covers: head size 128, no mask or causal, 16-byte aligned q / out / cache, the number of keys known
// on the host (skv > 0; skv_dev, if given, must hold skv - sq). Returns 1 when the shape is not
// covered (the caller then runs the mma.sync kernel). FB200_ATTN_TCGEN05=0 switches it off.
int fb200_launch_attention_prefill_tc(fb200_device* dev, const float* q, const __half* k, const __half* v, int b, int h,
                                      int hkv, int sq, int skv, const int* skv_dev, int cap, int d, float scale,
                                      int causal, float* out, int bshd) {
  static const bool off = getenv("FB200_ATTN_TCGEN05") && getenv("FB200_ATTN_TCGEN05")[0] == '0';
  if (off || d != XD || h % hkv || b > 65535 || h > 65535 || !(scale > 0.f) || skv <= 0 || skv > cap) return 1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(k) |
       reinterpret_cast<uintptr_t>(v)) & 15u)
    return 1;
  CUtensorMap kmap, vmap;
  if (!x_make_map(&kmap, k, skv, cap, b * hkv) || !x_make_map(&vmap, v, skv, cap, b * hkv)) return 1;
  XArgs a = {};
  a.q = q; a.k = k; a.v = v; a.out = out; a.skv_dev = skv_dev;
  a.b = b; a.h = h; a.hkv = hkv; a.sq = sq; a.skv = skv; a.cap = cap; a.groups = h / hkv; a.bshd = bshd;
  a.causal = causal; a.scale_log2 = scale * 1.4426950408889634f;
  a.k_lbo = 16;           // not used by a swizzled K-major operand
  a.v_lbo = X_BOX_BYTES;  // MN-major V: between the two 64-dim boxes
  a.v_sbo = 1024;         // ... and between groups of 8 keys
  a.status = dev->status;
  const dim3 grid((unsigned)((sq + XQ - 1) / XQ), (unsigned)h, (unsigned)b);
  static bool configured[64] = {false};
  if (!configured[dev->ordinal & 63]) {
    FB_CUDA(dev, cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, X_SMEM));
    configured[dev->ordinal & 63] = true;
  }
  return fb200_launch(dev, attn_prefill_tc_kernel, grid, dim3(X_BLOCK), (size_t)X_SMEM, false, a, kmap, vmap);
}
