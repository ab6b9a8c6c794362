// Prefill attention (many queries, optional causal mask) for sm_100a on the 5th-generation tensor
// cores.  Replaces the reference's ScaledDotProductAttention / SdpaKernel
// (src/ops/cuda/sequence.cu:105-163,451-472), whose scores live in shared memory (skv*4 bytes, so it
// cannot pass ~12 K keys) and whose P.V loop is thread-serial.
//
// fp16, head_dim 128: one CTA (four softmax warps + an MMA warp + a TMA warp, two CTAs per SM) per
// (block of 128 query rows, query head).  Q, K and V tiles are staged by TMA with 128-byte swizzle;
// S = Q.K^T (128 x 64 per tile of 64 keys) and O += P.V are tcgen05.mma (cta_group::1, kind::f16) with
// the accumulators in tensor memory (two S buffers and O: 256 columns per CTA); thread t owns query
// row t: it reads its scores with tcgen05.ld, does the online softmax in registers, writes P (fp16
// pairs) back over the first half of its S row with tcgen05.st - P.V takes its A operand from tensor
// memory, so P never crosses shared memory - and rescales its O row in tensor memory when the running
// maximum moves by more than a threshold.  One lane each of two more warps launches the MMAs and the
// TMA loads; the sides meet only on mbarriers (tcgen05.commit for MMA completion).  K/V tiles are
// multi-buffered and S is computed two tiles ahead, so tensor core and softmax overlap.  Every wait
// is bounded.  Other dtypes and head sizes run row by row on the decode kernels (correct, not fast).
//
// Semantics as the reference's CPU op (src/ops/cpu/sequence.cpp:236-301): q (sq,hq,d), k/v
// (skv,hkv,d) token-major, head h reads KV head h / (hq/hkv), scale 1/sqrt(d); with is_causal row t
// sees keys [0, t] when skv >= t+1 and all keys otherwise.
#include <math.h>

#include <mutex>

#include "common.cuh"

namespace axb {

// Row-by-row evaluation on the decode kernels (defined beside them).
int sdpa_rows_fallback(const void *q, const void *k, const void *v, void *out, int sq, int hq, int hkv,
                       int d, int64_t skv, int is_causal, int dtype, void *workspace,
                       size_t workspace_bytes, cudaStream_t st);
size_t sdpa_rows_workspace_bytes(int sq, int hq, int hkv, int d, int64_t skv);
// Tiled evaluation on the FMA pipe (prefill_tiled.cu): FLOAT32 and the head sizes the tensor-core kernels
// do not take.
bool sdpa_tiled_supported(int sq, int hq, int hkv, int d, int64_t skv);
int sdpa_tiled(const void *q, const void *k, const void *v, void *out, int sq, int hq, int hkv, int d, int64_t skv,
               int is_causal, int dtype, cudaStream_t st);

namespace {

constexpr int kBlockM = 128, kBlockN = 64, kD = 128;
constexpr int kSoftmaxWarps = 4;
constexpr int kMmaWarp = kSoftmaxWarps, kLoadWarp = kSoftmaxWarps + 1;
constexpr int kThreads = (kSoftmaxWarps + 2) * 32;  // + the MMA warp and the TMA warp
constexpr int kQTileBytes = kBlockM * kD * 2;   // 32 KB: two swizzled boxes of [128 rows][64 halves]
constexpr int kKvTileBytes = kBlockN * kD * 2;  // 16 KB: two swizzled boxes of [64 rows][64 halves]
constexpr int kKStages = 3, kVStages = 2;  // K runs ahead of V: S is computed two tiles before P.V
constexpr int kOffQ = 0, kOffK = kQTileBytes, kOffV = kOffK + kKStages * kKvTileBytes;
constexpr int kOffBar = kOffV + kVStages * kKvTileBytes;
constexpr int kSmemBytes = kOffBar + 256;  // 112 KB + barriers: two CTAs per SM
constexpr float kLog2e = 1.4426950408889634f;

struct PrefillParams {
  void *out;
  int sq, hq, hkv, skv, causal;
  float scale_log2;
};

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Shared-memory matrix descriptor: start address, leading / stride byte offsets (all >> 4),
// descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}

// The same with the A operand read from tensor memory (lane = row, one 32-bit column = two fp16
// elements along K, so 16 keys = 8 columns).
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The same load without the wait: several may be in flight before one tcgen05.wait::ld.
__device__ __forceinline__ void tmem_ld32_async(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

constexpr float kLazyLog2 = 8.0f;


// 192 threads.  Warps 0-3 (softmax): thread t owns query row t of the block (tensor-memory lane t)
// and all 64 key columns of a tile, so the row maximum and sum need no exchange.  Warp 4 (one lane)
// issues every MMA from descriptors built once; warp 5 (one lane) issues every TMA load, K and V tiles
// in rings of 3 and 2 stages freed by tcgen05.commit - a single thread doing both spent two thirds of
// a tile's time on instruction issue.  The sides meet only on mbarriers (full/empty per stage; bar_s:
// S_j ready; bar_p: P_j written; bar_o: P_j.V_j done; bar_fin: the last P.V done).  Software pipeline:
// S_{j+2} = Q.K_{j+2}^T is issued once P_j.V_j has completed, while the softmax warps are already in
// tile j+1 (two S buffers).  Two CTAs share an SM (112 KB of shared memory and 256 tensor-memory
// columns each).
__global__ void __launch_bounds__(kThreads, 2)
prefill_attn_f16_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const PrefillParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffBar);
  uint64_t *bar_q = bars;                                    // Q landed
  uint64_t *full_k = bars + 1, *empty_k = bars + 4;          // per K stage: tile landed / S that read it done
  uint64_t *full_v = bars + 7, *empty_v = bars + 9;          // per V stage: tile landed / P.V that read it done
  uint64_t *bar_s = bars + 11, *bar_o = bars + 13;           // S_j ready (per S buffer); P_j.V_j done
  uint64_t *bar_fin = bars + 14;  // the last P.V: the softmax warps skip phases of bar_o, a parity wait there would alias
  uint64_t *bar_p = bars + 15;    // P_j written (per S buffer), one arrival per softmax warp
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 17);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 18);

  // the swizzled tiles need a 1024-byte aligned base; refuse to run otherwise (nothing is written)
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicOr(&g_error_word, AXB200_ERR_WAIT_TIMEOUT);
    return;
  }
  // heaviest blocks first: under a causal mask the last query block has the most key tiles
  const int qb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y;
  const int hk = h / (p.hq / p.hkv);
  const int q0 = qb * kBlockM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t_last = min(q0 + kBlockM, p.sq) - 1;
  const int kv_end_max = p.causal ? min(t_last + 1, p.skv) : p.skv;  // reference rule: min(t+1, skv)
  const int nkv = (kv_end_max + kBlockN - 1) / kBlockN;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 15; ++i) mbar_init(&bars[i], 1);
    // one per S buffer: a softmax warp may run a tile ahead of the others, and with a single barrier
    // its second arrival would complete the phase the slower warps have not reached
    mbar_init(&bar_p[0], kSoftmaxWarps);
    mbar_init(&bar_p[1], kSoftmaxWarps);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(smem_u32(tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot, tmem_o = tmem_base + 128;  // S buffers at columns 0 and 64

  if (warp == kLoadWarp) {
    // ================= TMA warp (one lane): Q, then K and V tiles in the order they are consumed =====
    if (lane == 0) {
      tma_prefetch_descriptor(&tmQ);
      tma_prefetch_descriptor(&tmK);
      tma_prefetch_descriptor(&tmV);
      mbar_arrive_expect_tx(bar_q, kQTileBytes);
      tma_load_3d(smem + kOffQ, &tmQ, bar_q, 0, h, q0);
      tma_load_3d(smem + kOffQ + kQTileBytes / 2, &tmQ, bar_q, 64, h, q0);
      bool ok = true;
      auto load_k = [&](int j) {
        const int s = j % kKStages;
        if (j >= kKStages) ok = mbar_wait_bounded(&empty_k[s], (j / kKStages - 1) & 1, abort_flag);
        if (!ok) return;
        uint8_t *dst = smem + kOffK + s * kKvTileBytes;
        mbar_arrive_expect_tx(&full_k[s], kKvTileBytes);
        tma_load_3d(dst, &tmK, &full_k[s], 0, hk, j * kBlockN);
        tma_load_3d(dst + kKvTileBytes / 2, &tmK, &full_k[s], 64, hk, j * kBlockN);
      };
      auto load_v = [&](int j) {
        const int s = j % kVStages;
        if (j >= kVStages) ok = mbar_wait_bounded(&empty_v[s], (j / kVStages - 1) & 1, abort_flag);
        if (!ok) return;
        uint8_t *dst = smem + kOffV + s * kKvTileBytes;
        mbar_arrive_expect_tx(&full_v[s], kKvTileBytes);
        tma_load_3d(dst, &tmV, &full_v[s], 0, hk, j * kBlockN);
        tma_load_3d(dst + kKvTileBytes / 2, &tmV, &full_v[s], 64, hk, j * kBlockN);
      };
      // consumption order is S_0 S_1 (PV_0 S_2) (PV_1 S_3) ...: K_0 K_1 K_2 V_0 K_3 V_1 ...
      load_k(0);
      if (nkv > 1) load_k(1);
      for (int j = 0; j < nkv && ok; ++j) {
        if (j + 2 < nkv) load_k(j + 2);
        if (ok) load_v(j);
      }
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA warp (one lane) =================
    if (lane == 0) {
      // instruction descriptors: fp32 accumulate, fp16 operands, M = 128.  Q.K^T: N = 64 keys, B
      // K-major; P.V: N = 128 dims, B MN-major (a V tile is [keys][d], d contiguous)
      const uint32_t idesc_qk = (1u << 4) | ((kBlockN >> 3) << 17) | ((kBlockM >> 4) << 24);
      const uint32_t idesc_pv = (1u << 4) | (1u << 16) | ((kD >> 3) << 17) | ((kBlockM >> 4) << 24);
      // Shared-memory descriptors are built once: stepping a tile, a stage or 16 elements along K only
      // adds to the 14-bit address field (bytes >> 4), which cannot carry out of it (addresses < 256 KB).
      const uint64_t dq = smem_desc(smem_u32(smem + kOffQ), 16, 1024);
      const uint64_t dk = smem_desc(smem_u32(smem + kOffK), 16, 1024);
      const uint64_t dv = smem_desc(smem_u32(smem + kOffV), kKvTileBytes / 2, 1024);
      // S_j = Q . K_j^T into S buffer j&1; arrives on bar_s[j&1], and frees the K stage when done
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1, sk = j % kKStages;
        if (!mbar_wait_bounded(&full_k[sk], (j / kKStages) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint64_t dks = dk + (uint64_t)(sk * (kKvTileBytes >> 4));
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // head_dim 128 = 8 steps of 16; each 64-wide half of d is one box
          const uint32_t q_off = (ks >> 2) * (kQTileBytes / 2) + (ks & 3) * 32;
          const uint32_t k_off = (ks >> 2) * (kKvTileBytes / 2) + (ks & 3) * 32;
          umma_f16(tmem_base + s * kBlockN, dq + (q_off >> 4), dks + (k_off >> 4), idesc_qk, ks > 0);
        }
        umma_commit(&bar_s[s]);
        umma_commit(&empty_k[sk]);
        return true;
      };
      bool ok = mbar_wait_bounded(bar_q, 0, abort_flag) && issue_s(0);
      if (ok && nkv > 1) ok = issue_s(1);
      for (int j = 0; j < nkv && ok; ++j) {
        // P_j stands in the first 32 columns of S buffer j&1: O += P_j . V_j
        const int sv = j % kVStages;
        ok = mbar_wait_bounded(&bar_p[j & 1], (j >> 1) & 1, abort_flag) &&
             mbar_wait_bounded(&full_v[sv], (j / kVStages) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint64_t dvs = dv + (uint64_t)(sv * (kKvTileBytes >> 4));
        const uint32_t p_tmem = tmem_base + (j & 1) * kBlockN;
#pragma unroll
        for (int ks = 0; ks < kBlockN / 16; ++ks) {
          // V as the MN-major B operand: the two 64-wide d atoms are one box (8 KB) apart, 8-key
          // groups 1 KB apart, 16 keys per instruction = 2 KB
          umma_f16_ts(tmem_o, p_tmem + ks * 8, dvs + (uint64_t)(ks * (2048 >> 4)), idesc_pv, j > 0 || ks > 0);
        }
        umma_commit(bar_o);
        umma_commit(&empty_v[sv]);
        if (j == nkv - 1) umma_commit(bar_fin);
        if (j + 2 < nkv) {
          // P_j.V_j complete: P_j is consumed, so S_{j+2} may overwrite S buffer j&1 (queueing it behind
          // P_j.V_j instead would lean on issue-order execution, which is documented only for MMAs of
          // one shape; measured no faster)
          ok = mbar_wait_bounded(bar_o, j & 1, abort_flag);
          if (!ok) break;
          ok = issue_s(j + 2);
        }
      }
    }
  } else {
    // ================= softmax warps =================
    const int row = threadIdx.x;
    const int t_row = q0 + row;
    const int kv_end = p.causal ? min(t_row + 1, p.skv) : p.skv;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      const int sb = j & 1;
      ok = mbar_wait_bounded(&bar_s[sb], (j >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      // ---- this thread's row of scores: 64 keys ----
      const int n0 = j * kBlockN;
      uint32_t sr[2][32];
      tmem_ld32(tmem_base + sb * kBlockN + lane_base, sr[0]);
      tmem_ld32(tmem_base + sb * kBlockN + lane_base + 32, sr[1]);
      if (n0 + kBlockN > kv_end) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (n0 + c * 32 + i >= kv_end) sr[c][i] = 0xff800000u;  // -inf
      }
      // four independent chains keep the 64-long reductions off the critical path
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sr[c][i]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // Lazy maximum: the running maximum (and with it the rescale of O in tensor memory) moves only
      // when some row of the warp found a score more than kLazyLog2 above it; until then p = 2^(s - m)
      // may reach 2^kLazyLog2, which fp16 P and the fp32 sums hold without loss.
      const float m_tile = mx * p.scale_log2;
      float corr = 1.f;
      const bool corr_any = __any_sync(0xffffffffu, m_tile > m_run + kLazyLog2);
      if (corr_any) {
        const float m_new = fmaxf(m_run, m_tile);
        corr = fast_exp2(m_run - ((m_new == -INFINITY) ? 0.f : m_new));
        m_run = m_new;
      }
      const float m_safe = (m_run == -INFINITY) ? 0.f : m_run;
      uint32_t packed[32];
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float xa = fmaf(__uint_as_float(sr[c][i]), p.scale_log2, -m_safe);
          const float xb = fmaf(__uint_as_float(sr[c][i + 1]), p.scale_log2, -m_safe);
          const float a = fast_exp2(xa), b = fast_exp2(xb);
          sum4[(i >> 1) & 3] += a + b;
          packed[c * 16 + (i >> 1)] = pack_half2(a, b);
        }
      l_run = l_run * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));

      // P_j (fp16 pairs, 32 columns) over the first half of this thread's own S row
      tmem_st32(tmem_base + sb * kBlockN + lane_base, packed);
      // rescale this row of O in tensor memory when the warp moved a maximum; O is in use by
      // P_{j-1}.V_{j-1} until that completes (P_j.V_j is not issued before this warp arrives below,
      // so the barrier cannot be more than one phase ahead of the parity asked for)
      if (j > 0 && corr_any) {
        ok = mbar_wait_bounded(bar_o, (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_o + lane_base + c * 32, r);
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
          tmem_st32(tmem_o + lane_base + c * 32, r);
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_p[sb]);
    }
    // ---- epilogue: O / l -> out ----
    if (ok) ok = mbar_wait_bounded(bar_fin, 0, abort_flag);
    tc_fence_after();
    if (ok) {
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      __half *dst = reinterpret_cast<__half *>(p.out) + ((size_t)t_row * p.hq + h) * kD;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_o + lane_base + c * 32, r);
        if (t_row < p.sq) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w;
            w.x = pack_half2(__uint_as_float(r[u * 8 + 0]) * inv, __uint_as_float(r[u * 8 + 1]) * inv);
            w.y = pack_half2(__uint_as_float(r[u * 8 + 2]) * inv, __uint_as_float(r[u * 8 + 3]) * inv);
            w.z = pack_half2(__uint_as_float(r[u * 8 + 4]) * inv, __uint_as_float(r[u * 8 + 5]) * inv);
            w.w = pack_half2(__uint_as_float(r[u * 8 + 6]) * inv, __uint_as_float(r[u * 8 + 7]) * inv);
            *reinterpret_cast<uint4 *>(dst + c * 32 + u * 8) = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmem_base) : "memory");
}

// ---------------------------------------------------------------------------------------------------
// The 256-row form, for sq >= 256: one CTA per SM works on two query tiles of 128 rows against key
// tiles of 128, so that every MMA is 128 x 128 x 16 - at N = 64 the Q.K^T products re-read their A
// operand from shared memory so often that shared-memory bandwidth, not the tensor core, sets their
// pace - and each K/V tile staged in shared memory serves both query tiles.  Tensor memory (all 512
// columns): S_0, S_1, O_0, O_1, 128 columns each; P_g overwrites the first 64 columns of S_g.
// 320 threads: warps 0-3 own query tile 0 (thread t = row t), warps 4-7 tile 1, warp 8 issues the
// MMAs, warp 9 the TMA loads.  Per tile g the chain is S_g(j) -> softmax -> P_g(j) -> O_g += P_g(j).V_j
// -> S_g(j+1); the two tiles alternate on the tensor core, one computing while the other's softmax
// runs.  S_g(j+1) is queued directly behind P_g(j).V_j, whose A operand it overwrites: MMAs of one
// shape issued by one thread execute in issue order.  Its completion (bar_s) therefore also tells the
// softmax warps that P_g(j).V_j is done and O_g may be rescaled.
constexpr int kPairN = 128, kPairTileBytes = 128 * kD * 2;  // 32 KB: two swizzled boxes of [128 rows][64 halves]
constexpr int kPairThreads = 320, kPairMmaWarp = 8, kPairLoadWarp = 9;
constexpr int kPairOffQ = 0, kPairOffK = 2 * kPairTileBytes, kPairOffV = kPairOffK + 2 * kPairTileBytes;
constexpr int kPairOffBar = kPairOffV + 2 * kPairTileBytes;
constexpr int kPairSmemBytes = kPairOffBar + 256;  // 192 KB + barriers

__global__ void __launch_bounds__(kPairThreads, 1)
prefill_attn_f16_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                             const __grid_constant__ CUtensorMap tmV, const PrefillParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kPairOffBar);
  // K/V tiles travel in pairs (V_j, K_{j+1}) - what one key-tile step of the MMA warp consumes - under
  // one full and one empty barrier per pair slot j & 1, so that the MMA warp, which can do nothing else
  // while it waits, makes one wait and one commit per step instead of two.  Q and K_0 share bar_q.
  uint64_t *bar_q = bars, *full_kv = bars + 1, *empty_kv = bars + 3;
  uint64_t *bar_s = bars + 5, *bar_fin = bars + 7;  // per query tile: S_g(j) ready; last P.V done
  uint64_t *bar_p = bars + 9;                       // per query tile: P_g(j) written, one arrival per warp
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 11);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 12);

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicOr(&g_error_word, AXB200_ERR_WAIT_TIMEOUT);
    return;
  }
  // heaviest blocks first: under a causal mask the last query block has the most key tiles
  const int qb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y;
  const int hk = h / (p.hq / p.hkv);
  const int q0 = qb * 2 * kBlockM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // key tiles per query tile: none for a tile past the last query row; under the causal rule
  // min(t+1, skv) keys for its last row
  int nkv_g[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int first = q0 + g * kBlockM;
    const int t_last = min(first + kBlockM, p.sq) - 1;
    const int kv_end_max = p.causal ? min(t_last + 1, p.skv) : p.skv;
    nkv_g[g] = first < p.sq ? (kv_end_max + kPairN - 1) / kPairN : 0;
  }
  const int nkv = max(nkv_g[0], nkv_g[1]);

  if (threadIdx.x == 0) {
    for (int i = 0; i < 9; ++i) mbar_init(&bars[i], 1);
    mbar_init(&bar_p[0], 4);
    mbar_init(&bar_p[1], 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kPairMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;  // S_g at g * 128, O_g at 256 + g * 128

  if (warp == kPairLoadWarp) {
    // ================= TMA warp (one lane) =================
    if (lane == 0) {
      tma_prefetch_descriptor(&tmQ);
      tma_prefetch_descriptor(&tmK);
      tma_prefetch_descriptor(&tmV);
      mbar_arrive_expect_tx(bar_q, 3 * kPairTileBytes);
#pragma unroll
      for (int g = 0; g < 2; ++g) {  // rows past sq are zero-filled
        tma_load_3d(smem + kPairOffQ + g * kPairTileBytes, &tmQ, bar_q, 0, h, q0 + g * kBlockM);
        tma_load_3d(smem + kPairOffQ + g * kPairTileBytes + kPairTileBytes / 2, &tmQ, bar_q, 64, h, q0 + g * kBlockM);
      }
      tma_load_3d(smem + kPairOffK, &tmK, bar_q, 0, hk, 0);
      tma_load_3d(smem + kPairOffK + kPairTileBytes / 2, &tmK, bar_q, 64, hk, 0);
      bool ok = true;
      for (int j = 0; j < nkv && ok; ++j) {  // pair j: V_j into V stage j & 1, K_{j+1} into K stage (j+1) & 1
        const int s = j & 1;
        // slot s was last committed by step j - 2; for j = 1 by the prologue, which read K_0 out of the
        // K stage that K_2 goes to (so slot 1 is one phase further on than slot 0)
        if (j >= 1) ok = mbar_wait_bounded(&empty_kv[s], s ? ((j - 1) >> 1) & 1 : ((j >> 1) - 1) & 1, abort_flag);
        if (!ok) break;
        const bool with_k = j + 1 < nkv;
        mbar_arrive_expect_tx(&full_kv[s], with_k ? 2 * kPairTileBytes : kPairTileBytes);
        if (with_k) {  // first: S_g(j+1) is what the softmax warps wait for
          uint8_t *kd = smem + kPairOffK + (s ^ 1) * kPairTileBytes;
          tma_load_3d(kd, &tmK, &full_kv[s], 0, hk, (j + 1) * kPairN);
          tma_load_3d(kd + kPairTileBytes / 2, &tmK, &full_kv[s], 64, hk, (j + 1) * kPairN);
        }
        uint8_t *vd = smem + kPairOffV + s * kPairTileBytes;
        tma_load_3d(vd, &tmV, &full_kv[s], 0, hk, j * kPairN);
        tma_load_3d(vd + kPairTileBytes / 2, &tmV, &full_kv[s], 64, hk, j * kPairN);
      }
    }
  } else if (warp == kPairMmaWarp) {
    // ================= MMA warp (one lane) =================
    if (lane == 0) {
      // fp32 accumulate, fp16 operands, M = 128, N = 128; Q.K^T: B K-major; P.V: B MN-major
      const uint32_t idesc_qk = (1u << 4) | ((kPairN >> 3) << 17) | ((kBlockM >> 4) << 24);
      const uint32_t idesc_pv = idesc_qk | (1u << 16);
      const uint64_t dq = smem_desc(smem_u32(smem + kPairOffQ), 16, 1024);
      const uint64_t dk = smem_desc(smem_u32(smem + kPairOffK), 16, 1024);
      const uint64_t dv = smem_desc(smem_u32(smem + kPairOffV), kPairTileBytes / 2, 1024);
      auto issue_s = [&](int g, int j) {  // S_g(j) = Q_g . K_j^T; K_j is known to have landed
        const uint64_t dqg = dq + (uint64_t)(g * (kPairTileBytes >> 4));
        const uint64_t dks = dk + (uint64_t)((j & 1) * (kPairTileBytes >> 4));
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // head_dim 128 = 8 steps of 16; each 64-wide half of d is one box
          const uint32_t off = ((ks >> 2) * (kPairTileBytes / 2) + (ks & 3) * 32) >> 4;
          umma_f16(tmem_base + g * 128, dqg + off, dks + off, idesc_qk, ks > 0);
        }
        umma_commit(&bar_s[g]);
      };
      bool ok = mbar_wait_bounded(bar_q, 0, abort_flag);
      if (ok) {
        tc_fence_after();
        if (nkv_g[0] > 0) issue_s(0, 0);
        if (nkv_g[1] > 0) issue_s(1, 0);
        umma_commit(&empty_kv[1]);  // K_0 has been read: the stage may take K_2
      }
      for (int j = 0; j < nkv && ok; ++j) {
        ok = mbar_wait_bounded(&full_kv[j & 1], (j >> 1) & 1, abort_flag);
        if (!ok) break;
        const uint64_t dvs = dv + (uint64_t)((j & 1) * (kPairTileBytes >> 4));
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          if (j >= nkv_g[g]) continue;
          ok = mbar_wait_bounded(&bar_p[g], j & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          // O_g += P_g(j) . V_j: P from tensor memory (16 keys = 8 columns); V as the MN-major B
          // operand: the two 64-wide d atoms are one box (16 KB) apart, 8-key groups 1 KB apart
#pragma unroll
          for (int ks = 0; ks < kPairN / 16; ++ks)
            umma_f16_ts(tmem_base + 256 + g * 128, tmem_base + g * 128 + ks * 8, dvs + (uint64_t)(ks * (2048 >> 4)),
                        idesc_pv, j > 0 || ks > 0);
          if (j == nkv_g[g] - 1) umma_commit(&bar_fin[g]);
          if (j + 1 < nkv_g[g]) issue_s(g, j + 1);
        }
        if (!ok) break;
        umma_commit(&empty_kv[j & 1]);
      }
    }
  } else {
    // ================= softmax warps: query tile g, thread = row =================
    const int g = warp >> 2, row = threadIdx.x & (kBlockM - 1);
    const int my_nkv = g ? nkv_g[1] : nkv_g[0];
    const int t_row = q0 + g * kBlockM + row;
    const int kv_end = p.causal ? min(t_row + 1, p.skv) : p.skv;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem_base + g * 128 + lane_base, tmem_o = tmem_base + 256 + g * 128 + lane_base;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < my_nkv && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar_s[g], j & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      // ---- this thread's row of scores: 128 keys ----
      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32_async(tmem_s + c * 32, sr[c]);
      tmem_wait_ld();
      const int n0 = j * kPairN;
      if (n0 + kPairN > kv_end) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (n0 + c * 32 + i >= kv_end) sr[c][i] = 0xff800000u;  // -inf
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sr[c][i]));
      const float m_tile = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      // lazy maximum, as in the 128-row kernel
      float corr = 1.f;
      const bool moved = __any_sync(0xffffffffu, m_tile > m_run + kLazyLog2);
      if (moved) {
        const float m_new = fmaxf(m_run, m_tile);
        corr = fast_exp2(m_run - ((m_new == -INFINITY) ? 0.f : m_new));
        m_run = m_new;
      }
      const float m_safe = (m_run == -INFINITY) ? 0.f : m_run;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float xa = fmaf(__uint_as_float(sr[c][i]), p.scale_log2, -m_safe);
          const float xb = fmaf(__uint_as_float(sr[c][i + 1]), p.scale_log2, -m_safe);
          const float a = fast_exp2(xa), b = fast_exp2(xb);
          sum4[(i >> 1) & 3] += a + b;
          packed[i >> 1] = pack_half2(a, b);
        }
        // P: 32 keys = 16 columns over the front of this thread's own S row (all scores are in registers)
        tmem_st16(tmem_s + c * 16, packed);
      }
      l_run = l_run * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      // S_g(j) was queued behind P_g(j-1).V_{j-1}, so that product is complete: O_g may be rescaled
      if (j > 0 && moved) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_o + c * 32, r);
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
          tmem_st32(tmem_o + c * 32, r);
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_p[g]);
    }
    // ---- epilogue: O / l -> out ----
    if (ok && my_nkv > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar_fin[g], 0, abort_flag));
    tc_fence_after();
    if (ok && my_nkv > 0) {
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      __half *dst = reinterpret_cast<__half *>(p.out) + ((size_t)t_row * p.hq + h) * kD;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_o + c * 32, r);
        if (t_row < p.sq) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w;
            w.x = pack_half2(__uint_as_float(r[u * 8 + 0]) * inv, __uint_as_float(r[u * 8 + 1]) * inv);
            w.y = pack_half2(__uint_as_float(r[u * 8 + 2]) * inv, __uint_as_float(r[u * 8 + 3]) * inv);
            w.z = pack_half2(__uint_as_float(r[u * 8 + 4]) * inv, __uint_as_float(r[u * 8 + 5]) * inv);
            w.w = pack_half2(__uint_as_float(r[u * 8 + 6]) * inv, __uint_as_float(r[u * 8 + 7]) * inv);
            *reinterpret_cast<uint4 *>(dst + c * 32 + u * 8) = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kPairMmaWarp)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
}


using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encoder() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// (rows, heads, 128) fp16 token-major -> tensor map with boxes of [box_rows rows][64 halves], 128-byte swizzle
bool rows_map(CUtensorMap *map, const void *base, int64_t rows, int heads, int box_rows) {
  EncodeTiledFn fn = encoder();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)heads, (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)kD * 2, (cuuint64_t)heads * kD * 2};
  cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows}, es[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace axb

extern "C" {

size_t axb200_sdpa_workspace_bytes(int sq, int hq, int hkv, int d, int64_t skv, int dtype) {
  // the tensor-core kernels and the tiled FMA kernel keep everything on chip; only the row-by-row
  // evaluation on the decode kernels needs room for partials
  // (whatever the tensor-core path does not take - unaligned pointers, say - the tiled kernel does)
  if (hkv > 0 && hq % hkv == 0 && axb::sdpa_tiled_supported(sq, hq, hkv, d, skv)) return 0;
  return axb::sdpa_rows_workspace_bytes(sq, hq, hkv, d, skv);
}

int axb200_sdpa(const void *q, const void *k, const void *v, void *out, int sq, int hq, int hkv, int d,
                int64_t skv, int is_causal, int dtype, void *workspace, size_t workspace_bytes, void *stream) {
  if (dtype != AXB200_FLOAT16 && dtype != AXB200_FLOAT32) return AXB200_UNSUPPORTED_TYPE;
  if (!q || !k || !v || !out) return AXB200_INVALID_PTR;
  if (sq <= 0 || hq <= 0 || hkv <= 0 || d <= 0 || skv <= 0 || skv > 0x7fffffff - 4096) return AXB200_INVALID_ARGUMENT;
  if (hq % hkv != 0) return AXB200_SHAPE_MISMATCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool tensor_path = dtype == AXB200_FLOAT16 && d == axb::kD && hq <= 65535 && axb::aligned16(q) &&
                           axb::aligned16(k) && axb::aligned16(v) && axb::aligned16(out) && axb::encoder();
  if (!tensor_path) {
    if (axb::sdpa_tiled_supported(sq, hq, hkv, d, skv))
      return axb::sdpa_tiled(q, k, v, out, sq, hq, hkv, d, skv, is_causal, dtype, st);
    return axb::sdpa_rows_fallback(q, k, v, out, sq, hq, hkv, d, skv, is_causal, dtype, workspace, workspace_bytes, st);
  }
  // 256 query rows per CTA once there are that many; the 128-row form below that
  const bool pair = sq >= 2 * axb::kBlockM;
  const int kv_box = pair ? axb::kPairN : axb::kBlockN;
  CUtensorMap mq, mk, mv;
  if (!axb::rows_map(&mq, q, sq, hq, axb::kBlockM) || !axb::rows_map(&mk, k, skv, hkv, kv_box) ||
      !axb::rows_map(&mv, v, skv, hkv, kv_box))
    return AXB200_INTERNAL_ERROR;
  static std::mutex mu;
  static bool opted[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return AXB200_DEVICE_ERROR;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!opted[dev]) {
      if (cudaFuncSetAttribute(axb::prefill_attn_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               axb::kSmemBytes) != cudaSuccess ||
          cudaFuncSetAttribute(axb::prefill_attn_f16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               axb::kPairSmemBytes) != cudaSuccess)
        return AXB200_DEVICE_ERROR;
      opted[dev] = true;
    }
  }
  axb::PrefillParams p{};
  p.out = out;
  p.sq = sq;
  p.hq = hq;
  p.hkv = hkv;
  p.skv = (int)skv;
  p.causal = is_causal != 0;
  p.scale_log2 = (1.0f / sqrtf((float)d)) * axb::kLog2e;
  if (pair) {
    const dim3 grid((sq + 2 * axb::kBlockM - 1) / (2 * axb::kBlockM), hq);
    axb::prefill_attn_f16_pair_kernel<<<grid, axb::kPairThreads, axb::kPairSmemBytes, st>>>(mq, mk, mv, p);
  } else {
    const dim3 grid((sq + axb::kBlockM - 1) / axb::kBlockM, hq);
    axb::prefill_attn_f16_kernel<<<grid, axb::kThreads, axb::kSmemBytes, st>>>(mq, mk, mv, p);
  }
  return axb::launch_status();
}

}  // extern "C"
