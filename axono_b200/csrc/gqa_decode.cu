// Decode attention for sm_100a: split-K flash-decoding over the KV cache plus the
// log-sum-exp combine.  Replaces the reference's GqaDecodeAttention and its two kernels
// (src/ops/cuda/gqa.cu:31-92 split, :95-129 merge, :139-182 launcher).
//
// Split kernel: one CTA per (chunk of the sequence, KV head, sequence).  A producer warp
// streams 32 KB stages (K tile + V tile) from HBM into shared memory with TMA tensor copies
// that complete on mbarriers; four consumer warps compute, for all query heads that share
// the KV head, S = q.K^T, an online softmax and O += P.V per tile, so every K/V byte is read
// from HBM once.  fp16 uses mma.sync m16n8k16 with fp32 accumulators on 128-byte-swizzled
// tiles (query heads are the M rows); fp32 uses FMA on unswizzled tiles.  Each CTA leaves an
// unnormalised partial (m, l, O) in the workspace; the combine kernel merges a sequence's
// partials.  The number of chunks comes from the context length and the SM count.
//
// Layouts: q/out (batch,hq,d).  Cache either token-major contiguous (skv,hkv,d) - the
// reference's layout, one sequence - or paged (num_pages,hkv,page_tokens,d) with a block
// table, where one (page, head) tile is a contiguous run in HBM.
#include <math.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <set>
#include <utility>

#include "common.cuh"

namespace axb {

namespace {
constexpr int kMaxErrorReaders = 16;
ErrorReader g_error_readers[kMaxErrorReaders];
int g_num_error_readers = 0;
}  // namespace

void register_error_reader(ErrorReader fn) {
  if (g_num_error_readers < kMaxErrorReaders) g_error_readers[g_num_error_readers++] = fn;
}

namespace {

constexpr int kHeadDim = 128;
constexpr int kConsumerWarps = 4;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + one producer warp
constexpr int kStageBytes = 32768;               // K tile 16 KB + V tile 16 KB
constexpr int kTileTokensF16 = 64;
constexpr int kTileTokensF32 = 32;
constexpr int kMaxGroupMma = 16;
constexpr int kMaxChunks = 256;  // the reference's kMaxSplits (src/ops/cuda/gqa.cu:27)
constexpr float kLog2e = 1.4426950408889634f;

struct DecodeParams {
  const void *q;
  void *out;
  float *part_o;   // (batch, hq, max_chunks, d)
  float *part_ml;  // (batch, hq, max_chunks, 2): running max (log2 domain or raw), sum
  const int32_t *block_table;
  const int32_t *seq_lens;  // device lengths, or null -> fixed_len
  int fixed_len;
  int batch, hq, hkv, group, d;
  int page_tokens, max_blocks, num_pages;
  int chunk_tokens, max_chunks;
  // balanced != 0: the problem fits one wave of CTAs, so the chunk length is chosen by every CTA from
  // the lengths in device memory - the smallest one for which all sequences' chunks fit the `budget`
  // CTAs a KV head has - and the grid is (budget, hkv): CTA x finds its (sequence, chunk) by a prefix
  // sum of the chunk counts.  Every CTA of the wave then streams about the same number of bytes.
  int balanced, budget;
  float scale;  // 1/sqrt(d)
  int window;       // > 0: only the last `window` tokens of each sequence are visible (sliding window)
  int causal_rows;  // rows are the queries of one sequence: row b sees min(row_offset + b + 1, fixed_len) keys
  int row_offset;   // index of the launch's first row within that sequence
  // arrival_region >= 0: the CTA that finishes a (sequence, KV head) last merges its chunk partials and
  // writes the result itself (no combine kernel); the arrival counters are that region of g_arrival.
  // direct_ok: a sequence with a single chunk is normalised and written by its CTA, no partial.
  int arrival_region, direct_ok;
  int merge_pairs;  // the merging CTA takes a group's heads two at a time
  unsigned long long wait_ns;  // limit of every bounded wait in the launch
};

// The decode step in one launch (axb200_decode_step_paged): what the attention kernel needs to do the
// append itself - rotate q in registers, rotate the new key and put it and the new value into the
// cache and into the staged tile that holds their token, and leave seq_lens[b] + 1 behind.
constexpr int kStepHalfMax = 64;  // head_dim <= 128
struct StepParams {
  const void *k_new, *v_new;  // (batch, hkv, d)
  void *k_pages, *v_pages;
  int32_t *seq_lens;          // read once per CTA, bumped by the last CTA of a sequence to have read it
  const int64_t *pos;         // (batch), (3, batch) under M-RoPE, or null: position = tokens cached before
  const float *inv_freq_dev;  // (d / 2), or null: `table`
  int rotate, mrope, h_lim, w_lim;
  int stage_q;                // q lives in host memory: fetch it once per CTA through shared memory
  // The step straight from a QKV projection's output (the text tower's layer): row b of qkv holds hq query
  // heads, hkv key heads, hkv value heads of d elements, `ld` elements apart; q and k get a per-head RMS
  // norm (weights of d elements, or null) before the rotation.  qkv == null: q / k_new / v_new as above.
  const void *qkv;
  long long ld;
  const void *q_norm_w, *k_norm_w;
  float eps;
  int advance;                // 1: the launch adds the token's slot (first layer of a step); 0: the length
                              // already counts it (later layers: the token goes to slot length - 1)
  float table[kStepHalfMax];  // theta^(-2i/d), from the host's powf
};

// Peers of a launch whose result goes to other GPUs' memory (KV heads sharded, or one sequence's
// tokens spread over the GPUs).  world == 0: single GPU, the result goes to p.out.
constexpr int kMaxPeers = 8;
struct GatherParams {
  void *peer_out[kMaxPeers];           // each rank's gathered buffer for this call's slot
  unsigned int *peer_flags[kMaxPeers]; // each rank's flag array [world]; entry r = rank r's generation
  unsigned int *local_state;           // [0] items finished in this call, [1] this rank's generation
  int world, rank, hq_total;
  int mode;  // 0: all-gather of head outputs; 1: context-parallel exchange of (O, m, l) records
};

// Arrival counters of the fused merge: kArrivalRegions regions of kArrivalSlots counters, one counter
// per (sequence, KV head) of a launch.  Zero when the library is loaded; the CTA that completes a
// count resets it, so every launch finds and leaves zeros.  Launches that may overlap on the GPU use
// different regions (the host assigns a region per workspace pointer).
constexpr int kArrivalRegions = 64, kArrivalSlots = 4096;
static __device__ unsigned int g_arrival[kArrivalRegions * kArrivalSlots];
// Readers of seq_lens[b] in a one-launch decode step, same regions: every CTA of sequence b counts
// itself in after it has read the length; the one that completes the count stores the new length.
static __device__ unsigned int g_step_readers[kArrivalRegions * kArrivalSlots];

__global__ void zero_arrival_kernel() {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < kArrivalRegions * kArrivalSlots;
       i += gridDim.x * blockDim.x)
    g_arrival[i] = g_step_readers[i] = 0u;
}

__device__ __forceinline__ int seq_len_raw(const DecodeParams &p, int b) {
  if (p.seq_lens) return p.seq_lens[b];
  return p.causal_rows ? min(p.row_offset + b + 1, p.fixed_len) : p.fixed_len;
}

// Tokens a launch can reach in one sequence: what its pages hold and, with a host-planned chunk
// length, what the grid's chunks cover.
__device__ __forceinline__ int covered_tokens(const DecodeParams &p) {
  long long cover = p.seq_lens ? (long long)p.max_blocks * p.page_tokens : (long long)p.fixed_len;
  if (!p.balanced) cover = min(cover, (long long)p.max_chunks * p.chunk_tokens);
  return (int)min(cover, (long long)INT32_MAX - 4096);
}

// Length of sequence b as the launch sees it.  A length beyond what the launch covers (the host's
// bound was too small, or the length is corrupt) is cut there and AXB200_ERR_CAPACITY is recorded.
__device__ __forceinline__ int seq_len_of(const DecodeParams &p, int b) {
  const int L = seq_len_raw(p, b), cover = covered_tokens(p);
  if (L > cover) {
    atomicOr(&g_error_word, AXB200_ERR_CAPACITY);
    return cover;
  }
  return L < 0 ? 0 : L;
}

// First visible token of a sequence of length L: 0, or L - window under a sliding window.
__device__ __forceinline__ int first_visible(const DecodeParams &p, int L) {
  return (p.window > 0 && L > p.window) ? L - p.window : 0;
}

// ---- which (sequence, chunk) a CTA works on -----------------------------------------------------
constexpr int kMaxBalancedBatch = 320;  // sequences a balanced launch can have (148 SMs x 2 CTAs)
constexpr int kMinChunkTiles = 4;       // a chunk is at least 256 tokens
constexpr int kPlanWords = kMaxBalancedBatch + 4;

struct CtaWork {
  int b, chunk;  // sequence and chunk of this CTA
  int L;         // the sequence's length
  int ct;        // the sequence's chunk length in tokens (a multiple of 64)
  int n;         // the sequence's chunk count (>= 1: chunk 0 of an empty sequence writes the zero row)
};

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Chunk count of a sequence of `tiles` 64-token tiles under chunk length `c` tiles.
__host__ __device__ inline int chunks_at(int tiles, int c) { return tiles <= c ? 1 : ceil_div(tiles, c); }

// Chunk length (tokens) and count of one sequence once the launch's chunk length c is known: the
// sequence's tiles are spread evenly over its ceil(tiles / c) chunks.
__host__ __device__ inline void sequence_chunks(int L, int c, int *ct, int *n) {
  const int tiles = ceil_div(L, 64);
  const int n0 = chunks_at(tiles, c);
  const int per = tiles > 0 ? ceil_div(tiles, n0) : 1;
  *ct = per * 64;
  *n = tiles > 0 ? ceil_div(tiles, per) : 1;
}

// Smallest chunk length (in tiles, >= kMinChunkTiles) for which the sequences' chunks fit `budget`
// CTAs with at most max_chunks per sequence - host-side statement of what the CTAs compute.
inline int balanced_chunk_tiles_host(const int *lens, int batch, int budget, int max_chunks) {
  int hi = kMinChunkTiles;
  for (int i = 0; i < batch; ++i) hi = std::max(hi, ceil_div(std::max(lens[i], 0), 64));
  int lo = kMinChunkTiles;
  while (lo < hi) {
    const int mid = (lo + hi) / 2;
    long long sum = 0;
    int most = 0;
    for (int i = 0; i < batch; ++i) {
      const int n = chunks_at(ceil_div(std::max(lens[i], 0), 64), mid);
      sum += n;
      most = std::max(most, n);
    }
    if (sum <= budget && most <= max_chunks) hi = mid; else lo = mid + 1;
  }
  return lo;
}

// The same search by warp 0 of a CTA over the lengths staged in s_plan[0 .. batch); the result is
// left in s_plan[kMaxBalancedBatch].  All threads of the CTA call it (two __syncthreads).
__device__ __forceinline__ int balanced_chunk_tiles(const DecodeParams &p, int *s_plan) {
  for (int i = threadIdx.x; i < p.batch; i += blockDim.x) s_plan[i] = seq_len_of(p, i);
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int hi = kMinChunkTiles;
    for (int i = lane; i < p.batch; i += 32) hi = max(hi, ceil_div(s_plan[i], 64));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, off));
    int lo = kMinChunkTiles;
    while (lo < hi) {  // uniform across the warp
      const int mid = (lo + hi) >> 1;
      int sum = 0, most = 0;
      for (int i = lane; i < p.batch; i += 32) {
        const int n = chunks_at(ceil_div(s_plan[i], 64), mid);
        sum += n;
        most = max(most, n);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, off);
        most = max(most, __shfl_xor_sync(0xffffffffu, most, off));
      }
      if (sum <= p.budget && most <= p.max_chunks) hi = mid; else lo = mid + 1;
    }
    if (lane == 0) s_plan[kMaxBalancedBatch] = lo;
  }
  __syncthreads();
  return s_plan[kMaxBalancedBatch];
}

// Fills `w` for this CTA; false when the CTA has nothing to do.  All threads call it.
__device__ __forceinline__ bool cta_work(const DecodeParams &p, int *s_plan, CtaWork &w) {
  if (!p.balanced) {
    w.b = blockIdx.z;
    w.chunk = blockIdx.x;
    w.L = seq_len_of(p, w.b);
    w.ct = p.chunk_tokens;
    w.n = max(1, ceil_div(w.L, w.ct));
    return w.chunk < w.n;
  }
  const int c = balanced_chunk_tiles(p, s_plan);
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x, x = blockIdx.x;
    if (lane == 0) s_plan[kMaxBalancedBatch + 1] = -1;
    __syncwarp();
    int base = 0;
    for (int i0 = 0; i0 < p.batch; i0 += 32) {  // prefix sum of the chunk counts, 32 sequences a step
      const int i = i0 + lane;
      const int n = i < p.batch ? chunks_at(ceil_div(s_plan[i], 64), c) : 0;
      int incl = n;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += up;
      }
      const int excl = base + incl - n;
      if (n > 0 && x >= excl && x < excl + n) {
        s_plan[kMaxBalancedBatch + 1] = i;
        s_plan[kMaxBalancedBatch + 2] = x - excl;
      }
      base += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
  w.b = s_plan[kMaxBalancedBatch + 1];
  if (w.b < 0) return false;
  w.chunk = s_plan[kMaxBalancedBatch + 2];
  w.L = s_plan[w.b];
  sequence_chunks(w.L, c, &w.ct, &w.n);
  return w.chunk < w.n;
}

// Chunk length and count of sequence b for a kernel that merges (all threads call it).
__device__ __forceinline__ void sequence_plan(const DecodeParams &p, int b, int *s_plan, int *L, int *ct, int *n) {
  if (!p.balanced) {
    *L = seq_len_of(p, b);
    *ct = p.chunk_tokens;
    *n = max(1, ceil_div(*L, *ct));
    return;
  }
  const int c = balanced_chunk_tiles(p, s_plan);
  *L = s_plan[b];
  sequence_chunks(*L, c, ct, n);
}

// ---- the end of a (sequence, head): merge of the chunk partials and the final store ---------------
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Counts a CTA in on a device-scope counter.  Release: the stores of the whole CTA that a block
// barrier ordered before this thread become visible before the count does (release is cumulative);
// acquire: what the CTAs counted before this one stored is visible to this thread and, after the
// next block barrier, to the CTA's other threads.
__device__ __forceinline__ unsigned int atom_add_acq_rel_gpu(unsigned int *p, unsigned int v) {
  unsigned int old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void st_release_sys(unsigned int *p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Log-sum-exp merge of chunk partials [c0, n) of one (sequence, head) for output dim t: the
// un-normalised value relative to the maximum M, and the sum Ls.  `dom` is the exponent domain of
// the stored maxima.  Partials were written by other CTAs: read them past L1.
__device__ __forceinline__ void merge_row(const DecodeParams &p, size_t base, int c0, int n, int t,
                                          float dom, float &val, float &M, float &Ls) {
  // one pass with a running maximum: the loads of a step do not depend on the running state, so
  // several steps' loads are in flight together and the merge costs about one trip to L2
  M = -INFINITY;
  val = 0.f;
  Ls = 0.f;
#pragma unroll 4
  for (int c = c0; c < n; ++c) {
    const float2 ml = __ldcg(reinterpret_cast<const float2 *>(p.part_ml) + base + c);
    const float o = __ldcg(p.part_o + (base + c) * p.d + t);
    const float Mn = fmaxf(M, ml.x);
    const float keep = M == -INFINITY ? 0.f : exp2f((M - Mn) * dom);
    const float wgt = ml.x == -INFINITY ? 0.f : exp2f((ml.x - Mn) * dom);
    val = fmaf(wgt, o, val * keep);
    Ls = fmaf(wgt, ml.y, Ls * keep);
    M = Mn;
  }
}

// Final store of (sequence b, local head h), dim t.  val is un-normalised relative to the maximum M
// with sum Ls (an empty sequence: 0, -inf, 0).  Single GPU: out = val / Ls.  Heads sharded: the row
// goes into every rank's gathered buffer (batch, hq_total, d) at head rank*hq + h, plain stores over
// NVLink to peer-mapped pointers.  Context parallel: the un-normalised record [O(d), m, l] goes into
// every rank's record buffer (batch, hq, world, d + 2) at index `rank`.
template <typename OutT>
__device__ __forceinline__ void emit_final(const DecodeParams &p, const GatherParams &g, int b, int h,
                                           int t, float val, float M, float Ls) {
  if (g.world == 0) {
    reinterpret_cast<OutT *>(p.out)[((size_t)b * p.hq + h) * p.d + t] =
        static_cast<OutT>(Ls > 0.f ? val / Ls : 0.f);
  } else if (g.mode == 0) {
    const OutT v = static_cast<OutT>(Ls > 0.f ? val / Ls : 0.f);
    const size_t at = ((size_t)b * g.hq_total + (size_t)g.rank * p.hq + h) * p.d + t;
    for (int r = 0; r < g.world; ++r) reinterpret_cast<OutT *>(g.peer_out[r])[at] = v;
  } else {
    const size_t rec = (((size_t)b * p.hq + h) * g.world + g.rank) * (p.d + 2);
    for (int r = 0; r < g.world; ++r) {
      float *dst = reinterpret_cast<float *>(g.peer_out[r]) + rec;
      dst[t] = val;
      if (t == 0) {
        dst[p.d] = M;
        dst[p.d + 1] = Ls;
      }
    }
  }
}

// The merge of one (sequence, head): chunk partials [c_first, n) -> the final row, by the `nthreads`
// (a multiple of 32, at most 128) threads of a CTA.  The chunks are dealt to the warps and every lane owns
// four output dims, so that a warp's loads - one 16-byte read of O and one 8-byte read of (m, l) per
// chunk, up to four chunks in flight - are independent of one another: a sequence cut into dozens of
// chunks (one long sequence on an otherwise empty GPU) merges in a couple of trips to L2 instead of one
// trip per chunk.  The warps' running (M, sum, O) meet in `s_merge` (nwarps x 132 floats of shared
// memory, 16-byte aligned), and thread t < 128 finishes dim t.  Head sizes that are not a multiple of 4 take the
// element-wise loop.  Both the fused merge and the combine kernel come through here, and a head's
// arithmetic does not depend on which heads it is merged beside: identical bits.
constexpr int kMergeSlab = 128, kMergeRow = kMergeSlab + 4;  // rows stay 16-byte aligned
// kH heads (h, h + 1, ...) at once: their loads fly together and the two barriers are paid once.
template <typename OutT, int kH, typename Bar>
__device__ __forceinline__ void merge_heads(const DecodeParams &p, const GatherParams &g, int b, int h,
                                            int c_first, int n, float dom, int tid, int nthreads,
                                            float *s_merge, Bar bar) {
  const int d = p.d;
  if (d % 4 != 0) {
#pragma unroll
    for (int r = 0; r < kH; ++r) {
      const size_t base = ((size_t)b * p.hq + h + r) * p.max_chunks;
      for (int t = tid; t < d; t += nthreads) {
        float val, M, Ls;
        merge_row(p, base, c_first, n, t, dom, val, M, Ls);
        emit_final<OutT>(p, g, b, h + r, t, val, M, Ls);
      }
    }
    return;
  }
  const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
  for (int d0 = 0; d0 < d; d0 += kMergeSlab) {  // one pass per 128 dims (two for head_dim 256)
    const int t4 = d0 + lane * 4;
    const bool act = t4 < d;
    float M[kH], Ls[kH];
    float4 val[kH];
#pragma unroll
    for (int r = 0; r < kH; ++r) {
      M[r] = -INFINITY;
      Ls[r] = 0.f;
      val[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int c = c_first + warp; c < n; c += nwarps * 4) {
      float2 ml[kH][4];
      float4 o[kH][4];
#pragma unroll
      for (int r = 0; r < kH; ++r) {
        const size_t base = ((size_t)b * p.hq + h + r) * p.max_chunks;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int cc = c + u * nwarps;
          ml[r][u] = make_float2(-INFINITY, 0.f);
          o[r][u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (cc < n) {
            ml[r][u] = __ldcg(reinterpret_cast<const float2 *>(p.part_ml) + base + cc);
            if (act) o[r][u] = __ldcg(reinterpret_cast<const float4 *>(p.part_o + (base + cc) * d + t4));
          }
        }
      }
#pragma unroll
      for (int r = 0; r < kH; ++r) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (c + u * nwarps >= n) continue;
          const float Mn = fmaxf(M[r], ml[r][u].x);
          const float keep = M[r] == -INFINITY ? 0.f : exp2f((M[r] - Mn) * dom);
          const float wgt = ml[r][u].x == -INFINITY ? 0.f : exp2f((ml[r][u].x - Mn) * dom);
          val[r].x = fmaf(wgt, o[r][u].x, val[r].x * keep);
          val[r].y = fmaf(wgt, o[r][u].y, val[r].y * keep);
          val[r].z = fmaf(wgt, o[r][u].z, val[r].z * keep);
          val[r].w = fmaf(wgt, o[r][u].w, val[r].w * keep);
          Ls[r] = fmaf(wgt, ml[r][u].y, Ls[r] * keep);
          M[r] = Mn;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kH; ++r) {
      float *mine = s_merge + (r * nwarps + warp) * kMergeRow;
      if (act) *reinterpret_cast<float4 *>(mine + lane * 4) = val[r];
      if (lane == 0) {
        mine[kMergeSlab] = M[r];
        mine[kMergeSlab + 1] = Ls[r];
      }
    }
    bar();
    if (tid < kMergeSlab && d0 + tid < d) {
#pragma unroll
      for (int r = 0; r < kH; ++r) {
        const float *rows = s_merge + r * nwarps * kMergeRow;
        float Mx = -INFINITY;
        for (int w = 0; w < nwarps; ++w) Mx = fmaxf(Mx, rows[w * kMergeRow + kMergeSlab]);
        float v = 0.f, L = 0.f;
        for (int w = 0; w < nwarps; ++w) {
          const float mw = rows[w * kMergeRow + kMergeSlab];
          const float wgt = mw == -INFINITY ? 0.f : exp2f((mw - Mx) * dom);
          v = fmaf(wgt, rows[w * kMergeRow + tid], v);
          L = fmaf(wgt, rows[w * kMergeRow + kMergeSlab + 1], L);
        }
        emit_final<OutT>(p, g, b, h + r, d0 + tid, v, Mx, L);
      }
    }
    bar();  // s_merge is free for the next slab or heads
  }
}

// All `count` heads starting at h: in pairs, then a last single one.  s_merge: 2 x nwarps x 132 floats.
template <typename OutT, typename Bar>
__device__ __forceinline__ void merge_head_range(const DecodeParams &p, const GatherParams &g, int b, int h,
                                                 int count, int c_first, int n, float dom, int tid,
                                                 int nthreads, float *s_merge, Bar bar) {
  int r = 0;
  if (p.merge_pairs)
    for (; r + 2 <= count; r += 2) merge_heads<OutT, 2>(p, g, b, h + r, c_first, n, dom, tid, nthreads, s_merge, bar);
  for (; r < count; ++r) merge_heads<OutT, 1>(p, g, b, h + r, c_first, n, dom, tid, nthreads, s_merge, bar);
}

// Tail of a CTA that has stored a finished item into every peer's buffer.  Called by all `bar`
// threads of the CTA (thread index tid): every thread fences its stores system-wide, the CTA counts
// the item in, and the CTA that completes the launch's `total` items publishes this rank's new
// generation to every peer and waits (bounded by wait_ns) until every peer's generation has arrived
// here, so that when the kernel completes the local buffer is whole.  s_word: two shared words.
template <typename Bar>
__device__ __forceinline__ void publish_and_wait(const GatherParams &g, unsigned int total,
                                                 unsigned long long wait_ns, int tid,
                                                 volatile unsigned int *s_word, Bar bar) {
  __threadfence_system();
  bar();
  if (tid == 0) {
    const unsigned int last = atomicAdd(&g.local_state[0], 1u) == total - 1 ? 1u : 0u;
    s_word[0] = last;
    if (last) {
      __threadfence_system();
      const unsigned int gen = g.local_state[1] + 1;  // only the last CTA of a call touches the generation
      g.local_state[0] = 0;
      g.local_state[1] = gen;
      s_word[1] = gen;
    }
  }
  bar();
  if (!s_word[0]) return;
  const unsigned int gen = s_word[1];
  if (tid < g.world) {
    st_release_sys(g.peer_flags[tid] + g.rank, gen);
    const unsigned int *flag = g.peer_flags[g.rank] + tid;
    const unsigned long long t0 = global_timer_ns();
    // generations only grow; the signed difference keeps the comparison right across wrap-around
    while ((int)(ld_acquire_sys(flag) - gen) < 0) {
      if (global_timer_ns() - t0 > wait_ns) {
        atomicOr(&g_error_word, AXB200_ERR_WAIT_TIMEOUT);
        break;
      }
    }
  }
}

// What the `nthreads` compute threads of a split CTA do once the chunk's work is stored.  `direct`:
// the sequence had a single visible chunk and the CTA has already emitted the final rows.  Otherwise
// the partial is in the workspace: with arrival counters the CTA counts itself in and, when it is the
// last of its (sequence, KV head), merges the partials of the group's heads and emits the rows;
// without counters a combine kernel follows.  With peers, a finished item then joins the exchange.
template <typename OutT, typename Bar>
__device__ __forceinline__ void finish_item(const DecodeParams &p, const GatherParams &g,
                                            const CtaWork &w, int hk, int c_first, bool direct,
                                            float dom, int tid, int nthreads,
                                            volatile unsigned int *s_word, float *s_merge, Bar bar) {
  if (!direct) {
    if (p.arrival_region < 0) return;  // the combine kernel merges
    bar();  // every thread's partial is stored before thread 0 counts the CTA in
    if (tid == 0) {
      unsigned int *cnt = g_arrival + (size_t)p.arrival_region * kArrivalSlots + (size_t)w.b * p.hkv + hk;
      const unsigned int expected = (unsigned int)(w.n - c_first);
      // one release-acquire operation by one thread instead of a fence by every thread on either
      // side of the count: two trips to L2 less at the tail of every item
      const unsigned int last = atom_add_acq_rel_gpu(cnt, 1u) + 1 == expected ? 1u : 0u;
      if (last) *cnt = 0u;  // every other CTA of the item has arrived: leave zero for the next launch
      s_word[0] = last;
    }
    bar();
    if (!s_word[0]) return;
    merge_head_range<OutT>(p, g, w.b, hk * p.group, p.group, c_first, w.n, dom, tid, nthreads, s_merge, bar);
  }
  if (g.world) publish_and_wait(g, (unsigned int)(p.batch * p.hkv), p.wait_ns, tid, s_word, bar);
}

// An empty sequence: its one CTA (chunk 0) writes the zero rows.  Called by all threads of the CTA.
template <typename OutT>
__device__ __forceinline__ void emit_empty_item(const DecodeParams &p, const GatherParams &g, int b, int hk,
                                                volatile unsigned int *s_word) {
  if (p.arrival_region < 0 && !p.direct_ok) return;  // the combine kernel writes the zero rows
  for (int r = 0; r < p.group; ++r)
    for (int t = threadIdx.x; t < p.d; t += blockDim.x)
      emit_final<OutT>(p, g, b, hk * p.group + r, t, 0.f, -INFINITY, 0.f);
  if (g.world)
    publish_and_wait(g, (unsigned int)(p.batch * p.hkv), p.wait_ns, threadIdx.x, s_word, [] { __syncthreads(); });
}

// ---- producer ---------------------------------------------------------------------------
// Streams tiles [0, ntiles) of this CTA's chunk.  All 32 lanes run the loop (the page ids of
// the next 32 tiles are fetched one per lane); lane 0 issues the copies.
template <bool kPaged, int kStages, int kTile, int kBoxes, int kBoxElems, int kStage = kStageBytes>
__device__ __forceinline__ void produce_tiles(const CUtensorMap *tmK, const CUtensorMap *tmV,
                                              const DecodeParams &p, uint8_t *stages,
                                              uint64_t *full, uint64_t *empty,
                                              volatile int *abort_flag, int b, int hk, int start,
                                              int ntiles, int lane, int spec_start, int spec_page) {
  constexpr int kBoxBytes = (kStage / 2) / kBoxes;
  int page_cache = 0;
  for (int i = 0; i < ntiles; ++i) {
    const int s = i % kStages;
    const uint32_t phase = (i / kStages) & 1;
    const int tok0 = start + i * kTile;
    int page = 0, tok_in_page = tok0;
    if (kPaged) {
      if ((i & 31) == 0) {
        const int t = i + lane;
        const int slot = (start + t * kTile) / p.page_tokens;
        page_cache = 0;
        if (t < ntiles && slot < p.max_blocks) {
          // the first 32 page ids may have been fetched while the length was still on its way
          page_cache = (i == 0 && start == spec_start) ? spec_page
                                                       : p.block_table[(size_t)b * p.max_blocks + slot];
          if (page_cache < 0 || page_cache >= p.num_pages) {
            atomicOr(&g_error_word, AXB200_ERR_BAD_PAGE);
            page_cache = p.num_pages;  // out of range: the copy zero-fills
          }
        }
      }
      page = __shfl_sync(0xffffffffu, page_cache, i & 31);
      tok_in_page = tok0 % p.page_tokens;
    }
    if (lane == 0) {
      if (mbar_wait_bounded(&empty[s], phase ^ 1u, abort_flag, p.wait_ns)) {
        mbar_arrive_expect_tx(&full[s], kStage);
        uint8_t *st = stages + (size_t)s * kStage;
#pragma unroll
        for (int bx = 0; bx < kBoxes; ++bx) {
          if (kPaged) {
            tma_load_4d(st + bx * kBoxBytes, tmK, &full[s], bx * kBoxElems, tok_in_page, hk, page);
            tma_load_4d(st + kStage / 2 + bx * kBoxBytes, tmV, &full[s], bx * kBoxElems,
                        tok_in_page, hk, page);
          } else {
            tma_load_4d(st + bx * kBoxBytes, tmK, &full[s], bx * kBoxElems, hk, tok0, 0);
            tma_load_4d(st + kStage / 2 + bx * kBoxBytes, tmV, &full[s], bx * kBoxElems, hk,
                        tok0, 0);
          }
        }
      }
    }
    __syncwarp();
    if (*abort_flag) break;
  }
}

// ---- chunk epilogue shared by both dtypes ---------------------------------------------------
// Consumer warps have written their per-warp (m, l, O) for each query head of the group into
// shared memory; thread t owns output dim t.  m is in the exponent domain `dom` (so weights
// are exp2((m_w - M) * dom)).  direct: the chunk is the whole sequence - emit the final rows;
// otherwise store the chunk's partial.
template <typename OutT, int kD>
__device__ __forceinline__ void finalize_chunk(const DecodeParams &p, const GatherParams &gp,
                                               const float *mO, const float *mM, const float *mL,
                                               int b, int hk, int chunk, int t, float dom,
                                               bool direct) {
  if (t >= p.d) return;  // threads past the head size own no output dim (kD is the padded tile width)
  for (int r = 0; r < p.group; ++r) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) M = fmaxf(M, mM[w * kMaxGroupMma + r]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) {
      const float mw = mM[w * kMaxGroupMma + r];
      const float wgt = (mw == -INFINITY) ? 0.f : exp2f((mw - M) * dom);
      L += mL[w * kMaxGroupMma + r] * wgt;
      acc += mO[(w * kMaxGroupMma + r) * kD + t] * wgt;
    }
    const int h = hk * p.group + r;
    if (direct) {
      emit_final<OutT>(p, gp, b, h, t, acc, M, L);
    } else {
      const size_t slot = ((size_t)b * p.hq + h) * p.max_chunks + chunk;
      p.part_o[slot * p.d + t] = acc;
      if (t == 0) {
        p.part_ml[slot * 2 + 0] = M;
        p.part_ml[slot * 2 + 1] = L;
      }
    }
  }
}

// Shared-memory carve-up: [stages][full barriers][empty barriers][abort flag, 3 words for the end
// of the item]; the merge buffers alias the first two stages once the pipeline has drained.
template <int kStages, int kStage = kStageBytes>
struct SmemLayout {
  static constexpr int kBarOffset = kStages * kStage;
  static constexpr int kBytes = kBarOffset + 2 * kStages * 8 + 16;
  static constexpr int kDynamicBytes = kBytes + 1024;  // room to align the base to 1024 B
};

__device__ __forceinline__ uint8_t *align_1024(uint8_t *p) {
  return reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(p) + 1023) & ~uintptr_t(1023));
}

// ---- fp16 split kernel: tensor-core tiles ---------------------------------------------------
// Byte offset of the 16-byte chunk `c16` (0..15 across the 256-byte row) of token row `row`
// inside a K or V tile stored as two 128-byte-swizzled boxes [64 tokens][64 halves].
__device__ __forceinline__ uint32_t swz_off(int row, int c16) {
  return (uint32_t)((c16 >> 3) * 8192 + row * 128 + (((c16 & 7) ^ (row & 7)) << 4));
}

// kD: width of the staged tiles, 128 or 64 halves; the head size p.d is any multiple of 8 up to kD.  A
// stage is a 64-token K tile and V tile of kD halves each (256 * kD bytes); a tile is kD / 64 boxes of
// [64 tokens][64 halves], 128-byte swizzled.  Columns at and past p.d lie outside the tensor map, so the
// copy engine fills them with zeros (and reads nothing for them); q is padded with zeros in registers;
// zero columns add nothing to a dot product, and the output columns past p.d are never stored.
//
// kStep (paged, p.d == kD, host-planned chunks, no window): the launch is a whole decode step.  Thread 0
// reads the old length, every thread works with old + 1, and the CTA counts itself in as a reader of the
// length; the new token's K and V rows never come through the copy engine - the consumer warp that owns
// the token's row of the last tile rotates k_new, stores both rows to the sequence's page for the steps
// to come, and writes them over the staged tile once it has landed (whatever the page held there is
// replaced before any thread reads it).  q is rotated in registers; the caller's q is left as it is.
template <bool kPaged, int kStages, int kMinCtas, int kD, bool kStep = false>
__global__ void __launch_bounds__(kThreads, kMinCtas)
gqa_split_f16_kernel(const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const DecodeParams p,
                     const GatherParams gp, const __grid_constant__ StepParams sp) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_plan[kPlanWords];
  __shared__ float s_rope[kStep ? 2 * kStepHalfMax : 1];  // cos [0, 64), sin [64, 128) of the step's position
  __shared__ __align__(16) __half s_q[kStep ? kMaxGroupMma * kD : 8];  // the group's q rows as they came
  constexpr int kStage = 256 * kD, kKSteps = kD / 16, kNTiles = kD / 8;
  uint8_t *smem = align_1024(smem_raw);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + SmemLayout<kStages, kStage>::kBarOffset);
  uint64_t *empty = full + kStages;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + kStages);
  volatile unsigned int *s_word = reinterpret_cast<volatile unsigned int *>(abort_flag + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == kConsumerThreads) {  // the producer's first lane, while warp 0 plans
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  // The producer warp asks for its first page ids (and the tensor maps) before the sequence's length
  // is known: with a host-planned chunk length the chunk's first token does not depend on it, and the
  // two trips to memory overlap instead of following one another.
  int spec_start = -1, spec_page = 0;
  if (warp == kConsumerWarps && lane == 0) {
    tma_prefetch_descriptor(&tmK);
    tma_prefetch_descriptor(&tmV);
  }
  grid_dependency_wait();  // nothing above reads what the kernel before this one writes
  // A step kernel lets the next step's kernel be scheduled behind it: that kernel's CTAs take the slots this
  // one's leave, set up their barriers and descriptors, and wait at the line above until this grid is done.
  if (kStep) grid_dependency_launch();
  if (warp == kConsumerWarps) {
    if (kPaged && !p.balanced) {
      spec_start = blockIdx.x * p.chunk_tokens;
      const int slot = (spec_start + lane * kTileTokensF16) / p.page_tokens;
      if (slot < p.max_blocks) spec_page = p.block_table[(size_t)blockIdx.z * p.max_blocks + slot];
    }
  }
  CtaWork w;
  bool active;
  int appended = 0;  // kStep: 1 when this launch adds a token to the sequence
  if (kStep) {
    if (threadIdx.x == 0) {  // one read of the length per CTA: every thread works with the same value
      int len = sp.seq_lens[blockIdx.z];
      const int cover = covered_tokens(p);
      len = len < 0 ? 0 : len;
      int add = 1;
      if (!sp.advance) {  // a later layer of the step: the length already counts the token
        if (len > cover || len == 0) {
          atomicOr(&g_error_word, AXB200_ERR_CAPACITY);
          len = min(len, cover);
          add = 0;
        }
        s_plan[0] = len;
      } else {
        if (len + 1 > cover) {  // no room for the token: nothing is appended, the old tokens are attended
          atomicOr(&g_error_word, AXB200_ERR_CAPACITY);
          len = min(len, cover);
          add = 0;
        }
        s_plan[0] = len + add;
      }
      s_plan[1] = add;
    }
    __syncthreads();
    w.b = blockIdx.z;
    w.chunk = blockIdx.x;
    w.L = s_plan[0];
    appended = s_plan[1];
    w.ct = p.chunk_tokens;
    w.n = max(1, ceil_div(w.L, w.ct));
    active = w.chunk < w.n;
  } else {
    active = cta_work(p, s_plan, w);
    __syncthreads();
  }
  // kStep: thread 0 counts the CTA in as a reader of the length (release: after its read); the answer
  // is looked at later, when it has long arrived - by `settle`, before the thread's every way out.
  unsigned int readers_before = 0;
  unsigned int *readers = nullptr;
  if (kStep && threadIdx.x == 0 && sp.advance) {  // (a launch that does not advance leaves the length alone)
    readers = g_step_readers + (size_t)p.arrival_region * kArrivalSlots + blockIdx.z;
    readers_before = atom_add_acq_rel_gpu(readers, 1u);
  }
  auto settle = [&]() {
    if (kStep && threadIdx.x == 0 && sp.advance && readers_before + 1 == gridDim.x * gridDim.y) {
      *readers = 0u;  // every CTA of the sequence has read the old length
      if (appended) sp.seq_lens[blockIdx.z] = w.L;
    }
  };
  if (!active) {
    settle();
    return;
  }
  const int chunk = w.chunk, hk = blockIdx.y, b = w.b, L = w.L;
  if (L == 0) {
    settle();
    emit_empty_item<__half>(p, gp, b, hk, s_word);
    return;
  }
  const int first = first_visible(p, L);
  const int c_first = first / w.ct;  // chunks before it lie wholly outside the window
  int start = chunk * w.ct;
  const int end = min(L, start + w.ct);
  if (end <= first) {  // the whole chunk lies before the window
    settle();
    return;
  }
  if (start < first) start = first / kTileTokensF16 * kTileTokensF16;  // skip whole tiles before it
  const int ntiles = (end - start + kTileTokensF16 - 1) / kTileTokensF16;
  const bool direct = p.direct_ok && w.n - c_first == 1;

  if (warp == kConsumerWarps) {
    produce_tiles<kPaged, kStages, kTileTokensF16, kD / 64, 64, kStage>(&tmK, &tmV, p, smem, full, empty, abort_flag, b, hk,
                                                          start, ntiles, lane, spec_start, spec_page);
    return;
  }

  // ---- consumers: warp w owns tokens [16w, 16w+16) of every tile ----
  const int g = lane >> 2, tq = lane & 3;
  const bool use_hi = p.group > 8;  // rows 8..15 of the M dimension carry query heads too
  const __half *qh = reinterpret_cast<const __half *>(p.q);

  // Q as the A operand, resident in registers: kD / 16 k-steps x 4 regs.  Asked for first: the loads fly
  // while everything below up to the first use is worked out.
  uint32_t qa[kKSteps][4];
  auto load_q = [&](const __half *q0) {
    const __half *q1 = q0 + 8 * p.d;
    const bool v0 = g < p.group, v1 = g + 8 < p.group;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
      const int c = ks * 16 + tq * 2;  // even, and p.d is a multiple of 8: a pair is inside or outside as a whole
      const bool in0 = c < p.d, in1 = c + 8 < p.d;
      qa[ks][0] = v0 && in0 ? *reinterpret_cast<const uint32_t *>(q0 + c) : 0u;
      qa[ks][1] = v1 && in0 ? *reinterpret_cast<const uint32_t *>(q1 + c) : 0u;
      qa[ks][2] = v0 && in1 ? *reinterpret_cast<const uint32_t *>(q0 + c + 8) : 0u;
      qa[ks][3] = v1 && in1 ? *reinterpret_cast<const uint32_t *>(q1 + c + 8) : 0u;
    }
  };
  const bool staged = kStep && (sp.stage_q || sp.qkv != nullptr);  // q comes through shared memory
  if (!staged) load_q(qh + ((size_t)b * p.hq + (size_t)hk * p.group + g) * p.d);

  // ---- kStep, first half: what has to come from memory is asked for, the angles are worked out ----
  constexpr int kHalf = kD / 2, kPairs = kHalf / 32;  // rotary pairs per lane of the warp that appends
  const int new_row = L - 1 - (start + (ntiles - 1) * kTileTokensF16);  // the token's row in the last tile
  const bool patch = kStep && appended && chunk == w.n - 1 && warp == (new_row >> 4);
  __half k_lo[kPairs], k_hi[kPairs], v_lo[kPairs], v_hi[kPairs];
  int new_page = 0;
  if constexpr (kStep) {
    const __half *qkv_row = reinterpret_cast<const __half *>(sp.qkv) + (size_t)b * sp.ld;
    if (patch) {  // the token's rows and its page id on their way while the angles are worked out
      const __half *kn = sp.qkv ? qkv_row + (size_t)(p.hq + hk) * kD
                                : reinterpret_cast<const __half *>(sp.k_new) + ((size_t)b * p.hkv + hk) * kD;
      const __half *vn = sp.qkv ? qkv_row + (size_t)(p.hq + p.hkv + hk) * kD
                                : reinterpret_cast<const __half *>(sp.v_new) + ((size_t)b * p.hkv + hk) * kD;
#pragma unroll
      for (int j = 0; j < kPairs; ++j) {
        const int i = lane + 32 * j;
        k_lo[j] = kn[i], k_hi[j] = kn[i + kHalf], v_lo[j] = vn[i], v_hi[j] = vn[i + kHalf];
      }
      new_page = p.block_table[(size_t)b * p.max_blocks + (L - 1) / p.page_tokens];
    }
    // q in host memory (sp.stage_q): the group's rows come through shared memory, 16 bytes a thread, every
    // byte asked for once per CTA.  Fragment loads straight from q ask for each 32-byte sector from all
    // four warps; over PCIe every such request is a read transaction, and a launch of thousands of CTAs
    // saturates the link's request rate long before its bandwidth (measured: 0.35 ms instead of 0.27 ms
    // per host-buffer step for a quarter of the batch).  The loads are asked for here and stored after
    // the angles, so the two overlap.
    uint4 q_piece[2];
    const int q_pieces = p.group * (kD / 8);  // at most 16 heads x 16 pieces: two per thread
    if (staged) {
      const uint4 *src = reinterpret_cast<const uint4 *>(sp.qkv ? qkv_row + (size_t)hk * p.group * kD
                                                                : qh + ((size_t)b * p.hq + (size_t)hk * p.group) * kD);
#pragma unroll
      for (int u = 0; u < 2; ++u)
        if ((int)threadIdx.x + u * kConsumerThreads < q_pieces) q_piece[u] = src[threadIdx.x + u * kConsumerThreads];
    }
    if (sp.rotate && threadIdx.x < kHalf) {  // one angle per rotary pair, once per CTA
      const int i = threadIdx.x;
      float pt, ph, pw;
      if (sp.pos == nullptr) {
        pt = ph = pw = (float)(L - appended);  // tokens cached before this one
      } else if (sp.mrope) {
        pt = (float)sp.pos[b];
        ph = (float)sp.pos[p.batch + b];
        pw = (float)sp.pos[2 * p.batch + b];
      } else {
        pt = ph = pw = (float)sp.pos[b];
      }
      const float f = sp.mrope || sp.inv_freq_dev ? sp.inv_freq_dev[i] : sp.table[i];
      const float posv = sp.mrope ? mrope_pair_position(i, pt, ph, pw, sp.h_lim, sp.w_lim) : pt;
      sincosf(posv * f, &s_rope[kStepHalfMax + i], &s_rope[i]);
    }
    if (staged) {
#pragma unroll
      for (int u = 0; u < 2; ++u)
        if ((int)threadIdx.x + u * kConsumerThreads < q_pieces)
          reinterpret_cast<uint4 *>(s_q)[threadIdx.x + u * kConsumerThreads] = q_piece[u];
    }
    if (sp.qkv) {
      // The per-head RMS norm and the rotation of q where the rows lie, one warp per head, lane i and
      // i + 32 of each half as in the kernel that does this on its own (qkv_norm_rope_append_kernel): the
      // same sums in the same order, hence the same bits.  The rows go back as fp16, as that kernel's q_out.
      named_bar_sync(1, kConsumerThreads);  // rows and angles are in shared memory
      for (int r = warp; r < p.group; r += kConsumerWarps) {
        __half *row = s_q + r * kD;
        float a[kPairs], bb[kPairs], ss = 0.f;
#pragma unroll
        for (int j = 0; j < kPairs; ++j) {
          const int i = lane + 32 * j;
          a[j] = __half2float(row[i]);
          bb[j] = __half2float(row[i + kHalf]);
          ss = fmaf(a[j], a[j], ss);
          ss = fmaf(bb[j], bb[j], ss);
        }
        const __half *wq = reinterpret_cast<const __half *>(sp.q_norm_w);
        float inv = 1.f;
        if (wq) {
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
          inv = 1.0f / sqrtf(ss / (float)kD + sp.eps);
        }
#pragma unroll
        for (int j = 0; j < kPairs; ++j) {
          const int i = lane + 32 * j;
          float x0 = a[j], x1 = bb[j];
          if (wq) {
            x0 = x0 * inv * __half2float(wq[i]);
            x1 = x1 * inv * __half2float(wq[i + kHalf]);
          }
          if (sp.rotate) {
            const float sn = s_rope[kStepHalfMax + i], cs = s_rope[i];
            const float r0 = rope_lo(x0, x1, cs, sn), r1 = rope_hi(x0, x1, cs, sn);
            x0 = r0;
            x1 = r1;
          }
          row[i] = __float2half_rn(x0);
          row[i + kHalf] = __float2half_rn(x1);
        }
      }
    }
  }

  if (staged) {
    named_bar_sync(1, kConsumerThreads);  // the staged rows (and the angles) are there
    load_q(s_q + g * kD);
  }

  // ---- kStep, second half: rotate q in registers, rotate and store the new token's rows ----
  if constexpr (kStep) {
    if (!staged) named_bar_sync(1, kConsumerThreads);  // the angles are there (q's loads flew meanwhile)
    if (sp.rotate && !sp.qkv) {
      // pair (c, c + kHalf) sits in k-steps ks and ks + kKSteps / 2 of the same thread
#pragma unroll
      for (int ks = 0; ks < kKSteps / 2; ++ks) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = ks * 16 + tq * 2 + (j >> 1) * 8;
          const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&qa[ks][j]));
          const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&qa[ks + kKSteps / 2][j]));
          const float c0 = s_rope[c], s0 = s_rope[kStepHalfMax + c], c1 = s_rope[c + 1], s1 = s_rope[kStepHalfMax + c + 1];
          const __half2 rl = __halves2half2(__float2half_rn(rope_lo(lo.x, hi.x, c0, s0)), __float2half_rn(rope_lo(lo.y, hi.y, c1, s1)));
          const __half2 rh = __halves2half2(__float2half_rn(rope_hi(lo.x, hi.x, c0, s0)), __float2half_rn(rope_hi(lo.y, hi.y, c1, s1)));
          qa[ks][j] = *reinterpret_cast<const uint32_t *>(&rl);
          qa[ks + kKSteps / 2][j] = *reinterpret_cast<const uint32_t *>(&rh);
        }
      }
    }
    if (patch) {
      if (sp.rotate || (sp.qkv && sp.k_norm_w)) {
        float a[kPairs], bb[kPairs], ss = 0.f;
#pragma unroll
        for (int j = 0; j < kPairs; ++j) {
          a[j] = __half2float(k_lo[j]);
          bb[j] = __half2float(k_hi[j]);
          ss = fmaf(a[j], a[j], ss);
          ss = fmaf(bb[j], bb[j], ss);
        }
        const __half *wk = sp.qkv ? reinterpret_cast<const __half *>(sp.k_norm_w) : nullptr;
        float inv = 1.f;
        if (wk) {  // the key's RMS norm, summed as qkv_norm_rope_append_kernel sums it
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
          inv = 1.0f / sqrtf(ss / (float)kD + sp.eps);
        }
#pragma unroll
        for (int j = 0; j < kPairs; ++j) {
          const int i = lane + 32 * j;
          float x0 = a[j], x1 = bb[j];
          if (wk) {
            x0 = x0 * inv * __half2float(wk[i]);
            x1 = x1 * inv * __half2float(wk[i + kHalf]);
          }
          if (sp.rotate) {
            const float c = s_rope[i], sn = s_rope[kStepHalfMax + i];
            const float r0 = rope_lo(x0, x1, c, sn), r1 = rope_hi(x0, x1, c, sn);
            x0 = r0;
            x1 = r1;
          }
          k_lo[j] = __float2half_rn(x0);
          k_hi[j] = __float2half_rn(x1);
        }
      }
      if (new_page >= 0 && new_page < p.num_pages) {  // the rows in the cache, for the steps to come
        const size_t row = (((size_t)new_page * p.hkv + hk) * p.page_tokens + (L - 1) % p.page_tokens) * kD;
        __half *kd = reinterpret_cast<__half *>(sp.k_pages) + row, *vd = reinterpret_cast<__half *>(sp.v_pages) + row;
#pragma unroll
        for (int j = 0; j < kPairs; ++j) {
          const int i = lane + 32 * j;
          kd[i] = k_lo[j], kd[i + kHalf] = k_hi[j], vd[i] = v_lo[j], vd[i + kHalf] = v_hi[j];
        }
      } else if (lane == 0) {
        atomicOr(&g_error_word, AXB200_ERR_BAD_PAGE);
      }
    }
    settle();  // the count went out before the rows were asked for: its answer is here by now
  }

  float o[kNTiles][4];
#pragma unroll
  for (int nt = 0; nt < kNTiles; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY;  // running max (log2 domain) of rows g, g+8
  float l0 = 0.f, l1 = 0.f;              // this thread's share of the running sums
  const float sl2 = p.scale * kLog2e;

  // ldmatrix lane roles
  const int mat = lane >> 3, mrow = lane & 7;
  const int k_row = warp * 16 + (mat >> 1) * 8 + mrow;  // K: matrices (n-tile, k-half)
  const int k_c16 = mat & 1;
  const int v_row = warp * 16 + (mat & 1) * 8 + mrow;   // V: matrices (k-half, n-tile)
  const int v_c16 = mat >> 1;

  bool ok = true;
  for (int i = 0; i < ntiles && ok; ++i) {
    const int s = i % kStages;
    const uint32_t phase = (i / kStages) & 1;
    ok = mbar_wait_bounded(&full[s], phase, abort_flag, p.wait_ns);
    if (!ok) break;
    const uint32_t kbase = smem_u32(smem + (size_t)s * kStage);
    const uint32_t vbase = kbase + kStage / 2;
    if constexpr (kStep) if (patch && i == ntiles - 1) {  // the new token's rows over whatever the page held
      uint8_t *kt = smem + (size_t)s * kStage, *vt = kt + kStage / 2;
#pragma unroll
      for (int j = 0; j < kPairs; ++j) {
        const int e0 = lane + 32 * j, e1 = e0 + kHalf;
        const uint32_t o0 = swz_off(new_row, e0 >> 3) + (e0 & 7) * 2, o1 = swz_off(new_row, e1 >> 3) + (e1 & 7) * 2;
        *reinterpret_cast<__half *>(kt + o0) = k_lo[j];
        *reinterpret_cast<__half *>(kt + o1) = k_hi[j];
        *reinterpret_cast<__half *>(vt + o0) = v_lo[j];
        *reinterpret_cast<__half *>(vt + o1) = v_hi[j];
      }
      __syncwarp();
    }

    // S(16 heads x 16 tokens) = Q . K^T
    float sc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(b0, b1, b2, b3, kbase + swz_off(k_row, ks * 2 + k_c16));
      mma_16816(sc[0], qa[ks], b0, b1);
      mma_16816(sc[1], qa[ks], b2, b3);
    }

    // mask the tokens past the end of the sequence (last tile only)
    const int tile_tok = start + i * kTileTokensF16 + warp * 16;  // this warp's first token
    const int valid = end - tile_tok;                              // tokens of the warp that exist
    const int lo = first - tile_tok;                               // tokens below lo precede the window
    const bool edge = valid < 16 || lo > 0;
    if (edge) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int t0 = j * 8 + tq * 2;
        if (t0 >= valid || t0 < lo) sc[j][0] = sc[j][2] = -INFINITY;
        if (t0 + 1 >= valid || t0 + 1 < lo) sc[j][1] = sc[j][3] = -INFINITY;
      }
    }

    // online softmax in the log2 domain; rows are shared by the 4 lanes of a quad
    float mx0 = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1])) * sl2;
    float mx1 = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3])) * sl2;
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float ms0 = (mn0 == -INFINITY) ? 0.f : mn0;  // all-masked rows stay at weight 0
    const float ms1 = (mn1 == -INFINITY) ? 0.f : mn1;
    const float corr0 = fast_exp2(m0 - ms0), corr1 = fast_exp2(m1 - ms1);
    m0 = mn0;
    m1 = mn1;
    float pr[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      pr[j][0] = fast_exp2(fmaf(sc[j][0], sl2, -ms0));
      pr[j][1] = fast_exp2(fmaf(sc[j][1], sl2, -ms0));
      pr[j][2] = fast_exp2(fmaf(sc[j][2], sl2, -ms1));
      pr[j][3] = fast_exp2(fmaf(sc[j][3], sl2, -ms1));
    }
    l0 = l0 * corr0 + (pr[0][0] + pr[0][1] + pr[1][0] + pr[1][1]);
    l1 = l1 * corr1 + (pr[0][2] + pr[0][3] + pr[1][2] + pr[1][3]);
    const bool rescale = use_hi ? (corr0 != 1.f || corr1 != 1.f) : (corr0 != 1.f);
    if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
      for (int nt = 0; nt < kNTiles; ++nt) {
        o[nt][0] *= corr0;
        o[nt][1] *= corr0;
        o[nt][2] *= corr1;
        o[nt][3] *= corr1;
      }
    }

    // P (fp16) as the A operand of O += P . V
    uint32_t pa[4];
    pa[0] = pack_half2(pr[0][0], pr[0][1]);
    pa[1] = pack_half2(pr[0][2], pr[0][3]);
    pa[2] = pack_half2(pr[1][0], pr[1][1]);
    pa[3] = pack_half2(pr[1][2], pr[1][3]);
#pragma unroll
    for (int np = 0; np < kNTiles / 2; ++np) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(b0, b1, b2, b3, vbase + swz_off(v_row, np * 2 + v_c16));
      if (edge) {
        // rows outside [lo, valid) may hold stale bytes: zero them so 0 * NaN cannot appear.
        // b0/b2 hold tokens 2tq,2tq+1; b1/b3 hold tokens 8+2tq, 8+2tq+1.
        const int t0 = tq * 2;
        auto in = [&](int t) { return t < valid && t >= lo; };
        const uint32_t keep_lo = (in(t0) ? 0x0000ffffu : 0u) | (in(t0 + 1) ? 0xffff0000u : 0u);
        const uint32_t keep_hi = (in(t0 + 8) ? 0x0000ffffu : 0u) | (in(t0 + 9) ? 0xffff0000u : 0u);
        b0 &= keep_lo;
        b2 &= keep_lo;
        b1 &= keep_hi;
        b3 &= keep_hi;
      }
      mma_16816(o[np * 2], pa, b0, b1);
      mma_16816(o[np * 2 + 1], pa, b2, b3);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }

  // ---- merge the four warps' states and emit the chunk's partial ----
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  named_bar_sync(1, kConsumerThreads);  // every stage has been consumed: reuse stage memory
  if (*abort_flag) return;
  float *mO = reinterpret_cast<float *>(smem);                // [4][16][kD]: 256 * kD bytes, one stage
  float *mM = reinterpret_cast<float *>(smem + kStage);       // [4][16]
  float *mL = mM + kConsumerWarps * kMaxGroupMma;                  // [4][16]
  if (g < p.group) {
    float *dst = mO + (warp * kMaxGroupMma + g) * kD + tq * 2;
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt)
      *reinterpret_cast<float2 *>(dst + nt * 8) = make_float2(o[nt][0], o[nt][1]);
    if (tq == 0) {
      mM[warp * kMaxGroupMma + g] = m0;
      mL[warp * kMaxGroupMma + g] = l0;
    }
  }
  if (g + 8 < p.group) {
    float *dst = mO + (warp * kMaxGroupMma + g + 8) * kD + tq * 2;
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt)
      *reinterpret_cast<float2 *>(dst + nt * 8) = make_float2(o[nt][2], o[nt][3]);
    if (tq == 0) {
      mM[warp * kMaxGroupMma + g + 8] = m1;
      mL[warp * kMaxGroupMma + g + 8] = l1;
    }
  }
  named_bar_sync(1, kConsumerThreads);
  finalize_chunk<__half, kD>(p, gp, mO, mM, mL, b, hk, chunk, threadIdx.x, 1.0f, direct);
  finish_item<__half>(p, gp, w, hk, c_first, direct, 1.0f, threadIdx.x, kConsumerThreads, s_word, mO,
                      [] { named_bar_sync(1, kConsumerThreads); });
}

// ---- fp32 split kernel: FMA on unswizzled tiles ----------------------------------------------
// Tile = 32 tokens x 128 floats; warp w owns tokens [8w, 8w+8), lane owns dims [4*lane, +4).
template <bool kPaged, int kStages, int kGroup>
__global__ void __launch_bounds__(kThreads, 2)
gqa_split_f32_kernel(const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const DecodeParams p,
                     const GatherParams gp) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_plan[kPlanWords];
  uint8_t *smem = align_1024(smem_raw);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + SmemLayout<kStages>::kBarOffset);
  uint64_t *empty = full + kStages;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + kStages);
  volatile unsigned int *s_word = reinterpret_cast<volatile unsigned int *>(abort_flag + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == kConsumerThreads) {  // the producer's first lane, while warp 0 plans
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  // The producer warp asks for its first page ids (and the tensor maps) before the sequence's length
  // is known: with a host-planned chunk length the chunk's first token does not depend on it, and the
  // two trips to memory overlap instead of following one another.
  int spec_start = -1, spec_page = 0;
  if (warp == kConsumerWarps && lane == 0) {
    tma_prefetch_descriptor(&tmK);
    tma_prefetch_descriptor(&tmV);
  }
  grid_dependency_wait();  // nothing above reads what the kernel before this one writes
  if (warp == kConsumerWarps) {
    if (kPaged && !p.balanced) {
      spec_start = blockIdx.x * p.chunk_tokens;
      const int slot = (spec_start + lane * kTileTokensF32) / p.page_tokens;
      if (slot < p.max_blocks) spec_page = p.block_table[(size_t)blockIdx.z * p.max_blocks + slot];
    }
  }
  CtaWork w;
  const bool active = cta_work(p, s_plan, w);
  __syncthreads();
  if (!active) return;
  const int chunk = w.chunk, hk = blockIdx.y, b = w.b, L = w.L;
  if (L == 0) {
    emit_empty_item<float>(p, gp, b, hk, s_word);
    return;
  }
  const int first = first_visible(p, L);
  const int c_first = first / w.ct;  // chunks before it lie wholly outside the window
  int start = chunk * w.ct;
  const int end = min(L, start + w.ct);
  if (end <= first) return;  // the whole chunk lies before the window
  if (start < first) start = first / kTileTokensF32 * kTileTokensF32;  // skip whole tiles before it
  const int ntiles = (end - start + kTileTokensF32 - 1) / kTileTokensF32;
  const bool direct = p.direct_ok && w.n - c_first == 1;

  if (warp == kConsumerWarps) {
    produce_tiles<kPaged, kStages, kTileTokensF32, 1, 128>(&tmK, &tmV, p, smem, full, empty, abort_flag, b, hk,
                                                           start, ntiles, lane, spec_start, spec_page);
    return;
  }

  const float *qf = reinterpret_cast<const float *>(p.q);
  float4 qr[kGroup];
#pragma unroll
  for (int r = 0; r < kGroup; ++r)
    qr[r] = *reinterpret_cast<const float4 *>(
        qf + ((size_t)b * p.hq + (size_t)hk * kGroup + r) * kHeadDim + lane * 4);

  float4 o[kGroup];
  float m[kGroup], l[kGroup];  // m: running max of the raw dot products
#pragma unroll
  for (int r = 0; r < kGroup; ++r) {
    o[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    m[r] = -INFINITY;
    l[r] = 0.f;
  }
  const float sl2 = p.scale * kLog2e;

  bool ok = true;
  for (int i = 0; i < ntiles && ok; ++i) {
    const int s = i % kStages;
    const uint32_t phase = (i / kStages) & 1;
    ok = mbar_wait_bounded(&full[s], phase, abort_flag, p.wait_ns);
    if (!ok) break;
    const float *Ks = reinterpret_cast<const float *>(smem + (size_t)s * kStageBytes);
    const float *Vs = Ks + kTileTokensF32 * kHeadDim;
    const int valid = end - (start + i * kTileTokensF32 + warp * 8);  // tokens of this warp that exist
    const int lo = first - (start + i * kTileTokensF32 + warp * 8);   // tokens below lo precede the window

    float sc[kGroup][8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const float4 kv = *reinterpret_cast<const float4 *>(Ks + (warp * 8 + t) * kHeadDim + lane * 4);
#pragma unroll
      for (int r = 0; r < kGroup; ++r) {
        float a = qr[r].x * kv.x;
        a = fmaf(qr[r].y, kv.y, a);
        a = fmaf(qr[r].z, kv.z, a);
        a = fmaf(qr[r].w, kv.w, a);
        sc[r][t] = a;
      }
    }
#pragma unroll
    for (int r = 0; r < kGroup; ++r) {
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        float a = sc[r][t];
        a += __shfl_xor_sync(0xffffffffu, a, 16);
        a += __shfl_xor_sync(0xffffffffu, a, 8);
        a += __shfl_xor_sync(0xffffffffu, a, 4);
        a += __shfl_xor_sync(0xffffffffu, a, 2);
        a += __shfl_xor_sync(0xffffffffu, a, 1);
        sc[r][t] = (t < valid && t >= lo) ? a : -INFINITY;
      }
    }
#pragma unroll
    for (int r = 0; r < kGroup; ++r) {
      float mx = sc[r][0];
#pragma unroll
      for (int t = 1; t < 8; ++t) mx = fmaxf(mx, sc[r][t]);
      const float mn = fmaxf(m[r], mx);
      const float ms = (mn == -INFINITY) ? 0.f : mn;
      const float corr = exp2f((m[r] - ms) * sl2);
      m[r] = mn;
      float sum = 0.f;
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        sc[r][t] = exp2f((sc[r][t] - ms) * sl2);
        sum += sc[r][t];
      }
      l[r] = l[r] * corr + sum;
      o[r].x *= corr;
      o[r].y *= corr;
      o[r].z *= corr;
      o[r].w *= corr;
    }
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      float4 vv = *reinterpret_cast<const float4 *>(Vs + (warp * 8 + t) * kHeadDim + lane * 4);
      if (t >= valid || t < lo) vv = make_float4(0.f, 0.f, 0.f, 0.f);  // stale rows outside the range
#pragma unroll
      for (int r = 0; r < kGroup; ++r) {
        o[r].x = fmaf(sc[r][t], vv.x, o[r].x);
        o[r].y = fmaf(sc[r][t], vv.y, o[r].y);
        o[r].z = fmaf(sc[r][t], vv.z, o[r].z);
        o[r].w = fmaf(sc[r][t], vv.w, o[r].w);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }

  named_bar_sync(1, kConsumerThreads);
  if (*abort_flag) return;
  float *mO = reinterpret_cast<float *>(smem);
  float *mM = reinterpret_cast<float *>(smem + kStageBytes);
  float *mL = mM + kConsumerWarps * kMaxGroupMma;
#pragma unroll
  for (int r = 0; r < kGroup; ++r) {
    *reinterpret_cast<float4 *>(mO + (warp * kMaxGroupMma + r) * kHeadDim + lane * 4) = o[r];
    if (lane == 0) {
      mM[warp * kMaxGroupMma + r] = m[r];
      mL[warp * kMaxGroupMma + r] = l[r];
    }
  }
  named_bar_sync(1, kConsumerThreads);
  finalize_chunk<float, kHeadDim>(p, gp, mO, mM, mL, b, hk, chunk, threadIdx.x, sl2, direct);
  finish_item<float>(p, gp, w, hk, c_first, direct, sl2, threadIdx.x, kConsumerThreads, s_word, mO,
                     [] { named_bar_sync(1, kConsumerThreads); });
}

// ---- generic split kernel: any head_dim <= 256, any group, any alignment ---------------------------
// For the shapes the TMA kernels do not take (head_dim != 128, pointers off 16 bytes, odd groups).
// Same split-K scheme and partial format; tiles of keys are staged in shared memory as fp32 with plain
// coalesced loads (a warp reads a row), every query head of the KV head works on the staged tile:
//   scores   thread = (key, head subset): one K value from shared memory feeds all its heads
//   softmax  warp = head: tile maximum and sum by shuffles, once per tile instead of once per key
//   P.V      thread = (output column, head subset): one V value feeds all its heads
// Rows are padded to d + 1 floats so that "thread = key" reads are conflict-free.  Maxima are raw dot
// products; the scale enters inside the exponent (combine is told so).
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

constexpr int kGenThreads = 128, kGenMaxHeads = 16, kGenMaxAcc = 16, kGenLoadBatch = 8;
__host__ __device__ inline int gen_tile_tokens(int d) { return d <= 128 ? 64 : 32; }
// Row stride of the staged tiles in floats: d + 4 when head_dim is a multiple of 8 - rows stay 16-byte
// aligned and "thread = key" float4 reads are conflict-free ((d + 4) / 4 is odd) - else d + 1.
__host__ __device__ inline int gen_row_stride(int d) { return d % 8 == 0 ? d + 4 : d + 1; }
__host__ __device__ inline int gen_head_batch(int d, int group) {
  const int cap = d <= 128 ? kGenMaxHeads : kGenMaxHeads / 2;
  return group < cap ? group : cap;
}
inline size_t gen_smem_bytes(int d, int group) {
  const int tt = gen_tile_tokens(d), gb = gen_head_batch(d, group);
  return sizeof(float) * ((size_t)2 * tt * gen_row_stride(d) + (((size_t)gb * d + 3) & ~size_t(3)) + (size_t)gb * tt +
                          3 * kGenMaxHeads) +
         sizeof(long long) * 64 + 8;
}

// Scores of one key against kNh query heads (sub, sub + nsub, ...): the K value is read once per
// head_dim element; heads past `gb` are computed on a clamped index and not stored.
template <int kNh>
__device__ __forceinline__ void gen_scores(const float *Ks, const float *q_s, float *p_s, int key, int nt, int sub,
                                           int nsub, int gb, int d, int dp, int tt) {
  float sc[kNh];
  const float *qr[kNh];
#pragma unroll
  for (int hh = 0; hh < kNh; ++hh) {
    sc[hh] = 0.f;
    qr[hh] = q_s + min(sub + hh * nsub, gb - 1) * d;
  }
  if (key < nt) {
    const float *kr = Ks + key * dp;
    if (d % 8 == 0) {  // 16-byte reads, the same order of additions
      const float4 *kr4 = reinterpret_cast<const float4 *>(kr);
#pragma unroll 2
      for (int c4 = 0; c4 < d / 4; ++c4) {
        const float4 kv = kr4[c4];
#pragma unroll
        for (int hh = 0; hh < kNh; ++hh) {
          const float4 qv = reinterpret_cast<const float4 *>(qr[hh])[c4];
          sc[hh] = fmaf(qv.w, kv.w, fmaf(qv.z, kv.z, fmaf(qv.y, kv.y, fmaf(qv.x, kv.x, sc[hh]))));
        }
      }
    } else {
#pragma unroll 4
      for (int c = 0; c < d; ++c) {
        const float kv = kr[c];
#pragma unroll
        for (int hh = 0; hh < kNh; ++hh) sc[hh] = fmaf(qr[hh][c], kv, sc[hh]);
      }
    }
  }
#pragma unroll
  for (int hh = 0; hh < kNh; ++hh)
    if (sub + hh * nsub < gb) p_s[(sub + hh * nsub) * tt + key] = key < nt ? sc[hh] : -INFINITY;
}

// acc[0..kNh) = acc * corr + P . V for one output column and kNh heads (sub, sub + nsub, ...).
template <int kNh>
__device__ __forceinline__ void gen_pv(const float *Vs, const float *p_s, const float *corr_s, float *acc, int c,
                                       int nt, int sub, int nsub, int gb, int dp, int tt) {
  const float *pr[kNh];
#pragma unroll
  for (int hh = 0; hh < kNh; ++hh) {
    const int r = min(sub + hh * nsub, gb - 1);
    pr[hh] = p_s + r * tt;
    acc[hh] *= corr_s[r];
  }
  int t = 0;
  for (; t + 4 <= nt; t += 4) {  // four keys per step: the weights come as one 16-byte read per head
    const float v0 = Vs[t * dp + c], v1 = Vs[(t + 1) * dp + c], v2 = Vs[(t + 2) * dp + c], v3 = Vs[(t + 3) * dp + c];
#pragma unroll
    for (int hh = 0; hh < kNh; ++hh) {
      const float4 pw = *reinterpret_cast<const float4 *>(pr[hh] + t);
      acc[hh] = fmaf(pw.w, v3, fmaf(pw.z, v2, fmaf(pw.y, v1, fmaf(pw.x, v0, acc[hh]))));
    }
  }
  for (; t < nt; ++t) {
    const float vv = Vs[t * dp + c];
#pragma unroll
    for (int hh = 0; hh < kNh; ++hh) acc[hh] = fmaf(pr[hh][t], vv, acc[hh]);
  }
}

template <typename T, bool kPaged>
__global__ void __launch_bounds__(kGenThreads, 3)
gqa_split_generic_kernel(const T *k, const T *v, const DecodeParams p, const GatherParams gp, int d) {
  extern __shared__ __align__(16) float gsm[];
  __shared__ int s_plan[kPlanWords];
  __shared__ unsigned int s_word[2];
  grid_dependency_wait();
  CtaWork w;
  const bool active = cta_work(p, s_plan, w);
  __syncthreads();
  if (!active) return;
  const int chunk = w.chunk, hk = blockIdx.y, b = w.b, L = w.L;
  if (L == 0) {
    emit_empty_item<T>(p, gp, b, hk, s_word);
    return;
  }
  const int first = first_visible(p, L);
  const int c_first = first / w.ct;  // chunks before it lie wholly outside the window
  int start = chunk * w.ct;
  const int end = min(L, start + w.ct);
  if (end <= first) return;
  if (start < first) start = first;
  const bool direct = p.direct_ok && w.n - c_first == 1;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tt = gen_tile_tokens(d), gb_max = gen_head_batch(d, p.group), dp = gen_row_stride(d);
  float *Ks = gsm, *Vs = Ks + tt * dp, *q_s = Vs + tt * dp, *p_s = q_s + ((gb_max * d + 3) & ~3);  // all 16-byte aligned
  float *m_s = p_s + gb_max * tt, *l_s = m_s + kGenMaxHeads, *corr_s = l_s + kGenMaxHeads;
  long long *row_s = reinterpret_cast<long long *>(
      (reinterpret_cast<uintptr_t>(corr_s + kGenMaxHeads) + 7) & ~uintptr_t(7));  // [tt] element offsets of the tile's rows
  const T *qp = reinterpret_cast<const T *>(p.q);
  const float dom = p.scale * kLog2e;
  // thread roles
  const int nsub_qk = kGenThreads / tt, key = tid % tt, sub_qk = tid / tt;
  const int d_eff = d < kGenThreads ? d : kGenThreads;
  const int nsub_pv = kGenThreads / d_eff, col = tid % d_eff, sub_pv = tid / d_eff;
  const bool pv_active = sub_pv < nsub_pv;
  const int passes = (d + kGenThreads - 1) / kGenThreads;  // 1, or 2 for head_dim > 128

  for (int h0 = 0; h0 < p.group; h0 += gb_max) {  // head batches: one unless group > 16 (8 for head_dim > 128)
    const int gb = min(gb_max, p.group - h0);
    __syncthreads();  // the previous batch is done with shared memory
    for (int i = tid; i < gb * d; i += kGenThreads)
      q_s[i] = to_f32(qp[((size_t)b * p.hq + hk * p.group + h0 + i / d) * d + i % d]);
    if (tid < kGenMaxHeads) {
      m_s[tid] = -INFINITY;
      l_s[tid] = 0.f;
      corr_s[tid] = 1.f;
    }
    float acc[kGenMaxAcc];
#pragma unroll
    for (int a = 0; a < kGenMaxAcc; ++a) acc[a] = 0.f;
    const int nh_pv = pv_active ? (gb - sub_pv + nsub_pv - 1) / nsub_pv : 0;  // heads sub_pv, sub_pv + nsub_pv, ...
    const int nh_qk = (gb - sub_qk + nsub_qk - 1) / nsub_qk;

    for (int t0 = start; t0 < end; t0 += tt) {
      const int nt = min(tt, end - t0);
      // ---- stage the tile ----
      // Row offsets first (one page lookup per key), then the nt * d elements of K and of V spread
      // over the threads, consecutive threads on consecutive elements; eight loads of each are issued
      // before the first shared-memory store so that a CTA keeps ~8 KB in flight.
      if (tid < tt) {
        long long off = -1;
        if (tid < nt) {
          const int tok = t0 + tid;
          if (kPaged) {
            const int page = p.block_table[(size_t)b * p.max_blocks + tok / p.page_tokens];
            if (page >= 0 && page < p.num_pages)
              off = (long long)((((size_t)page * p.hkv + hk) * p.page_tokens + tok % p.page_tokens) * d);
            else
              atomicOr(&g_error_word, AXB200_ERR_BAD_PAGE);
          } else {
            off = (long long)(((size_t)tok * p.hkv + hk) * d);
          }
        }
        row_s[tid] = off;
      }
      __syncthreads();
      const int n_elem = nt * d;
      int er = tid / d, ec = tid % d;  // row and column of this thread's next element; they advance by 128
      for (int e0 = 0; e0 < n_elem; e0 += kGenThreads * kGenLoadBatch) {
        float kr[kGenLoadBatch], vr[kGenLoadBatch];
        int at[kGenLoadBatch];
#pragma unroll
        for (int u = 0; u < kGenLoadBatch; ++u) {
          kr[u] = vr[u] = 0.f;
          at[u] = -1;
          if (e0 + u * kGenThreads + tid < n_elem) {
            at[u] = er * dp + ec;
            const long long off = row_s[er];
            if (off >= 0) {
              kr[u] = to_f32(k[off + ec]);
              vr[u] = to_f32(v[off + ec]);
            }
          }
          ec += kGenThreads;
          while (ec >= d) {
            ec -= d;
            ++er;
          }
        }
#pragma unroll
        for (int u = 0; u < kGenLoadBatch; ++u)
          if (at[u] >= 0) {
            Ks[at[u]] = kr[u];
            Vs[at[u]] = vr[u];
          }
      }
      __syncthreads();
      // ---- scores ----
      if (nh_qk > 4) gen_scores<8>(Ks, q_s, p_s, key, nt, sub_qk, nsub_qk, gb, d, dp, tt);
      else if (nh_qk > 2) gen_scores<4>(Ks, q_s, p_s, key, nt, sub_qk, nsub_qk, gb, d, dp, tt);
      else if (nh_qk == 2) gen_scores<2>(Ks, q_s, p_s, key, nt, sub_qk, nsub_qk, gb, d, dp, tt);
      else if (nh_qk == 1) gen_scores<1>(Ks, q_s, p_s, key, nt, sub_qk, nsub_qk, gb, d, dp, tt);
      __syncthreads();
      // ---- online softmax of the tile, one warp per head ----
      for (int r = warp; r < gb; r += kGenThreads / 32) {
        float s0 = p_s[r * tt + lane], s1 = tt > 32 ? p_s[r * tt + 32 + lane] : -INFINITY;
        float mx = fmaxf(s0, s1);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        const float m_old = m_s[r], m_new = fmaxf(m_old, mx);
        const float corr = m_old == -INFINITY ? 0.f : exp2f((m_old - m_new) * dom);
        const float p0 = s0 == -INFINITY ? 0.f : exp2f((s0 - m_new) * dom);
        const float p1 = s1 == -INFINITY ? 0.f : exp2f((s1 - m_new) * dom);
        p_s[r * tt + lane] = p0;
        if (tt > 32) p_s[r * tt + 32 + lane] = p1;
        float ps = p0 + p1;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
        __syncwarp();
        if (lane == 0) {
          m_s[r] = m_new;
          l_s[r] = l_s[r] * corr + ps;
          corr_s[r] = corr;
        }
      }
      __syncthreads();
      // ---- O = O * corr + P . V ----
      // accumulators: head_dim <= 128: acc[hh], up to 16 heads; above: acc[pass * 8 + hh], up to 8 heads.
      // A head past the batch is computed on a clamped index; its accumulator is never written out.
      if (pv_active && passes == 1) {
        if (col < d) {
          if (nh_pv > 8) gen_pv<16>(Vs, p_s, corr_s, acc, col, nt, sub_pv, nsub_pv, gb, dp, tt);
          else if (nh_pv > 4) gen_pv<8>(Vs, p_s, corr_s, acc, col, nt, sub_pv, nsub_pv, gb, dp, tt);
          else if (nh_pv > 2) gen_pv<4>(Vs, p_s, corr_s, acc, col, nt, sub_pv, nsub_pv, gb, dp, tt);
          else if (nh_pv == 2) gen_pv<2>(Vs, p_s, corr_s, acc, col, nt, sub_pv, nsub_pv, gb, dp, tt);
          else if (nh_pv == 1) gen_pv<1>(Vs, p_s, corr_s, acc, col, nt, sub_pv, nsub_pv, gb, dp, tt);
        }
      } else if (pv_active) {
#pragma unroll
        for (int ps = 0; ps < 2; ++ps) {
          const int c = col + ps * kGenThreads;
          if (c < d) {
            float *a = acc + ps * (kGenMaxAcc / 2);
            if (nh_pv > 4) gen_pv<8>(Vs, p_s, corr_s, a, c, nt, 0, 1, gb, dp, tt);
            else if (nh_pv > 2) gen_pv<4>(Vs, p_s, corr_s, a, c, nt, 0, 1, gb, dp, tt);
            else if (nh_pv == 2) gen_pv<2>(Vs, p_s, corr_s, a, c, nt, 0, 1, gb, dp, tt);
            else if (nh_pv == 1) gen_pv<1>(Vs, p_s, corr_s, a, c, nt, 0, 1, gb, dp, tt);
          }
        }
      }
      __syncthreads();  // the tile buffers and p_s are free again
    }
    // ---- this chunk's result for the batch's heads ----
    if (pv_active) {
      auto emit = [&](int r, int c, float a) {
        const int h = hk * p.group + h0 + r;
        if (direct) {
          emit_final<T>(p, gp, b, h, c, a, m_s[r], l_s[r]);
        } else {
          const size_t slot = ((size_t)b * p.hq + h) * p.max_chunks + chunk;
          p.part_o[slot * d + c] = a;
        }
      };
      if (passes == 1) {
        if (col < d) {
#pragma unroll
          for (int hh = 0; hh < kGenMaxAcc; ++hh)
            if (hh < nh_pv) emit(sub_pv + hh * nsub_pv, col, acc[hh]);
        }
      } else {
#pragma unroll
        for (int ps = 0; ps < 2; ++ps) {
          const int c = col + ps * kGenThreads;
#pragma unroll
          for (int hh = 0; hh < kGenMaxAcc / 2; ++hh)
            if (c < d && hh < nh_pv) emit(hh, c, acc[ps * (kGenMaxAcc / 2) + hh]);
        }
      }
    }
    if (!direct && tid < gb) {
      const size_t slot = ((size_t)b * p.hq + hk * p.group + h0 + tid) * p.max_chunks + chunk;
      p.part_ml[slot * 2 + 0] = m_s[tid];
      p.part_ml[slot * 2 + 1] = l_s[tid];
    }
  }
  finish_item<T>(p, gp, w, hk, c_first, direct, dom, tid, kGenThreads, s_word, Ks, [] { __syncthreads(); });
}

// ---- combine: log-sum-exp merge of a sequence's chunk partials --------------------------------
// The separate form of the merge, used when a launch has no arrival counters (the fused merge is
// switched off, no counter region is free, or the launch has more items than a region holds).  One
// CTA per (sequence, query head); thread t owns output dims t, t + 128.  `dom` is the exponent domain
// of the stored maxima.  Same arithmetic, through the same functions, as the fused merge.  With
// peers, every CTA is an item of the exchange.
template <typename OutT>
__global__ void __launch_bounds__(128)
gqa_combine_kernel(const DecodeParams p, const GatherParams gp, float dom) {
  __shared__ int s_plan[kPlanWords];
  __shared__ unsigned int s_word[2];
  __shared__ __align__(16) float s_merge[2 * 4 * kMergeRow];
  const int h = blockIdx.x, b = blockIdx.y;
  int L, ct, n;
  sequence_plan(p, b, s_plan, &L, &ct, &n);
  const int c_first = first_visible(p, L) / ct;  // first chunk that holds visible tokens
  if (L > 0) {
    merge_head_range<OutT>(p, gp, b, h, 1, c_first, n, dom, threadIdx.x, blockDim.x, s_merge, [] { __syncthreads(); });
  } else {
    for (int t = threadIdx.x; t < p.d; t += blockDim.x) emit_final<OutT>(p, gp, b, h, t, 0.f, -INFINITY, 0.f);
  }
  if (gp.world)
    publish_and_wait(gp, gridDim.x * gridDim.y, p.wait_ns, threadIdx.x, s_word, [] { __syncthreads(); });
}

// ---- context-parallel decode: one sequence's tokens spread over the GPUs --------------------------
// Each rank caches a share of every sequence's tokens (softmax does not care which) and attends its
// share; the end of each (sequence, head) stores the un-normalised record [O_loc(d), m_loc, l_loc]
// into every rank's record buffer (emit_final) and the ranks exchange generation flags.  Merge kernel
// (next launch, local reads only): the log-sum-exp merge of the `world` records gives the same output
// on every rank.
template <typename OutT>
__global__ void __launch_bounds__(128)
cp_merge_kernel(const float *records, OutT *out, int world, int d, float dom) {
  const size_t bh = (size_t)blockIdx.y * gridDim.x + blockIdx.x;  // (b, h) row
  const float *rec = records + bh * world * (d + 2);
  float M = -INFINITY;
  for (int r = 0; r < world; ++r) M = fmaxf(M, rec[r * (d + 2) + d]);
  float L = 0.f;
  for (int r = 0; r < world; ++r) {
    const float m = rec[r * (d + 2) + d];
    if (m != -INFINITY) L = fmaf(rec[r * (d + 2) + d + 1], exp2f((m - M) * dom), L);
  }
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  for (int c0 = threadIdx.x; c0 < d; c0 += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < world; ++r) {
      const float m = rec[r * (d + 2) + d];
      if (m != -INFINITY) acc = fmaf(exp2f((m - M) * dom), rec[r * (d + 2) + c0], acc);
    }
    out[bh * d + c0] = static_cast<OutT>(acc * inv);
  }
}

// ---- host side ----------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// 4-D tensor map over a cache.  Paged: dims (d, page_tokens, hkv, num_pages), box
// (box_d, tile, 1, 1).  Token-major: dims (d, hkv, skv, 1), box (box_d, 1, tile, 1).
bool make_map(CUtensorMap *map, const void *base, int dtype, bool paged, int d, int hkv,
              int64_t tokens_or_page_tokens, int64_t num_pages, int tile) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const size_t es = dtype_size(dtype);
  const bool f16 = dtype == AXB200_FLOAT16;
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
  const cuuint32_t box_d = f16 ? 64 : 128;
  if (paged) {
    dims[0] = d; dims[1] = tokens_or_page_tokens; dims[2] = hkv; dims[3] = num_pages;
    strides[0] = d * es;
    strides[1] = tokens_or_page_tokens * d * es;
    strides[2] = (cuuint64_t)hkv * tokens_or_page_tokens * d * es;
    box[0] = box_d; box[1] = tile; box[2] = 1; box[3] = 1;
  } else {
    dims[0] = d; dims[1] = hkv; dims[2] = tokens_or_page_tokens; dims[3] = 1;
    strides[0] = d * es;
    strides[1] = (cuuint64_t)hkv * d * es;
    strides[2] = (cuuint64_t)tokens_or_page_tokens * hkv * d * es;
    box[0] = box_d; box[1] = 1; box[2] = tile; box[3] = 1;
  }
  CUresult r = fn(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
                  const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  f16 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// ---- host settings -------------------------------------------------------------------------------
std::mutex g_settings_mu;
unsigned long long g_wait_limit_ns = kWaitNanos;
bool g_fused_merge = true;
bool g_merge_pairs = true;
bool g_step_fused = true;  // axb200_decode_step_paged may use the one-launch form
bool g_dependent_launch = true;
bool g_device_plan = false;  // measured slower than the host plan on every one-wave case tried (see make_plan)
int g_forced_chunk_tiles = 0;  // > 0: overrides the planned chunk length (tuning and tests)

// ---- the chunk plan: "a split count chosen from the context length and SM count" -----------------
// `slots` CTAs are resident at once (2 per SM).  A large problem (more than about 8 waves of CTAs of
// 16 tiles) is cut on the host into chunks of 16..64 tiles of 64 tokens, one length for the whole
// launch: long enough to amortise a CTA's pipeline fill, many enough for the hardware scheduler to
// balance ragged lengths; CTAs past a sequence's end exit at once.  A problem whose (sequence, head)
// items fit one wave is planned on the device instead (`balanced`): the CTAs read the actual lengths
// and pick the smallest chunk length for which all chunks fit the wave, so every CTA of the wave
// streams about the same number of bytes whatever the mix of lengths.  In between (more items than
// slots, little work each) every sequence is one chunk.  At most kMaxChunks chunks per sequence.
struct Plan {
  int chunk_tokens, max_chunks;
  int balanced, budget;
  size_t part_o_bytes, part_ml_bytes;
};

Plan make_plan(int batch, int hq, int hkv, int d, int64_t max_len) {
  if (max_len < 1) max_len = 1;
  Plan pl{};
  const int64_t tiles = (max_len + 63) / 64;
  const int64_t slots = (int64_t)sm_count() * 2;
  const int64_t items = (int64_t)batch * hkv;
  const int64_t total = items * tiles;
  int64_t chunk_tiles;
  if (total >= 16 * 8 * slots) {
    chunk_tiles = (total + 8 * slots - 1) / (8 * slots);
    if (chunk_tiles < 16) chunk_tiles = 16;
    if (chunk_tiles > 64) chunk_tiles = 64;
  } else if (items <= slots && batch <= kMaxBalancedBatch && g_device_plan) {
    pl.balanced = 1;
    pl.budget = (int)(slots / hkv);
    chunk_tiles = kMinChunkTiles;
  } else {
    int64_t per_item = slots / items;  // chunks each (sequence, head) may have within one wave
    if (per_item < 1) per_item = 1;
    chunk_tiles = (tiles + per_item - 1) / per_item;
    if (chunk_tiles < kMinChunkTiles) chunk_tiles = kMinChunkTiles;
  }
  if (g_forced_chunk_tiles > 0) {
    pl.balanced = 0;
    chunk_tiles = g_forced_chunk_tiles;
  }
  while ((tiles + chunk_tiles - 1) / chunk_tiles > kMaxChunks) chunk_tiles *= 2;
  pl.chunk_tokens = (int)(chunk_tiles * 64);
  pl.max_chunks = (int)((max_len + pl.chunk_tokens - 1) / pl.chunk_tokens);
  if (pl.balanced && pl.max_chunks > pl.budget) pl.max_chunks = pl.budget;  // one sequence cannot have more
  if (pl.max_chunks < 1) pl.max_chunks = 1;
  pl.part_o_bytes = ((size_t)batch * hq * pl.max_chunks * d * sizeof(float) + 15) & ~size_t(15);  // (m, l) pairs are read as 8 bytes
  pl.part_ml_bytes = (size_t)batch * hq * pl.max_chunks * 2 * sizeof(float);
  return pl;
}

// Opts a kernel in to more than 48 KB of dynamic shared memory, once per (kernel, device).
bool set_smem(const void *kernel, int bytes) {
  static std::mutex mu;
  static std::set<std::pair<const void *, int>> done;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (done.count({kernel, dev})) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) !=
      cudaSuccess)
    return false;
  done.insert({kernel, dev});
  return true;
}

constexpr int kStagesDefault = 3;

// Launches a split kernel; with `dependent` the launch carries the programmatic-stream-serialization
// attribute, so its CTAs may be scheduled while the kernel before it in the stream (the append, in a
// decode step) is finishing - they stop at grid_dependency_wait() until that kernel is complete.
template <typename Kern, typename... Args>
int launch_split(Kern kern, dim3 grid, int threads, int smem, cudaStream_t st, bool dependent, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...) == cudaSuccess ? launch_status() : AXB200_DEVICE_ERROR;
}

// head_dim 64 has half the bytes per stage: twice the stages keep the same 96 KB per CTA in flight
template <bool kPaged, int kD, bool kStep>
int launch_f16_d(const CUtensorMap &mk, const CUtensorMap &mv, const DecodeParams &p,
                 const GatherParams &g, dim3 grid, cudaStream_t st, const StepParams &sp) {
  constexpr int kStages = kStagesDefault * 128 / kD;
  auto kern = gqa_split_f16_kernel<kPaged, kStages, 2, kD, kStep>;
  constexpr int smem = SmemLayout<kStages, 256 * kD>::kDynamicBytes;
  if (!set_smem(reinterpret_cast<const void *>(kern), smem)) return AXB200_DEVICE_ERROR;
  return launch_split(kern, grid, kThreads, smem, st, g_dependent_launch, mk, mv, p, g, sp);
}

// step: the launch appends the step's token itself (paged, head_dim 64 or 128 exactly)
template <bool kPaged>
int launch_f16(const CUtensorMap &mk, const CUtensorMap &mv, const DecodeParams &p,
               const GatherParams &g, dim3 grid, cudaStream_t st, const StepParams *step) {
  if (kPaged && step)
    return p.d == 64 ? launch_f16_d<true, 64, true>(mk, mv, p, g, grid, st, *step)
                     : launch_f16_d<true, 128, true>(mk, mv, p, g, grid, st, *step);
  static const StepParams none{};
  return p.d <= 64 ? launch_f16_d<kPaged, 64, false>(mk, mv, p, g, grid, st, none)
                   : launch_f16_d<kPaged, 128, false>(mk, mv, p, g, grid, st, none);
}

template <bool kPaged, int kGroup>
int launch_f32_g(const CUtensorMap &mk, const CUtensorMap &mv, const DecodeParams &p,
                 const GatherParams &g, dim3 grid, cudaStream_t st) {
  auto kern = gqa_split_f32_kernel<kPaged, kStagesDefault, kGroup>;
  constexpr int smem = SmemLayout<kStagesDefault>::kDynamicBytes;
  if (!set_smem(reinterpret_cast<const void *>(kern), smem)) return AXB200_DEVICE_ERROR;
  return launch_split(kern, grid, kThreads, smem, st, g_dependent_launch, mk, mv, p, g);
}

template <bool kPaged>
int launch_f32(const CUtensorMap &mk, const CUtensorMap &mv, const DecodeParams &p,
               const GatherParams &g, dim3 grid, cudaStream_t st) {
  switch (p.group) {
    case 1: return launch_f32_g<kPaged, 1>(mk, mv, p, g, grid, st);
    case 2: return launch_f32_g<kPaged, 2>(mk, mv, p, g, grid, st);
    case 4: return launch_f32_g<kPaged, 4>(mk, mv, p, g, grid, st);
    case 8: return launch_f32_g<kPaged, 8>(mk, mv, p, g, grid, st);
    default: return AXB200_UNSUPPORTED_TYPE;
  }
}

// ---- optional timing of the split kernel alone ---------------------------------------------------
// When enabled (axb200_profile_enable), every decode call brackets its split-kernel launch with
// a pair of CUDA events on the launching stream; axb200_profile_collect sums them.  Off by
// default; not for use during stream capture.
constexpr int kProfilePairs = 4096;
struct ProfileState {
  bool enabled = false;
  int used = 0;
  cudaEvent_t start[kProfilePairs];
  cudaEvent_t stop[kProfilePairs];
  bool created = false;
};
ProfileState g_profile;
std::mutex g_profile_mu;

int profile_slot() {
  std::lock_guard<std::mutex> lock(g_profile_mu);
  if (!g_profile.enabled || g_profile.used >= kProfilePairs) return -1;
  return g_profile.used++;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }


// Counter region of the fused merge for launches that use `workspace` on the current device.  Two
// launches may overlap on the GPU only if they use different workspaces (they would race on the
// partials otherwise), so a region per workspace pointer keeps their counters apart.  -1: none free.
int arrival_region_for(const void *workspace, int64_t items) {
  if (items > kArrivalSlots) return -1;
  static std::map<std::pair<int, const void *>, int> table;
  static int used[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  std::lock_guard<std::mutex> lock(g_settings_mu);
  if (!g_fused_merge) return -1;
  auto it = table.find({dev, workspace});
  if (it != table.end()) return it->second;
  if (used[dev] >= kArrivalRegions) return -1;
  const int region = used[dev]++;
  table[{dev, workspace}] = region;
  return region;
}

// Common launcher.  `paged` selects the cache layout; for the token-major layout `tokens` is skv.
int decode_impl(bool paged, const void *q, void *out, const void *k, const void *v,
                const int32_t *block_table, const int32_t *seq_lens, int fixed_len, int batch,
                int hq, int hkv, int d, int page_tokens, int max_blocks, int num_pages,
                int64_t max_len, int dtype, void *workspace, size_t workspace_bytes,
                cudaStream_t st, const GatherParams *gather = nullptr, int window = 0,
                int causal_rows = 0, int row_offset = 0, const StepParams *step = nullptr) {
  if (dtype != AXB200_FLOAT16 && dtype != AXB200_FLOAT32) return AXB200_UNSUPPORTED_TYPE;
  if (!q || (!out && !(gather && gather->mode == 0)) || !k || !v) return AXB200_INVALID_PTR;
  if (batch <= 0 || hq <= 0 || hkv <= 0 || d <= 0 || max_len <= 0) return AXB200_INVALID_ARGUMENT;
  if (hq % hkv != 0) return AXB200_SHAPE_MISMATCH;
  if (d > 256 || max_len > (int64_t)INT32_MAX - 4096) return AXB200_INVALID_ARGUMENT;
  if (paged && (!block_table || !seq_lens)) return AXB200_INVALID_PTR;
  if (paged && (page_tokens <= 0 || page_tokens % 64 != 0 || max_blocks <= 0 || num_pages <= 0))
    return AXB200_INVALID_ARGUMENT;
  if (paged && (int64_t)max_blocks * page_tokens < max_len) return AXB200_INVALID_ARGUMENT;
  if (batch > 65535 || hkv > 65535) return AXB200_INVALID_ARGUMENT;
  if (window < 0) return AXB200_INVALID_ARGUMENT;

  const Plan pl = make_plan(batch, hq, hkv, d, max_len);
  DecodeParams p{};
  p.q = q;
  p.out = out;
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.fixed_len = fixed_len;
  p.batch = batch;
  p.hq = hq;
  p.hkv = hkv;
  p.group = hq / hkv;
  p.d = d;
  p.page_tokens = paged ? page_tokens : 1;
  p.max_blocks = max_blocks;
  p.num_pages = num_pages;
  p.chunk_tokens = pl.chunk_tokens;
  p.max_chunks = pl.max_chunks;
  p.balanced = pl.balanced;
  p.budget = pl.budget;
  p.scale = 1.0f / sqrtf((float)d);
  p.window = window;
  p.causal_rows = causal_rows;
  p.row_offset = row_offset;
  {
    std::lock_guard<std::mutex> lock(g_settings_mu);
    p.wait_ns = g_wait_limit_ns;
  }
  const bool need_ws = pl.max_chunks > 1;
  if (need_ws) {
    if (!workspace || workspace_bytes < pl.part_o_bytes + pl.part_ml_bytes)
      return AXB200_INVALID_ARGUMENT;
    if (!aligned16(workspace)) return AXB200_INVALID_PTR;
    p.part_o = reinterpret_cast<float *>(workspace);
    p.part_ml = reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + pl.part_o_bytes);
  }
  // Who writes the result.  One chunk per sequence at most: the split CTA itself.  Else the last CTA
  // of each (sequence, KV head) when a counter region is to be had, else a combine kernel - which
  // then also emits the single-chunk sequences, so that every item passes through one place.
  p.arrival_region = need_ws || step ? arrival_region_for(workspace, (int64_t)batch * hkv) : -1;
  const bool combine_kernel = need_ws && p.arrival_region < 0;
  p.direct_ok = !combine_kernel;
  p.merge_pairs = g_merge_pairs;
  GatherParams g{};
  if (gather) g = *gather;
  const dim3 grid = pl.balanced ? dim3(pl.budget, hkv, 1) : dim3(pl.max_chunks, hkv, batch);
  const bool f16 = dtype == AXB200_FLOAT16;
  const float dom = p.scale * kLog2e;

  const bool f16_in = dtype == AXB200_FLOAT16;
  // fp16: any head size that is a multiple of 8 up to 128 (rows stay 16-byte multiples for the tensor
  // map; narrower heads ride in the 64- or 128-wide tile with zero fill); fp32: 128
  bool tiled = (d == kHeadDim || (f16_in && d % 8 == 0 && d <= kHeadDim)) && aligned16(k) && aligned16(v) &&
               aligned16(q) && encode_fn();
  if (tiled && f16 && p.group > kMaxGroupMma) tiled = false;
  if (tiled && !f16 && !(p.group == 1 || p.group == 2 || p.group == 4 || p.group == 8))
    tiled = false;
  // The step in one launch needs the fp16 TMA kernel at its full tile width, host-planned chunks and a
  // counter region (which is looked up by workspace pointer); nothing has been launched at this point.
  if (step && !(paged && f16 && tiled && (d == 64 || d == 128) && !pl.balanced && window == 0 && workspace &&
                aligned16(workspace) && p.arrival_region >= 0 && aligned16(step->k_new) && aligned16(step->v_new)))
    return kStepNotFused;

  CUtensorMap mk, mv;
  if (tiled) {
    const int tile = f16 ? kTileTokensF16 : kTileTokensF32;
    const int64_t tok = paged ? page_tokens : max_len;
    if (!make_map(&mk, k, dtype, paged, d, hkv, tok, num_pages, tile) ||
        !make_map(&mv, v, dtype, paged, d, hkv, tok, num_pages, tile))
      return AXB200_INTERNAL_ERROR;
  }
  int status;
  const int prof = profile_slot();
  if (prof >= 0) cudaEventRecord(g_profile.start[prof], st);
  if (tiled) {
    if (f16)
      status = paged ? launch_f16<true>(mk, mv, p, g, grid, st, step) : launch_f16<false>(mk, mv, p, g, grid, st, nullptr);
    else
      status = paged ? launch_f32<true>(mk, mv, p, g, grid, st) : launch_f32<false>(mk, mv, p, g, grid, st);
  } else {
    const int gsmem = (int)gen_smem_bytes(d, p.group);
    bool ok_attr = true;
    if (f16) {
      auto kk = reinterpret_cast<const __half *>(k), vv = reinterpret_cast<const __half *>(v);
      if (paged) {
        auto kern = gqa_split_generic_kernel<__half, true>;
        ok_attr = set_smem(reinterpret_cast<const void *>(kern), 100 * 1024);
        if (ok_attr) kern<<<grid, kGenThreads, gsmem, st>>>(kk, vv, p, g, d);
      } else {
        auto kern = gqa_split_generic_kernel<__half, false>;
        ok_attr = set_smem(reinterpret_cast<const void *>(kern), 100 * 1024);
        if (ok_attr) kern<<<grid, kGenThreads, gsmem, st>>>(kk, vv, p, g, d);
      }
    } else {
      auto kk = reinterpret_cast<const float *>(k), vv = reinterpret_cast<const float *>(v);
      if (paged) {
        auto kern = gqa_split_generic_kernel<float, true>;
        ok_attr = set_smem(reinterpret_cast<const void *>(kern), 100 * 1024);
        if (ok_attr) kern<<<grid, kGenThreads, gsmem, st>>>(kk, vv, p, g, d);
      } else {
        auto kern = gqa_split_generic_kernel<float, false>;
        ok_attr = set_smem(reinterpret_cast<const void *>(kern), 100 * 1024);
        if (ok_attr) kern<<<grid, kGenThreads, gsmem, st>>>(kk, vv, p, g, d);
      }
    }
    status = ok_attr ? launch_status() : AXB200_DEVICE_ERROR;
  }
  if (prof >= 0) cudaEventRecord(g_profile.stop[prof], st);  // recorded on every path once the start is
  if (status != AXB200_OK) return status;
  // The fp16 tiled kernel keeps its maxima in the log2 domain (already scaled); the fp32 and
  // generic kernels keep raw dot products and scale inside the exponent.
  const float cdom = (tiled && f16) ? 1.0f : dom;
  const dim3 cgrid(hq, batch);
  if (combine_kernel) {
    if (f16) gqa_combine_kernel<__half><<<cgrid, 128, 0, st>>>(p, g, cdom);
    else gqa_combine_kernel<float><<<cgrid, 128, 0, st>>>(p, g, cdom);
    status = launch_status();
    if (status != AXB200_OK) return status;
  }
  if (gather && gather->mode == 1) {  // every rank's records are here: merge them (local reads only)
    const float *records = static_cast<const float *>(gather->peer_out[gather->rank]);
    if (f16) cp_merge_kernel<__half><<<cgrid, 128, 0, st>>>(records, static_cast<__half *>(out), gather->world, d, cdom);
    else cp_merge_kernel<float><<<cgrid, 128, 0, st>>>(records, static_cast<float *>(out), gather->world, d, cdom);
    status = launch_status();
  }
  return status;
}

// ---- built-in scratch for callers that cannot allocate device memory -------------------------------
// One fixed array per GPU, part of the library image: every GPU that loads the library holds these
// bytes until the process exits.  Host code must not pass `g_static_scratch` to a kernel - in host
// code that name is only a handle for the runtime - so the device address is looked up once per
// device with cudaGetSymbolAddress and cached.
constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of the array on the current device, or null after a failed lookup.
void *static_scratch_ptr() {
  static std::mutex mu;
  static void *ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess) {
      cudaGetLastError();  // leave no sticky error behind
      return nullptr;
    }
    ptrs[dev] = ptr;
  }
  return ptrs[dev];
}

}  // namespace

// Prefill attention evaluated row by row on the decode kernels: query row t of q (sq,hq,d) is a
// "sequence" that sees min(t + 1, skv) keys (causal) or all skv keys of the one token-major cache.
// Correct for every dtype and head size the decode kernels take; K/V are re-read per row, so this is
// the parity path, not the fast one.
size_t sdpa_rows_workspace_bytes(int sq, int hq, int hkv, int d, int64_t skv) {
  if (sq <= 0 || hq <= 0 || hkv <= 0 || d <= 0 || skv <= 0) return 0;
  const Plan pl = make_plan(sq < 65535 ? sq : 65535, hq, hkv, d, skv);  // the largest slice
  return pl.part_o_bytes + pl.part_ml_bytes;
}

int sdpa_rows_fallback(const void *q, const void *k, const void *v, void *out, int sq, int hq, int hkv,
                       int d, int64_t skv, int is_causal, int dtype, void *workspace,
                       size_t workspace_bytes, cudaStream_t st) {
  // the rows are the launch's batch dimension (at most 65535 to a grid): long prompts go in slices
  constexpr int kSlice = 65535;
  const size_t row_bytes = (size_t)hq * d * dtype_size(dtype);
  for (int r0 = 0; r0 < sq; r0 += kSlice) {
    const int n = sq - r0 < kSlice ? sq - r0 : kSlice;
    const int status = decode_impl(false, static_cast<const uint8_t *>(q) + r0 * row_bytes,
                                   static_cast<uint8_t *>(out) + r0 * row_bytes, k, v, nullptr, nullptr, (int)skv, n,
                                   hq, hkv, d, 0, 0, 1, skv, dtype, workspace, workspace_bytes, st, nullptr, 0,
                                   is_causal ? 1 : 0, r0);
    if (status != AXB200_OK) return status;
  }
  return AXB200_OK;
}

// The decode step as ONE launch when that form applies (see the kStep notes at the fp16 kernel), else
// kStepNotFused with nothing launched.  q, k_new, v_new may live in page-locked host memory that the
// device can address; out too.
int decode_step_try_fused(const void *q, const void *k_new, const void *v_new, void *out, void *k_pages,
                          void *v_pages, const int32_t *block_table, int32_t *seq_lens, const int64_t *pos,
                          const float *inv_freq, float theta, int rotate, int mrope, int h_sec, int w_sec,
                          int batch, int hq, int hkv, int d, int page_tokens, int max_blocks, int num_pages,
                          int64_t max_seq_len, int dtype, void *workspace, size_t workspace_bytes,
                          void *stream) {
  {
    std::lock_guard<std::mutex> lock(g_settings_mu);
    if (!g_step_fused) return kStepNotFused;
  }
  if (dtype != AXB200_FLOAT16 || !(d == 64 || d == 128) || batch > kArrivalSlots) return kStepNotFused;
  if (!k_new || !v_new || !seq_lens) return AXB200_INVALID_PTR;
  if (rotate && mrope && !inv_freq) return AXB200_INVALID_PTR;
  StepParams sp{};
  sp.k_new = k_new;
  sp.v_new = v_new;
  sp.k_pages = k_pages;
  sp.v_pages = v_pages;
  sp.seq_lens = seq_lens;
  sp.pos = pos;
  sp.inv_freq_dev = inv_freq;
  sp.rotate = rotate;
  sp.mrope = mrope;
  sp.h_lim = h_sec * 3;
  sp.w_lim = w_sec * 3;
  sp.advance = 1;
  if (rotate && !inv_freq) rope_inv_freq_host(theta, d, sp.table);
  {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, q) != cudaSuccess) {
      cudaGetLastError();
    } else {
      sp.stage_q = attr.type == cudaMemoryTypeHost;
    }
  }
  return decode_impl(true, q, out, k_pages, v_pages, block_table, seq_lens, 0, batch, hq, hkv, d, page_tokens,
                     max_blocks, num_pages, max_seq_len, dtype, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream), nullptr, 0, 0, 0, &sp);
}

}  // namespace axb

extern "C" {

int axb200_qkv_decode_step_paged(const void *qkv, int64_t ld, const void *q_norm_w, const void *k_norm_w, float eps,
                                 void *out, void *k_pages, void *v_pages, const int32_t *block_table,
                                 int32_t *seq_lens, const int64_t *pos, const float *inv_freq, float theta,
                                 int rotate, int mrope, int h_sec, int w_sec, int batch, int hq, int hkv, int d,
                                 int page_tokens, int max_blocks, int num_pages, int64_t max_seq_len, int dtype,
                                 int slot_delta, int advance, void *workspace, size_t workspace_bytes,
                                 void *const *peer_out, void *const *peer_flags, void *local_state, int world,
                                 int rank, int hq_total, void *stream) {
  using namespace axb;
  const size_t es = dtype_size(dtype);
  if (es == 0) return AXB200_UNSUPPORTED_TYPE;
  if (!qkv || !k_pages || !v_pages || !block_table || !seq_lens || !workspace) return AXB200_INVALID_PTR;
  if (batch <= 0 || hq <= 0 || hkv <= 0 || d <= 0 || max_seq_len <= 0 || ld < (int64_t)(hq + 2 * hkv) * d)
    return AXB200_INVALID_ARGUMENT;
  if (!((slot_delta == 0 && advance == 1) || (slot_delta == -1 && advance == 0))) return AXB200_INVALID_ARGUMENT;
  if (rotate && mrope && !inv_freq) return AXB200_INVALID_PTR;
  if (workspace_bytes < axb200_decode_step_workspace_bytes(batch, hq, hkv, d, max_seq_len, dtype))
    return AXB200_INVALID_ARGUMENT;
  GatherParams g{};
  const bool peers = world > 0;
  if (peers) {
    if (!peer_out || !peer_flags || !local_state) return AXB200_INVALID_PTR;
    if (world > kMaxPeers || rank < 0 || rank >= world || hq_total != hq * world) return AXB200_INVALID_ARGUMENT;
    for (int r = 0; r < world; ++r) {
      if (!peer_out[r] || !peer_flags[r]) return AXB200_INVALID_PTR;
      g.peer_out[r] = peer_out[r];
      g.peer_flags[r] = static_cast<unsigned int *>(peer_flags[r]);
    }
    g.local_state = static_cast<unsigned int *>(local_state);
    g.world = world;
    g.rank = rank;
    g.hq_total = hq_total;
  } else if (!out) {
    return AXB200_INVALID_PTR;
  }
  const size_t attn_bytes = (axb200_gqa_workspace_bytes(batch, hq, hkv, d, max_seq_len, dtype) + 255) & ~size_t(255);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  bool fused;
  {
    std::lock_guard<std::mutex> lock(g_settings_mu);
    fused = g_step_fused;
  }
  fused = fused && dtype == AXB200_FLOAT16 && (d == 64 || d == 128) && batch <= kArrivalSlots && ld % 8 == 0 &&
          aligned16(qkv);
  if (fused) {
    StepParams sp{};
    sp.k_pages = k_pages;
    sp.v_pages = v_pages;
    sp.seq_lens = seq_lens;
    sp.pos = pos;
    sp.inv_freq_dev = inv_freq;
    sp.rotate = rotate;
    sp.mrope = mrope;
    sp.h_lim = h_sec * 3;
    sp.w_lim = w_sec * 3;
    sp.qkv = qkv;
    sp.ld = ld;
    sp.q_norm_w = q_norm_w;
    sp.k_norm_w = k_norm_w;
    sp.eps = eps;
    sp.advance = advance;
    if (rotate && !inv_freq) rope_inv_freq_host(theta, d, sp.table);
    const int rc = decode_impl(true, qkv, peers ? nullptr : out, k_pages, v_pages, block_table, seq_lens, 0, batch, hq,
                               hkv, d, page_tokens, max_blocks, num_pages, max_seq_len, dtype, workspace, attn_bytes,
                               st, peers ? &g : nullptr, 0, 0, 0, &sp);
    if (rc != kStepNotFused) return rc;
  }
  // two launches: the per-head norm + rotation + append kernel leaves q in the workspace, then attention
  void *q_rot = static_cast<uint8_t *>(workspace) + attn_bytes;
  int rc = axb200_qkv_norm_rope_append(qkv, ld, q_norm_w, k_norm_w, eps, q_rot, k_pages, v_pages, block_table, seq_lens,
                                       pos, inv_freq, theta, rotate, mrope, h_sec, w_sec, batch, hq, hkv, d, page_tokens,
                                       max_blocks, num_pages, dtype, slot_delta, advance, stream);
  if (rc != AXB200_OK) return rc;
  return decode_impl(true, q_rot, peers ? nullptr : out, k_pages, v_pages, block_table, seq_lens, 0, batch, hq, hkv, d,
                     page_tokens, max_blocks, num_pages, max_seq_len, dtype, workspace, attn_bytes, st,
                     peers ? &g : nullptr);
}

int axb200_set_step_fused(int on) {
  std::lock_guard<std::mutex> lock(axb::g_settings_mu);
  axb::g_step_fused = on != 0;
  return AXB200_OK;
}

size_t axb200_decode_step_workspace_bytes(int batch, int hq, int hkv, int d, int64_t max_seq_len, int dtype) {
  const size_t es = axb::dtype_size(dtype);
  if (es == 0 || batch <= 0 || hq <= 0 || hkv <= 0 || d <= 0 || max_seq_len <= 0) return 0;
  const size_t attn = (axb200_gqa_workspace_bytes(batch, hq, hkv, d, max_seq_len, dtype) + 255) & ~size_t(255);
  return attn + (((size_t)batch * hq * d * es + 255) & ~size_t(255));  // + the rotated q of the two-launch form
}

int axb200_decode_step_launches(int batch, int hq, int hkv, int d, int64_t max_seq_len, int dtype) {
  if (batch <= 0 || hq <= 0 || hkv <= 0 || d <= 0 || max_seq_len <= 0 || hq % hkv != 0) return 0;
  bool fused;
  {
    std::lock_guard<std::mutex> lock(axb::g_settings_mu);
    fused = axb::g_step_fused && axb::g_fused_merge;
  }
  const axb::Plan pl = axb::make_plan(batch, hq, hkv, d, max_seq_len);
  fused = fused && dtype == AXB200_FLOAT16 && (d == 64 || d == 128) && hq / hkv <= axb::kMaxGroupMma &&
          !pl.balanced && (int64_t)batch * hkv <= axb::kArrivalSlots;
  return fused ? 1 : 2;
}

int axb200_decode_step_paged(const void *q, const void *k_new, const void *v_new, void *out, void *k_pages,
                             void *v_pages, const int32_t *block_table, int32_t *seq_lens,
                             const int64_t *pos, const float *inv_freq, float theta, int rotate, int mrope,
                             int h_sec, int w_sec, int batch, int hq, int hkv, int d, int page_tokens,
                             int max_blocks, int num_pages, int64_t max_seq_len, int dtype, void *workspace,
                             size_t workspace_bytes, void *stream) {
  const size_t es = axb::dtype_size(dtype);
  if (es == 0) return AXB200_UNSUPPORTED_TYPE;
  if (!q || !k_new || !v_new || !out || !k_pages || !v_pages || !block_table || !seq_lens || !workspace)
    return AXB200_INVALID_PTR;
  if (batch <= 0 || hq <= 0 || hkv <= 0 || d <= 0 || max_seq_len <= 0) return AXB200_INVALID_ARGUMENT;
  if (workspace_bytes < axb200_decode_step_workspace_bytes(batch, hq, hkv, d, max_seq_len, dtype))
    return AXB200_INVALID_ARGUMENT;
  const size_t attn_bytes = (axb200_gqa_workspace_bytes(batch, hq, hkv, d, max_seq_len, dtype) + 255) & ~size_t(255);
  int rc = axb::decode_step_try_fused(q, k_new, v_new, out, k_pages, v_pages, block_table, seq_lens, pos, inv_freq,
                                      theta, rotate, mrope, h_sec, w_sec, batch, hq, hkv, d, page_tokens, max_blocks,
                                      num_pages, max_seq_len, dtype, workspace, attn_bytes, stream);
  if (rc != axb::kStepNotFused) return rc;
  // two launches: the append leaves the rotated q in the workspace (the caller's q stays as it is)
  void *q_rot = static_cast<uint8_t *>(workspace) + attn_bytes;
  const void *q_attn = q;
  if (rotate) {
    rc = axb::kv_append_rope_from(q_rot, q, k_new, v_new, k_pages, v_pages, block_table, seq_lens, pos, inv_freq, theta,
                                  1, mrope, h_sec, w_sec, batch, hq, hkv, d, page_tokens, max_blocks, num_pages,
                                  dtype, 0, 1, stream);
    q_attn = q_rot;
  } else {
    rc = axb::kv_append_rope_from(nullptr, nullptr, k_new, v_new, k_pages, v_pages, block_table, seq_lens, pos,
                                  inv_freq, theta, 0, mrope, h_sec, w_sec, batch, 0, hkv, d, page_tokens, max_blocks,
                                  num_pages, dtype, 0, 1, stream);
  }
  if (rc != AXB200_OK) return rc;
  return axb200_gqa_decode_paged(q_attn, out, k_pages, v_pages, block_table, seq_lens, batch, hq, hkv, d, page_tokens,
                                 max_blocks, num_pages, max_seq_len, dtype, workspace, attn_bytes, stream);
}

int axb200_set_wait_limit_ns(uint64_t ns) {
  if (ns == 0) return AXB200_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(axb::g_settings_mu);
  axb::g_wait_limit_ns = ns;
  return AXB200_OK;
}

int axb200_set_dependent_launch(int on) {
  std::lock_guard<std::mutex> lock(axb::g_settings_mu);
  axb::g_dependent_launch = on != 0;
  return AXB200_OK;
}

int axb200_set_chunk_tiles(int tiles) {
  if (tiles < 0) return AXB200_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(axb::g_settings_mu);
  axb::g_forced_chunk_tiles = tiles;
  return AXB200_OK;
}

int axb200_set_device_plan(int on) {
  std::lock_guard<std::mutex> lock(axb::g_settings_mu);
  axb::g_device_plan = on != 0;
  return AXB200_OK;
}

int axb200_set_fused_merge(int on) {
  std::lock_guard<std::mutex> lock(axb::g_settings_mu);
  axb::g_fused_merge = on != 0;
  axb::g_merge_pairs = on != 2;
  return AXB200_OK;
}

int axb200_gqa_chunk_plan(const int32_t *lens_host, int batch, int hq, int hkv, int d, int64_t max_seq_len,
                          int32_t *chunk_tokens_out, int32_t *n_chunks_out, int32_t *max_chunks_out,
                          int32_t *grid_ctas_out) {
  if (!lens_host || !chunk_tokens_out || !n_chunks_out) return AXB200_INVALID_PTR;
  if (batch <= 0 || hq <= 0 || hkv <= 0 || d <= 0 || max_seq_len <= 0) return AXB200_INVALID_ARGUMENT;
  const axb::Plan pl = axb::make_plan(batch, hq, hkv, d, max_seq_len);
  if (max_chunks_out) *max_chunks_out = pl.max_chunks;
  if (grid_ctas_out) *grid_ctas_out = pl.balanced ? pl.budget * hkv : pl.max_chunks * hkv * batch;
  const int c = pl.balanced ? axb::balanced_chunk_tiles_host(lens_host, batch, pl.budget, pl.max_chunks) : 0;
  for (int b = 0; b < batch; ++b) {
    int L = lens_host[b] < 0 ? 0 : lens_host[b];
    if (pl.balanced) {
      int ct, n;
      axb::sequence_chunks(L, c, &ct, &n);
      chunk_tokens_out[b] = ct;
      n_chunks_out[b] = n;
    } else {
      const int64_t cover = (int64_t)pl.max_chunks * pl.chunk_tokens;
      if (L > cover) L = (int)cover;
      chunk_tokens_out[b] = pl.chunk_tokens;
      n_chunks_out[b] = std::max(1, axb::ceil_div(L, pl.chunk_tokens));
    }
  }
  return AXB200_OK;
}

size_t axb200_static_scratch_bytes(void) { return axb::kStaticScratchBytes; }

int axb200_gqa_decode_static(const void *q, const void *k, const void *v, void *out, int hq,
                             int hkv, int d, int64_t skv, int dtype, void *stream) {
  if (hq <= 0 || hkv <= 0 || d <= 0 || skv <= 0) return AXB200_INVALID_ARGUMENT;
  const axb::Plan pl = axb::make_plan(1, hq, hkv, d, skv);
  if (pl.part_o_bytes + pl.part_ml_bytes > axb::kStaticScratchBytes) return AXB200_OUT_OF_MEMORY;
  void *scratch = axb::static_scratch_ptr();
  if (!scratch) return AXB200_DEVICE_ERROR;
  // Nothing in the array has to start at zero: the combine kernel reads only the partial records
  // that this call's split kernel has written.
  return axb::decode_impl(false, q, out, k, v, nullptr, nullptr, (int)skv, 1, hq, hkv, d, 0, 0, 1,
                          skv, dtype, scratch, axb::kStaticScratchBytes,
                          static_cast<cudaStream_t>(stream));
}

int axb200_gqa_decode_paged_gather(const void *q, const void *k_pages, const void *v_pages,
                                   const int32_t *block_table, const int32_t *seq_lens, int batch,
                                   int hq, int hkv, int d, int page_tokens, int max_blocks,
                                   int num_pages, int64_t max_seq_len, int dtype, void *workspace,
                                   size_t workspace_bytes, void *const *peer_out,
                                   void *const *peer_flags, void *local_state, int world, int rank,
                                   int hq_total, void *stream) {
  if (!peer_out || !peer_flags || !local_state) return AXB200_INVALID_PTR;
  if (world < 1 || world > axb::kMaxPeers || rank < 0 || rank >= world || hq_total != hq * world)
    return AXB200_INVALID_ARGUMENT;
  axb::GatherParams g{};
  for (int r = 0; r < world; ++r) {
    if (!peer_out[r] || !peer_flags[r]) return AXB200_INVALID_PTR;
    g.peer_out[r] = peer_out[r];
    g.peer_flags[r] = static_cast<unsigned int *>(peer_flags[r]);
  }
  g.local_state = static_cast<unsigned int *>(local_state);
  g.world = world;
  g.rank = rank;
  g.hq_total = hq_total;
  return axb::decode_impl(true, q, nullptr, k_pages, v_pages, block_table, seq_lens, 0, batch, hq,
                          hkv, d, page_tokens, max_blocks, num_pages, max_seq_len, dtype, workspace,
                          workspace_bytes, static_cast<cudaStream_t>(stream), &g);
}

int axb200_gqa_decode_paged_cp(const void *q, void *out, const void *k_pages, const void *v_pages,
                               const int32_t *block_table, const int32_t *seq_lens, int batch,
                               int hq, int hkv, int d, int page_tokens, int max_blocks,
                               int num_pages, int64_t max_seq_len, int dtype, void *workspace,
                               size_t workspace_bytes, void *const *peer_records,
                               void *const *peer_flags, void *local_state, int world, int rank,
                               void *stream) {
  if (!peer_records || !peer_flags || !local_state || !out) return AXB200_INVALID_PTR;
  if (world < 1 || world > axb::kMaxPeers || rank < 0 || rank >= world) return AXB200_INVALID_ARGUMENT;
  axb::GatherParams g{};
  for (int r = 0; r < world; ++r) {
    if (!peer_records[r] || !peer_flags[r]) return AXB200_INVALID_PTR;
    g.peer_out[r] = peer_records[r];
    g.peer_flags[r] = static_cast<unsigned int *>(peer_flags[r]);
  }
  g.local_state = static_cast<unsigned int *>(local_state);
  g.world = world;
  g.rank = rank;
  g.hq_total = hq;
  g.mode = 1;
  return axb::decode_impl(true, q, out, k_pages, v_pages, block_table, seq_lens, 0, batch, hq, hkv,
                          d, page_tokens, max_blocks, num_pages, max_seq_len, dtype, workspace,
                          workspace_bytes, static_cast<cudaStream_t>(stream), &g);
}

int axb200_gqa_decode_paged_window(const void *q, void *out, const void *k_pages,
                                   const void *v_pages, const int32_t *block_table,
                                   const int32_t *seq_lens, int batch, int hq, int hkv, int d,
                                   int page_tokens, int max_blocks, int num_pages,
                                   int64_t max_seq_len, int window, int dtype, void *workspace,
                                   size_t workspace_bytes, void *stream) {
  return axb::decode_impl(true, q, out, k_pages, v_pages, block_table, seq_lens, 0, batch, hq, hkv,
                          d, page_tokens, max_blocks, num_pages, max_seq_len, dtype, workspace,
                          workspace_bytes, static_cast<cudaStream_t>(stream), nullptr, window);
}

int axb200_p2p_alloc(size_t bytes, void **dev_ptr, void *handle64) {
  if (!dev_ptr || !handle64 || bytes == 0) return AXB200_INVALID_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void *ptr = nullptr;
  if (cudaMalloc(&ptr, bytes) != cudaSuccess) return AXB200_OUT_OF_MEMORY;
  if (cudaMemset(ptr, 0, bytes) != cudaSuccess) {
    cudaFree(ptr);
    return AXB200_DEVICE_ERROR;
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) {
    cudaFree(ptr);
    return AXB200_DEVICE_ERROR;
  }
  memcpy(handle64, &h, sizeof(h));
  *dev_ptr = ptr;
  return AXB200_OK;
}

int axb200_p2p_open(const void *handle64, void **dev_ptr) {
  if (!handle64 || !dev_ptr) return AXB200_INVALID_PTR;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void *ptr = nullptr;
  if (cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return AXB200_DEVICE_ERROR;
  }
  *dev_ptr = ptr;
  return AXB200_OK;
}

int axb200_p2p_close(void *dev_ptr) {
  return cudaIpcCloseMemHandle(dev_ptr) == cudaSuccess ? AXB200_OK : AXB200_DEVICE_ERROR;
}

int axb200_p2p_free(void *dev_ptr) {
  return cudaFree(dev_ptr) == cudaSuccess ? AXB200_OK : AXB200_DEVICE_ERROR;
}

const char *axb200_version(void) { return "axono_b200 0.2 (sm_100a)"; }

unsigned int axb200_last_error(void) {
  if (cudaDeviceSynchronize() != cudaSuccess) return 0x80000000u;
  unsigned int word = 0;
  for (int i = 0; i < axb::g_num_error_readers; ++i) word |= axb::g_error_readers[i]();
  if (word & AXB200_ERR_WAIT_TIMEOUT) {
    // a CTA that gave up never counted itself in: put the fused merge's counters back to zero
    axb::zero_arrival_kernel<<<64, 256>>>();
    cudaDeviceSynchronize();
  }
  return word;
}

int axb200_profile_enable(int on) {
  std::lock_guard<std::mutex> lock(axb::g_profile_mu);
  axb::ProfileState &ps = axb::g_profile;
  if (on && !ps.created) {
    for (int i = 0; i < axb::kProfilePairs; ++i) {
      if (cudaEventCreate(&ps.start[i]) != cudaSuccess || cudaEventCreate(&ps.stop[i]) != cudaSuccess)
        return AXB200_DEVICE_ERROR;
    }
    ps.created = true;
  }
  ps.enabled = on != 0;
  ps.used = 0;
  return AXB200_OK;
}

int axb200_profile_collect(double *split_ms_total, int *launches) {
  if (!split_ms_total || !launches) return AXB200_INVALID_PTR;
  if (cudaDeviceSynchronize() != cudaSuccess) return AXB200_DEVICE_ERROR;
  std::lock_guard<std::mutex> lock(axb::g_profile_mu);
  axb::ProfileState &ps = axb::g_profile;
  double total = 0.0;
  for (int i = 0; i < ps.used; ++i) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, ps.start[i], ps.stop[i]) != cudaSuccess)
      return AXB200_DEVICE_ERROR;
    total += ms;
  }
  *split_ms_total = total;
  *launches = ps.used;
  ps.used = 0;
  return AXB200_OK;
}

size_t axb200_gqa_workspace_bytes(int batch, int hq, int hkv, int d, int64_t max_seq_len,
                                  int dtype) {
  (void)dtype;
  if (batch <= 0 || hq <= 0 || hkv <= 0 || d <= 0 || max_seq_len <= 0) return 0;
  const axb::Plan pl = axb::make_plan(batch, hq, hkv, d, max_seq_len);
  return pl.part_o_bytes + pl.part_ml_bytes;
}

int axb200_gqa_decode(const void *q, const void *k, const void *v, void *out, int hq, int hkv,
                      int d, int64_t skv, int dtype, void *workspace, size_t workspace_bytes,
                      void *stream) {
  return axb::decode_impl(false, q, out, k, v, nullptr, nullptr, (int)skv, 1, hq, hkv, d, 0, 0, 1,
                          skv, dtype, workspace, workspace_bytes,
                          static_cast<cudaStream_t>(stream));
}

int axb200_gqa_decode_paged(const void *q, void *out, const void *k_pages, const void *v_pages,
                            const int32_t *block_table, const int32_t *seq_lens, int batch, int hq,
                            int hkv, int d, int page_tokens, int max_blocks, int num_pages,
                            int64_t max_seq_len, int dtype, void *workspace,
                            size_t workspace_bytes, void *stream) {
  return axb::decode_impl(true, q, out, k_pages, v_pages, block_table, seq_lens, 0, batch, hq, hkv,
                          d, page_tokens, max_blocks, num_pages, max_seq_len, dtype, workspace,
                          workspace_bytes, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
