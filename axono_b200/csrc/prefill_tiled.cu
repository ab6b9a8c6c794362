// Prefill attention on the FMA pipe: many queries, optional causal mask, FLOAT32 or FLOAT16 storage
// with fp32 arithmetic throughout, any head_dim that is a multiple of 4 up to 256.  It serves what the
// tensor-core kernel does not take - above all FLOAT32, the only type the reference's own
// ScaledDotProductAttention accepts (src/ops/cuda/sequence.cu:451-472), where a tensor-core product
// (fp16 or tf32 operands) could not hold the 1e-5 parity bound.  Before this kernel those shapes ran
// row by row on the decode kernels, which re-read K and V once per query row.
//
// One CTA per (block of query rows, KV head): the `group` query heads of the KV head times the rows
// of the block make 64 virtual rows that share every staged K / V tile.  Per tile of 64 keys:
//   stage    K and V rows into shared memory as fp32 (plain coalesced loads, four of each in flight per
//            thread before the first store)
//   scores   thread = 2 rows x 4 keys, 16-byte reads of Q and K rows: 6 shared-memory reads per 32 FMAs
//   softmax  warp = 4 rows: maximum and sum by shuffles, the causal rule applied here
//   P.V      thread = 2 rows x (head_dim / 16) columns, accumulators in registers
// Semantics as the reference's CPU op (src/ops/cpu/sequence.cpp:236-301): q (sq,hq,d), k / v
// (skv,hkv,d) token-major, head h reads KV head h / (hq / hkv), scale 1/sqrt(d); with is_causal row t
// sees keys [0, min(t + 1, skv)).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <mutex>
#include <set>

#include "axono_b200.h"
#include "common.cuh"

namespace axb {
namespace {

// Two CTA shapes, both 512 threads (16 warps hide the shared-memory latency): 64 virtual rows with 2
// rows per thread, and 128 virtual rows with 4 rows per thread - twice the FMAs per shared-memory byte -
// where its 166 KB of shared memory (head_dim 128) fit and the problem has that many rows.
constexpr int kTpKeys = 64, kTpThreads = 512, kTpLoadBatch = 4;
constexpr float kTpLog2e = 1.4426950408889634f;

struct TiledParams {
  const void *q, *k, *v;
  void *out;
  int sq, hq, hkv, group, skv, causal, d;
  int bq;  // query rows per CTA: virtual rows / group
  float scale;
};

template <typename T>
__device__ __forceinline__ float tp_f32(T v);
template <>
__device__ __forceinline__ float tp_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float tp_f32<__half>(__half v) { return __half2float(v); }

// Row stride of the staged tiles in floats: rows stay 16-byte aligned; (d + 4) / 4 is odd when d is a
// multiple of 8, which keeps "thread = key" 16-byte reads conflict-free.
__host__ __device__ inline int tp_stride(int d) { return d + 4; }
inline size_t tp_smem_bytes(int d, int rows) {
  return sizeof(float) * ((size_t)rows * d + 2 * (size_t)kTpKeys * tp_stride(d) + (size_t)rows * (kTpKeys + 4) +
                          3 * (size_t)rows);
}

// kCols: 16-byte column chunks per thread = head_dim / 64, rounded up; kTpRows virtual rows per CTA,
// kTpRpt of them per thread.
template <typename T, int kCols, int kTpRows, int kTpRpt>
__global__ void __launch_bounds__(kTpThreads)
sdpa_tiled_kernel(const TiledParams p) {
  static_assert((kTpRows / kTpRpt) * 16 == kTpThreads, "thread tile does not cover the CTA tile");
  extern __shared__ __align__(16) float tsm[];
  const int d = p.d, dp = tp_stride(d), pp = kTpKeys + 4;
  float *Qs = tsm, *Ks = Qs + kTpRows * d, *Vs = Ks + kTpKeys * dp, *Ps = Vs + kTpKeys * dp;
  float *m_s = Ps + kTpRows * pp, *l_s = m_s + kTpRows, *corr_s = l_s + kTpRows;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // heaviest blocks first under the causal mask
  const int qb = gridDim.x - 1 - blockIdx.x, hk = blockIdx.y;
  const int q0 = qb * p.bq;
  const T *qg = reinterpret_cast<const T *>(p.q), *kg = reinterpret_cast<const T *>(p.k),
          *vg = reinterpret_cast<const T *>(p.v);
  // virtual row r = g * bq + i: query head hk * group + g, query row q0 + i
  const int n_rows = p.group * p.bq;
  const int t_last = min(q0 + p.bq, p.sq) - 1;
  const int kv_end_max = p.causal ? min(t_last + 1, p.skv) : p.skv;

  for (int e = tid; e < kTpRows * d; e += kTpThreads) {
    const int r = e / d, c = e - r * d;
    const int g = r / p.bq, i = r - g * p.bq;
    float val = 0.f;
    if (r < n_rows && q0 + i < p.sq) val = tp_f32(qg[((size_t)(q0 + i) * p.hq + hk * p.group + g) * d + c]);
    Qs[e] = val;
  }
  if (tid < kTpRows) {
    m_s[tid] = -INFINITY;
    l_s[tid] = 0.f;
    corr_s[tid] = 1.f;
  }
  // thread tile: rows kTpRpt * ty ..; keys tx + 16 * j (scores); columns (tx + 16 * j) * 4 .. + 3 (output)
  const int ty = tid >> 4, tx = tid & 15;
  float acc[kTpRpt][kCols * 4];
#pragma unroll
  for (int a = 0; a < kTpRpt; ++a)
#pragma unroll
    for (int c = 0; c < kCols * 4; ++c) acc[a][c] = 0.f;
  const float dom = p.scale * kTpLog2e;

  for (int t0 = 0; t0 < kv_end_max; t0 += kTpKeys) {
    const int nt = min(kTpKeys, kv_end_max - t0);
    __syncthreads();  // the previous tile is done with Ks, Vs, Ps (and Qs is written)
    // ---- stage K and V: nt * d elements each, consecutive threads on consecutive elements ----
    {
      const int n_elem = nt * d;
      int er = tid / d, ec = tid % d;
      for (int e0 = 0; e0 < n_elem; e0 += kTpThreads * kTpLoadBatch) {
        float kr[kTpLoadBatch], vr[kTpLoadBatch];
        int at[kTpLoadBatch];
#pragma unroll
        for (int u = 0; u < kTpLoadBatch; ++u) {
          at[u] = -1;
          kr[u] = vr[u] = 0.f;
          if (e0 + u * kTpThreads + tid < n_elem) {
            at[u] = er * dp + ec;
            const size_t off = ((size_t)(t0 + er) * p.hkv + hk) * d + ec;
            kr[u] = tp_f32(kg[off]);
            vr[u] = tp_f32(vg[off]);
          }
          ec += kTpThreads;
          while (ec >= d) {
            ec -= d;
            ++er;
          }
        }
#pragma unroll
        for (int u = 0; u < kTpLoadBatch; ++u)
          if (at[u] >= 0) {
            Ks[at[u]] = kr[u];
            Vs[at[u]] = vr[u];
          }
      }
      // keys past the tile's end read as zeros in the score loop
      for (int e = n_elem + tid; e < kTpKeys * d; e += kTpThreads) {
        const int r = e / d, c = e - r * d;
        Ks[r * dp + c] = 0.f;
        Vs[r * dp + c] = 0.f;
      }
    }
    __syncthreads();
    // ---- scores: kTpRpt rows x 4 keys per thread ----
    {
      float sc[kTpRpt][4];
#pragma unroll
      for (int a = 0; a < kTpRpt; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) sc[a][b] = 0.f;
      const float4 *q4 = reinterpret_cast<const float4 *>(Qs + (kTpRpt * ty) * d);
      const float4 *k4 = reinterpret_cast<const float4 *>(Ks + tx * dp);
      const int qs4 = d / 4, ks4 = (16 * dp) / 4;
#pragma unroll 2
      for (int c4 = 0; c4 < d / 4; ++c4) {
        float4 qv[kTpRpt], kv[4];
#pragma unroll
        for (int a = 0; a < kTpRpt; ++a) qv[a] = q4[a * qs4 + c4];
#pragma unroll
        for (int b = 0; b < 4; ++b) kv[b] = k4[b * ks4 + c4];
#pragma unroll
        for (int a = 0; a < kTpRpt; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b)
            sc[a][b] = fmaf(qv[a].w, kv[b].w, fmaf(qv[a].z, kv[b].z, fmaf(qv[a].y, kv[b].y, fmaf(qv[a].x, kv[b].x, sc[a][b]))));
      }
#pragma unroll
      for (int a = 0; a < kTpRpt; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) Ps[(kTpRpt * ty + a) * pp + tx + 16 * b] = sc[a][b];
    }
    __syncthreads();
    // ---- online softmax: kTpRows / warps rows per warp, the causal rule per row ----
    constexpr int kRowsPerWarp = kTpRows / (kTpThreads / 32);
    for (int r = warp * kRowsPerWarp; r < warp * kRowsPerWarp + kRowsPerWarp; ++r) {
      const int g = r / p.bq, i = r - g * p.bq;
      const int t_row = q0 + i;
      const int kv_end = (r < n_rows && t_row < p.sq) ? (p.causal ? min(t_row + 1, p.skv) : p.skv) : 0;
      const int k0 = t0 + lane, k1 = t0 + 32 + lane;
      const float s0 = k0 < kv_end ? Ps[r * pp + lane] : -INFINITY;
      const float s1 = k1 < kv_end ? Ps[r * pp + 32 + lane] : -INFINITY;
      float mx = fmaxf(s0, s1);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_old = m_s[r], m_new = fmaxf(m_old, mx);
      const float corr = m_old == -INFINITY ? 0.f : exp2f((m_old - m_new) * dom);
      const float p0 = s0 == -INFINITY ? 0.f : exp2f((s0 - m_new) * dom);
      const float p1 = s1 == -INFINITY ? 0.f : exp2f((s1 - m_new) * dom);
      Ps[r * pp + lane] = p0;
      Ps[r * pp + 32 + lane] = p1;
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
    // ---- O = O * corr + P . V: kTpRpt rows x kCols chunks of 4 columns per thread ----
    {
#pragma unroll
      for (int a = 0; a < kTpRpt; ++a) {
        const float cr = corr_s[kTpRpt * ty + a];
#pragma unroll
        for (int c = 0; c < kCols * 4; ++c) acc[a][c] *= cr;
      }
      for (int t = 0; t < nt; t += 4) {  // Ps and Vs rows past nt hold zeros
        float4 pw[kTpRpt];
#pragma unroll
        for (int a = 0; a < kTpRpt; ++a) pw[a] = *reinterpret_cast<const float4 *>(Ps + (kTpRpt * ty + a) * pp + t);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int j = 0; j < kCols; ++j) {
            const int c = (tx + 16 * j) * 4;
            if (c < d) {
              const float4 vv = *reinterpret_cast<const float4 *>(Vs + (t + u) * dp + c);
#pragma unroll
              for (int a = 0; a < kTpRpt; ++a) {
                const float w = u == 0 ? pw[a].x : u == 1 ? pw[a].y : u == 2 ? pw[a].z : pw[a].w;
                acc[a][j * 4 + 0] = fmaf(w, vv.x, acc[a][j * 4 + 0]);
                acc[a][j * 4 + 1] = fmaf(w, vv.y, acc[a][j * 4 + 1]);
                acc[a][j * 4 + 2] = fmaf(w, vv.z, acc[a][j * 4 + 2]);
                acc[a][j * 4 + 3] = fmaf(w, vv.w, acc[a][j * 4 + 3]);
              }
            }
          }
        }
      }
    }
  }
  __syncthreads();
  // ---- O / l -> out ----
  T *og = reinterpret_cast<T *>(p.out);
#pragma unroll
  for (int a = 0; a < kTpRpt; ++a) {
    const int r = kTpRpt * ty + a;
    const int g = r / p.bq, i = r - g * p.bq;
    if (r >= n_rows || q0 + i >= p.sq) continue;
    const float l = l_s[r];
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T *row = og + ((size_t)(q0 + i) * p.hq + hk * p.group + g) * d;
#pragma unroll
    for (int j = 0; j < kCols; ++j) {
      const int c = (tx + 16 * j) * 4;
      if (c < d) {
#pragma unroll
        for (int e = 0; e < 4; ++e) row[c + e] = static_cast<T>(acc[a][j * 4 + e] * inv);
      }
    }
  }
}

bool tp_set_smem(const void *kernel, int bytes) {
  static std::mutex mu;
  static std::set<std::pair<const void *, int>> done;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (done.count({kernel, dev})) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
  done.insert({kernel, dev});
  return true;
}

template <typename T, int kCols, int kRows, int kRpt>
int tp_launch(const TiledParams &p, cudaStream_t st) {
  auto kern = sdpa_tiled_kernel<T, kCols, kRows, kRpt>;
  const int smem = (int)tp_smem_bytes(p.d, kRows);
  if (!tp_set_smem(reinterpret_cast<const void *>(kern), 200 * 1024)) return AXB200_DEVICE_ERROR;
  const dim3 grid((p.sq + p.bq - 1) / p.bq, p.hkv);
  kern<<<grid, kTpThreads, smem, st>>>(p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? AXB200_OK : AXB200_DEVICE_ERROR;
}

}  // namespace

// Whether the tiled kernel takes this problem; otherwise the caller runs it row by row.
bool sdpa_tiled_supported(int sq, int hq, int hkv, int d, int64_t skv) {
  const int group = hkv > 0 ? hq / hkv : 0;
  return sq >= 16 && d % 4 == 0 && d >= 4 && d <= 256 && group >= 1 && group <= 64 && hkv <= 65535 &&
         skv <= 0x7fffffff - kTpKeys && tp_smem_bytes(d, 64) <= 200 * 1024;
}

namespace {
template <typename T, int kRows, int kRpt>
int tp_dispatch_cols(const TiledParams &p, cudaStream_t st) {
  switch ((p.d + 63) / 64) {  // 16-byte chunks per thread
    case 1: return tp_launch<T, 1, kRows, kRpt>(p, st);
    case 2: return tp_launch<T, 2, kRows, kRpt>(p, st);
    case 3: return tp_launch<T, 3, kRows, kRpt>(p, st);
    default: return tp_launch<T, 4, kRows, kRpt>(p, st);
  }
}
}  // namespace

int sdpa_tiled(const void *q, const void *k, const void *v, void *out, int sq, int hq, int hkv, int d, int64_t skv,
               int is_causal, int dtype, cudaStream_t st) {
  TiledParams p{};
  p.q = q;
  p.k = k;
  p.v = v;
  p.out = out;
  p.sq = sq;
  p.hq = hq;
  p.hkv = hkv;
  p.group = hq / hkv;
  p.skv = (int)skv;
  p.causal = is_causal != 0;
  p.d = d;
  p.scale = 1.0f / sqrtf((float)d);
  // 128 virtual rows per CTA where they fit in shared memory and the problem fills them
  const bool big = tp_smem_bytes(d, 128) <= 200 * 1024 && (int64_t)sq * p.group >= 128 && d <= 128;
  p.bq = (big ? 128 : 64) / p.group;
  if (dtype == AXB200_FLOAT32)
    return big ? tp_dispatch_cols<float, 128, 4>(p, st) : tp_dispatch_cols<float, 64, 2>(p, st);
  return big ? tp_dispatch_cols<__half, 128, 4>(p, st) : tp_dispatch_cols<__half, 64, 2>(p, st);
}

}  // namespace axb
