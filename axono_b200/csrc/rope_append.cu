// RoPE / M-RoPE and the KV-cache append for sm_100a.  Replaces the reference's Rope
// (src/ops/cuda/sequence.cu:84-101,318-342), RopeThd (:186-212,421-449), RopeWithCosSin
// (:166-183,344-367), MropeCosSin (:372-419) and, for the decode step, the concat-based cache
// update (axono/python/axono/nn/kv_cache.py:96-102 -> src/ops/cuda/sequence.cu:474-521).
//
// Arithmetic follows the reference's CPU twins (src/ops/cpu/sequence.cpp:54-234): the angle is
// float(position) * inv_freq[i] in fp32, cos/sin are the full-range functions (positions reach
// tens of thousands, so the fast intrinsics would be wrong), and pair (i, i + dim/2) rotates as
// (a*c - b*s, b*c + a*s).  For plain rope the inverse frequencies theta^(-2i/dim) are computed
// on the host with the C library's powf - the function the reference's CPU op calls - and
// passed to the kernel by value, so the table is bit-identical to the reference's.
#include <math.h>

#include "common.cuh"

namespace axb {
namespace {

constexpr int kMaxHalf = 128;  // head_dim <= 256

struct InvFreqTable {
  float f[kMaxHalf];
};

template <typename T>
__device__ __forceinline__ float ld(const T *p);
template <>
__device__ __forceinline__ float ld<float>(const float *p) { return *p; }
template <>
__device__ __forceinline__ float ld<__half>(const __half *p) { return __half2float(*p); }
template <typename T>
__device__ __forceinline__ void st(T *p, float v);
template <>
__device__ __forceinline__ void st<float>(float *p, float v) { *p = v; }
template <>
__device__ __forceinline__ void st<__half>(__half *p, float v) { *p = __float2half_rn(v); }

// 16 bytes of T as floats and back (pointers 16-byte aligned): 4 floats or 8 halves.
template <typename T>
struct Vec16 {
  static constexpr int kN = 16 / (int)sizeof(T);
};
__device__ __forceinline__ void ld16(const float *p, float (&f)[4]) {
  const float4 v = *reinterpret_cast<const float4 *>(p);
  f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
}
__device__ __forceinline__ void ld16(const __half *p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4 *>(p);
  const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(h[i]);
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void st16(float *p, const float (&f)[4]) {
  *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
__device__ __forceinline__ void st16(__half *p, const float (&f)[8]) {
  uint4 v;
  __half2 *h = reinterpret_cast<__half2 *>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __halves2half2(__float2half_rn(f[2 * i]), __float2half_rn(f[2 * i + 1]));
  *reinterpret_cast<uint4 *>(p) = v;
}
// Rotates kN pairs (a[j], b[j]) = (x[i + j], x[i + j + half]) with the tables at i + j; the same
// expressions, element by element, as the scalar path.
template <int kN>
__device__ __forceinline__ void rotate_vec(float (&a)[kN], float (&b)[kN], const float *c0, const float *s0,
                                           const float *c1, const float *s1) {
#pragma unroll
  for (int j = 0; j < kN; ++j) {
    const float x = a[j], y = b[j];
    a[j] = rope_lo(x, y, c0[j], s0[j]);
    b[j] = rope_hi(x, y, c1[j], s1[j]);
  }
}

__device__ __forceinline__ float pair_position(int i, float pt, float ph, float pw, int h_lim, int w_lim) {
  return mrope_pair_position(i, pt, ph, pw, h_lim, w_lim);
}

enum RopeMode { kModeTheta = 0, kModeMrope = 1, kModeCosSin = 2 };

// One thread per (row, head, pair).  out may alias x: each thread reads its pair before writing.
template <typename T, int kMode>
__global__ void __launch_bounds__(256)
rope_kernel(const T *x, T *out, const int64_t *pos, const float *inv_freq_dev,
            const InvFreqTable table, const float *cos_t, const float *sin_t, int64_t rows,
            int heads, int dim, int h_lim, int w_lim) {
  const int half = dim / 2;
  const int64_t total = rows * heads * half;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % half);
    const int64_t rh = idx / half;
    const int64_t r = rh / heads;
    const T *src = x + rh * dim;
    T *dst = out + rh * dim;
    const float a = ld(src + i), b = ld(src + i + half);
    float c0, s0, c1, s1;
    if (kMode == kModeCosSin) {
      c0 = cos_t[r * dim + i];
      s0 = sin_t[r * dim + i];
      c1 = cos_t[r * dim + i + half];
      s1 = sin_t[r * dim + i + half];
    } else {
      float p, f;
      if (kMode == kModeMrope) {
        p = pair_position(i, (float)pos[r], (float)pos[rows + r], (float)pos[2 * rows + r], h_lim,
                          w_lim);
        f = inv_freq_dev[i];
      } else {
        p = (float)pos[r];
        f = table.f[i];
      }
      const float ang = p * f;
      sincosf(ang, &s0, &c0);
      c1 = c0;
      s1 = s0;
    }
    st(dst + i, rope_lo(a, b, c0, s0));
    st(dst + i + half, rope_hi(a, b, c1, s1));
  }
}

// One CTA per row (grid-stride): the row's cos / sin are computed once per rotary pair into shared
// memory and every head reuses them - with one thread per (row, head, pair) the range-reduced sincosf
// was evaluated `heads` times over and dominated the kernel.  Same arithmetic per element as
// rope_kernel; head_dim <= 256.
template <typename T, int kMode>
__global__ void __launch_bounds__(128)
rope_rows_kernel(const T *x, T *out, const int64_t *pos, const float *inv_freq_dev, const InvFreqTable table,
                 const float *cos_t, const float *sin_t, int64_t rows, int heads, int dim, int h_lim, int w_lim,
                 int vec) {  // vec: x and out 16-byte aligned and dim / 2 a multiple of 16 bytes' worth of T
  __shared__ float s_c0[kMaxHalf], s_s0[kMaxHalf], s_c1[kMaxHalf], s_s1[kMaxHalf];
  const int half = dim / 2;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    __syncthreads();  // the previous row's pairs are done with the tables
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      if (kMode == kModeCosSin) {
        s_c0[i] = cos_t[r * dim + i];
        s_s0[i] = sin_t[r * dim + i];
        s_c1[i] = cos_t[r * dim + i + half];
        s_s1[i] = sin_t[r * dim + i + half];
      } else {
        float p, f;
        if (kMode == kModeMrope) {
          p = pair_position(i, (float)pos[r], (float)pos[rows + r], (float)pos[2 * rows + r], h_lim, w_lim);
          f = inv_freq_dev[i];
        } else {
          p = (float)pos[r];
          f = table.f[i];
        }
        float sn, cs;
        sincosf(p * f, &sn, &cs);
        s_c0[i] = s_c1[i] = cs;
        s_s0[i] = s_s1[i] = sn;
      }
    }
    __syncthreads();
    const T *src = x + r * heads * dim;
    T *dst = out + r * heads * dim;
    if (vec) {
      constexpr int kN = Vec16<T>::kN;
      const int per_head = half / kN;
      for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
        const int h = idx / per_head, i = (idx - h * per_head) * kN;
        float a[kN], b[kN];
        ld16(src + h * dim + i, a);
        ld16(src + h * dim + i + half, b);
        rotate_vec<kN>(a, b, s_c0 + i, s_s0 + i, s_c1 + i, s_s1 + i);
        st16(dst + h * dim + i, a);
        st16(dst + h * dim + i + half, b);
      }
    } else {
      for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        const float a = ld(src + h * dim + i), b = ld(src + h * dim + i + half);
        st(dst + h * dim + i, rope_lo(a, b, s_c0[i], s_s0[i]));
        st(dst + h * dim + i + half, rope_hi(a, b, s_c1[i], s_s1[i]));
      }
    }
  }
}

__global__ void __launch_bounds__(256)
mrope_cos_sin_kernel(const int64_t *pos, const float *inv_freq, float *cos_out, float *sin_out,
                     int64_t rows, int half, int h_lim, int w_lim) {
  const int64_t total = rows * half;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % half);
    const int64_t r = idx / half;
    const float p = pair_position(i, (float)pos[r], (float)pos[rows + r], (float)pos[2 * rows + r],
                                  h_lim, w_lim);
    float s, c;
    sincosf(p * inv_freq[i], &s, &c);
    cos_out[r * 2 * half + i] = c;
    cos_out[r * 2 * half + i + half] = c;
    sin_out[r * 2 * half + i] = s;
    sin_out[r * 2 * half + i + half] = s;
  }
}

// ---- append + rotate ------------------------------------------------------------------------
struct AppendParams {
  void *q;
  const void *q_src;  // where q is read from; null = q itself (rotated in place)
  const void *k_new, *v_new;
  void *k_pages, *v_pages;
  const int32_t *block_table;
  int32_t *seq_lens;
  const int64_t *pos;
  const float *inv_freq_dev;
  int rotate, mrope, h_lim, w_lim;
  int batch, hq, hkv, d;
  int page_tokens, max_blocks, num_pages;
  int slot_delta;  // the token goes to slot seq_lens[b] + slot_delta (0, or -1 once a layer advanced)
  int advance;
};

// One CTA per sequence, one warp per head (query heads, then key heads, then value heads): rotates q
// in place, rotates k and copies v into slot seq_lens[b] + slot_delta of the sequence's pages (page
// layout (hkv, page_tokens, d)), then bumps seq_lens[b].  The kernel is a chain of dependent loads
// (length -> page id -> store address) over a few KB, so it is built for latency: every thread reads
// the length itself, each warp has its head's row in flight before the page id is known, cos / sin are
// computed once per sequence while those loads fly, and there is one block-wide barrier - which is
// also what orders every thread's read of the length before the bump.  In a multi-layer step the
// first layer appends with slot_delta 0 and advances, so that every layer's attention sees the new
// token; the later layers append with slot_delta -1 and do not advance.
template <typename T>
__global__ void __launch_bounds__(1024)
kv_append_rope_kernel(const AppendParams p, const InvFreqTable table) {
  __shared__ float s_cos[kMaxHalf], s_sin[kMaxHalf];
  grid_dependency_launch();  // the attention kernel that follows may be scheduled; it waits for this one's end
  const int b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int half = p.d / 2;
  const int q_heads = p.rotate ? p.hq : 0;  // without rotation q is left as it is
  const int n_heads = q_heads + 2 * p.hkv;
  const int len = p.seq_lens[b] + p.slot_delta;  // slot of the new token = tokens cached before it

  // this warp's first head: its row on the way before anything else is known
  T *q = reinterpret_cast<T *>(p.q) + (size_t)b * p.hq * p.d;
  const T *kn = reinterpret_cast<const T *>(p.k_new) + (size_t)b * p.hkv * p.d;
  const T *vn = reinterpret_cast<const T *>(p.v_new) + (size_t)b * p.hkv * p.d;
  const T *q_in = p.q_src ? reinterpret_cast<const T *>(p.q_src) + (size_t)b * p.hq * p.d : q;
  auto row_of = [&](int head) -> const T * {
    if (head < q_heads) return q_in + (size_t)head * p.d;
    if (head < q_heads + p.hkv) return kn + (size_t)(head - q_heads) * p.d;
    return vn + (size_t)(head - q_heads - p.hkv) * p.d;
  };
  constexpr int kPer = kMaxHalf / 32;  // pairs (i, i + half) per lane, i = lane + 32 j
  float a[kPer], bb[kPer];
  if (warp < n_heads) {
    const T *src = row_of(warp);
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int i = lane + 32 * j;
      a[j] = i < half ? ld(src + i) : 0.f;
      bb[j] = i < half ? ld(src + i + half) : 0.f;
    }
  }

  const int slot = len / p.page_tokens;
  int page = -1;
  if (len >= 0 && slot < p.max_blocks) page = p.block_table[(size_t)b * p.max_blocks + slot];
  const bool page_ok = page >= 0 && page < p.num_pages;
  if (!page_ok && threadIdx.x == 0)
    atomicOr(&g_error_word, (len >= 0 && slot < p.max_blocks) ? AXB200_ERR_BAD_PAGE
                                                              : AXB200_ERR_CAPACITY);
  const int tok = len % p.page_tokens;

  if (p.rotate) {  // cos/sin of each rotary pair once per sequence; every head reuses them
    float pt, ph, pw;
    if (p.pos == nullptr) {
      pt = ph = pw = (float)len;
    } else if (p.mrope) {
      pt = (float)p.pos[b];
      ph = (float)p.pos[p.batch + b];
      pw = (float)p.pos[2 * p.batch + b];
    } else {
      pt = ph = pw = (float)p.pos[b];
    }
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float f = p.mrope || p.inv_freq_dev ? p.inv_freq_dev[i] : table.f[i];
      const float posv = p.mrope ? pair_position(i, pt, ph, pw, p.h_lim, p.w_lim) : pt;
      sincosf(posv * f, &s_sin[i], &s_cos[i]);
    }
  }
  __syncthreads();  // tables ready; every thread has read the length

  for (int head = warp; head < n_heads; head += nwarps) {
    if (head != warp) {  // more heads than warps: fetch the next row
      const T *src = row_of(head);
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        const int i = lane + 32 * j;
        a[j] = i < half ? ld(src + i) : 0.f;
        bb[j] = i < half ? ld(src + i + half) : 0.f;
      }
    }
    const bool is_q = head < q_heads, is_k = !is_q && head < q_heads + p.hkv;
    T *dst;
    if (is_q) {
      dst = q + (size_t)head * p.d;
    } else {
      if (!page_ok) continue;
      const int h = is_k ? head - q_heads : head - q_heads - p.hkv;
      dst = reinterpret_cast<T *>(is_k ? p.k_pages : p.v_pages) +
            (((size_t)page * p.hkv + h) * p.page_tokens + tok) * p.d;
    }
    const bool rot = p.rotate && (is_q || is_k);
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int i = lane + 32 * j;
      if (i >= half) continue;
      if (rot) {
        const float c = s_cos[i], s = s_sin[i];
        st(dst + i, rope_lo(a[j], bb[j], c, s));
        st(dst + i + half, rope_hi(a[j], bb[j], c, s));
      } else {  // a value row, or a key row without rotation: the bits as they came
        const T *src = row_of(head);
        dst[i] = src[i];
        dst[i + half] = src[i + half];
      }
    }
  }
  if (p.advance && page_ok && threadIdx.x == 0) p.seq_lens[b] = len - p.slot_delta + 1;
}

// ---- prefill write: many tokens of ONE sequence into its pages -------------------------------------
// After a prefill the reference stores the whole (seq,hkv,d) K/V of the prompt as the cache
// (axono/python/axono/nn/kv_cache.py:96-100) with K already rotated by rope / rope_thd
// (examples/vlm/qwen3vl/model.py:358-362).  Here: one CTA per token; rotates q (in place, optional) and
// k with the token's own position(s) and scatters k/v into the sequence's pages at slots
// start .. start + n - 1.  The length is set by the host side afterwards (one store).
struct PrefillWriteParams {
  void *q;  // (n, hq, d) or null
  const void *k, *v;  // (n, hkv, d)
  void *k_pages, *v_pages;
  const int32_t *block_row;  // this sequence's row of the block table
  const int64_t *pos;        // (n) or (3, n) or null -> start + i
  const float *inv_freq_dev;
  int rotate, mrope, h_lim, w_lim;
  int n, hq, hkv, d, page_tokens, max_blocks, num_pages, start;
  int vec;  // every pointer 16-byte aligned and d / 2 a multiple of 16 bytes' worth of T
};

template <typename T>
__global__ void __launch_bounds__(256)
kv_prefill_write_kernel(const PrefillWriteParams p, const InvFreqTable table) {
  const int i_tok = blockIdx.x;
  const int slot_tok = p.start + i_tok;
  const int half = p.d / 2;
  float pt, ph, pw;
  if (p.pos == nullptr) {
    pt = ph = pw = (float)slot_tok;
  } else if (p.mrope) {
    pt = (float)p.pos[i_tok];
    ph = (float)p.pos[p.n + i_tok];
    pw = (float)p.pos[2 * p.n + i_tok];
  } else {
    pt = ph = pw = (float)p.pos[i_tok];
  }
  const int blk = slot_tok / p.page_tokens;
  int page = -1;
  if (blk < p.max_blocks) page = p.block_row[blk];
  const bool page_ok = page >= 0 && page < p.num_pages;
  if (!page_ok && threadIdx.x == 0)
    atomicOr(&g_error_word, blk < p.max_blocks ? AXB200_ERR_BAD_PAGE : AXB200_ERR_CAPACITY);
  const int tok = slot_tok % p.page_tokens;

  __shared__ float s_cos[kMaxHalf], s_sin[kMaxHalf];
  if (p.rotate) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float f = p.mrope || p.inv_freq_dev ? p.inv_freq_dev[i] : table.f[i];
      const float posv = p.mrope ? pair_position(i, pt, ph, pw, p.h_lim, p.w_lim) : pt;
      sincosf(posv * f, &s_sin[i], &s_cos[i]);
    }
    __syncthreads();
  }
  T *q = p.q ? reinterpret_cast<T *>(p.q) + (size_t)i_tok * p.hq * p.d : nullptr;
  const T *kn = reinterpret_cast<const T *>(p.k) + (size_t)i_tok * p.hkv * p.d;
  const T *vn = reinterpret_cast<const T *>(p.v) + (size_t)i_tok * p.hkv * p.d;
  if (p.vec) {  // 16 bytes per access: the same arithmetic per element as below
    constexpr int kN = Vec16<T>::kN;
    const int per_head = half / kN;
    const int q_items = (q && p.rotate) ? p.hq * per_head : 0, k_items = page_ok ? p.hkv * per_head : 0;
    for (int idx = threadIdx.x; idx < q_items + k_items; idx += blockDim.x) {
      const bool is_q = idx < q_items;
      const int j = is_q ? idx : idx - q_items;
      const int h = j / per_head, i = (j - h * per_head) * kN;
      const T *src = is_q ? q + (size_t)h * p.d : kn + (size_t)h * p.d;
      T *dst = is_q ? q + (size_t)h * p.d
                    : reinterpret_cast<T *>(p.k_pages) + (((size_t)page * p.hkv + h) * p.page_tokens + tok) * p.d;
      float a[kN], b[kN];
      ld16(src + i, a);
      ld16(src + i + half, b);
      if (p.rotate) rotate_vec<kN>(a, b, s_cos + i, s_sin + i, s_cos + i, s_sin + i);
      st16(dst + i, a);
      st16(dst + i + half, b);
    }
    if (page_ok) {
      const int per_row = p.d / kN;
      for (int idx = threadIdx.x; idx < p.hkv * per_row; idx += blockDim.x) {
        const int h = idx / per_row, c = (idx - h * per_row) * kN;
        *reinterpret_cast<uint4 *>(reinterpret_cast<T *>(p.v_pages) + (((size_t)page * p.hkv + h) * p.page_tokens + tok) * p.d + c) =
            *reinterpret_cast<const uint4 *>(vn + (size_t)h * p.d + c);
      }
    }
    return;
  }
  const int q_pairs = q ? p.hq * half : 0, k_pairs = p.hkv * half;
  for (int idx = threadIdx.x; idx < q_pairs + k_pairs; idx += blockDim.x) {
    const bool is_q = idx < q_pairs;
    const int j = is_q ? idx : idx - q_pairs;
    const int h = j / half, i = j % half;
    const float c = p.rotate ? s_cos[i] : 1.f, sn = p.rotate ? s_sin[i] : 0.f;
    if (is_q) {
      if (p.rotate) {
        T *row = q + (size_t)h * p.d;
        const float a = ld(row + i), bb = ld(row + i + half);
        st(row + i, rope_lo(a, bb, c, sn));
        st(row + i + half, rope_hi(a, bb, c, sn));
      }
    } else if (page_ok) {
      const T *row = kn + (size_t)h * p.d;
      T *dst = reinterpret_cast<T *>(p.k_pages) + (((size_t)page * p.hkv + h) * p.page_tokens + tok) * p.d;
      if (p.rotate) {
        const float a = ld(row + i), bb = ld(row + i + half);
        st(dst + i, rope_lo(a, bb, c, sn));
        st(dst + i + half, rope_hi(a, bb, c, sn));
      } else {
        dst[i] = row[i];
        dst[i + half] = row[i + half];
      }
    }
  }
  if (page_ok) {
    for (int idx = threadIdx.x; idx < p.hkv * p.d; idx += blockDim.x) {
      const int h = idx / p.d, c = idx % p.d;
      reinterpret_cast<T *>(p.v_pages)[(((size_t)page * p.hkv + h) * p.page_tokens + tok) * p.d + c] = vn[idx];
    }
  }
}

// ---- per-head norm + rotate + append straight from the QKV projection output ----------------------
// The reference's layer runs, after the QKV GEMM: reshape, rms_norm(q), rms_norm(k) over head_dim
// (examples/vlm/qwen3vl/model.py:353-357), rope on both (:358-359), cache.update (:362).  Here one
// launch does all of it: one CTA per sequence, one warp per head; the warp reads its head's row from
// the GEMM output (row stride `ld`), reduces the sum of squares with shuffles, scales by the norm
// weight, rotates, and writes q to a contiguous (batch,hq,d) buffer and k/v into the page slot.
struct FusedQkvParams {
  const void *qkv;  // (batch, ld): [q heads | k heads | v heads] per row
  long long ld;
  const void *q_norm_w, *k_norm_w;  // (d) or null
  float eps;
  void *q_out;  // (batch, hq, d)
};

template <typename T>
__global__ void __launch_bounds__(1024)
qkv_norm_rope_append_kernel(const AppendParams p, const FusedQkvParams f, const InvFreqTable table) {
  __shared__ int s_len;
  grid_dependency_launch();  // the layer's attention kernel may be scheduled; it waits for this one's end
  const int b = blockIdx.x;
  if (threadIdx.x == 0) s_len = p.seq_lens[b] + p.slot_delta;
  __syncthreads();
  const int len = s_len;
  const int half = p.d / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;

  float pt, ph, pw;
  if (p.pos == nullptr) {
    pt = ph = pw = (float)len;
  } else if (p.mrope) {
    pt = (float)p.pos[b];
    ph = (float)p.pos[p.batch + b];
    pw = (float)p.pos[2 * p.batch + b];
  } else {
    pt = ph = pw = (float)p.pos[b];
  }
  const int slot = len / p.page_tokens;
  int page = -1;
  if (len >= 0 && slot < p.max_blocks) page = p.block_table[(size_t)b * p.max_blocks + slot];
  const bool page_ok = page >= 0 && page < p.num_pages;
  if (!page_ok && threadIdx.x == 0)
    atomicOr(&g_error_word, (len >= 0 && slot < p.max_blocks) ? AXB200_ERR_BAD_PAGE
                                                              : AXB200_ERR_CAPACITY);
  const int tok = len % p.page_tokens;
  const T *row = reinterpret_cast<const T *>(f.qkv) + (size_t)b * f.ld;

  // cos/sin of each rotary pair once per sequence; every head reuses them
  __shared__ float s_cos[kMaxHalf], s_sin[kMaxHalf];
  if (p.rotate) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float fr = p.mrope || p.inv_freq_dev ? p.inv_freq_dev[i] : table.f[i];
      const float posv = p.mrope ? pair_position(i, pt, ph, pw, p.h_lim, p.w_lim) : pt;
      sincosf(posv * fr, &s_sin[i], &s_cos[i]);
    }
    __syncthreads();
  }

  for (int head = warp; head < p.hq + 2 * p.hkv; head += nwarps) {
    const bool is_q = head < p.hq, is_k = !is_q && head < p.hq + p.hkv;
    const T *src = row + (size_t)head * p.d;
    T *dst;
    if (is_q) {
      dst = reinterpret_cast<T *>(f.q_out) + ((size_t)b * p.hq + head) * p.d;
    } else {
      if (!page_ok) continue;
      const int h = is_k ? head - p.hq : head - p.hq - p.hkv;
      dst = reinterpret_cast<T *>(is_k ? p.k_pages : p.v_pages) +
            (((size_t)page * p.hkv + h) * p.page_tokens + tok) * p.d;
    }
    if (!is_q && !is_k) {  // v: copy
      for (int c = lane; c < p.d; c += 32) dst[c] = src[c];
      continue;
    }
    // pairs (i, i+half), i = lane + 32*j
    float a[4], bb[4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = lane + 32 * j;
      a[j] = i < half ? ld(src + i) : 0.f;
      bb[j] = i < half ? ld(src + i + half) : 0.f;
      ss = fmaf(a[j], a[j], ss);
      ss = fmaf(bb[j], bb[j], ss);
    }
    const T *w = reinterpret_cast<const T *>(is_q ? f.q_norm_w : f.k_norm_w);
    float inv = 1.f;
    if (w) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
      inv = 1.0f / sqrtf(ss / (float)p.d + f.eps);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = lane + 32 * j;
      if (i >= half) continue;
      float x0 = a[j], x1 = bb[j];
      if (w) {
        x0 = x0 * inv * ld(w + i);
        x1 = x1 * inv * ld(w + i + half);
      }
      if (p.rotate) {
        const float sn = s_sin[i], cs = s_cos[i];
        const float r0 = rope_lo(x0, x1, cs, sn), r1 = rope_hi(x0, x1, cs, sn);
        x0 = r0;
        x1 = r1;
      }
      st(dst + i, x0);
      st(dst + i + half, x1);
    }
  }
  if (p.advance && page_ok) {
    __syncthreads();
    if (threadIdx.x == 0) p.seq_lens[b] = len - p.slot_delta + 1;
  }
}

// theta^(-2i/dim) with the host C library's powf, as src/ops/cpu/sequence.cpp:83-84 computes it.
void fill_table(InvFreqTable *t, float theta, int dim) {
  for (int i = 0; i < dim / 2 && i < kMaxHalf; ++i)
    t->f[i] = powf(theta, -2.0f * static_cast<float>(i) / static_cast<float>(dim));
}
}  // namespace

void rope_inv_freq_host(float theta, int dim, float *out) {
  for (int i = 0; i < dim / 2; ++i) out[i] = powf(theta, -2.0f * static_cast<float>(i) / static_cast<float>(dim));
}

namespace {

int grid_for(int64_t total) {
  int64_t blocks = (total + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return (int)blocks;
}

template <int kMode>
int rope_dispatch(const void *x, void *out, const int64_t *pos, const float *inv_freq,
                  const InvFreqTable &table, const float *cos_t, const float *sin_t, int64_t rows,
                  int heads, int dim, int h_lim, int w_lim, int dtype, cudaStream_t st) {
  const int64_t total = rows * heads * (dim / 2);
  if (total == 0) return AXB200_OK;
  if (dim / 2 <= kMaxHalf) {  // cos / sin once per (row, pair)
    const int grid = (int)(rows < 148 * 16 ? rows : 148 * 16);
    const int es = dtype == AXB200_FLOAT32 ? 4 : 2;
    const int vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0 &&
                    ((dim / 2) * es) % 16 == 0;
    if (dtype == AXB200_FLOAT32)
      rope_rows_kernel<float, kMode><<<grid, 128, 0, st>>>(
          reinterpret_cast<const float *>(x), reinterpret_cast<float *>(out), pos, inv_freq, table,
          cos_t, sin_t, rows, heads, dim, h_lim, w_lim, vec);
    else
      rope_rows_kernel<__half, kMode><<<grid, 128, 0, st>>>(
          reinterpret_cast<const __half *>(x), reinterpret_cast<__half *>(out), pos, inv_freq, table,
          cos_t, sin_t, rows, heads, dim, h_lim, w_lim, vec);
    return launch_status();
  }
  const int grid = grid_for(total);
  if (dtype == AXB200_FLOAT32)
    rope_kernel<float, kMode><<<grid, 256, 0, st>>>(
        reinterpret_cast<const float *>(x), reinterpret_cast<float *>(out), pos, inv_freq, table,
        cos_t, sin_t, rows, heads, dim, h_lim, w_lim);
  else
    rope_kernel<__half, kMode><<<grid, 256, 0, st>>>(
        reinterpret_cast<const __half *>(x), reinterpret_cast<__half *>(out), pos, inv_freq, table,
        cos_t, sin_t, rows, heads, dim, h_lim, w_lim);
  return launch_status();
}

int check_rope_args(const void *x, const void *out, int64_t rows, int heads, int dim, int dtype) {
  if (dtype != AXB200_FLOAT32 && dtype != AXB200_FLOAT16) return AXB200_UNSUPPORTED_TYPE;
  if (!x || !out) return AXB200_INVALID_PTR;
  if (rows < 0 || heads <= 0 || dim <= 0 || dim % 2 != 0 || dim / 2 > kMaxHalf)
    return AXB200_INVALID_ARGUMENT;
  return AXB200_OK;
}

}  // namespace
}  // namespace axb

extern "C" {

int axb200_rope(const void *x, const int64_t *pos, float theta, void *out, int64_t rows, int heads,
                int dim, int dtype, void *stream) {
  int st = axb::check_rope_args(x, out, rows, heads, dim, dtype);
  if (st != AXB200_OK) return st;
  if (!pos) return AXB200_INVALID_PTR;
  axb::InvFreqTable table{};
  axb::fill_table(&table, theta, dim);
  return axb::rope_dispatch<axb::kModeTheta>(x, out, pos, nullptr, table, nullptr, nullptr, rows,
                                             heads, dim, 0, 0, dtype,
                                             static_cast<cudaStream_t>(stream));
}

int axb200_rope_thd(const void *x, const int64_t *pos, const float *inv_freq, int t_sec, int h_sec,
                    int w_sec, void *out, int64_t rows, int heads, int dim, int dtype,
                    void *stream) {
  (void)t_sec;
  int st = axb::check_rope_args(x, out, rows, heads, dim, dtype);
  if (st != AXB200_OK) return st;
  if (!pos || !inv_freq) return AXB200_INVALID_PTR;
  axb::InvFreqTable table{};
  return axb::rope_dispatch<axb::kModeMrope>(x, out, pos, inv_freq, table, nullptr, nullptr, rows,
                                             heads, dim, h_sec * 3, w_sec * 3, dtype,
                                             static_cast<cudaStream_t>(stream));
}

int axb200_rope_with_cos_sin(const void *x, const float *cos_t, const float *sin_t, void *out,
                             int64_t rows, int heads, int dim, int dtype, void *stream) {
  int st = axb::check_rope_args(x, out, rows, heads, dim, dtype);
  if (st != AXB200_OK) return st;
  if (!cos_t || !sin_t) return AXB200_INVALID_PTR;
  axb::InvFreqTable table{};
  return axb::rope_dispatch<axb::kModeCosSin>(x, out, nullptr, nullptr, table, cos_t, sin_t, rows,
                                              heads, dim, 0, 0, dtype,
                                              static_cast<cudaStream_t>(stream));
}

int axb200_mrope_cos_sin(const int64_t *pos, const float *inv_freq, int h_sec, int w_sec,
                         float *cos_out, float *sin_out, int64_t rows, int half, void *stream) {
  if (!pos || !inv_freq || !cos_out || !sin_out) return AXB200_INVALID_PTR;
  if (half <= 0 || rows < 0) return AXB200_INVALID_ARGUMENT;
  if (rows == 0) return AXB200_OK;
  axb::mrope_cos_sin_kernel<<<axb::grid_for(rows * half), 256, 0,
                              static_cast<cudaStream_t>(stream)>>>(
      pos, inv_freq, cos_out, sin_out, rows, half, h_sec * 3, w_sec * 3);
  return axb::launch_status();
}

int axb200_kv_append_rope(void *q, const void *k_new, const void *v_new, void *k_pages,
                          void *v_pages, const int32_t *block_table, int32_t *seq_lens,
                          const int64_t *pos, const float *inv_freq, float theta, int rotate,
                          int mrope, int h_sec, int w_sec, int batch, int hq, int hkv, int d,
                          int page_tokens, int max_blocks, int num_pages, int dtype, int slot_delta,
                          int advance, void *stream) {
  return axb::kv_append_rope_from(q, nullptr, k_new, v_new, k_pages, v_pages, block_table, seq_lens, pos, inv_freq,
                                  theta, rotate, mrope, h_sec, w_sec, batch, hq, hkv, d, page_tokens, max_blocks,
                                  num_pages, dtype, slot_delta, advance, stream);
}

}  // extern "C"

// The append with q read from somewhere else than where it is written (q_src; null = in place): the
// host-buffer step reads q, k_new and v_new straight from page-locked host memory.
int axb::kv_append_rope_from(void *q, const void *q_src, const void *k_new, const void *v_new, void *k_pages,
                             void *v_pages, const int32_t *block_table, int32_t *seq_lens,
                             const int64_t *pos, const float *inv_freq, float theta, int rotate,
                             int mrope, int h_sec, int w_sec, int batch, int hq, int hkv, int d,
                             int page_tokens, int max_blocks, int num_pages, int dtype, int slot_delta,
                             int advance, void *stream) {
  if (dtype != AXB200_FLOAT32 && dtype != AXB200_FLOAT16) return AXB200_UNSUPPORTED_TYPE;
  if (!k_new || !v_new || !k_pages || !v_pages || !block_table || !seq_lens)
    return AXB200_INVALID_PTR;
  if (rotate && !q && hq > 0) return AXB200_INVALID_PTR;
  if (batch <= 0 || hq < 0 || hkv <= 0 || d <= 0 || d % 2 != 0 || d / 2 > axb::kMaxHalf ||
      page_tokens <= 0 || max_blocks <= 0 || num_pages <= 0 || slot_delta > 0 || slot_delta < -1)
    return AXB200_INVALID_ARGUMENT;
  if (rotate && mrope && !inv_freq) return AXB200_INVALID_PTR;
  axb::AppendParams p{};
  p.q = q;
  p.q_src = (q && rotate) ? q_src : nullptr;
  p.k_new = k_new;
  p.v_new = v_new;
  p.k_pages = k_pages;
  p.v_pages = v_pages;
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.pos = pos;
  p.inv_freq_dev = inv_freq;
  p.rotate = rotate;
  p.mrope = mrope;
  p.h_lim = h_sec * 3;
  p.w_lim = w_sec * 3;
  p.batch = batch;
  p.hq = q ? hq : 0;
  p.hkv = hkv;
  p.d = d;
  p.page_tokens = page_tokens;
  p.max_blocks = max_blocks;
  p.num_pages = num_pages;
  p.slot_delta = slot_delta;
  p.advance = advance;
  axb::InvFreqTable table{};
  if (rotate && !inv_freq) axb::fill_table(&table, theta, d);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int heads = (rotate ? p.hq : 0) + 2 * hkv;  // one warp per head, up to the block limit
  const int threads = heads >= 32 ? 1024 : (heads < 2 ? 64 : heads * 32);
  if (dtype == AXB200_FLOAT32)
    axb::kv_append_rope_kernel<float><<<batch, threads, 0, st>>>(p, table);
  else
    axb::kv_append_rope_kernel<__half><<<batch, threads, 0, st>>>(p, table);
  return axb::launch_status();
}

extern "C" {

int axb200_kv_prefill_write(void *q, const void *k, const void *v, void *k_pages, void *v_pages,
                            const int32_t *block_row, const int64_t *pos, const float *inv_freq,
                            float theta, int rotate, int mrope, int h_sec, int w_sec, int64_t n, int hq,
                            int hkv, int d, int page_tokens, int max_blocks, int num_pages,
                            int64_t start, int dtype, void *stream) {
  if (dtype != AXB200_FLOAT32 && dtype != AXB200_FLOAT16) return AXB200_UNSUPPORTED_TYPE;
  if (!k || !v || !k_pages || !v_pages || !block_row) return AXB200_INVALID_PTR;
  if (n < 0 || n > 0x7fffffff || hq < 0 || hkv <= 0 || d <= 0 || d % 2 != 0 || d / 2 > axb::kMaxHalf ||
      page_tokens <= 0 || max_blocks <= 0 || num_pages <= 0 || start < 0 || start + n > 0x7fffffff)
    return AXB200_INVALID_ARGUMENT;
  if (rotate && mrope && !inv_freq) return AXB200_INVALID_PTR;
  if (n == 0) return AXB200_OK;
  axb::PrefillWriteParams p{};
  p.q = q;
  p.k = k;
  p.v = v;
  p.k_pages = k_pages;
  p.v_pages = v_pages;
  p.block_row = block_row;
  p.pos = pos;
  p.inv_freq_dev = inv_freq;
  p.rotate = rotate;
  p.mrope = mrope;
  p.h_lim = h_sec * 3;
  p.w_lim = w_sec * 3;
  p.n = (int)n;
  p.hq = hq;
  p.hkv = hkv;
  p.d = d;
  p.page_tokens = page_tokens;
  p.max_blocks = max_blocks;
  p.num_pages = num_pages;
  p.start = (int)start;
  const int es = dtype == AXB200_FLOAT32 ? 4 : 2;
  p.vec = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
            reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages)) & 15u) == 0 &&
          ((d / 2) * es) % 16 == 0;
  axb::InvFreqTable table{};
  if (rotate && !inv_freq) axb::fill_table(&table, theta, d);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == AXB200_FLOAT32)
    axb::kv_prefill_write_kernel<float><<<(unsigned)n, 256, 0, st>>>(p, table);
  else
    axb::kv_prefill_write_kernel<__half><<<(unsigned)n, 256, 0, st>>>(p, table);
  return axb::launch_status();
}

int axb200_qkv_norm_rope_append(const void *qkv, int64_t ld, const void *q_norm_w,
                                const void *k_norm_w, float eps, void *q_out, void *k_pages,
                                void *v_pages, const int32_t *block_table, int32_t *seq_lens,
                                const int64_t *pos, const float *inv_freq, float theta, int rotate,
                                int mrope, int h_sec, int w_sec, int batch, int hq, int hkv, int d,
                                int page_tokens, int max_blocks, int num_pages, int dtype,
                                int slot_delta, int advance, void *stream) {
  if (dtype != AXB200_FLOAT32 && dtype != AXB200_FLOAT16) return AXB200_UNSUPPORTED_TYPE;
  if (!qkv || !q_out || !k_pages || !v_pages || !block_table || !seq_lens) return AXB200_INVALID_PTR;
  if (batch <= 0 || hq <= 0 || hkv <= 0 || d <= 0 || d % 2 != 0 || d / 2 > axb::kMaxHalf ||
      page_tokens <= 0 || max_blocks <= 0 || num_pages <= 0 || slot_delta > 0 || slot_delta < -1 ||
      ld < (int64_t)(hq + 2 * hkv) * d)
    return AXB200_INVALID_ARGUMENT;
  if (rotate && mrope && !inv_freq) return AXB200_INVALID_PTR;
  axb::AppendParams p{};
  p.k_pages = k_pages;
  p.v_pages = v_pages;
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.pos = pos;
  p.inv_freq_dev = inv_freq;
  p.rotate = rotate;
  p.mrope = mrope;
  p.h_lim = h_sec * 3;
  p.w_lim = w_sec * 3;
  p.batch = batch;
  p.hq = hq;
  p.hkv = hkv;
  p.d = d;
  p.page_tokens = page_tokens;
  p.max_blocks = max_blocks;
  p.num_pages = num_pages;
  p.slot_delta = slot_delta;
  p.advance = advance;
  axb::FusedQkvParams f{};
  f.qkv = qkv;
  f.ld = ld;
  f.q_norm_w = q_norm_w;
  f.k_norm_w = k_norm_w;
  f.eps = eps;
  f.q_out = q_out;
  axb::InvFreqTable table{};
  if (rotate && !inv_freq) axb::fill_table(&table, theta, d);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // one warp per head (q, k and v heads) up to the block limit: the heads of a row are independent and
  // the kernel is a chain of dependent loads, so looping a warp over several heads only adds latency
  const int heads = hq + 2 * hkv;
  const int threads = heads >= 32 ? 1024 : (heads < 2 ? 64 : heads * 32);
  if (dtype == AXB200_FLOAT32)
    axb::qkv_norm_rope_append_kernel<float><<<batch, threads, 0, st>>>(p, f, table);
  else
    axb::qkv_norm_rope_append_kernel<__half><<<batch, threads, 0, st>>>(p, f, table);
  return axb::launch_status();
}

}  // extern "C"
