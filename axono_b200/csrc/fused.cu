// Fused norm / activation kernels around the decode attention, for sm_100a.  Replaces the
// reference's AddRmsNorm and SiluMul (src/ops/cuda/fused.cu:28-110), RmsNorm
// (src/ops/cuda/llm.cu:139-158,345-373) and Concat (src/ops/cuda/sequence.cu:474-521).
// All arithmetic is fp32 whatever the storage type; loads and stores are 128-bit where the
// pointers and row lengths allow.
#include <math.h>

#include "common.cuh"

namespace axb {
namespace {

template <typename T>
struct Vec;  // 16-byte vector of T
template <>
struct Vec<float> {
  static constexpr int kN = 4;
  float4 raw;
  __device__ __forceinline__ float get(int i) const { return reinterpret_cast<const float *>(&raw)[i]; }
  __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<float *>(&raw)[i] = v; }
};
template <>
struct Vec<__half> {
  static constexpr int kN = 8;
  uint4 raw;
  __device__ __forceinline__ float get(int i) const {
    return __half2float(reinterpret_cast<const __half *>(&raw)[i]);
  }
  __device__ __forceinline__ void set(int i, float v) {
    reinterpret_cast<__half *>(&raw)[i] = __float2half_rn(v);
  }
};

template <typename T>
__device__ __forceinline__ float ldf(const T *p);
template <>
__device__ __forceinline__ float ldf<float>(const float *p) { return *p; }
template <>
__device__ __forceinline__ float ldf<__half>(const __half *p) { return __half2float(*p); }
template <typename T>
__device__ __forceinline__ void stf(T *p, float v);
template <>
__device__ __forceinline__ void stf<float>(float *p, float v) { *p = v; }
template <>
__device__ __forceinline__ void stf<__half>(__half *p, float v) { *p = __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// Sum over the CTA; every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float *scratch /* >= 32 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < nwarps ? scratch[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// ---- add_rms_norm: y = x + res; out = y * rsqrt(mean(y^2) + eps) * w -----------------------------
// One CTA per row.  Vector path: each thread keeps up to kMaxVec 16-byte vectors of y in
// registers between the two phases, so x and res are read once and y/out written once.
constexpr int kNormThreads = 256;
constexpr int kMaxVec = 4;

template <typename T, bool kHasResidual>
__global__ void __launch_bounds__(kNormThreads)
add_rms_norm_vec_kernel(const T *x, const T *res, const T *w, float eps, T *y, T *out, int hidden) {
  __shared__ float scratch[32];
  using V = Vec<T>;
  const int64_t row = blockIdx.x;
  const int nvec = hidden / V::kN;
  const V *xv = reinterpret_cast<const V *>(x + row * hidden);
  const V *rv = kHasResidual ? reinterpret_cast<const V *>(res + row * hidden) : nullptr;
  const V *wv = reinterpret_cast<const V *>(w);
  V *yv = kHasResidual ? reinterpret_cast<V *>(y + row * hidden) : nullptr;
  V *ov = reinterpret_cast<V *>(out + row * hidden);

  float vals[kMaxVec][V::kN];
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int vi = threadIdx.x + j * kNormThreads;
    if (vi < nvec) {
      V a = xv[vi];
      if (kHasResidual) {
        const V r = rv[vi];
        V yy;
#pragma unroll
        for (int e = 0; e < V::kN; ++e) {
          vals[j][e] = a.get(e) + r.get(e);
          yy.set(e, vals[j][e]);
        }
        yv[vi] = yy;
      } else {
#pragma unroll
        for (int e = 0; e < V::kN; ++e) vals[j][e] = a.get(e);
      }
#pragma unroll
      for (int e = 0; e < V::kN; ++e) sum = fmaf(vals[j][e], vals[j][e], sum);
    }
  }
  sum = block_sum(sum, scratch);
  const float rms = 1.0f / sqrtf(sum / (float)hidden + eps);
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int vi = threadIdx.x + j * kNormThreads;
    if (vi < nvec) {
      V o;
      if (w) {
        const V ww = wv[vi];
#pragma unroll
        for (int e = 0; e < V::kN; ++e) o.set(e, vals[j][e] * rms * ww.get(e));
      } else {
#pragma unroll
        for (int e = 0; e < V::kN; ++e) o.set(e, vals[j][e] * rms);
      }
      ov[vi] = o;
    }
  }
}

// Any hidden size / alignment: two passes, the second recomputes x + res.
template <typename T, bool kHasResidual>
__global__ void __launch_bounds__(kNormThreads)
add_rms_norm_generic_kernel(const T *x, const T *res, const T *w, float eps, T *y, T *out,
                            int hidden) {
  __shared__ float scratch[32];
  const int64_t row = blockIdx.x;
  const T *xr = x + row * hidden;
  const T *rr = kHasResidual ? res + row * hidden : nullptr;
  float sum = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = ldf(xr + i);
    if (kHasResidual) {
      v += ldf(rr + i);
      stf(y + row * hidden + i, v);
    }
    sum = fmaf(v, v, sum);
  }
  sum = block_sum(sum, scratch);
  const float rms = 1.0f / sqrtf(sum / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = ldf(xr + i);
    if (kHasResidual) v += ldf(rr + i);
    v *= rms;
    if (w) v *= ldf(w + i);
    stf(out + row * hidden + i, v);
  }
}

// RMS norm over short rows (per-head q/k norm, cols <= 1024): one warp per row.
template <typename T>
__global__ void __launch_bounds__(256)
rms_norm_warp_kernel(const T *x, const T *w, float eps, T *out, int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T *xr = x + row * cols;
  float v[32];
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const int c = lane + 32 * j;
    v[j] = c < cols ? ldf(xr + c) : 0.f;
    sum = fmaf(v[j], v[j], sum);
  }
  sum = warp_sum(sum);
  const float inv = 1.0f / sqrtf(sum / (float)cols + eps);
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const int c = lane + 32 * j;
    if (c < cols) {
      const float normed = v[j] * inv;
      stf(out + row * cols + c, w ? normed * ldf(w + c) : normed);
    }
  }
}

// ---- silu_mul -----------------------------------------------------------------------------------
__device__ __forceinline__ float silu_mul1(float g, float u) { return g / (1.0f + expf(-g)) * u; }

template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_vec_kernel(const T *gate, const T *up, T *out, int64_t nvec) {
  using V = Vec<T>;
  const V *gv = reinterpret_cast<const V *>(gate);
  const V *uv = reinterpret_cast<const V *>(up);
  V *ov = reinterpret_cast<V *>(out);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    const V g = gv[i], u = uv[i];
    V o;
#pragma unroll
    for (int e = 0; e < V::kN; ++e) o.set(e, silu_mul1(g.get(e), u.get(e)));
    ov[i] = o;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_scalar_kernel(const T *gate, const T *up, T *out, int64_t begin, int64_t n) {
  for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    stf(out + i, silu_mul1(ldf(gate + i), ldf(up + i)));
}

// silu(gate) * up where gate and up are the two halves of each row of one matrix (the output of a
// fused gate|up projection): in (rows, ld) with gate = in[r, 0:n], up = in[r, n:2n]; out (rows, n).
template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_rows_kernel(const T *in, long long ld, int n, long long rows, T *out, bool vec) {
  using V = Vec<T>;
  if (vec) {
    const int nv = n / V::kN;
    const long long total = rows * nv;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
      const long long r = i / nv;
      const int c = (int)(i % nv);
      const V g = reinterpret_cast<const V *>(in + r * ld)[c];
      const V u = reinterpret_cast<const V *>(in + r * ld + n)[c];
      V o;
#pragma unroll
      for (int e = 0; e < V::kN; ++e) o.set(e, silu_mul1(g.get(e), u.get(e)));
      reinterpret_cast<V *>(out + r * n)[c] = o;
    }
  } else {
    const long long total = rows * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
      const long long r = i / n;
      const int c = (int)(i % n);
      stf(out + i, silu_mul1(ldf(in + r * ld + c), ldf(in + r * ld + n + c)));
    }
  }
}

// ---- embedding gather and argmax over the last dim (the ends of a decode step) -----------------
// Replaces the reference's EmbeddingKernel and ArgmaxKernel (src/ops/cuda/sequence.cu:75-81,262-292).
// Embedding: one CTA per id, 16-byte copies of the table row; an id outside [0, vocab) sets
// AXB200_ERR_BAD_INDEX and yields a zero row.
template <typename IdT>
__global__ void __launch_bounds__(256)
embedding_kernel(const IdT *ids, const uint8_t *table, uint8_t *out, long long vocab, size_t row_bytes,
                 bool vec) {
  const long long id = (long long)ids[blockIdx.x];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0) atomicOr(&g_error_word, AXB200_ERR_BAD_INDEX);
  const uint8_t *src = table + (size_t)(ok ? id : 0) * row_bytes;
  uint8_t *dst = out + (size_t)blockIdx.x * row_bytes;
  if (vec) {
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (size_t i = threadIdx.x; i < row_bytes / 16; i += blockDim.x)
      reinterpret_cast<uint4 *>(dst)[i] = ok ? reinterpret_cast<const uint4 *>(src)[i] : zero;
  } else {
    for (size_t i = threadIdx.x; i < row_bytes; i += blockDim.x) dst[i] = ok ? src[i] : 0;
  }
}

// Argmax with the reference's CPU rule (src/ops/cpu/sequence.cpp:370-400): best = 0, then
// `if (row[c] > row[best]) best = c` left to right, i.e. the lowest index among equal maxima and a
// NaN at index 0 is never displaced.  One CTA per row.
struct ArgBest {
  float v;
  int i;
};
__device__ __forceinline__ ArgBest arg_better(ArgBest a, ArgBest b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// 16 bytes of a row as floats (4 floats or 8 halves)
__device__ __forceinline__ void arg_ld16(const float *p, float (&f)[4]) {
  const float4 v = *reinterpret_cast<const float4 *>(p);
  f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
}
__device__ __forceinline__ void arg_ld16(const __half *p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4 *>(p);
  const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(h[i]);
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}

template <typename T>
__global__ void __launch_bounds__(1024)
argmax_kernel(const T *x, int64_t *out, int cols, int vec) {  // vec: rows are 16-byte aligned multiples of 16 bytes
  __shared__ ArgBest s_best[32];
  const T *row = x + (size_t)blockIdx.x * cols;
  ArgBest best{-INFINITY, 0x7fffffff};
  if (vec) {
    // a vocabulary-sized row is hundreds of KB per CTA: 16-byte loads, four in flight per thread
    constexpr int kN = 16 / (int)sizeof(T), kUnroll = 4;
    const int nvec = cols / kN;
    for (int v0 = threadIdx.x; v0 < nvec; v0 += blockDim.x * kUnroll) {
      float f[kUnroll][kN];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int vi = v0 + u * blockDim.x;
        if (vi < nvec) arg_ld16(row + (size_t)vi * kN, f[u]);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int vi = v0 + u * blockDim.x;
        if (vi < nvec) {
#pragma unroll
          for (int j = 0; j < kN; ++j) {
            const float v = f[u][j];
            const int c = vi * kN + j;
            if (v > best.v || (v == best.v && c < best.i)) best = ArgBest{v, c};  // NaN never wins
          }
        }
      }
    }
  } else {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float v = ldf(row + c);
      if (v > best.v || (v == best.v && c < best.i)) best = ArgBest{v, c};  // NaN never wins
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    ArgBest o{__shfl_xor_sync(0xffffffffu, best.v, off), __shfl_xor_sync(0xffffffffu, best.i, off)};
    best = arg_better(best, o);
  }
  if ((threadIdx.x & 31) == 0) s_best[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) best = arg_better(best, s_best[w]);
    const float first = ldf(row);
    // row[0] NaN: nothing compares greater; every value -inf or NaN: index 0 stays
    out[blockIdx.x] = (first != first || best.i == 0x7fffffff) ? 0 : best.i;
  }
}

// ---- fp16 <-> fp32 cast (IEEE, round to nearest even) -------------------------------------------
template <typename Src, typename Dst>
__global__ void __launch_bounds__(256)
cast_kernel(const Src *src, Dst *dst, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    stf(dst + i, ldf(src + i));
}

// ---- concat (bytes) -----------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
concat_bytes_kernel(const uint8_t *a, const uint8_t *b, uint8_t *out, int64_t outer, size_t a_bytes,
                    size_t b_bytes) {
  const size_t row = a_bytes + b_bytes;
  const size_t total = (size_t)outer * row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t o = i / row, c = i % row;
    out[i] = c < a_bytes ? a[o * a_bytes + c] : b[o * b_bytes + (c - a_bytes)];
  }
}

int blocks_for(int64_t work, int per_block) {
  int64_t blocks = (work + per_block - 1) / per_block;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return (int)blocks;
}

bool al16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T, bool kRes>
int norm_launch(const void *x, const void *res, const void *w, float eps, void *y, void *out,
                int64_t rows, int hidden, cudaStream_t st) {
  const T *xp = static_cast<const T *>(x), *rp = static_cast<const T *>(res),
          *wp = static_cast<const T *>(w);
  T *yp = static_cast<T *>(y), *op = static_cast<T *>(out);
  constexpr int n = Vec<T>::kN;
  const bool vec = hidden % n == 0 && hidden / n <= kNormThreads * kMaxVec && al16(x) &&
                   al16(out) && (!w || al16(w)) && (!kRes || (al16(res) && al16(y)));
  if (vec)
    add_rms_norm_vec_kernel<T, kRes><<<(unsigned)rows, kNormThreads, 0, st>>>(xp, rp, wp, eps, yp, op, hidden);
  else
    add_rms_norm_generic_kernel<T, kRes><<<(unsigned)rows, kNormThreads, 0, st>>>(xp, rp, wp, eps, yp, op, hidden);
  return launch_status();
}

}  // namespace
}  // namespace axb

extern "C" {

int axb200_add_rms_norm(const void *x, const void *residual, const void *weight, float eps,
                        void *y, void *out, int64_t rows, int hidden, int dtype, void *stream) {
  if (dtype != AXB200_FLOAT32 && dtype != AXB200_FLOAT16) return AXB200_UNSUPPORTED_TYPE;
  if (!x || !residual || !weight || !y || !out) return AXB200_INVALID_PTR;
  if (rows < 0 || hidden <= 0 || rows > 0x7fffffff) return AXB200_INVALID_ARGUMENT;
  if (rows == 0) return AXB200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == AXB200_FLOAT32
             ? axb::norm_launch<float, true>(x, residual, weight, eps, y, out, rows, hidden, st)
             : axb::norm_launch<__half, true>(x, residual, weight, eps, y, out, rows, hidden, st);
}

int axb200_rms_norm(const void *x, const void *weight, float eps, void *out, int64_t rows, int cols,
                    int dtype, void *stream) {
  if (dtype != AXB200_FLOAT32 && dtype != AXB200_FLOAT16) return AXB200_UNSUPPORTED_TYPE;
  if (!x || !out) return AXB200_INVALID_PTR;
  if (rows < 0 || cols <= 0 || rows > 0x7fffffff) return AXB200_INVALID_ARGUMENT;
  if (rows == 0) return AXB200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cols <= 1024 && rows >= 16) {
    const unsigned grid = (unsigned)((rows + 7) / 8);
    if (dtype == AXB200_FLOAT32)
      axb::rms_norm_warp_kernel<float><<<grid, 256, 0, st>>>(
          static_cast<const float *>(x), static_cast<const float *>(weight), eps,
          static_cast<float *>(out), rows, cols);
    else
      axb::rms_norm_warp_kernel<__half><<<grid, 256, 0, st>>>(
          static_cast<const __half *>(x), static_cast<const __half *>(weight), eps,
          static_cast<__half *>(out), rows, cols);
    return axb::launch_status();
  }
  return dtype == AXB200_FLOAT32
             ? axb::norm_launch<float, false>(x, nullptr, weight, eps, nullptr, out, rows, cols, st)
             : axb::norm_launch<__half, false>(x, nullptr, weight, eps, nullptr, out, rows, cols, st);
}

int axb200_silu_mul(const void *gate, const void *up, void *out, int64_t n, int dtype,
                    void *stream) {
  if (dtype != AXB200_FLOAT32 && dtype != AXB200_FLOAT16) return AXB200_UNSUPPORTED_TYPE;
  if (!gate || !up || !out) return AXB200_INVALID_PTR;
  if (n < 0) return AXB200_INVALID_ARGUMENT;
  if (n == 0) return AXB200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool aligned = axb::al16(gate) && axb::al16(up) && axb::al16(out);
  if (dtype == AXB200_FLOAT32) {
    auto g = static_cast<const float *>(gate), u = static_cast<const float *>(up);
    auto o = static_cast<float *>(out);
    const int64_t nvec = aligned ? n / 4 : 0;
    if (nvec) axb::silu_mul_vec_kernel<float><<<axb::blocks_for(nvec, 256), 256, 0, st>>>(g, u, o, nvec);
    if (nvec * 4 < n)
      axb::silu_mul_scalar_kernel<float><<<axb::blocks_for(n - nvec * 4, 256), 256, 0, st>>>(g, u, o, nvec * 4, n);
  } else {
    auto g = static_cast<const __half *>(gate), u = static_cast<const __half *>(up);
    auto o = static_cast<__half *>(out);
    const int64_t nvec = aligned ? n / 8 : 0;
    if (nvec) axb::silu_mul_vec_kernel<__half><<<axb::blocks_for(nvec, 256), 256, 0, st>>>(g, u, o, nvec);
    if (nvec * 8 < n)
      axb::silu_mul_scalar_kernel<__half><<<axb::blocks_for(n - nvec * 8, 256), 256, 0, st>>>(g, u, o, nvec * 8, n);
  }
  return axb::launch_status();
}

int axb200_silu_mul_rows(const void *gate_up, int64_t ld, int n, int64_t rows, void *out, int dtype,
                         void *stream) {
  if (dtype != AXB200_FLOAT32 && dtype != AXB200_FLOAT16) return AXB200_UNSUPPORTED_TYPE;
  if (!gate_up || !out) return AXB200_INVALID_PTR;
  if (n <= 0 || rows < 0 || ld < 2 * (int64_t)n) return AXB200_INVALID_ARGUMENT;
  if (rows == 0) return AXB200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == AXB200_FLOAT32) {
    const bool vec = n % 4 == 0 && ld % 4 == 0 && axb::al16(gate_up) && axb::al16(out);
    axb::silu_mul_rows_kernel<float><<<axb::blocks_for(rows * n / (vec ? 4 : 1), 256), 256, 0, st>>>(
        static_cast<const float *>(gate_up), ld, n, rows, static_cast<float *>(out), vec);
  } else {
    const bool vec = n % 8 == 0 && ld % 8 == 0 && axb::al16(gate_up) && axb::al16(out);
    axb::silu_mul_rows_kernel<__half><<<axb::blocks_for(rows * n / (vec ? 8 : 1), 256), 256, 0, st>>>(
        static_cast<const __half *>(gate_up), ld, n, rows, static_cast<__half *>(out), vec);
  }
  return axb::launch_status();
}

int axb200_embedding(const void *ids, int ids_dtype, const void *table, void *out, int64_t n,
                     int64_t vocab, int hidden, int dtype, void *stream) {
  const size_t es = axb::dtype_size(dtype);
  if (es == 0 || (ids_dtype != AXB200_INT32 && ids_dtype != AXB200_INT64)) return AXB200_UNSUPPORTED_TYPE;
  if (!ids || !table || !out) return AXB200_INVALID_PTR;
  if (n < 0 || vocab <= 0 || hidden <= 0 || n > 0x7fffffff) return AXB200_INVALID_ARGUMENT;
  if (n == 0) return AXB200_OK;
  const size_t row_bytes = (size_t)hidden * es;
  const bool vec = row_bytes % 16 == 0 && axb::al16(table) && axb::al16(out);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ids_dtype == AXB200_INT64)
    axb::embedding_kernel<int64_t><<<(unsigned)n, 256, 0, st>>>(
        static_cast<const int64_t *>(ids), static_cast<const uint8_t *>(table), static_cast<uint8_t *>(out), vocab,
        row_bytes, vec);
  else
    axb::embedding_kernel<int32_t><<<(unsigned)n, 256, 0, st>>>(
        static_cast<const int32_t *>(ids), static_cast<const uint8_t *>(table), static_cast<uint8_t *>(out), vocab,
        row_bytes, vec);
  return axb::launch_status();
}

int axb200_argmax_last_dim(const void *x, int64_t *out, int64_t rows, int cols, int dtype, void *stream) {
  if (dtype != AXB200_FLOAT32 && dtype != AXB200_FLOAT16) return AXB200_UNSUPPORTED_TYPE;
  if (!x || !out) return AXB200_INVALID_PTR;
  if (rows < 0 || cols <= 0 || rows > 0x7fffffff) return AXB200_INVALID_ARGUMENT;
  if (rows == 0) return AXB200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t row_bytes = (size_t)cols * (dtype == AXB200_FLOAT32 ? 4 : 2);
  const int vec = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && row_bytes % 16 == 0;
  if (dtype == AXB200_FLOAT32)
    axb::argmax_kernel<float><<<(unsigned)rows, cols >= 8192 ? 1024 : 256, 0, st>>>(static_cast<const float *>(x), out, cols, vec);
  else
    axb::argmax_kernel<__half><<<(unsigned)rows, cols >= 8192 ? 1024 : 256, 0, st>>>(static_cast<const __half *>(x), out, cols, vec);
  return axb::launch_status();
}

int axb200_cast(const void *src, int src_dtype, void *dst, int dst_dtype, int64_t n, void *stream) {
  if (!src || !dst) return AXB200_INVALID_PTR;
  if (n < 0) return AXB200_INVALID_ARGUMENT;
  if (n == 0) return AXB200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = axb::blocks_for(n, 256);
  if (src_dtype == AXB200_FLOAT16 && dst_dtype == AXB200_FLOAT32)
    axb::cast_kernel<__half, float><<<grid, 256, 0, st>>>(static_cast<const __half *>(src), static_cast<float *>(dst), n);
  else if (src_dtype == AXB200_FLOAT32 && dst_dtype == AXB200_FLOAT16)
    axb::cast_kernel<float, __half><<<grid, 256, 0, st>>>(static_cast<const float *>(src), static_cast<__half *>(dst), n);
  else
    return AXB200_UNSUPPORTED_TYPE;
  return axb::launch_status();
}

int axb200_concat(const void *a, const void *b, void *out, int64_t outer, size_t a_bytes,
                  size_t b_bytes, void *stream) {
  if (!out || (a_bytes && !a) || (b_bytes && !b)) return AXB200_INVALID_PTR;
  if (outer < 0) return AXB200_INVALID_ARGUMENT;
  if (outer == 0 || a_bytes + b_bytes == 0) return AXB200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (outer == 1) {
    // Axis 0: two device-to-device copies, as the reference does (src/ops/cuda/sequence.cu:500-519).
    if (a_bytes && cudaMemcpyAsync(out, a, a_bytes, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
      return AXB200_DEVICE_ERROR;
    if (b_bytes && cudaMemcpyAsync(static_cast<uint8_t *>(out) + a_bytes, b, b_bytes,
                                   cudaMemcpyDeviceToDevice, st) != cudaSuccess)
      return AXB200_DEVICE_ERROR;
    return AXB200_OK;
  }
  const int64_t total = outer * (int64_t)(a_bytes + b_bytes);
  axb::concat_bytes_kernel<<<axb::blocks_for(total, 256), 256, 0, st>>>(
      static_cast<const uint8_t *>(a), static_cast<const uint8_t *>(b), static_cast<uint8_t *>(out),
      outer, a_bytes, b_bytes);
  return axb::launch_status();
}

}  // extern "C"
