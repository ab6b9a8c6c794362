// C shim over the reference's own CUDA operators (namespace axono::ops::cuda), linked against the
// reference's sources compiled for sm_100 where they lie (oracle/Makefile, target `refcuda`).
// TEST INFRASTRUCTURE ONLY: it gives the "reference kernels on a B200" timing and a second,
// GPU-side parity check; no product code loads it.
//
// Host buffers go in and out: inputs are wrapped as CPU tensors (Tensor::FromBorrowed,
// src/core/tensor.cpp:138-144) and moved with Tensor::to("cuda") (:146-177), the op runs on the
// reference's own stream and allocator, the result is moved back with to("cpu").  Timed loops
// bracket `iters` calls with CUDA events on the legacy default stream, the stream the reference
// launches on (src/core/cuda/graph.cu:58-62).
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <cstring>

#include "axono/core/tensor.h"
#include "axono/core/types.h"
#include "axono/ops/cuda/fused.h"
#include "axono/ops/cuda/gqa.h"
#include "axono/ops/cuda/sequence.h"

namespace {
using axono::core::Context;
using axono::core::DataType;
using axono::core::Shape;
using axono::core::Status;
using axono::core::Tensor;

Tensor ToCuda(DataType dt, const Shape &shape, const void *p) {
  return Tensor::FromBorrowed(dt, shape, p).to("cuda");
}
int Code(Status s) { return static_cast<int>(s); }

// Runs `fn` once for the result and `iters` more times between two events; returns ms per call.
template <typename Fn>
int Timed(Fn fn, int iters, double *ms_per_call) {
  Status st = fn();
  if (st != Status::OK) return Code(st);
  if (iters <= 0 || !ms_per_call) return 0;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  cudaDeviceSynchronize();
  cudaEventRecord(e0, 0);
  for (int i = 0; i < iters; ++i) fn();
  cudaEventRecord(e1, 0);
  cudaEventSynchronize(e1);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *ms_per_call = ms / iters;
  return 0;
}
}  // namespace

extern "C" {

// GqaDecodeAttention (src/ops/cuda/gqa.cu:139-182): q (1,hq,d), k/v (skv,hkv,d) fp32 host buffers.
int refcu_gqa_decode_f32(const float *q, const float *k, const float *v, float *out, size_t hq,
                         size_t hkv, size_t d, size_t skv, int iters, double *ms_per_call) {
  Context ctx;
  Tensor tq = ToCuda(DataType::FLOAT32, {1, hq, d}, q);
  Tensor tk = ToCuda(DataType::FLOAT32, {skv, hkv, d}, k);
  Tensor tv = ToCuda(DataType::FLOAT32, {skv, hkv, d}, v);
  Tensor res(DataType::FLOAT32, {1, hq, d}, "cuda");
  int rc = Timed([&] { return axono::ops::cuda::GqaDecodeAttention(ctx, tq, tk, tv, res); }, iters,
                 ms_per_call);
  if (rc != 0) return rc;
  Tensor host = res.to("cpu");
  std::memcpy(out, host.data(), hq * d * sizeof(float));
  return 0;
}

// ScaledDotProductAttention (src/ops/cuda/sequence.cu:451-472): q (sq,hq,d), k/v (skv,hkv,d) fp32 host
// buffers; the reference's kernel keeps skv scores per query in shared memory.
int refcu_sdpa_f32(const float *q, const float *k, const float *v, float *out, size_t sq, size_t hq, size_t hkv,
                   size_t d, size_t skv, int is_causal, int iters, double *ms_per_call) {
  Context ctx;
  Tensor tq = ToCuda(DataType::FLOAT32, {sq, hq, d}, q);
  Tensor tk = ToCuda(DataType::FLOAT32, {skv, hkv, d}, k);
  Tensor tv = ToCuda(DataType::FLOAT32, {skv, hkv, d}, v);
  Tensor res(DataType::FLOAT32, {sq, hq, d}, "cuda");
  int rc = Timed([&] { return axono::ops::cuda::ScaledDotProductAttention(ctx, tq, tk, tv, is_causal != 0, res); },
                 iters, ms_per_call);
  if (rc != 0) return rc;
  Tensor host = res.to("cpu");
  std::memcpy(out, host.data(), sq * hq * d * sizeof(float));
  return 0;
}

// AddRmsNorm (src/ops/cuda/fused.cu:91-110).
int refcu_add_rms_norm_f32(const float *x, const float *res_in, const float *w, float eps, float *y,
                           float *out, size_t rows, size_t hidden, int iters, double *ms_per_call) {
  Context ctx;
  Tensor tx = ToCuda(DataType::FLOAT32, {rows, hidden}, x);
  Tensor tr = ToCuda(DataType::FLOAT32, {rows, hidden}, res_in);
  Tensor tw = ToCuda(DataType::FLOAT32, {hidden}, w);
  Tensor ty(DataType::FLOAT32, {rows, hidden}, "cuda"), to(DataType::FLOAT32, {rows, hidden}, "cuda");
  int rc = Timed([&] { return axono::ops::cuda::AddRmsNorm(ctx, tx, tr, tw, eps, ty, to); }, iters,
                 ms_per_call);
  if (rc != 0) return rc;
  std::memcpy(y, ty.to("cpu").data(), rows * hidden * sizeof(float));
  std::memcpy(out, to.to("cpu").data(), rows * hidden * sizeof(float));
  return 0;
}

// SiluMul (src/ops/cuda/fused.cu:76-89).
int refcu_silu_mul_f32(const float *g, const float *u, float *y, size_t n, int iters,
                       double *ms_per_call) {
  Context ctx;
  Tensor tg = ToCuda(DataType::FLOAT32, {n}, g);
  Tensor tu = ToCuda(DataType::FLOAT32, {n}, u);
  Tensor ty(DataType::FLOAT32, {n}, "cuda");
  int rc = Timed([&] { return axono::ops::cuda::SiluMul(ctx, tg, tu, ty); }, iters, ms_per_call);
  if (rc != 0) return rc;
  std::memcpy(y, ty.to("cpu").data(), n * sizeof(float));
  return 0;
}

// Rope (src/ops/cuda/sequence.cu:318-342).
int refcu_rope_f32(const float *x, const int64_t *pos, float theta, float *out, size_t rows,
                   size_t heads, size_t dim, int iters, double *ms_per_call) {
  Context ctx;
  Tensor tx = ToCuda(DataType::FLOAT32, {rows, heads, dim}, x);
  Tensor tp = ToCuda(DataType::INT64, {rows}, pos);
  Tensor to(DataType::FLOAT32, {rows, heads, dim}, "cuda");
  int rc = Timed([&] { return axono::ops::cuda::Rope(ctx, tx, tp, theta, to); }, iters, ms_per_call);
  if (rc != 0) return rc;
  std::memcpy(out, to.to("cpu").data(), rows * heads * dim * sizeof(float));
  return 0;
}

}  // extern "C"
