// C shim over the reference's own CPU operators (namespace axono::ops::cpu),
// linked against the reference's sources compiled where they lie (see
// oracle/Makefile).  TEST INFRASTRUCTURE ONLY: it exists to pin the C
// restatement in axono_oracle.c and to time the reference's CPU path; no
// product code loads it.
//
// Buffers are wrapped with Tensor::FromBorrowed (src/core/tensor.cpp:138-144),
// so the reference reads and writes the caller's memory in place: its ops call
// result.Resize(shape), which keeps the storage when the element count is
// unchanged (src/core/tensor.cpp:245-255).
#include <chrono>
#include <cstddef>
#include <cstdint>

#include "axono/core/half.h"
#include "axono/core/tensor.h"
#include "axono/core/types.h"
#include "axono/ops/cpu/fused.h"
#include "axono/ops/cpu/llm.h"
#include "axono/ops/cpu/sequence.h"

namespace {
using axono::core::Context;
using axono::core::DataType;
using axono::core::Shape;
using axono::core::Status;
using axono::core::Tensor;

Tensor Wrap(DataType dt, const Shape &shape, const void *p) {
  return Tensor::FromBorrowed(dt, shape, p);
}
int Code(Status s) { return static_cast<int>(s); }
}  // namespace

extern "C" {

int ref_sdpa_f32(const float *q, const float *k, const float *v, float *out,
                 size_t sq, size_t hq, size_t hkv, size_t d, size_t skv,
                 int is_causal) {
  Context ctx;
  Tensor tq = Wrap(DataType::FLOAT32, {sq, hq, d}, q);
  Tensor tk = Wrap(DataType::FLOAT32, {skv, hkv, d}, k);
  Tensor tv = Wrap(DataType::FLOAT32, {skv, hkv, d}, v);
  Tensor to = Wrap(DataType::FLOAT32, {sq, hq, d}, out);
  return Code(axono::ops::cpu::ScaledDotProductAttention(ctx, tq, tk, tv,
                                                         is_causal != 0, to));
}

// Calls the op `iters` times on the same wrapped buffers and writes each call's
// wall time in milliseconds to ms_out; wrapping stays outside the timed region.
int ref_sdpa_f32_timed(const float *q, const float *k, const float *v,
                       float *out, size_t sq, size_t hq, size_t hkv, size_t d,
                       size_t skv, int iters, double *ms_out) {
  Context ctx;
  Tensor tq = Wrap(DataType::FLOAT32, {sq, hq, d}, q);
  Tensor tk = Wrap(DataType::FLOAT32, {skv, hkv, d}, k);
  Tensor tv = Wrap(DataType::FLOAT32, {skv, hkv, d}, v);
  Tensor to = Wrap(DataType::FLOAT32, {sq, hq, d}, out);
  for (int i = 0; i < iters; ++i) {
    auto t0 = std::chrono::steady_clock::now();
    Status st =
        axono::ops::cpu::ScaledDotProductAttention(ctx, tq, tk, tv, false, to);
    auto t1 = std::chrono::steady_clock::now();
    if (st != Status::OK) return Code(st);
    ms_out[i] = std::chrono::duration<double, std::milli>(t1 - t0).count();
  }
  return 0;
}

// A prepared call: the four tensors wrapped once, so repeated runs pay only for the op itself
// (FromBorrowed allocates and zero-fills a same-sized buffer before it adopts the caller's
// pointer, src/core/tensor.cpp:138-144, which would otherwise dominate a timed call).
struct SdpaCall {
  Tensor q, k, v, out;
};

void *ref_sdpa_prepare(const float *q, const float *k, const float *v, float *out, size_t sq,
                       size_t hq, size_t hkv, size_t d, size_t skv) {
  return new SdpaCall{Wrap(DataType::FLOAT32, {sq, hq, d}, q), Wrap(DataType::FLOAT32, {skv, hkv, d}, k),
                      Wrap(DataType::FLOAT32, {skv, hkv, d}, v), Wrap(DataType::FLOAT32, {sq, hq, d}, out)};
}

int ref_sdpa_run(void *call) {
  SdpaCall *c = static_cast<SdpaCall *>(call);
  Context ctx;
  return Code(axono::ops::cpu::ScaledDotProductAttention(ctx, c->q, c->k, c->v, false, c->out));
}

void ref_sdpa_release(void *call) { delete static_cast<SdpaCall *>(call); }

int ref_rope_f32(const float *x, const int64_t *pos, float theta, float *out,
                 size_t rows, size_t heads, size_t dim) {
  Context ctx;
  Tensor tx = Wrap(DataType::FLOAT32, {rows, heads, dim}, x);
  Tensor tp = Wrap(DataType::INT64, {rows}, pos);
  Tensor to = Wrap(DataType::FLOAT32, {rows, heads, dim}, out);
  return Code(axono::ops::cpu::Rope(ctx, tx, tp, theta, to));
}

int ref_rope_with_cos_sin_f32(const float *x, const float *c, const float *s,
                              float *out, size_t rows, size_t heads,
                              size_t dim) {
  Context ctx;
  Tensor tx = Wrap(DataType::FLOAT32, {rows, heads, dim}, x);
  Tensor tc = Wrap(DataType::FLOAT32, {rows, dim}, c);
  Tensor ts = Wrap(DataType::FLOAT32, {rows, dim}, s);
  Tensor to = Wrap(DataType::FLOAT32, {rows, heads, dim}, out);
  return Code(axono::ops::cpu::RopeWithCosSin(ctx, tx, tc, ts, to));
}

int ref_mrope_cos_sin_f32(const int64_t *pos, const float *inv_freq, int h_sec,
                          int w_sec, float *c, float *s, size_t rows,
                          size_t half) {
  Context ctx;
  Tensor tp = Wrap(DataType::INT64, {3, rows}, pos);
  Tensor tf = Wrap(DataType::FLOAT32, {half}, inv_freq);
  Tensor tc = Wrap(DataType::FLOAT32, {rows, 2 * half}, c);
  Tensor ts = Wrap(DataType::FLOAT32, {rows, 2 * half}, s);
  return Code(axono::ops::cpu::MropeCosSin(ctx, tp, tf, h_sec, w_sec, tc, ts));
}

int ref_rope_thd_f32(const float *x, const int64_t *pos, const float *inv_freq,
                     int t_sec, int h_sec, int w_sec, float *out, size_t rows,
                     size_t heads, size_t dim) {
  Context ctx;
  Tensor tx = Wrap(DataType::FLOAT32, {rows, heads, dim}, x);
  Tensor tp = Wrap(DataType::INT64, {3, rows}, pos);
  Tensor tf = Wrap(DataType::FLOAT32, {dim / 2}, inv_freq);
  Tensor to = Wrap(DataType::FLOAT32, {rows, heads, dim}, out);
  return Code(
      axono::ops::cpu::RopeThd(ctx, tx, tp, tf, t_sec, h_sec, w_sec, to));
}

// Concat along axis 0 of two (rows, inner) byte matrices, as
// DynamicKVCache.update does; dtype INT8 makes it a byte copy.
int ref_concat_axis0_bytes(const void *a, const void *b, void *out,
                           size_t a_rows, size_t b_rows, size_t row_bytes) {
  Context ctx;
  Tensor ta = Wrap(DataType::INT8, {a_rows, row_bytes}, a);
  Tensor tb = Wrap(DataType::INT8, {b_rows, row_bytes}, b);
  Tensor to = Wrap(DataType::INT8, {a_rows + b_rows, row_bytes}, out);
  return Code(axono::ops::cpu::Concat(ctx, ta, tb, 0, to));
}

int ref_silu_mul_f32(const float *g, const float *u, float *y, size_t n) {
  Context ctx;
  Tensor tg = Wrap(DataType::FLOAT32, {n}, g);
  Tensor tu = Wrap(DataType::FLOAT32, {n}, u);
  Tensor ty = Wrap(DataType::FLOAT32, {n}, y);
  return Code(axono::ops::cpu::SiluMul(ctx, tg, tu, ty));
}

int ref_add_rms_norm_f32(const float *x, const float *res, const float *w,
                         float eps, float *y, float *out, size_t rows,
                         size_t hidden) {
  Context ctx;
  Tensor tx = Wrap(DataType::FLOAT32, {rows, hidden}, x);
  Tensor tr = Wrap(DataType::FLOAT32, {rows, hidden}, res);
  Tensor tw = Wrap(DataType::FLOAT32, {hidden}, w);
  Tensor ty = Wrap(DataType::FLOAT32, {rows, hidden}, y);
  Tensor to = Wrap(DataType::FLOAT32, {rows, hidden}, out);
  return Code(axono::ops::cpu::AddRmsNorm(ctx, tx, tr, tw, eps, ty, to));
}

int ref_rms_norm_f32(const float *x, const float *w, float eps, float *out,
                     size_t rows, size_t cols) {
  Context ctx;
  Tensor tx = Wrap(DataType::FLOAT32, {rows, cols}, x);
  Tensor tw = Wrap(DataType::FLOAT32, {cols}, w);
  Tensor to = Wrap(DataType::FLOAT32, {rows, cols}, out);
  return Code(axono::ops::cpu::RmsNorm(ctx, tx, tw, eps, to));
}

int ref_embedding_f32(const int64_t *ids, const float *table, float *out, size_t n, size_t vocab,
                      size_t hidden) {
  Context ctx;
  Tensor ti = Wrap(DataType::INT64, {n}, ids);
  Tensor tt = Wrap(DataType::FLOAT32, {vocab, hidden}, table);
  Tensor to = Wrap(DataType::FLOAT32, {n, hidden}, out);
  return Code(axono::ops::cpu::Embedding(ctx, ti, tt, to));
}

int ref_argmax_last_dim_f32(const float *x, int64_t *out, size_t rows, size_t cols) {
  Context ctx;
  Tensor tx = Wrap(DataType::FLOAT32, {rows, cols}, x);
  Tensor to = Wrap(DataType::INT64, {rows}, out);
  return Code(axono::ops::cpu::ArgmaxLastDim(ctx, tx, to));
}

void ref_half_to_float(const uint16_t *h, float *out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = axono::core::detail::Half2Float(h[i]);
}

void ref_float_to_half(const float *x, uint16_t *out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = axono::core::detail::Float2Half(x[i]);
}

}  // extern "C"
