#include "axono_ops.h"

#include <algorithm>
#include <initializer_list>

#include "axono_b200.h"

namespace axono {
namespace ops {
namespace cuda {
namespace {

using core::DataType;
using core::Shape;

int Dt(DataType t) { return static_cast<int>(t); }        // same enum values as the C ABI
Status St(int s) { return static_cast<Status>(s); }       // same enum values as the C ABI
void *Stream() { return core::cuda::CurrentStream(); }
bool Float(DataType t) { return t == DataType::FLOAT32 || t == DataType::FLOAT16; }
bool Cuda(const Tensor &t) { return t.is_cuda(); }

// Every operand in device memory of one GPU: a host pointer (or another GPU's) handed to a kernel is a
// fault that takes the context with it, so this is checked before anything is resized or launched.
// Null operands (optional arguments) are skipped.
bool OneDevice(std::initializer_list<const Tensor *> ts) {
  int dev = -2;
  for (const Tensor *t : ts) {
    if (!t) continue;
    if (!t->is_cuda()) return false;
    if (dev == -2) dev = t->device_index();
    else if (t->device_index() != dev) return false;
  }
  return true;
}

// Scratch comes from the caching pool, like the reference's three workspace tensors
// (src/ops/cuda/gqa.cu:166-168); after the first call of a shape it is a pool hit.
Tensor Scratch(size_t bytes, const std::string &device) {
  return Tensor::Uninitialized(DataType::INT8, {std::max<size_t>(bytes, 16)}, device);
}

}  // namespace

Status GqaDecodeAttention(const Context &, const Tensor &q, const Tensor &k, const Tensor &v, Tensor &result) {
  if (!OneDevice({&q, &k, &v})) return Status::DEVICE_MISMATCH;
  if (q.ndim() != 3 || k.ndim() != 3 || v.ndim() != 3 || !Float(q.dtype())) return Status::UNSUPPORTED_TYPE;
  if (k.dtype() != q.dtype() || v.dtype() != q.dtype()) return Status::UNSUPPORTED_TYPE;
  if (!Cuda(q) || !Cuda(k) || !Cuda(v)) return Status::DEVICE_MISMATCH;
  const size_t sq = q.shape()[0], hq = q.shape()[1], d = q.shape()[2];
  const size_t skv = k.shape()[0], hkv = k.shape()[1];
  if (sq != 1) return Status::INVALID_ARGUMENT;
  if (k.shape()[2] != d || v.shape()[0] != skv || v.shape()[1] != hkv || v.shape()[2] != d || hkv == 0 || hq % hkv != 0)
    return Status::SHAPE_MISMATCH;
  Status st = result.Resize({1, hq, d});
  if (st != Status::OK) return st;
  const size_t ws = axb200_gqa_workspace_bytes(1, (int)hq, (int)hkv, (int)d, (int64_t)skv, Dt(q.dtype()));
  Tensor scratch = Scratch(ws, q.device());
  return St(axb200_gqa_decode(q.data(), k.data(), v.data(), result.data(), (int)hq, (int)hkv, (int)d, (int64_t)skv,
                              Dt(q.dtype()), scratch.data(), scratch.num_bytes(), Stream()));
}

Status ScaledDotProductAttention(const Context &, const Tensor &q, const Tensor &k, const Tensor &v, bool is_causal,
                                 Tensor &result) {
  if (!OneDevice({&q, &k, &v})) return Status::DEVICE_MISMATCH;
  if (q.ndim() != 3 || k.ndim() != 3 || v.ndim() != 3) return Status::INVALID_ARGUMENT;
  if (!Float(q.dtype()) || k.dtype() != q.dtype() || v.dtype() != q.dtype()) return Status::UNSUPPORTED_TYPE;
  const size_t sq = q.shape()[0], hq = q.shape()[1], d = q.shape()[2];
  const size_t skv = k.shape()[0], hkv = k.shape()[1];
  if (k.shape()[2] != d || v.shape()[0] != skv || v.shape()[1] != hkv || v.shape()[2] != d) return Status::SHAPE_MISMATCH;
  if (hkv == 0 || hq % hkv != 0) return Status::SHAPE_MISMATCH;
  Status st = result.Resize({sq, hq, d});
  if (st != Status::OK) return st;
  const size_t ws = axb200_sdpa_workspace_bytes((int)sq, (int)hq, (int)hkv, (int)d, (int64_t)skv, Dt(q.dtype()));
  Tensor scratch = Scratch(ws, q.device());
  return St(axb200_sdpa(q.data(), k.data(), v.data(), result.data(), (int)sq, (int)hq, (int)hkv, (int)d, (int64_t)skv,
                        is_causal ? 1 : 0, Dt(q.dtype()), scratch.data(), scratch.num_bytes(), Stream()));
}

Status SiluMul(const Context &, const Tensor &gate, const Tensor &up, Tensor &result) {
  if (!OneDevice({&gate, &up})) return Status::DEVICE_MISMATCH;
  if (!Float(gate.dtype()) || gate.dtype() != up.dtype() || gate.shape() != up.shape()) return Status::SHAPE_MISMATCH;
  Status st = result.Resize(gate.shape());
  if (st != Status::OK) return st;
  return St(axb200_silu_mul(gate.data(), up.data(), result.data(), (int64_t)gate.num_elements(), Dt(gate.dtype()), Stream()));
}

Status AddRmsNorm(const Context &, const Tensor &x, const Tensor &residual, const Tensor &weight, float eps, Tensor &y,
                  Tensor &out) {
  if (!OneDevice({&x, &residual, &weight})) return Status::DEVICE_MISMATCH;
  if (!Float(x.dtype()) || x.shape() != residual.shape() || residual.dtype() != x.dtype()) return Status::SHAPE_MISMATCH;
  if (x.ndim() < 1) return Status::INVALID_ARGUMENT;
  const size_t hidden = x.shape().back();
  if (weight.ndim() != 1 || weight.shape()[0] != hidden || weight.dtype() != x.dtype()) return Status::SHAPE_MISMATCH;
  Status st = y.Resize(x.shape());
  if (st != Status::OK) return st;
  st = out.Resize(x.shape());
  if (st != Status::OK) return st;
  return St(axb200_add_rms_norm(x.data(), residual.data(), weight.data(), eps, y.data(), out.data(),
                                (int64_t)(x.num_elements() / hidden), (int)hidden, Dt(x.dtype()), Stream()));
}

Status RmsNorm(const Context &, const Tensor &x, const Tensor &weight, float eps, Tensor &result) {
  if (!OneDevice({&x, weight.num_elements() ? &weight : nullptr})) return Status::DEVICE_MISMATCH;
  if (x.ndim() < 1) return Status::INVALID_ARGUMENT;
  const size_t cols = x.shape().back();
  Status st = result.Resize(x.shape());
  if (st != Status::OK) return st;
  if (!Float(x.dtype())) return Status::UNSUPPORTED_TYPE;
  if (cols == 0) return Status::INVALID_ARGUMENT;
  const bool has_w = weight.num_elements() != 0;
  if (has_w && (weight.ndim() != 1 || weight.shape()[0] != cols || weight.dtype() != x.dtype())) return Status::SHAPE_MISMATCH;
  return St(axb200_rms_norm(x.data(), has_w ? weight.data() : nullptr, eps, result.data(),
                            (int64_t)(x.num_elements() / cols), (int)cols, Dt(x.dtype()), Stream()));
}

Status Rope(const Context &, const Tensor &x, const Tensor &pos_ids, float theta, Tensor &result) {
  if (!OneDevice({&x, &pos_ids})) return Status::DEVICE_MISMATCH;
  if (x.ndim() != 3 || !Float(x.dtype())) return Status::UNSUPPORTED_TYPE;
  const size_t rows = x.shape()[0], heads = x.shape()[1], dim = x.shape()[2];
  if (dim % 2 != 0) return Status::INVALID_ARGUMENT;
  if (pos_ids.num_elements() != rows || pos_ids.dtype() != DataType::INT64) return Status::UNSUPPORTED_TYPE;
  Status st = result.Resize(x.shape());
  if (st != Status::OK) return st;
  return St(axb200_rope(x.data(), pos_ids.data<int64_t>(), theta, result.data(), (int64_t)rows, (int)heads, (int)dim,
                        Dt(x.dtype()), Stream()));
}

Status RopeThd(const Context &, const Tensor &x, const Tensor &pos, const Tensor &inv_freq, int t_sec, int h_sec,
               int w_sec, Tensor &result) {
  if (!OneDevice({&x, &pos, &inv_freq})) return Status::DEVICE_MISMATCH;
  if (x.ndim() != 3 || !Float(x.dtype())) return Status::UNSUPPORTED_TYPE;
  const size_t rows = x.shape()[0], heads = x.shape()[1], dim = x.shape()[2];
  if (dim % 2 != 0) return Status::INVALID_ARGUMENT;
  if (pos.ndim() != 2 || pos.shape()[0] != 3 || pos.shape()[1] != rows || pos.dtype() != DataType::INT64)
    return Status::SHAPE_MISMATCH;
  if (inv_freq.ndim() != 1 || inv_freq.shape()[0] != dim / 2 || inv_freq.dtype() != DataType::FLOAT32)
    return Status::SHAPE_MISMATCH;
  Status st = result.Resize(x.shape());
  if (st != Status::OK) return st;
  return St(axb200_rope_thd(x.data(), pos.data<int64_t>(), inv_freq.data<float>(), t_sec, h_sec, w_sec, result.data(),
                            (int64_t)rows, (int)heads, (int)dim, Dt(x.dtype()), Stream()));
}

Status RopeWithCosSin(const Context &, const Tensor &x, const Tensor &cos, const Tensor &sin, Tensor &result) {
  if (!OneDevice({&x, &cos, &sin})) return Status::DEVICE_MISMATCH;
  if (x.ndim() != 3 || !Float(x.dtype())) return Status::UNSUPPORTED_TYPE;
  const size_t rows = x.shape()[0], heads = x.shape()[1], dim = x.shape()[2];
  if (dim % 2 != 0) return Status::INVALID_ARGUMENT;
  if (cos.ndim() != 2 || sin.ndim() != 2 || cos.shape()[0] != rows || cos.shape()[1] != dim || sin.shape()[0] != rows ||
      sin.shape()[1] != dim || cos.dtype() != DataType::FLOAT32 || sin.dtype() != DataType::FLOAT32)
    return Status::SHAPE_MISMATCH;
  Status st = result.Resize(x.shape());
  if (st != Status::OK) return st;
  return St(axb200_rope_with_cos_sin(x.data(), cos.data<float>(), sin.data<float>(), result.data(), (int64_t)rows,
                                     (int)heads, (int)dim, Dt(x.dtype()), Stream()));
}

Status MropeCosSin(const Context &, const Tensor &pos, const Tensor &inv_freq, int h_sec, int w_sec, Tensor &cos_out,
                   Tensor &sin_out) {
  if (!OneDevice({&pos, &inv_freq})) return Status::DEVICE_MISMATCH;
  if (pos.ndim() != 2 || pos.shape()[0] != 3 || pos.dtype() != DataType::INT64) return Status::SHAPE_MISMATCH;
  const size_t rows = pos.shape()[1], half = inv_freq.ndim() ? inv_freq.shape()[0] : 0;
  if (half == 0) return Status::INVALID_ARGUMENT;
  Status st = cos_out.Resize({rows, 2 * half});
  if (st != Status::OK) return st;
  st = sin_out.Resize({rows, 2 * half});
  if (st != Status::OK) return st;
  return St(axb200_mrope_cos_sin(pos.data<int64_t>(), inv_freq.data<float>(), h_sec, w_sec, cos_out.data<float>(),
                                 sin_out.data<float>(), (int64_t)rows, (int)half, Stream()));
}

Status Concat(const Context &, const Tensor &a, const Tensor &b, int axis, Tensor &result) {
  if (!OneDevice({&a, &b})) return Status::DEVICE_MISMATCH;
  if (a.ndim() < 1 || a.ndim() != b.ndim() || a.dtype() != b.dtype()) return Status::INVALID_ARGUMENT;
  const size_t nd = a.ndim();
  const size_t ax = axis < 0 ? nd + axis : (size_t)axis;
  if (ax >= nd) return Status::INVALID_ARGUMENT;
  for (size_t i = 0; i < nd; ++i)
    if (i != ax && a.shape()[i] != b.shape()[i]) return Status::SHAPE_MISMATCH;
  Shape shape = a.shape();
  shape[ax] += b.shape()[ax];
  Status st = result.Resize(shape);
  if (st != Status::OK) return st;
  size_t outer = 1;
  for (size_t i = 0; i < ax; ++i) outer *= a.shape()[i];
  const size_t es = core::GetDataTypeSize(a.dtype());
  return St(axb200_concat(a.data(), b.data(), result.data(), (int64_t)outer, a.num_elements() / outer * es,
                          b.num_elements() / outer * es, Stream()));
}

Status Embedding(const Context &, const Tensor &ids, const Tensor &table, Tensor &result) {
  if (!OneDevice({&ids, &table})) return Status::DEVICE_MISMATCH;
  if (ids.ndim() < 1 || table.ndim() != 2) return Status::INVALID_ARGUMENT;
  if (!Float(table.dtype())) return Status::UNSUPPORTED_TYPE;
  if (ids.dtype() != DataType::INT32 && ids.dtype() != DataType::INT64) return Status::UNSUPPORTED_TYPE;
  Shape out_shape = ids.shape();
  out_shape.push_back(table.shape()[1]);
  Status st = result.Resize(out_shape);
  if (st != Status::OK) return st;
  return St(axb200_embedding(ids.data(), Dt(ids.dtype()), table.data(), result.data(), (int64_t)ids.num_elements(),
                             (int64_t)table.shape()[0], (int)table.shape()[1], Dt(table.dtype()), Stream()));
}

Status ArgmaxLastDim(const Context &, const Tensor &x, Tensor &result) {
  if (!OneDevice({&x})) return Status::DEVICE_MISMATCH;
  if (x.ndim() < 1) return Status::INVALID_ARGUMENT;
  const size_t cols = x.shape().back();
  const size_t rows = cols ? x.num_elements() / cols : 0;
  Status st = result.Resize({rows});
  if (st != Status::OK) return st;
  if (result.dtype() != DataType::INT64 || !Float(x.dtype())) return Status::UNSUPPORTED_TYPE;
  return St(axb200_argmax_last_dim(x.data(), result.data<int64_t>(), (int64_t)rows, (int)cols, Dt(x.dtype()), Stream()));
}

Status LinearNoBias(const Context &, const Tensor &x, const Tensor &w, Tensor &result) {
  if (!OneDevice({&x, &w})) return Status::DEVICE_MISMATCH;
  if (x.ndim() != 2 || w.ndim() != 2 || x.shape()[1] != w.shape()[1]) return Status::SHAPE_MISMATCH;
  if (!Float(x.dtype()) || w.dtype() != x.dtype()) return Status::UNSUPPORTED_TYPE;
  if (!Cuda(x) || !Cuda(w)) return Status::DEVICE_MISMATCH;
  Status st = result.Resize({x.shape()[0], w.shape()[0]});
  if (st != Status::OK) return st;
  return St(axb200_linear_nobias(x.data(), w.data(), result.data(), (int64_t)x.shape()[0], (int64_t)w.shape()[0],
                                 (int64_t)x.shape()[1], Dt(x.dtype()), Stream()));
}

Status SiluMulRows(const Context &, const Tensor &gate_up, int n, Tensor &result) {
  if (!OneDevice({&gate_up})) return Status::DEVICE_MISMATCH;
  if (gate_up.ndim() != 2 || n <= 0 || gate_up.shape()[1] != (size_t)(2 * n)) return Status::SHAPE_MISMATCH;
  if (!Float(gate_up.dtype())) return Status::UNSUPPORTED_TYPE;
  Status st = result.Resize({gate_up.shape()[0], (size_t)n});
  if (st != Status::OK) return st;
  return St(axb200_silu_mul_rows(gate_up.data(), (int64_t)gate_up.shape()[1], n, (int64_t)gate_up.shape()[0],
                                 result.data(), Dt(gate_up.dtype()), Stream()));
}

Status QkvNormRopeAppend(const Context &, const Tensor &qkv, int hq, const Tensor *q_norm_w, const Tensor *k_norm_w,
                         float eps, axb200_kv_arena *arena, int layer, const Tensor *pos, const Tensor *inv_freq,
                         float theta, bool rotate, bool mrope, int h_sec, int w_sec, int slot_delta, bool advance,
                         Tensor &q_out) {
  if (!OneDevice({&qkv, q_norm_w, k_norm_w, pos, inv_freq})) return Status::DEVICE_MISMATCH;
  if (!arena || qkv.ndim() != 2 || !Float(qkv.dtype())) return Status::UNSUPPORTED_TYPE;
  int n_layers, num_pages, hkv, page_tokens, d, dtype, max_seqs, max_blocks;
  if (axb200_kv_arena_geometry(arena, &n_layers, &num_pages, &hkv, &page_tokens, &d, &dtype, &max_seqs, &max_blocks) != 0)
    return Status::INVALID_PTR;
  if ((int)qkv.shape()[0] != max_seqs || qkv.shape()[1] != (size_t)((hq + 2 * hkv) * d) || Dt(qkv.dtype()) != dtype ||
      layer < 0 || layer >= n_layers)
    return Status::SHAPE_MISMATCH;
  Status st = q_out.Resize({(size_t)max_seqs, (size_t)hq, (size_t)d});
  if (st != Status::OK) return st;
  return St(axb200_qkv_norm_rope_append(qkv.data(), (int64_t)qkv.shape()[1], q_norm_w ? q_norm_w->data() : nullptr,
                                        k_norm_w ? k_norm_w->data() : nullptr, eps, q_out.data(),
                                        axb200_kv_arena_k_pages(arena, layer), axb200_kv_arena_v_pages(arena, layer),
                                        axb200_kv_arena_block_table(arena), axb200_kv_arena_seq_lens(arena),
                                        pos ? pos->data<int64_t>() : nullptr, inv_freq ? inv_freq->data<float>() : nullptr,
                                        theta, rotate, mrope, h_sec, w_sec, max_seqs, hq, hkv, d, page_tokens, max_blocks,
                                        num_pages, dtype, slot_delta, advance, Stream()));
}

Status KvAppendRope(const Context &, Tensor *q, const Tensor &k_new, const Tensor &v_new, axb200_kv_arena *arena,
                    int layer, const Tensor *pos, const Tensor *inv_freq, float theta, bool rotate, bool mrope, int h_sec,
                    int w_sec, int slot_delta, bool advance) {
  if (!OneDevice({q, &k_new, &v_new, pos, inv_freq})) return Status::DEVICE_MISMATCH;
  if (!arena || k_new.ndim() != 3 || v_new.shape() != k_new.shape() || !Float(k_new.dtype())) return Status::SHAPE_MISMATCH;
  int n_layers, num_pages, hkv, page_tokens, d, dtype, max_seqs, max_blocks;
  if (axb200_kv_arena_geometry(arena, &n_layers, &num_pages, &hkv, &page_tokens, &d, &dtype, &max_seqs, &max_blocks) != 0)
    return Status::INVALID_PTR;
  if ((int)k_new.shape()[0] != max_seqs || (int)k_new.shape()[1] != hkv || (int)k_new.shape()[2] != d ||
      Dt(k_new.dtype()) != dtype || layer < 0 || layer >= n_layers)
    return Status::SHAPE_MISMATCH;
  const int hq = q ? (int)q->shape()[1] : 0;
  return St(axb200_kv_append_rope(q ? q->data() : nullptr, k_new.data(), v_new.data(), axb200_kv_arena_k_pages(arena, layer),
                                  axb200_kv_arena_v_pages(arena, layer), axb200_kv_arena_block_table(arena),
                                  axb200_kv_arena_seq_lens(arena), pos ? pos->data<int64_t>() : nullptr,
                                  inv_freq ? inv_freq->data<float>() : nullptr, theta, rotate, mrope, h_sec, w_sec,
                                  max_seqs, hq, hkv, d, page_tokens, max_blocks, num_pages, dtype, slot_delta, advance,
                                  Stream()));
}

Status GqaDecodeAttentionPaged(const Context &, const Tensor &q, axb200_kv_arena *arena, int layer, int64_t max_seq_len,
                               Tensor &result) {
  if (!OneDevice({&q})) return Status::DEVICE_MISMATCH;
  if (!arena || q.ndim() != 3 || !Float(q.dtype())) return Status::UNSUPPORTED_TYPE;
  int n_layers, num_pages, hkv, page_tokens, d, dtype, max_seqs, max_blocks;
  if (axb200_kv_arena_geometry(arena, &n_layers, &num_pages, &hkv, &page_tokens, &d, &dtype, &max_seqs, &max_blocks) != 0)
    return Status::INVALID_PTR;
  const int hq = (int)q.shape()[1];
  if ((int)q.shape()[0] != max_seqs || (int)q.shape()[2] != d || Dt(q.dtype()) != dtype || layer < 0 || layer >= n_layers)
    return Status::SHAPE_MISMATCH;
  Status st = result.Resize(q.shape());
  if (st != Status::OK) return st;
  const size_t ws = axb200_gqa_workspace_bytes(max_seqs, hq, hkv, d, max_seq_len, dtype);
  Tensor scratch = Scratch(ws, q.device());
  return St(axb200_gqa_decode_paged(q.data(), result.data(), axb200_kv_arena_k_pages(arena, layer),
                                    axb200_kv_arena_v_pages(arena, layer), axb200_kv_arena_block_table(arena),
                                    axb200_kv_arena_seq_lens(arena), max_seqs, hq, hkv, d, page_tokens, max_blocks,
                                    num_pages, max_seq_len, dtype, scratch.data(), scratch.num_bytes(), Stream()));
}

Status DecodeStepPaged(const Context &, const Tensor &q, const Tensor &k_new, const Tensor &v_new, axb200_kv_arena *arena,
                       int layer, const Tensor *pos, const Tensor *inv_freq, float theta, bool rotate, bool mrope, int h_sec,
                       int w_sec, int64_t max_seq_len, Tensor &result) {
  if (!OneDevice({&q, &k_new, &v_new, pos, inv_freq})) return Status::DEVICE_MISMATCH;
  if (!arena || q.ndim() != 3 || k_new.ndim() != 3 || v_new.shape() != k_new.shape() || !Float(q.dtype()))
    return Status::SHAPE_MISMATCH;
  int n_layers, num_pages, hkv, page_tokens, d, dtype, max_seqs, max_blocks;
  if (axb200_kv_arena_geometry(arena, &n_layers, &num_pages, &hkv, &page_tokens, &d, &dtype, &max_seqs, &max_blocks) != 0)
    return Status::INVALID_PTR;
  const int hq = (int)q.shape()[1];
  if ((int)q.shape()[0] != max_seqs || (int)q.shape()[2] != d || Dt(q.dtype()) != dtype || (int)k_new.shape()[0] != max_seqs ||
      (int)k_new.shape()[1] != hkv || (int)k_new.shape()[2] != d || k_new.dtype() != q.dtype() || layer < 0 || layer >= n_layers)
    return Status::SHAPE_MISMATCH;
  Status st = result.Resize(q.shape());
  if (st != Status::OK) return st;
  const size_t ws = axb200_decode_step_workspace_bytes(max_seqs, hq, hkv, d, max_seq_len, dtype);
  Tensor scratch = Scratch(ws, q.device());
  return St(axb200_decode_step_paged(q.data(), k_new.data(), v_new.data(), result.data(), axb200_kv_arena_k_pages(arena, layer),
                                     axb200_kv_arena_v_pages(arena, layer), axb200_kv_arena_block_table(arena),
                                     axb200_kv_arena_seq_lens(arena), pos ? pos->data<int64_t>() : nullptr,
                                     inv_freq ? inv_freq->data<float>() : nullptr, theta, rotate, mrope, h_sec, w_sec, max_seqs,
                                     hq, hkv, d, page_tokens, max_blocks, num_pages, max_seq_len, dtype, scratch.data(),
                                     scratch.num_bytes(), Stream()));
}

}  // namespace cuda
}  // namespace ops
}  // namespace axono
