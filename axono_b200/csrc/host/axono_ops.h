// The reference's CUDA operator entry points for the decode path, with their signatures
// (include/axono/ops/cuda/{gqa,fused,sequence,llm}.h), now thin adapters from Tensor to the C ABI of
// axono_b200.h.  FLOAT16 tensors are accepted wherever the reference took FLOAT32 only.
#pragma once

#include "axono_core.h"

struct axb200_kv_arena;

namespace axono {
namespace ops {
namespace cuda {

using core::Context;
using core::Status;
using core::Tensor;

Status GqaDecodeAttention(const Context &ctx, const Tensor &q, const Tensor &k, const Tensor &v, Tensor &result);
Status ScaledDotProductAttention(const Context &ctx, const Tensor &q, const Tensor &k, const Tensor &v,
                                 bool is_causal, Tensor &result);
Status SiluMul(const Context &ctx, const Tensor &gate, const Tensor &up, Tensor &result);
Status AddRmsNorm(const Context &ctx, const Tensor &x, const Tensor &residual, const Tensor &weight, float eps,
                  Tensor &y, Tensor &out);
Status RmsNorm(const Context &ctx, const Tensor &x, const Tensor &weight, float eps, Tensor &result);
Status Rope(const Context &ctx, const Tensor &x, const Tensor &pos_ids, float theta, Tensor &result);
Status RopeThd(const Context &ctx, const Tensor &x, const Tensor &pos, const Tensor &inv_freq, int t_sec, int h_sec,
               int w_sec, Tensor &result);
Status RopeWithCosSin(const Context &ctx, const Tensor &x, const Tensor &cos, const Tensor &sin, Tensor &result);
Status MropeCosSin(const Context &ctx, const Tensor &pos, const Tensor &inv_freq, int h_sec, int w_sec,
                   Tensor &cos_out, Tensor &sin_out);
Status Concat(const Context &ctx, const Tensor &a, const Tensor &b, int axis, Tensor &result);
Status Embedding(const Context &ctx, const Tensor &ids, const Tensor &table, Tensor &result);
Status ArgmaxLastDim(const Context &ctx, const Tensor &x, Tensor &result);

// x (rows, in) . w (out, in)^T -> (rows, out): the projection GEMM of the text tower, a plain cuBLASLt
// call as in the reference (src/ops/cuda/linear.cu:105-203, Python linear_nobias); FLOAT16 with fp32
// accumulation, or FLOAT32.  A library GEMM, outside the rewritten path.
Status LinearNoBias(const Context &ctx, const Tensor &x, const Tensor &w, Tensor &result);

// Glue kernels of the tower (new): silu_mul on the halves of a fused gate|up projection, and per-head
// norm + rope + append straight from the QKV projection's output.
Status SiluMulRows(const Context &ctx, const Tensor &gate_up, int n, Tensor &result);
Status QkvNormRopeAppend(const Context &ctx, const Tensor &qkv, int hq, const Tensor *q_norm_w, const Tensor *k_norm_w,
                         float eps, axb200_kv_arena *arena, int layer, const Tensor *pos, const Tensor *inv_freq,
                         float theta, bool rotate, bool mrope, int h_sec, int w_sec, int slot_delta, bool advance,
                         Tensor &q_out);

// Paged cache (new operators; the cache lives in a KV arena).
// kv_append_rope followed by gqa_decode_attention_paged as one operator (one launch where the library's
// one-launch step applies): q is read, not rotated in place; the arena's lengths grow by one.
Status DecodeStepPaged(const Context &ctx, const Tensor &q, const Tensor &k_new, const Tensor &v_new, axb200_kv_arena *arena,
                       int layer, const Tensor *pos, const Tensor *inv_freq, float theta, bool rotate, bool mrope, int h_sec,
                       int w_sec, int64_t max_seq_len, Tensor &result);
Status KvAppendRope(const Context &ctx, Tensor *q, const Tensor &k_new, const Tensor &v_new, axb200_kv_arena *arena,
                    int layer, const Tensor *pos, const Tensor *inv_freq, float theta, bool rotate, bool mrope,
                    int h_sec, int w_sec, int slot_delta, bool advance);
Status GqaDecodeAttentionPaged(const Context &ctx, const Tensor &q, axb200_kv_arena *arena, int layer,
                               int64_t max_seq_len, Tensor &result);

}  // namespace cuda
}  // namespace ops
}  // namespace axono
