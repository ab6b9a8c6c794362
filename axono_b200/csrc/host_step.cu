// One decode step for callers whose activations live in host memory - the situation of the
// reference's binding, where every step's inputs arrive as host arrays and the result is read back
// (axono/python/examples/vlm/qwen3vl/model.py:738-761: ids/positions are written into device tensors
// with copy_from_numpy, the logits come back with to_numpy).  The call stages q / k_new / v_new
// from (pinned) host buffers, runs RoPE + append and the paged decode attention, copies the
// attention output back and waits for it: one call through the C ABI instead of six.
//
// When all four host buffers are page-locked memory the GPU can address under the same pointer
// (cudaHostAlloc, or registered memory where the device reports that property), no copy engine is
// involved at all: the append kernel reads q / k_new / v_new from host memory itself (a few KB per
// sequence, each byte read once; the rotated q goes to the device staging buffer, where the attention
// kernel reads it many times), and the attention kernel's final rows are stored straight into the host
// output buffer; where the one-launch step applies (fp16, head_dim 64 or 128) there is no append kernel
// either.  Each copy saved is a separate DMA operation with its own few microseconds of latency
// on a step that is itself tens to hundreds of microseconds.  Pageable memory takes the copying path.
#include "common.cuh"

namespace {
// True when a kernel may dereference `p`: page-locked host memory mapped at the same address.
bool device_addressable_host(const void *p) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeHost && attr.devicePointer == p;
}
}  // namespace

extern "C" int axb200_decode_step_host(
    const void *q_host, const void *k_new_host, const void *v_new_host, void *out_host, void *q_dev,
    void *k_new_dev, void *v_new_dev, void *out_dev, void *k_pages, void *v_pages,
    const int32_t *block_table, int32_t *seq_lens, const int64_t *pos, const float *inv_freq,
    float theta, int rotate, int mrope, int h_sec, int w_sec, int batch, int hq, int hkv, int d,
    int page_tokens, int max_blocks, int num_pages, int64_t max_seq_len, int dtype, void *workspace,
    size_t workspace_bytes, void *stream) {
  const size_t es = axb::dtype_size(dtype);
  if (es == 0) return AXB200_UNSUPPORTED_TYPE;
  if (!q_host || !k_new_host || !v_new_host || !out_host || !q_dev || !k_new_dev || !v_new_dev ||
      !out_dev)
    return AXB200_INVALID_PTR;
  if (batch <= 0 || hq <= 0 || hkv <= 0 || d <= 0) return AXB200_INVALID_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t qb = (size_t)batch * hq * d * es, kb = (size_t)batch * hkv * d * es;
  if (rotate && device_addressable_host(q_host) && device_addressable_host(k_new_host) &&
      device_addressable_host(v_new_host) && device_addressable_host(out_host)) {
    // one launch when that form applies: the attention kernel reads q, k_new, v_new from host memory itself
    int rc = axb::decode_step_try_fused(q_host, k_new_host, v_new_host, out_host, k_pages, v_pages, block_table,
                                        seq_lens, pos, inv_freq, theta, rotate, mrope, h_sec, w_sec, batch, hq, hkv, d,
                                        page_tokens, max_blocks, num_pages, max_seq_len, dtype, workspace,
                                        workspace_bytes, stream);
    if (rc == AXB200_OK) return cudaStreamSynchronize(st) == cudaSuccess ? AXB200_OK : AXB200_DEVICE_ERROR;
    if (rc != axb::kStepNotFused) return rc;
    rc = axb::kv_append_rope_from(q_dev, q_host, k_new_host, v_new_host, k_pages, v_pages, block_table, seq_lens,
                                      pos, inv_freq, theta, rotate, mrope, h_sec, w_sec, batch, hq, hkv, d,
                                      page_tokens, max_blocks, num_pages, dtype, 0, 1, stream);
    if (rc != AXB200_OK) return rc;
    rc = axb200_gqa_decode_paged(q_dev, out_host, k_pages, v_pages, block_table, seq_lens, batch, hq, hkv, d,
                                 page_tokens, max_blocks, num_pages, max_seq_len, dtype, workspace,
                                 workspace_bytes, stream);
    if (rc != AXB200_OK) return rc;
    return cudaStreamSynchronize(st) == cudaSuccess ? AXB200_OK : AXB200_DEVICE_ERROR;
  }
  if (cudaMemcpyAsync(q_dev, q_host, qb, cudaMemcpyHostToDevice, st) != cudaSuccess ||
      cudaMemcpyAsync(k_new_dev, k_new_host, kb, cudaMemcpyHostToDevice, st) != cudaSuccess ||
      cudaMemcpyAsync(v_new_dev, v_new_host, kb, cudaMemcpyHostToDevice, st) != cudaSuccess)
    return AXB200_DEVICE_ERROR;
  int rc = axb200_kv_append_rope(q_dev, k_new_dev, v_new_dev, k_pages, v_pages, block_table,
                                 seq_lens, pos, inv_freq, theta, rotate, mrope, h_sec, w_sec, batch,
                                 hq, hkv, d, page_tokens, max_blocks, num_pages, dtype, 0, 1, stream);
  if (rc != AXB200_OK) return rc;
  rc = axb200_gqa_decode_paged(q_dev, out_dev, k_pages, v_pages, block_table, seq_lens, batch, hq,
                               hkv, d, page_tokens, max_blocks, num_pages, max_seq_len, dtype,
                               workspace, workspace_bytes, stream);
  if (rc != AXB200_OK) return rc;
  if (cudaMemcpyAsync(out_host, out_dev, qb, cudaMemcpyDeviceToHost, st) != cudaSuccess)
    return AXB200_DEVICE_ERROR;
  return cudaStreamSynchronize(st) == cudaSuccess ? AXB200_OK : AXB200_DEVICE_ERROR;
}
