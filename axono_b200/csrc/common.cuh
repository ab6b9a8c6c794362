// Shared device/host helpers for the sm_100a decode-path kernels: status and dtype codes,
// the device error word, and thin inline-PTX wrappers (mbarrier, TMA tensor copies,
// ldmatrix, mma.sync).
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "axono_b200.h"

namespace axb {

// Set by kernels instead of trapping; read and cleared by axb200_last_error().  Each
// translation unit has its own copy (no relocatable device code is needed) and registers a
// reader for it at load time.
static __device__ unsigned int g_error_word = 0;

using ErrorReader = unsigned int (*)();
void register_error_reader(ErrorReader fn);  // defined once, beside axb200_last_error()

static unsigned int read_clear_error_word() {
  unsigned int word = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&word, g_error_word, sizeof(word)) != cudaSuccess) return 0x80000000u;
  if (word) cudaMemcpyToSymbol(g_error_word, &zero, sizeof(zero));
  return word;
}

namespace {
struct ErrorReaderRegistration {
  ErrorReaderRegistration() { register_error_reader(&read_clear_error_word); }
};
static ErrorReaderRegistration g_error_reader_registration;
}  // namespace

// axb200_kv_append_rope with q read from q_src (null: in place); defined in rope_append.cu.
int kv_append_rope_from(void *q, const void *q_src, const void *k_new, const void *v_new, void *k_pages,
                        void *v_pages, const int32_t *block_table, int32_t *seq_lens, const int64_t *pos,
                        const float *inv_freq, float theta, int rotate, int mrope, int h_sec, int w_sec,
                        int batch, int hq, int hkv, int d, int page_tokens, int max_blocks, int num_pages,
                        int dtype, int slot_delta, int advance, void *stream);

// The decode step as one launch when that form applies, else kStepNotFused with nothing launched;
// defined in gqa_decode.cu.
constexpr int kStepNotFused = -1000;
int decode_step_try_fused(const void *q, const void *k_new, const void *v_new, void *out, void *k_pages,
                          void *v_pages, const int32_t *block_table, int32_t *seq_lens, const int64_t *pos,
                          const float *inv_freq, float theta, int rotate, int mrope, int h_sec, int w_sec,
                          int batch, int hq, int hkv, int d, int page_tokens, int max_blocks, int num_pages,
                          int64_t max_seq_len, int dtype, void *workspace, size_t workspace_bytes,
                          void *stream);

inline size_t dtype_size(int dtype) {
  switch (dtype) {
    case AXB200_FLOAT16: return 2;
    case AXB200_FLOAT32: return 4;
    default: return 0;
  }
}

inline int launch_status() {
  return cudaGetLastError() == cudaSuccess ? AXB200_OK : AXB200_DEVICE_ERROR;
}

// ---- bounded waiting ---------------------------------------------------------------------
// Every spin in these kernels is limited: a waiter that has polled for the wait limit of wall time
// records AXB200_ERR_WAIT_TIMEOUT, raises the CTA's abort flag and the kernel winds down
// instead of hanging the GPU.  The limit is a host-side setting (axb200_set_wait_limit_ns, 2 s by
// default) that the launchers pass to their kernels by value.
constexpr unsigned long long kWaitNanos = 2000000000ull;  // 2 s, the default limit
unsigned long long wait_limit_ns();                        // defined beside axb200_set_wait_limit_ns

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Waits for the phase with the given parity to complete, or until the time limit or the
// CTA's abort flag ends the wait.  Returns false when it gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity,
                                                  volatile int *abort_flag,
                                                  unsigned long long limit_ns = kWaitNanos) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > limit_ns) break;
    }
  }
  *abort_flag = 1;
  atomicOr(&g_error_word, AXB200_ERR_WAIT_TIMEOUT);
  return false;
}

// ---- programmatic dependent launch ------------------------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may be scheduled while the
// kernel before it in the stream is still running; grid_dependency_wait() blocks until that kernel has
// completed and its writes are visible, so everything above the call (barrier set-up, descriptor
// prefetch) overlaps the predecessor's tail and the launch latency.  Without the attribute the call
// returns at once.  grid_dependency_launch() in the predecessor lets the dependents be scheduled early.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- rotary position embedding: the arithmetic every kernel that rotates shares ------------------
// Pair (a, b) = (x[i], x[i + half]) turned by the angle whose cosine and sine are (c, s).  The
// roundings are spelled out (one product rounded, then one fused multiply-add) so that the append
// kernel, the prefill write, the standalone rope kernels and the decode step that rotates inside the
// attention kernel produce the same bits whatever the compiler would contract on its own.
__device__ __forceinline__ float rope_lo(float a, float b, float c, float s) { return __fmaf_rn(a, c, -__fmul_rn(b, s)); }
__device__ __forceinline__ float rope_hi(float a, float b, float c, float s) { return __fmaf_rn(b, c, __fmul_rn(a, s)); }

// Position of rotary pair i under M-RoPE: the stride-3 rule (src/ops/cpu/sequence.cpp:222-227).
__device__ __forceinline__ float mrope_pair_position(int i, float pt, float ph, float pw, int h_lim, int w_lim) {
  if (i % 3 == 1 && i < h_lim) return ph;
  if (i % 3 == 2 && i < w_lim) return pw;
  return pt;
}

// theta^(-2i/dim) for i < dim/2 with the host C library's powf (src/ops/cpu/sequence.cpp:83-84);
// defined in rope_append.cu.
void rope_inv_freq_host(float theta, int dim, float *out);

// ---- TMA (cp.async.bulk.tensor), 4-D tiled load, completion on an mbarrier -----------------
// The innermost coordinate c0 times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *map, uint64_t *bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor-core fragments ------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3,
                                            uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                                  uint32_t &r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&h);
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace axb
