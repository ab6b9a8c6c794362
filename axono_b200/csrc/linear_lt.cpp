// Projection GEMM of the tower: out (rows, out_features) = x (rows, in_features) . w (out_features,
// in_features)^T, one cuBLASLt call.  A library GEMM - the reference's own choice for its projections
// (src/ops/cuda/linear.cu:105-203) and outside the rewritten path; it is here so that the native
// runtime and the torch-tensor mirror share one tuned call: on the first use of a shape up to eight
// heuristic candidates are timed on the real operands and the fastest is kept (at a few dozen rows
// the heuristic's first choice is often not it).
#include <cublasLt.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <tuple>

#include "axono_b200.h"

namespace {

// cuBLASLt is opened on first use, by its soname first: a process that also holds PyTorch then shares
// the copy PyTorch loaded (two different builds under one soname cannot live side by side - import
// torch before the first projection in such a process), and a process without it gets the toolkit's.
struct LtApi {
  decltype(&cublasLtCreate) Create = nullptr;
  decltype(&cublasLtMatmulDescCreate) DescCreate = nullptr;
  decltype(&cublasLtMatmulDescSetAttribute) DescSet = nullptr;
  decltype(&cublasLtMatrixLayoutCreate) LayoutCreate = nullptr;
  decltype(&cublasLtMatmulPreferenceCreate) PrefCreate = nullptr;
  decltype(&cublasLtMatmulPreferenceSetAttribute) PrefSet = nullptr;
  decltype(&cublasLtMatmulPreferenceDestroy) PrefDestroy = nullptr;
  decltype(&cublasLtMatmulAlgoGetHeuristic) Heuristic = nullptr;
  decltype(&cublasLtMatmul) Matmul = nullptr;
  bool ok = false;
};
const LtApi &lt_api() {
  static LtApi api = [] {
    LtApi a;
    void *h = dlopen("libcublasLt.so.12", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("/usr/local/cuda/lib64/libcublasLt.so.12", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return a;
#define AXONO_LT_SYM(field, name) a.field = reinterpret_cast<decltype(a.field)>(dlsym(h, #name))
    AXONO_LT_SYM(Create, cublasLtCreate);
    AXONO_LT_SYM(DescCreate, cublasLtMatmulDescCreate);
    AXONO_LT_SYM(DescSet, cublasLtMatmulDescSetAttribute);
    AXONO_LT_SYM(LayoutCreate, cublasLtMatrixLayoutCreate);
    AXONO_LT_SYM(PrefCreate, cublasLtMatmulPreferenceCreate);
    AXONO_LT_SYM(PrefSet, cublasLtMatmulPreferenceSetAttribute);
    AXONO_LT_SYM(PrefDestroy, cublasLtMatmulPreferenceDestroy);
    AXONO_LT_SYM(Heuristic, cublasLtMatmulAlgoGetHeuristic);
    AXONO_LT_SYM(Matmul, cublasLtMatmul);
#undef AXONO_LT_SYM
    a.ok = a.Create && a.DescCreate && a.DescSet && a.LayoutCreate && a.PrefCreate && a.PrefSet && a.PrefDestroy &&
           a.Heuristic && a.Matmul;
    return a;
  }();
  return api;
}

// One cuBLASLt handle and one 32 MB workspace per device, made on first use (outside graph capture:
// the warm-up run of CUDAGraph.capture makes that first call); one matmul plan per (rows, out, in, dtype,
// alignment class).  The workspace is shared by every call on the device: calls that may overlap on the
// GPU (different streams) would race on it - keep the projections of one device on one stream.
struct LtState {
  cublasLtHandle_t handle = nullptr;
  void *workspace = nullptr;
  size_t workspace_bytes = size_t(32) << 20;
  struct Plan {
    cublasLtMatmulDesc_t op = nullptr;
    cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;
    cublasLtMatmulAlgo_t algo;
  };
  std::map<std::tuple<int64_t, int64_t, int64_t, int>, Plan> plans;
};
std::mutex g_lt_mu;
LtState g_lt[64];


}  // namespace

extern "C" int axb200_linear_nobias(const void *x, const void *w, void *out, int64_t rows, int64_t out_features,
                                    int64_t in_features, int dtype, void *stream) {
  if (dtype != AXB200_FLOAT16 && dtype != AXB200_FLOAT32) return AXB200_UNSUPPORTED_TYPE;
  if (!x || !w || !out) return AXB200_INVALID_PTR;
  if (rows <= 0 || out_features <= 0 || in_features <= 0) return AXB200_INVALID_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) return AXB200_DEVICE_ERROR;
  const bool capturing = cap != cudaStreamCaptureStatusNone;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return AXB200_DEVICE_ERROR;
  const LtApi &api = lt_api();
  if (!api.ok) return AXB200_INTERNAL_ERROR;
  std::lock_guard<std::mutex> lock(g_lt_mu);
  LtState &lt = g_lt[dev];
  if (!lt.handle) {
    if (capturing) return AXB200_INVALID_ARGUMENT;  // first use must be outside a capture
    // the workspace first: a handle is only published together with the memory every later call assumes
    void *ws = nullptr;
    if (cudaMalloc(&ws, lt.workspace_bytes) != cudaSuccess) {
      cudaGetLastError();
      return AXB200_OUT_OF_MEMORY;
    }
    cublasLtHandle_t h = nullptr;
    if (api.Create(&h) != CUBLAS_STATUS_SUCCESS) {
      cudaFree(ws);
      return AXB200_DEVICE_ERROR;
    }
    lt.workspace = ws;
    lt.handle = h;
  }
  const bool half = dtype == AXB200_FLOAT16;
  const cudaDataType_t dt = half ? CUDA_R_16F : CUDA_R_32F;
  const int64_t in = in_features, outf = out_features;
  // The algorithm is chosen for the operands' alignment too: a plan made for 256-byte aligned pointers
  // may not be valid for less aligned ones, so alignment classes (16 bytes and up, or less) are
  // separate plans.
  const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out);
  const int align_class = (bits & 255u) == 0 ? 2 : (bits & 15u) == 0 ? 1 : 0;
  auto key = std::make_tuple(rows, outf, in, (int)half * 4 + align_class);
  auto it = lt.plans.find(key);
  if (it == lt.plans.end()) {
    if (capturing) return AXB200_INVALID_ARGUMENT;  // plans are made (and timed) in a warm-up run
    // Row-major result (rows, out) = x . w^T is column-major (out, rows) = w_cm^T . x_cm, where the
    // row-major buffers read column-major are w_cm (in, out) and x_cm (in, rows).
    LtState::Plan pl;
    const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
    bool ok = api.DescCreate(&pl.op, CUBLAS_COMPUTE_32F, CUDA_R_32F) == CUBLAS_STATUS_SUCCESS;
    ok = ok && api.DescSet(pl.op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta)) == CUBLAS_STATUS_SUCCESS;
    ok = ok && api.DescSet(pl.op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb)) == CUBLAS_STATUS_SUCCESS;
    ok = ok && api.LayoutCreate(&pl.a, dt, in, outf, in) == CUBLAS_STATUS_SUCCESS;    // w_cm
    ok = ok && api.LayoutCreate(&pl.b, dt, in, rows, in) == CUBLAS_STATUS_SUCCESS;   // x_cm
    ok = ok && api.LayoutCreate(&pl.c, dt, outf, rows, outf) == CUBLAS_STATUS_SUCCESS; // result_cm
    cublasLtMatmulPreference_t pref = nullptr;
    ok = ok && api.PrefCreate(&pref) == CUBLAS_STATUS_SUCCESS;
    ok = ok && api.PrefSet(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &lt.workspace_bytes,
                                                    sizeof(lt.workspace_bytes)) == CUBLAS_STATUS_SUCCESS;
    // Up to eight candidates from the heuristic, each timed on the real operands (beta = 0, so the
    // trial runs are idempotent): at a few dozen rows the first candidate is often not the fastest.
    constexpr int kCandidates = 8;
    cublasLtMatmulHeuristicResult_t heur[kCandidates];
    int found = 0;
    ok = ok && api.Heuristic(lt.handle, pl.op, pl.a, pl.b, pl.c, pl.c, pref, kCandidates, heur, &found) ==
                   CUBLAS_STATUS_SUCCESS && found > 0;
    if (pref) api.PrefDestroy(pref);
    if (!ok) return AXB200_INTERNAL_ERROR;
    int best = -1;
    for (int c = 0; c < found && best < 0; ++c)  // the first usable candidate, unless a timed one beats it
      if (heur[c].state == CUBLAS_STATUS_SUCCESS && heur[c].workspaceSize <= lt.workspace_bytes) best = c;
    if (best < 0) return AXB200_INTERNAL_ERROR;  // nothing the library offers fits
    if (found > 1) {
      const float one = 1.f, zero = 0.f;
      cudaStream_t ts = st;
      cudaEvent_t e0 = nullptr, e1 = nullptr;
      float best_ms = -1.f;
      if (cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess) {
        for (int c = 0; c < found; ++c) {
          if (heur[c].state != CUBLAS_STATUS_SUCCESS || heur[c].workspaceSize > lt.workspace_bytes) continue;
          bool run_ok = true;
          for (int rep = 0; rep < 13 && run_ok; ++rep) {
            if (rep == 3) cudaEventRecord(e0, ts);  // three warm-up runs, ten timed
            run_ok = api.Matmul(lt.handle, pl.op, &one, w, pl.a, x, pl.b, &zero, out, pl.c,
                                out, pl.c, &heur[c].algo, lt.workspace, lt.workspace_bytes, ts) ==
                     CUBLAS_STATUS_SUCCESS;
          }
          float ms = 0.f;
          if (!run_ok || cudaEventRecord(e1, ts) != cudaSuccess || cudaEventSynchronize(e1) != cudaSuccess ||
              cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) {
            cudaGetLastError();
            continue;
          }
          if (best_ms < 0.f || ms < best_ms) {
            best_ms = ms;
            best = c;
          }
        }
      }
      if (e0) cudaEventDestroy(e0);
      if (e1) cudaEventDestroy(e1);
    }
    pl.algo = heur[best].algo;
    it = lt.plans.emplace(key, pl).first;
  }
  const LtState::Plan &pl = it->second;
  const float alpha = 1.f, beta = 0.f;
  const cublasStatus_t cs = api.Matmul(lt.handle, pl.op, &alpha, w, pl.a, x, pl.b, &beta, out, pl.c, out, pl.c, &pl.algo,
                                       lt.workspace, lt.workspace_bytes, st);
  return cs == CUBLAS_STATUS_SUCCESS ? AXB200_OK : AXB200_DEVICE_ERROR;
}
