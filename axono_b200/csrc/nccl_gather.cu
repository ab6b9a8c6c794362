// The library collective of the decode path: an NCCL all-gather of per-head attention outputs for KV
// heads sharded over the GPUs of one node (one process per GPU).  The reference has no collective
// (its WITH_NCCL build option is reserved and unused, CMakeLists.txt:78,91-92); this is the plain form
// a maintainer would write first - attention, ncclAllGather, output projection - and the baseline the
// fused attention + gather kernel (gqa_decode.cu) is measured against.
//
// NCCL is opened by soname on first use, so a process that never shards heads does not load it.  The
// communicator is created - and used once - by axb200_nccl_init, which every rank must call before
// any stream capture: creation allocates and synchronises, neither of which a capture allows.  After
// that axb200_nccl_all_gather only enqueues the collective on the given stream and may be captured.
// Every rank must issue the same sequence of collectives; like any collective it waits for its peers.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace {

struct NcclApi {
  decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
  decltype(&ncclCommInitRank) CommInitRank = nullptr;
  decltype(&ncclAllGather) AllGather = nullptr;
  decltype(&ncclCommDestroy) CommDestroy = nullptr;
  bool ok = false;
};

const NcclApi &nccl_api() {
  static NcclApi api = [] {
    NcclApi a;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return a;
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    a.ok = a.GetUniqueId && a.CommInitRank && a.AllGather && a.CommDestroy;
    return a;
  }();
  return api;
}

// dst (n1, n0, row) = src (n0, n1, row): the gathered buffer comes rank-major, (world, batch, heads*d);
// the projection reads (batch, world, heads*d).  16 bytes per thread and access.
__global__ void __launch_bounds__(256)
swap_leading_dims_kernel(const uint4 *src, uint4 *dst, int n0, int n1, int row16) {
  const int64_t total = (int64_t)n0 * n1 * row16;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    // i runs over dst in its own order: dst[(j1 * n0 + j0) * row16 + c]
    const int c = (int)(i % row16);
    const int64_t r = i / row16;
    const int j0 = (int)(r % n0), j1 = (int)(r / n0);
    dst[i] = src[((int64_t)j0 * n1 + j1) * row16 + c];
  }
}

}  // namespace

extern "C" {

int axb200_nccl_unique_id(void *id128) {
  if (!id128) return AXB200_INVALID_PTR;
  const NcclApi &api = nccl_api();
  if (!api.ok) return AXB200_INTERNAL_ERROR;
  static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique id size");
  ncclUniqueId id;
  if (api.GetUniqueId(&id) != ncclSuccess) return AXB200_DEVICE_ERROR;
  memcpy(id128, &id, sizeof(id));
  return AXB200_OK;
}

int axb200_nccl_init(const void *id128, int world, int rank, void **comm_out) {
  if (!id128 || !comm_out) return AXB200_INVALID_PTR;
  if (world < 1 || rank < 0 || rank >= world) return AXB200_INVALID_ARGUMENT;
  const NcclApi &api = nccl_api();
  if (!api.ok) return AXB200_INTERNAL_ERROR;
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  ncclComm_t comm = nullptr;
  if (api.CommInitRank(&comm, world, id, rank) != ncclSuccess) return AXB200_DEVICE_ERROR;
  // one collective now, outside any capture: NCCL sets up its channels and buffers on first use
  void *probe = nullptr;
  bool ok = cudaMalloc(&probe, 256 * (size_t)(world + 1)) == cudaSuccess;
  ok = ok && api.AllGather(probe, static_cast<char *>(probe) + 256, 256, ncclChar, comm, nullptr) == ncclSuccess;
  ok = ok && cudaDeviceSynchronize() == cudaSuccess;
  if (probe) cudaFree(probe);
  if (!ok) {
    api.CommDestroy(comm);
    return AXB200_DEVICE_ERROR;
  }
  *comm_out = comm;
  return AXB200_OK;
}

int axb200_nccl_all_gather(void *comm, const void *send, void *recv, size_t bytes_per_rank, void *stream) {
  if (!comm || !send || !recv) return AXB200_INVALID_PTR;
  if (bytes_per_rank == 0) return AXB200_INVALID_ARGUMENT;
  const NcclApi &api = nccl_api();
  if (!api.ok) return AXB200_INTERNAL_ERROR;
  return api.AllGather(send, recv, bytes_per_rank, ncclChar, static_cast<ncclComm_t>(comm),
                       static_cast<cudaStream_t>(stream)) == ncclSuccess
             ? AXB200_OK
             : AXB200_DEVICE_ERROR;
}

int axb200_nccl_destroy(void *comm) {
  if (!comm) return AXB200_INVALID_PTR;
  const NcclApi &api = nccl_api();
  if (!api.ok) return AXB200_INTERNAL_ERROR;
  return api.CommDestroy(static_cast<ncclComm_t>(comm)) == ncclSuccess ? AXB200_OK : AXB200_DEVICE_ERROR;
}

int axb200_swap_leading_dims(const void *src, void *dst, int n0, int n1, size_t row_bytes, void *stream) {
  if (!src || !dst) return AXB200_INVALID_PTR;
  if (n0 <= 0 || n1 <= 0 || row_bytes == 0 || row_bytes % 16 != 0 ||
      ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u))
    return AXB200_INVALID_ARGUMENT;
  const int row16 = (int)(row_bytes / 16);
  const int64_t total = (int64_t)n0 * n1 * row16;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  swap_leading_dims_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4 *>(src), static_cast<uint4 *>(dst), n0, n1, row16);
  return axb::launch_status();
}

}  // extern "C"
