// KV page arena: the allocator side of the paged cache.  Replaces what the reference does for KV
// tensors - every step `concat` allocates a new, ever larger tensor from the size-bucketed caching
// pool (axono/python/axono/nn/kv_cache.py:96-102, src/core/cuda/detail.cu:41-146,153-275), which can
// never reuse a block because no size repeats - by fixed pools of pages with a free list:
//   * per layer one K pool and one V pool (num_pages, hkv, page_tokens, d), allocated once,
//     zero-filled once (as the reference zero-fills new storage), addresses stable for the life of
//     the arena (CUDA-graph replay depends on that), never evicted, never re-zeroed on reuse (the
//     kernels mask by sequence length, so stale bytes in a recycled page cannot be read);
//   * sequences own pages through a block table (max_seqs, max_blocks) shared by all layers; a
//     sequence slot is the batch row the kernels see;
//   * alloc / reserve / free are host-side and O(pages touched); the device copies of the block
//     table are refreshed by axb200_kv_arena_sync (one H2D copy of the dirty rows' span).
// With device_memory == 0 only the bookkeeping exists (no CUDA call is made): that mode is what the
// CPU tests drive.
#include <mutex>
#include <new>
#include <utility>
#include <vector>

#include "common.cuh"

struct axb200_kv_arena {
  int n_layers, num_pages, hkv, page_tokens, d, dtype, max_seqs, max_blocks;
  bool device;
  std::mutex mu;
  std::vector<int32_t> free_pages;           // stack of free page ids
  std::vector<int32_t> table;                // host block table (max_seqs * max_blocks), -1 = none
  std::vector<int32_t> blocks_of;            // pages held per sequence slot
  std::vector<uint8_t> live;                 // slot in use
  int dirty_lo, dirty_hi;                    // rows whose device copy is stale: [lo, hi)
  std::vector<void *> k_pools, v_pools;      // per layer
  int32_t *table_dev = nullptr;
  int32_t *seq_lens_dev = nullptr;
  size_t pool_bytes = 0;
};

namespace {

void mark_dirty(axb200_kv_arena *a, int row) {
  if (a->dirty_lo > row) a->dirty_lo = row;
  if (a->dirty_hi < row + 1) a->dirty_hi = row + 1;
}

// Grows `seq` to hold `tokens`; all-or-nothing.
int reserve_locked(axb200_kv_arena *a, int seq, int64_t tokens) {
  if (seq < 0 || seq >= a->max_seqs || !a->live[seq] || tokens < 0) return AXB200_INVALID_ARGUMENT;
  const int64_t need = (tokens + a->page_tokens - 1) / a->page_tokens;
  if (need > a->max_blocks) return AXB200_INVALID_ARGUMENT;
  const int have = a->blocks_of[seq];
  if (need <= have) return AXB200_OK;
  if ((int64_t)a->free_pages.size() < need - have) return AXB200_OUT_OF_MEMORY;
  for (int64_t blk = have; blk < need; ++blk) {
    a->table[(size_t)seq * a->max_blocks + blk] = a->free_pages.back();
    a->free_pages.pop_back();
  }
  a->blocks_of[seq] = (int)need;
  mark_dirty(a, seq);
  return AXB200_OK;
}

}  // namespace

extern "C" {

int axb200_kv_arena_create(int n_layers, int num_pages, int hkv, int page_tokens, int d, int dtype,
                           int max_seqs, int max_blocks, int device_memory,
                           axb200_kv_arena **out) {
  if (!out) return AXB200_INVALID_PTR;
  if (n_layers <= 0 || num_pages <= 0 || hkv <= 0 || page_tokens <= 0 || page_tokens % 64 != 0 ||
      d <= 0 || max_seqs <= 0 || max_blocks <= 0 || axb::dtype_size(dtype) == 0)
    return AXB200_INVALID_ARGUMENT;
  axb200_kv_arena *a = new (std::nothrow) axb200_kv_arena();
  if (!a) return AXB200_OUT_OF_MEMORY;
  a->n_layers = n_layers;
  a->num_pages = num_pages;
  a->hkv = hkv;
  a->page_tokens = page_tokens;
  a->d = d;
  a->dtype = dtype;
  a->max_seqs = max_seqs;
  a->max_blocks = max_blocks;
  a->device = device_memory != 0;
  a->free_pages.resize(num_pages);
  for (int i = 0; i < num_pages; ++i) a->free_pages[i] = num_pages - 1 - i;  // page 0 is handed out first
  a->table.assign((size_t)max_seqs * max_blocks, -1);
  a->blocks_of.assign(max_seqs, 0);
  a->live.assign(max_seqs, 0);
  a->dirty_lo = 0;
  a->dirty_hi = max_seqs;
  a->pool_bytes = (size_t)num_pages * hkv * page_tokens * d * axb::dtype_size(dtype);
  if (a->device) {
    bool ok = true;
    for (int l = 0; l < n_layers && ok; ++l) {
      void *k = nullptr, *v = nullptr;
      ok = cudaMalloc(&k, a->pool_bytes) == cudaSuccess && cudaMalloc(&v, a->pool_bytes) == cudaSuccess;
      if (k) a->k_pools.push_back(k);
      if (v) a->v_pools.push_back(v);
      if (ok) ok = cudaMemset(k, 0, a->pool_bytes) == cudaSuccess && cudaMemset(v, 0, a->pool_bytes) == cudaSuccess;
    }
    ok = ok && cudaMalloc(&a->table_dev, a->table.size() * sizeof(int32_t)) == cudaSuccess &&
         cudaMalloc(&a->seq_lens_dev, max_seqs * sizeof(int32_t)) == cudaSuccess &&
         cudaMemset(a->seq_lens_dev, 0, max_seqs * sizeof(int32_t)) == cudaSuccess;
    if (!ok) {
      cudaGetLastError();
      for (void *p : a->k_pools) cudaFree(p);
      for (void *p : a->v_pools) cudaFree(p);
      if (a->table_dev) cudaFree(a->table_dev);
      if (a->seq_lens_dev) cudaFree(a->seq_lens_dev);
      delete a;
      return AXB200_OUT_OF_MEMORY;
    }
  }
  *out = a;
  return AXB200_OK;
}

int axb200_kv_arena_shuffle_free(axb200_kv_arena *a, uint64_t seed) {
  if (!a) return AXB200_INVALID_PTR;
  std::lock_guard<std::mutex> lock(a->mu);
  // Fisher-Yates over the free stack with a fixed 64-bit LCG stream (Knuth's MMIX constants), so the
  // same seed gives the same order everywhere
  uint64_t x = seed * 6364136223846793005ull + 1442695040888963407ull;
  for (size_t i = a->free_pages.size(); i > 1; --i) {
    x = x * 6364136223846793005ull + 1442695040888963407ull;
    const size_t j = (size_t)((x >> 33) % i);
    std::swap(a->free_pages[i - 1], a->free_pages[j]);
  }
  return AXB200_OK;
}

int axb200_kv_arena_destroy(axb200_kv_arena *a) {
  if (!a) return AXB200_INVALID_PTR;
  if (a->device) {
    cudaDeviceSynchronize();
    for (void *p : a->k_pools) cudaFree(p);
    for (void *p : a->v_pools) cudaFree(p);
    cudaFree(a->table_dev);
    cudaFree(a->seq_lens_dev);
  }
  delete a;
  return AXB200_OK;
}

// Takes a free sequence slot (the lowest) and pages for `reserve_tokens`.
int axb200_kv_arena_alloc_seq(axb200_kv_arena *a, int64_t reserve_tokens, int *seq_id) {
  if (!a || !seq_id) return AXB200_INVALID_PTR;
  std::lock_guard<std::mutex> lock(a->mu);
  int slot = -1;
  for (int s = 0; s < a->max_seqs; ++s)
    if (!a->live[s]) {
      slot = s;
      break;
    }
  if (slot < 0) return AXB200_OUT_OF_MEMORY;
  a->live[slot] = 1;
  const int rc = reserve_locked(a, slot, reserve_tokens);
  if (rc != AXB200_OK) {
    a->live[slot] = 0;
    return rc;
  }
  *seq_id = slot;
  return AXB200_OK;
}

// Makes room for `tokens` tokens in total (call before the step that crosses a page boundary).
int axb200_kv_arena_reserve(axb200_kv_arena *a, int seq_id, int64_t tokens) {
  if (!a) return AXB200_INVALID_PTR;
  std::lock_guard<std::mutex> lock(a->mu);
  return reserve_locked(a, seq_id, tokens);
}

// Returns the sequence's pages to the free list and zeroes its device length on `stream`.
int axb200_kv_arena_free_seq(axb200_kv_arena *a, int seq_id, void *stream) {
  if (!a) return AXB200_INVALID_PTR;
  std::lock_guard<std::mutex> lock(a->mu);
  if (seq_id < 0 || seq_id >= a->max_seqs || !a->live[seq_id]) return AXB200_INVALID_ARGUMENT;
  for (int blk = a->blocks_of[seq_id] - 1; blk >= 0; --blk) {
    int32_t &e = a->table[(size_t)seq_id * a->max_blocks + blk];
    a->free_pages.push_back(e);
    e = -1;
  }
  a->blocks_of[seq_id] = 0;
  a->live[seq_id] = 0;
  mark_dirty(a, seq_id);
  if (a->device &&
      cudaMemsetAsync(a->seq_lens_dev + seq_id, 0, sizeof(int32_t), static_cast<cudaStream_t>(stream)) != cudaSuccess)
    return AXB200_DEVICE_ERROR;
  return AXB200_OK;
}

// Uploads the block-table rows changed since the last sync (one H2D copy on `stream`).  The host
// table is pageable memory, so the copy is staged by the runtime before the call returns.
int axb200_kv_arena_sync(axb200_kv_arena *a, void *stream) {
  if (!a) return AXB200_INVALID_PTR;
  std::lock_guard<std::mutex> lock(a->mu);
  if (!a->device || a->dirty_lo >= a->dirty_hi) {
    a->dirty_lo = a->max_seqs;
    a->dirty_hi = 0;
    return AXB200_OK;
  }
  const size_t off = (size_t)a->dirty_lo * a->max_blocks, n = (size_t)(a->dirty_hi - a->dirty_lo) * a->max_blocks;
  const cudaError_t e = cudaMemcpyAsync(a->table_dev + off, a->table.data() + off, n * sizeof(int32_t),
                                        cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
  a->dirty_lo = a->max_seqs;
  a->dirty_hi = 0;
  return e == cudaSuccess ? AXB200_OK : AXB200_DEVICE_ERROR;
}

int axb200_kv_arena_stats(axb200_kv_arena *a, int64_t *pages_total, int64_t *pages_free,
                          int64_t *seqs_live, int64_t *device_bytes) {
  if (!a) return AXB200_INVALID_PTR;
  std::lock_guard<std::mutex> lock(a->mu);
  int64_t live = 0;
  for (uint8_t l : a->live) live += l;
  if (pages_total) *pages_total = a->num_pages;
  if (pages_free) *pages_free = (int64_t)a->free_pages.size();
  if (seqs_live) *seqs_live = live;
  if (device_bytes) *device_bytes = a->device ? (int64_t)(2 * a->pool_bytes * a->n_layers) : 0;
  return AXB200_OK;
}

// Host view of one block-table row (for tests and debugging): copies blocks_of entries.
int axb200_kv_arena_seq_pages(axb200_kv_arena *a, int seq_id, int32_t *pages_out, int capacity) {
  if (!a || !pages_out) return -1;
  std::lock_guard<std::mutex> lock(a->mu);
  if (seq_id < 0 || seq_id >= a->max_seqs || !a->live[seq_id]) return -1;
  const int n = a->blocks_of[seq_id];
  for (int i = 0; i < n && i < capacity; ++i) pages_out[i] = a->table[(size_t)seq_id * a->max_blocks + i];
  return n;
}

int axb200_kv_arena_geometry(axb200_kv_arena *a, int *n_layers, int *num_pages, int *hkv, int *page_tokens,
                             int *d, int *dtype, int *max_seqs, int *max_blocks) {
  if (!a) return AXB200_INVALID_PTR;
  if (n_layers) *n_layers = a->n_layers;
  if (num_pages) *num_pages = a->num_pages;
  if (hkv) *hkv = a->hkv;
  if (page_tokens) *page_tokens = a->page_tokens;
  if (d) *d = a->d;
  if (dtype) *dtype = a->dtype;
  if (max_seqs) *max_seqs = a->max_seqs;
  if (max_blocks) *max_blocks = a->max_blocks;
  return AXB200_OK;
}

void *axb200_kv_arena_k_pages(axb200_kv_arena *a, int layer) {
  return (a && a->device && layer >= 0 && layer < a->n_layers) ? a->k_pools[layer] : nullptr;
}
void *axb200_kv_arena_v_pages(axb200_kv_arena *a, int layer) {
  return (a && a->device && layer >= 0 && layer < a->n_layers) ? a->v_pools[layer] : nullptr;
}
int32_t *axb200_kv_arena_block_table(axb200_kv_arena *a) { return a ? a->table_dev : nullptr; }
int32_t *axb200_kv_arena_seq_lens(axb200_kv_arena *a) { return a ? a->seq_lens_dev : nullptr; }

}  // extern "C"
