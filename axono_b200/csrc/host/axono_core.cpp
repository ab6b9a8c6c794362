// Implementation of the native host runtime declared in axono_core.h.
#include "axono_core.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <unordered_map>

#include "axono_b200.h"

namespace axono {
namespace core {

size_t GetDataTypeSize(DataType dtype) {
  switch (dtype) {
    case DataType::INT8: case DataType::BOOLEAN: return 1;
    case DataType::INT16: case DataType::FLOAT16: return 2;
    case DataType::INT32: case DataType::FLOAT32: return 4;
    case DataType::INT64: case DataType::FLOAT64: return 8;
  }
  return 0;
}

size_t CalculateNumElements(const Shape &shape) {
  if (shape.empty()) return 0;
  size_t n = 1;
  for (size_t d : shape) n *= d;
  return n;
}

namespace cuda {
namespace {

int ParseDevice(const std::string &device) {  // "cuda" -> 0, "cuda:3" -> 3, anything else -> -1
  if (device.compare(0, 4, "cuda") != 0) return -1;
  if (device.size() == 4) return 0;
  if (device[4] != ':') return -1;
  return std::atoi(device.c_str() + 5);
}

// ---- caching allocator: exact-size free lists, budget with FIFO eviction, <= 8 blocks per size ----
struct Cache {
  std::mutex mu;
  std::unordered_map<size_t, std::deque<void *>> free_lists;  // keyed by (device, bytes) folded below
  std::deque<std::pair<size_t, void *>> fifo;                 // insertion order, for eviction
  size_t cached_bytes = 0;
  size_t budget = size_t(2) << 30;
};
Cache &cache() {
  static Cache c;
  return c;
}
size_t Key(int dev, size_t bytes) { return bytes * 64 + (size_t)dev; }  // dev < 64

void EvictLocked(Cache &c) {
  while (c.cached_bytes > c.budget && !c.fifo.empty()) {
    auto [key, ptr] = c.fifo.front();
    c.fifo.pop_front();
    auto &lst = c.free_lists[key];
    for (auto it = lst.begin(); it != lst.end(); ++it)
      if (*it == ptr) {
        lst.erase(it);
        cudaFree(ptr);
        c.cached_bytes -= key / 64;
        break;
      }
  }
}

void *CacheAcquire(int dev, size_t bytes) {
  Cache &c = cache();
  std::lock_guard<std::mutex> lock(c.mu);
  auto it = c.free_lists.find(Key(dev, bytes));
  if (it == c.free_lists.end() || it->second.empty()) return nullptr;
  void *p = it->second.back();
  it->second.pop_back();
  for (auto f = c.fifo.begin(); f != c.fifo.end(); ++f)
    if (f->second == p) {
      c.fifo.erase(f);
      break;
    }
  c.cached_bytes -= bytes;
  return p;
}

void CacheRelease(int dev, size_t bytes, void *p) {
  Cache &c = cache();
  std::lock_guard<std::mutex> lock(c.mu);
  auto &lst = c.free_lists[Key(dev, bytes)];
  if (lst.size() >= 8 || bytes > c.budget) {
    cudaFree(p);
    return;
  }
  lst.push_back(p);
  c.fifo.emplace_back(Key(dev, bytes), p);
  c.cached_bytes += bytes;
  EvictLocked(c);
}

// ---- capture state (per thread) and capture pool ----
thread_local cudaStream_t t_capture_stream = nullptr;
thread_local bool t_capturing = false;
thread_local uint64_t t_capture_gen = 0;  // which capture of this thread an in-graph allocation belongs to
thread_local std::vector<void *> t_capture_owned;  // pool blocks the running capture has taken

struct PoolEntry {
  int dev;
  size_t bytes;
  void *ptr;
};
struct CapturePool {
  std::mutex mu;
  std::vector<PoolEntry> entries;
  bool recording = false;
};
CapturePool &pool() {
  static CapturePool p;
  return p;
}

}  // namespace

bool Available() {
  int n = 0;
  return cudaGetDeviceCount(&n) == cudaSuccess && n > 0;
}

Status SetDevice(int index) { return cudaSetDevice(index) == cudaSuccess ? Status::OK : Status::DEVICE_ERROR; }
int CurrentDevice() {
  int dev = -1;
  return cudaGetDevice(&dev) == cudaSuccess ? dev : -1;
}
std::string DevicePciBusId(int index) {
  char buf[32] = {0};
  if (cudaDeviceGetPCIBusId(buf, sizeof(buf), index) != cudaSuccess) {
    cudaGetLastError();
    return "";
  }
  return buf;
}
void *AllocatePinnedHost(size_t bytes) {
  void *p = nullptr;
  if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}
void FreePinnedHost(void *ptr) {
  if (ptr) cudaFreeHost(ptr);
}
EventTimer::EventTimer() {
  cudaEvent_t a = nullptr, b = nullptr;
  if (cudaEventCreate(&a) == cudaSuccess && cudaEventCreate(&b) == cudaSuccess) {
    start_ = a;
    stop_ = b;
  } else {
    if (a) cudaEventDestroy(a);
    cudaGetLastError();
  }
}
EventTimer::~EventTimer() {
  if (start_) cudaEventDestroy(static_cast<cudaEvent_t>(start_));
  if (stop_) cudaEventDestroy(static_cast<cudaEvent_t>(stop_));
}
Status EventTimer::Start() {
  if (!start_) return Status::DEVICE_ERROR;
  return cudaEventRecord(static_cast<cudaEvent_t>(start_), static_cast<cudaStream_t>(CurrentStream())) == cudaSuccess
             ? Status::OK : Status::DEVICE_ERROR;
}
Status EventTimer::Stop() {
  if (!stop_) return Status::DEVICE_ERROR;
  return cudaEventRecord(static_cast<cudaEvent_t>(stop_), static_cast<cudaStream_t>(CurrentStream())) == cudaSuccess
             ? Status::OK : Status::DEVICE_ERROR;
}
Status EventTimer::ElapsedMs(float *ms) {
  if (!start_ || !stop_ || !ms) return Status::DEVICE_ERROR;
  if (cudaEventSynchronize(static_cast<cudaEvent_t>(stop_)) != cudaSuccess) return Status::DEVICE_ERROR;
  return cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start_), static_cast<cudaEvent_t>(stop_)) == cudaSuccess
             ? Status::OK : Status::DEVICE_ERROR;
}
Status DeviceSynchronize() { return cudaDeviceSynchronize() == cudaSuccess ? Status::OK : Status::DEVICE_ERROR; }
Status MemInfo(size_t *free_bytes, size_t *total_bytes) {
  return cudaMemGetInfo(free_bytes, total_bytes) == cudaSuccess ? Status::OK : Status::DEVICE_ERROR;
}
Status CopyToHost(void *dst, const void *device_src, size_t bytes) {
  return cudaMemcpy(dst, device_src, bytes, cudaMemcpyDeviceToHost) == cudaSuccess ? Status::OK : Status::DEVICE_ERROR;
}

Status CopyToDevice(void *device_dst, const void *src, size_t bytes) {
  return cudaMemcpy(device_dst, src, bytes, cudaMemcpyHostToDevice) == cudaSuccess ? Status::OK : Status::DEVICE_ERROR;
}

Status CopyOnDevice(void *device_dst, const void *device_src, size_t bytes) {
  return cudaMemcpy(device_dst, device_src, bytes, cudaMemcpyDeviceToDevice) == cudaSuccess ? Status::OK : Status::DEVICE_ERROR;
}

void SetCacheBudget(size_t bytes) {
  Cache &c = cache();
  std::lock_guard<std::mutex> lock(c.mu);
  c.budget = bytes;
  EvictLocked(c);
}
size_t GetCacheBudget() { return cache().budget; }
size_t GetCachedBytes() { return cache().cached_bytes; }
void ClearDeviceCache() {
  Cache &c = cache();
  std::lock_guard<std::mutex> lock(c.mu);
  for (auto &kv : c.free_lists)
    for (void *p : kv.second) cudaFree(p);
  c.free_lists.clear();
  c.fifo.clear();
  c.cached_bytes = 0;
}

void *CurrentStream() { return t_capturing ? t_capture_stream : nullptr; }
bool IsCapturing() { return t_capturing; }

void ResetCapturePool() {
  CapturePool &p = pool();
  std::lock_guard<std::mutex> lock(p.mu);
  for (auto &e : p.entries) cudaFree(e.ptr);
  p.entries.clear();
  p.recording = false;
}
void SetCapturePoolRecording(bool on) {
  CapturePool &p = pool();
  std::lock_guard<std::mutex> lock(p.mu);
  p.recording = on;
}

std::shared_ptr<void> AllocateStorage(size_t bytes, const std::string &device, bool zero) {
  const int dev = ParseDevice(device);
  if (dev < 0) throw std::runtime_error("bad device string: " + device);
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || dev >= count)
    throw std::runtime_error("CUDA device not available: " + device);
  cudaSetDevice(dev);
  cudaStream_t st = static_cast<cudaStream_t>(CurrentStream());
  CapturePool &cp = pool();
  if (IsCapturing()) {
    // same sizes in the same order as the warm-up run: the addresses repeat
    std::lock_guard<std::mutex> lock(cp.mu);
    for (size_t i = 0; i < cp.entries.size(); ++i) {
      PoolEntry &e = cp.entries[i];
      if (e.dev == dev && e.bytes == bytes) {
        void *ptr = e.ptr;
        cp.entries.erase(cp.entries.begin() + i);  // first match: the warm-up run's order
        t_capture_owned.push_back(ptr);            // from now on it belongs to the graph being captured
        if (zero) cudaMemsetAsync(ptr, 0, bytes, st);  // a memset node: storage starts at zero on every replay
        return std::shared_ptr<void>(ptr, [](void *) {});
      }
    }
  }
  if (IsCapturing()) {
    // No pool entry (the block form of capture has no warm-up run): a stream-ordered allocation,
    // recorded as an allocation node.  Freed inside the same capture it becomes a free node; kept
    // past the end of the capture (an output) it belongs to the graph, which is instantiated with
    // auto-free-on-launch so that it can be launched again.
    void *p = nullptr;
    if (cudaMallocAsync(&p, bytes, st) != cudaSuccess) {
      cudaGetLastError();
      throw std::runtime_error("stream-ordered allocation failed during graph capture");
    }
    if (zero) cudaMemsetAsync(p, 0, bytes, st);
    const uint64_t gen = t_capture_gen;
    return std::shared_ptr<void>(p, [gen, st](void *q) {
      if (t_capturing && t_capture_gen == gen) cudaFreeAsync(q, st);
    });
  }
  void *p = CacheAcquire(dev, bytes);
  if (p) {
    if (zero) cudaMemsetAsync(p, 0, bytes, st);
  } else {
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
      cudaGetLastError();
      ClearDeviceCache();  // drain the pool and retry once
      if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        throw std::bad_alloc();
      }
    }
    if (zero) cudaMemsetAsync(p, 0, bytes, st);
  }
  bool recorded = false;
  {
    std::lock_guard<std::mutex> lock(cp.mu);
    if (cp.recording) {
      cp.entries.push_back(PoolEntry{dev, bytes, p});
      recorded = true;
    }
  }
  if (recorded) return std::shared_ptr<void>(p, [](void *) {});  // the capture pool owns it now
  return std::shared_ptr<void>(p, [dev, bytes](void *q) { CacheRelease(dev, bytes, q); });
}

// ---- graph capture ----
namespace {
void DropCaptureOwned() {  // a capture that did not become a graph gives its pool blocks back to the device
  for (void *ptr : t_capture_owned) cudaFree(ptr);
  t_capture_owned.clear();
}
}  // namespace

Status BeginGraphCapture(void **stream_out) {
  if (t_capturing) return Status::INVALID_ARGUMENT;
  cudaStream_t st = nullptr;
  if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) return Status::DEVICE_ERROR;
  if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
    cudaGetLastError();
    cudaStreamDestroy(st);
    return Status::DEVICE_ERROR;
  }
  t_capture_stream = st;
  t_capturing = true;
  ++t_capture_gen;
  SetCapturePoolRecording(false);  // also re-arms the pool entries for this run
  if (stream_out) *stream_out = st;
  return Status::OK;
}

Status EndGraphCapture(void *stream, GraphExec *out) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  t_capturing = false;
  t_capture_stream = nullptr;
  cudaGraph_t graph = nullptr;
  if (cudaStreamEndCapture(st, &graph) != cudaSuccess || !graph) {
    cudaGetLastError();
    cudaStreamDestroy(st);
    DropCaptureOwned();
    return Status::INTERNAL_ERROR;
  }
  size_t n = 0;
  cudaGraphGetNodes(graph, nullptr, &n);
  if (n == 0) {  // nothing was launched: an empty graph is an error
    cudaGraphDestroy(graph);
    cudaStreamDestroy(st);
    DropCaptureOwned();
    return Status::INVALID_ARGUMENT;
  }
  cudaGraphExec_t exec = nullptr;
  const cudaError_t e = cudaGraphInstantiate(&exec, graph, cudaGraphInstantiateFlagAutoFreeOnLaunch);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    cudaGetLastError();
    cudaStreamDestroy(st);
    DropCaptureOwned();
    return Status::INTERNAL_ERROR;
  }
  out->Reset();
  out->exec_ = exec;
  out->stream_ = st;
  out->num_nodes_ = n;
  out->owned_.swap(t_capture_owned);
  return Status::OK;
}

void AbortGraphCapture(void *stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  t_capturing = false;
  t_capture_stream = nullptr;
  cudaGraph_t graph = nullptr;
  cudaStreamEndCapture(st, &graph);
  cudaGetLastError();
  if (graph) cudaGraphDestroy(graph);
  cudaStreamDestroy(st);
  DropCaptureOwned();
}

GraphExec::~GraphExec() { Reset(); }
void GraphExec::Reset() {
  if (stream_) cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));
  if (exec_) cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(exec_));
  if (stream_) cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
  for (void *ptr : owned_) cudaFree(ptr);
  owned_.clear();
  exec_ = nullptr;
  stream_ = nullptr;
  num_nodes_ = 0;
}
Status GraphExec::Replay() {
  if (!exec_) return Status::INVALID_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (cudaGraphLaunch(static_cast<cudaGraphExec_t>(exec_), st) != cudaSuccess) return Status::DEVICE_ERROR;
  return cudaStreamSynchronize(st) == cudaSuccess ? Status::OK : Status::DEVICE_ERROR;
}
Status GraphExec::ReplayTimed(int times, float *ms_per_launch) {
  if (!exec_ || times <= 0 || !ms_per_launch) return Status::INVALID_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return Status::DEVICE_ERROR;
  bool ok = cudaStreamSynchronize(st) == cudaSuccess && cudaEventRecord(e0, st) == cudaSuccess;
  for (int i = 0; i < times && ok; ++i) ok = cudaGraphLaunch(static_cast<cudaGraphExec_t>(exec_), st) == cudaSuccess;
  ok = ok && cudaEventRecord(e1, st) == cudaSuccess && cudaEventSynchronize(e1) == cudaSuccess;
  float ms = 0.f;
  ok = ok && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *ms_per_launch = ms / (float)times;
  return ok ? Status::OK : Status::DEVICE_ERROR;
}
Status GraphExec::Sync() {
  if (!stream_) return Status::OK;
  return cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)) == cudaSuccess ? Status::OK : Status::DEVICE_ERROR;
}

}  // namespace cuda

// ---- Tensor ----
Tensor::Tensor(DataType dtype, const Shape &shape) : dtype_(dtype), shape_(shape) {
  num_elements_ = CalculateNumElements(shape);
  Allocate();
}
Tensor::Tensor(DataType dtype, const Shape &shape, const std::string &device)
    : dtype_(dtype), shape_(shape), device_(device) {
  num_elements_ = CalculateNumElements(shape);
  Allocate();
}

void Tensor::Allocate() {
  data_.reset();
  const size_t bytes = num_bytes();
  if (bytes == 0) return;
  if (is_cuda()) {
    data_ = cuda::AllocateStorage(bytes, device_, zero_fill_);
  } else {
    void *p = std::calloc(1, bytes);  // new storage is zero-filled
    if (!p) throw std::bad_alloc();
    data_ = std::shared_ptr<void>(p, std::free);
  }
}

Tensor Tensor::Uninitialized(DataType dtype, const Shape &shape, const std::string &device) {
  Tensor t(dtype);
  t.device_ = device;
  t.zero_fill_ = !t.is_cuda();  // host storage stays calloc'ed
  t.shape_ = shape;
  t.num_elements_ = CalculateNumElements(shape);
  t.Allocate();
  return t;
}

Tensor Tensor::FromBorrowed(DataType dtype, const Shape &shape, const void *data) {
  Tensor t(dtype);
  t.shape_ = shape;
  t.num_elements_ = CalculateNumElements(shape);
  t.data_ = std::shared_ptr<void>(const_cast<void *>(data), [](void *) {});
  return t;
}

Tensor Tensor::FromBorrowedDevice(DataType dtype, const Shape &shape, void *device_ptr, const std::string &device) {
  Tensor t(dtype);
  t.device_ = device;
  t.zero_fill_ = false;
  t.shape_ = shape;
  t.num_elements_ = CalculateNumElements(shape);
  t.data_ = std::shared_ptr<void>(device_ptr, [](void *) {});
  return t;
}

int Tensor::device_index() const {
  if (!is_cuda()) return -1;
  return device_.size() > 5 ? std::atoi(device_.c_str() + 5) : 0;
}

Status Tensor::CopyFrom(const Tensor &src) {
  if (src.num_elements_ != num_elements_ || src.dtype_ != dtype_) return Status::SHAPE_MISMATCH;
  const size_t bytes = num_bytes();
  if (bytes == 0) return Status::OK;
  if (!is_cuda() && !src.is_cuda()) {
    std::memcpy(data_.get(), src.data_.get(), bytes);
    return Status::OK;
  }
  // Blocking copies on the legacy default stream order after the kernels launched on it; while
  // capturing, device-to-device copies join the captured stream.
  cudaStream_t st = static_cast<cudaStream_t>(cuda::CurrentStream());
  cudaError_t e;
  if (is_cuda() && src.is_cuda())
    e = cudaMemcpyAsync(data_.get(), src.data_.get(), bytes, cudaMemcpyDeviceToDevice, st);
  else if (is_cuda())
    e = cudaMemcpy(data_.get(), src.data_.get(), bytes, cudaMemcpyHostToDevice);
  else
    e = cudaMemcpy(data_.get(), src.data_.get(), bytes, cudaMemcpyDeviceToHost);
  return e == cudaSuccess ? Status::OK : Status::DEVICE_ERROR;
}

Tensor Tensor::to(const std::string &device) const {
  if (device == device_) return *this;  // same device: share the storage
  Tensor out(dtype_, shape_, device);
  if (out.CopyFrom(*this) != Status::OK) throw std::runtime_error("Tensor::to: copy failed");
  return out;
}
Status Tensor::to_(const std::string &device) {
  if (device == device_) return Status::OK;
  *this = to(device);
  return Status::OK;
}

Tensor Tensor::CastTo(DataType target) const {
  if (target == dtype_) return *this;
  const bool h2f = dtype_ == DataType::FLOAT16 && target == DataType::FLOAT32;
  const bool f2h = dtype_ == DataType::FLOAT32 && target == DataType::FLOAT16;
  if (!h2f && !f2h) throw std::runtime_error("CastTo: only FLOAT16 <-> FLOAT32");
  Tensor out(target, shape_, device_);
  if (is_cuda()) {
    const int st = axb200_cast(data_.get(), static_cast<int>(dtype_), out.data(), static_cast<int>(target),
                               (int64_t)num_elements_, cuda::CurrentStream());
    if (st != 0) throw std::runtime_error("CastTo failed, status " + std::to_string(st));
  } else if (h2f) {
    const __half *s = data<__half>();
    float *d = out.data<float>();
    for (size_t i = 0; i < num_elements_; ++i) d[i] = __half2float(s[i]);
  } else {
    const float *s = data<float>();
    __half *d = out.data<__half>();
    for (size_t i = 0; i < num_elements_; ++i) d[i] = __float2half_rn(s[i]);
  }
  return out;
}

Status Tensor::Reshape(const Shape &shape) {
  if (CalculateNumElements(shape) != num_elements_) throw std::runtime_error("Reshape requires the same element count");
  shape_ = shape;
  return Status::OK;
}
Status Tensor::Resize(const Shape &shape) {
  const size_t n = CalculateNumElements(shape);
  shape_ = shape;
  if (n != num_elements_) {
    num_elements_ = n;
    Allocate();
  }
  return Status::OK;
}
Status Tensor::FillZero() {
  if (!data_) return Status::INVALID_ARGUMENT;
  if (is_cuda())
    return cudaMemsetAsync(data_.get(), 0, num_bytes(), static_cast<cudaStream_t>(cuda::CurrentStream())) == cudaSuccess
               ? Status::OK : Status::DEVICE_ERROR;
  std::memset(data_.get(), 0, num_bytes());
  return Status::OK;
}
std::string Tensor::ToString() const {
  std::ostringstream os;
  os << "Tensor(dtype=" << static_cast<int>(dtype_) << ", shape=[";
  for (size_t i = 0; i < shape_.size(); ++i) os << (i ? ", " : "") << shape_[i];
  os << "], device=" << device_ << ")";
  return os.str();
}

}  // namespace core
}  // namespace axono
