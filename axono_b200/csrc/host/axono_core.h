// Native host runtime of the drop-in: the container types and device services the reference's
// operators rely on, re-implemented for this library (no PyTorch anywhere in this layer).
//
//   axono::core::{DataType, Status, Context, Shape, Tensor}   include/axono/core/types.h:18-72,
//                                                             include/axono/core/tensor.h:24-129
//   axono::core::cuda caching allocator                       src/core/cuda/detail.cu:41-146,153-275
//   current stream, graph capture, capture pool               src/core/cuda/{graph,capture_pool}.cu
//
// Semantics kept: contiguous row-major tensors; copy = share storage; new storage is zero-filled;
// device is a string "cpu" | "cuda" | "cuda:<id>"; FLOAT16 is raw IEEE bits; operators launch on the
// current stream (legacy default stream, or the capture stream while capturing) and never
// synchronise; allocations made while a graph is being captured come from the capture pool that the
// warm-up run filled, so addresses repeat.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace axono {
namespace core {

enum class DataType { INT8, INT16, INT32, INT64, FLOAT16, FLOAT32, FLOAT64, BOOLEAN };
enum class Status {
  OK, INVALID_ARGUMENT, OUT_OF_MEMORY, UNSUPPORTED_TYPE, SHAPE_MISMATCH, INTERNAL_ERROR, DEVICE_ERROR,
  INVALID_PTR, DEVICE_MISMATCH
};
struct Context { int device_id = 0; };
using Shape = std::vector<size_t>;

size_t GetDataTypeSize(DataType dtype);
size_t CalculateNumElements(const Shape &shape);  // 0 for an empty shape, as in the reference

class Tensor {
 public:
  Tensor() = default;
  explicit Tensor(DataType dtype) : dtype_(dtype) {}
  Tensor(DataType dtype, const Shape &shape);
  Tensor(DataType dtype, const Shape &shape, const std::string &device);
  // copy = share storage; move = take storage (defaults do exactly that)

  static Tensor FromBorrowed(DataType dtype, const Shape &shape, const void *data);  // host memory, not owned
  // Device memory owned by somebody else (a peer-mapped buffer, a KV pool): a view, never freed here.
  static Tensor FromBorrowedDevice(DataType dtype, const Shape &shape, void *device_ptr, const std::string &device);
  // Device storage without the zero fill, for results an operator overwrites completely (the binding
  // layer's outputs): the fill would be one more memset per operator in every captured graph.  Storage
  // the tensor takes later through Resize is not filled either.
  static Tensor Uninitialized(DataType dtype, const Shape &shape, const std::string &device);

  const std::string &device() const { return device_; }
  bool is_cuda() const { return device_.compare(0, 4, "cuda") == 0; }
  int device_index() const;  // -1 for cpu
  DataType dtype() const { return dtype_; }
  const Shape &shape() const { return shape_; }
  size_t ndim() const { return shape_.size(); }
  size_t num_elements() const { return num_elements_; }
  size_t num_bytes() const { return num_elements_ * GetDataTypeSize(dtype_); }
  void *data() { return data_.get(); }
  const void *data() const { return data_.get(); }
  template <typename T> T *data() { return static_cast<T *>(data_.get()); }
  template <typename T> const T *data() const { return static_cast<const T *>(data_.get()); }

  Tensor to(const std::string &device) const;  // same device: returns a tensor sharing the storage
  Status to_(const std::string &device);
  Status CopyFrom(const Tensor &src);          // element counts must match; any device pair
  Tensor CastTo(DataType target) const;        // FLOAT16 <-> FLOAT32 (same device)
  Status Reshape(const Shape &shape);          // throws when the element count differs
  Status Resize(const Shape &shape);           // reallocates only when the element count changes
  Status FillZero();
  bool IsSameShape(const Tensor &o) const { return shape_ == o.shape_; }
  std::string ToString() const;

 private:
  void Allocate();
  DataType dtype_ = DataType::FLOAT32;
  Shape shape_;
  std::string device_ = "cpu";
  size_t num_elements_ = 0;
  bool zero_fill_ = true;
  std::shared_ptr<void> data_;
};

namespace cuda {

bool Available();
Status SetDevice(int index);  // makes the device current for this thread (one process per GPU picks its own)
int CurrentDevice();          // -1 without a device
std::string DevicePciBusId(int index);  // "" on failure; lets a monitor find the same GPU through NVML
Status DeviceSynchronize();
void *AllocatePinnedHost(size_t bytes);  // page-locked host memory for asynchronous copies; nullptr on failure
void FreePinnedHost(void *ptr);
// A pair of events on the current stream: Start / Stop bracket a region, ElapsedMs waits for Stop.
class EventTimer {
 public:
  EventTimer();
  ~EventTimer();
  EventTimer(const EventTimer &) = delete;
  EventTimer &operator=(const EventTimer &) = delete;
  Status Start();
  Status Stop();
  Status ElapsedMs(float *ms);
 private:
  void *start_ = nullptr, *stop_ = nullptr;  // cudaEvent_t
};
Status MemInfo(size_t *free_bytes, size_t *total_bytes);  // of the current device
Status CopyToHost(void *dst, const void *device_src, size_t bytes);  // blocking, legacy default stream
Status CopyToDevice(void *device_dst, const void *src, size_t bytes);  // blocking, legacy default stream
Status CopyOnDevice(void *device_dst, const void *device_src, size_t bytes);  // blocking, legacy default stream
// --- caching allocator ---
void SetCacheBudget(size_t bytes);
size_t GetCacheBudget();
size_t GetCachedBytes();
void ClearDeviceCache();
std::shared_ptr<void> AllocateStorage(size_t bytes, const std::string &device, bool zero = true);

// --- current stream and graph capture ---
void *CurrentStream();  // cudaStream_t: legacy default stream, or this thread's capture stream
bool IsCapturing();
void ResetCapturePool();
void SetCapturePoolRecording(bool on);

class GraphExec {
 public:
  GraphExec() = default;
  ~GraphExec();
  GraphExec(const GraphExec &) = delete;
  GraphExec &operator=(const GraphExec &) = delete;
  Status Replay();  // launch on the capture stream and wait for it
  // `times` launches back to back between two events on the capture stream; milliseconds per launch
  Status ReplayTimed(int times, float *ms_per_launch);
  Status Sync();
  void Reset();
  bool IsCaptured() const { return exec_ != nullptr; }
  size_t NumNodes() const { return num_nodes_; }

 private:
  friend Status EndGraphCapture(void *stream, GraphExec *out);
  void *exec_ = nullptr;    // cudaGraphExec_t
  void *stream_ = nullptr;  // cudaStream_t the graph was captured on
  size_t num_nodes_ = 0;
  // Device blocks the captured run took from the capture pool: the graph's nodes and its output
  // tensors point into them, so they live exactly as long as the graph (Reset frees them).  Another
  // capture never touches them, so several graphs can be alive at once.
  std::vector<void *> owned_;
};

Status BeginGraphCapture(void **stream_out);
Status EndGraphCapture(void *stream, GraphExec *out);  // an empty graph is an error
void AbortGraphCapture(void *stream);

}  // namespace cuda
}  // namespace core
}  // namespace axono
