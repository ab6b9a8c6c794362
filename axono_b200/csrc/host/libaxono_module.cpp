// Python module `libaxono`: the binding surface of the reference's module for the decode path
// (axono/python/src/nanobind_module.cpp:185-372 Tensor/DataType/Status, :398-400 cache controls,
// :905-1210 operators, :1211-1324 CUDA graph), over this library's native runtime.  No PyTorch.
// Operators run on CUDA tensors only: a CPU tensor raises, there is no host fallback.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "axono_b200.h"
#include "axono_core.h"
#include "axono_ops.h"

namespace py = pybind11;
using axono::core::Context;
using axono::core::DataType;
using axono::core::Shape;
using axono::core::Status;
using axono::core::Tensor;
namespace acuda = axono::core::cuda;
namespace aops = axono::ops::cuda;

namespace {

[[noreturn]] void Fail(const char *op, Status st) {
  throw std::runtime_error(std::string(op) + " failed, status " + std::to_string(static_cast<int>(st)) +
                           " (device error bits " + std::to_string(axb200_last_error()) + ")");
}
void Check(const char *op, Status st) {
  if (st != Status::OK) Fail(op, st);
}
void NeedCuda(const char *op, const Tensor &t) {
  if (!t.is_cuda()) throw std::runtime_error(std::string(op) + ": CUDA tensors only (this build has no CPU operators)");
}

py::dtype NumpyDtype(DataType t) {
  switch (t) {
    case DataType::INT8: return py::dtype::of<int8_t>();
    case DataType::INT16: return py::dtype::of<int16_t>();
    case DataType::INT32: return py::dtype::of<int32_t>();
    case DataType::INT64: return py::dtype::of<int64_t>();
    case DataType::FLOAT16: return py::dtype("float16");
    case DataType::FLOAT32: return py::dtype::of<float>();
    case DataType::FLOAT64: return py::dtype::of<double>();
    case DataType::BOOLEAN: return py::dtype::of<bool>();
  }
  throw std::runtime_error("unknown dtype");
}

DataType FromNumpyDtype(const py::dtype &dt) {
  const char k = dt.kind();
  const auto sz = dt.itemsize();
  if (k == 'f' && sz == 2) return DataType::FLOAT16;
  if (k == 'f' && sz == 4) return DataType::FLOAT32;
  if (k == 'f' && sz == 8) return DataType::FLOAT64;
  if (k == 'i' && sz == 1) return DataType::INT8;
  if (k == 'i' && sz == 2) return DataType::INT16;
  if (k == 'i' && sz == 4) return DataType::INT32;
  if (k == 'i' && sz == 8) return DataType::INT64;
  if (k == 'u' && sz == 2) return DataType::FLOAT16;  // raw half bits, as the reference passes them
  if (k == 'b') return DataType::BOOLEAN;
  throw std::runtime_error("unsupported numpy dtype");
}

Shape ShapeOf(const py::array &a) {
  Shape s;
  for (py::ssize_t i = 0; i < a.ndim(); ++i) s.push_back(static_cast<size_t>(a.shape(i)));
  return s;
}

// A host copy of the tensor as a numpy array of its dtype (device tensors are read back).
py::array ToNumpy(const Tensor &t) {
  std::vector<py::ssize_t> shp(t.shape().begin(), t.shape().end());
  py::array out(NumpyDtype(t.dtype()), shp);
  if (t.num_bytes() == 0) return out;
  Tensor host = Tensor::FromBorrowed(t.dtype(), t.shape(), out.mutable_data());
  Check("numpy", host.CopyFrom(t));
  return out;
}

Tensor FromNumpy(const py::array &arr, const std::string &device) {
  py::array a = py::array::ensure(arr, py::array::c_style);
  if (!a) throw std::runtime_error("from_numpy: not an array");
  const DataType dt = FromNumpyDtype(a.dtype());
  Tensor host = Tensor::FromBorrowed(dt, ShapeOf(a), a.data());
  Tensor out(dt, ShapeOf(a), device);
  if (out.num_bytes()) Check("from_numpy", out.CopyFrom(host));
  return out;
}

template <typename T>
py::array Accessor(const Tensor &t, DataType want, const char *name) {
  if (t.dtype() != want) throw std::runtime_error(std::string(name) + ": tensor has another dtype");
  return ToNumpy(t);
}

struct Arena {
  axb200_kv_arena *h = nullptr;
  ~Arena() {
    if (h) axb200_kv_arena_destroy(h);
  }
};

}  // namespace

PYBIND11_MODULE(libaxono, m) {
  m.doc() = "Axono decode-path operators on B200 (native runtime, no PyTorch)";

  py::enum_<DataType>(m, "DataType")
      .value("INT8", DataType::INT8).value("INT16", DataType::INT16).value("INT32", DataType::INT32)
      .value("INT64", DataType::INT64).value("FLOAT16", DataType::FLOAT16).value("FLOAT32", DataType::FLOAT32)
      .value("FLOAT64", DataType::FLOAT64).value("BOOLEAN", DataType::BOOLEAN);
  py::enum_<Status>(m, "Status")
      .value("OK", Status::OK).value("INVALID_ARGUMENT", Status::INVALID_ARGUMENT)
      .value("OUT_OF_MEMORY", Status::OUT_OF_MEMORY).value("UNSUPPORTED_TYPE", Status::UNSUPPORTED_TYPE)
      .value("SHAPE_MISMATCH", Status::SHAPE_MISMATCH).value("INTERNAL_ERROR", Status::INTERNAL_ERROR)
      .value("DEVICE_ERROR", Status::DEVICE_ERROR).value("INVALID_PTR", Status::INVALID_PTR)
      .value("DEVICE_MISMATCH", Status::DEVICE_MISMATCH);

  py::class_<Tensor>(m, "Tensor")
      .def(py::init<>())
      .def(py::init<DataType>())
      .def(py::init<DataType, const Shape &>(), py::arg("dtype"), py::arg("shape"))
      .def(py::init<DataType, const Shape &, const std::string &>(), py::arg("dtype"), py::arg("shape"),
           py::arg("device"))
      .def_static("from_numpy", &FromNumpy, py::arg("array"), py::arg("device") = "cpu")
      .def_static(
          "from_borrowed",
          [](py::array arr) {
            if (!(arr.flags() & py::array::c_style)) throw std::runtime_error("from_borrowed: array must be C-contiguous");
            const DataType dt = FromNumpyDtype(arr.dtype());
            if (dt != DataType::FLOAT32 && dt != DataType::FLOAT16)
              throw std::runtime_error("from_borrowed: FLOAT32 / FLOAT16 only");
            return Tensor::FromBorrowed(dt, ShapeOf(arr), arr.data());
          },
          py::arg("array"), py::keep_alive<0, 1>())
      .def_static(
          "from_borrowed_i64",
          [](py::array arr) {
            if (!(arr.flags() & py::array::c_style) || FromNumpyDtype(arr.dtype()) != DataType::INT64)
              throw std::runtime_error("from_borrowed_i64: C-contiguous INT64 only");
            return Tensor::FromBorrowed(DataType::INT64, ShapeOf(arr), arr.data());
          },
          py::arg("array"), py::keep_alive<0, 1>())
      .def_static(
          "from_device_ptr",  // a view of device memory that somebody else owns (peer-mapped buffers, KV pools)
          [](uintptr_t ptr, DataType dtype, const Shape &shape, const std::string &device) {
            if (!ptr) throw std::runtime_error("from_device_ptr: null pointer");
            return Tensor::FromBorrowedDevice(dtype, shape, reinterpret_cast<void *>(ptr), device);
          },
          py::arg("ptr"), py::arg("dtype"), py::arg("shape"), py::arg("device") = "cuda")
      .def("to", &Tensor::to, py::arg("device"))
      .def("to_", &Tensor::to_, py::arg("device"))
      .def("copy_from", [](Tensor &self, const Tensor &src) { Check("copy_from", self.CopyFrom(src)); }, py::arg("src"))
      .def("copy_from_numpy",
           [](Tensor &self, const py::array &arr) {
             py::array a = py::array::ensure(arr, py::array::c_style);
             if (!a || FromNumpyDtype(a.dtype()) != self.dtype() || (size_t)a.size() != self.num_elements())
               throw std::runtime_error("copy_from_numpy: dtype or element count differs");
             Check("copy_from_numpy", self.CopyFrom(Tensor::FromBorrowed(self.dtype(), self.shape(), a.data())));
           },
           py::arg("array"))
      .def("reshape", &Tensor::Reshape)
      .def("resize", &Tensor::Resize)
      .def("fill_zero", &Tensor::FillZero)
      .def("is_same_shape", &Tensor::IsSameShape)
      .def("cast_to", &Tensor::CastTo)
      .def("_orig_cast_to", &Tensor::CastTo)
      .def_property_readonly("is_cuda", &Tensor::is_cuda)
      .def_property_readonly("device", &Tensor::device)
      .def_property_readonly("dtype", &Tensor::dtype)
      .def_property_readonly("shape", [](const Tensor &t) { return py::tuple(py::cast(t.shape())); })
      .def_property_readonly("ndim", &Tensor::ndim)
      .def_property_readonly("num_elements", &Tensor::num_elements)
      .def_property_readonly("num_bytes", &Tensor::num_bytes)
      .def_property_readonly("data_ptr", [](const Tensor &t) { return reinterpret_cast<uintptr_t>(t.data()); })
      .def("numpy", &ToNumpy)
      .def("to_numpy", &ToNumpy)
      .def("data_int8", [](const Tensor &t) { return Accessor<int8_t>(t, DataType::INT8, "data_int8"); })
      .def("data_int16", [](const Tensor &t) { return Accessor<int16_t>(t, DataType::INT16, "data_int16"); })
      .def("data_int32", [](const Tensor &t) { return Accessor<int32_t>(t, DataType::INT32, "data_int32"); })
      .def("data_int64", [](const Tensor &t) { return Accessor<int64_t>(t, DataType::INT64, "data_int64"); })
      .def("data_float16",  // raw bits as int16, viewed as float16 by the caller (as the reference exposes them)
           [](const Tensor &t) {
             if (t.dtype() != DataType::FLOAT16) throw std::runtime_error("data_float16: tensor is not FLOAT16");
             return ToNumpy(t).attr("view")(py::dtype::of<int16_t>());
           })
      .def("data_float32", [](const Tensor &t) { return Accessor<float>(t, DataType::FLOAT32, "data_float32"); })
      .def("data_float64", [](const Tensor &t) { return Accessor<double>(t, DataType::FLOAT64, "data_float64"); })
      .def("data_bool", [](const Tensor &t) { return Accessor<bool>(t, DataType::BOOLEAN, "data_bool"); })
      .def("__repr__", &Tensor::ToString)
      .def("__str__", &Tensor::ToString)
      .def("__copy__", [](const Tensor &t) { return Tensor(t); })
      .def("__deepcopy__", [](const Tensor &t, py::dict) {
        Tensor out(t.dtype(), t.shape(), t.device());
        if (t.num_bytes()) Check("deepcopy", out.CopyFrom(t));
        return out;
      });

  // ---- allocator controls ----
  m.def("cuda_available", &acuda::Available);
  m.def("cached_bytes", &acuda::GetCachedBytes);
  m.def("set_cache_budget", &acuda::SetCacheBudget, py::arg("bytes"));
  m.def("cache_budget", &acuda::GetCacheBudget);
  m.def("clear_cache", &acuda::ClearDeviceCache);
  m.def("mem_info", []() {  // (free, total) bytes of the current device
    size_t f = 0, t = 0;
    Check("mem_info", acuda::MemInfo(&f, &t));
    return py::make_tuple(f, t);
  });
  m.def("set_device", [](int index) { Check("set_device", acuda::SetDevice(index)); }, py::arg("index"));
  m.def("current_device", &acuda::CurrentDevice);
  m.def("device_pci_bus_id", &acuda::DevicePciBusId, py::arg("index"));
  m.def("synchronize", []() { Check("synchronize", acuda::DeviceSynchronize()); });
  m.def("current_stream", []() {  // cudaStream_t as an integer: 0 = legacy default stream, else the capture stream
    return reinterpret_cast<uintptr_t>(acuda::CurrentStream());
  });
  m.def("set_fused_merge", [](bool on) { axb200_set_fused_merge(on ? 1 : 0); }, py::arg("on"));
  m.def("set_wait_limit_ns", [](uint64_t ns) { Check("set_wait_limit_ns", static_cast<Status>(axb200_set_wait_limit_ns(ns))); },
        py::arg("ns"));
  m.def("profile_enable", [](bool on) { Check("profile_enable", static_cast<Status>(axb200_profile_enable(on ? 1 : 0))); },
        py::arg("on"));
  m.def("profile_collect", []() {  // (summed milliseconds of the split kernel, launches) since the last collect
    double ms = 0.0;
    int launches = 0;
    Check("profile_collect", static_cast<Status>(axb200_profile_collect(&ms, &launches)));
    return py::make_tuple(ms, launches);
  });
  m.def(
      "pinned_empty",  // a numpy array in page-locked host memory (asynchronous copies need it)
      [](const std::vector<py::ssize_t> &shape, DataType dtype) {
        size_t n = 1;
        for (auto d : shape) n *= (size_t)d;
        void *p = acuda::AllocatePinnedHost(n * axono::core::GetDataTypeSize(dtype));
        if (!p) throw std::runtime_error("pinned_empty: allocation failed");
        py::capsule owner(p, [](void *q) { acuda::FreePinnedHost(q); });
        return py::array(NumpyDtype(dtype), shape, p, owner);
      },
      py::arg("shape"), py::arg("dtype"));
  m.def(
      "randn",  // seeded N(mean, std) on the device; values depend only on (seed, element index)
      [](const Shape &shape, DataType dtype, const std::string &device, uint64_t seed, float mean, float stddev) {
        Tensor out = Tensor::Uninitialized(dtype, shape, device);
        Check("randn", static_cast<Status>(axb200_randn(out.data(), (int64_t)out.num_elements(), static_cast<int>(dtype), mean,
                                                        stddev, seed, acuda::CurrentStream())));
        return out;
      },
      py::arg("shape"), py::arg("dtype"), py::arg("device") = "cuda", py::arg("seed") = 0, py::arg("mean") = 0.f,
      py::arg("std") = 1.f);
  py::class_<acuda::EventTimer>(m, "EventTimer")
      .def(py::init<>())
      .def("start", [](acuda::EventTimer &t) { Check("EventTimer.start", t.Start()); })
      .def("stop", [](acuda::EventTimer &t) { Check("EventTimer.stop", t.Stop()); })
      .def("elapsed_ms", [](acuda::EventTimer &t) {
        float ms = 0.f;
        Check("EventTimer.elapsed_ms", t.ElapsedMs(&ms));
        return ms;
      });
  m.def("device_error_bits", []() { return axb200_last_error(); });
  m.def("version", []() { return std::string(axb200_version()); });

  // ---- operators ----
  m.def("gqa_decode_attention",
        [](const Tensor &q, const Tensor &k, const Tensor &v) {
          Tensor result = Tensor::Uninitialized(q.dtype(), q.shape(), q.device());
          Check("gqa_decode_attention", aops::GqaDecodeAttention(Context(), q, k, v, result));
          return result;
        },
        py::arg("q"), py::arg("k"), py::arg("v"));
  m.def("scaled_dot_product_attention",
        [](const Tensor &q, const Tensor &k, const Tensor &v, bool is_causal) {
          NeedCuda("scaled_dot_product_attention", q);
          Tensor result = Tensor::Uninitialized(q.dtype(), q.shape(), q.device());
          Check("scaled_dot_product_attention", aops::ScaledDotProductAttention(Context(), q, k, v, is_causal, result));
          return result;
        },
        py::arg("q"), py::arg("k"), py::arg("v"), py::arg("is_causal") = false);
  m.def("silu_mul",
        [](const Tensor &gate, const Tensor &up) {
          NeedCuda("silu_mul", gate);
          Tensor result = Tensor::Uninitialized(gate.dtype(), gate.shape(), gate.device());
          Check("silu_mul", aops::SiluMul(Context(), gate, up, result));
          return result;
        },
        py::arg("gate"), py::arg("up"));
  m.def("add_rms_norm",
        [](const Tensor &x, const Tensor &residual, const Tensor &weight, float eps) {
          NeedCuda("add_rms_norm", x);
          Tensor y = Tensor::Uninitialized(x.dtype(), x.shape(), x.device()), out = Tensor::Uninitialized(x.dtype(), x.shape(), x.device());
          Check("add_rms_norm", aops::AddRmsNorm(Context(), x, residual, weight, eps, y, out));
          return py::make_tuple(y, out);
        },
        py::arg("x"), py::arg("residual"), py::arg("weight"), py::arg("eps"));
  m.def("rms_norm",
        [](const Tensor &x, const Tensor &weight, float eps) {
          NeedCuda("rms_norm", x);
          if (x.is_cuda() != weight.is_cuda() || x.dtype() != weight.dtype())
            throw std::runtime_error("rms_norm: inputs differ in device or dtype");
          Tensor result = Tensor::Uninitialized(x.dtype(), x.shape(), x.device());
          Check("rms_norm", aops::RmsNorm(Context(), x, weight, eps, result));
          return result;
        },
        py::arg("x"), py::arg("weight"), py::arg("eps") = 1e-5f);
  m.def("rope",
        [](const Tensor &x, const Tensor &pos_ids, float theta) {
          NeedCuda("rope", x);
          Tensor result = Tensor::Uninitialized(x.dtype(), x.shape(), x.device());
          Check("rope", aops::Rope(Context(), x, pos_ids, theta, result));
          return result;
        },
        py::arg("x"), py::arg("pos_ids"), py::arg("theta"));
  m.def("rope_with_cos_sin",
        [](const Tensor &x, const Tensor &cos, const Tensor &sin) {
          NeedCuda("rope_with_cos_sin", x);
          Tensor result = Tensor::Uninitialized(x.dtype(), x.shape(), x.device());
          Check("rope_with_cos_sin", aops::RopeWithCosSin(Context(), x, cos, sin, result));
          return result;
        },
        py::arg("x"), py::arg("cos"), py::arg("sin"));
  m.def("rope_thd",
        [](const Tensor &x, const Tensor &pos, const Tensor &inv_freq, int t_sec, int h_sec, int w_sec) {
          NeedCuda("rope_thd", x);
          Tensor result = Tensor::Uninitialized(x.dtype(), x.shape(), x.device());
          Check("rope_thd", aops::RopeThd(Context(), x, pos, inv_freq, t_sec, h_sec, w_sec, result));
          return result;
        },
        py::arg("x"), py::arg("pos"), py::arg("inv_freq"), py::arg("t_sec"), py::arg("h_sec"), py::arg("w_sec"));
  m.def("mrope_cos_sin",
        [](const Tensor &pos, const Tensor &inv_freq, int h_sec, int w_sec) {
          NeedCuda("mrope_cos_sin", pos);
          Tensor cos_out = Tensor::Uninitialized(DataType::FLOAT32, {}, pos.device()), sin_out = Tensor::Uninitialized(DataType::FLOAT32, {}, pos.device());
          Check("mrope_cos_sin", aops::MropeCosSin(Context(), pos, inv_freq, h_sec, w_sec, cos_out, sin_out));
          return py::make_tuple(cos_out, sin_out);
        },
        py::arg("pos"), py::arg("inv_freq"), py::arg("h_sec"), py::arg("w_sec"));
  m.def("concat",
        [](const Tensor &a, const Tensor &b, int axis) {
          NeedCuda("concat", a);
          if (a.is_cuda() != b.is_cuda() || a.dtype() != b.dtype())
            throw std::runtime_error("concat: inputs differ in device or dtype");
          Tensor result = Tensor::Uninitialized(a.dtype(), {}, a.device());
          Check("concat", aops::Concat(Context(), a, b, axis, result));
          return result;
        },
        py::arg("a"), py::arg("b"), py::arg("axis"));
  m.def("embedding",
        [](const Tensor &ids, const Tensor &table) {
          NeedCuda("embedding", table);
          if (ids.is_cuda() != table.is_cuda()) throw std::runtime_error("embedding: inputs are on different devices");
          Tensor result = Tensor::Uninitialized(table.dtype(), {}, table.device());
          Check("embedding", aops::Embedding(Context(), ids, table, result));
          return result;
        },
        py::arg("ids"), py::arg("table"));
  m.def("argmax",
        [](const Tensor &x) {
          NeedCuda("argmax", x);
          Tensor result = Tensor::Uninitialized(DataType::INT64, {}, x.device());
          Check("argmax", aops::ArgmaxLastDim(Context(), x, result));
          return result;
        },
        py::arg("x"));

  m.def("linear_nobias",
        [](const Tensor &x, const Tensor &w) {
          Tensor result = Tensor::Uninitialized(x.dtype(), {}, x.device());
          Check("linear_nobias", aops::LinearNoBias(Context(), x, w, result));
          return result;
        },
        py::arg("x"), py::arg("weight"));
  m.def("silu_mul_rows",
        [](const Tensor &gate_up, int n) {
          NeedCuda("silu_mul_rows", gate_up);
          Tensor result = Tensor::Uninitialized(gate_up.dtype(), {}, gate_up.device());
          Check("silu_mul_rows", aops::SiluMulRows(Context(), gate_up, n, result));
          return result;
        },
        py::arg("gate_up"), py::arg("n"));

  // ---- paged KV arena (new operators) ----
  py::class_<Arena>(m, "KVArena")
      .def(py::init([](int n_layers, int num_pages, int hkv, int page_tokens, int d, DataType dtype, int max_seqs,
                       int max_blocks) {
             auto a = std::make_unique<Arena>();
             Check("KVArena", static_cast<Status>(axb200_kv_arena_create(n_layers, num_pages, hkv, page_tokens, d,
                                                                         static_cast<int>(dtype), max_seqs, max_blocks,
                                                                         1, &a->h)));
             return a;
           }),
           py::arg("n_layers"), py::arg("num_pages"), py::arg("hkv"), py::arg("page_tokens"), py::arg("d"),
           py::arg("dtype"), py::arg("max_seqs"), py::arg("max_blocks"))
      .def("alloc_seq",
           [](Arena &a, int64_t reserve_tokens) {
             int id = -1;
             Check("alloc_seq", static_cast<Status>(axb200_kv_arena_alloc_seq(a.h, reserve_tokens, &id)));
             return id;
           },
           py::arg("reserve_tokens"))
      .def("reserve", [](Arena &a, int seq, int64_t tokens) {
        Check("reserve", static_cast<Status>(axb200_kv_arena_reserve(a.h, seq, tokens)));
      })
      .def("free_seq", [](Arena &a, int seq) {
        Check("free_seq", static_cast<Status>(axb200_kv_arena_free_seq(a.h, seq, acuda::CurrentStream())));
      })
      .def("sync", [](Arena &a) { Check("sync", static_cast<Status>(axb200_kv_arena_sync(a.h, acuda::CurrentStream()))); })
      .def("stats",
           [](Arena &a) {
             int64_t total, free_pages, live, bytes;
             Check("stats", static_cast<Status>(axb200_kv_arena_stats(a.h, &total, &free_pages, &live, &bytes)));
             py::dict d;
             d["pages_total"] = total;
             d["pages_free"] = free_pages;
             d["seqs_live"] = live;
             d["device_bytes"] = bytes;
             return d;
           })
      .def_property_readonly("handle", [](Arena &a) { return reinterpret_cast<uintptr_t>(a.h); })
      .def("geometry",
           [](Arena &a) {
             int nl, np, hkv, pt, d, dt, ms, mb;
             axb200_kv_arena_geometry(a.h, &nl, &np, &hkv, &pt, &d, &dt, &ms, &mb);
             py::dict g;
             g["n_layers"] = nl; g["num_pages"] = np; g["hkv"] = hkv; g["page_tokens"] = pt; g["d"] = d;
             g["dtype"] = static_cast<DataType>(dt); g["max_seqs"] = ms; g["max_blocks"] = mb;
             return g;
           })
      .def("k_pages_ptr", [](Arena &a, int layer) { return reinterpret_cast<uintptr_t>(axb200_kv_arena_k_pages(a.h, layer)); })
      .def("v_pages_ptr", [](Arena &a, int layer) { return reinterpret_cast<uintptr_t>(axb200_kv_arena_v_pages(a.h, layer)); })
      .def_property_readonly("block_table_ptr", [](Arena &a) { return reinterpret_cast<uintptr_t>(axb200_kv_arena_block_table(a.h)); })
      .def_property_readonly("seq_lens_ptr", [](Arena &a) { return reinterpret_cast<uintptr_t>(axb200_kv_arena_seq_lens(a.h)); })
      .def("shuffle_free", [](Arena &a, uint64_t seed) {
        Check("shuffle_free", static_cast<Status>(axb200_kv_arena_shuffle_free(a.h, seed)));
      }, py::arg("seed"))
      .def("fill_normal",  // every K and V pool of every layer <- std * N(0,1), seeded per pool
           [](Arena &a, uint64_t seed, float stddev) {
             int nl, np, hkv, pt, d, dt, ms, mb;
             axb200_kv_arena_geometry(a.h, &nl, &np, &hkv, &pt, &d, &dt, &ms, &mb);
             const int64_t n = (int64_t)np * hkv * pt * d;
             for (int l = 0; l < nl; ++l)
               for (int kv = 0; kv < 2; ++kv)
                 Check("fill_normal", static_cast<Status>(axb200_randn(
                                          kv ? axb200_kv_arena_v_pages(a.h, l) : axb200_kv_arena_k_pages(a.h, l), n, dt, 0.f,
                                          stddev, seed * 1000003ull + (uint64_t)(2 * l + kv), acuda::CurrentStream())));
           },
           py::arg("seed"), py::arg("std") = 1.f)
      .def("gather",  // the first n cached tokens of one sequence as token-major (n, hkv, d) host arrays (for checks)
           [](Arena &a, int layer, int seq, int64_t n) {
             int nl, np, hkv, pt, d, dt, ms, mb;
             axb200_kv_arena_geometry(a.h, &nl, &np, &hkv, &pt, &d, &dt, &ms, &mb);
             if (layer < 0 || layer >= nl || n < 0) throw std::runtime_error("gather: bad layer or length");
             std::vector<int32_t> pages(mb);
             const int have = axb200_kv_arena_seq_pages(a.h, seq, pages.data(), mb);
             if (have < 0 || (int64_t)have * pt < n) throw std::runtime_error("gather: the sequence holds fewer pages");
             const size_t es = dt == static_cast<int>(DataType::FLOAT16) ? 2 : 4;
             const DataType dtype = static_cast<DataType>(dt);
             std::vector<py::ssize_t> shp{(py::ssize_t)n, hkv, d};
             py::array k_out(NumpyDtype(dtype), shp), v_out(NumpyDtype(dtype), shp);
             std::vector<char> page((size_t)hkv * pt * d * es);
             for (int kv = 0; kv < 2; ++kv) {
               const char *pool = static_cast<const char *>(kv ? axb200_kv_arena_v_pages(a.h, layer) : axb200_kv_arena_k_pages(a.h, layer));
               char *dst = static_cast<char *>(kv ? v_out.mutable_data() : k_out.mutable_data());
               for (int64_t blk = 0; blk * pt < n; ++blk) {
                 Check("gather", acuda::CopyToHost(page.data(), pool + (size_t)pages[blk] * page.size(), page.size()));
                 const int64_t toks = std::min<int64_t>(pt, n - blk * pt);
                 for (int64_t t = 0; t < toks; ++t)
                   for (int h = 0; h < hkv; ++h)
                     std::memcpy(dst + (((blk * pt + t) * hkv + h) * d) * es, page.data() + (((size_t)h * pt + t) * d) * es, d * es);
               }
             }
             return py::make_tuple(k_out, v_out);
           },
           py::arg("layer"), py::arg("seq"), py::arg("n"))
      .def("fill_pages",  // every K and V pool of every layer <- repetitions of `chunk` (benchmarks: non-zero cache contents)
           [](Arena &a, py::array chunk) {
             int nl, np, hkv, pt, d, dt, ms, mb;
             axb200_kv_arena_geometry(a.h, &nl, &np, &hkv, &pt, &d, &dt, &ms, &mb);
             py::array c = py::array::ensure(chunk, py::array::c_style);
             const size_t es = dt == static_cast<int>(DataType::FLOAT16) ? 2 : 4;
             const size_t pool = (size_t)np * hkv * pt * d * es, cb = (size_t)c.nbytes();
             if (!c || (size_t)c.itemsize() != es || cb == 0 || cb > pool) throw std::runtime_error("fill_pages: bad chunk");
             for (int l = 0; l < nl; ++l)
               for (int kv = 0; kv < 2; ++kv) {
                 char *base = static_cast<char *>(kv ? axb200_kv_arena_v_pages(a.h, l) : axb200_kv_arena_k_pages(a.h, l));
                 Check("fill_pages", acuda::CopyToDevice(base, c.data(), cb));
                 for (size_t have = cb; have < pool; have *= 2)  // doubling device-to-device copies
                   Check("fill_pages", acuda::CopyOnDevice(base + have, base, std::min(have, pool - have)));
               }
           },
           py::arg("chunk"))
      .def("set_seq_lens",  // overwrites the device-side lengths (a cache filled by other means, tests, benchmarks)
           [](Arena &a, py::array_t<int32_t, py::array::c_style | py::array::forcecast> lens) {
             int nl, np, hkv, pt, d, dt, ms, mb;
             axb200_kv_arena_geometry(a.h, &nl, &np, &hkv, &pt, &d, &dt, &ms, &mb);
             if (lens.size() != ms) throw std::runtime_error("set_seq_lens: one length per sequence slot");
             for (py::ssize_t i = 0; i < lens.size(); ++i)
               if (lens.data()[i] < 0 || lens.data()[i] > (int64_t)mb * pt) throw std::runtime_error("set_seq_lens: length out of range");
             Check("set_seq_lens", acuda::CopyToDevice(axb200_kv_arena_seq_lens(a.h), lens.data(), ms * sizeof(int32_t)));
           },
           py::arg("lens"))
      .def("seq_lens", [](Arena &a) {  // host copy of the device-side lengths
        int nl, np, hkv, pt, d, dt, ms, mb;
        axb200_kv_arena_geometry(a.h, &nl, &np, &hkv, &pt, &d, &dt, &ms, &mb);
        py::array_t<int32_t> out(ms);
        Check("seq_lens", acuda::CopyToHost(out.mutable_data(), axb200_kv_arena_seq_lens(a.h), ms * sizeof(int32_t)));
        return out;
      });
  m.def("kv_append_rope",
        [](Arena &arena, int layer, py::object q, const Tensor &k_new, const Tensor &v_new, py::object pos,
           py::object inv_freq, float theta, bool rotate, py::object mrope_section, int slot_delta, bool advance) {
          Tensor *qp = q.is_none() ? nullptr : q.cast<Tensor *>();
          const Tensor *pp = pos.is_none() ? nullptr : pos.cast<const Tensor *>();
          const Tensor *fp = inv_freq.is_none() ? nullptr : inv_freq.cast<const Tensor *>();
          int h_sec = 0, w_sec = 0;
          const bool mrope = !mrope_section.is_none();
          if (mrope) {
            auto sec = mrope_section.cast<std::vector<int>>();
            if (sec.size() != 3) throw std::runtime_error("mrope_section: (t, h, w)");
            h_sec = sec[1];
            w_sec = sec[2];
          }
          Check("kv_append_rope", aops::KvAppendRope(Context(), qp, k_new, v_new, arena.h, layer, pp, fp, theta, rotate,
                                                     mrope, h_sec, w_sec, slot_delta, advance));
        },
        py::arg("arena"), py::arg("layer"), py::arg("q"), py::arg("k_new"), py::arg("v_new"),
        py::arg("pos") = py::none(), py::arg("inv_freq") = py::none(), py::arg("theta") = 1e6f,
        py::arg("rotate") = true, py::arg("mrope_section") = py::none(), py::arg("slot_delta") = 0,
        py::arg("advance") = true);
  m.def("qkv_norm_rope_append",
        [](Arena &arena, int layer, const Tensor &qkv, int hq, py::object q_norm_w, py::object k_norm_w, float eps,
           py::object pos, py::object inv_freq, float theta, bool rotate, py::object mrope_section, int slot_delta,
           bool advance) {
          const Tensor *qn = q_norm_w.is_none() ? nullptr : q_norm_w.cast<const Tensor *>();
          const Tensor *kn = k_norm_w.is_none() ? nullptr : k_norm_w.cast<const Tensor *>();
          const Tensor *pp = pos.is_none() ? nullptr : pos.cast<const Tensor *>();
          const Tensor *fp = inv_freq.is_none() ? nullptr : inv_freq.cast<const Tensor *>();
          int h_sec = 0, w_sec = 0;
          const bool mrope = !mrope_section.is_none();
          if (mrope) {
            auto sec = mrope_section.cast<std::vector<int>>();
            if (sec.size() != 3) throw std::runtime_error("mrope_section: (t, h, w)");
            h_sec = sec[1];
            w_sec = sec[2];
          }
          Tensor q_out = Tensor::Uninitialized(qkv.dtype(), {}, qkv.device());
          Check("qkv_norm_rope_append",
                aops::QkvNormRopeAppend(Context(), qkv, hq, qn, kn, eps, arena.h, layer, pp, fp, theta, rotate, mrope,
                                        h_sec, w_sec, slot_delta, advance, q_out));
          return q_out;
        },
        py::arg("arena"), py::arg("layer"), py::arg("qkv"), py::arg("hq"), py::arg("q_norm_w") = py::none(),
        py::arg("k_norm_w") = py::none(), py::arg("eps") = 1e-6f, py::arg("pos") = py::none(),
        py::arg("inv_freq") = py::none(), py::arg("theta") = 1e6f, py::arg("rotate") = true,
        py::arg("mrope_section") = py::none(), py::arg("slot_delta") = 0, py::arg("advance") = true);
  m.def("gqa_decode_attention_paged",
        [](const Tensor &q, Arena &arena, int layer, int64_t max_seq_len, py::object out) {
          Tensor result = out.is_none() ? Tensor::Uninitialized(q.dtype(), q.shape(), q.device()) : out.cast<Tensor>();
          if (!out.is_none() && (result.dtype() != q.dtype() || result.shape() != q.shape() || result.device() != q.device()))
            throw std::runtime_error("gqa_decode_attention_paged: out must match q in dtype, shape and device");
          Check("gqa_decode_attention_paged", aops::GqaDecodeAttentionPaged(Context(), q, arena.h, layer, max_seq_len, result));
          return result;
        },
        py::arg("q"), py::arg("arena"), py::arg("layer"), py::arg("max_seq_len"), py::arg("out") = py::none());
  m.def("decode_step_paged",  // rope(q), rope(k_new), append, attention: one operator, one launch where the library can
        [](const Tensor &q, const Tensor &k_new, const Tensor &v_new, Arena &arena, int layer, int64_t max_seq_len,
           py::object out, py::object pos, py::object inv_freq, float theta, bool rotate, py::object mrope_section) {
          const Tensor *pp = pos.is_none() ? nullptr : pos.cast<const Tensor *>();
          const Tensor *fp = inv_freq.is_none() ? nullptr : inv_freq.cast<const Tensor *>();
          int h_sec = 0, w_sec = 0;
          const bool mrope = !mrope_section.is_none();
          if (mrope) {
            auto sec = mrope_section.cast<std::vector<int>>();
            if (sec.size() != 3) throw std::runtime_error("mrope_section: (t, h, w)");
            h_sec = sec[1];
            w_sec = sec[2];
          }
          Tensor result = out.is_none() ? Tensor::Uninitialized(q.dtype(), q.shape(), q.device()) : out.cast<Tensor>();
          if (!out.is_none() && (result.dtype() != q.dtype() || result.shape() != q.shape() || result.device() != q.device()))
            throw std::runtime_error("decode_step_paged: out must match q in dtype, shape and device");
          Check("decode_step_paged", aops::DecodeStepPaged(Context(), q, k_new, v_new, arena.h, layer, pp, fp, theta, rotate,
                                                           mrope, h_sec, w_sec, max_seq_len, result));
          return result;
        },
        py::arg("q"), py::arg("k_new"), py::arg("v_new"), py::arg("arena"), py::arg("layer"), py::arg("max_seq_len"),
        py::arg("out") = py::none(), py::arg("pos") = py::none(), py::arg("inv_freq") = py::none(),
        py::arg("theta") = 1e6f, py::arg("rotate") = true, py::arg("mrope_section") = py::none());
  m.def("decode_step_launches", [](int batch, int hq, int hkv, int d, int64_t max_seq_len, DataType dtype) {
    return axb200_decode_step_launches(batch, hq, hkv, d, max_seq_len, static_cast<int>(dtype));
  });
  m.def("set_step_fused", [](bool on) { axb200_set_step_fused(on ? 1 : 0); }, py::arg("on"));
  m.def(
      "decode_step_host",  // one decode step with HOST activations (pinned arrays): copies in, rope + append, attention, copy out, wait
      [](Arena &arena, int layer, py::array q_host, py::array k_host, py::array v_host, py::array out_host, Tensor &q_dev,
         Tensor &k_dev, Tensor &v_dev, Tensor &out_dev, Tensor &scratch, int64_t max_seq_len, float theta) {
        int nl, np, hkv, pt, d, dt, ms, mb;
        axb200_kv_arena_geometry(arena.h, &nl, &np, &hkv, &pt, &d, &dt, &ms, &mb);
        if (q_dev.ndim() != 3 || (int)q_dev.shape()[0] != ms || (int)q_dev.shape()[2] != d || k_dev.ndim() != 3 ||
            (int)k_dev.shape()[1] != hkv || static_cast<int>(q_dev.dtype()) != dt || layer < 0 || layer >= nl)
          throw std::runtime_error("decode_step_host: staging tensors do not match the arena");
        const size_t qb = q_dev.num_bytes(), kb = k_dev.num_bytes();
        if ((size_t)q_host.nbytes() != qb || (size_t)out_host.nbytes() != qb || (size_t)k_host.nbytes() != kb ||
            (size_t)v_host.nbytes() != kb || v_dev.num_bytes() != kb || out_dev.num_bytes() != qb)
          throw std::runtime_error("decode_step_host: host and staging buffers differ in size");
        const int hq = (int)q_dev.shape()[1];
        Check("decode_step_host",
              static_cast<Status>(axb200_decode_step_host(
                  q_host.data(), k_host.data(), v_host.data(), out_host.mutable_data(), q_dev.data(), k_dev.data(), v_dev.data(),
                  out_dev.data(), axb200_kv_arena_k_pages(arena.h, layer), axb200_kv_arena_v_pages(arena.h, layer),
                  axb200_kv_arena_block_table(arena.h), axb200_kv_arena_seq_lens(arena.h), nullptr, nullptr, theta, 1, 0, 0, 0,
                  ms, hq, hkv, d, pt, mb, np, max_seq_len, dt, scratch.data(), scratch.num_bytes(), acuda::CurrentStream())));
      },
      py::arg("arena"), py::arg("layer"), py::arg("q_host"), py::arg("k_new_host"), py::arg("v_new_host"), py::arg("out_host"),
      py::arg("q_dev"), py::arg("k_new_dev"), py::arg("v_new_dev"), py::arg("out_dev"), py::arg("scratch"),
      py::arg("max_seq_len"), py::arg("theta") = 1e6f);
  m.def("gqa_workspace_bytes", [](int batch, int hq, int hkv, int d, int64_t max_seq_len, DataType dtype) {
    return axb200_gqa_workspace_bytes(batch, hq, hkv, d, max_seq_len, static_cast<int>(dtype));
  });

  // ---- CUDA graph ----
  m.def("_graph_begin_capture", []() {
    acuda::DeviceSynchronize();  // the capture stream does not order against work already submitted
    void *stream = nullptr;
    if (acuda::BeginGraphCapture(&stream) != Status::OK) throw std::runtime_error("_graph_begin_capture failed");
    return reinterpret_cast<intptr_t>(stream);
  });
  m.def("_graph_end_capture", [](intptr_t handle, acuda::GraphExec &exec) {
    if (acuda::EndGraphCapture(reinterpret_cast<void *>(handle), &exec) != Status::OK)
      throw std::runtime_error("_graph_end_capture: the body made an illegal call (sync / H2D / allocation) or launched nothing");
  });
  m.def("_graph_abort_capture", [](intptr_t handle) { acuda::AbortGraphCapture(reinterpret_cast<void *>(handle)); });

  py::class_<acuda::GraphExec>(m, "CUDAGraph")
      .def(py::init<>())
      .def("capture",
           [](acuda::GraphExec &self, py::function fn) {
             // 1) warm-up in recording mode: every device allocation enters the capture pool
             acuda::ResetCapturePool();
             acuda::SetCapturePoolRecording(true);
             try {
               fn();
             } catch (...) {
               acuda::SetCapturePoolRecording(false);
               throw;
             }
             acuda::SetCapturePoolRecording(false);
             acuda::DeviceSynchronize();
             // 2) capture: same-size allocations hit the pool in order, addresses repeat
             void *stream = nullptr;
             if (acuda::BeginGraphCapture(&stream) != Status::OK) throw std::runtime_error("CUDAGraph.capture: begin failed");
             try {
               fn();
             } catch (...) {
               acuda::AbortGraphCapture(stream);
               throw;
             }
             if (acuda::EndGraphCapture(stream, &self) != Status::OK)
               throw std::runtime_error("CUDAGraph.capture: the body made an illegal call (sync / allocation / H2D copy) or launched nothing");
           },
           py::arg("fn"))
      .def("replay", [](acuda::GraphExec &self) {
        if (self.Replay() != Status::OK) throw std::runtime_error("CUDAGraph.replay: not captured, or the launch failed");
      })
      .def("sync", [](acuda::GraphExec &self) {
        if (self.Sync() != Status::OK) throw std::runtime_error("CUDAGraph.sync failed");
      })
      .def("replay_timed",  // `times` launches between two CUDA events on the capture stream: ms per launch
           [](acuda::GraphExec &self, int times) {
             float ms = 0.f;
             if (self.ReplayTimed(times, &ms) != Status::OK) throw std::runtime_error("CUDAGraph.replay_timed failed");
             return ms;
           },
           py::arg("times"))
      .def("reset", [](acuda::GraphExec &self) {
        self.Reset();
        acuda::ResetCapturePool();
      })
      .def_property_readonly("is_captured", &acuda::GraphExec::IsCaptured)
      .def_property_readonly("num_nodes", &acuda::GraphExec::NumNodes);
}
