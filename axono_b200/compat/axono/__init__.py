"""`axono` as the decode path sees it, served by the B200 library's native module.  Names, argument
order and defaults follow the reference package (axono/python/axono/__init__.py and the modules it
re-exports); see axono_b200.compat for what is and is not covered."""
from __future__ import annotations

import numpy as np

from axono_b200 import native as _native

_l = _native.load()

DataType, Status, Tensor = _l.DataType, _l.Status, _l.Tensor
CUDAGraph, cuda_graph, compile = _native.CUDAGraph, _native.cuda_graph, _native.compile  # noqa: A001
cuda_available = _l.cuda_available
cached_bytes, set_cache_budget = _l.cached_bytes, _l.set_cache_budget

_DEFAULT_DEVICE = "cpu"


def set_default_device(device: str) -> None:
    """Device of tensors made by Tensor.from_numpy / zeros / ones / full when none is given:
    "cpu" | "cuda" | "cuda:<id>" (axono/python/axono/core/tensor.py:45-66)."""
    global _DEFAULT_DEVICE
    if device != "cpu" and not device.startswith("cuda"):
        raise ValueError(f"unknown device {device!r}")
    if device.startswith("cuda") and not cuda_available():
        raise RuntimeError("no CUDA device")
    _DEFAULT_DEVICE = device


def get_default_device() -> str:
    return _DEFAULT_DEVICE


def set_backend(name: str) -> None:
    """"cuda" or "cpu": the reference's global switch (core/backend.py).  Host tensors can be made and
    moved under "cpu", but this library has no CPU operators."""
    set_default_device("cuda" if name == "cuda" else "cpu")


def get_backend() -> str:
    return "cuda" if _DEFAULT_DEVICE.startswith("cuda") else "cpu"


# ---- conveniences the reference attaches to the bound Tensor class (core/tensor.py:108-470) ----
_NP_OF = {DataType.INT8: np.int8, DataType.INT16: np.int16, DataType.INT32: np.int32, DataType.INT64: np.int64,
          DataType.FLOAT16: np.float16, DataType.FLOAT32: np.float32, DataType.FLOAT64: np.float64,
          DataType.BOOLEAN: np.bool_}


if not hasattr(_l, "_native_from_numpy"):  # keep the bound constructor: the name is re-pointed below
    _l._native_from_numpy = _l.Tensor.from_numpy


def _from_numpy(array, device=None):
    array = np.ascontiguousarray(array)
    if array.dtype.type not in _NP_OF.values():
        array = array.astype(np.float32)
    return _l._native_from_numpy(array, device or _DEFAULT_DEVICE)


def _to_numpy(self):
    # FLOAT16 comes back as raw int16 bits, to be viewed as float16 by the caller, as in the reference
    return self.data_float16() if self.dtype == DataType.FLOAT16 else self.numpy()


def _full(shape, value, dtype=DataType.FLOAT32, device=None):
    return _from_numpy(np.full(tuple(shape), value, dtype=_NP_OF[dtype]), device)


def _fill(self, value):
    self.copy_from_numpy(np.full(tuple(self.shape), value, dtype=_NP_OF[self.dtype]))
    return self


def _randn(shape, dtype=DataType.FLOAT32, device=None, mean=0.0, stddev=1.0):
    a = np.random.standard_normal(tuple(shape)).astype(np.float32) * stddev + mean
    return _from_numpy(a.astype(_NP_OF[dtype]), device)


Tensor.from_numpy = staticmethod(_from_numpy)
Tensor.to_numpy = _to_numpy
Tensor.fill = _fill
Tensor.full = staticmethod(_full)
Tensor.zeros = staticmethod(lambda shape, dtype=DataType.FLOAT32, device=None: _full(shape, 0, dtype, device))
Tensor.ones = staticmethod(lambda shape, dtype=DataType.FLOAT32, device=None: _full(shape, 1, dtype, device))
Tensor.randn = staticmethod(_randn)
Tensor.create_like = staticmethod(lambda other: _l.Tensor(other.dtype, list(other.shape), other.device))


# ---- operators of the path (core/ops/sequence.py:17-75, core/ops/llm.py:99-109, gqa.py, fused.py) ----
def gqa_decode_attention(q, k, v):
    return _l.gqa_decode_attention(q, k, v)


def rope(x, pos_ids, theta: float = 10000.0):
    return _l.rope(x, pos_ids, theta)


def rope_with_cos_sin(x, cos, sin):
    return _l.rope_with_cos_sin(x, cos, sin)


def rope_thd(x, pos, inv_freq, mrope_section):
    t_sec, h_sec, w_sec = (list(mrope_section) + [0, 0, 0])[:3]
    return _l.rope_thd(x, pos, inv_freq, int(t_sec), int(h_sec), int(w_sec))


def mrope_cos_sin(pos, inv_freq, h_sec: int, w_sec: int):
    return _l.mrope_cos_sin(pos, inv_freq, h_sec, w_sec)


def scaled_dot_product_attention(q, k, v, is_causal: bool = False):
    return _l.scaled_dot_product_attention(q, k, v, is_causal)


def embedding(ids, table):
    return _l.embedding(ids, table)


def concat(a, b, axis: int):
    return _l.concat(a, b, axis)


def argmax(x):
    return _l.argmax(x)


def rms_norm(x, weight, eps: float = 1e-5):
    return _l.rms_norm(x, weight, eps)


from . import fused, gqa, nn  # noqa: E402,F401
