"""CPU checkers for the decode hot path.  TEST INFRASTRUCTURE ONLY.

Two interchangeable numpy front ends over two shared libraries:

* ``port()``      - ``oracle/_build/libaxono_oracle.so``: the plain-C restatement
  (``axono_oracle.c``) of the reference's CPU operators;
* ``reference()`` - ``oracle/_ref/libaxono_ref_cpu.so``: the reference's own CPU
  sources compiled in place plus ``ref_shim.cpp`` (present only where it was built).

Only the tests, ``__graft_entry__.smoke()`` and the benchmark's CPU-baseline leg may
import this package; the product (``axono_b200``) never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_LIB = os.path.join(_HERE, "_build", "libaxono_oracle.so")
REF_LIB = os.path.join(_HERE, "_ref", "libaxono_ref_cpu.so")
REF_CUDA_LIB = os.path.join(_HERE, "_ref", "libaxono_ref_cuda.so")

_sz = C.c_size_t
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i64p = np.ctypeslib.ndpointer(np.int64, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")


def build(ref_root: str = "") -> None:
    """Compile the C restatement, and the reference libraries when its sources are present (their
    location: argument, else $AXONO_REFERENCE_ROOT, else a checkout named `reference` beside this
    repository)."""
    ref_root = ref_root or os.environ.get("AXONO_REFERENCE_ROOT", "") or _sibling_reference()
    subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])
    if ref_root and os.path.isdir(os.path.join(ref_root, "src")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REF={ref_root}"])
        subprocess.check_call(["make", "-s", "-C", _HERE, "refcuda", f"REF={ref_root}"])


def _sibling_reference() -> str:
    path = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return path if os.path.isdir(path) else ""


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class _Checker:
    """numpy wrappers shared by both libraries; `prefix` is ``orc_`` or ``ref_``."""

    def __init__(self, path: str, prefix: str, kind: str):
        self.lib = C.CDLL(path)
        self.prefix = prefix
        self.kind = kind
        self.path = path

    def _fn(self, name, argtypes, restype=C.c_int):
        fn = getattr(self.lib, self.prefix + name)
        fn.argtypes = argtypes
        fn.restype = restype
        return fn

    @staticmethod
    def _check(st, what):
        if st != 0:
            raise RuntimeError(f"{what} failed, status {st}")

    # attention ---------------------------------------------------------
    def sdpa(self, q, k, v, is_causal=False):
        q, k, v = _f32(q), _f32(k), _f32(v)
        sq, hq, d = q.shape
        skv, hkv, _ = k.shape
        out = np.empty_like(q)
        fn = self._fn("sdpa_f32", [_f32p, _f32p, _f32p, _f32p, _sz, _sz, _sz, _sz, _sz, C.c_int])
        self._check(fn(q, k, v, out, sq, hq, hkv, d, skv, int(is_causal)), "sdpa")
        return out

    def gqa_decode(self, q, k, v):
        """q (1,hq,d), k/v (skv,hkv,d) -> (1,hq,d); the reference's decode op equals
        non-causal SDPA (axono/python/axono/gqa.py:32)."""
        return self.sdpa(q, k, v, False)

    def gqa_decode_batched(self, q, ks, vs):
        """q (B,hq,d); ks/vs lists of per-sequence (L_b,hkv,d) arrays -> (B,hq,d)."""
        q = _f32(q)
        out = np.empty_like(q)
        for b in range(q.shape[0]):
            out[b] = self.sdpa(q[b : b + 1], ks[b], vs[b], False)[0]
        return out

    # rope ---------------------------------------------------------------
    def rope(self, x, pos, theta):
        x = _f32(x)
        pos = np.ascontiguousarray(pos, dtype=np.int64).reshape(-1)
        rows, heads, dim = x.shape
        out = np.empty_like(x)
        fn = self._fn("rope_f32", [_f32p, _i64p, C.c_float, _f32p, _sz, _sz, _sz])
        self._check(fn(x, pos, theta, out, rows, heads, dim), "rope")
        return out

    def rope_with_cos_sin(self, x, cos, sin):
        x, cos, sin = _f32(x), _f32(cos), _f32(sin)
        rows, heads, dim = x.shape
        out = np.empty_like(x)
        fn = self._fn("rope_with_cos_sin_f32", [_f32p, _f32p, _f32p, _f32p, _sz, _sz, _sz])
        self._check(fn(x, cos, sin, out, rows, heads, dim), "rope_with_cos_sin")
        return out

    def mrope_cos_sin(self, pos3, inv_freq, h_sec, w_sec):
        pos3 = np.ascontiguousarray(pos3, dtype=np.int64)
        inv_freq = _f32(inv_freq)
        rows, half = pos3.shape[1], inv_freq.shape[0]
        cos = np.empty((rows, 2 * half), np.float32)
        sin = np.empty((rows, 2 * half), np.float32)
        fn = self._fn("mrope_cos_sin_f32", [_i64p, _f32p, C.c_int, C.c_int, _f32p, _f32p, _sz, _sz])
        self._check(fn(pos3, inv_freq, h_sec, w_sec, cos, sin, rows, half), "mrope_cos_sin")
        return cos, sin

    def rope_thd(self, x, pos3, inv_freq, sections):
        x = _f32(x)
        pos3 = np.ascontiguousarray(pos3, dtype=np.int64)
        inv_freq = _f32(inv_freq)
        rows, heads, dim = x.shape
        out = np.empty_like(x)
        t, h, w = sections
        fn = self._fn(
            "rope_thd_f32",
            [_f32p, _i64p, _f32p, C.c_int, C.c_int, C.c_int, _f32p, _sz, _sz, _sz],
        )
        self._check(fn(x, pos3, inv_freq, t, h, w, out, rows, heads, dim), "rope_thd")
        return out

    # append ---------------------------------------------------------------
    def concat_axis0(self, a, b):
        a = np.ascontiguousarray(a)
        b = np.ascontiguousarray(b)
        assert a.dtype == b.dtype and a.shape[1:] == b.shape[1:]
        out = np.empty((a.shape[0] + b.shape[0],) + a.shape[1:], a.dtype)
        row_bytes = int(np.prod(a.shape[1:], dtype=np.int64)) * a.dtype.itemsize
        av, bv, ov = (t.view(np.uint8).reshape(-1) for t in (a, b, out))
        if self.prefix == "orc_":
            fn = self._fn("concat_bytes", [_u8p, _u8p, _u8p, _sz, _sz, _sz])
            self._check(fn(av, bv, ov, 1, a.shape[0] * row_bytes, b.shape[0] * row_bytes), "concat")
        else:
            fn = self._fn("concat_axis0_bytes", [_u8p, _u8p, _u8p, _sz, _sz, _sz])
            self._check(fn(av, bv, ov, a.shape[0], b.shape[0], row_bytes), "concat")
        return out

    # fused ---------------------------------------------------------------
    def silu_mul(self, gate, up):
        gate, up = _f32(gate), _f32(up)
        out = np.empty_like(gate)
        fn = self._fn("silu_mul_f32", [_f32p, _f32p, _f32p, _sz])
        self._check(fn(gate.reshape(-1), up.reshape(-1), out.reshape(-1), gate.size), "silu_mul")
        return out

    def add_rms_norm(self, x, residual, weight, eps=1e-6):
        x, residual, weight = _f32(x), _f32(residual), _f32(weight)
        hidden = x.shape[-1]
        rows = x.size // hidden
        y = np.empty_like(x)
        out = np.empty_like(x)
        fn = self._fn("add_rms_norm_f32", [_f32p, _f32p, _f32p, C.c_float, _f32p, _f32p, _sz, _sz])
        self._check(
            fn(x.reshape(-1), residual.reshape(-1), weight, eps, y.reshape(-1), out.reshape(-1), rows, hidden),
            "add_rms_norm",
        )
        return y, out

    def rms_norm(self, x, weight, eps=1e-5):
        x, weight = _f32(x), _f32(weight)
        cols = x.shape[-1]
        rows = x.size // cols
        out = np.empty_like(x)
        fn = self._fn("rms_norm_f32", [_f32p, _f32p, C.c_float, _f32p, _sz, _sz])
        self._check(fn(x.reshape(-1), weight, eps, out.reshape(-1), rows, cols), "rms_norm")
        return out

    # embedding / argmax ------------------------------------------------------
    def embedding(self, ids, table):
        ids = np.ascontiguousarray(ids, dtype=np.int64)
        table = _f32(table)
        out = np.empty(ids.shape + (table.shape[1],), np.float32)
        if self.prefix == "orc_":
            fn = self._fn("embedding_f32", [_i64p, _f32p, _f32p, _sz, _sz])
            self._check(fn(ids.reshape(-1), table, out.reshape(-1), ids.size, table.shape[1]), "embedding")
        else:
            fn = self._fn("embedding_f32", [_i64p, _f32p, _f32p, _sz, _sz, _sz])
            self._check(fn(ids.reshape(-1), table, out.reshape(-1), ids.size, table.shape[0], table.shape[1]),
                        "embedding")
        return out

    def argmax_last_dim(self, x):
        x = _f32(x)
        cols = x.shape[-1]
        out = np.empty(x.shape[:-1], np.int64)
        fn = self._fn("argmax_last_dim_f32", [_f32p, _i64p, _sz, _sz])
        self._check(fn(x.reshape(-1), out.reshape(-1), x.size // cols, cols), "argmax")
        return out

    # fp16 bits ---------------------------------------------------------------
    def half_to_float(self, bits):
        bits = np.ascontiguousarray(bits, dtype=np.uint16)
        out = np.empty(bits.shape, np.float32)
        fn = self._fn("half_to_float", [_u16p, _f32p, _sz], None)
        fn(bits.reshape(-1), out.reshape(-1), bits.size)
        return out

    def float_to_half(self, x):
        x = _f32(x)
        out = np.empty(x.shape, np.uint16)
        fn = self._fn("float_to_half", [_f32p, _u16p, _sz], None)
        fn(x.reshape(-1), out.reshape(-1), x.size)
        return out


class _Port(_Checker):
    def rope_inv_freq(self, theta, dim):
        out = np.empty(dim // 2, np.float32)
        fn = self._fn("rope_inv_freq", [C.c_float, _sz, _f32p], None)
        fn(theta, dim, out)
        return out

    def build_mrope_pos3(self, n, img_start, want, llm_h, llm_w):
        pos3 = np.zeros((3, n), np.int64)
        fn = self._fn("build_mrope_pos3", [_i64p, _sz, _sz, _sz, _sz, _sz], None)
        fn(pos3, n, img_start, want, llm_h, llm_w)
        return pos3

    def prepare_sdpa(self, q, k, v):
        """Same interface as the reference checker's: (run, out, release)."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        sq, hq, d = q.shape
        skv, hkv, _ = k.shape
        out = np.empty_like(q)
        fn = self._fn("sdpa_f32", [_f32p, _f32p, _f32p, _f32p, _sz, _sz, _sz, _sz, _sz, C.c_int])

        def _run():
            self._check(fn(q, k, v, out, sq, hq, hkv, d, skv, 0), "sdpa")

        return _run, out, (lambda: None)

    def num_threads(self):
        fn = self._fn("num_threads", [], C.c_int)
        return int(fn())


class _Reference(_Checker):
    def sdpa_timed(self, q, k, v, iters):
        """Times `iters` calls of the reference's CPU SDPA on the same buffers; returns
        (out, ms_per_call array)."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        sq, hq, d = q.shape
        skv, hkv, _ = k.shape
        out = np.empty_like(q)
        ms = np.zeros(iters, np.float64)
        fn = self._fn(
            "sdpa_f32_timed",
            [_f32p, _f32p, _f32p, _f32p, _sz, _sz, _sz, _sz, _sz, C.c_int,
             np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")],
        )
        self._check(fn(q, k, v, out, sq, hq, hkv, d, skv, iters, ms), "sdpa_timed")
        return out, ms


    def prepare_sdpa(self, q, k, v):
        """Wraps the buffers once; returns (run, out, release): run() executes the reference's
        non-causal SDPA into `out`."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        sq, hq, d = q.shape
        skv, hkv, _ = k.shape
        out = np.empty_like(q)
        prep = self._fn("sdpa_prepare", [_f32p, _f32p, _f32p, _f32p, _sz, _sz, _sz, _sz, _sz], C.c_void_p)
        run = self._fn("sdpa_run", [C.c_void_p])
        rel = self._fn("sdpa_release", [C.c_void_p], None)
        handle = C.c_void_p(prep(q, k, v, out, sq, hq, hkv, d, skv))
        keep = [q, k, v, out]  # the wrapped buffers must outlive the handle

        def _run():
            self._check(run(handle), "sdpa_run")

        def _release():
            rel(handle)
            keep.clear()

        return _run, out, _release


class _ReferenceCuda:
    """The reference's own CUDA operators (fp32), compiled for sm_100: host arrays in and out, with
    an optional timed loop (`iters` calls between CUDA events; returns milliseconds per call)."""

    kind = "reference-cuda"

    def __init__(self, path):
        self.lib = C.CDLL(path)
        self._ms = C.c_double(0.0)

    def _run(self, name, argtypes, *args, iters=0):
        fn = getattr(self.lib, "refcu_" + name)
        fn.argtypes = argtypes + [C.c_int, C.POINTER(C.c_double)]
        fn.restype = C.c_int
        self._ms.value = 0.0
        st = fn(*args, int(iters), C.byref(self._ms))
        if st != 0:
            raise RuntimeError(f"reference CUDA {name} failed, status {st}")
        return self._ms.value

    def gqa_decode(self, q, k, v, iters=0):
        q, k, v = _f32(q), _f32(k), _f32(v)
        _, hq, d = q.shape
        skv, hkv, _ = k.shape
        out = np.empty_like(q)
        ms = self._run("gqa_decode_f32", [_f32p, _f32p, _f32p, _f32p, _sz, _sz, _sz, _sz], q, k, v, out, hq, hkv, d,
                       skv, iters=iters)
        return out, ms

    def sdpa(self, q, k, v, is_causal=False, iters=0):
        q, k, v = _f32(q), _f32(k), _f32(v)
        sq, hq, d = q.shape
        skv, hkv, _ = k.shape
        out = np.empty_like(q)
        ms = self._run("sdpa_f32", [_f32p, _f32p, _f32p, _f32p, _sz, _sz, _sz, _sz, _sz, C.c_int], q, k, v, out, sq, hq,
                       hkv, d, skv, int(bool(is_causal)), iters=iters)
        return out, ms

    def add_rms_norm(self, x, residual, weight, eps=1e-6, iters=0):
        x, residual, weight = _f32(x), _f32(residual), _f32(weight)
        hidden = x.shape[-1]
        y, out = np.empty_like(x), np.empty_like(x)
        ms = self._run("add_rms_norm_f32", [_f32p, _f32p, _f32p, C.c_float, _f32p, _f32p, _sz, _sz],
                       x.reshape(-1), residual.reshape(-1), weight, eps, y.reshape(-1), out.reshape(-1),
                       x.size // hidden, hidden, iters=iters)
        return y, out, ms

    def silu_mul(self, gate, up, iters=0):
        gate, up = _f32(gate), _f32(up)
        out = np.empty_like(gate)
        ms = self._run("silu_mul_f32", [_f32p, _f32p, _f32p, _sz], gate.reshape(-1), up.reshape(-1), out.reshape(-1),
                       gate.size, iters=iters)
        return out, ms

    def rope(self, x, pos, theta, iters=0):
        x = _f32(x)
        pos = np.ascontiguousarray(pos, dtype=np.int64).reshape(-1)
        rows, heads, dim = x.shape
        out = np.empty_like(x)
        ms = self._run("rope_f32", [_f32p, _i64p, C.c_float, _f32p, _sz, _sz, _sz], x, pos, theta, out, rows, heads,
                       dim, iters=iters)
        return out, ms


_port = None
_reference = None
_reference_cuda = None


def have_reference_cuda() -> bool:
    return os.path.exists(REF_CUDA_LIB)


def reference_cuda() -> _ReferenceCuda:
    global _reference_cuda
    if _reference_cuda is None:
        if not have_reference_cuda():
            raise FileNotFoundError(f"{REF_CUDA_LIB} is not built (make -C oracle refcuda)")
        _reference_cuda = _ReferenceCuda(REF_CUDA_LIB)
    return _reference_cuda


def port() -> _Port:
    global _port
    if _port is None:
        if not os.path.exists(PORT_LIB):
            build()
        _port = _Port(PORT_LIB, "orc_", "port")
    return _port


def have_reference() -> bool:
    return os.path.exists(REF_LIB)


def reference() -> _Reference:
    global _reference
    if _reference is None:
        if not have_reference():
            raise FileNotFoundError(f"{REF_LIB} is not built (needs the reference sources: make -C oracle ref)")
        _reference = _Reference(REF_LIB, "ref_", "reference")
    return _reference


def best() -> _Checker:
    """The reference's own code where it was built, else the C restatement."""
    return reference() if have_reference() else port()


def rel_err(out, ref) -> float:
    """Parity metric used throughout the tests: max|out-ref| / max|ref| per tensor."""
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = float(np.max(np.abs(ref))) if ref.size else 0.0
    if denom == 0.0:
        return float(np.max(np.abs(out - ref))) if ref.size else 0.0
    return float(np.max(np.abs(out - ref)) / denom)
