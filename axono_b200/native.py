"""Loader of the native module `libaxono` (no PyTorch): the reference's binding surface for the
decode path - Tensor, DataType, Status, the operators, CUDAGraph, the allocator controls
(axono/python/src/nanobind_module.cpp) - plus the KV arena operators.

    from axono_b200 import native
    lx = native.load()            # also registers it as `libaxono` in sys.modules
    q = lx.Tensor.from_numpy(q_np, "cuda")
    out = lx.gqa_decode_attention(q, k, v).numpy()

`cuda_graph()` mirrors the reference's context manager (axono/python/axono/core/cuda_graph.py).
"""
from __future__ import annotations

import contextlib
import importlib.util
import os
import sys

_MODULE = None


def load():
    """Imports the in-tree extension module; raises when it has not been built (python -m axono_b200.build)."""
    global _MODULE
    if _MODULE is not None:
        return _MODULE
    from . import build as _build

    path = _build.native_module_path()
    if not os.path.exists(path):
        raise ImportError(f"native module not built: {path} (run `python -m axono_b200.build`)")
    spec = importlib.util.spec_from_file_location("libaxono", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["libaxono"] = mod
    _MODULE = mod
    return mod


class CUDAGraph:
    """capture (with its own warm-up run) -> replay any number of times -> reset; `output` / `outputs`
    hold what the captured function returned (buffers that every replay rewrites)."""

    def __init__(self):
        lx = load()
        if not lx.cuda_available():
            raise RuntimeError("CUDA graphs need a CUDA device")
        self._impl = lx.CUDAGraph()
        self.output = None
        self.outputs = []

    def capture(self, fn):
        box = {}

        def body():
            box["r"] = fn()

        self._impl.capture(body)
        r = box.get("r")
        self.outputs = list(r) if isinstance(r, (tuple, list)) else [r]
        self.output = self.outputs[0]
        return self

    def replay(self):
        self._impl.replay()
        return self.output

    def sync(self):
        self._impl.sync()

    def reset(self):
        self._impl.reset()
        self.output, self.outputs = None, []

    @property
    def is_captured(self):
        return self._impl.is_captured

    @property
    def num_nodes(self):
        return self._impl.num_nodes


@contextlib.contextmanager
def cuda_graph():
    """Captures the block itself (no warm-up re-run): tensors created inside it are stream-ordered
    allocations recorded in the graph; set `g.output` (a tensor or a tuple) inside the block."""
    lx = load()
    g = CUDAGraph()
    handle = lx._graph_begin_capture()
    try:
        yield g
    except BaseException:
        lx._graph_abort_capture(handle)
        raise
    lx._graph_end_capture(handle, g._impl)
    out = g.output
    if isinstance(out, (tuple, list)):
        g.outputs, g.output = list(out), out[0]
    elif out is not None:
        g.outputs = [out]
