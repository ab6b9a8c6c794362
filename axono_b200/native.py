"""Loader of the native module `libaxono` (no PyTorch): the reference's binding surface for the
decode path - Tensor, DataType, Status, the operators, CUDAGraph, the allocator controls
(axono/python/src/nanobind_module.cpp) - plus the KV arena operators.

    from axono_b200 import native
    lx = native.load()            # also registers it as `libaxono` in sys.modules
    q = lx.Tensor.from_numpy(q_np, "cuda")
    out = lx.gqa_decode_attention(q, k, v).numpy()

`CUDAGraph` / `cuda_graph()` mirror the reference's wrappers (axono/python/axono/core/cuda_graph.py),
`compile()` its graph-replay model wrapper (axono/python/axono/core/compile.py:69-174).
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

    def replay_timed(self, times: int) -> float:
        """`times` launches back to back between two CUDA events on the capture stream: ms per launch."""
        return self._impl.replay_timed(times)

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


def _is_tensor(a) -> bool:
    return hasattr(a, "shape") and hasattr(a, "dtype") and hasattr(a, "copy_from")


def _signature(args, kwargs):
    """Call signature that selects a cached graph: shape / dtype / device of tensors, repr of the rest."""
    parts = []
    for a in args:
        parts.append(("T", tuple(a.shape), str(a.dtype), str(a.device)) if _is_tensor(a) else ("S", repr(a)))
    for k in sorted(kwargs):
        v = kwargs[k]
        parts.append((k, "T", tuple(v.shape), str(v.dtype), str(v.device)) if _is_tensor(v) else (k, "S", repr(v)))
    return tuple(parts)


class CompiledModel:
    """`model` wrapped for graph replay.  The first call with a new signature runs the model once
    eagerly on the real inputs, then captures it (capture's own warm-up run records the allocations);
    that call's tensors become the static inputs and later calls copy their inputs into them; outputs
    are static buffers that the next replay overwrites.  Attribute access passes through to the model."""

    def __init__(self, model, mode: str = "normal"):
        if mode != "normal":
            raise ValueError(f"compile: unsupported mode {mode!r} (only 'normal')")
        if not load().cuda_available():
            raise RuntimeError("compile needs a CUDA device")
        object.__setattr__(self, "_model", model)
        object.__setattr__(self, "_mode", mode)
        object.__setattr__(self, "_graphs", {})

    def __getattr__(self, name):
        return getattr(object.__getattribute__(self, "_model"), name)

    def __setattr__(self, name, value):
        if name.startswith("_"):
            object.__setattr__(self, name, value)
        else:
            setattr(object.__getattribute__(self, "_model"), name, value)

    def __call__(self, *args, **kwargs):
        sig = _signature(args, kwargs)
        entry = self._graphs.get(sig)
        if entry is None:
            self._model(*args, **kwargs)
            g = CUDAGraph().capture(lambda: self._model(*args, **kwargs))
            entry = (g, args, kwargs)
            self._graphs[sig] = entry
        g, s_args, s_kwargs = entry
        for s, a in zip(s_args, args):
            if _is_tensor(s) and s is not a:
                s.copy_from(a)
        for k, s in s_kwargs.items():
            if _is_tensor(s) and s is not kwargs[k]:
                s.copy_from(kwargs[k])
        g.replay()
        outs = g.outputs
        return outs[0] if len(outs) == 1 else tuple(outs)

    forward = __call__

    @property
    def num_graphs(self) -> int:
        return len(self._graphs)

    def __repr__(self):
        return f"CompiledModel(mode={self._mode!r}, graphs={len(self._graphs)}, model={self._model!r})"


def compile(model, mode: str = "normal") -> CompiledModel:  # noqa: A001 - the reference's name
    return CompiledModel(model, mode=mode)
