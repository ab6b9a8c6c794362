"""CUDA-graph capture with the reference's `CUDAGraph` / `cuda_graph` / `compile` semantics
(axono/python/axono/core/cuda_graph.py:54-190, axono/python/axono/core/compile.py:69-174):

* `CUDAGraph().capture(fn)` warms `fn` up once, then records every operator `fn` launches into
  one graph; `fn`'s return value(s) become static output buffers (`output`, `outputs`);
* `replay()` launches the graph and waits for it; outputs are overwritten in place each time;
* replay before capture, and a capture that launched no operator, raise `RuntimeError`
  (tests/core/test_cuda_graph.py:148-165 of the reference);
* `compile(model)` keys graphs by the call signature (shapes/dtypes/devices of tensor arguments,
  repr of the others); the first call of a signature runs eagerly once and captures; later calls
  copy new inputs into the captured input tensors and replay.

The operators are launch-only on the current stream and never allocate, which is what capture
needs.  PyTorch supplies the capture stream and the private memory pool that keeps temporaries of
the captured region at fixed addresses (the job of the reference's capture pool,
src/core/cuda/capture_pool.cu:21-51).  What lets a decode step replay at all is the paged cache:
its lengths live on the device and advance inside the graph (the reference's concat-grown cache
changes shapes and addresses every step and cannot be replayed).
"""
from __future__ import annotations

import torch

from . import ops


class CUDAGraph:
    def __init__(self) -> None:
        if not torch.cuda.is_available():
            raise RuntimeError("CUDAGraph needs a CUDA device")
        self._graph = None
        self._outputs = []
        self._output = None
        self._num_nodes = 0

    # -- capture ----------------------------------------------------------------------------------
    def capture(self, fn, warmup: bool = True) -> "CUDAGraph":
        """Records everything `fn()` launches.  With `warmup` (the reference's behaviour) `fn` runs
        once eagerly first - so state that `fn` advances (cache lengths) advances once here."""
        if warmup:
            fn()
            torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(graph):
            out = fn()
        nodes = ops.launch_count() - before
        if nodes == 0:
            raise RuntimeError("CUDAGraph.capture: the captured region launched no operator")
        self._graph = graph
        self._num_nodes = nodes
        self._set_outputs(out)
        return self

    def _set_outputs(self, value) -> None:
        self._outputs = list(value) if isinstance(value, (tuple, list)) else [value]
        self._output = self._outputs[0] if self._outputs else None

    # -- replay -----------------------------------------------------------------------------------
    def replay(self) -> "CUDAGraph":
        if self._graph is None:
            raise RuntimeError("CUDAGraph.replay: nothing has been captured")
        self._graph.replay()
        torch.cuda.current_stream().synchronize()
        return self

    def replay_async(self) -> "CUDAGraph":
        """Launch without waiting (for back-to-back decode steps)."""
        if self._graph is None:
            raise RuntimeError("CUDAGraph.replay: nothing has been captured")
        self._graph.replay()
        return self

    def sync(self) -> "CUDAGraph":
        torch.cuda.current_stream().synchronize()
        return self

    def reset(self) -> None:
        if self._graph is not None:
            self._graph.reset()
        self._graph = None
        self._outputs, self._output, self._num_nodes = [], None, 0

    @property
    def output(self):
        return self._output

    @output.setter
    def output(self, value):
        self._set_outputs(value)

    @property
    def outputs(self):
        return list(self._outputs)

    @outputs.setter
    def outputs(self, values):
        self._set_outputs(values)

    @property
    def is_captured(self) -> bool:
        return self._graph is not None

    @property
    def num_nodes(self) -> int:
        """Operator launches recorded in the graph."""
        return self._num_nodes


class cuda_graph:  # noqa: N801 - context-manager spelling of the reference
    """`with cuda_graph() as g: y = op(...); g.output = y` - captures the block, no warm-up."""

    def __init__(self):
        self.graph = CUDAGraph()
        self._ctx = None
        self._before = 0

    def __enter__(self) -> CUDAGraph:
        self.graph._graph = torch.cuda.CUDAGraph()
        self._before = ops.launch_count()
        self._ctx = torch.cuda.graph(self.graph._graph)
        self._ctx.__enter__()
        return self.graph

    def __exit__(self, exc_type, exc, tb):
        self._ctx.__exit__(exc_type, exc, tb)
        if exc_type is None:
            self.graph._num_nodes = ops.launch_count() - self._before
            if self.graph._num_nodes == 0:
                self.graph._graph = None
                raise RuntimeError("cuda_graph: the captured block launched no operator")
        else:
            self.graph._graph = None
        return False


def _is_tensor(a) -> bool:
    return hasattr(a, "shape") and hasattr(a, "dtype")


def _signature(args, kwargs):
    parts = []
    for a in args:
        parts.append(("T", tuple(a.shape), str(a.dtype), str(a.device)) if _is_tensor(a) else ("S", repr(a)))
    for k in sorted(kwargs):
        v = kwargs[k]
        parts.append((k, "T", tuple(v.shape), str(v.dtype), str(v.device)) if _is_tensor(v) else (k, "S", repr(v)))
    return tuple(parts)


class CompiledModel:
    """A callable wrapped for graph replay; see the module docstring for the contract."""

    def __init__(self, model, mode: str = "normal"):
        if mode != "normal":
            raise ValueError(f"compile: unsupported mode {mode!r} (only 'normal')")
        if not torch.cuda.is_available():
            raise RuntimeError("compile needs a CUDA device")
        self._model, self._mode, self._graphs = model, mode, {}

    def __call__(self, *args, **kwargs):
        sig = _signature(args, kwargs)
        entry = self._graphs.get(sig)
        if entry is None:
            self._model(*args, **kwargs)  # eager warm-up on the real inputs
            g = CUDAGraph().capture(lambda: self._model(*args, **kwargs), warmup=False)
            entry = (g, args, kwargs)
            self._graphs[sig] = entry
        g, s_args, s_kwargs = entry
        for s, a in zip(s_args, args):
            if _is_tensor(s) and s is not a:
                s.copy_(a)
        for k, s in s_kwargs.items():
            if _is_tensor(s) and s is not kwargs[k]:
                s.copy_(kwargs[k])
        g.replay()
        outs = g.outputs
        return outs[0] if len(outs) == 1 else tuple(outs)

    forward = __call__

    @property
    def num_graphs(self) -> int:
        return len(self._graphs)


def compile(model, mode: str = "normal") -> CompiledModel:  # noqa: A001 - the reference's name
    return CompiledModel(model, mode=mode)
