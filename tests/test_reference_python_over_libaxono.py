"""The reference's OWN Python files, unchanged, on top of this library's `libaxono` module.

The drop-in promise is that Axono's pure-Python layer keeps working when the native module under it is
replaced.  These tests load the reference's `axono/gqa.py`, `axono/fused.py`, `axono/core/cuda_graph.py`
and `axono/core/compile.py` from a reference checkout by path (they are never copied into this
repository) after registering this library's module as `libaxono`, and drive the operators, the
`CUDAGraph` wrapper and `compile()` through them.

They need the reference's sources (`$AXONO_REFERENCE_ROOT`, else a checkout named `reference` beside this
repository) and are skipped where those are absent.  Without a GPU the import surface and the error behaviour are checked; with a
GPU the same files run the decode-path operators against the CPU checker.
"""
import importlib
import os
import sys
import types

import numpy as np
import pytest

REF = os.environ.get("AXONO_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
PKG = os.path.join(REF, "axono", "python", "axono")

pytestmark = pytest.mark.skipif(not os.path.isfile(os.path.join(PKG, "gqa.py")),
                                reason="no reference checkout at $AXONO_REFERENCE_ROOT")


@pytest.fixture(scope="module")
def ref():
    """The reference's modules, imported from its tree under a private package name so that its
    package __init__ (which pulls in the whole library) is not run."""
    from axono_b200 import native

    lx = native.load()  # registers sys.modules["libaxono"]
    root = types.ModuleType("axono_reference_files")
    root.__path__ = [PKG]
    core = types.ModuleType("axono_reference_files.core")
    core.__path__ = [os.path.join(PKG, "core")]
    sys.modules["axono_reference_files"] = root
    sys.modules["axono_reference_files.core"] = core
    mods = types.SimpleNamespace(
        lx=lx,
        gqa=importlib.import_module("axono_reference_files.gqa"),
        fused=importlib.import_module("axono_reference_files.fused"),
        cuda_graph=importlib.import_module("axono_reference_files.core.cuda_graph"),
        compile=importlib.import_module("axono_reference_files.core.compile"),
    )
    for m in (mods.gqa, mods.fused, mods.cuda_graph, mods.compile):
        assert os.path.realpath(m.__file__).startswith(os.path.realpath(REF))
    return mods


def test_reference_files_import_against_this_module(ref):
    """Every name the four files take from `libaxono` exists here."""
    for name in ("gqa_decode_attention", "silu_mul", "add_rms_norm", "CUDAGraph", "cuda_available",
                 "_graph_begin_capture", "_graph_end_capture", "_graph_abort_capture"):
        assert hasattr(ref.lx, name), name
    assert ref.gqa._l is ref.lx and ref.compile._l is ref.lx


def test_errors_surface_as_runtime_error_without_cuda(ref):
    """What the reference's tests assert (pytest.raises(RuntimeError)): a CPU tensor has no operator
    here, and without a device CUDAGraph() and compile() refuse, as the reference's wrappers do."""
    if ref.lx.cuda_available():
        pytest.skip("a CUDA device is present")
    T = ref.lx.Tensor
    q = T.from_numpy(np.zeros((1, 16, 128), np.float32))
    k = T.from_numpy(np.zeros((4, 8, 128), np.float32))
    with pytest.raises(RuntimeError):
        ref.gqa.gqa_decode_attention(q, k, k)
    with pytest.raises(RuntimeError):
        ref.fused.silu_mul(q, q)
    with pytest.raises(RuntimeError):
        ref.fused.add_rms_norm(q, q, T.from_numpy(np.ones(128, np.float32)))
    with pytest.raises(RuntimeError):
        ref.cuda_graph.CUDAGraph()
    with pytest.raises(RuntimeError):
        ref.compile.compile(lambda x: x)


@pytest.mark.gpu
def test_reference_wrappers_run_the_decode_path(ref):
    import oracle

    lx, orc = ref.lx, oracle.best()
    rng = np.random.default_rng(3)
    dev = lambda a: lx.Tensor.from_numpy(np.ascontiguousarray(a, dtype=np.float32), "cuda")  # noqa: E731
    q = rng.standard_normal((1, 16, 128)).astype(np.float32)
    for skv in (300, 4096):
        k = rng.standard_normal((skv, 8, 128)).astype(np.float32)
        v = rng.standard_normal((skv, 8, 128)).astype(np.float32)
        out = ref.gqa.gqa_decode_attention(dev(q), dev(k), dev(v)).numpy()
        assert oracle.rel_err(out, orc.gqa_decode(q, k, v)) <= 1e-5
    g, u = rng.standard_normal((37, 53)).astype(np.float32), rng.standard_normal((37, 53)).astype(np.float32)
    np.testing.assert_allclose(ref.fused.silu_mul(dev(g), dev(u)).numpy(), orc.silu_mul(g, u), rtol=1e-5, atol=1e-6)
    x, r = rng.standard_normal((4, 128)).astype(np.float32), rng.standard_normal((4, 128)).astype(np.float32)
    w = (1 + 0.02 * rng.standard_normal(128)).astype(np.float32)
    y, o = ref.fused.add_rms_norm(dev(x), dev(r), dev(w))  # the reference's default eps
    ry, ro = orc.add_rms_norm(x, r, w, 1e-6)
    np.testing.assert_allclose(y.numpy(), ry, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(o.numpy(), ro, rtol=1e-4, atol=1e-5)

    # the reference's CUDAGraph wrapper: capture, replay, outputs rewritten in place
    xs, rs, ws = dev(x), dev(r), dev(w)
    graph = ref.cuda_graph.CUDAGraph().capture(lambda: ref.fused.add_rms_norm(xs, rs, ws))
    assert len(graph.outputs) == 2
    xs.copy_from(dev(2 * x))
    graph.replay()
    ry2, _ = orc.add_rms_norm(2 * x, r, w, 1e-6)
    np.testing.assert_allclose(graph.outputs[0].numpy(), ry2, rtol=1e-5, atol=1e-6)

    # the reference's compile(): first call captures, later calls copy the inputs in and replay
    model = ref.compile.compile(lambda a, b: ref.fused.silu_mul(a, b))
    first = model(dev(g), dev(u)).numpy().copy()
    second = model(dev(u), dev(g)).numpy()
    np.testing.assert_allclose(first, orc.silu_mul(g, u), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(second, orc.silu_mul(u, g), rtol=1e-5, atol=1e-6)
    assert lx.device_error_bits() == 0
