"""CPU-side checks of the native `libaxono` module: it imports without PyTorch, the host Tensor keeps
the reference's container semantics (include/axono/core/tensor.h:24-129), and operators refuse CPU
tensors instead of falling back to host code."""
import subprocess
import sys

import numpy as np
import pytest

from axono_b200 import native


@pytest.fixture(scope="module")
def lx():
    return native.load()


def test_import_without_torch():
    code = ("import sys; from axono_b200 import native; lx = native.load(); "
            "assert 'torch' not in sys.modules, 'torch was imported'; "
            "print(lx.version(), int(lx.DataType.FLOAT16), int(lx.Status.DEVICE_MISMATCH))")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    assert out.stdout.split()[-2:] == ["4", "8"]  # enum values of include/axono/core/types.h:18-43


def test_enums_match_reference_values(lx):
    assert [int(getattr(lx.DataType, n)) for n in
            ("INT8", "INT16", "INT32", "INT64", "FLOAT16", "FLOAT32", "FLOAT64", "BOOLEAN")] == list(range(8))
    assert int(lx.Status.OK) == 0 and int(lx.Status.SHAPE_MISMATCH) == 4 and int(lx.Status.DEVICE_ERROR) == 6


def test_host_tensor_semantics(lx):
    t = lx.Tensor(lx.DataType.FLOAT32, [2, 3])
    assert t.shape == (2, 3) and t.ndim == 2 and t.num_elements == 6 and t.num_bytes == 24
    assert t.device == "cpu" and not t.is_cuda
    assert np.array_equal(t.numpy(), np.zeros((2, 3), np.float32))  # new storage is zero-filled
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    u = lx.Tensor.from_numpy(a)
    assert np.array_equal(u.data_float32(), a)
    t.copy_from(u)
    assert np.array_equal(t.numpy(), a)
    t.reshape([3, 2])
    assert t.shape == (3, 2) and np.array_equal(t.numpy().ravel(), a.ravel())
    with pytest.raises(RuntimeError):
        t.reshape([4, 2])
    t.resize([4])
    assert t.num_elements == 4 and np.array_equal(t.numpy(), np.zeros(4, np.float32))
    with pytest.raises(RuntimeError):  # element counts differ
        t.copy_from(u)
    empty = lx.Tensor(lx.DataType.FLOAT32, [])
    assert empty.num_elements == 0  # an empty shape holds nothing, as in the reference


def test_half_tensors_carry_raw_bits(lx):
    a = np.array([1.0, -2.5, 65504.0, 6e-8], dtype=np.float16)
    t = lx.Tensor.from_numpy(a)
    assert t.dtype == lx.DataType.FLOAT16
    assert np.array_equal(t.data_float16().view(np.float16), a)
    f = t.cast_to(lx.DataType.FLOAT32)
    assert np.array_equal(f.numpy(), a.astype(np.float32))
    assert np.array_equal(f.cast_to(lx.DataType.FLOAT16).numpy(), a)
    b = lx.Tensor.from_borrowed(a.view(np.uint16))
    assert b.dtype == lx.DataType.FLOAT16 and np.array_equal(b.numpy(), a)


def test_copy_shares_storage_deepcopy_does_not(lx):
    import copy

    t = lx.Tensor.from_numpy(np.ones(4, np.float32))
    s, d = copy.copy(t), copy.deepcopy(t)
    t.fill_zero()
    assert np.array_equal(s.numpy(), np.zeros(4, np.float32))
    assert np.array_equal(d.numpy(), np.ones(4, np.float32))


def test_operators_refuse_cpu_tensors(lx):
    x = lx.Tensor.from_numpy(np.ones((2, 8), np.float32))
    w = lx.Tensor.from_numpy(np.ones(8, np.float32))
    for call in (lambda: lx.silu_mul(x, x), lambda: lx.add_rms_norm(x, x, w, 1e-6), lambda: lx.rms_norm(x, w),
                 lambda: lx.argmax(x), lambda: lx.concat(x, x, 0)):
        with pytest.raises(RuntimeError):
            call()
    q = lx.Tensor.from_numpy(np.ones((1, 4, 64), np.float32))
    kv = lx.Tensor.from_numpy(np.ones((16, 2, 64), np.float32))
    with pytest.raises(RuntimeError, match="status 8"):  # DEVICE_MISMATCH, src/ops/cuda/gqa.cu:143-154
        lx.gqa_decode_attention(q, kv, kv)


def test_every_operator_checks_every_operand_before_launching(lx):
    """A host pointer handed to a kernel would be an illegal-address fault that takes the context with
    it.  No operator gets that far: each one refuses unless every tensor operand is in device memory
    (status 8, DEVICE_MISMATCH, or the binding's own message) - nothing is launched, so this needs no GPU.
    The reference checks the first operand at most (its ops ignore ctx, e.g. src/ops/cuda/fused.cu:78)."""
    f32, i64 = np.float32, np.int64
    T = lx.Tensor.from_numpy
    x3 = T(np.ones((2, 4, 8), f32))
    x2 = T(np.ones((2, 8), f32))
    w = T(np.ones(8, f32))
    pos = T(np.zeros(2, i64))
    pos3 = T(np.zeros((3, 2), i64))
    inv = T(np.ones(4, f32))
    cs = T(np.ones((2, 8), f32))
    ids = T(np.zeros(3, i64))
    calls = {
        "gqa_decode_attention": lambda: lx.gqa_decode_attention(T(np.ones((1, 4, 8), f32)), x3, x3),
        "scaled_dot_product_attention": lambda: lx.scaled_dot_product_attention(x3, x3, x3, True),
        "silu_mul": lambda: lx.silu_mul(x2, x2),
        "add_rms_norm": lambda: lx.add_rms_norm(x2, x2, w, 1e-6),
        "rms_norm": lambda: lx.rms_norm(x2, w, 1e-6),
        "rope": lambda: lx.rope(x3, pos, 1e4),
        "rope_thd": lambda: lx.rope_thd(x3, pos3, inv, 1, 1, 1),
        "rope_with_cos_sin": lambda: lx.rope_with_cos_sin(x3, cs, cs),
        "mrope_cos_sin": lambda: lx.mrope_cos_sin(pos3, inv, 1, 1),
        "concat": lambda: lx.concat(x2, x2, 0),
        "embedding": lambda: lx.embedding(ids, x2),
        "argmax": lambda: lx.argmax(x2),
        "linear_nobias": lambda: lx.linear_nobias(x2, x2),
        "silu_mul_rows": lambda: lx.silu_mul_rows(x2, 4),
    }
    for name, call in calls.items():
        with pytest.raises(RuntimeError):
            call()
    for name in ("linear_nobias", "gqa_decode_attention"):  # these reach the operator layer: its own status
        with pytest.raises(RuntimeError, match="status 8"):
            calls[name]()


def test_axono_compat_package_host_side():
    """`import axono` resolves to the compatibility package; host tensors, default device and the
    KV-cache contract need no GPU; operators on host tensors raise instead of falling back."""
    import axono_b200.compat as compat

    compat.install()
    import axono
    from axono import nn

    assert axono.get_default_device() == "cpu" and axono.get_backend() == "cpu"
    with pytest.raises(ValueError):
        axono.set_default_device("tpu")
    t = axono.Tensor.from_numpy(np.arange(6).reshape(2, 3))  # ints stay ints
    assert t.dtype == axono.DataType.INT64 and np.array_equal(t.to_numpy(), np.arange(6).reshape(2, 3))
    assert np.array_equal(axono.Tensor.ones([2, 2]).to_numpy(), np.ones((2, 2), np.float32))
    assert np.array_equal(axono.Tensor.zeros([3]).fill(2.5).to_numpy(), np.full(3, 2.5, np.float32))
    cache = nn.DynamicKVCache(2)
    assert len(cache) == 0
    with pytest.raises(RuntimeError):
        cache.get(0)
    k = axono.Tensor.from_numpy(np.zeros((3, 2, 4), np.float32))
    cache.update(0, k, k)
    assert len(cache) == 3 and cache.get(0)[0] is k
    with pytest.raises(RuntimeError):  # second update concatenates: a CUDA operator, refused for host tensors
        cache.update(0, k, k)
    with pytest.raises(RuntimeError):
        axono.fused.silu_mul(k, k)
    assert not hasattr(axono, "matmul")  # outside this library
