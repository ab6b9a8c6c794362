"""The library collective's pieces on one GPU (-m gpu): the re-layout kernel against numpy, and an NCCL
communicator of one rank - created before any capture, its all-gather recorded into a CUDA graph and
replayed - which is the sequence the head-sharded tower runs on several GPUs."""
import ctypes as C

import numpy as np
import pytest

from axono_b200 import _capi, native

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lx():
    m = native.load()
    assert m.cuda_available()
    return m


def test_swap_leading_dims_matches_numpy(lx):
    lib = _capi.lib()
    rng = np.random.default_rng(5)
    for n0, n1, row in ((8, 32, 256), (2, 5, 8), (3, 1, 1024), (1, 7, 64)):
        a = rng.standard_normal((n0, n1, row)).astype(np.float16)
        src = lx.Tensor.from_numpy(a, "cuda")
        dst = lx.Tensor(lx.DataType.FLOAT16, [n1, n0, row], "cuda")
        assert lib.axb200_swap_leading_dims(src.data_ptr, dst.data_ptr, n0, n1, row * 2, None) == 0
        assert np.array_equal(dst.numpy(), a.transpose(1, 0, 2))
    t = lx.Tensor(lx.DataType.FLOAT16, [64], "cuda")
    assert lib.axb200_swap_leading_dims(t.data_ptr, t.data_ptr, 2, 2, 8, None) == 1  # rows must be 16-byte multiples
    assert lib.axb200_swap_leading_dims(None, t.data_ptr, 2, 2, 16, None) == 7


_NCCL_CHILD = r"""
import ctypes as C, sys
import numpy as np
from axono_b200 import _capi, native
lx = native.load(); lib = _capi.lib()
uid = C.create_string_buffer(128)
if lib.axb200_nccl_unique_id(uid) != 0:
    print("SKIP: libnccl.so.2 is not loadable here"); sys.exit(0)
comm = C.c_void_p()
assert lib.axb200_nccl_init(uid, 1, 0, C.byref(comm)) == 0  # before any capture: it allocates and synchronises
a = np.arange(4 * 2 * 128, dtype=np.float32).astype(np.float16).reshape(4, 2, 128)
send = lx.Tensor.from_numpy(a, "cuda")
recv = lx.Tensor(lx.DataType.FLOAT16, [1, 4, 2, 128], "cuda")
def body():
    _capi.check(lib.axb200_nccl_all_gather(comm, send.data_ptr, recv.data_ptr, send.num_bytes, lx.current_stream()),
                "nccl_all_gather")
    return recv
g = native.CUDAGraph().capture(body)
assert np.array_equal(recv.numpy().reshape(a.shape), a)
send.copy_from_numpy((a * 2).astype(np.float16))
g.replay()
assert np.array_equal(recv.numpy().reshape(a.shape), (a * 2).astype(np.float16))
g.reset()
assert lib.axb200_nccl_destroy(comm) == 0
assert lib.axb200_nccl_all_gather(None, send.data_ptr, recv.data_ptr, 16, None) == 7  # INVALID_PTR
assert lx.device_error_bits() == 0
print("OK")
"""


def test_nccl_all_gather_of_one_rank_inside_a_graph():
    """In a child process with a time limit: a communicator's set-up talks to the host's network stack,
    and a stall there should fail this test, not hold up the others."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    out = subprocess.run([sys.executable, "-c", _NCCL_CHILD], capture_output=True, text=True, timeout=240, env=env, cwd=root)
    if "SKIP" in out.stdout:
        pytest.skip(out.stdout.strip())
    assert out.returncode == 0 and "OK" in out.stdout, out.stdout + out.stderr
