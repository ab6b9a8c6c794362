"""The allocation-free decode entry point (axb200_gqa_decode_static) against the regular one.

Some hosts of this library cannot hand it a workspace: the GPU's memory belongs to their own
allocator, or a cudaMalloc in the decode loop would synchronise the whole device.  For them the
library carries a fixed 4 MiB scratch array of its own.  This file is named to be collected last,
and it must pass both on its own in a fresh process and after every other GPU test has run.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, q, k, v, dtype_code):
    """Runs the regular entry point (caller-provided workspace) and the static-scratch one on the
    same inputs, through the C ABI, and returns both outputs."""
    _, hq, d = q.shape
    skv, hkv, _ = k.shape
    stream = torch.cuda.current_stream().cuda_stream
    need = lib.axb200_gqa_workspace_bytes(1, hq, hkv, d, skv, dtype_code)
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device="cuda")
    ref = torch.empty_like(q)
    out = torch.full_like(q, float("nan"))
    st = lib.axb200_gqa_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), ref.data_ptr(), hq, hkv, d, skv,
                               dtype_code, ws.data_ptr(), ws.numel(), stream)
    assert st == 0
    st = lib.axb200_gqa_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), hq, hkv, d, skv,
                                      dtype_code, stream)
    assert st == 0
    torch.cuda.synchronize()
    return ref, out


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2e-3), (torch.float32, 1e-5)])
def test_static_scratch_matches_workspace_entry_point_twice(dtype, tol):
    from axono_b200 import _capi

    lib = _capi.lib()
    code = _capi.FLOAT16 if dtype == torch.float16 else _capi.FLOAT32
    assert lib.axb200_static_scratch_bytes() == 4 << 20
    gen = torch.Generator(device="cuda").manual_seed(7)
    # second call is shorter, so the array still holds the first call's records beyond what it uses
    for skv in (9000, 2500):
        q = torch.randn((1, 16, 128), generator=gen, device="cuda").to(dtype)
        k = torch.randn((skv, 8, 128), generator=gen, device="cuda").to(dtype)
        v = torch.randn((skv, 8, 128), generator=gen, device="cuda").to(dtype)
        ref, out = _both(lib, q, k, v, code)
        assert torch.isfinite(out).all()
        err = (out.float() - ref.float()).abs().max().item() / ref.float().abs().max().item()
        assert err <= tol, f"skv={skv}: {err:.3e}"
    assert lib.axb200_last_error() == 0


def test_static_scratch_rejects_oversize_and_allocates_nothing():
    from axono_b200 import _capi

    lib = _capi.lib()
    # 512 query heads x 256 dims x many chunks needs more than the 4 MiB the library carries
    hq, hkv, d, skv = 512, 8, 256, 200000
    assert lib.axb200_gqa_workspace_bytes(1, hq, hkv, d, skv, _capi.FLOAT32) > lib.axb200_static_scratch_bytes()
    dummy = torch.zeros(16, device="cuda")
    st = lib.axb200_gqa_decode_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                      hq, hkv, d, skv, _capi.FLOAT32, None)
    assert st == 2  # AXB200_OUT_OF_MEMORY: beyond the built-in scratch, nothing was launched
    # a fitting call leaves the driver's allocated-memory figure where it was
    q = torch.randn((1, 16, 128), device="cuda")
    k = torch.randn((4096, 8, 128), device="cuda")
    out = torch.empty_like(q)
    lib.axb200_gqa_decode_static(q.data_ptr(), k.data_ptr(), k.data_ptr(), out.data_ptr(), 16, 8, 128, 4096,
                                 _capi.FLOAT32, None)
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        st = lib.axb200_gqa_decode_static(q.data_ptr(), k.data_ptr(), k.data_ptr(), out.data_ptr(), 16, 8, 128,
                                          4096, _capi.FLOAT32, None)
        assert st == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
