"""GPU-side parity: this package's fp32 kernels against the reference's own CUDA kernels compiled for
sm_100 (oracle/_ref/libaxono_ref_cuda.so), on the same seeded inputs.  Skipped where that library was
not built.  The reference's kernels are fp32 and single-sequence."""
import numpy as np
import pytest
import torch

import cases
import oracle

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not oracle.have_reference_cuda(), reason="reference CUDA library not built")]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_gqa_decode_matches_reference_cuda_kernels():
    from axono_b200 import ops

    ref = oracle.reference_cuda()
    for name in ("gqa_rs3_skv7", "gqa_rs3_skv1024", "gqa_skv2048", "gqa_skv2049", "gqa_c1_skv4096"):
        q, k, v = cases.all_gqa_cases()[name]
        want, _ = ref.gqa_decode(q, k, v)  # SDPA fallback below 2048 keys, split-K kernels from 2048
        got = ops.gqa_decode_attention(dev(q), dev(k), dev(v)).cpu().numpy()
        assert oracle.rel_err(got, want) <= 1e-5, name


def test_fused_and_rope_match_reference_cuda_kernels():
    from axono_b200 import ops

    ref = oracle.reference_cuda()
    f = cases.fused_cases()
    x, r, w, eps = f["addrms_c2"]
    y, out, _ = ref.add_rms_norm(x, r, w, eps)
    my_y, my_out = ops.add_rms_norm(dev(x), dev(r), dev(w), eps)
    assert np.array_equal(my_y.cpu().numpy(), y)
    assert oracle.rel_err(my_out.cpu().numpy(), out) <= 1e-5
    g, u = f["silu_rs0"]
    want, _ = ref.silu_mul(g, u)
    np.testing.assert_allclose(ops.silu_mul(dev(g), dev(u)).cpu().numpy(), want, rtol=1e-5, atol=1e-6)
    xq, pos, theta = cases.rope_cases()["rope_small"]
    want, _ = ref.rope(xq, pos, theta)
    assert oracle.rel_err(ops.rope(dev(xq), dev(pos), theta).cpu().numpy(), want) <= 1e-5
