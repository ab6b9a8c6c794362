"""Pins the CPU oracle (the C restatement) before anything is checked against it:
against the golden vectors produced by the reference's own CPU library, against the
numpy restatements the reference's tests use (at the reference's tolerances), and -
where the reference library was built in this tree - directly against it."""
import math

import numpy as np
import pytest

import cases
import oracle

# the restatement and the reference library agree bit-for-bit when built by the same compiler;
# the tolerance only allows for a different FMA-contraction choice by another compiler.
TIGHT = 1e-6


def _close(a, b, tol=TIGHT):
    assert a.shape == b.shape
    assert oracle.rel_err(a, b) <= tol


def _np_gqa(q, k, v):
    """numpy statement of the op as in axono/python/tests/core/test_gqa.py:11-25."""
    _, hq, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    out = np.zeros((1, hq, d), np.float32)
    for h in range(hq):
        s = (q[0, h] @ k[:, h // group].T) / math.sqrt(d)
        w = np.exp(s - s.max())
        out[0, h] = (w / w.sum()) @ v[:, h // group]
    return out


@pytest.mark.parametrize("name", sorted(cases.all_gqa_cases()))
def test_gqa_matches_golden_and_numpy(port, golden, name):
    q, k, v = cases.all_gqa_cases()[name]
    out = port.gqa_decode(q, k, v)
    _close(out, golden[name])
    # the reference's own test tolerance (test_gqa.py:42)
    np.testing.assert_allclose(out, _np_gqa(q, k, v), rtol=1e-4, atol=1e-4)


def test_sdpa_causal(port, golden):
    q, k, v = cases.sdpa_causal_case()
    _close(port.sdpa(q, k, v, True), golden["sdpa_causal"])
    _close(port.sdpa(q, k, v, False), golden["sdpa_noncausal"])
    # causal rule of src/ops/cpu/sequence.cpp:269-270: row t sees keys [0, t]
    ref = np.zeros_like(q)
    for t in range(q.shape[0]):
        ref[t] = _np_gqa(q[t : t + 1], k[: t + 1], v[: t + 1])[0]
    np.testing.assert_allclose(port.sdpa(q, k, v, True), ref, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("name", sorted(cases.rope_cases()))
def test_rope(port, golden, name):
    x, pos, theta = cases.rope_cases()[name]
    out = port.rope(x, pos, theta)
    _close(out, golden[name])
    if name == "rope_small":  # numpy statement of test_sequence_ops.py:68-79
        half = x.shape[-1] // 2
        inv = theta ** (-2.0 * np.arange(0, half, dtype=np.float32) / x.shape[-1])
        ref = np.empty_like(x)
        for t in range(x.shape[0]):
            c, s = np.cos(pos[t] * inv), np.sin(pos[t] * inv)
            ref[t, :, :half] = x[t, :, :half] * c - x[t, :, half:] * s
            ref[t, :, half:] = x[t, :, half:] * c + x[t, :, :half] * s
        np.testing.assert_allclose(out, ref, rtol=1e-4, atol=1e-5)


def _np_mrope_cos_sin(pos3, inv, h_sec, w_sec):
    """numpy statement of the stride-3 rule as in test_sequence_ops.py:241-249."""
    freqs = pos3[:, :, None].astype(np.float32) * inv[None, None, :]
    out = freqs[0].copy()
    hi = np.arange(1, h_sec * 3, 3)
    wi = np.arange(2, w_sec * 3, 3)
    out[:, hi] = freqs[1][:, hi]
    out[:, wi] = freqs[2][:, wi]
    ang = np.concatenate([out, out], -1)
    return np.cos(ang), np.sin(ang)


@pytest.mark.parametrize("name", sorted(cases.mrope_cases()))
def test_mrope(port, golden, name):
    case = cases.mrope_cases()[name]
    if name.startswith("mrope_cs"):
        pos3, inv, h, w = case
        c, s = port.mrope_cos_sin(pos3, inv, h, w)
        _close(c, golden[name + "_cos"])
        _close(s, golden[name + "_sin"])
        rc, rs = _np_mrope_cos_sin(pos3, inv, h, w)
        np.testing.assert_allclose(c, rc, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(s, rs, rtol=1e-5, atol=1e-6)
    else:
        x, pos3, inv, sec = case
        out = port.rope_thd(x, pos3, inv, sec)
        _close(out, golden[name])
        # rope_thd == rope_with_cos_sin over the mrope tables (same angles)
        c, s = port.mrope_cos_sin(pos3, inv, sec[1], sec[2])
        _close(out, port.rope_with_cos_sin(x, c, s))


def test_mrope_positions_bit_exact(port):
    for n, s, want, h, w in ((1536, 0, 1024, 32, 32), (40, 5, 12, 3, 4), (20, 3, 8, 2, 4)):
        a = port.build_mrope_pos3(n, s, want, h, w)
        b = cases.build_mrope_pos3(n, s, want, h, w)
        assert np.array_equal(a, b)
    # decode position rule (examples/vlm/qwen3vl/model.py:724-727, 746-748)
    full = cases.build_mrope_pos3(1536, 0, 1024, 32, 32)
    rope_delta = max(32, 32) - 1024
    assert full[0, -1] + 1 == 1536 + rope_delta


def test_fused(port, golden):
    f = cases.fused_cases()
    g, u = f["silu_rs0"]
    y = port.silu_mul(g, u)
    _close(y, golden["silu_rs0"])
    np.testing.assert_allclose(y, g / (1.0 + np.exp(-g)) * u, rtol=1e-5, atol=1e-6)
    _close(port.silu_mul(*f["silu_edge"]), golden["silu_edge"])
    for name in ("addrms_rs1", "addrms_c2"):
        x, r, w, eps = f[name]
        yy, out = port.add_rms_norm(x, r, w, eps)
        _close(yy, golden[name + "_y"])
        _close(out, golden[name + "_out"])
        s = x + r
        np.testing.assert_allclose(yy, s, rtol=1e-5, atol=1e-6)
        ref = s / np.sqrt((s**2).mean(-1, keepdims=True) + eps) * w
        np.testing.assert_allclose(out, ref, rtol=1e-4, atol=1e-5)
    for name in ("rms_8x16", "rms_qnorm"):
        x, w, eps = f[name]
        out = port.rms_norm(x, w, eps)
        _close(out, golden[name])
        ref = x / np.sqrt((x**2).mean(-1, keepdims=True) + eps) * w
        np.testing.assert_allclose(out, ref, rtol=1e-4, atol=1e-5)


def test_add_rms_norm_chain(port):
    """y feeds the next layer's residual: tests/core/test_fused.py:69-78 (RandomState(2))."""
    rng = np.random.RandomState(2)
    h = rng.randn(2, 64).astype(np.float32)
    a1 = rng.randn(2, 64).astype(np.float32)
    a2 = rng.randn(2, 64).astype(np.float32)
    w = np.ones(64, np.float32)
    h1, _ = port.add_rms_norm(a1, h, w, 1e-6)
    h2, _ = port.add_rms_norm(a2, h1, w, 1e-6)
    np.testing.assert_allclose(h2, a2 + a1 + h, rtol=1e-5, atol=1e-6)


def test_concat_and_half_bits(port, golden):
    a, b = cases.concat_case()
    out = port.concat_axis0(a, b)
    assert np.array_equal(out.view(np.uint16), golden["concat_fp16_bits"])
    assert np.array_equal(out.view(np.uint16), np.concatenate([a, b]).view(np.uint16))
    bits = np.arange(65536, dtype=np.uint16)
    mine = port.half_to_float(bits).view(np.uint32)
    assert np.array_equal(mine, golden["half_to_float_all_bits"])
    # normal numbers, zeros and infinities widen exactly as IEEE; the reference's subnormal
    # branch (include/axono/core/half.h:63-72) yields half the IEEE value, restated as written.
    ieee = bits.view(np.float16).astype(np.float32).view(np.uint32)
    exp = (bits >> 10) & 0x1F
    normal = (exp != 0) & (exp != 0x1F)
    zero_or_inf = (bits & 0x7FFF == 0) | (bits & 0x7FFF == 0x7C00)
    assert np.array_equal(mine[normal | zero_or_inf], ieee[normal | zero_or_inf])
    sub = (exp == 0) & (bits & 0x3FF != 0)
    assert np.array_equal(mine[sub].view(np.float32) * 2, ieee[sub].view(np.float32))


def test_decode_with_cache_equals_causal_last_row(port):
    """tests/nn/test_kv_cache.py:117-148: attention of the newest token over the appended cache
    equals the last row of a full causal forward."""
    rng = np.random.default_rng(1060)
    s, hq, hkv, d = 9, 4, 2, 16
    q = rng.standard_normal((s, hq, d)).astype(np.float32)
    k = rng.standard_normal((s, hkv, d)).astype(np.float32)
    v = rng.standard_normal((s, hkv, d)).astype(np.float32)
    full = port.sdpa(q, k, v, True)
    kc, vc = k[:1], v[:1]
    for t in range(1, s):
        kc = port.concat_axis0(kc, k[t : t + 1])
        vc = port.concat_axis0(vc, v[t : t + 1])
    last = port.gqa_decode(q[s - 1 : s], kc, vc)
    assert np.array_equal(last[0], full[s - 1])


@pytest.mark.skipif(not oracle.have_reference(), reason="reference library not built in this tree")
def test_port_equals_reference_library(port):
    ref = oracle.reference()
    rng = np.random.default_rng(1070)
    for skv in (1, 3, 64, 65, 1000):
        q = rng.standard_normal((1, 16, 128)).astype(np.float32)
        k = rng.standard_normal((skv, 8, 128)).astype(np.float32)
        v = rng.standard_normal((skv, 8, 128)).astype(np.float32)
        _close(port.gqa_decode(q, k, v), ref.gqa_decode(q, k, v))
    x = rng.standard_normal((6, 8, 128)).astype(np.float32)
    pos = rng.integers(0, 40000, 6)
    _close(port.rope(x, pos, 1e6), ref.rope(x, pos, 1e6))
    pos3 = rng.integers(0, 40000, (3, 6))
    inv = cases.inv_freq(1e6)
    _close(port.rope_thd(x, pos3, inv, (24, 20, 20)), ref.rope_thd(x, pos3, inv, (24, 20, 20)))
    xs = (rng.standard_normal(20000) * 100).astype(np.float32)
    assert np.array_equal(port.float_to_half(xs), ref.float_to_half(xs))
    # the inverse-frequency table equals what the rope op computes internally: rope() and
    # rope_with_cos_sin over cos/sin of float(pos) * table agree bit for bit
    inv_t = port.rope_inv_freq(1e6, 128)
    ang = pos.astype(np.float32)[:, None] * inv_t[None, :]
    one = np.ones((6, 1, 128), np.float32)
    c = ref.rope(one, pos, 1e6)  # a=b=1: out[:half] = c - s, out[half:] = c + s
    cc, ss = port.mrope_cos_sin(np.stack([pos] * 3), inv_t, 0, 0)
    _close(c[:, 0, :64], cc[:, :64] - ss[:, :64], 0.0)
    assert ang.dtype == np.float32


def test_embedding_and_argmax(port):
    rng = np.random.default_rng(1080)
    table = rng.standard_normal((50, 16)).astype(np.float32)
    ids = rng.integers(0, 50, (3, 4))
    assert np.array_equal(port.embedding(ids, table), table[ids])  # tests/core/test_sequence_ops.py:51-55
    x = rng.standard_normal((6, 1000)).astype(np.float32)
    x[1, 10] = x[1, 900] = 99.0  # a tie: the first maximum wins
    x[2, :] = -np.inf
    x[3, 0] = np.nan  # nothing compares greater than NaN: index 0 stays
    x[4, 5] = np.nan
    got = port.argmax_last_dim(x)
    assert got[0] == x[0].argmax() and got[1] == 10 and got[2] == 0 and got[3] == 0
    assert got[4] == np.nanargmax(x[4]) and got[5] == x[5].argmax()
    if oracle.have_reference():
        ref = oracle.reference()
        assert np.array_equal(ref.embedding(ids, table), port.embedding(ids, table))
        assert np.array_equal(ref.argmax_last_dim(x), got)
