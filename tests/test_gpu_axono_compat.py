"""`import axono` (the compatibility package over the native module) used the way the reference's
own tests use the reference (axono/python/tests/core/{test_gqa,test_fused,test_sequence_ops}.py,
tests/nn/test_kv_cache.py): numpy restatements of the math, the reference's seeds, shapes and
tolerances (rtol = atol = 1e-4 for attention and rope, 1e-5 / 1e-4 for the fused ops), plus the split-K
sizes (skv >= 2048) that the reference's tests never reach.  No PyTorch."""
import math

import numpy as np
import pytest

import axono_b200.compat as compat

compat.install()
import axono  # noqa: E402
from axono import Tensor, nn  # noqa: E402
import axono.fused as F  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture()
def cuda_env():
    assert axono.cuda_available()
    axono.set_backend("cuda")
    yield
    axono.set_backend("cpu")


def _ref_gqa(q, k, v):
    sq, hq, d = q.shape
    skv, hkv = k.shape[:2]
    group = hq // hkv
    out = np.zeros((sq, hq, d), np.float32)
    for h in range(hq):
        scores = (q[0, h].astype(np.float64) @ k[:, h // group].T.astype(np.float64)) / math.sqrt(d)
        w = np.exp(scores - scores.max())
        out[0, h] = (w / w.sum()) @ v[:, h // group]
    return out


def _t(arr, device="cuda"):
    return Tensor.from_numpy(np.ascontiguousarray(arr, dtype=np.float32)).to(device)


def test_gqa_decode_matches_numpy(cuda_env):
    rng = np.random.RandomState(3)
    for skv in (1, 7, 256, 512, 1024, 2048, 4096, 10000):
        q, k, v = (rng.randn(*s).astype(np.float32) for s in ((1, 16, 128), (skv, 8, 128), (skv, 8, 128)))
        out = axono.gqa_decode_attention(_t(q), _t(k), _t(v)).to_numpy()
        np.testing.assert_allclose(out, _ref_gqa(q, k, v), rtol=1e-4, atol=1e-4)


def test_gqa_decode_matches_sdpa_op(cuda_env):
    rng = np.random.RandomState(4)
    q, k, v = (rng.randn(*s).astype(np.float32) for s in ((1, 16, 128), (300, 8, 128), (300, 8, 128)))
    qt, kt, vt = _t(q), _t(k), _t(v)
    a1 = axono.gqa.gqa_decode_attention(qt, kt, vt).to_numpy()
    a2 = axono.scaled_dot_product_attention(qt, kt, vt, False).to_numpy()
    np.testing.assert_allclose(a1, a2, rtol=1e-4, atol=1e-4)


def test_fused_ops(cuda_env):
    rng = np.random.RandomState(0)
    g, u = rng.randn(4, 37).astype(np.float32), rng.randn(4, 37).astype(np.float32)
    np.testing.assert_allclose(F.silu_mul(_t(g), _t(u)).to_numpy(), g / (1 + np.exp(-g)) * u, rtol=1e-5, atol=1e-6)
    rng = np.random.RandomState(1)
    x, r, w = rng.randn(6, 64).astype(np.float32), rng.randn(6, 64).astype(np.float32), rng.randn(64).astype(np.float32)
    y, out = F.add_rms_norm(_t(x), _t(r), _t(w), 1e-6)
    yy = x + r
    np.testing.assert_allclose(y.to_numpy(), yy, rtol=1e-6)
    np.testing.assert_allclose(out.to_numpy(), yy / np.sqrt((yy * yy).mean(-1, keepdims=True) + 1e-6) * w, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(axono.rms_norm(_t(x), _t(w)).to_numpy(),
                               x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-5) * w, rtol=1e-4, atol=1e-5)


def test_rope_default_theta_and_thd(cuda_env):
    rng = np.random.RandomState(5)
    s, h, d = 6, 2, 8
    x = rng.randn(s, h, d).astype(np.float32)
    pos = np.arange(s, dtype=np.int64)
    out = axono.rope(_t(x), Tensor.from_numpy(pos).to("cuda")).to_numpy()  # theta defaults to 10000
    inv = (1.0 / (10000.0 ** (np.arange(0, d, 2, dtype=np.float32) / d))).astype(np.float32)
    ang = pos[:, None].astype(np.float32) * inv[None]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., : d // 2], x[..., d // 2:]
    np.testing.assert_allclose(out, np.concatenate([a * cos - b * sin, b * cos + a * sin], -1), rtol=1e-4, atol=1e-4)
    # rope_thd with equal t / h / w positions is plain rope with the same inv_freq
    pos3 = np.stack([pos, pos, pos]).astype(np.int64)
    thd = axono.rope_thd(_t(x), Tensor.from_numpy(pos3).to("cuda"), _t(inv), [2, 1, 1]).to_numpy()
    np.testing.assert_allclose(thd, out, rtol=1e-4, atol=1e-4)


def _kv(seq, heads, d, seed):
    return _t(np.random.RandomState(seed).randn(seq, heads, d))


def test_dynamic_kv_cache_contract(cuda_env):
    cache = nn.DynamicKVCache(2, device="cuda")
    assert len(cache) == 0
    with pytest.raises(RuntimeError):
        cache.get(0)
    k1, v1 = _kv(3, 2, 4, 0), _kv(3, 2, 4, 1)
    cache.update(0, k1, v1)
    assert len(cache) == 3 and cache.get(0)[0].data_ptr == k1.data_ptr  # the first update stores the tensor itself
    k2, v2 = _kv(1, 2, 4, 2), _kv(1, 2, 4, 3)
    cache.update(0, k2, v2)
    k, v = cache.get(0)
    assert len(cache) == 4 and v.shape == (4, 2, 4)
    assert np.array_equal(k.to_numpy()[:3], k1.to_numpy()) and np.array_equal(k.to_numpy()[3], k2.to_numpy()[0])
    cache.update(1, _kv(5, 1, 4, 4), _kv(5, 1, 4, 5))
    assert cache.get(1)[0].shape == (5, 1, 4) and len(cache) == 4  # layers are independent
    cache.reset()
    assert len(cache) == 0
    assert isinstance(cache, nn.KVCache)


def test_decode_with_cache_equals_causal_forward(cuda_env):
    """Token-by-token decode over a DynamicKVCache gives the rows of one causal attention over the whole
    sequence (axono/python/tests/nn/test_kv_cache.py:116-148)."""
    rng = np.random.RandomState(6)
    s, hq, hkv, d = 9, 4, 2, 16
    q, k, v = (rng.randn(*sh).astype(np.float32) for sh in ((s, hq, d), (s, hkv, d), (s, hkv, d)))
    full = axono.scaled_dot_product_attention(_t(q), _t(k), _t(v), True).to_numpy()
    cache = nn.DynamicKVCache(1, device="cuda")
    for t in range(s):
        cache.update(0, _t(k[t:t + 1]), _t(v[t:t + 1]))
        kc, vc = cache.get(0)
        step = axono.gqa_decode_attention(_t(q[t:t + 1]), kc, vc).to_numpy()
        np.testing.assert_allclose(step[0], full[t], rtol=1e-4, atol=1e-4)


def test_paged_cache_decode_matches_dynamic_cache(cuda_env):
    """The paged cache (append with rope in one launch, attention from pages) against the reference's
    operator sequence rope -> DynamicKVCache.update -> gqa_decode_attention, three sequences, two layers."""
    rng = np.random.RandomState(7)
    batch, hq, hkv, d, layers = 3, 8, 2, 128, 2
    paged = nn.PagedKVCache(layers, batch, hkv, d, 256, dtype=axono.DataType.FLOAT32)
    dyn = [nn.DynamicKVCache(layers, device="cuda") for _ in range(batch)]
    for step in range(4):
        for layer in range(layers):
            q, k, v = (rng.randn(*sh).astype(np.float32) for sh in ((batch, hq, d), (batch, hkv, d), (batch, hkv, d)))
            qd = _t(q)
            paged.update(layer, _t(k), _t(v), q=qd, theta=1e6)
            got = paged.attend(layer, qd).to_numpy()
            pos = Tensor.from_numpy(np.array([step], np.int64)).to("cuda")
            for b in range(batch):
                dyn[b].update(layer, axono.rope(_t(k[b:b + 1]), pos, 1e6), _t(v[b:b + 1]))
                kc, vc = dyn[b].get(layer)
                ref = axono.gqa_decode_attention(axono.rope(_t(q[b:b + 1]), pos, 1e6), kc, vc).to_numpy()
                np.testing.assert_allclose(got[b:b + 1], ref, rtol=1e-5, atol=1e-5)
    assert len(paged) == 4
    paged.reset()
    assert len(paged) == 0


def test_compile_and_graph_through_axono(cuda_env):
    w = _t(np.ones(64))

    def block(x, r):
        y, xn = F.add_rms_norm(x, r, w, 1e-6)
        return F.silu_mul(xn, y)

    rng = np.random.RandomState(8)
    x, r = rng.randn(4, 64).astype(np.float32), rng.randn(4, 64).astype(np.float32)
    m = axono.compile(block)
    out = m(_t(x), _t(r)).to_numpy().copy()
    yy = x + r
    xn = yy / np.sqrt((yy * yy).mean(-1, keepdims=True) + 1e-6)
    np.testing.assert_allclose(out, xn / (1 + np.exp(-xn)) * yy, rtol=1e-4, atol=1e-5)
    xt, rt = _t(x), _t(r)
    with axono.cuda_graph() as g:
        g.output = block(xt, rt)
    g.replay()
    g.sync()
    np.testing.assert_allclose(g.output.to_numpy(), out, rtol=1e-6)
    g.reset()


def test_half_tensors_round_trip(cuda_env):
    a = np.random.RandomState(9).randn(5, 7).astype(np.float32)
    h = _t(a).cast_to(axono.DataType.FLOAT16)
    assert h.to_numpy().dtype == np.int16  # raw bits, viewed as float16 by the caller
    np.testing.assert_array_equal(h.to_numpy().view(np.float16), a.astype(np.float16))
