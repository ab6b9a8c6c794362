"""Parity of the CUDA path against the CPU oracle, through the C ABI (-m gpu).

Tolerances (per tensor, max|out-ref| / max|ref|): fp32 <= 1e-5; fp16 storage with fp32
accumulation <= 2e-3; cache indexing, appended bytes and positions bit-exact.  The fp16 oracle is
the fp32 oracle run on the exactly-widened fp16 inputs.
"""
import numpy as np
import pytest
import torch

import cases
import oracle

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
F16_TOL = 2e-3


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available()
    from axono_b200 import ops as _ops

    return _ops


@pytest.fixture(scope="module")
def orc():
    return oracle.best()


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def host(t):
    return t.detach().float().cpu().numpy()


def widen(a):
    """fp32 array holding the values an fp16 tensor stores."""
    return a.astype(np.float16).astype(np.float32)


def assert_close(out, ref, tol):
    err = oracle.rel_err(out, ref)
    assert err <= tol, f"rel err {err:.3e} > {tol:.1e}"


# ---- decode attention, reference layout -------------------------------------------------------


@pytest.mark.parametrize("name", sorted(cases.all_gqa_cases()))
def test_gqa_fp32_golden(ops, golden, name):
    q, k, v = cases.all_gqa_cases()[name]
    out = host(ops.gqa_decode_attention(dev(q), dev(k), dev(v)))
    assert_close(out, golden[name], F32_TOL)
    np.testing.assert_allclose(out, golden[name], rtol=1e-4, atol=1e-4)  # the reference's own bar
    assert ops.last_error() == 0


@pytest.mark.parametrize("name", sorted(cases.all_gqa_cases()))
def test_gqa_fp16_golden_inputs(ops, orc, name):
    q, k, v = cases.all_gqa_cases()[name]
    ref = orc.gqa_decode(widen(q), widen(k), widen(v))
    out = host(ops.gqa_decode_attention(dev(q, torch.float16), dev(k, torch.float16), dev(v, torch.float16)))
    assert_close(out, ref, F16_TOL)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("hq,hkv,d", [(16, 8, 128), (8, 8, 128), (32, 8, 128), (64, 8, 128), (16, 1, 128),
                                      (24, 2, 128), (6, 2, 128), (4, 2, 8), (8, 4, 64), (4, 4, 256),
                                      # the generic kernel: other head sizes, groups past one head batch
                                      (32, 2, 80), (16, 8, 96), (40, 2, 64), (18, 1, 256), (3, 3, 48)])
@pytest.mark.parametrize("skv", [1, 63, 64, 65, 255, 257, 2049, 8193])
def test_gqa_shapes(ops, orc, dtype, hq, hkv, d, skv):
    rng = np.random.default_rng(hq * 1000 + hkv * 100 + d + skv)
    q = rng.standard_normal((1, hq, d)).astype(np.float32)
    k = rng.standard_normal((skv, hkv, d)).astype(np.float32)
    v = rng.standard_normal((skv, hkv, d)).astype(np.float32)
    if dtype == torch.float16:
        q, k, v = widen(q), widen(k), widen(v)
    ref = orc.gqa_decode(q, k, v)
    out = host(ops.gqa_decode_attention(dev(q, dtype), dev(k, dtype), dev(v, dtype)))
    assert_close(out, ref, F32_TOL if dtype == torch.float32 else F16_TOL)
    assert ops.last_error() == 0


def test_gqa_sharp_softmax_and_large_logits(ops, orc):
    """One dominant key per head and logits of magnitude ~40: the online max must track it."""
    rng = np.random.default_rng(77)
    skv = 3000
    q = (rng.standard_normal((1, 16, 128)) * 3).astype(np.float32)
    k = rng.standard_normal((skv, 8, 128)).astype(np.float32)
    v = rng.standard_normal((skv, 8, 128)).astype(np.float32)
    k[2999] = q[0, ::2] * 1.5  # the very last token dominates
    k[5] = q[0, 1::2] * 1.2
    for dtype, tol in ((torch.float32, F32_TOL), (torch.float16, F16_TOL)):
        qq, kk, vv = (widen(a) if dtype == torch.float16 else a for a in (q, k, v))
        ref = orc.gqa_decode(qq, kk, vv)
        out = host(ops.gqa_decode_attention(dev(qq, dtype), dev(kk, dtype), dev(vv, dtype)))
        assert_close(out, ref, tol)


def test_gqa_argument_errors(ops):
    q = torch.zeros(1, 16, 128, device="cuda")
    k = torch.zeros(10, 8, 128, device="cuda")
    with pytest.raises(RuntimeError):
        ops.gqa_decode_attention(torch.zeros(2, 16, 128, device="cuda"), k, k)  # sq != 1
    with pytest.raises(RuntimeError):
        ops.gqa_decode_attention(q, k, torch.zeros(10, 8, 64, device="cuda"))  # shape mismatch
    with pytest.raises(RuntimeError):
        ops.gqa_decode_attention(q.double(), k.double(), k.double())  # unsupported dtype
    with pytest.raises(RuntimeError):
        ops.gqa_decode_attention(torch.zeros(1, 12, 128, device="cuda"), k, k)  # hq % hkv != 0


# ---- decode attention, paged and batched ---------------------------------------------------------


def _paged_case(ops, orc, dtype, lens, page_tokens, hq=16, hkv=8, d=128, seed=0, shuffle=True, check=None):
    from axono_b200.kv_cache import PagedKVCache

    rng = np.random.default_rng(seed)
    B, Lmax = len(lens), max(lens)
    q = rng.standard_normal((B, hq, d)).astype(np.float32)
    k = (0.5 * rng.standard_normal((B, Lmax, hkv, d))).astype(np.float32)
    v = (0.5 * rng.standard_normal((B, Lmax, hkv, d))).astype(np.float32)
    if dtype == torch.float16:
        q, k, v = widen(q), widen(k), widen(v)
    cache = PagedKVCache(1, B, hkv, d, Lmax, dtype=dtype, page_tokens=page_tokens)
    if shuffle:
        perm = torch.from_numpy(rng.permutation(cache.num_pages).astype(np.int32))
        cache.block_table = perm.reshape(B, cache.max_blocks).contiguous().cuda()
    # poison the pools so stale bytes past each sequence's end would show up
    cache.k_pages[0].fill_(float("nan"))
    cache.v_pages[0].fill_(float("nan"))
    cache.fill(0, dev(k, dtype), dev(v, dtype), lens)
    for b, n in enumerate(lens):  # re-poison the tail of each sequence's last page
        kb, vb = cache.gather(0, b)
        assert kb.shape[0] == n
    out = host(cache.attend(0, dev(q, dtype)))
    which = range(B) if check is None else check
    tol = F32_TOL if dtype == torch.float32 else F16_TOL
    for b in which:
        ref = orc.gqa_decode(q[b : b + 1], k[b, : lens[b]], v[b, : lens[b]])
        assert_close(out[b : b + 1], ref, tol)
    assert ops.last_error() == 0
    return cache, q, out


def _poison_tail(cache, lens):
    """NaNs in every slot past a sequence's end inside its last page."""
    for b, n in enumerate(lens):
        slot, tok = divmod(n, cache.page_tokens)
        if tok and slot < cache.max_blocks:
            page = int(cache.block_table[b, slot])
            cache.k_pages[0][page, :, tok:, :] = float("nan")
            cache.v_pages[0][page, :, tok:, :] = float("nan")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("page_tokens", [64, 128])
def test_paged_ragged_batch(ops, orc, dtype, page_tokens):
    lens = [1, 63, 64, 65, 700, 2048, 2500]
    cache, q, out = _paged_case(ops, orc, dtype, lens, page_tokens, seed=5)
    _poison_tail(cache, lens)
    out2 = host(cache.attend(0, dev(q, dtype)))
    assert np.array_equal(out, out2), "bytes past the end of a sequence leaked into the result"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_paged_matches_reference_layout_bitwise(ops, dtype):
    """The paged kernel on sequence b and the single-sequence kernel on the gathered cache see the
    same tiles in the same order: identical bits."""
    from axono_b200.kv_cache import PagedKVCache

    rng = np.random.default_rng(9)
    B, L = 3, 4096
    q = dev(rng.standard_normal((B, 16, 128)).astype(np.float32), dtype)
    k = dev(rng.standard_normal((B, L, 8, 128)).astype(np.float32), dtype)
    v = dev(rng.standard_normal((B, L, 8, 128)).astype(np.float32), dtype)
    cache = PagedKVCache(1, B, 8, 128, L, dtype=dtype)
    cache.fill(0, k, v, [L, L, L])
    out = cache.attend(0, q)
    for b in range(B):
        kb, vb = cache.gather(0, b)
        assert torch.equal(kb, k[b]) and torch.equal(vb, v[b])
    # same chunking requires the same (batch, max_len) plan: run the contiguous op per sequence and
    # compare within tolerance, and the paged op against itself with permuted pages bit for bit
    single = torch.cat([ops.gqa_decode_attention(q[b : b + 1], k[b], v[b]) for b in range(B)])
    assert_close(host(out), host(single), F32_TOL if dtype == torch.float32 else F16_TOL)
    perm = torch.randperm(cache.num_pages, generator=torch.Generator().manual_seed(1)).to(torch.int32)
    cache2 = PagedKVCache(1, B, 8, 128, L, dtype=dtype, page_order=perm)
    cache2.fill(0, k, v, [L, L, L])
    assert torch.equal(cache2.attend(0, q), out)


def test_paged_long_context_fp16_properties(ops, orc):
    """Full-size ragged lengths (16K..32K) on a reduced batch: oracle on two sequences, page
    permutation invariance on all."""
    rng = np.random.default_rng(3000)
    lens = rng.integers(16384, 32769, 6).tolist()
    lens[0] = 32768
    _paged_case(ops, orc, torch.float16, lens, 64, seed=11, check=[0, 3])


def test_empty_sequence_in_batch(ops, orc):
    """A sequence of length 0 yields zeros and does not disturb its neighbours."""
    from axono_b200.kv_cache import PagedKVCache

    rng = np.random.default_rng(21)
    lens = [300, 0, 5000]
    q = rng.standard_normal((3, 16, 128)).astype(np.float32)
    k = rng.standard_normal((3, 5000, 8, 128)).astype(np.float32)
    v = rng.standard_normal((3, 5000, 8, 128)).astype(np.float32)
    cache = PagedKVCache(1, 3, 8, 128, 5000, dtype=torch.float32)
    cache.fill(0, dev(k), dev(v), lens)
    out = host(cache.attend(0, dev(q)))
    assert np.all(out[1] == 0)
    for b in (0, 2):
        assert_close(out[b : b + 1], orc.gqa_decode(q[b : b + 1], k[b, : lens[b]], v[b, : lens[b]]), F32_TOL)


# ---- append with RoPE / M-RoPE ---------------------------------------------------------------------


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("mode", ["rope_pos", "rope_len", "mrope", "plain"])
def test_kv_append_rope(ops, orc, dtype, mode):
    from axono_b200.kv_cache import PagedKVCache

    rng = np.random.default_rng(31)
    B, hq, hkv, d = 8, 16, 8, 128
    lens = [0, 1, 63, 64, 127, 128, 500, 8192]
    Lcap = 8192 + 64
    cache = PagedKVCache(1, B, hkv, d, Lcap, dtype=dtype,
                         page_order=torch.from_numpy(rng.permutation(B * ((Lcap + 63) // 64)).astype(np.int32)))
    k0 = rng.standard_normal((B, 8192, hkv, d)).astype(np.float32)
    v0 = rng.standard_normal((B, 8192, hkv, d)).astype(np.float32)
    cache.fill(0, dev(k0, dtype), dev(v0, dtype), lens)
    q = rng.standard_normal((B, hq, d)).astype(np.float32)
    kn = rng.standard_normal((B, hkv, d)).astype(np.float32)
    vn = rng.standard_normal((B, hkv, d)).astype(np.float32)
    if dtype == torch.float16:
        q, kn, vn = widen(q), widen(kn), widen(vn)
    qd, knd, vnd = dev(q, dtype), dev(kn, dtype), dev(vn, dtype)
    theta = 1e6
    inv = cases.inv_freq(theta)
    if mode == "rope_pos":
        pos = rng.integers(0, 40000, B).astype(np.int64)
        cache.append_rope(0, qd, knd, vnd, pos=dev(pos), theta=theta)
        q_ref, k_ref = orc.rope(q, pos, theta), orc.rope(kn, pos, theta)
    elif mode == "rope_len":
        cache.append_rope(0, qd, knd, vnd, theta=theta)
        pos = np.asarray(lens, np.int64)
        q_ref, k_ref = orc.rope(q, pos, theta), orc.rope(kn, pos, theta)
    elif mode == "mrope":
        pos3 = rng.integers(0, 40000, (3, B)).astype(np.int64)
        cache.append_rope(0, qd, knd, vnd, pos=dev(pos3), inv_freq=dev(inv), mrope_section=(24, 20, 20))
        q_ref = orc.rope_thd(q, pos3, inv, (24, 20, 20))
        k_ref = orc.rope_thd(kn, pos3, inv, (24, 20, 20))
    else:
        cache.update(0, knd, vnd)
        q_ref, k_ref = q, kn
    tol = F32_TOL if dtype == torch.float32 else F16_TOL
    assert_close(host(qd), q_ref, tol)
    assert cache.seq_lens.cpu().tolist() == [n + 1 for n in lens]  # positions advance by exactly one
    for b, n in enumerate(lens):
        kb, vb = cache.gather(0, b)
        assert kb.shape[0] == n + 1
        # everything already cached is untouched, the new value row is a byte copy (the reference's
        # concat semantics, src/ops/cpu/sequence.cpp:303-338)
        assert torch.equal(kb[:n], dev(k0[b, :n], dtype)) and torch.equal(vb[:n], dev(v0[b, :n], dtype))
        assert torch.equal(vb[n], vnd[b])
        if mode == "plain":
            assert torch.equal(kb[n], knd[b])
        else:
            assert_close(host(kb[n]), k_ref[b], tol)
    assert ops.last_error() == 0


def test_append_reports_bad_page_and_capacity(ops):
    """Bounds are checked in the kernel: a page id outside the pool or a full sequence sets a bit of
    the error word and writes nothing."""
    from axono_b200.kv_cache import PagedKVCache

    cache = PagedKVCache(1, 2, 8, 128, 128, dtype=torch.float32)
    kn = torch.ones(2, 8, 128, device="cuda")
    cache.block_table[1, 0] = cache.num_pages + 3
    cache.update(0, kn, kn)
    assert ops.last_error() == 2  # AXB200_ERR_BAD_PAGE
    assert cache.seq_lens.cpu().tolist() == [1, 0]
    cache.block_table[1, 0] = 2
    cache.seq_lens.fill_(128)  # at capacity (2 blocks x 64)
    cache.update(0, kn, kn)
    assert ops.last_error() == 4  # AXB200_ERR_CAPACITY
    assert cache.seq_lens.cpu().tolist() == [128, 128]
    assert ops.last_error() == 0


def test_decode_with_cache_equals_causal_last_row(ops, orc):
    """tests/nn/test_kv_cache.py:117-148 of the reference, through the paged cache: appending token by
    token and attending equals the last row of a full causal forward."""
    from axono_b200.kv_cache import PagedKVCache

    rng = np.random.default_rng(41)
    s, hq, hkv, d = 70, 4, 2, 128
    q = rng.standard_normal((s, hq, d)).astype(np.float32)
    k = rng.standard_normal((s, hkv, d)).astype(np.float32)
    v = rng.standard_normal((s, hkv, d)).astype(np.float32)
    full = orc.sdpa(q, k, v, True)
    cache = PagedKVCache(1, 1, hkv, d, 128, dtype=torch.float32)
    for t in range(s):
        cache.update(0, dev(k[t : t + 1]), dev(v[t : t + 1]))
        if t in (0, 1, 63, 64, 69):
            out = host(cache.attend(0, dev(q[t : t + 1])))
            assert_close(out[0], full[t], F32_TOL)
    assert len(cache) == s
    cache.reset()
    assert len(cache) == 0


# ---- stand-alone RoPE family ----------------------------------------------------------------------------


@pytest.mark.parametrize("name", sorted(cases.rope_cases()))
def test_rope_golden(ops, golden, name):
    x, pos, theta = cases.rope_cases()[name]
    out = host(ops.rope(dev(x), dev(pos), theta))
    assert_close(out, golden[name], F32_TOL)
    out16 = host(ops.rope(dev(x, torch.float16), dev(pos), theta))
    assert_close(out16, oracle.port().rope(widen(x), pos, theta), F16_TOL)


@pytest.mark.parametrize("name", sorted(cases.mrope_cases()))
def test_mrope_golden(ops, golden, name):
    case = cases.mrope_cases()[name]
    if name.startswith("mrope_cs"):
        pos3, inv, h, w = case
        c, s = ops.mrope_cos_sin(dev(pos3), dev(inv), h, w)
        np.testing.assert_allclose(host(c), golden[name + "_cos"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(host(s), golden[name + "_sin"], rtol=1e-5, atol=1e-6)
    else:
        x, pos3, inv, sec = case
        out = host(ops.rope_thd(dev(x), dev(pos3), dev(inv), sec))
        assert_close(out, golden[name], F32_TOL)
        c, s = ops.mrope_cos_sin(dev(pos3), dev(inv), sec[1], sec[2])
        out2 = host(ops.rope_with_cos_sin(dev(x), c, s))
        assert_close(out2, golden[name], F32_TOL)


# ---- fused norm / activation -----------------------------------------------------------------------------


def test_fused_golden(ops, golden):
    f = cases.fused_cases()
    for name in ("silu_rs0", "silu_edge"):
        g, u = f[name]
        out = host(ops.silu_mul(dev(g), dev(u)))
        np.testing.assert_allclose(out, golden[name], rtol=1e-5, atol=1e-6)  # tests/core/test_fused.py:25
    for name in ("addrms_rs1", "addrms_c2"):
        x, r, w, eps = f[name]
        y, out = ops.add_rms_norm(dev(x), dev(r), dev(w), eps)
        assert np.array_equal(host(y), golden[name + "_y"])  # one fp32 add: bit-exact
        assert_close(host(out), golden[name + "_out"], F32_TOL)
        np.testing.assert_allclose(host(out), golden[name + "_out"], rtol=1e-4, atol=1e-5)
    for name in ("rms_8x16", "rms_qnorm"):
        x, w, eps = f[name]
        assert_close(host(ops.rms_norm(dev(x), dev(w), eps)), golden[name], F32_TOL)


@pytest.mark.parametrize("shape", [(8, 2048), (8, 6144), (3, 53), (1, 8192), (5, 10000), (37, 128)])
def test_fused_fp16_and_odd_shapes(ops, orc, shape):
    rng = np.random.default_rng(sum(shape))
    x = widen(rng.standard_normal(shape).astype(np.float32))
    r = widen(rng.standard_normal(shape).astype(np.float32))
    w = widen((1 + 0.02 * rng.standard_normal(shape[-1])).astype(np.float32))
    for dtype, tol in ((torch.float32, F32_TOL), (torch.float16, F16_TOL)):
        y, out = ops.add_rms_norm(dev(x, dtype), dev(r, dtype), dev(w, dtype), 1e-6)
        ry, ro = orc.add_rms_norm(x, r, w, 1e-6)
        assert_close(host(y), ry, tol)
        assert_close(host(out), ro, tol)
        assert_close(host(ops.silu_mul(dev(x, dtype), dev(r, dtype))), orc.silu_mul(x, r), tol)
        assert_close(host(ops.rms_norm(dev(x, dtype), dev(w, dtype), 1e-5)), orc.rms_norm(x, w, 1e-5), tol)
    # unaligned views take the scalar paths
    xo = dev(np.concatenate([[0.0], x.reshape(-1)]).astype(np.float32))[1:]
    ro_ = dev(np.concatenate([[0.0], r.reshape(-1)]).astype(np.float32))[1:]
    assert_close(host(ops.silu_mul(xo, ro_)).reshape(shape), orc.silu_mul(x, r), F32_TOL)


def test_add_rms_norm_chain(ops):
    rng = np.random.RandomState(2)
    h, a1, a2 = (rng.randn(2, 64).astype(np.float32) for _ in range(3))
    w = np.ones(64, np.float32)
    h1, _ = ops.add_rms_norm(dev(a1), dev(h), dev(w), 1e-6)
    h2, _ = ops.add_rms_norm(dev(a2), h1, dev(w), 1e-6)
    np.testing.assert_allclose(host(h2), a2 + a1 + h, rtol=1e-5, atol=1e-6)


def test_concat_bit_exact(ops, golden):
    a, b = cases.concat_case()
    out = ops.concat(dev(a), dev(b), 0)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), golden["concat_fp16_bits"])
    rng = np.random.default_rng(51)
    a = rng.standard_normal((2, 3, 4)).astype(np.float32)
    b = rng.standard_normal((2, 3, 5)).astype(np.float32)
    assert np.array_equal(ops.concat(dev(a), dev(b), -1).cpu().numpy(), np.concatenate([a, b], -1))
    b1 = rng.standard_normal((2, 7, 4)).astype(np.float32)
    assert np.array_equal(ops.concat(dev(a), dev(b1), 1).cpu().numpy(), np.concatenate([a, b1], 1))


@pytest.mark.parametrize("pinned", [True, False])
def test_decode_step_host_matches_separate_calls(ops, pinned):
    """The host-buffer step (one C-ABI call: inputs in, rope + append, attend, output out, wait) gives the
    same bits as the device-resident calls it composes - with page-locked buffers, which the kernels read
    and write directly, and with pageable ones, which go through copies."""
    from axono_b200.kv_cache import PagedKVCache

    rng = np.random.default_rng(61)
    B, hq, hkv, d, L = 4, 16, 8, 128, 3000
    lens = [L, 1, 64, 2049]
    k0 = dev((0.5 * rng.standard_normal((B, L, hkv, d))).astype(np.float32), torch.float16)
    v0 = dev((0.5 * rng.standard_normal((B, L, hkv, d))).astype(np.float32), torch.float16)
    caches = []
    for _ in range(2):
        c = PagedKVCache(1, B, hkv, d, L + 64, dtype=torch.float16)
        c.fill(0, k0, v0, lens)
        caches.append(c)
    pin = (lambda t: t.pin_memory()) if pinned else (lambda t: t)
    host = lambda *s: pin(torch.from_numpy(rng.standard_normal(s).astype(np.float16)))  # noqa: E731
    for step in range(3):
        q_h, k_h, v_h = host(B, hq, d), host(B, hkv, d), host(B, hkv, d)
        q_before = q_h.clone()
        out_h = pin(torch.empty_like(q_h))
        caches[0].step_host(q_h, k_h, v_h, out_h, theta=1e6)
        qd = q_h.cuda()
        caches[1].append_rope(0, qd, k_h.cuda(), v_h.cuda(), theta=1e6)
        want = caches[1].attend(0, qd).cpu()
        assert torch.equal(out_h, want), f"step {step}"
        assert torch.equal(q_h, q_before)  # the host's q is an input: it is not rotated in place
    assert torch.equal(caches[0].seq_lens, caches[1].seq_lens)
    assert ops.last_error() == 0


def test_embedding_and_argmax(ops, orc):
    rng = np.random.default_rng(91)
    table = rng.standard_normal((1000, 2048)).astype(np.float32)
    ids = rng.integers(0, 1000, (4, 8))
    for dtype in (torch.float32, torch.float16):
        t = dev(table, dtype)
        for idt in (torch.int64, torch.int32):
            out = ops.embedding(dev(ids).to(idt), t)
            assert torch.equal(out, t[dev(ids)])  # a row copy: bit-exact
    assert np.array_equal(host(ops.embedding(dev(ids), dev(table))), orc.embedding(ids, table))
    odd = rng.standard_normal((7, 37)).astype(np.float32)  # rows that are not 16-byte multiples
    assert torch.equal(ops.embedding(dev(np.array([6, 0, 3])), dev(odd)), dev(odd)[[6, 0, 3]])
    bad = ops.embedding(dev(np.array([1, 1000, -1])), dev(table))
    assert ops.last_error() == 8 and torch.all(bad[1:] == 0) and torch.equal(bad[0], dev(table)[1])
    x = rng.standard_normal((6, 151936)).astype(np.float32)
    x[1, 10] = x[1, 90000] = 99.0
    x[2, :] = -np.inf
    x[3, 0] = np.nan
    x[4, 5] = np.nan
    want = orc.argmax_last_dim(x)
    assert np.array_equal(ops.argmax_last_dim(dev(x)).cpu().numpy(), want)
    x16 = widen(x)
    assert np.array_equal(ops.argmax_last_dim(dev(x16, torch.float16)).cpu().numpy(), orc.argmax_last_dim(x16))
    # rows that are not 16-byte multiples take the element-wise loop; ties at both ends of a row
    y = rng.standard_normal((5, 1001)).astype(np.float32)
    y[0, 0] = y[0, 1000] = 50.0
    y[1, 999] = y[1, 1000] = 50.0
    assert np.array_equal(ops.argmax_last_dim(dev(y)).cpu().numpy(), orc.argmax_last_dim(y))
    y16 = widen(y)
    assert np.array_equal(ops.argmax_last_dim(dev(y16, torch.float16)).cpu().numpy(), orc.argmax_last_dim(y16))
    assert ops.last_error() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("window", [1, 63, 64, 100, 1000, 4096])
def test_sliding_window_attention(ops, orc, dtype, window):
    """Only the last `window` tokens are visible; equals the oracle on the sliced cache."""
    from axono_b200.kv_cache import SlidingWindowKVCache

    rng = np.random.default_rng(window)
    B, hq, hkv, d, Lmax = 6, 16, 8, 128, 5000
    lens = [5000, 1, 64, 65, 2049, 777]
    q = rng.standard_normal((B, hq, d)).astype(np.float32)
    k = (0.5 * rng.standard_normal((B, Lmax, hkv, d))).astype(np.float32)
    v = (0.5 * rng.standard_normal((B, Lmax, hkv, d))).astype(np.float32)
    if dtype == torch.float16:
        q, k, v = widen(q), widen(k), widen(v)
    cache = SlidingWindowKVCache(window, 1, B, hkv, d, Lmax, dtype=dtype)
    cache.fill(0, dev(k, dtype), dev(v, dtype), lens)
    # poison everything before each window: those tokens must not be read into the result
    for b, n in enumerate(lens):
        lo = max(0, n - window)
        for t0 in range(0, lo, 64):
            page = int(cache.block_table[b, t0 // 64])
            hi = min(64, lo - t0)
            cache.k_pages[0][page, :, :hi, :] = float("nan")
            cache.v_pages[0][page, :, :hi, :] = float("nan")
    out = host(cache.attend(0, dev(q, dtype)))
    tol = F32_TOL if dtype == torch.float32 else F16_TOL
    for b, n in enumerate(lens):
        lo = max(0, n - window)
        assert_close(out[b : b + 1], orc.gqa_decode(q[b : b + 1], k[b, lo:n], v[b, lo:n]), tol)
    assert len(cache) == min(max(lens), window)
    assert ops.last_error() == 0


# ---- prefill attention (the SDPA op) ------------------------------------------------------------------------


def test_sdpa_reference_shapes_fp32(ops, golden):
    """The reference's own SDPA test shape (sq 4, skv 6, 4 q / 2 kv heads, d 8), causal and not:
    tests/core/test_sequence_ops.py:85-111 -> golden vectors from the reference's CPU library."""
    q, k, v = cases.sdpa_causal_case()
    assert_close(host(ops.scaled_dot_product_attention(dev(q), dev(k), dev(v), True)), golden["sdpa_causal"], F32_TOL)
    assert_close(host(ops.scaled_dot_product_attention(dev(q), dev(k), dev(v), False)), golden["sdpa_noncausal"], F32_TOL)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sq,skv", [(1, 1), (5, 5), (127, 127), (128, 128), (129, 129), (300, 300), (1000, 1000),
                                    (64, 700), (700, 64), (257, 2049)])
def test_sdpa_fp16_tensor_core_path(ops, orc, causal, sq, skv):
    """fp16, head_dim 128: the tcgen05 kernel against the oracle (causal rule: row t sees min(t+1, skv) keys
    when skv >= t+1, else all)."""
    rng = np.random.default_rng(sq * 7 + skv)
    q = widen(rng.standard_normal((sq, 16, 128)).astype(np.float32))
    k = widen(rng.standard_normal((skv, 8, 128)).astype(np.float32))
    v = widen(rng.standard_normal((skv, 8, 128)).astype(np.float32))
    ref = orc.sdpa(q, k, v, causal)
    out = host(ops.scaled_dot_product_attention(dev(q, torch.float16), dev(k, torch.float16), dev(v, torch.float16), causal))
    assert_close(out, ref, F16_TOL)
    assert ops.last_error() == 0


@pytest.mark.parametrize("dtype,hq,hkv,d", [(torch.float32, 16, 8, 128), (torch.float32, 4, 2, 64), (torch.float16, 4, 4, 64)])
def test_sdpa_row_fallback(ops, orc, dtype, hq, hkv, d):
    rng = np.random.default_rng(d + hq)
    sq, skv = 70, 300
    q = rng.standard_normal((sq, hq, d)).astype(np.float32)
    k = rng.standard_normal((skv, hkv, d)).astype(np.float32)
    v = rng.standard_normal((skv, hkv, d)).astype(np.float32)
    if dtype == torch.float16:
        q, k, v = widen(q), widen(k), widen(v)
    for causal in (False, True):
        out = host(ops.scaled_dot_product_attention(dev(q, dtype), dev(k, dtype), dev(v, dtype), causal))
        assert_close(out, orc.sdpa(q, k, v, causal), F32_TOL if dtype == torch.float32 else F16_TOL)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("hq,hkv,d", [(16, 8, 128), (4, 4, 64), (6, 2, 80), (16, 2, 96), (3, 1, 8), (8, 8, 192)])
@pytest.mark.parametrize("sq,skv", [(16, 16), (70, 300), (300, 70), (257, 257), (1000, 1000), (33, 2049)])
def test_sdpa_tiled_fma_path(ops, orc, dtype, hq, hkv, d, sq, skv):
    """The tiled FMA prefill kernel (FLOAT32, and head sizes other than 128): both mask modes, query
    blocks that do not divide sq, groups 1 / 2 / 3 / 8, more queries than keys and the reverse."""
    rng = np.random.default_rng(sq * 31 + skv * 7 + d + hq)
    q = rng.standard_normal((sq, hq, d)).astype(np.float32)
    k = rng.standard_normal((skv, hkv, d)).astype(np.float32)
    v = rng.standard_normal((skv, hkv, d)).astype(np.float32)
    if dtype == torch.float16:
        if d == 128:
            pytest.skip("fp16 at head_dim 128 runs on the tensor-core kernel")
        q, k, v = widen(q), widen(k), widen(v)
    for causal in (False, True):
        out = host(ops.scaled_dot_product_attention(dev(q, dtype), dev(k, dtype), dev(v, dtype), causal))
        assert_close(out, orc.sdpa(q, k, v, causal), F32_TOL if dtype == torch.float32 else F16_TOL)
    assert ops.last_error() == 0


def test_sdpa_prefill_then_decode_consistency(ops, orc):
    """Prefill's last causal row equals decode attention of that query over the same cache
    (tests/nn/test_kv_cache.py:117-148 of the reference, at a length its SDPA kernel cannot reach)."""
    rng = np.random.default_rng(123)
    s = 2500
    q = dev(rng.standard_normal((s, 16, 128)).astype(np.float32), torch.float16)
    k = dev(rng.standard_normal((s, 8, 128)).astype(np.float32), torch.float16)
    v = dev(rng.standard_normal((s, 8, 128)).astype(np.float32), torch.float16)
    full = ops.scaled_dot_product_attention(q, k, v, True)
    last = ops.gqa_decode_attention(q[s - 1 : s].contiguous(), k, v)
    assert_close(host(full[s - 1 : s]), host(last), 1e-3)


def test_cast_half_float_round_trip(ops):
    """Tensor.cast_to on the device: float32 -> float16 rounds to nearest even, float16 -> float32 is exact."""
    a = torch.randn(1000, 37, device="cuda") * 100
    h = ops.cast(a, torch.float16)
    assert h.dtype == torch.float16 and torch.equal(h, a.half())
    assert torch.equal(ops.cast(h, torch.float32), h.float())
    assert ops.cast(a, torch.float32) is a


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.float16, 4e-3)])
def test_linear_nobias_is_x_wT(ops, dtype, tol):
    """The tower's projection through the C ABI: one cuBLASLt call, algorithm timed on first use."""
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((32, 384), generator=g, device="cuda").to(dtype)
    w = (0.05 * torch.randn((640, 384), generator=g, device="cuda")).to(dtype)
    for _ in range(2):  # the second call reuses the chosen plan
        y = ops.linear_nobias(x, w)
        ref = x.float() @ w.float().t()
        assert y.shape == (32, 640) and oracle.rel_err(y.float().cpu().numpy(), ref.cpu().numpy()) <= tol
    with pytest.raises(RuntimeError):
        ops.linear_nobias(x, w[:, :100].contiguous())


def test_sdpa_long_prefill_rows_match_decode(ops):
    """Full-size property: at 16384 tokens (128 key tiles per query block, both query tiles of a CTA, the
    heaviest-first block order) every sampled causal row equals decode attention of that query over its
    prefix of the same K / V."""
    g = torch.Generator(device="cuda").manual_seed(77)
    s = 16384
    q = torch.randn((s, 16, 128), generator=g, device="cuda").half()
    k = (0.5 * torch.randn((s, 8, 128), generator=g, device="cuda")).half()
    v = (0.5 * torch.randn((s, 8, 128), generator=g, device="cuda")).half()
    full = ops.scaled_dot_product_attention(q, k, v, True)
    for t in (0, 1, 127, 128, 255, 256, 383, 4095, 8191, 8192, 16255, 16383):
        row = ops.gqa_decode_attention(q[t : t + 1].contiguous(), k[: t + 1].contiguous(), v[: t + 1].contiguous())
        assert_close(host(full[t : t + 1]), host(row), 2e-3)
    assert ops.last_error() == 0


@pytest.mark.parametrize("d", [128, 64])
def test_sdpa_tiled_long_rows_match_decode(ops, d):
    """The tiled FMA prefill kernel at 3000 tokens in FLOAT32 (both CTA shapes: 128 virtual rows at
    head_dim 128, and the same at 64): sampled causal rows against decode attention over their prefixes."""
    g = torch.Generator(device="cuda").manual_seed(78 + d)
    s = 3000
    q = torch.randn((s, 16, d), generator=g, device="cuda")
    k = torch.randn((s, 8, d), generator=g, device="cuda")
    v = torch.randn((s, 8, d), generator=g, device="cuda")
    full = ops.scaled_dot_product_attention(q, k, v, True)
    for t in (0, 31, 32, 63, 64, 127, 1000, 2047, 2048, 2999):
        row = ops.gqa_decode_attention(q[t : t + 1].contiguous(), k[: t + 1].contiguous(), v[: t + 1].contiguous())
        assert_close(host(full[t : t + 1]), host(row), 2e-5)
    assert ops.last_error() == 0
