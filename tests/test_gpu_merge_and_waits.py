"""The end of a decode call on the GPU (-m gpu): the merge of the chunk partials by the last CTA of each
(sequence, KV head) against the separate combine kernel, the device-planned chunk lengths, the
capacity flag, and a bounded wait that runs out (a peer that never answers) without hanging anything.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def widen(a):
    return a.astype(np.float16).astype(np.float32)


@pytest.fixture(scope="module")
def lib():
    from axono_b200 import _capi

    return _capi.lib()


@pytest.fixture(params=["host_plan", "device_plan"])
def plan_mode(request, lib):
    """Both ways a one-wave call can be cut into chunks: on the host from the bound (default), on the
    device from the lengths in device memory."""
    lib.axb200_set_device_plan(1 if request.param == "device_plan" else 0)
    yield request.param
    lib.axb200_set_device_plan(0)


@pytest.fixture()
def both_merges(lib):
    """Runs a callable once with the merge fused into the split kernel and once with the separate
    combine kernel; always leaves the default (fused) behind."""

    def run(fn):
        try:
            lib.axb200_set_fused_merge(0)
            separate = fn()
            torch.cuda.synchronize()
        finally:
            lib.axb200_set_fused_merge(1)
        fused = fn()
        torch.cuda.synchronize()
        return fused, separate

    return run


def _cache(dtype, lens, hq, hkv, d, seed, capacity=None):
    from axono_b200.kv_cache import PagedKVCache

    rng = np.random.default_rng(seed)
    B, Lmax = len(lens), max(max(lens), 1)
    q = rng.standard_normal((B, hq, d)).astype(np.float32)
    k = (0.5 * rng.standard_normal((B, Lmax, hkv, d))).astype(np.float32)
    v = (0.5 * rng.standard_normal((B, Lmax, hkv, d))).astype(np.float32)
    if dtype == torch.float16:
        q, k, v = widen(q), widen(k), widen(v)
    cache = PagedKVCache(1, B, hkv, d, capacity or Lmax, dtype=dtype)
    perm = torch.from_numpy(rng.permutation(cache.num_pages).astype(np.int32))
    cache.block_table = perm.reshape(B, cache.max_blocks).contiguous().cuda()
    cache.k_pages[0].fill_(float("nan"))
    cache.v_pages[0].fill_(float("nan"))
    cache.fill(0, dev(k, dtype), dev(v, dtype), lens)
    return cache, q, k, v


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("hq,hkv,d", [(16, 8, 128), (6, 2, 80), (16, 1, 128), (8, 2, 64)])
def test_fused_merge_equals_combine_kernel_bit_for_bit(both_merges, plan_mode, dtype, hq, hkv, d):
    from axono_b200 import ops

    lens = [9000, 0, 1, 300, 4097, 64, 2500]
    cache, q, k, v = _cache(dtype, lens, hq, hkv, d, seed=31)
    qd = dev(q, dtype)
    fused, separate = both_merges(lambda: cache.attend(0, qd).clone())
    assert torch.equal(fused, separate)
    orc = oracle.best()
    tol = 1e-5 if dtype == torch.float32 else 2e-3
    out = fused.float().cpu().numpy()
    assert np.all(out[1] == 0)
    for b in (0, 2, 3, 4, 6):
        assert oracle.rel_err(out[b : b + 1], orc.gqa_decode(q[b : b + 1], k[b, : lens[b]], v[b, : lens[b]])) <= tol
    # under a window, chunks that lie wholly before it never arrive: the count must not wait for them
    fw, sw = both_merges(lambda: cache.attend(0, qd, window=1000).clone())
    assert torch.equal(fw, sw)
    ref = orc.gqa_decode(q[0:1], k[0, lens[0] - 1000 : lens[0]], v[0, lens[0] - 1000 : lens[0]])
    assert oracle.rel_err(fw[0:1].float().cpu().numpy(), ref) <= tol
    # the merge leaves its counters at zero: a second pass over the same workspace gives the same bits
    assert torch.equal(cache.attend(0, qd), fused)
    assert ops.last_error() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_fused_merge_reference_layout(both_merges, plan_mode, dtype):
    """One sequence in the reference's layout: the host-visible op, long enough for many chunks."""
    from axono_b200 import ops

    rng = np.random.default_rng(32)
    for d, skv in ((128, 20000), (64, 9000)):
        q = dev(rng.standard_normal((1, 16, d)).astype(np.float32), dtype)
        k = dev((0.5 * rng.standard_normal((skv, 8, d))).astype(np.float32), dtype)
        v = dev((0.5 * rng.standard_normal((skv, 8, d))).astype(np.float32), dtype)
        fused, separate = both_merges(lambda: ops.gqa_decode_attention(q, k, v))
        assert torch.equal(fused, separate)
        ref = oracle.best().gqa_decode(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy())
        assert oracle.rel_err(fused.float().cpu().numpy(), ref) <= (1e-5 if dtype == torch.float32 else 2e-3)
    assert ops.last_error() == 0


def test_one_wave_of_very_ragged_lengths(plan_mode):
    """Lengths from 1 to 32768 in one small batch: the device picks the chunk length from them; results
    against the oracle, and bit-identical when the same sequences sit in other batch rows (another
    prefix sum, the same chunks)."""
    from axono_b200 import ops

    lens = [32768, 1, 17000, 300, 25000]
    cache, q, k, v = _cache(torch.float16, lens, 16, 8, 128, seed=33)
    out = cache.attend(0, dev(q, torch.float16))
    orc = oracle.best()
    for b in (0, 1, 3):
        ref = orc.gqa_decode(q[b : b + 1], k[b, : lens[b]], v[b, : lens[b]])
        assert oracle.rel_err(out[b : b + 1].float().cpu().numpy(), ref) <= 2e-3
    order = [4, 2, 0, 3, 1]
    cache2, _, _, _ = _cache(torch.float16, lens, 16, 8, 128, seed=33)
    cache2.block_table = cache2.block_table[order].contiguous()
    cache2.seq_lens.copy_(torch.tensor([lens[i] for i in order], dtype=torch.int32))
    out2 = cache2.attend(0, dev(q[order], torch.float16))
    assert torch.equal(out2, out[order])
    assert ops.last_error() == 0


def test_length_beyond_the_host_bound_sets_the_capacity_flag():
    """A caller whose host-side bound lags behind the device lengths (a replayed graph that was not
    noted) used to get a silently truncated result.  Large launch (host-planned chunk length): the
    flag is raised and the covered prefix is what is attended; small launch (planned on the device from
    the real lengths): the whole sequence is attended and nothing is flagged."""
    from axono_b200 import _capi, ops

    from axono_b200.kv_cache import PagedKVCache

    B, hq, hkv, d = 64, 16, 8, 128
    lens = [6000] * B
    lens[5] = 11000
    cache = PagedKVCache(1, B, hkv, d, 11008, dtype=torch.float16)
    gen = torch.Generator(device="cuda").manual_seed(34)
    for pool in (cache.k_pages[0], cache.v_pages[0]):  # contents straight on the device: 1.4 GB a pool
        for p0 in range(0, pool.shape[0], 1024):
            n = min(1024, pool.shape[0] - p0)
            pool[p0 : p0 + n] = (0.5 * torch.randn((n,) + tuple(pool.shape[1:]), generator=gen, device="cuda")).half()
    cache.seq_lens.copy_(torch.tensor(lens, dtype=torch.int32))
    qd = torch.randn((B, hq, d), generator=gen, device="cuda").half()
    q = qd.float().cpu().numpy()

    def kv(b, n):  # the first n cached tokens of sequence b, token-major, as the oracle wants them
        kb, vb = cache.gather(0, b)
        return kb[:n].float().cpu().numpy(), vb[:n].float().cpu().numpy()

    bound = 8192
    ct = np.zeros(B, np.int32)
    n = np.zeros(B, np.int32)
    mc = C.c_int32(0)
    _capi.lib().axb200_gqa_chunk_plan(np.asarray(lens, np.int32).ctypes.data, B, hq, hkv, d, bound, ct.ctypes.data,
                                      n.ctypes.data, C.byref(mc), None)
    cover = int(ct[5]) * mc.value
    assert bound <= cover < lens[5]
    out = ops.gqa_decode_attention_paged(qd, cache.k_pages[0], cache.v_pages[0], cache.block_table, cache.seq_lens, bound)
    torch.cuda.synchronize()
    assert ops.last_error() & 4
    orc = oracle.best()
    assert oracle.rel_err(out[5:6].float().cpu().numpy(), orc.gqa_decode(q[5:6], *kv(5, cover))) <= 2e-3
    assert oracle.rel_err(out[6:7].float().cpu().numpy(), orc.gqa_decode(q[6:7], *kv(6, 6000))) <= 2e-3
    assert ops.last_error() == 0
    # four sequences only, planned on the device from the real lengths: the bound does not matter
    _capi.lib().axb200_set_device_plan(1)
    small = ops.gqa_decode_attention_paged(qd[4:8].contiguous(), cache.k_pages[0], cache.v_pages[0],
                                           cache.block_table[4:8].contiguous(), cache.seq_lens[4:8].contiguous(), bound)
    assert ops.last_error() == 0
    _capi.lib().axb200_set_device_plan(0)
    assert oracle.rel_err(small[1:2].float().cpu().numpy(), orc.gqa_decode(q[5:6], *kv(5, 11000))) <= 2e-3


def test_peer_wait_runs_out_and_the_context_survives(lib):
    """Failure detection without a fault: rank 0 of a two-rank head-sharded call whose peer never
    publishes (the "peer" buffers are local allocations nobody writes to).  With a 2 ms limit the wait
    gives up, the call returns, AXB200_ERR_WAIT_TIMEOUT is reported, this rank's own rows are in place,
    and the next ordinary call is clean."""
    from axono_b200 import _capi, ops

    B, hq, hkv, d, L = 4, 4, 2, 128, 3000
    lens = [L, 700, 64, 2049]
    cache, q, k, v = _cache(torch.float16, lens, hq, hkv, d, seed=35)
    qd = dev(q, torch.float16)
    want = cache.attend(0, qd)
    hq_total = 2 * hq
    out_bytes = B * hq_total * d * 2

    def alloc(nbytes):
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        _capi.check(lib.axb200_p2p_alloc(nbytes, C.byref(ptr), handle), "p2p_alloc")
        return ptr.value

    outs = [alloc(out_bytes), alloc(out_bytes)]        # mine, and the absent peer's
    flags = [alloc(256), alloc(256)]
    state = alloc(256)
    arr = C.c_void_p * 2
    ws = ops.workspace("cuda", ops.gqa_workspace_bytes(B, hq, hkv, d, L))
    try:
        assert lib.axb200_set_wait_limit_ns(2_000_000) == 0
        st = lib.axb200_gqa_decode_paged_gather(
            qd.data_ptr(), cache.k_pages[0].data_ptr(), cache.v_pages[0].data_ptr(), cache.block_table.data_ptr(),
            cache.seq_lens.data_ptr(), B, hq, hkv, d, cache.page_tokens, cache.max_blocks, cache.num_pages, L,
            _capi.FLOAT16, ws.data_ptr(), ws.numel(), arr(*outs), arr(*flags), state, 2, 0, hq_total,
            torch.cuda.current_stream().cuda_stream)
        assert st == 0
        torch.cuda.synchronize()  # returns: the wait gave up after its limit
        assert ops.last_error() == 1  # AXB200_ERR_WAIT_TIMEOUT, and the word is cleared by the read
    finally:
        lib.axb200_set_wait_limit_ns(2_000_000_000)
    from axono_b200.kv_cache import _DeviceView

    mine = torch.as_tensor(_DeviceView(outs[0], (B, hq_total, d), "<f2"), device="cuda")
    assert torch.equal(mine[:, :hq], want)  # rank 0's heads landed in its own gathered buffer
    peer = torch.as_tensor(_DeviceView(outs[1], (B, hq_total, d), "<f2"), device="cuda")
    assert torch.equal(peer[:, :hq], want)  # ... and in the peer's
    assert torch.equal(cache.attend(0, qd), want) and ops.last_error() == 0
    del mine, peer
    for p in outs + flags + [state]:
        lib.axb200_p2p_free(p)


def test_setting_validation(lib):
    assert lib.axb200_set_wait_limit_ns(0) == 1  # INVALID_ARGUMENT
    assert lib.axb200_set_wait_limit_ns(2_000_000_000) == 0


def test_chunk_length_override_changes_nothing_but_rounding(lib):
    from axono_b200 import ops

    lens = [5000, 300, 2049]
    cache, q, k, v = _cache(torch.float32, lens, 16, 8, 128, seed=36)
    qd = dev(q)
    base = cache.attend(0, qd).clone()
    try:
        for tiles in (4, 7, 64):
            assert lib.axb200_set_chunk_tiles(tiles) == 0
            got = cache.attend(0, qd)
            assert oracle.rel_err(got.cpu().numpy(), base.cpu().numpy()) <= 2e-6
    finally:
        lib.axb200_set_chunk_tiles(0)
    assert ops.last_error() == 0


@pytest.mark.parametrize("hq,hkv", [(16, 8), (32, 8), (8, 8), (12, 4)])
def test_head_dim_64_on_the_tma_kernel(hq, hkv):
    """fp16 with head_dim 64 runs on the TMA / tensor-core split kernel (one 64 x 64 box per tile): ragged
    paged batch against the oracle, page-permutation invariance, and the reference layout."""
    from axono_b200 import ops

    lens = [4100, 1, 63, 64, 65, 9000, 2500]
    cache, q, k, v = _cache(torch.float16, lens, hq, hkv, 64, seed=37)
    qd = dev(q, torch.float16)
    out = cache.attend(0, qd)
    orc = oracle.best()
    for b in range(len(lens)):
        ref = orc.gqa_decode(q[b : b + 1], k[b, : lens[b]], v[b, : lens[b]])
        assert oracle.rel_err(out[b : b + 1].float().cpu().numpy(), ref) <= 2e-3, b
    cache2, _, _, _ = _cache(torch.float16, lens, hq, hkv, 64, seed=37)
    perm = torch.randperm(cache2.num_pages, generator=torch.Generator().manual_seed(5)).to(torch.int32)
    from axono_b200.kv_cache import PagedKVCache

    cache3 = PagedKVCache(1, len(lens), hkv, 64, max(lens), dtype=torch.float16, page_order=perm)
    cache3.fill(0, dev(k, torch.float16), dev(v, torch.float16), lens)
    assert torch.equal(cache3.attend(0, qd), out)
    single = ops.gqa_decode_attention(qd[5:6].contiguous(), dev(k[5, :9000], torch.float16), dev(v[5, :9000], torch.float16))
    assert oracle.rel_err(single.float().cpu().numpy(), orc.gqa_decode(q[5:6], k[5, :9000], v[5, :9000])) <= 2e-3
    assert ops.last_error() == 0


@pytest.mark.parametrize("seed", range(12))
def test_random_paged_batches_against_the_oracle(seed, lib):
    """Seeded random configurations of the batched decode call - batch, head counts, head_dim (both TMA
    shapes and a generic one), dtype, page size, ragged lengths with empty and one-token sequences, an
    optional sliding window, either chunk plan, either merge - every sequence against the oracle."""
    from axono_b200 import ops
    from axono_b200.kv_cache import PagedKVCache

    rng = np.random.default_rng(9000 + seed)
    d = int(rng.choice([128, 128, 64, 80]))
    hkv = int(rng.choice([1, 2, 4, 8]))
    group = int(rng.choice([1, 2, 4]) if d != 80 else rng.choice([1, 3]))
    hq = hkv * group
    dtype = torch.float16 if (d == 64 or rng.random() < 0.6) else torch.float32
    B = int(rng.integers(1, 7))
    lens = [int(x) for x in rng.choice([0, 1, 63, 64, 65, 700, 2049, 5000, 9000], B)]
    if max(lens) == 0:
        lens[0] = 300
    page_tokens = int(rng.choice([64, 128]))
    window = int(rng.choice([0, 0, 100, 1000]))
    lib.axb200_set_device_plan(int(rng.integers(0, 2)))
    lib.axb200_set_fused_merge(int(rng.integers(0, 2)))
    try:
        Lmax = max(lens)
        q = rng.standard_normal((B, hq, d)).astype(np.float32)
        k = (0.5 * rng.standard_normal((B, Lmax, hkv, d))).astype(np.float32)
        v = (0.5 * rng.standard_normal((B, Lmax, hkv, d))).astype(np.float32)
        if dtype == torch.float16:
            q, k, v = widen(q), widen(k), widen(v)
        cache = PagedKVCache(1, B, hkv, d, Lmax, dtype=dtype, page_tokens=page_tokens)
        perm = torch.from_numpy(rng.permutation(cache.num_pages).astype(np.int32))
        cache.block_table = perm.reshape(B, cache.max_blocks).contiguous().cuda()
        cache.k_pages[0].fill_(float("nan"))
        cache.v_pages[0].fill_(float("nan"))
        cache.fill(0, dev(k, dtype), dev(v, dtype), lens)
        out = cache.attend(0, dev(q, dtype), window=window).float().cpu().numpy()
        torch.cuda.synchronize()
    finally:
        lib.axb200_set_device_plan(0)
        lib.axb200_set_fused_merge(1)
    assert ops.last_error() == 0
    orc = oracle.best()
    tol = 1e-5 if dtype == torch.float32 else 2e-3
    for b, n in enumerate(lens):
        if n == 0:
            assert np.all(out[b] == 0)
            continue
        lo = max(0, n - window) if window else 0
        ref = orc.gqa_decode(q[b : b + 1], k[b, lo:n], v[b, lo:n])
        err = oracle.rel_err(out[b : b + 1], ref)
        assert err <= tol, f"seed {seed} d={d} hq={hq} hkv={hkv} {dtype} lens={lens} window={window} b={b}: {err:.3e}"


@pytest.mark.parametrize("d,hq,hkv", [(8, 4, 2), (48, 6, 2), (72, 8, 8), (80, 32, 2), (96, 16, 8), (120, 4, 4)])
def test_fp16_head_sizes_below_the_tile_width(d, hq, hkv):
    """fp16 head sizes that are multiples of 8 up to 128 ride in the 64- or 128-wide TMA tile: the columns
    past the head size lie outside the tensor map and read as zeros.  Paged and reference layout, against
    the oracle; NaN poison in every unused slot shows that nothing beyond a row's own bytes is read."""
    from axono_b200 import ops

    lens = [3000, 65, 1, 8200]
    cache, q, k, v = _cache(torch.float16, lens, hq, hkv, d, seed=38)
    qd = dev(q, torch.float16)
    out = cache.attend(0, qd).float().cpu().numpy()
    orc = oracle.best()
    for b in range(len(lens)):
        ref = orc.gqa_decode(q[b : b + 1], k[b, : lens[b]], v[b, : lens[b]])
        assert oracle.rel_err(out[b : b + 1], ref) <= 2e-3, (d, b)
    single = ops.gqa_decode_attention(qd[3:4].contiguous(), dev(k[3, :8200], torch.float16), dev(v[3, :8200], torch.float16))
    assert oracle.rel_err(single.float().cpu().numpy(), orc.gqa_decode(q[3:4], k[3, :8200], v[3, :8200])) <= 2e-3
    assert np.isfinite(out).all() and ops.last_error() == 0
