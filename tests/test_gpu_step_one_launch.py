"""The decode step as one operator on the GPU (-m gpu): `axb200_decode_step_paged` - rope(q), rope(k_new),
append, attention - against the two kernels it replaces (kv_append_rope, then gqa_decode_attention_paged),
bit for bit: the attention output, every byte of the pages, the lengths; q is left as it was.  Where the
one-launch form applies (fp16, head_dim 64 or 128) it is the attention kernel itself that appends; elsewhere
the operator runs the two kernels.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    from axono_b200 import _capi

    return _capi.lib()


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def _two_caches(dtype, lens, hkv, d, seed, capacity):
    """Two caches with the same scattered pages and the same contents (unused slots hold NaN)."""
    from axono_b200.kv_cache import PagedKVCache

    rng = np.random.default_rng(seed)
    B, Lmax = len(lens), max(max(lens), 1)
    k = (0.5 * rng.standard_normal((B, Lmax, hkv, d))).astype(np.float32)
    v = (0.5 * rng.standard_normal((B, Lmax, hkv, d))).astype(np.float32)
    perm = None
    caches = []
    for _ in range(2):
        cache = PagedKVCache(1, B, hkv, d, capacity, dtype=dtype)
        if perm is None:
            perm = torch.from_numpy(rng.permutation(cache.num_pages).astype(np.int32))
        cache.block_table = perm.reshape(B, cache.max_blocks).contiguous().cuda()
        cache.k_pages[0].fill_(float("nan"))
        cache.v_pages[0].fill_(float("nan"))
        cache.fill(0, dev(k, dtype), dev(v, dtype), lens)
        caches.append(cache)
    return caches


def _same_bytes(a, b):
    """Equal as bytes (NaN-filled unused slots compare equal to themselves)."""
    return torch.equal(a.view(torch.int16 if a.dtype == torch.float16 else torch.int32),
                       b.view(torch.int16 if b.dtype == torch.float16 else torch.int32))


def _steps(lib, dtype, lens, hq, hkv, d, seed, capacity, n_steps=3, pos_mode="length", expect_launches=None):
    from axono_b200 import _capi, ops

    one, two = _two_caches(dtype, lens, hkv, d, seed, capacity)
    rng = np.random.default_rng(seed + 1)
    B = len(lens)
    code = _capi.FLOAT16 if dtype == torch.float16 else _capi.FLOAT32
    if expect_launches is not None:
        assert lib.axb200_decode_step_launches(B, hq, hkv, d, capacity, code) == expect_launches
    inv_freq = dev((1e4 ** (-np.arange(d // 2, dtype=np.float32) * 2 / d)).astype(np.float32))
    for step in range(n_steps):
        q = dev(rng.standard_normal((B, hq, d)).astype(np.float32), dtype)
        kn = dev((0.5 * rng.standard_normal((B, hkv, d))).astype(np.float32), dtype)
        vn = dev((0.5 * rng.standard_normal((B, hkv, d))).astype(np.float32), dtype)
        kw = {}
        if pos_mode == "explicit":
            kw = {"pos": dev(rng.integers(0, 40000, B).astype(np.int64))}
        elif pos_mode == "mrope":
            kw = {"pos": dev(rng.integers(0, 40000, (3, B)).astype(np.int64)), "inv_freq": inv_freq,
                  "mrope_section": (d // 2 - 2 * (d // 6), d // 6, d // 6)}
        q_before = q.clone()
        out_one = one.step(0, q, kn, vn, theta=1e6, **kw)
        assert torch.equal(q, q_before), "the step operator must not rotate the caller's q"
        q2 = q.clone()
        two.append_rope(0, q2, kn, vn, theta=1e6, **kw)
        out_two = two.attend(0, q2)
        torch.cuda.synchronize()
        assert ops.last_error() == 0
        assert torch.equal(one.seq_lens, two.seq_lens), f"step {step}"
        assert _same_bytes(one.k_pages[0], two.k_pages[0]) and _same_bytes(one.v_pages[0], two.v_pages[0]), f"step {step}"
        assert _same_bytes(out_one, out_two), f"step {step}"
    return one, out_one, q2


@pytest.mark.parametrize("hq,hkv,d", [(16, 8, 128), (8, 8, 128), (32, 2, 128), (8, 2, 64), (16, 4, 64)])
@pytest.mark.parametrize("pos_mode", ["length", "explicit", "mrope"])
def test_one_launch_step_equals_the_two_kernels(lib, hq, hkv, d, pos_mode):
    # lengths on every edge: empty, the token opens a tile / a page, closes one, many chunks
    lens = [0, 1, 62, 63, 64, 127, 128, 300, 4095, 4096, 9000]
    _steps(lib, torch.float16, lens, hq, hkv, d, seed=5, capacity=9216, pos_mode=pos_mode, expect_launches=1)


def test_one_launch_step_in_one_wave_and_in_many(lib):
    # one wave (few long sequences, several chunks each) and a large ragged batch (host-planned chunk grid)
    _steps(lib, torch.float16, [8192] * 8, 16, 8, 128, seed=6, capacity=8192 + 64, expect_launches=1)
    rng = np.random.default_rng(7)
    _steps(lib, torch.float16, rng.integers(1, 3000, 96).tolist(), 16, 8, 128, seed=8, capacity=3072, n_steps=2,
           expect_launches=1)


def test_step_result_against_the_cpu_checker(lib):
    lens = [700, 64, 2500]
    hq, hkv, d = 16, 8, 128
    one, out, q_rot = _steps(lib, torch.float16, lens, hq, hkv, d, seed=9, capacity=2624, n_steps=2)
    orc = oracle.best()
    for b in range(len(lens)):
        k, v = one.gather(0, b)
        ref = orc.gqa_decode(q_rot[b : b + 1].float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy())
        assert oracle.rel_err(out[b : b + 1].float().cpu().numpy(), ref) <= 2e-3


@pytest.mark.parametrize("dtype,hq,hkv,d", [(torch.float32, 16, 8, 128), (torch.float16, 6, 2, 80), (torch.float16, 4, 2, 256)])
def test_step_operator_runs_the_two_kernels_where_one_launch_does_not_apply(lib, dtype, hq, hkv, d):
    _steps(lib, dtype, [0, 63, 64, 300, 2100], hq, hkv, d, seed=11, capacity=2176, n_steps=2, expect_launches=2)


def test_one_launch_form_can_be_switched_off(lib):
    try:
        lib.axb200_set_step_fused(0)
        _steps(lib, torch.float16, [5, 64, 1000], 16, 8, 128, seed=12, capacity=1088, n_steps=2, expect_launches=2)
    finally:
        lib.axb200_set_step_fused(1)


def test_full_sequence_sets_the_capacity_flag_and_appends_nothing(lib):
    from axono_b200 import ops

    hq, hkv, d = 16, 8, 128
    lens = [128, 100]  # the first sequence fills its two pages
    one, _ = _two_caches(torch.float16, lens, hkv, d, seed=13, capacity=128)
    rng = np.random.default_rng(14)
    q = dev(rng.standard_normal((2, hq, d)).astype(np.float32), torch.float16)
    kn = dev(rng.standard_normal((2, hkv, d)).astype(np.float32), torch.float16)
    vn = dev(rng.standard_normal((2, hkv, d)).astype(np.float32), torch.float16)
    pages_before = one.k_pages[0].clone()
    out = one.step(0, q, kn, vn, theta=1e6)
    torch.cuda.synchronize()
    assert ops.last_error() & 4  # AXB200_ERR_CAPACITY (reading clears it)
    assert one.seq_lens.tolist() == [128, 101]
    idx = one.block_table[0, :2].long()
    assert _same_bytes(one.k_pages[0][idx], pages_before[idx])  # nothing written for the full sequence
    assert torch.isfinite(out.float()).all()  # the old tokens were attended


def test_multi_wave_batch(lib):
    # more (sequence, head, tile) work than eight waves of CTAs: fixed chunks of 16-64 tiles, CTAs past a
    # sequence's end exit at once - and still count as readers of its length
    rng = np.random.default_rng(17)
    _steps(lib, torch.float16, rng.integers(5000, 6400, 64).tolist(), 16, 8, 128, seed=18, capacity=6464, n_steps=2,
           expect_launches=1)


def test_step_captured_in_a_graph_follows_the_growing_cache(lib):
    from axono_b200 import _capi, ops

    hq, hkv, d = 16, 8, 128
    lens = [60, 4090, 700]
    one, two = _two_caches(torch.float16, lens, hkv, d, seed=15, capacity=4224)
    rng = np.random.default_rng(16)
    q = dev(rng.standard_normal((3, hq, d)).astype(np.float32), torch.float16)
    kn = dev(rng.standard_normal((3, hkv, d)).astype(np.float32), torch.float16)
    vn = dev(rng.standard_normal((3, hkv, d)).astype(np.float32), torch.float16)
    out = torch.empty_like(q)
    # the scratch of the captured call (sized for the capacity) exists before the capture
    ops.workspace(q.device, lib.axb200_decode_step_workspace_bytes(3, hq, hkv, d, one.max_seq_len, _capi.FLOAT16))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        one.step(0, q, kn, vn, out=out, theta=1e6)
    for _ in range(8):  # the sequence of 60 crosses a tile and a page boundary
        g.replay()
        q2 = q.clone()
        two.append_rope(0, q2, kn, vn, theta=1e6)
        # planned for the capacity, as the captured call is: the same chunks, hence the same bits
        want = ops.gqa_decode_attention_paged(q2, two.k_pages[0], two.v_pages[0], two.block_table, two.seq_lens,
                                              two.max_seq_len)
        torch.cuda.synchronize()
        assert torch.equal(one.seq_lens, two.seq_lens)
        assert _same_bytes(out, want)
    assert _same_bytes(one.k_pages[0], two.k_pages[0])


@pytest.mark.parametrize("dtype,hq,hkv,d,launches", [(torch.float16, 16, 8, 128, 1), (torch.float16, 8, 2, 64, 1),
                                                     (torch.float16, 6, 2, 80, 2), (torch.float32, 16, 8, 128, 2)])
@pytest.mark.parametrize("norms,mrope", [(True, True), (False, False)])
def test_step_from_the_qkv_projection_output(lib, dtype, hq, hkv, d, launches, norms, mrope):
    """`axb200_qkv_decode_step_paged` (per-head norms + rope + append + attention from one QKV row) against
    qkv_norm_rope_append followed by the attention call: bit for bit, as the first layer of a step (slot =
    length, the length advances) and as a later one (slot = length - 1, it does not), with strided rows."""
    from axono_b200 import _capi, ops

    lens = [0, 63, 64, 127, 300, 2100]
    one, two = _two_caches(dtype, lens, hkv, d, seed=31, capacity=2176)
    B = len(lens)
    code = _capi.FLOAT16 if dtype == torch.float16 else _capi.FLOAT32
    assert lib.axb200_decode_step_launches(B, hq, hkv, d, one.max_seq_len, code) == launches
    rng = np.random.default_rng(32)
    width = (hq + 2 * hkv) * d
    wq = dev((1 + 0.1 * rng.standard_normal(d)).astype(np.float32), dtype) if norms else None
    wk = dev((1 + 0.1 * rng.standard_normal(d)).astype(np.float32), dtype) if norms else None
    kw = {"theta": 1e6}
    if mrope:
        kw = {"inv_freq": dev((1e6 ** (-np.arange(d // 2, dtype=np.float32) * 2 / d)).astype(np.float32)),
              "mrope_section": (d // 2 - 2 * (d // 6), d // 6, d // 6)}
    for step in range(2):
        for advance, slot_delta in ((True, 0), (False, -1)):  # first layer, then a later layer, of the same step
            wide = dev(rng.standard_normal((B, width + 64)).astype(np.float32), dtype)
            qkv = wide[:, :width]  # rows 64 elements apart from dense
            bound = min(one.max_seq_len, max(lens) + step + 1)
            got = ops.qkv_decode_step_paged(qkv, hq, wq, wk, 1e-6, one.k_pages[0], one.v_pages[0], one.block_table,
                                            one.seq_lens, bound, advance=advance, slot_delta=slot_delta, **kw)
            q2 = ops.qkv_norm_rope_append(qkv, hq, wq, wk, 1e-6, two.k_pages[0], two.v_pages[0], two.block_table,
                                          two.seq_lens, advance=advance, slot_delta=slot_delta, **kw)
            want = ops.gqa_decode_attention_paged(q2, two.k_pages[0], two.v_pages[0], two.block_table, two.seq_lens, bound)
            torch.cuda.synchronize()
            assert ops.last_error() == 0
            assert torch.equal(one.seq_lens, two.seq_lens)
            assert _same_bytes(one.k_pages[0], two.k_pages[0]) and _same_bytes(one.v_pages[0], two.v_pages[0])
            assert _same_bytes(got, want), f"step {step}, advance {advance}"
    assert one.seq_lens.tolist() == [n + 2 for n in lens]
