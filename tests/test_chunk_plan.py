"""The decode calls' chunk plan, evaluated on the host (no GPU): the library exports the functions its
kernels run on the device-resident lengths (axb200_gqa_chunk_plan), so the index arithmetic - how many
chunks each sequence gets, how long they are, that they fit one wave of CTAs - is checked here."""
import ctypes as C

import numpy as np
import pytest

from axono_b200 import _capi

@pytest.fixture(autouse=True)
def device_plan():
    """These tests are about the plan made from the device-resident lengths, an option that is off by
    default (the host plan measured faster); the last test covers the default."""
    _capi.lib().axb200_set_device_plan(1)
    yield
    _capi.lib().axb200_set_device_plan(0)
    _capi.lib().axb200_set_chunk_tiles(0)


SLOTS = 2 * 148  # CTAs resident at once on the part the plan is made for (the library's default without a GPU)


def plan(lens, hq=16, hkv=8, d=128, max_len=None):
    lens = np.ascontiguousarray(lens, dtype=np.int32)
    ct = np.zeros(len(lens), np.int32)
    n = np.zeros(len(lens), np.int32)
    mc, grid = C.c_int32(0), C.c_int32(0)
    st = _capi.lib().axb200_gqa_chunk_plan(lens.ctypes.data, len(lens), hq, hkv, d, int(max_len or max(1, lens.max())),
                                           ct.ctypes.data, n.ctypes.data, C.byref(mc), C.byref(grid))
    assert st == 0
    return ct, n, mc.value, grid.value


def test_one_wave_plan_balances_bytes_per_cta():
    rng = np.random.default_rng(3000)
    lens = rng.integers(16384, 32769, 8)
    ct, n, max_chunks, grid = plan(lens, max_len=32768)
    budget = SLOTS // 8
    assert grid == budget * 8 and n.sum() <= budget and n.max() <= max_chunks
    assert np.all(ct % 64 == 0) and np.all(ct * n >= lens) and np.all(ct * (n - 1) < lens)
    # every CTA of the wave streams about the same run: the longest chunk is within one tile of the
    # smallest chunk length that fits the wave at all
    tiles = -(-lens // 64)
    best = next(c for c in range(4, tiles.max() + 1) if np.maximum(1, -(-tiles // c)).sum() <= budget)
    assert ct.max() <= best * 64 and ct.max() >= best * 64 - 64 * 2
    # the old one-length-for-all rule gave ceil(512 / 4) = 128 tiles to every sequence
    assert ct.max() < 128 * 64


def test_one_wave_plan_edge_lengths():
    ct, n, max_chunks, _ = plan([0, 1, 63, 64, 65, 300, 32768], max_len=32768)
    assert n[0] == 1  # an empty sequence keeps one CTA: it writes the zero rows
    assert list(n[1:5]) == [1, 1, 1, 1]
    assert n.sum() <= SLOTS // 8 and n.max() <= max_chunks
    assert np.all(ct >= 64) and ct[6] * n[6] >= 32768
    # a chunk is never shorter than four tiles unless the sequence is
    assert all(c >= 256 or k == 1 for c, k in zip(ct, n))


def test_lengths_above_the_bound_are_still_covered_in_one_wave():
    # the device plans from the real lengths: a bound that was too small costs nothing here
    ct, n, max_chunks, _ = plan([20000, 100], max_len=4096)
    assert ct[0] * n[0] >= 20000 and n[0] <= max_chunks


def test_many_sequences_single_kv_head():
    lens = np.full(32, 16385)
    ct, n, max_chunks, grid = plan(lens, hq=2, hkv=1, max_len=16448)
    assert grid == SLOTS and n.sum() <= SLOTS and np.all(n == n[0]) and n[0] == SLOTS // 32


def test_large_problem_keeps_one_host_planned_length():
    rng = np.random.default_rng(1)
    lens = rng.integers(16384, 32769, 64)
    ct, n, max_chunks, grid = plan(lens, max_len=32768)
    assert np.all(ct == 4096) and np.all(n == -(-lens // 4096)) and max_chunks == 8 and grid == 8 * 8 * 64
    # a length beyond what the grid covers is cut at the cover (the kernel also raises AXB200_ERR_CAPACITY)
    ct2, n2, mc2, _ = plan([40000] + [30000] * 63, max_len=32768)
    assert n2[0] == mc2


@pytest.mark.parametrize("seed", range(5))
def test_plan_invariants_random(seed):
    rng = np.random.default_rng(seed)
    batch = int(rng.integers(1, 30))
    hkv = int(rng.choice([1, 2, 4, 8]))
    lens = rng.integers(0, 40000, batch)
    ct, n, max_chunks, grid = plan(lens, hq=hkv * 2, hkv=hkv, max_len=40000)
    assert np.all(n >= 1) and np.all(n <= max_chunks) and np.all(ct % 64 == 0)
    assert np.all(ct.astype(np.int64) * n >= np.minimum(lens, ct.astype(np.int64) * max_chunks))
    if grid == (SLOTS // hkv) * hkv:  # planned on the device lengths
        assert n.sum() <= SLOTS // hkv


def test_default_host_plan_and_the_override():
    lib = _capi.lib()
    lib.axb200_set_device_plan(0)
    lens = np.asarray([16384, 32768, 20000, 100] + [24000] * 4)
    ct, n, max_chunks, grid = plan(lens, max_len=32768)
    # one wave: 296 slots / 64 (sequence, head) items = 4 chunks for a sequence at the bound
    assert np.all(ct == 8192) and list(n[:4]) == [2, 4, 3, 1] and max_chunks == 4 and grid == 4 * 8 * 8
    assert lib.axb200_set_chunk_tiles(32) == 0
    ct, n, max_chunks, _ = plan(lens, max_len=32768)
    assert np.all(ct == 2048) and max_chunks == 16 and n[1] == 16
    assert lib.axb200_set_chunk_tiles(1) == 0  # doubled until a sequence has at most 256 chunks
    ct, _, max_chunks, _ = plan(lens, max_len=32768)
    assert np.all(ct == 128) and max_chunks == 256
    assert lib.axb200_set_chunk_tiles(-1) == 1
    lib.axb200_set_chunk_tiles(0)


def test_how_many_launches_a_decode_step_takes():
    """`axb200_decode_step_paged` is one launch where the attention kernel can append the token itself
    (fp16, head_dim 64 or 128, at most 16 query heads per KV head, host-planned chunks), two otherwise."""
    lib = _capi.lib()
    lib.axb200_set_device_plan(0)
    launches = lib.axb200_decode_step_launches
    assert launches(64, 16, 8, 128, 32768, _capi.FLOAT16) == 1
    assert launches(8, 8, 2, 64, 8192, _capi.FLOAT16) == 1
    assert launches(1, 32, 2, 128, 100, _capi.FLOAT16) == 1
    assert launches(64, 16, 8, 128, 32768, _capi.FLOAT32) == 2  # the fp32 kernels do not append
    assert launches(8, 6, 2, 80, 8192, _capi.FLOAT16) == 2      # rides in a wider tile: not the step form
    assert launches(8, 32, 1, 128, 8192, _capi.FLOAT16) == 2    # 32 query heads per KV head: generic kernel
    assert launches(8, 16, 8, 128, 0, _capi.FLOAT16) == 0 and launches(8, 16, 5, 128, 64, _capi.FLOAT16) == 0
    lib.axb200_set_device_plan(1)  # a launch planned on the device lengths reads them in every CTA's prologue
    assert launches(8, 16, 8, 128, 8192, _capi.FLOAT16) == 2
    lib.axb200_set_device_plan(0)
    try:
        lib.axb200_set_step_fused(0)
        assert launches(64, 16, 8, 128, 32768, _capi.FLOAT16) == 2
    finally:
        lib.axb200_set_step_fused(1)
    assert lib.axb200_decode_step_workspace_bytes(8, 16, 8, 128, 8192, _capi.FLOAT16) >= \
        lib.axb200_gqa_workspace_bytes(8, 16, 8, 128, 8192, _capi.FLOAT16) + 8 * 16 * 128 * 2


def test_step_entry_points_refuse_bad_arguments_before_touching_the_device():
    """Argument checks of the step operators come before any CUDA call, so they can be exercised without a
    GPU: status codes as the reference's enum (3 UNSUPPORTED_TYPE, 7 INVALID_PTR, 1 INVALID_ARGUMENT)."""
    lib = _capi.lib()
    buf = (C.c_char * 4096)()
    ptr = C.addressof(buf)
    F16 = _capi.FLOAT16
    ok_ws = lib.axb200_decode_step_workspace_bytes(2, 4, 2, 128, 256, F16)
    assert ok_ws > 0 and lib.axb200_decode_step_workspace_bytes(2, 4, 2, 128, 256, 99) == 0

    def step(q=ptr, k=ptr, v=ptr, out=ptr, dtype=F16, batch=2, ws=ptr, ws_bytes=ok_ws, max_len=256):
        return lib.axb200_decode_step_paged(q, k, v, out, ptr, ptr, ptr, ptr, None, None, 1e6, 1, 0, 0, 0, batch, 4, 2, 128,
                                            64, 4, 8, max_len, dtype, ws, ws_bytes, None)

    assert step(dtype=99) == 3
    assert step(q=None) == 7 and step(out=None) == 7 and step(ws=None) == 7
    assert step(batch=0) == 1 and step(max_len=0) == 1
    assert step(ws_bytes=ok_ws - 1) == 1

    def qkv_step(qkv=ptr, ld=(4 + 4) * 128, slot_delta=0, advance=1, world=0, out=ptr, peer=None, hq_total=4, dtype=F16):
        return lib.axb200_qkv_decode_step_paged(qkv, ld, None, None, 1e-6, out, ptr, ptr, ptr, ptr, None, None, 1e6, 1, 0, 0, 0,
                                                2, 4, 2, 128, 64, 4, 8, 256, dtype, slot_delta, advance, ptr, ok_ws, peer, peer,
                                                peer, world, 0, hq_total, None)

    assert qkv_step(dtype=99) == 3
    assert qkv_step(qkv=None) == 7 and qkv_step(out=None) == 7
    assert qkv_step(ld=100) == 1                      # a row must hold hq + 2 hkv heads
    assert qkv_step(slot_delta=-1, advance=1) == 1    # first layer: (0, 1); later layers: (-1, 0)
    assert qkv_step(slot_delta=0, advance=0) == 1
    assert qkv_step(world=2) == 7                     # peers asked for, none given
    assert qkv_step(world=9, peer=ptr) == 1 and qkv_step(world=2, peer=ptr, hq_total=5) == 1
