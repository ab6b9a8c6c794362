"""KV page arena: host-side bookkeeping on CPU (no device memory), and on a GPU the arena-backed cache
against the plain paged cache."""
import numpy as np
import pytest
import torch

from axono_b200.kv_cache import KVArena


def test_bookkeeping_without_device_memory():
    a = KVArena(n_layers=2, num_pages=10, n_kv_heads=8, head_dim=128, max_seqs=4, max_seq_len=64 * 6,
                device_memory=False)
    assert a.stats() == {"pages_total": 10, "pages_free": 10, "seqs_live": 0, "device_bytes": 0}
    s0 = a.alloc_seq(100)  # 2 pages
    s1 = a.alloc_seq(64)  # 1 page
    assert (s0, s1) == (0, 1)
    assert a.seq_pages(s0) == [0, 1] and a.seq_pages(s1) == [2]
    a.reserve(s0, 128)  # still 2 pages
    assert a.seq_pages(s0) == [0, 1]
    a.reserve(s0, 129)  # crosses a page boundary
    assert a.seq_pages(s0) == [0, 1, 3]
    assert a.stats()["pages_free"] == 6
    with pytest.raises(RuntimeError):
        a.reserve(s0, 64 * 7)  # beyond max_blocks
    with pytest.raises(RuntimeError):
        a.reserve(s1, 64 * 6 + 0 + 64 * 3)  # beyond max_blocks as well
    # exhaustion is all-or-nothing
    s2 = a.alloc_seq(64 * 5)
    assert a.stats()["pages_free"] == 1
    with pytest.raises(RuntimeError):
        a.alloc_seq(64 * 2)
    assert a.stats() == {"pages_total": 10, "pages_free": 1, "seqs_live": 3, "device_bytes": 0}
    # freed pages are handed out again, lowest slot first
    a.free_seq(s0)
    assert a.stats()["pages_free"] == 4 and a.stats()["seqs_live"] == 2
    s3 = a.alloc_seq(64 * 3)
    assert s3 == 0 and sorted(a.seq_pages(s3) ) == [0, 1, 3]
    with pytest.raises(RuntimeError):
        a.free_seq(3)  # never allocated
    with pytest.raises(RuntimeError):
        a.seq_pages(3)
    # slots run out
    a.alloc_seq(0)
    with pytest.raises(RuntimeError):
        a.alloc_seq(0)
    a.free_seq(s2)
    a.close()


@pytest.mark.gpu
def test_arena_backed_cache_matches_plain_paged_cache():
    """Sequences come and go; a recycled page still holds the previous owner's bytes (never re-zeroed)
    and the results stay exact because the kernels mask by length."""
    import oracle
    from axono_b200 import ops

    orc = oracle.best()
    rng = np.random.default_rng(71)
    hq, hkv, d = 16, 8, 128
    arena = KVArena(1, num_pages=40, n_kv_heads=hkv, head_dim=d, max_seqs=4, max_seq_len=1024, dtype=torch.float32)
    cache = arena.cache()
    assert arena.stats()["device_bytes"] == 2 * 40 * hkv * 64 * d * 4

    def grow(slot, n_tokens, kstore, vstore):
        """Appends n_tokens one by one (reserving ahead), remembering what went in."""
        for _ in range(n_tokens):
            arena.reserve(slot, len(kstore[slot]) + 1)
            arena.sync()
            kn = rng.standard_normal((1, hkv, d)).astype(np.float32)
            vn = rng.standard_normal((1, hkv, d)).astype(np.float32)
            kstore[slot].append(kn[0].copy())
            vstore[slot].append(vn[0].copy())
            # a one-row step on this sequence's row of the shared table and length vector
            ops.kv_append_rope(None, torch.from_numpy(kn).cuda(), torch.from_numpy(vn).cuda(), cache.k_pages[0],
                               cache.v_pages[0], cache.block_table[slot : slot + 1], cache.seq_lens[slot : slot + 1],
                               rotate=False, advance=True)

    ks = {s: [] for s in range(4)}
    vs = {s: [] for s in range(4)}
    a = arena.alloc_seq(1)
    b = arena.alloc_seq(1)
    arena.sync()
    grow(a, 70, ks, vs)
    grow(b, 130, ks, vs)
    q = rng.standard_normal((4, hq, d)).astype(np.float32)
    cache._host_len_bound = 1024
    out = cache.attend(0, torch.from_numpy(q).cuda()).cpu().numpy()
    for s in (a, b):
        ref = orc.gqa_decode(q[s : s + 1], np.stack(ks[s]), np.stack(vs[s]))
        assert oracle.rel_err(out[s : s + 1], ref) <= 1e-5
    assert np.all(out[2:] == 0)  # unused slots have length 0
    # free a, start a new sequence in the recycled pages
    pages_a = arena.seq_pages(a)
    arena.free_seq(a)
    c = arena.alloc_seq(1)
    arena.sync()
    assert c == a and arena.seq_pages(c)[0] in pages_a
    ks[c], vs[c] = [], []
    grow(c, 5, ks, vs)
    out = cache.attend(0, torch.from_numpy(q).cuda()).cpu().numpy()
    for s in (c, b):
        ref = orc.gqa_decode(q[s : s + 1], np.stack(ks[s]), np.stack(vs[s]))
        assert oracle.rel_err(out[s : s + 1], ref) <= 1e-5
    assert ops.last_error() == 0
    arena.close()
