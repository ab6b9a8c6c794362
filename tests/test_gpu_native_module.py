"""The native `libaxono` module on the GPU, written the way the reference tests its binding
(axono/python/tests/core/{test_gqa,test_fused,test_llm_ops,test_sequence_ops,test_cuda_graph}.py):
numpy in, Tensor through the operators, numpy out, checked against the CPU oracle.  PyTorch appears only in
the tower comparison (and is imported first: one cuBLASLt per process); tolerances: fp32 1e-5, fp16 2e-3
(max|out - ref| / max|ref|)."""
import numpy as np
import pytest
import torch  # noqa: F401 - before the native module's first projection: one process, one cuBLASLt (see axono_ops.cpp)

import oracle
from axono_b200 import native

pytestmark = pytest.mark.gpu
TOL = {np.float32: 1e-5, np.float16: 2e-3}


@pytest.fixture(scope="module")
def lx():
    m = native.load()
    assert m.cuda_available(), "no CUDA device"
    return m


@pytest.fixture(scope="module")
def chk():
    return oracle.best()


def dev(lx, a):
    return lx.Tensor.from_numpy(np.ascontiguousarray(a), "cuda")


def f32(a):
    return np.asarray(a, dtype=np.float32)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("hq,hkv,d,skv", [(16, 8, 128, 777), (32, 8, 128, 4096), (8, 8, 64, 33), (12, 4, 80, 300)])
def test_gqa_decode_attention(lx, chk, dtype, hq, hkv, d, skv):
    rng = np.random.default_rng(hq * 1000 + skv)
    q = rng.standard_normal((1, hq, d), dtype=np.float32).astype(dtype)
    k = rng.standard_normal((skv, hkv, d), dtype=np.float32).astype(dtype)
    v = rng.standard_normal((skv, hkv, d), dtype=np.float32).astype(dtype)
    out = lx.gqa_decode_attention(dev(lx, q), dev(lx, k), dev(lx, v))
    assert out.shape == (1, hq, d) and out.is_cuda and out.dtype == (lx.DataType.FLOAT32 if dtype is np.float32 else lx.DataType.FLOAT16)
    ref = chk.gqa_decode(f32(q), f32(k), f32(v))
    assert oracle.rel_err(f32(out.numpy()), ref) <= TOL[dtype]


def test_gqa_decode_attention_status_codes(lx):
    """Argument checks in the reference's order (src/ops/cuda/gqa.cu:143-154)."""
    rng = np.random.default_rng(0)
    q = dev(lx, rng.standard_normal((1, 8, 64), dtype=np.float32))
    k = dev(lx, rng.standard_normal((16, 2, 64), dtype=np.float32))
    with pytest.raises(RuntimeError, match="status 1"):  # Sq must be 1
        lx.gqa_decode_attention(dev(lx, np.zeros((2, 8, 64), np.float32)), k, k)
    with pytest.raises(RuntimeError, match="status 4"):  # Hq not a multiple of Hkv
        lx.gqa_decode_attention(dev(lx, np.zeros((1, 7, 64), np.float32)), k, k)
    with pytest.raises(RuntimeError, match="status 3"):  # dtype
        lx.gqa_decode_attention(dev(lx, np.zeros((1, 8, 64), np.int32)), k, k)
    with pytest.raises(RuntimeError, match="status 8"):  # device
        lx.gqa_decode_attention(q, k.to("cpu"), k)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_fused_elementwise(lx, chk, dtype):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((5, 2048), dtype=np.float32).astype(dtype)
    r = rng.standard_normal((5, 2048), dtype=np.float32).astype(dtype)
    w = (1 + 0.1 * rng.standard_normal(2048, dtype=np.float32)).astype(dtype)
    y, out = lx.add_rms_norm(dev(lx, x), dev(lx, r), dev(lx, w), 1e-6)
    y_ref, out_ref = chk.add_rms_norm(f32(x), f32(r), f32(w), 1e-6)
    if dtype is np.float32:
        assert np.array_equal(y.numpy(), y_ref)  # one rounded add
    assert oracle.rel_err(f32(y.numpy()), y_ref) <= TOL[dtype]
    assert oracle.rel_err(f32(out.numpy()), out_ref) <= TOL[dtype]
    act = lx.silu_mul(dev(lx, x), dev(lx, r))
    assert oracle.rel_err(f32(act.numpy()), chk.silu_mul(f32(x), f32(r))) <= TOL[dtype]
    n = lx.rms_norm(dev(lx, x), dev(lx, w), 1e-5)
    assert oracle.rel_err(f32(n.numpy()), chk.rms_norm(f32(x), f32(w), 1e-5)) <= TOL[dtype]


def test_rope_family(lx, chk):
    rng = np.random.default_rng(2)
    s, h, d = 9, 4, 128
    x = rng.standard_normal((s, h, d), dtype=np.float32)
    pos = rng.integers(0, 40000, size=s).astype(np.int64)
    out = lx.rope(dev(lx, x), dev(lx, pos), 1e6)
    assert oracle.rel_err(out.numpy(), chk.rope(x, pos, 1e6)) <= 1e-5
    pos3 = rng.integers(0, 5000, size=(3, s)).astype(np.int64)
    inv = oracle.port().rope_inv_freq(1e6, d)
    cos, sin = lx.mrope_cos_sin(dev(lx, pos3), dev(lx, inv), 20, 20)
    cos_ref, sin_ref = chk.mrope_cos_sin(pos3, inv, 20, 20)
    assert cos.shape == (s, d) and oracle.rel_err(cos.numpy(), cos_ref) <= 1e-5
    assert oracle.rel_err(sin.numpy(), sin_ref) <= 1e-5
    rot = lx.rope_with_cos_sin(dev(lx, x), cos, sin)
    assert oracle.rel_err(rot.numpy(), chk.rope_with_cos_sin(x, cos_ref, sin_ref)) <= 1e-5
    thd = lx.rope_thd(dev(lx, x), dev(lx, pos3), dev(lx, inv), 24, 20, 20)
    assert oracle.rel_err(thd.numpy(), chk.rope_thd(x, pos3, inv, (24, 20, 20))) <= 1e-5


def test_sequence_ops_bit_exact(lx, chk):
    rng = np.random.default_rng(3)
    a = rng.standard_normal((7, 4, 64), dtype=np.float32)
    b = rng.standard_normal((1, 4, 64), dtype=np.float32)
    cat = lx.concat(dev(lx, a), dev(lx, b), 0)
    assert cat.shape == (8, 4, 64) and np.array_equal(cat.numpy(), np.concatenate([a, b], 0))
    cat2 = lx.concat(dev(lx, a), dev(lx, a), -1)
    assert np.array_equal(cat2.numpy(), np.concatenate([a, a], -1))
    table = rng.standard_normal((1000, 96), dtype=np.float32)
    ids = rng.integers(0, 1000, size=(3, 5)).astype(np.int64)
    emb = lx.embedding(dev(lx, ids), dev(lx, table))
    assert emb.shape == (3, 5, 96) and np.array_equal(emb.numpy(), table[ids])
    logits = rng.standard_normal((6, 151936), dtype=np.float32)
    logits[2, 77] = logits[2, 150000] = 99.0  # a tie: the lowest index wins
    am = lx.argmax(dev(lx, logits))
    assert am.dtype == lx.DataType.INT64 and np.array_equal(am.numpy(), chk.argmax_last_dim(logits))
    assert am.numpy()[2] == 77


def test_cast_and_device_moves(lx):
    a = np.random.default_rng(4).standard_normal((33, 65), dtype=np.float32)
    t = dev(lx, a)
    assert t.device == "cuda" and t.is_cuda and np.array_equal(t.to("cpu").numpy(), a)
    h = t.cast_to(lx.DataType.FLOAT16)
    assert h.dtype == lx.DataType.FLOAT16 and np.array_equal(h.numpy(), a.astype(np.float16))
    assert np.array_equal(h.cast_to(lx.DataType.FLOAT32).numpy(), a.astype(np.float16).astype(np.float32))
    fresh = lx.Tensor(lx.DataType.FLOAT32, [1000], "cuda")
    assert not fresh.numpy().any()  # device storage starts at zero, also when it comes from the pool


def test_caching_allocator_reuses_and_respects_budget(lx):
    lx.clear_cache()
    assert lx.cached_bytes() == 0
    t = lx.Tensor(lx.DataType.INT8, [1 << 20], "cuda")
    ptr = t.data_ptr
    t.copy_from_numpy(np.full(1 << 20, 7, np.int8))
    del t
    assert lx.cached_bytes() == 1 << 20
    u = lx.Tensor(lx.DataType.INT8, [1 << 20], "cuda")  # exact-size hit, zeroed again
    assert u.data_ptr == ptr and lx.cached_bytes() == 0 and not u.numpy().any()
    del u
    old = lx.cache_budget()
    try:
        lx.set_cache_budget(1 << 19)  # below what is cached: evicted
        assert lx.cached_bytes() == 0
        v = lx.Tensor(lx.DataType.INT8, [1 << 20], "cuda")
        del v
        assert lx.cached_bytes() == 0  # larger than the budget: freed, not cached
    finally:
        lx.set_cache_budget(old)


def _decode_chain(lx, x, r, w, q, k, v):
    y, xn = lx.add_rms_norm(x, r, w, 1e-6)
    attn = lx.gqa_decode_attention(q, k, v)
    return y, xn, attn, lx.silu_mul(xn, y)


def test_cuda_graph_capture_replay(lx, chk):
    """capture(fn) warms up, records allocations, captures; replays rewrite the same output buffers
    and follow in-place changes of the inputs (axono/python/tests/core/test_cuda_graph.py:26-80)."""
    rng = np.random.default_rng(5)
    x_np, r_np = rng.standard_normal((4, 1024), dtype=np.float32), rng.standard_normal((4, 1024), dtype=np.float32)
    w_np = np.ones(1024, np.float32)
    q_np = rng.standard_normal((1, 16, 128), dtype=np.float32)
    k_np, v_np = (rng.standard_normal((2000, 8, 128), dtype=np.float32) for _ in range(2))
    x, r, w, q, k, v = (dev(lx, a) for a in (x_np, r_np, w_np, q_np, k_np, v_np))
    g = native.CUDAGraph()
    g.capture(lambda: _decode_chain(lx, x, r, w, q, k, v))
    assert g.is_captured and g.num_nodes >= 3  # norm, attention (split + merge in one kernel), silu
    y, xn, attn, act = g.outputs
    for _ in range(3):
        g.replay()
        g.sync()
        assert oracle.rel_err(attn.numpy(), chk.gqa_decode(q_np, k_np, v_np)) <= 1e-5
        assert np.array_equal(y.numpy(), x_np + r_np)
    q2 = rng.standard_normal((1, 16, 128), dtype=np.float32)
    q.copy_from_numpy(q2)  # same address, new contents
    g.replay()
    g.sync()
    assert oracle.rel_err(attn.numpy(), chk.gqa_decode(q2, k_np, v_np)) <= 1e-5
    eager = _decode_chain(lx, x, r, w, q, k, v)
    assert np.array_equal(eager[3].numpy(), act.numpy())
    g.reset()
    assert not g.is_captured


def test_cuda_graph_block_form_and_errors(lx):
    rng = np.random.default_rng(6)
    a_np, b_np = rng.standard_normal((8, 512), dtype=np.float32), rng.standard_normal((8, 512), dtype=np.float32)
    a, b = dev(lx, a_np), dev(lx, b_np)
    with native.cuda_graph() as g:
        tmp = lx.silu_mul(a, b)  # a temporary allocated inside the graph
        g.output = lx.silu_mul(tmp, b)
        del tmp
    assert g.is_captured and g.num_nodes >= 2
    ref = None
    for _ in range(4):
        g.replay()
        g.sync()
        cur = g.output.numpy()
        ref = cur if ref is None else ref
        assert np.array_equal(cur, ref)
    s1 = oracle.port().silu_mul(a_np, b_np)
    assert oracle.rel_err(ref, oracle.port().silu_mul(s1, b_np)) <= 1e-5
    g.reset()
    with pytest.raises(RuntimeError):  # replay before capture
        native.CUDAGraph().replay()
    with pytest.raises(RuntimeError):  # nothing launched: an empty graph is an error
        native.CUDAGraph().capture(lambda: None)
    # the runtime is usable after the failed capture
    assert np.array_equal(lx.silu_mul(a, b).numpy(), lx.silu_mul(a, b).numpy())


def test_kv_arena_decode_steps(lx, chk):
    """Append-with-rope into arena pages, then paged attention, for three sequences over five steps;
    the oracle runs rope -> concat -> gqa_decode per sequence on contiguous arrays."""
    hq, hkv, d, page = 8, 2, 128, 64
    lens = [130, 5, 64]
    rng = np.random.default_rng(7)
    arena = lx.KVArena(1, 32, hkv, page, d, lx.DataType.FLOAT32, 3, 8)
    hist_k = [np.zeros((0, hkv, d), np.float32) for _ in lens]
    hist_v = [np.zeros((0, hkv, d), np.float32) for _ in lens]
    for n in lens:
        arena.alloc_seq(n + 3)
    arena.sync()
    assert list(arena.seq_lens()) == [0, 0, 0]
    st = arena.stats()
    assert st["seqs_live"] == 3 and st["pages_total"] == 32 and st["pages_free"] == 32 - sum((n + 3 + page - 1) // page for n in lens)
    for step in range(5):
        k_new = rng.standard_normal((3, hkv, d), dtype=np.float32)
        v_new = rng.standard_normal((3, hkv, d), dtype=np.float32)
        q = rng.standard_normal((3, hq, d), dtype=np.float32)
        qd = dev(lx, q)
        lx.kv_append_rope(arena, 0, qd, dev(lx, k_new), dev(lx, v_new), theta=1e6)
        out = lx.gqa_decode_attention_paged(qd, arena, 0, 64)
        pos = np.full(1, step, np.int64)
        for b in range(3):
            hist_k[b] = np.concatenate([hist_k[b], chk.rope(k_new[b:b + 1], pos, 1e6)], 0)
            hist_v[b] = np.concatenate([hist_v[b], v_new[b:b + 1]], 0)
            q_rot = chk.rope(q[b:b + 1], pos, 1e6)
            ref = chk.gqa_decode(q_rot, hist_k[b], hist_v[b])
            assert oracle.rel_err(out.numpy()[b:b + 1], ref) <= 1e-5
    assert list(arena.seq_lens()) == [5, 5, 5]
    arena.free_seq(1)
    assert arena.stats()["seqs_live"] == 2 and list(arena.seq_lens()) == [5, 0, 5]


def test_compile_caches_one_graph_per_signature(lx, chk):
    """compile(): first call warms up and captures, later calls copy inputs into the first call's
    tensors and replay; a new shape captures a second graph (axono/python/axono/core/compile.py:69-174)."""
    rng = np.random.default_rng(8)
    w = dev(lx, np.ones(512, np.float32))

    class Block:
        eps = 1e-6

        def __call__(self, x, r):
            y, xn = lx.add_rms_norm(x, r, w, self.eps)
            return lx.silu_mul(xn, y)

    m = native.compile(Block())
    assert m.eps == 1e-6  # attribute access passes through to the model
    x1, r1 = rng.standard_normal((4, 512), dtype=np.float32), rng.standard_normal((4, 512), dtype=np.float32)
    out = m(dev(lx, x1), dev(lx, r1))
    y_ref, xn_ref = chk.add_rms_norm(x1, r1, np.ones(512, np.float32), 1e-6)
    assert oracle.rel_err(out.to_numpy(), chk.silu_mul(xn_ref, y_ref)) <= 1e-5
    x2, r2 = rng.standard_normal((4, 512), dtype=np.float32), rng.standard_normal((4, 512), dtype=np.float32)
    out2 = m(dev(lx, x2), dev(lx, r2))  # same signature: replay on refreshed static inputs
    y_ref, xn_ref = chk.add_rms_norm(x2, r2, np.ones(512, np.float32), 1e-6)
    assert m.num_graphs == 1 and oracle.rel_err(out2.to_numpy(), chk.silu_mul(xn_ref, y_ref)) <= 1e-5
    assert out2.data_ptr == out.data_ptr  # outputs are static buffers
    x3 = rng.standard_normal((2, 512), dtype=np.float32)
    m(dev(lx, x3), dev(lx, x3))
    assert m.num_graphs == 2
    with pytest.raises(ValueError):
        native.compile(Block(), mode="max")


def test_linear_nobias_and_glue(lx):
    """linear_nobias is a cuBLASLt call (x . w^T, row-major); silu_mul_rows works on the halves of a
    fused gate|up output."""
    rng = np.random.default_rng(10)
    for dtype, tol in ((np.float32, 1e-4), (np.float16, 4e-3)):  # fp32 runs as TF32-free SGEMM; fp16 accumulates in fp32
        x = rng.standard_normal((5, 192), dtype=np.float32).astype(dtype)
        w = (0.1 * rng.standard_normal((320, 192), dtype=np.float32)).astype(dtype)
        y = lx.linear_nobias(dev(lx, x), dev(lx, w))
        assert y.shape == (5, 320)
        ref = f32(x) @ f32(w).T
        assert oracle.rel_err(f32(y.numpy()), ref) <= tol
    gu = rng.standard_normal((4, 256), dtype=np.float32)
    act = lx.silu_mul_rows(dev(lx, gu), 128)
    assert oracle.rel_err(act.numpy(), oracle.port().silu_mul(gu[:, :128].copy(), gu[:, 128:].copy())) <= 1e-5
    with pytest.raises(RuntimeError):
        lx.linear_nobias(dev(lx, np.zeros((2, 8), np.float32)), dev(lx, np.zeros((4, 9), np.float32)))


def test_native_tower_matches_torch_tower():
    """The tower's decode step on the native runtime against the same step on the torch-tensor mirror,
    same weights, three steps eagerly and three more as one captured graph."""
    import torch

    from axono_b200.decode import TextTower
    from axono_b200.native_tower import NativeTextTower
    from axono_b200.tower_config import TextTowerConfig

    cfg = TextTowerConfig(hidden=256, intermediate=512, n_q_heads=4, n_kv_heads=2, head_dim=128, vocab=1000, n_layers=3)
    batch, lens = 3, [70, 5, 129]
    nt = NativeTextTower(cfg, batch, 256, seed=3)
    tt = TextTower(cfg, batch, 256, page_tokens=64)
    hw = nt.host_weights
    tt.embed.copy_(torch.from_numpy(hw["embed"]))
    tt.final_ln.copy_(torch.from_numpy(hw["final_ln"]))
    for lw_t, lw_n in zip(tt.layers, hw["layers"]):
        for k in lw_t:
            lw_t[k].copy_(torch.from_numpy(lw_n[k]))
    ids = [1, 2, 3]
    nt.set_state(ids, lens)
    tt.set_state(ids, lens)
    for _ in range(3):
        n_ids, t_ids = nt.decode_step().numpy(), tt.decode_step().cpu().numpy()
        ref = tt.last_logits.float().cpu().numpy()
        assert oracle.rel_err(nt.last_logits.numpy().astype(np.float32), ref) <= 2e-2
        assert np.array_equal(n_ids, t_ids)
    assert list(nt.arena.seq_lens()) == [n + 3 for n in lens]
    g = native.CUDAGraph().capture(nt.decode_step)
    # capture's warm-up run was a real step: put the state back one token
    nt.set_state(t_ids, [n + 3 for n in lens])
    for _ in range(3):
        g.replay()
        t_ids = tt.decode_step().cpu().numpy()
        assert oracle.rel_err(nt.last_logits.numpy().astype(np.float32), tt.last_logits.float().cpu().numpy()) <= 2e-2
        assert np.array_equal(g.output.numpy(), t_ids)
    assert g.replay_timed(5) > 0


def test_runtime_returns_its_memory(lx):
    """Allocate / free cycles and capture / replay / reset cycles leave the device where it was: blocks go
    back to the pool (bounded by the budget), the capture pool is released by reset, graphs are destroyed."""
    rng = np.random.default_rng(11)
    a, b = dev(lx, rng.standard_normal((64, 1024), dtype=np.float32)), dev(lx, rng.standard_normal((64, 1024), dtype=np.float32))
    w = dev(lx, np.ones(1024, np.float32))

    def body():
        y, xn = lx.add_rms_norm(a, b, w, 1e-6)
        return lx.silu_mul(xn, y)

    def cycle():
        for n in (1 << 20, 3 << 20, 1 << 20, 5 << 20):
            t = lx.Tensor(lx.DataType.INT8, [n], "cuda")
            del t
        g = native.CUDAGraph().capture(body)
        for _ in range(3):
            g.replay()
        ref = g.output.numpy().copy()
        g.reset()
        return ref

    first = cycle()  # warms the pool and every lazily created handle
    lx.clear_cache()
    free0, _ = lx.mem_info()
    for _ in range(20):
        assert np.array_equal(cycle(), first)
    lx.clear_cache()
    free1, _ = lx.mem_info()
    assert abs(free0 - free1) <= (8 << 20), (free0, free1)  # nothing accumulates over 20 cycles
    assert lx.cached_bytes() == 0


def test_several_graphs_alive_at_once(lx):
    """A later capture must not touch the buffers of an earlier graph: each graph owns the pool blocks
    its captured run took (compile() keeps one graph per call signature alive)."""
    rng = np.random.default_rng(12)
    w = dev(lx, np.ones(256, np.float32))

    def block(x, r):
        y, xn = lx.add_rms_norm(x, r, w, 1e-6)
        return lx.silu_mul(xn, y)

    m = native.compile(block)
    xs = {n: (rng.standard_normal((n, 256), dtype=np.float32), rng.standard_normal((n, 256), dtype=np.float32)) for n in (4, 9, 17)}
    ref = {}
    for n, (x, r) in xs.items():  # three signatures -> three live graphs
        ref[n] = m(dev(lx, x), dev(lx, r)).numpy().copy()
    assert m.num_graphs == 3
    for _ in range(3):
        for n, (x, r) in xs.items():  # replay them in turn, with scratch allocations in between
            junk = lx.Tensor(lx.DataType.FLOAT32, [n * 256], "cuda")
            junk.copy_from_numpy(np.full(n * 256, 7.0, np.float32))
            out = m(dev(lx, x), dev(lx, r)).numpy()
            assert np.array_equal(out, ref[n])
            del junk
    a4, b4, a9, b9 = (dev(lx, t) for t in (*xs[4], *xs[9]))  # inputs are made outside the captured bodies
    g1 = native.CUDAGraph().capture(lambda: block(a4, b4))
    g1.replay()
    first = g1.output.numpy().copy()
    assert np.array_equal(first, ref[4])
    g2 = native.CUDAGraph().capture(lambda: block(a9, b9))
    g2.replay()
    g1.replay()
    assert np.array_equal(g1.output.numpy(), first)
    g2.reset()  # releasing one graph leaves the other intact
    g1.replay()
    assert np.array_equal(g1.output.numpy(), first)
    g1.reset()


def test_framework_free_services(lx, chk):
    """What a program without any framework takes from the module besides the operators: device choice,
    the seeded device fill, page-locked arrays, event timing, views of foreign device memory, and the
    arena's read-back - exercised the way bench.py's default arm uses them."""
    assert lx.current_device() == 0 and isinstance(lx.device_pci_bus_id(0), str) and lx.device_pci_bus_id(0)
    assert lx.current_stream() == 0  # legacy default stream outside capture
    f16 = lx.DataType.FLOAT16
    a = lx.randn([1 << 16], f16, "cuda", 7, 0.0, 0.5).numpy().astype(np.float32)
    b = lx.randn([1 << 16], f16, "cuda", 7, 0.0, 0.5).numpy().astype(np.float32)
    c = lx.randn([1 << 16], f16, "cuda", 8, 0.0, 0.5).numpy().astype(np.float32)
    assert np.array_equal(a, b) and not np.array_equal(a, c)  # (seed, index) decides the value
    assert abs(a.mean()) < 0.01 and abs(a.std() - 0.5) < 0.01 and np.isfinite(a).all()
    short = lx.randn([1000], f16, "cuda", 7, 0.0, 0.5).numpy().astype(np.float32)
    assert np.array_equal(short, a[:1000])  # the launch shape does not matter
    p = lx.pinned_empty([4, 8], lx.DataType.FLOAT32)
    assert p.shape == (4, 8) and p.dtype == np.float32
    p[...] = 3.0
    t = lx.Tensor.from_numpy(p, "cuda")
    view = lx.Tensor.from_device_ptr(t.data_ptr, lx.DataType.FLOAT32, [32], "cuda")
    assert np.array_equal(view.numpy(), np.full(32, 3.0, np.float32))
    timer = lx.EventTimer()
    timer.start()
    lx.randn([1 << 24], f16, "cuda", 1)
    timer.stop()
    assert 0.0 < timer.elapsed_ms() < 100.0

    # an arena with scattered pages, filled on the device, read back token-major
    hkv, d, page, cap, B = 2, 128, 64, 1000, 3
    blocks = (cap + page - 1) // page
    arena = lx.KVArena(1, B * blocks, hkv, page, d, f16, B, blocks)
    arena.shuffle_free(5)
    for _ in range(B):
        arena.alloc_seq(cap)
    arena.sync()
    arena.fill_normal(3, 0.5)
    lens = np.asarray([1000, 70, 0], np.int32)
    arena.set_seq_lens(lens)
    rng = np.random.default_rng(1)
    q = rng.standard_normal((B, 4, d)).astype(np.float16)
    out = lx.Tensor(f16, [B, 4, d], "cuda")
    got = lx.gqa_decode_attention_paged(dev(lx, q), arena, 0, cap, out=out)
    assert got.data_ptr == out.data_ptr  # written in place
    res = out.numpy().astype(np.float32)
    for b in (0, 1):
        k, v = arena.gather(0, b, int(lens[b]))
        assert k.shape == (lens[b], hkv, d)
        assert oracle.rel_err(res[b : b + 1], chk.gqa_decode(f32(q[b : b + 1]), f32(k), f32(v))) <= 2e-3
    assert np.all(res[2] == 0)

    # the host-buffer step on page-locked arrays: same bits as append + attention on device tensors
    twin = lx.KVArena(1, B * blocks, hkv, page, d, f16, B, blocks)
    twin.shuffle_free(5)
    for _ in range(B):
        twin.alloc_seq(cap)
    twin.sync()
    twin.fill_normal(3, 0.5)
    twin.set_seq_lens(lens)
    qh, oh = lx.pinned_empty([B, 4, d], f16), lx.pinned_empty([B, 4, d], f16)
    kh, vh = lx.pinned_empty([B, hkv, d], f16), lx.pinned_empty([B, hkv, d], f16)
    qh[...] = q
    kh[...] = rng.standard_normal((B, hkv, d)).astype(np.float16)
    vh[...] = rng.standard_normal((B, hkv, d)).astype(np.float16)
    stage = [lx.Tensor(f16, [B, 4, d], "cuda"), lx.Tensor(f16, [B, hkv, d], "cuda"), lx.Tensor(f16, [B, hkv, d], "cuda"),
             lx.Tensor(f16, [B, 4, d], "cuda")]
    ws = lx.Tensor(lx.DataType.INT8, [max(256, lx.gqa_workspace_bytes(B, 4, hkv, d, cap, f16))], "cuda")
    lx.decode_step_host(arena, 0, qh, kh, vh, oh, stage[0], stage[1], stage[2], stage[3], ws, cap, 1e6)
    qd = dev(lx, qh.copy())
    lx.kv_append_rope(twin, 0, qd, dev(lx, kh.copy()), dev(lx, vh.copy()), theta=1e6)
    want = lx.gqa_decode_attention_paged(qd, twin, 0, cap).numpy()
    assert np.array_equal(oh, want)
    assert np.array_equal(arena.seq_lens(), lens + 1)
    assert lx.device_error_bits() == 0


def test_decode_step_operator(lx, chk):
    """`decode_step_paged` on the native runtime: one launch, the bits of kv_append_rope + attention, q left
    as it was, lengths advanced - over several steps on scattered pages."""
    f16 = lx.DataType.FLOAT16
    hq, hkv, d, page, cap, B = 16, 8, 128, 64, 2200, 3
    blocks = (cap + page - 1) // page
    arenas = []
    for _ in range(2):
        a = lx.KVArena(1, B * blocks, hkv, page, d, f16, B, blocks)
        a.shuffle_free(9)
        for _ in range(B):
            a.alloc_seq(cap)
        a.sync()
        a.fill_normal(4, 0.5)
        a.set_seq_lens(np.asarray([2100, 63, 0], np.int32))
        arenas.append(a)
    one, two = arenas
    assert lx.decode_step_launches(B, hq, hkv, d, cap, f16) == 1
    rng = np.random.default_rng(2)
    for step in range(3):
        q = rng.standard_normal((B, hq, d)).astype(np.float16)
        kn = (0.5 * rng.standard_normal((B, hkv, d))).astype(np.float16)
        vn = (0.5 * rng.standard_normal((B, hkv, d))).astype(np.float16)
        qd = dev(lx, q)
        got = lx.decode_step_paged(qd, dev(lx, kn), dev(lx, vn), one, 0, cap, theta=1e6)
        assert np.array_equal(qd.numpy(), q)  # only read
        q2 = dev(lx, q)
        lx.kv_append_rope(two, 0, q2, dev(lx, kn), dev(lx, vn), theta=1e6)
        want = lx.gqa_decode_attention_paged(q2, two, 0, cap)
        assert np.array_equal(got.numpy(), want.numpy()), f"step {step}"
        assert np.array_equal(one.seq_lens(), two.seq_lens())
    for b in range(B):
        n = int(one.seq_lens()[b])
        k1, v1 = one.gather(0, b, n)
        k2, v2 = two.gather(0, b, n)
        assert np.array_equal(k1, k2) and np.array_equal(v1, v2)
    k, v = one.gather(0, 1, 66)
    ref = chk.gqa_decode(q2.numpy()[1:2].astype(np.float32), k.astype(np.float32), v.astype(np.float32))
    assert oracle.rel_err(got.numpy()[1:2].astype(np.float32), ref) <= 2e-3
    assert lx.device_error_bits() == 0


@pytest.mark.parametrize("use_mrope,qk_norm,heads", [(True, True, (4, 2)), (False, False, (16, 8)), (True, False, (8, 1))])
def test_native_tower_one_launch_layer_step_equals_the_two_kernels(use_mrope, qk_norm, heads):
    """The tower with each layer's norm + rope + append + attention as the one operator (one launch) against
    the same tower running qkv_norm_rope_append and the attention call: identical logits, tokens and pages,
    eagerly and as a captured graph, with lengths on tile and page edges."""
    from axono_b200.native_tower import NativeTextTower
    from axono_b200.tower_config import TextTowerConfig

    cfg = TextTowerConfig(hidden=256, intermediate=512, n_q_heads=heads[0], n_kv_heads=heads[1], head_dim=128, vocab=1000,
                          n_layers=3, use_mrope=use_mrope, qk_norm=qk_norm)
    batch, lens = 4, [70, 63, 127, 1200]
    one = NativeTextTower(cfg, batch, 1408, seed=5)
    two = NativeTextTower(cfg, batch, 1408, seed=5, weights=one.host_weights, fused_step=False)
    assert one.fused_step and not two.fused_step
    for t in (one, two):
        t.arena.fill_normal(21, 0.5)
        t.set_state([7, 8, 9, 10], lens)
    for step in range(3):
        a, b = one.decode_step().numpy(), two.decode_step().numpy()
        assert np.array_equal(one.last_logits.numpy(), two.last_logits.numpy()), f"step {step}"
        assert np.array_equal(a, b)
    g = native.CUDAGraph().capture(one.decode_step)  # its warm-up run is a real step
    two.decode_step()
    for step in range(3):
        g.replay()
        two.decode_step()
        assert np.array_equal(one.last_logits.numpy(), two.last_logits.numpy()), f"replay {step}"
    assert list(one.arena.seq_lens()) == list(two.arena.seq_lens()) == [n + 7 for n in lens]
    for li in range(cfg.n_layers):
        for bi in range(batch):
            k1, v1 = one.arena.gather(li, bi, lens[bi] + 7)
            k2, v2 = two.arena.gather(li, bi, lens[bi] + 7)
            assert np.array_equal(k1, k2) and np.array_equal(v1, v2)
    lx = native.load()
    assert lx.device_error_bits() == 0
    g2 = native.CUDAGraph().capture(two.decode_step)
    assert g.num_nodes == g2.num_nodes - cfg.n_layers  # one launch less per layer: the operator really is one launch
    g.reset()
    g2.reset()
