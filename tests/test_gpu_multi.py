"""Two-GPU tests of the head-sharded path: attention fused with the all-gather over peer memory, and
the text-tower step built on it.  Each rank is its own process on its own GPU (ranks that wait on one
another never share a GPU).  Skipped on a single-GPU box."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _widen(a):
    return a.astype(np.float16).astype(np.float32)


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)  # host-side exchange only
    try:
        from axono_b200 import ops, sharding
        from axono_b200.cuda_graph import CUDAGraph
        from axono_b200.decode import TextTower, TextTowerConfig
        from axono_b200.kv_cache import PagedKVCache
        from axono_b200.p2p import PeerGather

        h = torch.float16
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda().to(h)  # noqa: E731

        # ---- fused attention + all-gather against the same attention on all heads locally ----
        rng = np.random.default_rng(7000)
        B, hq, hkv, d, L = 5, 8, 4, 128, 3000
        lens = [L, L - 1, 64, 1000, 2049]
        q = _widen(rng.standard_normal((B, hq, d)).astype(np.float32))
        k = _widen((0.5 * rng.standard_normal((B, L, hkv, d))).astype(np.float32))
        v = _widen((0.5 * rng.standard_normal((B, L, hkv, d))).astype(np.float32))
        full = PagedKVCache(1, B, hkv, d, L, dtype=h)
        full.fill(0, dev(k), dev(v), lens)
        kvh, qh = sharding.shard_kv_heads(hq, hkv, world, rank)
        local = PagedKVCache(1, B, len(kvh), d, L, dtype=h)
        local.fill(0, dev(k[:, :, kvh.start:kvh.stop]), dev(v[:, :, kvh.start:kvh.stop]), lens)
        pg = PeerGather(B, hq, d, h, slots=2)
        for it in range(40):  # many generations, alternating buffers, a different q every time
            qi = dev(q * (1.0 + 0.01 * it))
            want = full.attend(0, qi)
            got = local.attend(0, qi[:, qh.start:qh.stop].contiguous(), gather=(pg, it % 2))
            torch.cuda.synchronize()
            err = (got.float() - want.float()).abs().max().item() / want.float().abs().max().item()
            assert err <= 1e-3, f"rank {rank} iteration {it}: {err:.3e}"
        assert ops.last_error() == 0

        # ---- context-parallel decode: pages of every sequence dealt round-robin to the ranks ----
        Lc = 3000
        clens = [Lc, 40, 64, 65, 1500]  # 40 tokens: only rank 0 holds any
        pe = PeerGather(B, hq, d, h, slots=2, kind="records")
        cp = PagedKVCache(1, B, hkv, d, Lc, dtype=h)
        local_lens, kl, vl = [], np.zeros_like(k), np.zeros_like(v)
        for b_, n in enumerate(clens):
            mine = [t for t in range(n) if (t // 64) % world == rank]
            local_lens.append(len(mine))
            kl[b_, : len(mine)] = k[b_, mine]
            vl[b_, : len(mine)] = v[b_, mine]
        cp.fill(0, dev(kl), dev(vl), local_lens)
        full2 = PagedKVCache(1, B, hkv, d, Lc, dtype=h)
        full2.fill(0, dev(k), dev(v), clens)
        for it in range(6):
            qi = dev(q * (1.0 + 0.02 * it))
            want = full2.attend(0, qi)
            got = cp.attend(0, qi, context_parallel=(pe, it % 2))
            torch.cuda.synchronize()
            err = (got.float() - want.float()).abs().max().item() / want.float().abs().max().item()
            assert err <= 1e-3, f"rank {rank} context-parallel iteration {it}: {err:.3e}"
        assert ops.last_error() == 0

        # ---- text tower: sharded ranks agree with each other and with the unsharded tower ----
        cfg = TextTowerConfig(hidden=256, intermediate=512, n_q_heads=4, n_kv_heads=2, head_dim=128, vocab=1000,
                              n_layers=4)
        Bt, L0 = 4, 300
        r = np.random.default_rng(7001)
        k0 = [_widen((0.5 * r.standard_normal((Bt, L0, 2, 128))).astype(np.float32)) for _ in range(cfg.n_layers)]
        v0 = [_widen((0.5 * r.standard_normal((Bt, L0, 2, 128))).astype(np.float32)) for _ in range(cfg.n_layers)]
        tlens = [L0, L0 - 7, 64, 129]
        tok = r.integers(0, cfg.vocab, Bt)

        def make(w, rk):
            tw = TextTower(cfg, Bt, 512, dtype=h, seed=3, world=w, rank=rk)
            kv, _ = sharding.shard_kv_heads(4, 2, w, rk)
            for li in range(cfg.n_layers):
                tw.cache.fill(li, dev(k0[li][:, :, kv.start:kv.stop]), dev(v0[li][:, :, kv.start:kv.stop]), tlens)
            tw.set_state(tok, tlens)
            return tw

        single, shard = make(1, 0), make(world, rank)
        ops.workspace("cuda", ops.gqa_workspace_bytes(Bt, 4, 2, 128, 512))
        g = None
        for step in range(4):
            if step == 0:
                shard.decode_step()  # eager
            else:
                if g is None:  # capture after the eager step; a capture run executes nothing
                    g = CUDAGraph().capture(shard.decode_step, warmup=False)
                g.replay()
                shard.cache.note_replayed()
            single.decode_step()
            torch.cuda.synchronize()
            a, b = shard.last_logits.float(), single.last_logits.float()
            err = (a - b).abs().max().item() / b.abs().max().item()
            assert err <= 2e-2, f"rank {rank} step {step}: logits differ {err:.3e}"
            toks = [None] * world
            dist.all_gather_object(toks, shard.token_ids.cpu().tolist())
            assert all(t == toks[0] for t in toks), "ranks disagree on the next tokens"
            single.token_ids.copy_(shard.token_ids)  # keep the two on the same trajectory
        assert ops.last_error() == 0
        shard.peer_gather.close()
        pe.close()
        pg.close()
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.timeout(240)
def test_fused_gather_and_sharded_tower_two_gpus(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def _run_native_ranks(phase, tmp_path, limit):
    """The ranks of tests/native_two_gpu_worker.py as clean interpreter processes (no PyTorch in them), each
    with a hard time limit: a rank that is still running when the limit is up is ended by its PID and the
    test fails - nothing is left waiting.  NVLS is switched off in the library the workers may load: a rank
    that is ended must not hold memory bound to an in-switch reduction group."""
    import subprocess
    import sys
    import time

    world = 2
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    key = f"test.{os.getpid()}.{_free_port()}"
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""), NCCL_NVLS_ENABLE="0")
    logs = [open(tmp_path / f"rank{r}.log", "w+") for r in range(world)]
    procs = [subprocess.Popen([sys.executable, os.path.join(root, "tests", "native_two_gpu_worker.py"), phase, str(r),
                               str(world), key, str(tmp_path)], stdout=logs[r], stderr=subprocess.STDOUT, env=env, cwd=root)
             for r in range(world)]
    deadline = time.monotonic() + limit
    for p in procs:
        try:
            p.wait(max(1.0, deadline - time.monotonic()))
        except subprocess.TimeoutExpired:
            pass
    late = [p.poll() is None for p in procs]
    for p in procs:
        if p.poll() is None:
            p.kill()
            p.wait(20)
    out = []
    for r, f in enumerate(logs):
        f.seek(0)
        out.append(f"--- rank {r} ---\n" + f.read()[-3000:])
        f.close()
    assert not any(late), f"ranks still running after {limit} s were ended: {late}\n" + "\n".join(out)
    assert all(p.returncode == 0 for p in procs), "\n".join(out)
    assert all((tmp_path / f"native_{phase}_ok{r}").exists() for r in range(world))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.timeout(240)
def test_native_runtime_two_gpus(tmp_path):
    _run_native_ranks("fused", tmp_path, limit=150)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.timeout(240)
def test_native_runtime_two_gpus_nccl_gather_in_the_graph(tmp_path):
    """The library form of the gather.  The workers are clean processes, so `libnccl.so.2` resolves as it does
    for `bench.py --gather nccl`: to the system's library, not to the copy a framework bundles."""
    _run_native_ranks("nccl", tmp_path, limit=150)
