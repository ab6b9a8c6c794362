"""One rank of the native-runtime two-GPU checks, run as a process of its own by tests/test_gpu_multi.py:

    python tests/native_two_gpu_worker.py <fused|nccl> <rank> <world> <rendezvous key> <out dir>

No PyTorch in this process (the product path has none): ranks meet over the package's own host
rendezvous, and the NCCL form loads the system's libnccl.so.2 exactly as `bench.py` does.
fused: the two cross-GPU forms of attention against local attention, then the head-sharded native tower
against the unsharded one (eager step, captured step, replays).  nccl: the library form of the gather
(ncclAllGather + re-layout recorded into the step's graph) against the unsharded tower."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _setup(rank, world, key):
    from axono_b200 import native
    from axono_b200.rendezvous import Rendezvous
    from axono_b200.tower_config import TextTowerConfig

    lx = native.load()
    lx.set_device(rank)
    rdv = Rendezvous(rank, world, key, timeout=60.0)
    cfg = TextTowerConfig(hidden=256, intermediate=512, n_q_heads=8, n_kv_heads=4, head_dim=128, vocab=1000, n_layers=3)
    return native, lx, rdv, cfg, f"cuda:{rank}"


BT, L0, FULL_SEED = 4, 300, 11
LENS = [L0, L0 - 7, 64, 129]


def _fill_shard(full, shard, cfg, rank, world):
    """The sharded arena holds this rank's KV heads of the full one."""
    from axono_b200.native_multi import write_tokens

    per = cfg.n_kv_heads // world
    for li in range(cfg.n_layers):
        for b in range(BT):
            kf, vf = full.arena.gather(li, b, LENS[b])
            write_tokens(shard.arena, li, b, np.ascontiguousarray(kf[:, rank * per:(rank + 1) * per]),
                         np.ascontiguousarray(vf[:, rank * per:(rank + 1) * per]))


def fused(rank, world, key):
    from axono_b200.native_multi import multi_gpu_parity
    from axono_b200.native_tower import NativeTextTower

    native, lx, rdv, cfg, device = _setup(rank, world, key)
    res = multi_gpu_parity(rdv, device)
    assert res["gather"] <= 1e-3 and res["cp"] <= 1e-3 and res["device_error_bits"] == 0, res
    tok = np.random.default_rng(7001).integers(0, cfg.vocab, BT)
    shard = NativeTextTower(cfg, BT, 512, seed=3, device=device, rdv=rdv)
    single = NativeTextTower(cfg, BT, 512, seed=3, device=device, weights=shard.host_weights)
    single.arena.fill_normal(FULL_SEED, 0.5)
    _fill_shard(single, shard, cfg, rank, world)
    shard.set_state(tok, LENS)
    single.set_state(tok, LENS)
    g = None
    for step in range(4):
        if step == 0:
            shard.decode_step()  # eager
        elif g is None:
            g = native.CUDAGraph().capture(shard.decode_step)  # its warm-up run is a real step
        else:
            g.replay()
        single.decode_step()
        lx.synchronize()
        a, b_ = shard.last_logits.numpy().astype(np.float32), single.last_logits.numpy().astype(np.float32)
        err = float(np.abs(a - b_).max() / np.abs(b_).max())
        assert err <= 2e-2, f"rank {rank} step {step}: logits differ {err:.3e}"
        toks = rdv.all_gather_object(shard.token_ids.numpy().tolist())
        assert all(t == toks[0] for t in toks), "ranks disagree on the next tokens"
        single.token_ids.copy_from(shard.token_ids)  # keep the two on the same trajectory
    assert lx.device_error_bits() == 0
    if g is not None:
        g.reset()
    shard.close()
    rdv.close()
    assert "torch" not in sys.modules


def nccl(rank, world, key):
    from axono_b200.native_tower import NativeTextTower

    native, lx, rdv, cfg, device = _setup(rank, world, key)
    tok = np.random.default_rng(7001).integers(0, cfg.vocab, BT)
    ref = NativeTextTower(cfg, BT, 512, seed=3, device=device)
    coll = NativeTextTower(cfg, BT, 512, seed=3, device=device, rdv=rdv, weights=ref.host_weights, gather="nccl")
    ref.arena.fill_normal(FULL_SEED, 0.5)
    _fill_shard(ref, coll, cfg, rank, world)
    coll.set_state(tok, LENS)
    ref.set_state(tok, LENS)
    print("towers ready", flush=True)
    gc = native.CUDAGraph().capture(coll.decode_step)  # warm-up run = step 1, then captured with the collective inside
    print("captured", gc.num_nodes, flush=True)
    ref.decode_step()
    for step in range(2):
        lx.synchronize()
        print("step", step, "synchronised", flush=True)
        a, b_ = coll.last_logits.numpy().astype(np.float32), ref.last_logits.numpy().astype(np.float32)
        err = float(np.abs(a - b_).max() / np.abs(b_).max())
        assert err <= 2e-2, f"rank {rank} NCCL step {step}: logits differ {err:.3e}"
        ref.token_ids.copy_from(coll.token_ids)
        gc.replay()
        ref.decode_step()
    lx.synchronize()
    assert gc.num_nodes > 0 and lx.device_error_bits() == 0
    gc.reset()  # ncclCommDestroy waits for every graph that recorded work of the communicator to be gone
    coll.close()
    rdv.close()
    assert "torch" not in sys.modules


if __name__ == "__main__":
    import faulthandler

    # a rank that is stuck says where (the Python frame of the call that does not return) and ends by itself,
    # before the parent's limit ends it without a word
    faulthandler.dump_traceback_later(100, exit=True)
    phase, rank, world, key, out_dir = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], sys.argv[5]
    {"fused": fused, "nccl": nccl}[phase](rank, world, key)
    open(os.path.join(out_dir, f"native_{phase}_ok{rank}"), "w").close()
