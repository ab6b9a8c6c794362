"""Host-side rendezvous of the ranks (CPU only): the exchanges the multi-GPU paths make on the host, and
failure detection on the host - a rank that leaves between steps, or never starts, turns into
`RankLost` on the ranks that wait for it, within the time limit, instead of a hang."""
import multiprocessing as mp
import os
import time

import pytest

from axono_b200.rendezvous import RankLost, Rendezvous


def _key():
    return f"test.{os.getpid()}.{time.monotonic_ns()}"


def _rank_main(rank, world, key, leave_after, out):
    try:
        rdv = Rendezvous(rank, world, key, timeout=5.0)
        parts = rdv.all_gather(bytes([rank]) * (rank + 1))
        out.put((rank, "gather", [p.hex() for p in parts]))
        out.put((rank, "max", rdv.max(10.0 * rank), rdv.sum(float(rank))))
        for step in range(4):
            if rank == leave_after[0] and step == leave_after[1]:
                rdv.close()  # this rank leaves between steps: nothing of its is in flight
                out.put((rank, "left", step))
                return
            rdv.barrier()
        out.put((rank, "done"))
        rdv.close()
    except RankLost as e:
        out.put((rank, "lost", str(e)))


def _run(world, leave_after=(-1, -1)):
    ctx = mp.get_context("spawn")
    out, key = ctx.Queue(), _key()
    procs = [ctx.Process(target=_rank_main, args=(r, world, key, leave_after, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive()
    msgs = []
    while not out.empty():
        msgs.append(out.get())
    return msgs


@pytest.mark.parametrize("world", [2, 3])
def test_all_gather_barrier_and_reductions(world):
    msgs = _run(world)
    want = [(bytes([r]) * (r + 1)).hex() for r in range(world)]
    for r in range(world):
        assert (r, "gather", want) in msgs
        assert (r, "max", 10.0 * (world - 1), float(sum(range(world)))) in msgs
        assert (r, "done") in msgs


def test_a_rank_that_leaves_between_steps_is_detected():
    t0 = time.monotonic()
    msgs = _run(3, leave_after=(2, 1))
    assert (2, "left", 1) in msgs
    lost = {m[0] for m in msgs if m[1] == "lost"}
    assert lost == {0, 1}, msgs  # both survivors learn of it at their next barrier
    assert time.monotonic() - t0 < 30


def test_a_rank_that_never_starts_is_detected():
    t0 = time.monotonic()
    with pytest.raises(RankLost):
        Rendezvous(0, 2, _key(), timeout=0.5)
    with pytest.raises(RankLost):
        Rendezvous(1, 2, _key(), timeout=0.5)
    assert time.monotonic() - t0 < 10


def test_single_rank_needs_no_socket():
    rdv = Rendezvous(0, 1, "unused")
    assert rdv.all_gather(b"x") == [b"x"] and rdv.max(3.0) == 3.0 and rdv.sum(2.0) == 2.0
    rdv.barrier()
    rdv.close()
