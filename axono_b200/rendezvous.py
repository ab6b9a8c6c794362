"""Host-side rendezvous of the ranks of one node (one process per GPU), without PyTorch.

The decode path has no data-path collective that needs a library: what the ranks exchange on the
host is small and rare - the 64-byte IPC handles of the peer-mapped buffers at set-up, a barrier on
both sides of a timed region, the maximum of the ranks' times.  This module does that over one
abstract-namespace Unix socket: rank 0 listens, the others connect, and every operation is an
all-gather of one small blob per rank through rank 0.  It also is the host side of failure
detection: every wait has a time limit, so a rank that has left between steps shows up as
`RankLost` at the next barrier of the others instead of as a hang.

    rdv = Rendezvous.from_env()        # RANK / WORLD_SIZE / MASTER_PORT as torchrun exports them
    handles = rdv.all_gather(handle)   # list of bytes, one per rank
    rdv.barrier()
    slowest = rdv.max(my_seconds)
"""
from __future__ import annotations

import os
import pickle
import socket
import struct
import time
from typing import List, Optional


class RankLost(RuntimeError):
    """A peer did not take part in a host-side exchange within the time limit (it exited, or it never
    started).  Raised on every rank that was waiting for it."""


def _send(sock: socket.socket, blob: bytes) -> None:
    sock.sendall(struct.pack("<Q", len(blob)) + blob)


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        part = sock.recv(n - len(buf))
        if not part:
            raise ConnectionError("peer closed the connection")
        buf += part
    return bytes(buf)


def _recv(sock: socket.socket) -> bytes:
    (n,) = struct.unpack("<Q", _recv_exact(sock, 8))
    return _recv_exact(sock, n)


class Rendezvous:
    def __init__(self, rank: int, world: int, key: str, timeout: float = 120.0):
        """`key` names the job on this host (all its ranks pass the same one); `timeout` (seconds)
        bounds the start-up wait and every later exchange."""
        if not 0 <= rank < world:
            raise ValueError("rank outside the world")
        self.rank, self.world, self.timeout = rank, world, float(timeout)
        self._peers: List[Optional[socket.socket]] = [None] * world
        self._server: Optional[socket.socket] = None
        self._up: Optional[socket.socket] = None
        if world == 1:
            return
        addr = "\0axono_b200." + key  # abstract namespace: no file, gone with the process
        deadline = time.monotonic() + self.timeout
        if rank == 0:
            srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            srv.bind(addr)
            srv.listen(world)
            self._server = srv
            joined = 0
            while joined < world - 1:
                srv.settimeout(max(0.01, deadline - time.monotonic()))
                try:
                    conn, _ = srv.accept()
                except (socket.timeout, TimeoutError):
                    missing = [r for r in range(1, world) if self._peers[r] is None]
                    self.close()
                    raise RankLost(f"ranks {missing} did not join within {self.timeout:.0f} s") from None
                conn.settimeout(self.timeout)
                (r,) = struct.unpack("<I", _recv_exact(conn, 4))
                self._peers[r] = conn
                joined += 1
        else:
            while True:
                s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
                try:
                    s.connect(addr)
                    break
                except (FileNotFoundError, ConnectionRefusedError):
                    s.close()
                    if time.monotonic() > deadline:
                        raise RankLost(f"rank 0 did not open the rendezvous within {self.timeout:.0f} s") from None
                    time.sleep(0.02)
            s.settimeout(self.timeout)
            s.sendall(struct.pack("<I", rank))
            self._up = s

    @classmethod
    def from_env(cls, timeout: float = 120.0) -> "Rendezvous":
        """Rank, world and job key from the variables a one-node launcher exports (RANK, WORLD_SIZE,
        MASTER_PORT; the run id when there is one)."""
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        key = os.environ.get("MASTER_PORT", "0") + "." + os.environ.get("TORCHELASTIC_RUN_ID", "job")
        return cls(rank, world, key, timeout)

    # ---- the one primitive: every rank gives a blob, every rank gets all of them ----
    def all_gather(self, blob: bytes) -> List[bytes]:
        if self.world == 1:
            return [bytes(blob)]
        try:
            if self.rank == 0:
                parts = [bytes(blob)] + [b""] * (self.world - 1)
                for r in range(1, self.world):
                    parts[r] = _recv(self._peers[r])
                packed = pickle.dumps(parts)
                for r in range(1, self.world):
                    _send(self._peers[r], packed)
                return parts
            _send(self._up, bytes(blob))
            return pickle.loads(_recv(self._up))
        except (socket.timeout, TimeoutError, ConnectionError, OSError) as e:
            raise RankLost(f"rank {self.rank}: a peer left the job ({type(e).__name__}: {e})") from None

    def barrier(self) -> None:
        self.all_gather(b"")

    def all_gather_object(self, obj) -> list:
        return [pickle.loads(b) for b in self.all_gather(pickle.dumps(obj))]

    def max(self, x: float) -> float:
        return max(self.all_gather_object(float(x)))

    def sum(self, x: float) -> float:
        return sum(self.all_gather_object(float(x)))

    def close(self) -> None:
        for s in self._peers + [self._up, self._server]:
            if s is not None:
                try:
                    s.close()
                except OSError:
                    pass
        self._peers = [None] * self.world
        self._up = self._server = None
