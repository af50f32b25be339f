"""A minimal TCP rendezvous for one-process-per-GPU runs, standard library only.

The reference drives all GPUs from one process (flyvec/train_flyvec.py:141-146)
and so does ``flyvec_train --gpus N`` by default.  When a launcher starts one
process per GPU instead (``RANK`` / ``WORLD_SIZE`` / ``MASTER_ADDR`` /
``MASTER_PORT`` in the environment, as ``torch.distributed.run``, ``srun`` or
``mpirun`` wrappers set them), the ranks only need two things from each other
before the library's own exchange takes over: the 128-byte communicator id and
rank 0's initial weights.  Rank 0 serves both over a socket on
``MASTER_PORT + 1``; nothing here imports torch.
"""
from __future__ import annotations

import os
import socket
import struct
import time

import numpy as np


def env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        part = sock.recv(min(1 << 20, n - len(buf)))
        if not part:
            raise ConnectionError("rendezvous peer closed the connection early")
        buf += part
    return bytes(buf)


class Rendezvous:
    """``broadcast(payload)``: rank 0's bytes to every rank; ``barrier()``: all ranks meet.
    The connections stay open for the lifetime of the object."""

    def __init__(self, rank: int, world: int, addr: str | None = None, port: int | None = None, timeout: float = 300.0):
        self.rank, self.world = rank, world
        self.peers: list[socket.socket] = []
        if world == 1:
            return
        addr = addr or os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = port if port is not None else int(os.environ.get("MASTER_PORT", "29500")) + 1
        if rank == 0:
            srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            srv.bind(("", port))
            srv.listen(world)
            srv.settimeout(timeout)
            slots: dict[int, socket.socket] = {}
            while len(slots) < world - 1:
                conn, _ = srv.accept()
                conn.settimeout(timeout)
                (r,) = struct.unpack("<i", _recv_exact(conn, 4))
                slots[r] = conn
            srv.close()
            self.peers = [slots[r] for r in sorted(slots)]
        else:
            deadline = time.time() + timeout
            while True:
                try:
                    s = socket.create_connection((addr, port), timeout=5.0)
                    break
                except OSError:
                    if time.time() > deadline:
                        raise
                    time.sleep(0.2)
            s.settimeout(timeout)
            s.sendall(struct.pack("<i", rank))
            self.peers = [s]

    def broadcast(self, payload: bytes | None) -> bytes:
        if self.world == 1:
            return payload
        if self.rank == 0:
            head = struct.pack("<q", len(payload))
            for p in self.peers:
                p.sendall(head + payload)
            return payload
        (n,) = struct.unpack("<q", _recv_exact(self.peers[0], 8))
        return _recv_exact(self.peers[0], n)

    def broadcast_array(self, a: np.ndarray | None, shape, dtype) -> np.ndarray:
        raw = self.broadcast(np.ascontiguousarray(a, dtype).tobytes() if self.rank == 0 else None)
        return np.frombuffer(raw, dtype=dtype).reshape(shape).copy() if self.rank != 0 else np.ascontiguousarray(a, dtype)

    def barrier(self):
        if self.world == 1:
            return
        if self.rank == 0:
            for p in self.peers:
                _recv_exact(p, 1)
            for p in self.peers:
                p.sendall(b"\x01")
        else:
            self.peers[0].sendall(b"\x01")
            _recv_exact(self.peers[0], 1)

    def close(self):
        for p in self.peers:
            try:
                p.close()
            except OSError:
                pass
        self.peers = []
