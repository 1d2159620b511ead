"""One transport contract for everything that moves messages between ranks on the host.

``Transport``            send / recv / barrier / close between numbered ranks; a dead or departed peer surfaces at once
                         as ``PeerLost`` naming that rank (never as a hang or an anonymous socket error)
``DeviceTransport``      the same for device buffers (the peer-memory communicator of ``parallel.comm``)
``MemoryTransport``      ranks as threads of one process (tests, the simulator's default wire); can corrupt on purpose
``SharedMemoryTransport`` single-producer single-consumer rings in POSIX shared memory with a doorbell word per ring
``FramedTcpTransport``   length-prefixed frames over TCP with credit flow control, ``bye`` (orderly leave) and
                         ``abandon`` (peer gone) frames, and an HMAC-authenticated rendezvous
``TorchDistTransport``   torch.distributed point-to-point (gloo or NCCL) behind the same calls

``as_exchange()`` adapts any of them to the simultaneous send+receive primitive the host collectives are written on, so
the simulator, gloo ranks and the shared-memory / TCP transports run the same collective algorithms.

Reference: ITransport / IDeviceTransport (src/Idrak.Abstraction/Cluster), FramedTransport
(src/Idrak.Network/Abstractions/FramedTransport.cs:29,335-363,477), SharedMemoryTransport
(src/Idrak.Network/Transports/SharedMemoryTransport.cs:30,264), Rendezvous (Transports/Rendezvous.cs:28,302).
"""
from __future__ import annotations

import hashlib
import hmac
import os
import queue
import socket
import struct
import threading
import time
from typing import Any, Callable, Dict, List, Optional, Sequence

import numpy as np
import torch


class PeerLost(ConnectionError):
    """A peer can no longer be reached. ``rank`` is the peer; ``orderly`` says it announced its leave (``bye``)."""

    def __init__(self, rank: int, why: str = "", orderly: bool = False):
        super().__init__(f"rank {rank} {'left' if orderly else 'is gone'}{': ' + why if why else ''}")
        self.rank, self.orderly = rank, orderly


class WireCorruption(ValueError):
    """A frame failed its check (length, magic or checksum)."""


class Transport:
    """Ordered, reliable messages of flat tensors between ranks ``0 .. world - 1``."""
    rank: int
    world: int

    def send(self, dst: int, values: torch.Tensor) -> None:
        raise NotImplementedError

    def recv(self, src: int, timeout: Optional[float] = None) -> torch.Tensor:
        raise NotImplementedError

    def close(self, orderly: bool = True) -> None:
        """Leaves the group; peers blocked on this rank get ``PeerLost`` (``orderly`` tells them it was announced)."""

    def barrier(self, timeout: Optional[float] = None) -> None:
        """Dissemination barrier over send / recv: log2(world) rounds, no root."""
        token = torch.zeros(1)
        k = 1
        while k < self.world:
            self.send((self.rank + k) % self.world, token)
            self.recv((self.rank - k) % self.world, timeout)
            k *= 2

    def as_exchange(self):
        return _ExchangeAdapter(self)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close(orderly=exc[0] is None)
        return False


class DeviceTransport:
    """Device-side counterpart: collectives over buffers that live in GPU memory. ``parallel.comm.Communicator``
    satisfies it; the contract is stated here so host-side code can be written against either."""
    rank: int
    world: int

    def all_reduce(self, values: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def all_gather(self, piece: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def reduce_scatter(self, values: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def barrier(self) -> None:
        raise NotImplementedError


class _ExchangeAdapter:
    """Send and receive at once on top of an ordered transport. The send runs on a helper thread while this thread
    receives: with bounded buffering (a ring smaller than the message, exhausted credit) every rank of a ring would
    otherwise sit in its send while nobody receives."""

    def __init__(self, t: Transport):
        self.t, self.rank, self.world = t, t.rank, t.world
        self._jobs: "queue.Queue" = queue.Queue()
        self._done: "queue.Queue" = queue.Queue()
        self._worker: Optional[threading.Thread] = None

    def _sender(self):
        while True:
            job = self._jobs.get()
            if job is None:
                return
            try:
                self.t.send(*job)
                self._done.put(None)
            except BaseException as e:      # handed to the thread that asked for the exchange
                self._done.put(e)

    def exchange(self, dst, out, src, count, dtype):
        if dst is not None and src is None:
            self.t.send(dst, out)
            return None
        if dst is not None:
            if self._worker is None:
                self._worker = threading.Thread(target=self._sender, daemon=True)
                self._worker.start()
            self._jobs.put((dst, out))
        got = None
        try:
            if src is not None:
                got = self.t.recv(src)
        finally:
            if dst is not None:
                err = self._done.get()
                if err is not None:
                    raise err
        return got.to(dtype) if got is not None and got.dtype != dtype else got


# --------------------------------------------------------------------------- in-process
class MemoryTransport(Transport):
    """Ranks as threads of one process. ``MemoryTransport.hub(world)`` makes the group; ``hub.run(fn)`` runs
    ``fn(rank, transport)`` on one thread per rank and returns the results in rank order."""

    class Hub:
        def __init__(self, world: int, corrupt: bool = False, timeout: float = 20.0):
            self.world, self.corrupt, self.timeout = world, corrupt, timeout
            self.boxes = {(s, d): queue.Queue() for s in range(world) for d in range(world)}
            self.left: Dict[int, bool] = {}              # rank -> orderly
            self.ends = [MemoryTransport(self, r) for r in range(world)]

        def run(self, fn: Callable[[int, "MemoryTransport"], Any]) -> List[Any]:
            results: List[Any] = [None] * self.world
            errors: List[Optional[BaseException]] = [None] * self.world

            def main(r):
                try:
                    results[r] = fn(r, self.ends[r])
                except BaseException as e:          # surfaced below, with the rank
                    errors[r] = e
                    self.ends[r].close(orderly=False)
            threads = [threading.Thread(target=main, args=(r,), daemon=True) for r in range(self.world)]
            for t in threads:
                t.start()
            for t in threads:
                t.join(self.timeout * 4)
            for r, e in enumerate(errors):
                if e is not None and not isinstance(e, PeerLost):
                    raise RuntimeError(f"rank {r} failed: {e}") from e
            for e in errors:
                if e is not None:
                    raise e
            return results

    @classmethod
    def hub(cls, world: int, corrupt: bool = False, timeout: float = 20.0) -> "MemoryTransport.Hub":
        return cls.Hub(world, corrupt, timeout)

    def __init__(self, hub: "MemoryTransport.Hub", rank: int):
        self.hub_, self.rank, self.world = hub, rank, hub.world
        self._sent = 0

    def send(self, dst, values):
        if dst in self.hub_.left:
            raise PeerLost(dst, "send to a rank that left", self.hub_.left[dst])
        v = values.detach().clone()
        self._sent += 1
        if self.hub_.corrupt and v.numel() and v.is_floating_point() and self._sent % 3 == 0:
            v.view(-1)[0] += 1.0            # the deliberately broken wire: one value off every third message
        self.hub_.boxes[(self.rank, dst)].put(v)

    def recv(self, src, timeout=None):
        deadline = time.monotonic() + (timeout if timeout is not None else self.hub_.timeout)
        box = self.hub_.boxes[(src, self.rank)]
        while True:
            try:
                return box.get(timeout=0.02)
            except queue.Empty:
                if src in self.hub_.left and box.empty():
                    raise PeerLost(src, "while waiting for its message", self.hub_.left[src])
                if time.monotonic() > deadline:
                    raise PeerLost(src, "no message within the time limit")

    def close(self, orderly=True):
        self.hub_.left.setdefault(self.rank, orderly)


# --------------------------------------------------------------------------- frames shared by the byte transports
_MAGIC = 0x4B524449            # "IDRK"
_KIND_DATA, _KIND_CREDIT, _KIND_BYE, _KIND_ABANDON = 1, 2, 3, 4
_DTYPES = [torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64, torch.uint8, torch.int8,
           torch.float64]
_HEADER = struct.Struct("<IBBHQI")     # magic, kind, dtype, reserved, payload bytes, crc of the payload


def _crc(b: bytes) -> int:
    import zlib
    return zlib.crc32(b) & 0xFFFFFFFF


def encode_frame(kind: int, values: Optional[torch.Tensor] = None) -> bytes:
    if values is None:
        return _HEADER.pack(_MAGIC, kind, 0, 0, 0, 0)
    flat = values.detach().contiguous().reshape(-1).cpu()
    raw = flat.view(torch.uint8).numpy().tobytes()
    return _HEADER.pack(_MAGIC, kind, _DTYPES.index(flat.dtype), 0, len(raw), _crc(raw)) + raw


def decode_header(head: bytes):
    magic, kind, dt, _, nbytes, crc = _HEADER.unpack(head)
    if magic != _MAGIC or kind not in (_KIND_DATA, _KIND_CREDIT, _KIND_BYE, _KIND_ABANDON) or dt >= len(_DTYPES):
        raise WireCorruption("frame header does not parse")
    return kind, _DTYPES[dt], nbytes, crc


def decode_payload(raw: bytes, dtype: torch.dtype, crc: int) -> torch.Tensor:
    if _crc(raw) != crc:
        raise WireCorruption("frame checksum mismatch")
    return torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dtype).clone() if raw else torch.empty(0, dtype=dtype)


# --------------------------------------------------------------------------- rendezvous (HMAC-authenticated)
def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            raise EOFError("connection closed")
        buf += chunk
    return bytes(buf)


def _send_blob(sock, b: bytes) -> None:
    sock.sendall(struct.pack("<I", len(b)) + b)


def _recv_blob(sock, limit: int = 1 << 20) -> bytes:
    (n,) = struct.unpack("<I", _recv_exact(sock, 4))
    if n > limit:
        raise WireCorruption("rendezvous message too long")
    return _recv_exact(sock, n)


def _prove(sock, secret: bytes, who: bytes) -> None:
    """Client side of the handshake: answer the server's nonce with HMAC(secret, nonce + who)."""
    nonce = _recv_blob(sock)
    _send_blob(sock, who)
    _send_blob(sock, hmac.new(secret, nonce + who, hashlib.sha256).digest())
    if _recv_blob(sock) != b"ok":
        raise PermissionError("rendezvous refused the shared secret")


def _challenge(sock, secret: bytes) -> bytes:
    """Server side: returns who the peer says it is once it proved knowledge of the secret."""
    nonce = os.urandom(32)
    _send_blob(sock, nonce)
    who = _recv_blob(sock)
    proof = _recv_blob(sock)
    if not hmac.compare_digest(proof, hmac.new(secret, nonce + who, hashlib.sha256).digest()):
        _send_blob(sock, b"no")
        raise PermissionError("peer failed the shared-secret check")
    _send_blob(sock, b"ok")
    return who


class Rendezvous:
    """Rank 0 listens on ``(host, port)``; every rank proves the shared secret, posts the address it accepts peers on
    and gets back the full table once all ``world`` ranks arrived."""

    def __init__(self, host: str, port: int, world: int, secret: bytes, timeout: float = 30.0):
        self.host, self.port, self.world, self.secret, self.timeout = host, port, world, secret, timeout

    def serve(self) -> threading.Thread:
        srv = socket.socket()
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        srv.bind((self.host, self.port))
        srv.listen(self.world)
        srv.settimeout(self.timeout)
        if self.port == 0:
            self.port = srv.getsockname()[1]

        def main():
            table: Dict[int, str] = {}
            conns = []
            try:
                while len(table) < self.world:
                    c, _ = srv.accept()
                    c.settimeout(self.timeout)
                    try:
                        who = _challenge(c, self.secret)
                    except (PermissionError, EOFError, WireCorruption, OSError):
                        c.close()          # a stranger does not count toward the world
                        continue
                    rank_s, addr = who.decode().split("@", 1)
                    table[int(rank_s)] = addr
                    conns.append(c)
                blob = ";".join(f"{r}@{a}" for r, a in sorted(table.items())).encode()
                for c in conns:
                    _send_blob(c, blob)
            finally:
                for c in conns:
                    c.close()
                srv.close()
        t = threading.Thread(target=main, daemon=True)
        t.start()
        return t

    def join(self, rank: int, my_address: str) -> Dict[int, str]:
        deadline = time.monotonic() + self.timeout
        while True:
            try:
                s = socket.create_connection((self.host, self.port), timeout=self.timeout)
                break
            except OSError:
                if time.monotonic() > deadline:
                    raise PeerLost(0, "rendezvous host does not answer")
                time.sleep(0.05)
        with s:
            s.settimeout(self.timeout)
            _prove(s, self.secret, f"{rank}@{my_address}".encode())
            blob = _recv_blob(s).decode()
        return {int(e.split("@", 1)[0]): e.split("@", 1)[1] for e in blob.split(";")}


# --------------------------------------------------------------------------- framed TCP
class FramedTcpTransport(Transport):
    """Full mesh of TCP connections carrying checked frames.

    Flow control is by credit: a sender may have ``credits`` data frames per peer outstanding; the receiver returns one
    credit when the application takes a message, so a slow consumer stalls its producers instead of growing a queue.
    ``close(orderly=True)`` sends ``bye`` to every peer; a connection that ends without it, or a failed checksum, is an
    ``abandon``: whoever waits on that rank gets ``PeerLost`` at once."""

    def __init__(self, rank: int, world: int, rendezvous: Rendezvous, credits: int = 8, host: str = "127.0.0.1",
                 timeout: float = 30.0):
        self.rank, self.world, self.credits, self.timeout = rank, world, credits, timeout
        self._inbox = {r: queue.Queue() for r in range(world) if r != rank}
        self._credit = {r: threading.Semaphore(credits) for r in range(world) if r != rank}
        self._gone: Dict[int, bool] = {}
        self._socks: Dict[int, socket.socket] = {}
        self._locks = {r: threading.Lock() for r in range(world) if r != rank}
        self._closed = False
        lst = socket.socket()
        lst.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        lst.bind((host, 0))
        lst.listen(world)
        lst.settimeout(timeout)
        if rank == 0:
            rendezvous.serve()
        table = rendezvous.join(rank, f"{host}:{lst.getsockname()[1]}")
        # the higher rank dials the lower one; both ends prove the secret again on the data connection
        for peer in range(rank):
            h, p = table[peer].rsplit(":", 1)
            s = socket.create_connection((h, int(p)), timeout=timeout)
            _prove(s, rendezvous.secret, str(rank).encode())
            self._adopt(peer, s)
        for _ in range(world - 1 - rank):
            c, _addr = lst.accept()
            c.settimeout(timeout)
            peer = int(_challenge(c, rendezvous.secret).decode())
            self._adopt(peer, c)
        lst.close()

    def _adopt(self, peer: int, s: socket.socket) -> None:
        s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        s.settimeout(None)
        self._socks[peer] = s
        threading.Thread(target=self._reader, args=(peer, s), daemon=True).start()

    def _mark_gone(self, peer: int, orderly: bool) -> None:
        self._gone.setdefault(peer, orderly)
        self._inbox[peer].put(None)                  # wakes a waiting recv
        for _ in range(self.credits):
            self._credit[peer].release()             # and a sender waiting for credit

    def _reader(self, peer: int, s: socket.socket) -> None:
        try:
            while True:
                kind, dtype, nbytes, crc = decode_header(_recv_exact(s, _HEADER.size))
                if kind == _KIND_DATA:
                    self._inbox[peer].put(decode_payload(_recv_exact(s, nbytes), dtype, crc))
                elif kind == _KIND_CREDIT:
                    self._credit[peer].release()
                elif kind == _KIND_BYE:
                    self._mark_gone(peer, True)
                    return
                else:
                    self._mark_gone(peer, False)
                    return
        except (EOFError, OSError, WireCorruption, struct.error):
            if not self._closed:
                self._mark_gone(peer, False)

    def _write(self, peer: int, frame: bytes) -> None:
        try:
            with self._locks[peer]:
                self._socks[peer].sendall(frame)
        except OSError as e:
            self._gone.setdefault(peer, False)
            raise PeerLost(peer, f"send failed ({e})")

    def send(self, dst, values):
        if dst in self._gone:
            raise PeerLost(dst, "send to a rank that left", self._gone[dst])
        if not self._credit[dst].acquire(timeout=self.timeout):
            raise PeerLost(dst, "no credit returned within the time limit")
        if dst in self._gone:
            raise PeerLost(dst, "left while this rank waited for credit", self._gone[dst])
        self._write(dst, encode_frame(_KIND_DATA, values))

    def recv(self, src, timeout=None):
        try:
            got = self._inbox[src].get(timeout=timeout if timeout is not None else self.timeout)
        except queue.Empty:
            raise PeerLost(src, "no message within the time limit")
        if got is None:
            self._inbox[src].put(None)               # stays lost for later calls
            raise PeerLost(src, "while waiting for its message", self._gone.get(src, False))
        if src not in self._gone:
            try:
                self._write(src, encode_frame(_KIND_CREDIT))
            except PeerLost:
                pass                                 # the message itself arrived; the loss shows on the next call
        return got

    def close(self, orderly=True):
        if self._closed:
            return
        self._closed = True
        for peer, s in self._socks.items():
            try:
                if peer not in self._gone:
                    with self._locks[peer]:
                        s.sendall(encode_frame(_KIND_BYE if orderly else _KIND_ABANDON))
                s.shutdown(socket.SHUT_RDWR)
            except OSError:
                pass
            s.close()


# --------------------------------------------------------------------------- shared-memory rings
class _Ring:
    """Single-producer single-consumer byte ring in a shared-memory block.

    Layout: [head u64 | tail u64 | doorbell u64 | state u64 | heartbeat f64 | pad to 64] + data. ``head`` counts bytes
    written, ``tail`` bytes consumed; the doorbell is bumped after every write so a consumer polls one word."""
    HEADER = 64

    def __init__(self, name: str, capacity: int, create: bool):
        from multiprocessing import shared_memory
        if create:
            self.shm = shared_memory.SharedMemory(name=name, create=True, size=self.HEADER + capacity)
            self.shm.buf[: self.HEADER] = bytes(self.HEADER)
        else:
            self.shm = shared_memory.SharedMemory(name=name)
        self.capacity = self.shm.size - self.HEADER if not create else capacity
        self.words = np.ndarray((4,), dtype=np.uint64, buffer=self.shm.buf, offset=0)
        self.beat = np.ndarray((1,), dtype=np.float64, buffer=self.shm.buf, offset=32)
        self.data = np.ndarray((self.capacity,), dtype=np.uint8, buffer=self.shm.buf, offset=self.HEADER)
        self.owner = create

    def free(self) -> int:
        return self.capacity - int(self.words[0] - self.words[1])

    def write(self, b: bytes) -> None:
        n, pos = len(b), int(self.words[0]) % self.capacity
        first = min(n, self.capacity - pos)
        self.data[pos:pos + first] = np.frombuffer(b[:first], dtype=np.uint8)
        if first < n:
            self.data[: n - first] = np.frombuffer(b[first:], dtype=np.uint8)
        self.words[0] += np.uint64(n)
        self.words[2] += np.uint64(1)

    def available(self) -> int:
        return int(self.words[0] - self.words[1])

    def read(self, n: int) -> bytes:
        pos = int(self.words[1]) % self.capacity
        first = min(n, self.capacity - pos)
        out = self.data[pos:pos + first].tobytes()
        if first < n:
            out += self.data[: n - first].tobytes()
        self.words[1] += np.uint64(n)
        return out

    def close(self):
        self.words = self.beat = self.data = None
        self.shm.close()
        if self.owner:
            try:
                self.shm.unlink()
            except FileNotFoundError:
                pass


class SharedMemoryTransport(Transport):
    """Ranks of one machine over rings in shared memory: ring (s, d) is created by its consumer d and written by s.

    A message larger than the ring streams through it in pieces. A departing rank writes 2 (bye) or 3 (abandon) into
    the state word of the rings it produces into; a rank that died without a word stops refreshing its heartbeat and
    is declared gone after ``stale_after`` seconds."""
    STATE_PRESENT, STATE_BYE, STATE_ABANDON = 1, 2, 3

    def __init__(self, rank: int, world: int, session: str, capacity: int = 1 << 20, timeout: float = 30.0,
                 stale_after: float = 5.0):
        self.rank, self.world, self.timeout, self.stale_after = rank, world, timeout, stale_after
        self._in = {s: _Ring(f"{session}-{s}-{rank}", capacity, True) for s in range(world) if s != rank}
        self._out: Dict[int, _Ring] = {}
        deadline = time.monotonic() + timeout
        for d in range(world):
            if d == rank:
                continue
            while True:
                try:
                    self._out[d] = _Ring(f"{session}-{rank}-{d}", capacity, False)
                    break
                except FileNotFoundError:
                    if time.monotonic() > deadline:
                        raise PeerLost(d, "never created its ring")
                    time.sleep(0.01)
            self._out[d].words[3] = np.uint64(self.STATE_PRESENT)
            self._out[d].beat[0] = time.time()
        self._stop = threading.Event()
        threading.Thread(target=self._heartbeat, daemon=True).start()

    def _heartbeat(self):
        while not self._stop.wait(0.2):
            now = time.time()
            for r in self._out.values():
                if r.beat is not None:
                    r.beat[0] = now

    def _check(self, peer: int, ring: _Ring) -> None:
        state = int(ring.words[3])
        if state in (self.STATE_BYE, self.STATE_ABANDON) and ring.available() == 0:
            raise PeerLost(peer, "while waiting for its message", state == self.STATE_BYE)
        if state == self.STATE_PRESENT and time.time() - float(ring.beat[0]) > self.stale_after:
            raise PeerLost(peer, "heartbeat went stale")

    def _pull(self, src: int, n: int, deadline: float) -> bytes:
        ring, out = self._in[src], bytearray()
        while len(out) < n:
            have = ring.available()
            if have:
                out += ring.read(min(have, n - len(out)))
                continue
            self._check(src, ring)
            if time.monotonic() > deadline:
                raise PeerLost(src, "no message within the time limit")
            time.sleep(0.0002)
        return bytes(out)

    def send(self, dst, values):
        ring = self._out[dst]
        frame = encode_frame(_KIND_DATA, values)
        deadline = time.monotonic() + self.timeout
        back = self._in[dst]                        # the peer's own outbound ring tells whether it is still there
        at = 0
        while at < len(frame):
            room = ring.free()
            if room:
                step = min(room, len(frame) - at)
                ring.write(frame[at:at + step])
                at += step
                continue
            if int(back.words[3]) in (self.STATE_BYE, self.STATE_ABANDON):
                raise PeerLost(dst, "left with this rank's message unread", int(back.words[3]) == self.STATE_BYE)
            if time.monotonic() > deadline:
                raise PeerLost(dst, "ring stayed full for the time limit")
            time.sleep(0.0002)

    def recv(self, src, timeout=None):
        deadline = time.monotonic() + (timeout if timeout is not None else self.timeout)
        kind, dtype, nbytes, crc = decode_header(self._pull(src, _HEADER.size, deadline))
        return decode_payload(self._pull(src, nbytes, deadline), dtype, crc)

    def close(self, orderly=True):
        if self._stop.is_set():
            return
        self._stop.set()
        for r in self._out.values():
            r.words[3] = np.uint64(self.STATE_BYE if orderly else self.STATE_ABANDON)
        time.sleep(0.05)            # lets the heartbeat thread see the stop before the views go away
        for r in list(self._out.values()) + list(self._in.values()):
            r.close()


# --------------------------------------------------------------------------- torch.distributed
class TorchDistTransport(Transport):
    """Point-to-point over a torch.distributed group (gloo on the host, NCCL for device tensors). A peer that does not
    answer inside the group's timeout surfaces as ``PeerLost`` naming it."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

    def _g(self, r):
        return self.dist.get_global_rank(self.group, r) if self.group is not None else r

    def send(self, dst, values):
        flat = values.detach().contiguous().reshape(-1)
        head = torch.tensor([flat.numel(), _DTYPES.index(flat.dtype)], dtype=torch.int64, device=flat.device)
        try:
            self.dist.send(head, self._g(dst), group=self.group)
            if flat.numel():
                self.dist.send(flat, self._g(dst), group=self.group)
        except RuntimeError as e:
            raise PeerLost(dst, str(e)[:120])

    def recv(self, src, timeout=None, device="cpu"):
        head = torch.zeros(2, dtype=torch.int64, device=device)
        try:
            self.dist.recv(head, self._g(src), group=self.group)
            out = torch.empty(int(head[0]), dtype=_DTYPES[int(head[1])], device=device)
            if out.numel():
                self.dist.recv(out, self._g(src), group=self.group)
        except RuntimeError as e:
            raise PeerLost(src, str(e)[:120])
        return out

    def barrier(self, timeout=None):
        self.dist.barrier(group=self.group)
