"""Network key/value client speaking the Redis serialisation protocol (RESP2) over a TCP socket, with the helper
surface the heuristics use: strings with TTL / NX, counters, lists, hashes, JSON values, tuning choices and pipelines.

Parity: crates/st-kv/src/lib.rs — `redis_get_raw` … `redis_pipeline` (:35-290), the `Choice` helpers (:291-432) and
the connection-holding `RedisKv` (:443-560).  The reference links the `redis` crate; this client needs nothing beyond
the standard library.  `RespKv` has the same methods as the in-process `logic.MemoryKv`, so callers take either;
`connect("redis://host:port/db")` returns a `RespKv`, `connect("memory://name")` the in-process store.

`MiniRespServer` is a small single-process server for the same command subset backed by a `MemoryKv`: the test-suite's
peer, and a stand-in when several local processes (ranks of one box) want to share tuning choices without an external
daemon.
"""
from __future__ import annotations

import json
import socket
import socketserver
import threading
from dataclasses import asdict
from typing import Any, Callable, List, Optional
from urllib.parse import urlparse

from .logic import Choice, KvError, MemoryKv
from .logic import connect as _connect_memory


# ---- wire format ------------------------------------------------------------------------------------------------------
def encode_command(*parts) -> bytes:
    out = [b"*%d\r\n" % len(parts)]
    for p in parts:
        b = p if isinstance(p, bytes) else str(p).encode()
        out.append(b"$%d\r\n%s\r\n" % (len(b), b))
    return b"".join(out)


class _Reader:
    def __init__(self, sock):
        self._f = sock.makefile("rb")

    def _line(self) -> bytes:
        line = self._f.readline()
        if not line.endswith(b"\r\n"):
            raise KvError("connection closed while reading a reply")
        return line[:-2]

    def read(self):
        line = self._line()
        kind, rest = line[:1], line[1:]
        if kind == b"+":
            return rest.decode()
        if kind == b"-":
            raise KvError(rest.decode())
        if kind == b":":
            return int(rest)
        if kind == b"$":
            n = int(rest)
            if n < 0:
                return None
            data = self._f.read(n + 2)
            if len(data) != n + 2:
                raise KvError("connection closed inside a bulk reply")
            return data[:-2].decode()
        if kind == b"*":
            n = int(rest)
            return None if n < 0 else [self.read() for _ in range(n)]
        raise KvError(f"unexpected reply type {kind!r}")

    def close(self) -> None:
        self._f.close()


class RespKv:
    """One connection; every method is a round trip unless issued inside :meth:`pipeline`."""

    def __init__(self, host: str = "127.0.0.1", port: int = 6379, db: int = 0, password: Optional[str] = None,
                 timeout: float = 5.0):
        try:
            self._sock = socket.create_connection((host, port), timeout=timeout)
        except OSError as exc:
            raise KvError(f"cannot connect to {host}:{port}: {exc}") from exc
        self._sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        self._reader = _Reader(self._sock)
        self._lock = threading.RLock()
        self._queue: Optional[list] = None
        if password:
            self._call("AUTH", password)
        if db:
            self._call("SELECT", db)

    @classmethod
    def from_url(cls, url: str, timeout: float = 5.0) -> "RespKv":
        u = urlparse(url)
        if u.scheme != "redis":
            raise KvError(f"not a redis:// URL: {url!r}")
        db = int(u.path.lstrip("/") or 0)
        return cls(u.hostname or "127.0.0.1", u.port or 6379, db, u.password, timeout)

    def close(self) -> None:
        with self._lock:
            try:
                self._reader.close()
                self._sock.close()
            except OSError:
                pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    def _call(self, *parts):
        with self._lock:
            if self._queue is not None:
                self._queue.append(parts)
                return None
            try:
                self._sock.sendall(encode_command(*parts))
                return self._reader.read()
            except OSError as exc:
                raise KvError(f"connection error during {parts[0]}: {exc}") from exc

    # strings ------------------------------------------------------------------------------------------------------
    def get(self, key: str):
        return self._call("GET", key)

    def set(self, key: str, value) -> None:
        self._call("SET", key, value)

    def set_ex(self, key: str, value, seconds: float) -> None:
        self._call("SET", key, value, "PX", max(int(round(seconds * 1000)), 1))

    def set_nx(self, key: str, value) -> bool:
        return self._call("SET", key, value, "NX") is not None

    def getset(self, key: str, value):
        return self._call("GETSET", key, value)

    def delete(self, key: str) -> int:
        return int(self._call("DEL", key) or 0)

    del_ = delete

    def exists(self, key: str) -> bool:
        return bool(self._call("EXISTS", key))

    def expire(self, key: str, seconds: float) -> bool:
        return bool(self._call("PEXPIRE", key, max(int(round(seconds * 1000)), 1)))

    def ttl(self, key: str) -> int:
        """-2 for a missing key, -1 without expiry, else whole seconds left (rounded up)."""
        ms = self._call("PTTL", key)
        return ms if ms is None or ms < 0 else -(-ms // 1000)

    def incr_by(self, key: str, amount):
        if isinstance(amount, int):
            return self._call("INCRBY", key, amount)
        r = self._call("INCRBYFLOAT", key, repr(float(amount)))
        return None if r is None else float(r)

    # lists --------------------------------------------------------------------------------------------------------
    def lpush(self, key: str, *values) -> int:
        return self._call("LPUSH", key, *values)

    def rpush(self, key: str, *values) -> int:
        return self._call("RPUSH", key, *values)

    def lrange(self, key: str, start: int, stop: int) -> list:
        return self._call("LRANGE", key, start, stop) or []

    def ltrim(self, key: str, start: int, stop: int) -> None:
        self._call("LTRIM", key, start, stop)

    # hashes -------------------------------------------------------------------------------------------------------
    def hset(self, key: str, field_name: str, value) -> bool:
        return bool(self._call("HSET", key, field_name, value))

    def hget(self, key: str, field_name: str):
        return self._call("HGET", key, field_name)

    def hdel(self, key: str, field_name: str) -> int:
        return int(self._call("HDEL", key, field_name) or 0)

    def hgetall(self, key: str) -> dict:
        flat = self._call("HGETALL", key) or []
        return dict(zip(flat[0::2], flat[1::2]))

    # JSON ---------------------------------------------------------------------------------------------------------
    def set_json(self, key: str, value, *, ex: Optional[float] = None, nx: bool = False) -> bool:
        parts = ["SET", key, json.dumps(value, sort_keys=True)]
        if ex is not None:
            parts += ["PX", max(int(round(ex * 1000)), 1)]
        if nx:
            parts.append("NX")
        reply = self._call(*parts)
        return True if self._queue is not None else reply is not None

    def get_json(self, key: str):
        raw = self.get(key)
        if raw is None:
            return None
        try:
            return json.loads(raw)
        except (TypeError, ValueError) as exc:
            raise KvError(f"value at {key!r} is not JSON: {exc}") from exc

    def get_or_set_json(self, key: str, default: Callable[[], Any], *, ex: Optional[float] = None):
        """Reads the key; if it is absent, stores ``default()`` with NX and returns whichever value won the race."""
        cur = self.get_json(key)
        if cur is not None:
            return cur
        value = default()
        if self.set_json(key, value, ex=ex, nx=True):
            return value
        cur = self.get_json(key)
        return value if cur is None else cur

    def lpush_json(self, key: str, value) -> int:
        return self.lpush(key, json.dumps(value, sort_keys=True))

    def rpush_json(self, key: str, value) -> int:
        return self.rpush(key, json.dumps(value, sort_keys=True))

    def lrange_json(self, key: str, start: int, stop: int) -> list:
        return [json.loads(v) for v in self.lrange(key, start, stop)]

    # tuning choices ---------------------------------------------------------------------------------------------------
    def set_choice(self, key: str, choice: Choice, *, ex: Optional[float] = None, nx: bool = False) -> bool:
        return self.set_json(key, asdict(choice), ex=ex, nx=nx)

    def get_choice(self, key: str) -> Optional[Choice]:
        d = self.get_json(key)
        return None if d is None else Choice(**d)

    def get_or_set_choice(self, key: str, default: Callable[[], Choice]) -> Choice:
        return Choice(**self.get_or_set_json(key, lambda: asdict(default())))

    def push_choice(self, key: str, choice: Choice, *, left: bool = True, keep: Optional[int] = None) -> int:
        n = (self.lpush_json if left else self.rpush_json)(key, asdict(choice))
        if keep is not None:
            self.ltrim(key, 0, keep - 1) if left else self.ltrim(key, -keep, -1)
            n = min(n, keep)
        return n

    def lrange_choice(self, key: str, start: int, stop: int) -> List[Choice]:
        return [Choice(**d) for d in self.lrange_json(key, start, stop)]

    # pipeline -----------------------------------------------------------------------------------------------------
    def pipeline(self, build: Callable[["RespKv"], Any]) -> list:
        """Queues every command ``build`` issues, sends them as one MULTI / EXEC transaction in a single write and
        returns the list of their replies (the calls themselves return ``None`` while queued)."""
        with self._lock:
            if self._queue is not None:
                raise KvError("pipelines do not nest")
            self._queue = []
            try:
                build(self)
                queued = self._queue
            finally:
                self._queue = None
            if not queued:
                return []
            payload = encode_command("MULTI") + b"".join(encode_command(*c) for c in queued) + encode_command("EXEC")
            try:
                self._sock.sendall(payload)
                self._reader.read()                      # +OK for MULTI
                for _ in queued:
                    self._reader.read()                  # +QUEUED for each
                return self._reader.read() or []
            except OSError as exc:
                raise KvError(f"connection error during a pipeline: {exc}") from exc


def connect(url: str = "memory://default"):
    """``memory://<name>``: the process-wide in-process store; ``redis://host:port/db``: a network client."""
    if url.startswith("redis://"):
        return RespKv.from_url(url)
    return _connect_memory(url)


# ---- loopback server --------------------------------------------------------------------------------------------------
class _Handler(socketserver.StreamRequestHandler):
    def handle(self):
        store: MemoryKv = self.server.store          # type: ignore[attr-defined]
        reader = _Reader(self.connection)
        queued: Optional[list] = None
        while True:
            try:
                cmd = reader.read()
            except (KvError, ValueError, OSError):
                return
            if not cmd:
                return
            name = str(cmd[0]).upper()
            if name == "MULTI":
                queued = []
                self.wfile.write(b"+OK\r\n")
            elif name == "EXEC":
                replies = [self._run(store, c) for c in (queued or [])]
                queued = None
                self.wfile.write(b"*%d\r\n" % len(replies) + b"".join(replies))
            elif queued is not None:
                queued.append(cmd)
                self.wfile.write(b"+QUEUED\r\n")
            else:
                self.wfile.write(self._run(store, cmd))
            self.wfile.flush()

    @staticmethod
    def _enc(v) -> bytes:
        if v is None:
            return b"$-1\r\n"
        if isinstance(v, bool):
            return b":%d\r\n" % int(v)
        if isinstance(v, int):
            return b":%d\r\n" % v
        if isinstance(v, (list, tuple)):
            return b"*%d\r\n" % len(v) + b"".join(_Handler._enc(x) for x in v)
        if isinstance(v, _Status):
            return b"+" + v.text.encode() + b"\r\n"
        b = (repr(v) if isinstance(v, float) else str(v)).encode()
        return b"$%d\r\n%s\r\n" % (len(b), b)

    def _run(self, s: MemoryKv, cmd: list) -> bytes:
        name, a = str(cmd[0]).upper(), cmd[1:]
        try:
            return self._enc(self._dispatch(s, name, a))
        except KvError as exc:
            return b"-ERR " + str(exc).encode() + b"\r\n"
        except (IndexError, ValueError) as exc:
            return b"-ERR wrong arguments for '" + name.encode() + b"': " + str(exc).encode() + b"\r\n"

    @staticmethod
    def _dispatch(s: MemoryKv, name: str, a: list):
        ok = _Status("OK")
        if name in ("PING",):
            return _Status("PONG")
        if name in ("AUTH", "SELECT"):
            return ok
        if name == "GET":
            v = s.get(a[0])
            if isinstance(v, (list, dict)):
                raise KvError("WRONGTYPE Operation against a key holding the wrong kind of value")
            return v
        if name == "SET":
            opts = [str(x).upper() for x in a[2:]]
            nx = "NX" in opts
            px = int(a[2 + opts.index("PX") + 1]) / 1000.0 if "PX" in opts else (float(a[2 + opts.index("EX") + 1]) if "EX" in opts else None)
            with s._lock:
                if nx and s.exists(a[0]):
                    return None
                s.set_ex(a[0], a[1], px) if px is not None else s.set(a[0], a[1])
            return ok
        if name == "GETSET":
            return s.getset(a[0], a[1])
        if name == "DEL":
            return sum(s.delete(k) for k in a)
        if name == "EXISTS":
            return sum(int(s.exists(k)) for k in a)
        if name in ("EXPIRE", "PEXPIRE"):
            return int(s.expire(a[0], float(a[1]) / (1000.0 if name == "PEXPIRE" else 1.0)))
        if name in ("TTL", "PTTL"):
            with s._lock:
                if not s.exists(a[0]):
                    return -2
                t = s._exp.get(a[0])
                if t is None:
                    return -1
                left = max(t - s._clock(), 0.0)
                return int(round(left * 1000)) if name == "PTTL" else int(-(-left // 1))
        if name in ("INCRBY", "INCRBYFLOAT"):
            with s._lock:
                cur = s.get(a[0])
                try:
                    base = 0 if cur is None else (int(cur) if name == "INCRBY" else float(cur))
                    new = base + (int(a[1]) if name == "INCRBY" else float(a[1]))
                except (TypeError, ValueError):
                    raise KvError("value is not an integer or out of range") from None
                s._d[a[0]] = str(new) if name == "INCRBY" else repr(new)
                return new if name == "INCRBY" else repr(new)
        if name == "LPUSH":
            return s.lpush(a[0], *a[1:])
        if name == "RPUSH":
            return s.rpush(a[0], *a[1:])
        if name == "LRANGE":
            return s.lrange(a[0], int(a[1]), int(a[2]))
        if name == "LTRIM":
            s.ltrim(a[0], int(a[1]), int(a[2]))
            return ok
        if name == "HSET":
            return int(s.hset(a[0], a[1], a[2]))
        if name == "HGET":
            return s.hget(a[0], a[1])
        if name == "HDEL":
            return s.hdel(a[0], a[1])
        if name == "HGETALL":
            return [x for kv in s.hgetall(a[0]).items() for x in kv]
        raise KvError(f"unknown command '{name}'")


class _Status:
    def __init__(self, text: str):
        self.text = text


class _Server(socketserver.ThreadingMixIn, socketserver.TCPServer):
    allow_reuse_address = True
    daemon_threads = True


class MiniRespServer:
    """``with MiniRespServer() as srv: kv = connect(srv.url)`` — serves on 127.0.0.1 and a free port."""

    def __init__(self, store: Optional[MemoryKv] = None, host: str = "127.0.0.1", port: int = 0):
        self.store = store or MemoryKv()
        self._server = _Server((host, port), _Handler)
        self._server.store = self.store              # type: ignore[attr-defined]
        self.host, self.port = self._server.server_address[:2]
        self._thread = threading.Thread(target=self._server.serve_forever, kwargs={"poll_interval": 0.05}, daemon=True)

    @property
    def url(self) -> str:
        return f"redis://{self.host}:{self.port}/0"

    def start(self) -> "MiniRespServer":
        self._thread.start()
        return self

    def stop(self) -> None:
        self._server.shutdown()
        self._server.server_close()
        self._thread.join(timeout=2.0)

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
        return False
