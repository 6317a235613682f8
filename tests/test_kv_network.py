"""Network key/value client against the loopback RESP server: the same helper surface as the in-process store
(behaviour of crates/st-kv/src/lib.rs), the wire encoding, pipelines as one transaction, errors and expiry."""
import time

import pytest

from spiraltorch_b200 import kv
from spiraltorch_b200.logic import Choice, KvError, MemoryKv


def test_wire_encoding():
    assert kv.encode_command("SET", "k", 1) == b"*3\r\n$3\r\nSET\r\n$1\r\nk\r\n$1\r\n1\r\n"
    assert kv.encode_command("GET", b"\xff") == b"*2\r\n$3\r\nGET\r\n$1\r\n\xff\r\n"


def test_client_round_trips_against_loopback_server():
    with kv.MiniRespServer() as srv, kv.connect(srv.url) as c:
        assert isinstance(c, kv.RespKv) and c.get("missing") is None
        c.set("a", "1")
        assert c.get("a") == "1" and c.exists("a") and not c.exists("b")
        assert c.set_nx("a", "2") is False and c.set_nx("b", "2") is True and c.getset("b", "3") == "2"
        assert c.incr_by("n", 5) == 5 and c.incr_by("n", -2) == 3 and c.incr_by("f", 0.5) == 0.5
        assert c.ttl("a") == -1 and c.ttl("missing") == -2
        c.set_ex("t", "x", 30.0)
        assert 29 <= c.ttl("t") <= 30 and c.expire("a", 10.0) and 9 <= c.ttl("a") <= 10 and not c.expire("missing", 1.0)
        assert c.delete("a") == 1 and c.delete("a") == 0
        assert c.rpush("l", "x", "y") == 2 and c.lpush("l", "w") == 3 and c.lrange("l", 0, -1) == ["w", "x", "y"]
        c.ltrim("l", 1, -1)
        assert c.lrange("l", 0, -1) == ["x", "y"] and c.lrange("none", 0, -1) == []
        assert c.hset("h", "f", "1") is True and c.hset("h", "f", "2") is False and c.hget("h", "f") == "2"
        assert c.hgetall("h") == {"f": "2"} and c.hdel("h", "f") == 1 and c.hget("h", "f") is None
        with pytest.raises(KvError):
            c.get("l")                                                # wrong type travels back as an error reply
        with pytest.raises(KvError):
            c._call("NOSUCH")
        assert c.get("b") == "3"                                      # the connection stays usable after errors


def test_json_choices_and_pipeline():
    store = MemoryKv()
    with kv.MiniRespServer(store) as srv, kv.RespKv.from_url(srv.url) as c:
        assert c.set_json("j", {"b": 2, "a": [1, 2]}) and c.get_json("j") == {"a": [1, 2], "b": 2}
        assert c.set_json("j", {"x": 1}, nx=True) is False
        calls = []
        assert c.get_or_set_json("d", lambda: calls.append(1) or {"v": 7}) == {"v": 7}
        assert c.get_or_set_json("d", lambda: calls.append(1) or {"v": 8}) == {"v": 7} and len(calls) == 1
        c.set("bad", "{not json")
        with pytest.raises(KvError):
            c.get_json("bad")
        ch = Choice(use_2ce=True, wg=128, kl=16, ch=4096)
        assert c.set_choice("tune", ch) and c.get_choice("tune") == ch and c.get_choice("nope") is None
        assert c.get_or_set_choice("tune2", lambda: ch) == ch
        for i in range(5):
            n = c.push_choice("hist", Choice(wg=32 * (i + 1)), keep=3)
        assert n == 3 and [x.wg for x in c.lrange_choice("hist", 0, -1)] == [160, 128, 96]
        replies = c.pipeline(lambda p: (p.set("p1", "a"), p.incr_by("cnt", 2), p.rpush("pl", "z"), p.get("p1")))
        assert replies == ["OK", 2, 1, "a"] and c.get("p1") == "a" and c.pipeline(lambda p: None) == []
        with pytest.raises(KvError):
            c.pipeline(lambda p: p.pipeline(lambda q: None))
        assert store.get("p1") == "a"                                  # the server's store is the one handed in
        # two clients see each other's writes (the point of a shared store)
        with kv.connect(srv.url) as other:
            other.set("shared", "yes")
            assert c.get("shared") == "yes"


def test_expiry_and_connection_errors():
    with kv.MiniRespServer() as srv, kv.connect(srv.url) as c:
        c.set_json("e", {"v": 1}, ex=0.05)
        assert c.get_json("e") == {"v": 1}
        time.sleep(0.12)
        assert c.get_json("e") is None and c.ttl("e") == -2
        port = srv.port
    with pytest.raises(KvError):
        kv.RespKv("127.0.0.1", port, timeout=0.5)                      # nothing listens there any more
    with pytest.raises(KvError):
        kv.RespKv.from_url("http://127.0.0.1:1")
    assert isinstance(kv.connect("memory://kv-test"), MemoryKv)
