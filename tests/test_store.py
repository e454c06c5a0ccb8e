import threading
import time

import pytest

from tensorplay_b200.distributed.store import (FileStore, HashStore, PrefixStore, StoreTimeoutError,
                                                TCPStore)


def _exercise(make_client):
    a, b = make_client(), make_client()
    a.set("k", b"v1")
    assert b.get("k") == b"v1"
    assert a.add("ctr", 3) == 3 and b.add("ctr", 4) == 7
    assert a.compare_set("cas", b"", b"first") == b"first"
    assert b.compare_set("cas", b"nope", b"x") == b"first"
    assert b.compare_set("cas", b"first", b"second") == b"second"
    assert a.check(["k", "cas"]) and not a.check(["missing"])
    assert a.has("k")
    t0 = time.time()
    with pytest.raises(StoreTimeoutError):
        a.get("missing", timeout=0.2)
    assert time.time() - t0 < 5

    def later():
        time.sleep(0.1)
        b.set("late", b"x")
    th = threading.Thread(target=later)
    th.start()
    a.wait(["late"], timeout=5)
    th.join()
    assert a.delete_key("late") and not a.check(["late"])
    p = PrefixStore("ns", a)
    p.set("k", b"inner")
    assert p.get("k") == b"inner" and a.get("k") == b"v1" and a.get("ns/k") == b"inner"


def test_tcp_store_native():
    master = TCPStore("127.0.0.1", 0, is_master=True, timeout=10)
    try:
        _exercise(lambda: TCPStore("127.0.0.1", master.port, timeout=10))
        assert master.num_keys() >= 3
    finally:
        master.close()


def test_hash_store():
    hs = HashStore(timeout=5)
    _exercise(lambda: hs)


def test_file_store(tmp_path):
    path = tmp_path / "store.json"
    _exercise(lambda: FileStore(str(path), timeout=5))


def test_tcp_store_backs_process_group():
    import torch
    import torch.distributed as dist
    master = TCPStore("127.0.0.1", 0, is_master=True, timeout=20)
    try:
        dist.init_process_group("gloo", store=master, rank=0, world_size=1)
        t = torch.ones(3)
        dist.all_reduce(t)
        assert t.sum() == 3
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()
        master.close()


def test_native_store_server_rejects_malformed_requests():
    """A request whose key count does not fit its operation gets an error reply (the connection
    stays usable); a request that announces an oversized value is dropped without growing a buffer."""
    import socket
    import struct

    from tensorplay_b200.distributed.store import TCPStore
    srv = TCPStore("127.0.0.1", 0, is_master=True, timeout=5)
    try:
        def req(sock, op, keys, v1=b"", v2=b"", arg=0):
            msg = struct.pack("<BI", op, len(keys))
            for k in keys:
                msg += struct.pack("<I", len(k)) + k
            msg += struct.pack("<Q", len(v1)) + v1 + struct.pack("<Q", len(v2)) + v2 + struct.pack("<q", arg)
            sock.sendall(msg)
            hdr = b""
            while len(hdr) < 12:
                chunk = sock.recv(12 - len(hdr))
                if not chunk:
                    return None
                hdr += chunk
            status, n = struct.unpack("<iQ", hdr)
            body = b""
            while len(body) < n:
                body += sock.recv(n - len(body))
            return status, body

        with socket.create_connection(("127.0.0.1", srv.port), timeout=5) as c:
            assert req(c, 1, [])[0] == 3            # SET without a key: error, not a crash
            assert req(c, 2, [b"a", b"b"])[0] == 3  # GET with two keys
            assert req(c, 7, [])[0] == 3            # CHECK needs at least one key
            assert req(c, 1, [b"k"], b"v")[0] == 0  # the connection still serves good requests
            assert req(c, 2, [b"k"], arg=1000) == (0, b"v")
        with socket.create_connection(("127.0.0.1", srv.port), timeout=5) as c:
            # announce a 1 TiB value: the server closes the connection instead of allocating
            c.sendall(struct.pack("<BI", 1, 1) + struct.pack("<I", 1) + b"k" + struct.pack("<Q", 1 << 40))
            assert c.recv(16) == b""
        srv.set("still", "alive")
        assert srv.get("still") in (b"alive", "alive")
    finally:
        srv.close()
