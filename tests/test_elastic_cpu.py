"""Elastic components on the host: the dynamic rendezvous (joins, late comers, fencing of stale
writers, eviction of silent nodes, closing), the file-based watchdog timers and the agent's
health-check endpoint. Failures are made on the host only (a node that stops its keep-alive, a
worker that overstays its timer)."""
import json
import subprocess
import sys
import threading
import time
import urllib.error
import urllib.request

import pytest

from tensorplay_b200.distributed.elastic.agent.server import HealthCheckServer
from tensorplay_b200.distributed.elastic.rendezvous import (DynamicRendezvousHandler, RendezvousClosedError,
                                                            RendezvousSettings, RendezvousTimeoutError)
from tensorplay_b200.distributed.elastic.timer import FileTimerClient, FileTimerServer, expires
from tensorplay_b200.distributed.store import HashStore


def _join_all(handlers):
    out = [None] * len(handlers)

    def run(i):
        out[i] = handlers[i].next_rendezvous()

    ts = [threading.Thread(target=run, args=(i,)) for i in range(len(handlers))]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=30)
    return out


def test_dynamic_rendezvous_rounds_wait_list_and_eviction():
    store = HashStore()
    s = RendezvousSettings("job", min_nodes=2, max_nodes=3, last_call_s=0.2, join_timeout_s=10, keep_alive_s=0.05,
                           keep_alive_max_attempts=4)
    hs = [DynamicRendezvousHandler(store, s, node_name=f"node{i}") for i in range(3)]
    res = _join_all(hs)
    assert sorted(r[1] for r in res) == [0, 1, 2] and all(r[2] == 3 for r in res)
    # the round's store is shared by its members and separate from the state record
    res[0][0].set("k", "v")
    assert res[2][0].get("k") == b"v"
    # a fourth node arrives while the round runs: it waits, the members see it
    late = DynamicRendezvousHandler(store, RendezvousSettings("job", 2, 3, join_timeout_s=0.5, keep_alive_s=0.05), "node9")
    with pytest.raises(RendezvousTimeoutError):
        late.next_rendezvous()
    # (it left the wait list when it gave up)
    assert hs[0].num_nodes_waiting() == 0
    # node2 falls silent: after its keep-alive expires the round is void and the survivors form a new one
    hs[2]._stop.set()
    time.sleep(0.5)
    res2 = _join_all(hs[:2])
    assert sorted(r[1] for r in res2) == [0, 1] and all(r[2] == 2 for r in res2)
    state = json.loads(store.get("rdzv/job/state"))
    assert "node2" not in state["participants"] and state["round"] >= 1
    # closing: nobody joins any more
    hs[0].set_closed()
    assert hs[1].is_closed()
    with pytest.raises(RendezvousClosedError):
        DynamicRendezvousHandler(store, s, "node7").next_rendezvous()
    for h in hs:
        h.shutdown()


def test_rendezvous_state_updates_are_fenced():
    """Two writers race on the record: the compare-and-set lets exactly one through per version, the
    loser re-reads and re-applies, so no update is lost."""
    store = HashStore()
    s = RendezvousSettings("race", 1, 64)
    hs = [DynamicRendezvousHandler(store, s, f"n{i}") for i in range(8)]

    def bump(h):
        for _ in range(50):
            def fn(state):
                state.setdefault("counter", 0)
                state["counter"] += 1
                return state
            h._update(fn)

    ts = [threading.Thread(target=bump, args=(h,)) for h in hs]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert json.loads(store.get("rdzv/race/state"))["counter"] == 400


def test_file_timer_reaps_a_worker_that_overstays(tmp_path):
    path = str(tmp_path / "timers")
    server = FileTimerServer(path, max_interval=0.05)
    server.start()
    try:
        code = (f"import sys, time; sys.path.insert(0, {sys.path[0]!r});\n"
                "from tensorplay_b200.distributed.elastic.timer import FileTimerClient, configure, expires\n"
                f"configure(FileTimerClient({path!r}))\n"
                "with expires(after=30): pass\n"          # released in time: nothing happens
                "print('first done', flush=True)\n"
                "with expires(after=0.2): time.sleep(60)\n")
        child = subprocess.Popen([sys.executable, "-c", code], stdout=subprocess.PIPE, cwd=sys.path[0] or ".")
        assert child.stdout.readline().strip() == b"first done"
        rc = child.wait(timeout=20)
        assert rc == -9 and server.expired and server.expired[0][0] == child.pid
        # in-process: a timer that is released never fires
        with expires(after=0.1, client=FileTimerClient(path)):
            pass
        time.sleep(0.3)
        assert len(server.expired) == 1
    finally:
        server.stop()


def test_health_check_server_reports_a_wedged_agent():
    last = {"t": time.time()}
    srv = HealthCheckServer(lambda: last["t"], port=0, timeout=0.3)
    srv.start()
    try:
        with urllib.request.urlopen(f"http://127.0.0.1:{srv.port}/healthz", timeout=5) as r:
            assert r.status == 200 and json.loads(r.read())["healthy"] is True
        time.sleep(0.5)   # the agent's loop stopped reporting
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(f"http://127.0.0.1:{srv.port}/", timeout=5)
        assert e.value.code == 503
        last["t"] = time.time()
        with urllib.request.urlopen(f"http://127.0.0.1:{srv.port}/", timeout=5) as r:
            assert r.status == 200
    finally:
        srv.stop()
