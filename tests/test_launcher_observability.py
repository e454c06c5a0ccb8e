"""tprun restart-on-failure with a flaky worker, ChildFailedError, watchdog and flight recorder
(host-side fault injection only, as in the reference's test_distributed_elastic.py:208-219)."""
import json
import os
import sys
import textwrap
import time

import pytest

from tensorplay_b200.distributed import flight_recorder as fr
from tensorplay_b200.distributed.run import ChildFailedError, LaunchConfig, elastic_launch
from tensorplay_b200.distributed.watchdog import PeerHeartbeat, Watchdog, WatchdogTimeout


def _script(tmp_path, body):
    p = tmp_path / "worker.py"
    p.write_text(textwrap.dedent(body))
    return str(p)


def test_tprun_restarts_flaky_worker(tmp_path):
    marker = tmp_path / "done"
    s = _script(tmp_path, f"""
        import os, sys
        rank = int(os.environ["RANK"]); attempt = int(os.environ["TP_RESTART_COUNT"])
        assert os.environ["WORLD_SIZE"] == "2" and "MASTER_PORT" in os.environ
        if attempt == 0 and rank == 1:
            sys.exit(3)          # first generation: rank 1 fails
        open(r"{marker}" + str(rank), "w").write(str(attempt))
    """)
    rc = elastic_launch(LaunchConfig(nproc_per_node=2, max_restarts=2, log_dir=str(tmp_path / "logs")),
                        [sys.executable, s])
    assert rc == 0
    assert (tmp_path / "done0").read_text() == "1" and (tmp_path / "done1").read_text() == "1"
    assert os.path.exists(tmp_path / "logs" / "attempt0_rank1.log")


def test_tprun_raises_when_restarts_exhausted(tmp_path):
    s = _script(tmp_path, "import sys; sys.exit(5)")
    with pytest.raises(ChildFailedError) as ei:
        elastic_launch(LaunchConfig(nproc_per_node=2, max_restarts=1), [sys.executable, s])
    assert 5 in ei.value.failures.values()


def test_watchdog_trips_and_raises():
    wd = Watchdog(cpu_timeout=0.15, action="raise", poll_interval=0.02)
    try:
        wd.heartbeat()
        time.sleep(0.4)
        with pytest.raises(WatchdogTimeout):
            wd.heartbeat()
        wd.heartbeat()  # recovered
    finally:
        wd.close()


def test_peer_heartbeat_detects_silent_rank():
    from tensorplay_b200.distributed.store import HashStore
    st = HashStore()
    a, b = PeerHeartbeat(st, 0, 2, timeout=0.1), PeerHeartbeat(st, 1, 2, timeout=0.1)
    a.beat(); b.beat()
    assert a.missing() == []
    time.sleep(0.25)
    a.beat()
    assert a.missing() == [1]   # rank 1 stopped beating
    b.beat()
    assert a.missing() == []


def test_flight_recorder_dump_and_analyze(tmp_path):
    paths = []
    for rank, ops in enumerate([["all_gather", "reduce_scatter", "all_gather"], ["all_gather", "all_reduce"]]):
        fr.clear()
        for o in ops:
            fr.record(o, numel=8, group="dp")
        paths.append(fr.dump(str(tmp_path / f"fr{rank}.json"), rank=rank))
    rep = fr.analyze(paths)
    assert rep["mismatch"]["index"] == 1 and rep["behind"] == [1]
    assert json.load(open(paths[0]))["entries"][0]["op"] == "all_gather"


def test_debug_server_and_package_surface():
    import json
    import urllib.request

    import tensorplay_b200 as tp
    d = tp.distributed
    # own sub-packages win over torch's modules of the same name
    assert d.algorithms.__name__.startswith("tensorplay_b200") and d.optim.__name__.startswith("tensorplay_b200")
    assert d.elastic.LocalElasticAgent is d.launcher.LocalElasticAgent
    port = d.debug.start_debug_server(0)
    try:
        root = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/", timeout=5).read())
        assert "/stacks" in root["endpoints"]
        stacks = urllib.request.urlopen(f"http://127.0.0.1:{port}/stacks", timeout=5).read().decode()
        assert "MainThread" in stacks and "test_debug_server_and_package_surface" in stacks
        json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/flight", timeout=5).read())
    finally:
        d.debug.stop_debug_server()


def test_debug_handler_registry_and_flight_recorder_object(tmp_path):
    import json
    import urllib.request

    from tensorplay_b200.distributed import debug, flight_recorder as fr
    assert {"/stacks", "/native", "/flight", "/store"} <= set(debug.list_handlers())

    class Hello(debug.DebugHandler):
        path = "/hello"

        def handle(self, request_path):
            return "hi " + request_path

    debug.register_handler(Hello())
    port = debug.start_debug_server(0)
    try:
        assert urllib.request.urlopen(f"http://127.0.0.1:{port}/hello?x=1").read().decode() == "hi /hello?x=1"
        idx = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/").read())
        assert "/hello" in idx["endpoints"]
        rec = fr.start_flight_recorder(str(tmp_path / "fr.json"), size=4)
        fr.clear()
        for i in range(6):
            rec.record("all_reduce", numel=i)
        assert [e["numel"] for e in rec.entries()] == [2, 3, 4, 5]            # ring of four
        flight = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/flight").read())
        assert len(flight["entries"]) == 4
        try:
            with rec:
                raise ValueError("boom")
        except ValueError:
            pass
        assert json.load(open(tmp_path / "fr.json"))["entries"][-1]["numel"] == 5
        assert fr.dump_flight_recorder(str(tmp_path / "fr2.json")).endswith("fr2.json")
    finally:
        debug.stop_debug_server()
        fr.start_flight_recorder(size=2048)


def test_private_module_paths_and_rpc_probe():
    import importlib
    import tensorplay_b200.distributed as dist
    assert importlib.import_module("tensorplay_b200.distributed._watchdog").Watchdog is dist.watchdog.Watchdog
    assert importlib.import_module("tensorplay_b200.distributed.distributed_core") is dist
    assert importlib.import_module("tensorplay_b200.distributed._store").TCPStore is dist.TCPStore
    for n in ("_mesh_layout", "_pycute", "config", "_tensor"):
        assert importlib.import_module("tensorplay_b200.distributed." + n) is not None
    assert not hasattr(dist.rpc, "init_rpc") and not dist.autograd.is_available()


def test_tprun_interrupted_launcher_takes_its_workers_down(tmp_path):
    """SIGTERM to the launcher: the ranks (sessions of their own) are signalled and gone afterwards."""
    import signal
    import subprocess
    s = _script(tmp_path, f"""
        import os, time
        open(r"{tmp_path}/pid" + os.environ["RANK"], "w").write(str(os.getpid()))
        time.sleep(120)
    """)
    launcher = subprocess.Popen([sys.executable, "-m", "tensorplay_b200.distributed.run", "--nproc-per-node", "2", s],
                                cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    deadline = time.time() + 60
    while time.time() < deadline and not all((tmp_path / f"pid{r}").exists() for r in range(2)):
        time.sleep(0.1)
    time.sleep(0.2)
    pids = [int((tmp_path / f"pid{r}").read_text()) for r in range(2)]
    launcher.send_signal(signal.SIGTERM)
    launcher.wait(timeout=30)

    def alive(pid):
        try:
            os.kill(pid, 0)
        except ProcessLookupError:
            return False
        # a zombie of another parent counts as gone
        try:
            return open(f"/proc/{pid}/stat").read().split(")")[1].split()[0] != "Z"
        except OSError:
            return False

    deadline = time.time() + 15
    while time.time() < deadline and any(alive(p) for p in pids):
        time.sleep(0.1)
    assert not any(alive(p) for p in pids)


def test_tprun_namespace_form_and_tee(tmp_path, capfd):
    from tensorplay_b200.distributed import run as tprun
    s = _script(tmp_path, "import os; print('hello from', os.environ['RANK'], flush=True)")
    ns = tprun.get_args_parser().parse_args(["--nproc-per-node", "2", "--log-dir", str(tmp_path / "lg"), "--tee", s])
    assert tprun.run(ns) == 0
    out = capfd.readouterr().out
    assert "[rank0] hello from 0" in out and "[rank1] hello from 1" in out
    assert "hello from 1" in (tmp_path / "lg" / "attempt0_rank1.log").read_text()
