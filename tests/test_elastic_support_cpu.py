"""Elastic support modules: events, metric streams, process contexts with error files / redirects / tee, store
helpers, and the launcher reporting a failed rank's exception."""
import io
import json
import os
import sys
import threading

import pytest

from tensorplay_b200.distributed.elastic import events, metrics, multiprocessing as emp, utils
from tensorplay_b200.distributed.store import HashStore


def test_events_round_trip_and_destinations(tmp_path, monkeypatch):
    e = events.Event("worker_start", events.EventSource.WORKER, metadata={"rank": 3, "ok": True})
    back = events.Event.deserialize(e.serialize())
    assert back == e and back.source is events.EventSource.WORKER and back.timestamp > 0
    path = tmp_path / "events.jsonl"
    monkeypatch.setenv("TPB_EVENTS_FILE", str(path))
    events.register_destination("file", events._destinations["file"])   # drop a logger cached without the path
    events.record(e, "file")
    events.record(e)                                                      # "null": dropped
    monkeypatch.setenv("TPB_RDZV_EVENTS_DESTINATION", "file")
    try:
        raise RuntimeError("boom")
    except RuntimeError:
        events.construct_and_record_rdzv_event("job7", "join failed", events.NodeState.FAILED, rank=1)
    for h in events._logger("file").handlers:
        h.flush()
    lines = [json.loads(x) for x in path.read_text().splitlines()]
    assert lines[0]["name"] == "worker_start" and lines[0]["metadata"]["rank"] == 3
    rd = events.RdzvEvent.deserialize(json.dumps(lines[1]))
    assert rd.run_id == "job7" and rd.node_state is events.NodeState.FAILED and "boom" in rd.error_trace
    assert rd.name == "test_events_round_trip_and_destinations" and rd.pid == os.getpid()


def test_metric_streams_and_prof():
    class Keep(metrics.MetricHandler):
        def __init__(self):
            self.seen = []

        def emit(self, m):
            self.seen.append((m.group_name, m.name, m.value))

    default, agent = Keep(), Keep()
    metrics.configure(default)
    metrics.configure(agent, group="agent")
    metrics.put_metric("restarts", 2, "agent")
    metrics.put_metric("loss", 0.5)

    class Worker:
        @metrics.prof(group="agent")
        def step(self, fail):
            if fail:
                raise ValueError("x")
            return 7

    assert Worker().step(False) == 7
    with pytest.raises(ValueError):
        Worker().step(True)
    names = [n for _, n, _ in agent.seen]
    assert names == ["restarts", "worker.step.success", "worker.step.duration.ms", "worker.step.failure",
                     "worker.step.duration.ms"]
    assert default.seen == [("tensorplay_elastic", "loss", 0.5)]
    metrics.configure(metrics.NullMetricHandler())


def _square(x, fail_rank):
    import os
    print(f"hello from {os.environ['LOCAL_RANK']}", flush=True)
    if int(os.environ["LOCAL_RANK"]) == fail_rank:
        raise ValueError(f"rank {fail_rank} gives up")
    return x * x


def test_function_workers_return_values_redirects_and_error_files(tmp_path):
    args = {r: (r + 2, -1) for r in range(3)}
    envs = {r: {"LOCAL_RANK": r} for r in range(3)}
    ctx = emp.start_processes("sq", _square, args, envs, logs_dir=str(tmp_path / "ok"), redirects=emp.Std.OUT)
    res = ctx.wait(timeout=120)
    assert res is not None and not res.is_failed() and res.return_values == {0: 4, 1: 9, 2: 16}
    assert open(res.stdouts[1]).read().strip() == "hello from 1"
    assert set(ctx.pids()) == {0, 1, 2}
    # one rank raises: its exception and traceback come back through the error file, the others are ended
    ctx = emp.start_processes("sq", _square, {r: (r, 1) for r in range(2)}, {r: {"LOCAL_RANK": r} for r in range(2)},
                              logs_dir=str(tmp_path / "bad"))
    res = ctx.wait(timeout=120)
    assert res.is_failed() and set(res.failures) == {1}
    f = res.failures[1]
    assert f.exitcode == 1 and "rank 1 gives up" in f.message and "_square" in f.traceback()
    err = emp.ChildFailedError("sq", res.failures)
    assert err.get_first_failure()[0] == 1 and "rank 1 gives up" in str(err) and "traceback:" in str(err)


def test_program_workers_tee_and_signal_failure(tmp_path):
    out = io.StringIO()
    prog = "import os,sys; print('tick', os.environ['LOCAL_RANK'], sys.argv[1], flush=True)"
    ctx = emp.SubprocessContext("w", sys.executable, {0: ("-c", prog, "a"), 1: ("-c", prog, "b")},
                                {0: {"LOCAL_RANK": 0}, 1: {"LOCAL_RANK": 1}}, str(tmp_path), emp.Std.NONE, emp.Std.OUT)
    ctx._tails[0].dst = out
    ctx.start()
    res = ctx.wait(timeout=60)
    assert res is not None and not res.is_failed()
    text = out.getvalue()
    assert "[w0]:tick 0 a" in text and "[w1]:tick 1 b" in text
    # a worker that ends on a signal: negative exit code, the signal is named
    ctx = emp.start_processes("k", sys.executable, {0: ("-c", "import os,signal; os.kill(os.getpid(), signal.SIGKILL)")},
                              {0: {}}, logs_dir=str(tmp_path / "k"))
    res = ctx.wait(timeout=60)
    assert res.failures[0].exitcode == -9 and res.failures[0].signal_name() == "SIGKILL"
    assert emp.Std.from_str("3") == emp.Std.ALL and emp.Std.from_str("0:3,1:0") == {0: emp.Std.ALL, 1: emp.Std.NONE}
    with pytest.raises(ValueError):
        emp.Std.from_str("x")


def test_store_helpers():
    store, world = HashStore(), 3
    got = {}

    def rank_fn(r):
        got[r] = utils.synchronize(store, f"blob{r}".encode(), r, world, "sync/", timeout=30)
        utils.barrier(store, world, "bar", barrier_timeout=30, rank=r)

    ts = [threading.Thread(target=rank_fn, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert all(got[r] == [b"blob0", b"blob1", b"blob2"] for r in range(world))
    # a rank that never arrives is named by rank 0
    with pytest.raises(Exception, match="did not arrive: 1"):
        utils.barrier(store, 2, "late", barrier_timeout=0.3, rank=0)
    assert utils.macros.substitute(["--r=${local_rank}", 5], "2") == ["--r=2", 5]
    with pytest.raises(ValueError):
        utils.get_env_variable_or_raise("TPB_SURELY_NOT_SET")
    assert 0 < utils.get_free_port() < 65536


def test_launcher_reports_the_failing_ranks_exception(tmp_path):
    from tensorplay_b200.distributed.run import ChildFailedError, LaunchConfig, elastic_launch
    script = tmp_path / "w.py"
    script.write_text(
        "import os\n"
        "from tensorplay_b200.distributed.elastic.multiprocessing import record\n"
        "@record\n"
        "def main():\n"
        "    if os.environ['RANK'] == '1':\n"
        "        raise KeyError('missing shard 17')\n"
        "    import time; time.sleep(30)\n"
        "main()\n")
    env = {"PYTHONPATH": os.pathsep.join([os.getcwd()] + sys.path)}
    with pytest.raises(ChildFailedError) as ei:
        elastic_launch(LaunchConfig(nproc_per_node=2, log_dir=str(tmp_path / "logs"), env=env), [sys.executable, str(script)])
    assert ei.value.failures == {1: 1}
    assert "missing shard 17" in str(ei.value) and "KeyError" in str(ei.value) and "in main" in str(ei.value)


def test_rendezvous_helpers_backend_and_registry():
    from datetime import timedelta
    from tensorplay_b200.distributed.elastic import rendezvous as R
    assert R.parse_rendezvous_endpoint("node3:29400", 1) == ("node3", 29400)
    assert R.parse_rendezvous_endpoint("node3", 29500) == ("node3", 29500)
    assert R.parse_rendezvous_endpoint("[::1]:80", 1) == ("::1", 80) and R.parse_rendezvous_endpoint("", 7) == ("localhost", 7)
    with pytest.raises(ValueError):
        R.parse_rendezvous_endpoint("host:99999", 1)
    assert R._parse_rendezvous_config("timeout=30, read_timeout = 5") == {"timeout": "30", "read_timeout": "5"}
    with pytest.raises(ValueError):
        R._parse_rendezvous_config("timeout")
    assert R._matches_machine_hostname("localhost") and R._matches_machine_hostname("127.0.0.1")
    t = R.RendezvousTimeout(join=timedelta(seconds=3))
    assert t.join.total_seconds() == 3 and t.heartbeat.total_seconds() == 5
    with pytest.raises(ValueError):
        R.RendezvousTimeout(close=timedelta(0))
    ticks = []
    timer = R._PeriodicTimer(timedelta(milliseconds=20), ticks.append, 1)
    timer.start()
    import time
    time.sleep(0.3)
    timer.cancel()
    n_ticks = len(ticks)
    assert 1 <= n_ticks <= 16
    time.sleep(0.06)
    assert len(ticks) == n_ticks                      # cancelled: no tick after cancel() returned
    # fenced state back end: a writer with a stale token loses and is told the current state
    be = R.StoreRendezvousBackend(HashStore(), "job")
    assert be.get_state() is None
    state, token, ok = be.set_state(b"v1")
    assert ok and state == b"v1"
    _, _, ok_stale = be.set_state(b"v2-from-stale", token=b"something-else")
    assert not ok_stale and be.get_state()[0] == b"v1"
    _, token2, ok2 = be.set_state(b"v2", token=token)
    assert ok2 and be.get_state()[0] == b"v2" and token2 == b"v2"
    # registry: the static handler needs no negotiation; the dynamic one is reachable by name
    reg = R.get_registry()
    assert {"static", "dynamic"} <= set(reg.backends())
    h = reg.create_handler("dynamic", HashStore(), "j2", 1, 1)
    store, rank, world = h.next_rendezvous()
    assert (rank, world) == (0, 1)
    h.shutdown()
    with pytest.raises(ValueError):
        reg.create_handler("nope")


def test_logs_specs_layout(tmp_path):
    specs = emp.DefaultLogsSpecs(str(tmp_path), redirects=emp.Std.OUT, tee={1: emp.Std.ERR}, local_ranks_filter={1})
    dest = specs.reify({0: {"TORCHELASTIC_RUN_ID": "jobx", "TORCHELASTIC_RESTART_COUNT": 2}, 1: {}})
    assert specs.root_log_dir == str(tmp_path)
    assert dest.stdouts[0].endswith("attempt_2/0/stdout.log") and "jobx_" in dest.stdouts[0]
    assert dest.stderrs[0] == "" and dest.stderrs[1].endswith("1/stderr.log") and dest.tee_stderrs == {1: dest.stderrs[1]}
    assert os.path.isdir(os.path.dirname(dest.error_files[1])) and emp.Redirects is emp.Std
    e = emp.SignalException("got it", __import__("signal").SIGTERM)
    assert e.sigval.name == "SIGTERM"
