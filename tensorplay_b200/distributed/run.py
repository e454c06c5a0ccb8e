"""``tprun``: elastic single-node launcher.

    python -m tensorplay_b200.distributed.run --nproc-per-node 8 [--max-restarts 3] train.py args...

Starts one worker process per rank with RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT,
hosts the native TCP store for rendezvous, monitors the workers, and on a failure tears the group
down and restarts all of them (new restart generation, ``TP_RESTART_COUNT``) up to
``--max-restarts`` times; when restarts are exhausted it raises ``ChildFailedError`` carrying the
first failure. Worker output can be teed into per-rank log files. Plays the role of
tensorplay/distributed/run.py:52-118 + elastic/agent/server/local_elastic_agent.py:205-434.
"""
from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .store import TCPStore


class ChildFailedError(RuntimeError):
    """``failures`` maps rank to exit code; ``details`` (when the agent could read them) maps rank to the
    ``ProcessFailure`` built from the rank's error file: the exception and traceback that a worker wrapped in
    ``elastic.multiprocessing.errors.record`` wrote before it died."""

    def __init__(self, name: str, failures: Dict[int, int], details: Optional[dict] = None):
        self.name, self.failures, self.details = name, failures, details or {}
        first = min(failures)
        msg = f"{name} failed: rank {first} exited with code {failures[first]} (all failures: {failures})"
        d = self.details.get(first)
        if d is not None and d.message:
            msg += f"\nrank {first}: {d.message}"
            tb = d.traceback()
            if tb:
                msg += "\n" + tb.rstrip()
        super().__init__(msg)


@dataclass
class LaunchConfig:
    nproc_per_node: int = 1
    max_restarts: int = 0
    monitor_interval: float = 0.1
    master_addr: str = "127.0.0.1"
    master_port: int = 0
    log_dir: Optional[str] = None
    tee: bool = False
    env: Dict[str, str] = field(default_factory=dict)


class LocalElasticAgent:
    def __init__(self, config: LaunchConfig, cmd: List[str]):
        self.cfg, self.cmd = config, cmd
        if config.master_addr in ("127.0.0.1", "localhost"):
            # one node: the rendezvous store listens on loopback only
            os.environ.setdefault("TPB_STORE_BIND_ADDR", "127.0.0.1")
        self.store = TCPStore(config.master_addr, config.master_port, is_master=True, timeout=60)
        self.procs: List[subprocess.Popen] = []
        self.restart_count = 0
        self.logs = []
        self._tees: List[threading.Thread] = []
        self._error_dir: Optional[str] = None

    def _start_workers(self) -> None:
        n = self.cfg.nproc_per_node
        # torch's own env:// rendezvous needs a second port (its TCPStore); pick a free one
        import socket
        with socket.socket() as s:
            s.bind((self.cfg.master_addr, 0))
            port = s.getsockname()[1]
        self.procs, self.logs = [], []
        for r in range(n):
            env = dict(os.environ)
            env.update(self.cfg.env)
            env.update({"RANK": str(r), "LOCAL_RANK": str(r), "WORLD_SIZE": str(n), "LOCAL_WORLD_SIZE": str(n),
                        "MASTER_ADDR": self.cfg.master_addr, "MASTER_PORT": str(port),
                        "TP_STORE_ADDR": self.cfg.master_addr, "TP_STORE_PORT": str(self.store.port),
                        "TP_RESTART_COUNT": str(self.restart_count),
                        "TORCHELASTIC_RESTART_COUNT": str(self.restart_count),
                        "TORCHELASTIC_ERROR_FILE": self._error_file(r)})
            out = None
            if self.cfg.log_dir:
                os.makedirs(self.cfg.log_dir, exist_ok=True)
                out = open(os.path.join(self.cfg.log_dir, f"attempt{self.restart_count}_rank{r}.log"), "w")
                self.logs.append(out)
            tee = self.cfg.tee and out is not None
            p = subprocess.Popen(self.cmd, env=env, stdout=subprocess.PIPE if tee else out,
                                 stderr=subprocess.STDOUT if out else None, start_new_session=True)
            if tee:
                # the rank's output goes to its log file and, prefixed, to the launcher's stdout
                t = threading.Thread(target=self._tee, args=(p.stdout, out, r), daemon=True)
                t.start()
                self._tees.append(t)
            self.procs.append(p)

    def _error_file(self, rank: int) -> str:
        if self._error_dir is None:
            import tempfile
            self._error_dir = self.cfg.log_dir or tempfile.mkdtemp(prefix="tprun_errors_")
            os.makedirs(self._error_dir, exist_ok=True)
        return os.path.join(self._error_dir, f"attempt{self.restart_count}_rank{rank}_error.json")

    def _failure_details(self, failed: Dict[int, int]) -> dict:
        from .elastic.multiprocessing import ProcessFailure
        return {r: ProcessFailure(r, self.procs[r].pid, c, self._error_file(r)) for r, c in failed.items()}

    @staticmethod
    def _tee(pipe, log, rank: int) -> None:
        for line in iter(pipe.readline, b""):
            text = line.decode("utf-8", "replace")
            log.write(text)
            log.flush()
            sys.stdout.write(f"[rank{rank}] {text}")
            sys.stdout.flush()
        pipe.close()

    def _stop_workers(self) -> None:
        for p in self.procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)
                except ProcessLookupError:
                    pass
        deadline = time.time() + 10
        for p in self.procs:
            try:
                p.wait(timeout=max(0.1, deadline - time.time()))
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
        for t in self._tees:
            t.join(timeout=2)
        self._tees = []
        for f in self.logs:
            f.close()
        self.logs = []

    def _monitor(self) -> Dict[int, int]:
        """Blocks until all workers exited 0 (returns {}) or one failed (returns {rank: code})."""
        while True:
            codes = [p.poll() for p in self.procs]
            failed = {r: c for r, c in enumerate(codes) if c not in (None, 0)}
            if failed:
                return failed
            if all(c == 0 for c in codes):
                return {}
            time.sleep(self.cfg.monitor_interval)

    def run(self) -> int:
        """Runs the group to completion. Whatever ends the launcher (a worker failure past the restart
        budget, Ctrl-C, SIGTERM, an exception in here) also ends every worker: the ranks run in
        sessions of their own and would otherwise outlive the launcher holding their GPUs."""

        def _on_signal(signum, _frame):
            raise KeyboardInterrupt(f"tprun: signal {signum}")

        previous = {}
        if threading.current_thread() is threading.main_thread():
            for sig in (signal.SIGTERM, signal.SIGINT):
                previous[sig] = signal.signal(sig, _on_signal)
        try:
            while True:
                self._start_workers()
                failed = self._monitor()
                if not failed:
                    self._stop_workers()  # all exited 0: joins the tee threads, closes the logs
                    return 0
                self._stop_workers()
                if self.restart_count >= self.cfg.max_restarts:
                    raise ChildFailedError(" ".join(self.cmd[:3]), failed, self._failure_details(failed))
                self.restart_count += 1
                self.store.set(f"restart/{self.restart_count}", str(failed))
        finally:
            self._stop_workers()
            for sig, h in previous.items():
                signal.signal(sig, h)
            self.store.close()


def elastic_launch(config: LaunchConfig, cmd: List[str]) -> int:
    return LocalElasticAgent(config, cmd).run()


def run(args) -> int:
    """Launch from a parsed argument namespace (as ``get_args_parser().parse_args`` returns it) or
    an argv list: the function form of ``tprun``."""
    if isinstance(args, argparse.Namespace):
        return _launch(args)
    return main(list(args) if args is not None else None)


def get_args_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="tprun")
    ap.add_argument("--nproc-per-node", "--nproc_per_node", type=int, default=int(os.environ.get("TP_NPROC", "1")))
    ap.add_argument("--max-restarts", "--max_restarts", type=int, default=0)
    ap.add_argument("--master-addr", default="127.0.0.1")
    ap.add_argument("--master-port", type=int, default=0)
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("--tee", action="store_true", help="with --log-dir: also print every rank's output, prefixed")
    ap.add_argument("--no-python", action="store_true")
    ap.add_argument("script")
    ap.add_argument("script_args", nargs=argparse.REMAINDER)
    return ap


def main(argv=None) -> int:
    return _launch(get_args_parser().parse_args(argv))


def _launch(a: argparse.Namespace) -> int:
    cmd = ([] if a.no_python else [sys.executable, "-u"]) + [a.script] + list(a.script_args)
    cfg = LaunchConfig(a.nproc_per_node, a.max_restarts, master_addr=a.master_addr, master_port=a.master_port,
                       log_dir=a.log_dir, tee=getattr(a, "tee", False))
    try:
        return elastic_launch(cfg, cmd)
    except ChildFailedError as e:
        print(f"tprun: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
