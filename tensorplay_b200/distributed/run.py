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
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .store import TCPStore


class ChildFailedError(RuntimeError):
    def __init__(self, name: str, failures: Dict[int, int]):
        self.name, self.failures = name, failures
        first = min(failures)
        super().__init__(f"{name} failed: rank {first} exited with code {failures[first]} "
                         f"(all failures: {failures})")


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
        self.store = TCPStore(config.master_addr, config.master_port, is_master=True, timeout=60)
        self.procs: List[subprocess.Popen] = []
        self.restart_count = 0
        self.logs = []

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
                        "TORCHELASTIC_RESTART_COUNT": str(self.restart_count)})
            out = None
            if self.cfg.log_dir:
                os.makedirs(self.cfg.log_dir, exist_ok=True)
                out = open(os.path.join(self.cfg.log_dir, f"attempt{self.restart_count}_rank{r}.log"), "w")
                self.logs.append(out)
            self.procs.append(subprocess.Popen(self.cmd, env=env, stdout=out, stderr=subprocess.STDOUT if out else None,
                                               start_new_session=True))

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
        for f in self.logs:
            f.close()

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
        try:
            while True:
                self._start_workers()
                failed = self._monitor()
                if not failed:
                    for f in self.logs:
                        f.close()
                    return 0
                self._stop_workers()
                if self.restart_count >= self.cfg.max_restarts:
                    raise ChildFailedError(" ".join(self.cmd[:3]), failed)
                self.restart_count += 1
                self.store.set(f"restart/{self.restart_count}", str(failed))
        finally:
            self.store.close()


def elastic_launch(config: LaunchConfig, cmd: List[str]) -> int:
    return LocalElasticAgent(config, cmd).run()


def run(args) -> int:
    """Launch from a parsed argument namespace or an argv list (the function form of ``tprun``)."""
    return main(args if isinstance(args, (list, tuple)) else None)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="tprun")
    ap.add_argument("--nproc-per-node", "--nproc_per_node", type=int, default=int(os.environ.get("TP_NPROC", "1")))
    ap.add_argument("--max-restarts", "--max_restarts", type=int, default=0)
    ap.add_argument("--master-addr", default="127.0.0.1")
    ap.add_argument("--master-port", type=int, default=0)
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("--no-python", action="store_true")
    ap.add_argument("script")
    ap.add_argument("script_args", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = ([] if a.no_python else [sys.executable, "-u"]) + [a.script] + a.script_args
    cfg = LaunchConfig(a.nproc_per_node, a.max_restarts, master_addr=a.master_addr, master_port=a.master_port,
                       log_dir=a.log_dir)
    try:
        return elastic_launch(cfg, cmd)
    except ChildFailedError as e:
        print(f"tprun: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
