"""Starting, watching and ending the worker processes of one node, with per-rank log files, teeing and error
files (tensorplay/distributed/elastic/multiprocessing/api.py: ``Std``, ``RunProcsResult`` :329, ``PContext`` :343,
``MultiprocessContext`` :592, ``SubprocessContext`` :777, ``start_processes`` :875; errors/__init__.py:
``ProcessFailure`` :44, ``ChildFailedError`` :115, ``record`` :220; tail_log.py).

A worker whose entry point is wrapped in ``errors.record`` writes the exception and its traceback as JSON to the
file named by ``TORCHELASTIC_ERROR_FILE`` (set per rank by ``start_processes``) before it dies; the parent reads
it into the ``ProcessFailure`` of that rank, so the launcher reports WHY a rank failed, not only its exit code.
"""
from __future__ import annotations

import abc
import json
import multiprocessing as mp
import os
import signal
import subprocess
import sys
import threading
import time
import traceback
from dataclasses import dataclass, field
from enum import IntFlag
from functools import wraps
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

ERROR_FILE_ENV = "TORCHELASTIC_ERROR_FILE"


class Std(IntFlag):
    NONE = 0
    OUT = 1
    ERR = 2
    ALL = 3

    @classmethod
    def from_str(cls, vm: str) -> Union["Std", Dict[int, "Std"]]:
        """``"3"`` -> ``Std.ALL``; ``"0:3,1:0"`` -> ``{0: Std.ALL, 1: Std.NONE}``."""
        vm = vm.strip()
        if vm.isdigit() and int(vm) in (0, 1, 2, 3):
            return cls(int(vm))
        out: Dict[int, Std] = {}
        try:
            for part in vm.split(","):
                r, v = part.split(":")
                out[int(r)] = cls(int(v))
        except ValueError:
            raise ValueError(f"{vm!r} does not match: <0|1|2|3> or <rank>:<0|1|2|3>[,...]") from None
        return out


def to_map(val_or_map: Union[Std, Dict[int, Std]], local_world_size: int) -> Dict[int, Std]:
    if isinstance(val_or_map, dict):
        return {r: val_or_map.get(r, Std.NONE) for r in range(local_world_size)}
    return {r: val_or_map for r in range(local_world_size)}


class SignalException(Exception):
    """Raised in the launcher when it receives a termination signal, so that ``finally`` blocks end the workers."""

    def __init__(self, msg: str, sigval: signal.Signals):
        super().__init__(msg)
        self.sigval = sigval


Redirects = Std   # older name of the same flags


# ------------------------------------------------------------------------------------------- errors
@dataclass
class ProcessFailure:
    local_rank: int
    pid: int
    exitcode: int
    error_file: str
    error_file_data: Any = field(init=False, default=None)
    message: str = field(init=False, default="")
    timestamp: int = field(init=False, default=0)

    def __post_init__(self):
        self.timestamp = int(time.time())
        if self.error_file and os.path.isfile(self.error_file):
            try:
                with open(self.error_file) as f:
                    self.error_file_data = json.load(f)
                msg = self.error_file_data["message"]
                if isinstance(msg, dict):
                    self.message = msg.get("message", "")
                    self.timestamp = int(msg.get("extraInfo", {}).get("timestamp", self.timestamp))
                else:
                    self.message = str(msg)
            except Exception as e:   # a torn or foreign file must not hide the failure itself
                self.message = f"<could not read the error file {self.error_file}: {e}>"
        elif self.exitcode < 0:
            self.message = f"Signal {-self.exitcode} ({self.signal_name()}) received by PID {self.pid}"
        else:
            self.message = "To enable traceback wrap the entry point in errors.record"

    def signal_name(self) -> str:
        if self.exitcode < 0:
            try:
                return signal.Signals(-self.exitcode).name
            except ValueError:
                return "<Unknown signal>"
        return "<N/A>"

    def traceback(self) -> str:
        try:
            return self.error_file_data["message"]["extraInfo"]["py_callstack"]
        except Exception:
            return ""


class ChildFailedError(Exception):
    def __init__(self, name: str, failures: Dict[int, ProcessFailure]):
        self.name, self.failures = name, failures
        if not failures:
            raise ValueError("ChildFailedError needs at least one failure")
        super().__init__(self.format_msg())

    def get_first_failure(self) -> Tuple[int, ProcessFailure]:
        rank = min(self.failures, key=lambda r: self.failures[r].timestamp)
        return rank, self.failures[rank]

    def format_msg(self) -> str:
        rank, first = self.get_first_failure()
        lines = [f"{self.name} FAILED", "-" * 60, "Root cause (first observed failure):",
                 f"  local_rank {rank} (pid {first.pid}) exitcode {first.exitcode}: {first.message}"]
        tb = first.traceback()
        if tb:
            lines += ["  traceback:"] + ["    " + ln for ln in tb.rstrip().splitlines()]
        others = [r for r in sorted(self.failures) if r != rank]
        if others:
            lines.append("Other failures:")
            lines += [f"  local_rank {r} (pid {self.failures[r].pid}) exitcode {self.failures[r].exitcode}: "
                      f"{self.failures[r].message}" for r in others]
        return "\n".join(lines)


def _write_error_file(path: str, exc: BaseException) -> None:
    data = {"message": {"message": f"{type(exc).__name__}: {exc}",
                        "extraInfo": {"py_callstack": traceback.format_exc(), "timestamp": str(int(time.time()))}}}
    tmp = f"{path}.{os.getpid()}.tmp"
    with open(tmp, "w") as f:
        json.dump(data, f)
    os.replace(tmp, path)   # the parent never sees half a file


def record(fn: Optional[Callable] = None, *, error_file: Optional[str] = None):
    """Decorator for a worker's entry point: an exception that leaves it is written to the error file first."""
    def wrap(f):
        @wraps(f)
        def wrapper(*args, **kwargs):
            try:
                return f(*args, **kwargs)
            except SystemExit:
                raise
            except BaseException as e:
                path = error_file or os.environ.get(ERROR_FILE_ENV)
                if path:
                    try:
                        _write_error_file(path, e)
                    except OSError:
                        pass
                raise
        return wrapper
    return wrap(fn) if fn is not None else wrap


# ------------------------------------------------------------------------------------------- tail
class TailLog:
    """Copies lines appended to per-rank log files to ``dst`` with a ``[name rank]:`` prefix until stopped."""

    def __init__(self, name: str, log_files: Dict[int, str], dst=None, interval_sec: float = 0.1):
        self.name, self.files, self.dst, self.interval = name, log_files, dst or sys.stdout, interval_sec
        self._stop = threading.Event()
        self._threads: List[threading.Thread] = []

    def start(self) -> "TailLog":
        for r, path in self.files.items():
            t = threading.Thread(target=self._tail, args=(r, path), daemon=True)
            t.start()
            self._threads.append(t)
        return self

    def _tail(self, rank: int, path: str) -> None:
        while not os.path.exists(path):
            if self._stop.is_set():
                return
            time.sleep(self.interval)
        with open(path, errors="replace") as f:
            while True:
                line = f.readline()
                if line:
                    self.dst.write(f"[{self.name}{rank}]:{line}")
                    continue
                if self._stop.is_set():
                    return
                time.sleep(self.interval)

    def stop(self) -> None:
        self._stop.set()
        for t in self._threads:
            t.join(timeout=5)
        self._threads = []


def tail_logfile(header: str, file: str, dst, finished: threading.Event, interval_sec: float = 0.1) -> None:
    """Copies lines appended to ``file`` to ``dst`` behind ``header`` until ``finished`` is set and the file is read
    to its end."""
    while not os.path.exists(file):
        if finished.is_set():
            return
        time.sleep(interval_sec)
    with open(file, errors="replace") as f:
        while True:
            line = f.readline()
            if line:
                dst.write(f"{header}{line}")
            elif finished.is_set():
                return
            else:
                time.sleep(interval_sec)


# ------------------------------------------------------------------------------------------- log destinations
@dataclass
class LogsDest:
    """Per local rank: files for redirected stdout / stderr, the subset that is also teed, and the error files."""
    stdouts: Dict[int, str] = field(default_factory=dict)
    stderrs: Dict[int, str] = field(default_factory=dict)
    tee_stdouts: Dict[int, str] = field(default_factory=dict)
    tee_stderrs: Dict[int, str] = field(default_factory=dict)
    error_files: Dict[int, str] = field(default_factory=dict)


class LogsSpecs(abc.ABC):
    def __init__(self, log_dir: Optional[str] = None, redirects: Union[Std, Dict[int, Std]] = Std.NONE,
                 tee: Union[Std, Dict[int, Std]] = Std.NONE, local_ranks_filter: Optional[set] = None):
        self._root_log_dir, self._redirects, self._tee, self._local_ranks_filter = log_dir, redirects, tee, local_ranks_filter

    @abc.abstractmethod
    def reify(self, envs: Dict[int, Dict[str, str]]) -> LogsDest: ...

    @property
    @abc.abstractmethod
    def root_log_dir(self) -> str: ...


class DefaultLogsSpecs(LogsSpecs):
    """``<log_dir>/<run id>_<random>/attempt_<n>/<local rank>/{stdout,stderr}.log`` and ``error.json``."""

    def __init__(self, log_dir=None, redirects=Std.NONE, tee=Std.NONE, local_ranks_filter=None):
        import tempfile
        if log_dir is None:
            log_dir = tempfile.mkdtemp(prefix="tensorplay_elastic_")
        elif not os.path.exists(log_dir):
            os.makedirs(log_dir, exist_ok=True)
        super().__init__(log_dir, redirects, tee, local_ranks_filter)
        self._run_log_dir: Optional[str] = None

    @property
    def root_log_dir(self) -> str:
        return str(self._root_log_dir)

    def reify(self, envs: Dict[int, Dict[str, str]]) -> LogsDest:
        import tempfile
        n = len(envs)
        first = envs.get(0, {}) if n else {}
        if self._run_log_dir is None:
            run_id = str(first.get("TORCHELASTIC_RUN_ID", first.get("TP_RUN_ID", "run")))
            self._run_log_dir = tempfile.mkdtemp(prefix=f"{run_id}_", dir=self._root_log_dir)
        attempt = os.path.join(self._run_log_dir, f"attempt_{first.get('TORCHELASTIC_RESTART_COUNT', first.get('TP_RESTART_COUNT', 0))}")
        red, te = to_map(self._redirects, n), to_map(self._tee, n)
        dest = LogsDest()
        for r in range(n):
            d = os.path.join(attempt, str(r))
            os.makedirs(d, exist_ok=True)
            want = red[r] | te[r]
            dest.stdouts[r] = os.path.join(d, "stdout.log") if want & Std.OUT else ""
            dest.stderrs[r] = os.path.join(d, "stderr.log") if want & Std.ERR else ""
            shown = self._local_ranks_filter is None or r in self._local_ranks_filter
            if te[r] & Std.OUT and shown:
                dest.tee_stdouts[r] = dest.stdouts[r]
            if te[r] & Std.ERR and shown:
                dest.tee_stderrs[r] = dest.stderrs[r]
            dest.error_files[r] = os.path.join(d, "error.json")
        return dest


# ------------------------------------------------------------------------------------------- contexts
@dataclass
class RunProcsResult:
    return_values: Dict[int, Any] = field(default_factory=dict)
    failures: Dict[int, ProcessFailure] = field(default_factory=dict)
    stdouts: Dict[int, str] = field(default_factory=dict)
    stderrs: Dict[int, str] = field(default_factory=dict)

    def is_failed(self) -> bool:
        return bool(self.failures)


class PContext(abc.ABC):
    def __init__(self, name: str, entrypoint, args: Dict[int, Tuple], envs: Dict[int, Dict[str, str]],
                 logs_dir: Optional[str], redirects: Union[Std, Dict[int, Std]], tee: Union[Std, Dict[int, Std]]):
        n = len(args)
        if sorted(args) != list(range(n)) or sorted(envs) != list(range(n)):
            raise RuntimeError(f"args and envs must have one entry for each local rank 0..{n - 1}")
        self.name, self.entrypoint, self.args, self.envs, self.nprocs = name, entrypoint, args, envs, n
        red, te = to_map(redirects, n), to_map(tee, n)
        if logs_dir is None and (any(red.values()) or any(te.values())):
            import tempfile
            logs_dir = tempfile.mkdtemp(prefix=f"{name}_")
        self.logs_dir = logs_dir
        self.stdouts: Dict[int, str] = {}
        self.stderrs: Dict[int, str] = {}
        self.error_files: Dict[int, str] = {}
        tee_out, tee_err = {}, {}
        for r in range(n):
            d = None
            if logs_dir is not None:
                d = os.path.join(logs_dir, str(r))
                os.makedirs(d, exist_ok=True)
                self.error_files[r] = os.path.join(d, "error.json")
            want = red[r] | te[r]          # teeing reads the file, so it implies the redirect
            self.stdouts[r] = os.path.join(d, "stdout.log") if d and want & Std.OUT else ""
            self.stderrs[r] = os.path.join(d, "stderr.log") if d and want & Std.ERR else ""
            if te[r] & Std.OUT:
                tee_out[r] = self.stdouts[r]
            if te[r] & Std.ERR:
                tee_err[r] = self.stderrs[r]
        self._tails = [TailLog(name, tee_out, sys.stdout), TailLog(name, tee_err, sys.stderr)]
        self._started = False

    def start(self) -> None:
        self._start()
        for t in self._tails:
            t.start()
        self._started = True

    @abc.abstractmethod
    def _start(self) -> None: ...

    @abc.abstractmethod
    def _poll(self) -> Optional[RunProcsResult]: ...

    @abc.abstractmethod
    def pids(self) -> Dict[int, int]: ...

    @abc.abstractmethod
    def _close(self, death_sig: signal.Signals, timeout: float) -> None: ...

    def wait(self, timeout: float = -1, period: float = 0.1) -> Optional[RunProcsResult]:
        """The result once every process ended (or one failed: the others are then ended too); None when
        ``timeout`` seconds passed first (``0``: poll once, negative: no limit)."""
        deadline = None if timeout < 0 else time.time() + timeout
        while True:
            res = self._poll()
            if res is not None:
                return res
            if deadline is not None and time.time() >= deadline:
                return None
            time.sleep(period)

    def close(self, death_sig: Optional[signal.Signals] = None, timeout: float = 30) -> None:
        self._close(death_sig or signal.SIGTERM, timeout)
        for t in self._tails:
            t.stop()

    def _env_for(self, r: int) -> Dict[str, str]:
        env = dict(os.environ)
        env.update({k: str(v) for k, v in self.envs[r].items()})
        if r in self.error_files:
            env[ERROR_FILE_ENV] = self.error_files[r]
        return env

    def _failure(self, r: int, pid: int, code: int) -> ProcessFailure:
        return ProcessFailure(r, pid, code, self.error_files.get(r, ""))


class SubprocessContext(PContext):
    """``entrypoint`` is a program (path or name on PATH); ``args[r]`` its arguments for local rank ``r``."""

    def _start(self) -> None:
        self._procs: Dict[int, subprocess.Popen] = {}
        self._files = []
        for r in range(self.nprocs):
            out = open(self.stdouts[r], "w") if self.stdouts[r] else None
            err = open(self.stderrs[r], "w") if self.stderrs[r] else None
            self._files += [f for f in (out, err) if f]
            self._procs[r] = subprocess.Popen([self.entrypoint, *map(str, self.args[r])], env=self._env_for(r),
                                              stdout=out, stderr=err, start_new_session=True)

    def pids(self) -> Dict[int, int]:
        return {r: p.pid for r, p in self._procs.items()}

    def _poll(self) -> Optional[RunProcsResult]:
        codes = {r: p.poll() for r, p in self._procs.items()}
        failed = {r: c for r, c in codes.items() if c not in (None, 0)}
        if failed:
            self.close()
            return RunProcsResult(failures={r: self._failure(r, self._procs[r].pid, c) for r, c in failed.items()},
                                  stdouts=self.stdouts, stderrs=self.stderrs)
        if all(c == 0 for c in codes.values()):
            self.close()
            return RunProcsResult(return_values={r: None for r in codes}, stdouts=self.stdouts, stderrs=self.stderrs)
        return None

    def _close(self, death_sig, timeout) -> None:
        for p in self._procs.values():
            if p.poll() is None:
                try:
                    os.killpg(p.pid, death_sig)    # the process group this context started, nothing else
                except ProcessLookupError:
                    pass
        end = time.time() + timeout
        for p in self._procs.values():
            try:
                p.wait(timeout=max(0.05, end - time.time()))
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
                p.wait()
        for f in self._files:
            f.close()
        self._files = []


def _mp_entry(fn, args, env, stdout, stderr, rank, queue):
    os.environ.update(env)
    for path, fd in ((stdout, 1), (stderr, 2)):
        if path:
            f = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o644)
            os.dup2(f, fd)
            os.close(f)
    queue.put((rank, record(fn)(*args)))


class MultiprocessContext(PContext):
    """``entrypoint`` is a picklable function; each local rank runs ``entrypoint(*args[r])`` in a process of its
    own and its return value comes back in ``RunProcsResult.return_values``."""

    def __init__(self, *a, start_method: str = "spawn", **kw):
        super().__init__(*a, **kw)
        self._ctx = mp.get_context(start_method)

    def _start(self) -> None:
        self._queue = self._ctx.SimpleQueue()
        self._procs: Dict[int, Any] = {}
        self._returns: Dict[int, Any] = {}
        for r in range(self.nprocs):
            env = {k: str(v) for k, v in self.envs[r].items()}
            if r in self.error_files:
                env[ERROR_FILE_ENV] = self.error_files[r]
            p = self._ctx.Process(target=_mp_entry, args=(self.entrypoint, self.args[r], env, self.stdouts[r],
                                                          self.stderrs[r], r, self._queue), daemon=False)
            p.start()
            self._procs[r] = p

    def pids(self) -> Dict[int, int]:
        return {r: p.pid for r, p in self._procs.items()}

    def _poll(self) -> Optional[RunProcsResult]:
        while not self._queue.empty():
            r, v = self._queue.get()
            self._returns[r] = v
        codes = {r: p.exitcode for r, p in self._procs.items()}
        failed = {r: c for r, c in codes.items() if c not in (None, 0)}
        if failed:
            self.close()
            return RunProcsResult(failures={r: self._failure(r, self._procs[r].pid, c) for r, c in failed.items()},
                                  stdouts=self.stdouts, stderrs=self.stderrs)
        if all(c == 0 for c in codes.values()):
            while not self._queue.empty():
                r, v = self._queue.get()
                self._returns[r] = v
            self.close()
            return RunProcsResult(return_values=dict(self._returns), stdouts=self.stdouts, stderrs=self.stderrs)
        return None

    def _close(self, death_sig, timeout) -> None:
        for p in self._procs.values():
            if p.is_alive():
                try:
                    os.kill(p.pid, death_sig)
                except ProcessLookupError:
                    pass
        end = time.time() + timeout
        for p in self._procs.values():
            p.join(max(0.05, end - time.time()))
            if p.is_alive():
                p.kill()
                p.join()


def start_processes(name: str, entrypoint: Union[Callable, str], args: Dict[int, Tuple], envs: Dict[int, Dict[str, str]],
                    logs_dir: Optional[str] = None, redirects: Union[Std, Dict[int, Std]] = Std.NONE,
                    tee: Union[Std, Dict[int, Std]] = Std.NONE, start_method: str = "spawn") -> PContext:
    """Starts one process per local rank and returns their context (already started): a program when
    ``entrypoint`` is a string, a function otherwise."""
    if isinstance(entrypoint, str):
        ctx: PContext = SubprocessContext(name, entrypoint, args, envs, logs_dir, redirects, tee)
    else:
        ctx = MultiprocessContext(name, entrypoint, args, envs, logs_dir, redirects, tee, start_method=start_method)
    ctx.start()
    return ctx


from . import errors  # noqa: E402,F401  (sub-module view of ProcessFailure / ChildFailedError / record)
