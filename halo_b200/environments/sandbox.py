"""Sandboxed program execution behind one interface (halo/environments/sandbox/base.py:12-69, factory.py:28).

``SubprocessSandbox`` runs a program in a child Python process with CPU-time, memory and wall-clock limits,
an empty environment and a scratch working directory. ``InProcessSandbox`` evaluates in this process (tests
and trusted tasks only). Remote and container backends plug in through ``register_sandbox``."""

from __future__ import annotations

import os
import resource
import subprocess
import sys
import tempfile
from dataclasses import dataclass


@dataclass
class ExecResult:
    stdout: str
    stderr: str
    exit_code: int
    timed_out: bool = False


class Sandbox:
    def run(self, source: str, stdin: str = "", timeout_s: float = 10.0) -> ExecResult:
        raise NotImplementedError

    def close(self) -> None: ...


class SubprocessSandbox(Sandbox):
    def __init__(self, memory_mb: int = 512, cpu_seconds: int = 10):
        self.memory_mb, self.cpu_seconds = memory_mb, cpu_seconds
        self._dir = tempfile.TemporaryDirectory(prefix="halo_sbx_")

    def _limits(self):
        resource.setrlimit(resource.RLIMIT_CPU, (self.cpu_seconds, self.cpu_seconds))
        mem = self.memory_mb << 20
        resource.setrlimit(resource.RLIMIT_AS, (mem, mem))
        resource.setrlimit(resource.RLIMIT_NPROC, (64, 64))
        os.setsid()

    def run(self, source: str, stdin: str = "", timeout_s: float = 10.0) -> ExecResult:
        path = os.path.join(self._dir.name, "main.py")
        with open(path, "w") as f:
            f.write(source)
        try:
            p = subprocess.run([sys.executable, "-I", path], input=stdin, capture_output=True, text=True, timeout=timeout_s,
                               cwd=self._dir.name, env={"PATH": "/usr/bin:/bin"}, preexec_fn=self._limits)
            return ExecResult(p.stdout, p.stderr, p.returncode)
        except subprocess.TimeoutExpired as exc:
            return ExecResult(exc.stdout or "", exc.stderr or "", -9, timed_out=True)

    def close(self) -> None:
        self._dir.cleanup()


class InProcessSandbox(Sandbox):
    def run(self, source: str, stdin: str = "", timeout_s: float = 10.0) -> ExecResult:
        import contextlib
        import io

        out, err = io.StringIO(), io.StringIO()
        code = 0
        old_stdin = sys.stdin
        sys.stdin = io.StringIO(stdin)
        try:
            with contextlib.redirect_stdout(out), contextlib.redirect_stderr(err):
                exec(compile(source, "<sandbox>", "exec"), {"__name__": "__main__"})  # noqa: S102
        except SystemExit as exc:
            code = int(exc.code or 0)
        except BaseException as exc:  # noqa: BLE001
            err.write(f"{type(exc).__name__}: {exc}")
            code = 1
        finally:
            sys.stdin = old_stdin
        return ExecResult(out.getvalue(), err.getvalue(), code)


_BACKENDS = {"subprocess": SubprocessSandbox, "inprocess": InProcessSandbox}


def register_sandbox(name: str, cls) -> None:
    _BACKENDS[name] = cls


def make_sandbox(name: str = "subprocess", **kw) -> Sandbox:
    if name not in _BACKENDS:
        raise KeyError(f"unknown sandbox backend {name!r}; registered: {sorted(_BACKENDS)}")
    return _BACKENDS[name](**kw)
