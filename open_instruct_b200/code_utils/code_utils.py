"""Run untrusted programs against test cases, one OS process per test with a hard timeout.

Contract of the reference's code-execution helpers (``open_instruct/code_utils/code_utils.py:146-191``,
``:314``): ``get_successful_tests_fast(program, tests, max_execution_time)`` returns a 0/1 list (assert-style
tests appended to the program) plus runtimes; ``get_successful_tests_stdio`` feeds ``input`` on stdin and
compares stdout with ``output``; ``reliability_guard`` disables destructive builtins inside the child.
"""

from __future__ import annotations

import contextlib
import faulthandler
import io
import multiprocessing as mp
import os
import sys
import time


def reliability_guard(max_memory_bytes: int | None = None) -> None:
    """Neuter functions that could damage the host (called inside the child process only)."""
    if max_memory_bytes is not None:
        import resource

        resource.setrlimit(resource.RLIMIT_AS, (max_memory_bytes, max_memory_bytes))
    faulthandler.disable()
    import builtins
    import shutil
    import subprocess

    builtins.exit = builtins.quit = None
    os.environ["OMP_NUM_THREADS"] = "1"
    for name in ("kill", "system", "putenv", "remove", "removedirs", "rmdir", "fchdir", "setuid", "fork", "forkpty", "killpg", "rename",
                 "renames", "truncate", "replace", "unlink", "fchmod", "fchown", "chmod", "chown", "chroot", "lchown", "chdir"):
        if hasattr(os, name):
            setattr(os, name, None)
    shutil.rmtree = shutil.move = shutil.chown = None
    subprocess.Popen = None


def _run_assert_test(program: str, test: str, q) -> None:
    reliability_guard()
    t0 = time.perf_counter()
    try:
        with contextlib.redirect_stdout(io.StringIO()), contextlib.redirect_stderr(io.StringIO()):
            exec(compile(program + "\n" + test, "<program>", "exec"), {"__name__": "__main__"})  # noqa: S102
        q.put((1, time.perf_counter() - t0))
    except BaseException:  # noqa: BLE001
        q.put((0, time.perf_counter() - t0))


def _run_stdio_test(program: str, stdin_text: str, expected: str, q) -> None:
    reliability_guard()
    t0 = time.perf_counter()
    out = io.StringIO()
    try:
        sys.stdin = io.StringIO(stdin_text)
        with contextlib.redirect_stdout(out), contextlib.redirect_stderr(io.StringIO()):
            exec(compile(program, "<program>", "exec"), {"__name__": "__main__"})  # noqa: S102
        ok = out.getvalue().strip().split() == str(expected).strip().split()
        q.put((int(ok), time.perf_counter() - t0))
    except BaseException:  # noqa: BLE001
        q.put((0, time.perf_counter() - t0))


def _run_isolated(target, args, timeout: float) -> tuple[int, float]:
    ctx = mp.get_context("fork")
    q = ctx.Queue()
    p = ctx.Process(target=target, args=(*args, q), daemon=True)
    p.start()
    p.join(timeout)
    if p.is_alive():
        p.kill()
        p.join()
        return 0, timeout
    try:
        return q.get(timeout=0.5)
    except Exception:  # noqa: BLE001 - child died without reporting (segfault, os._exit)
        return 0, timeout


def get_successful_tests_fast(program: str, tests: list[str], max_execution_time: float = 1.0):
    """(results, runtimes): one isolated process per assert-style test."""
    if not tests:
        return [], []
    if not should_execute(program, tests):
        return [0] * len(tests), [-1.0] * len(tests)
    out = [_run_isolated(_run_assert_test, (program, t), max_execution_time) for t in tests]
    return [r for r, _ in out], [t for _, t in out]


def get_successful_tests_stdio(program: str, tests: list[dict], max_execution_time: float = 1.0):
    if not tests:
        return [], []
    if not should_execute(program, tests):
        return [0] * len(tests), [-1.0] * len(tests)
    out = [_run_isolated(_run_stdio_test, (program, t.get("input", ""), t.get("output", "")), max_execution_time) for t in tests]
    return [r for r, _ in out], [t for _, t in out]


def should_execute(program: str, tests) -> bool:
    """Cheap static screen: refuse programs that reach for the threading / process machinery."""
    banned = ("import threading", "from threading", "import multiprocessing", "from multiprocessing", "os.fork", "subprocess")
    return not any(b in program for b in banned)
