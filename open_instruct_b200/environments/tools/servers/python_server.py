"""HTTP service behind the ``python`` tool: ``POST /execute {code, timeout} -> {output, error}``.

Each request runs in a worker process of a pool whose workers import the common scientific
packages once at start, so a call does not pay the import time
(cf. ``open_instruct/environments/tools/servers/python_server/tool_server.py:95-120``).

    uvicorn open_instruct_b200.environments.tools.servers.python_server:app --port 1212
"""

from __future__ import annotations

import contextlib
import io
import multiprocessing as mp
import traceback
from concurrent.futures import ProcessPoolExecutor, TimeoutError as FutTimeout

from fastapi import FastAPI
from pydantic import BaseModel

PREIMPORT = ("math", "json", "re", "itertools", "collections", "fractions", "statistics", "numpy", "sympy")


def _warm():
    for m in PREIMPORT:
        try:
            __import__(m)
        except ImportError:
            pass


def _run(code: str) -> dict:
    out = io.StringIO()
    try:
        with contextlib.redirect_stdout(out), contextlib.redirect_stderr(out):
            exec(compile(code, "<tool>", "exec"), {"__name__": "__main__"})  # noqa: S102
        return {"output": out.getvalue(), "error": None}
    except BaseException:  # noqa: BLE001
        return {"output": out.getvalue(), "error": traceback.format_exc(limit=3)}


app = FastAPI()
_pool: ProcessPoolExecutor | None = None


def pool() -> ProcessPoolExecutor:
    global _pool
    if _pool is None:
        _pool = ProcessPoolExecutor(max_workers=8, mp_context=mp.get_context("spawn"), initializer=_warm)
    return _pool


class ExecRequest(BaseModel):
    code: str
    timeout: float = 5.0


@app.get("/health")
def health():
    return {"status": "healthy"}


@app.post("/execute")
def execute(req: ExecRequest):
    global _pool
    fut = pool().submit(_run, req.code)
    try:
        return fut.result(timeout=req.timeout)
    except FutTimeout:
        # a stuck worker cannot be cancelled: replace the pool
        old, _pool = _pool, None
        old.shutdown(wait=False, cancel_futures=True)
        return {"output": "", "error": f"Timeout after {req.timeout} seconds"}
