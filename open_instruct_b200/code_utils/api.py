"""HTTP service for code-execution rewards (``POST /test_program``, ``POST /test_program_stdio``, ``GET /health``).

    uvicorn open_instruct_b200.code_utils.api:app --host 127.0.0.1 --port 1234

Request ``{program, tests, max_execution_time}`` -> ``{results: [0/1...], runtimes: [...]}``
(cf. ``open_instruct/code_utils/api.py``)."""

from __future__ import annotations

from fastapi import FastAPI, HTTPException
from pydantic import BaseModel

from .code_utils import get_successful_tests_fast, get_successful_tests_stdio

app = FastAPI()


class TestRequest(BaseModel):
    program: str
    tests: list
    max_execution_time: float = 1.0


@app.get("/health")
def health():
    return {"status": "healthy"}


@app.post("/test_program")
def test_program(req: TestRequest):
    try:
        results, runtimes = get_successful_tests_fast(req.program, req.tests, req.max_execution_time)
        return {"results": results, "runtimes": runtimes}
    except Exception as e:  # noqa: BLE001
        raise HTTPException(status_code=500, detail=str(e)) from e


@app.post("/test_program_stdio")
def test_program_stdio(req: TestRequest):
    try:
        results, runtimes = get_successful_tests_stdio(req.program, req.tests, req.max_execution_time)
        return {"results": results, "runtimes": runtimes}
    except Exception as e:  # noqa: BLE001
        raise HTTPException(status_code=500, detail=str(e)) from e
