"""Generate completions from an OpenAI-compatible endpoint: concurrent chat calls for small jobs, the batch API
(upload jsonl -> create batch -> poll -> download) for large ones (``open_instruct/experimental/oai_generate.py``).

Input jsonl rows: ``{"custom_id": ..., "body": {"messages": [...], ...}}``; output rows add ``"response"``.
Endpoint and key come from ``OPENAI_BASE_URL`` / ``OPENAI_API_KEY`` (or the ``AZURE_OPENAI_*`` pair).
"""

from __future__ import annotations

import asyncio
import json
import os
import time
from dataclasses import dataclass


@dataclass
class Args:
    input_file: str = "input.jsonl"
    output_file: str = "output.jsonl"
    model: str = "gpt-4o"
    batch: bool = False
    max_parallel_requests: int = 32
    poll_seconds: float = 30.0
    max_tokens: int = 2048


def endpoint() -> tuple[str, dict]:
    base = os.environ.get("OPENAI_BASE_URL") or os.environ.get("AZURE_OPENAI_ENDPOINT") or "https://api.openai.com/v1"
    key = os.environ.get("OPENAI_API_KEY") or os.environ.get("AZURE_OPENAI_API_KEY") or ""
    return base.rstrip("/"), {"Authorization": f"Bearer {key}", "api-key": key}


def read_jsonl(path: str) -> list[dict]:
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]


def write_jsonl(path: str, rows: list[dict]) -> None:
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")


async def run_chat(rows: list[dict], args: Args, post=None) -> list[dict]:
    """``post(url, json, headers) -> dict`` can be injected (tests); default is aiohttp."""
    base, headers = endpoint()
    sem = asyncio.Semaphore(args.max_parallel_requests)

    async def default_post(url, payload, hdrs):
        import aiohttp

        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=600)) as s:
            async with s.post(url, json=payload, headers=hdrs) as r:
                r.raise_for_status()
                return await r.json()

    post = post or default_post

    async def one(row):
        body = {"model": args.model, "max_tokens": args.max_tokens, **row.get("body", {})}
        async with sem:
            for attempt in range(4):
                try:
                    out = await post(base + "/chat/completions", body, headers)
                    return {**row, "response": out["choices"][0]["message"]["content"], "usage": out.get("usage")}
                except Exception as e:  # noqa: BLE001
                    err = str(e)
                    await asyncio.sleep(min(2**attempt, 8) * 0.01 if post is not default_post else 2**attempt)
            return {**row, "response": None, "error": err}

    return await asyncio.gather(*[one(r) for r in rows])


def run_batch(rows: list[dict], args: Args, http=None) -> list[dict]:
    """Batch API flow.  ``http(method, url, **kw) -> dict | bytes`` can be injected; default uses ``requests``."""
    base, headers = endpoint()

    def default_http(method, url, **kw):
        import requests

        r = requests.request(method, url, headers=headers, timeout=600, **kw)
        r.raise_for_status()
        return r.content if kw.pop("raw", False) or url.endswith("/content") else r.json()

    http = http or default_http
    lines = [json.dumps({"custom_id": r.get("custom_id", str(i)), "method": "POST", "url": "/v1/chat/completions",
                         "body": {"model": args.model, "max_tokens": args.max_tokens, **r.get("body", {})}}) for i, r in enumerate(rows)]
    up = http("POST", base + "/files", files={"file": ("batch.jsonl", "\n".join(lines).encode())}, data={"purpose": "batch"})
    job = http("POST", base + "/batches", json={"input_file_id": up["id"], "endpoint": "/v1/chat/completions", "completion_window": "24h"})
    while job["status"] not in ("completed", "failed", "expired", "cancelled"):
        time.sleep(args.poll_seconds)
        job = http("GET", base + f"/batches/{job['id']}")
    if job["status"] != "completed":
        raise RuntimeError(f"batch {job['id']} ended as {job['status']}")
    content = http("GET", base + f"/files/{job['output_file_id']}/content")
    by_id = {}
    for line in content.decode().splitlines():
        if line.strip():
            o = json.loads(line)
            by_id[o["custom_id"]] = o["response"]["body"]["choices"][0]["message"]["content"]
    return [{**r, "response": by_id.get(r.get("custom_id", str(i)))} for i, r in enumerate(rows)]


def main(args: Args) -> list[dict]:
    rows = read_jsonl(args.input_file)
    out = run_batch(rows, args) if args.batch else asyncio.run(run_chat(rows, args))
    write_jsonl(args.output_file, out)
    return out


if __name__ == "__main__":
    from ..config.argparser import ArgumentParserPlus

    main(ArgumentParserPlus((Args,)).parse())
