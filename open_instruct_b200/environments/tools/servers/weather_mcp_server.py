"""Deterministic fake-weather MCP server for tests of the MCP tool client (JSON-RPC over HTTP POST /mcp):
``tools/list`` and ``tools/call`` for ``get_current_weather`` and ``get_forecast``."""

from __future__ import annotations

import hashlib

from fastapi import FastAPI, Request

app = FastAPI()
TOOLS = [
    {"name": "get_current_weather", "description": "Current weather for a city",
     "inputSchema": {"type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}},
    {"name": "get_forecast", "description": "Forecast for the next days",
     "inputSchema": {"type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}}, "required": ["city"]}},
]


def _temp(city: str, day: int = 0) -> int:
    return int(hashlib.sha256(f"{city.lower()}:{day}".encode()).hexdigest(), 16) % 35


@app.post("/mcp")
async def mcp(request: Request):
    body = await request.json()
    rid, method, params = body.get("id"), body.get("method"), body.get("params", {})
    if method == "tools/list":
        return {"jsonrpc": "2.0", "id": rid, "result": {"tools": TOOLS}}
    if method == "tools/call":
        name, args = params.get("name"), params.get("arguments", {})
        city = args.get("city", "")
        if name == "get_current_weather":
            text = f"{city}: {_temp(city)} C, clear"
        elif name == "get_forecast":
            text = "\n".join(f"day {d + 1}: {_temp(city, d + 1)} C" for d in range(int(args.get("days", 3))))
        else:
            return {"jsonrpc": "2.0", "id": rid, "error": {"code": -32601, "message": f"unknown tool {name}"}}
        return {"jsonrpc": "2.0", "id": rid, "result": {"content": [{"type": "text", "text": text}]}}
    return {"jsonrpc": "2.0", "id": rid, "error": {"code": -32601, "message": f"unknown method {method}"}}
