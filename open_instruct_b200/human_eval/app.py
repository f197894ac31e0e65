"""Annotation server for pairwise human evaluation (FastAPI + sqlite3; the reference's is Flask + SQLAlchemy,
``human_eval/app.py``).

Routes: ``POST /signup`` / ``POST /login`` (JSON ``{username, password}`` -> session token, also set as a cookie),
``GET /instances/{i}`` (annotation page), ``GET /api/model-outputs/{i}`` (prompt + the two completions in random order),
``POST /api/submit-evaluation``, ``POST /api/submit-feedback``, ``GET /summary``.  Comparison instances are a JSON(L)
file of ``{"id", "prompt", "completions": [{"model", "completion"}, {"model", "completion"}]}``.

    python -m open_instruct_b200.human_eval.app --comparison_data_path data/eval_instances.json --port 5001
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import random
import secrets
import sqlite3
import threading
import time

from fastapi import FastAPI, HTTPException, Request, Response
from fastapi.responses import HTMLResponse

from .metrics import summarize

FIELDS = ("instance_index", "instance_id", "prompt", "model_a", "model_b", "completion_a", "completion_b",
          "completion_a_is_acceptable", "completion_b_is_acceptable", "preference", "instance_quality", "comment", "evaluator",
          "timestamp")

PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>Human evaluation</title>
<style>body{font-family:sans-serif;max-width:1100px;margin:2em auto}.c{display:flex;gap:1em}.c pre{flex:1;white-space:pre-wrap;
border:1px solid #ccc;padding:1em}</style></head><body><h2>Instance __INDEX__</h2><pre id="prompt"></pre>
<div class="c"><pre id="a"></pre><pre id="b"></pre></div>
<p>A acceptable? <select id="acc_a"><option>yes</option><option>no</option></select>
B acceptable? <select id="acc_b"><option>yes</option><option>no</option></select>
Preference <select id="pref"><option>a-is-better</option><option>a-is-slightly-better</option><option>tie</option>
<option>b-is-slightly-better</option><option>b-is-better</option></select> <button onclick="submit()">Submit</button>
<a href="/instances/__NEXT__">next</a></p>
<script>let d;fetch('/api/model-outputs/__INDEX__').then(r=>r.json()).then(j=>{d=j;prompt.textContent=j.prompt;
a.textContent=j.completions[0].completion;b.textContent=j.completions[1].completion});
function submit(){fetch('/api/submit-evaluation',{method:'POST',headers:{'Content-Type':'application/json'},body:JSON.stringify({
index:__INDEX__,prompt:d.prompt,model_a:d.completions[0].model,model_b:d.completions[1].model,completion_a:d.completions[0].completion,
completion_b:d.completions[1].completion,completion_a_is_acceptable:acc_a.value,completion_b_is_acceptable:acc_b.value,
preference:pref.value})}).then(r=>{if(r.ok)location='/instances/__NEXT__';else alert('log in first: POST /login')})}</script></body></html>"""


def load_instances(path: str) -> list[dict]:
    with open(path) as fh:
        text = fh.read().strip()
    return json.loads(text) if text.startswith("[") else [json.loads(line) for line in text.splitlines() if line.strip()]


class Store:
    """sqlite3 behind a lock (annotation traffic is a few writes per minute)."""

    def __init__(self, path: str):
        self.db = sqlite3.connect(path, check_same_thread=False)
        self.db.row_factory = sqlite3.Row
        self.lock = threading.Lock()
        with self.lock:
            self.db.execute("CREATE TABLE IF NOT EXISTS users (username TEXT PRIMARY KEY, salt TEXT, password TEXT)")
            self.db.execute(f"CREATE TABLE IF NOT EXISTS records (id INTEGER PRIMARY KEY AUTOINCREMENT, {', '.join(f + ' TEXT' for f in FIELDS)})")
            self.db.commit()

    @staticmethod
    def _hash(password: str, salt: str) -> str:
        return hashlib.pbkdf2_hmac("sha256", password.encode(), salt.encode(), 100_000).hex()

    def add_user(self, username: str, password: str) -> bool:
        salt = secrets.token_hex(8)
        with self.lock:
            try:
                self.db.execute("INSERT INTO users VALUES (?, ?, ?)", (username, salt, self._hash(password, salt)))
                self.db.commit()
                return True
            except sqlite3.IntegrityError:
                return False

    def check_user(self, username: str, password: str) -> bool:
        with self.lock:
            row = self.db.execute("SELECT salt, password FROM users WHERE username = ?", (username,)).fetchone()
        return row is not None and secrets.compare_digest(row["password"], self._hash(password, row["salt"]))

    def users(self) -> list[str]:
        with self.lock:
            return [r["username"] for r in self.db.execute("SELECT username FROM users")]

    def add_record(self, rec: dict) -> None:
        with self.lock:
            self.db.execute(f"INSERT INTO records ({', '.join(FIELDS)}) VALUES ({', '.join('?' * len(FIELDS))})",
                            tuple(str(rec.get(f, "")) if f != "instance_index" else int(rec[f]) for f in FIELDS))
            self.db.commit()

    def records(self) -> list[dict]:
        with self.lock:
            rows = self.db.execute(f"SELECT {', '.join(FIELDS)} FROM records ORDER BY id").fetchall()
        return [dict(r, instance_index=int(r["instance_index"])) for r in rows]


def create_app(instances: list[dict], db_path: str = ":memory:", seed: int | None = None):
    app = FastAPI(title="human evaluation")
    store = Store(db_path)
    sessions: dict[str, str] = {}
    rng = random.Random(seed)
    app.state.store = store

    def user_of(request: Request) -> str:
        token = request.cookies.get("session") or request.headers.get("authorization", "").removeprefix("Bearer ").strip()
        if token not in sessions:
            raise HTTPException(status_code=401, detail="log in first")
        return sessions[token]

    def _login(username: str, response: Response) -> dict:
        token = secrets.token_urlsafe(24)
        sessions[token] = username
        response.set_cookie("session", token, httponly=True)
        return {"username": username, "token": token}

    @app.post("/signup")
    async def signup(request: Request, response: Response):
        body = await request.json()
        if not body.get("username") or not body.get("password"):
            raise HTTPException(status_code=400, detail="username and password required")
        if not store.add_user(body["username"], body["password"]):
            raise HTTPException(status_code=409, detail="username already exists")
        return _login(body["username"], response)

    @app.post("/login")
    async def login(request: Request, response: Response):
        body = await request.json()
        if not store.check_user(body.get("username", ""), body.get("password", "")):
            raise HTTPException(status_code=401, detail="wrong username or password")
        return _login(body["username"], response)

    @app.get("/logout")
    def logout(request: Request):
        sessions.pop(request.cookies.get("session", ""), None)
        return {"message": "logged out"}

    @app.get("/", response_class=HTMLResponse)
    def index():
        return PAGE.replace("__INDEX__", "0").replace("__NEXT__", "1")

    @app.get("/instances/{index}", response_class=HTMLResponse)
    def instance_page(index: int):
        return PAGE.replace("__INDEX__", str(index)).replace("__NEXT__", str(min(index + 1, len(instances) - 1)))

    @app.get("/api/model-outputs/{index}")
    def model_outputs(index: int):
        if not 0 <= index < len(instances):
            return {"error": "Index out of range"}
        completions = list(instances[index]["completions"])
        rng.shuffle(completions)   # the annotator must not learn which side is which model
        return {"prompt": instances[index]["prompt"], "completions": completions}

    def _record(body: dict, evaluator: str, judged: bool) -> dict:
        idx = int(body["index"])
        if not 0 <= idx < len(instances):
            raise HTTPException(status_code=400, detail="index out of range")
        rec = {f: body.get(f, "") for f in FIELDS}
        rec.update(instance_index=idx, instance_id=str(instances[idx]["id"]), evaluator=evaluator,
                   timestamp=time.strftime("%Y-%m-%d %H:%M:%S", time.localtime()))
        if judged:
            rec.update(instance_quality="", comment="")
        else:
            rec.update(completion_a_is_acceptable="", completion_b_is_acceptable="", preference="")
        return rec

    @app.post("/api/submit-evaluation")
    async def submit_evaluation(request: Request):
        store.add_record(_record(await request.json(), user_of(request), judged=True))
        return {"message": "Evaluation data submitted successfully"}

    @app.post("/api/submit-feedback")
    async def submit_feedback(request: Request):
        store.add_record(_record(await request.json(), user_of(request), judged=False))
        return {"message": "Feedback submitted successfully"}

    @app.get("/summary")
    def summary(request: Request):
        user_of(request)
        return summarize(store.records(), store.users(), len(instances))

    return app


def export_records(db_path: str, out_path: str) -> int:
    """Dump the annotation table to JSONL or, by extension, CSV (``human_eval/export_db.py`` writes Excel)."""
    recs = Store(db_path).records()
    if out_path.endswith(".csv"):
        import csv

        with open(out_path, "w", newline="") as fh:
            w = csv.DictWriter(fh, fieldnames=FIELDS)
            w.writeheader()
            w.writerows(recs)
    else:
        with open(out_path, "w") as fh:
            for r in recs:
                fh.write(json.dumps(r) + "\n")
    return len(recs)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--comparison_data_path", required=True)
    ap.add_argument("--db", default="human_eval.sqlite3")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=5001)
    ap.add_argument("--export", default=None, help="write the records to this .jsonl / .csv file and exit")
    args = ap.parse_args(argv)
    if args.export:
        print(f"exported {export_records(args.db, args.export)} records to {args.export}")
        return
    import uvicorn

    uvicorn.run(create_app(load_instances(args.comparison_data_path), args.db), host=args.host, port=args.port)


if __name__ == "__main__":
    main()
