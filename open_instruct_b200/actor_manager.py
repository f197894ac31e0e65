"""Run-wide coordination state: the ``should_stop`` flag engines poll, queue depths, token and
timing statistics, and an optional HTTP status endpoint (``/api/status``) for a live dashboard
(cf. ``open_instruct/actor_manager.py``)."""

from __future__ import annotations

import collections
import json
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer


class ActorManager:
    def __init__(self, queues: dict | None = None, enable_dashboard: bool = False, port: int | None = None, window: int = 100):
        self._should_stop = False
        self._lock = threading.Lock()
        self.queues = queues or {}
        self.token_stats = collections.deque(maxlen=window)   # (time, prompt tokens, response tokens)
        self.training_times = collections.deque(maxlen=window)
        self.generation_times = collections.deque(maxlen=window)
        self.kv_cache_max_concurrency = None
        self.start_time = time.time()
        self._server = None
        if enable_dashboard:
            self._start_server(port or 0)

    def set_should_stop(self, flag: bool) -> None:
        with self._lock:
            self._should_stop = bool(flag)

    def should_stop(self) -> bool:
        with self._lock:
            return self._should_stop

    def report_token_statistics(self, prompt_tokens: int, response_tokens: int, generation_time: float) -> None:
        with self._lock:
            self.token_stats.append((time.time(), prompt_tokens, response_tokens))
            self.generation_times.append(generation_time)

    def report_training_step_time(self, seconds: float) -> None:
        with self._lock:
            self.training_times.append(seconds)

    def set_kv_cache_max_concurrency(self, n: int) -> None:
        self.kv_cache_max_concurrency = n

    def status(self) -> dict:
        with self._lock:
            ts = list(self.token_stats)
            span = (ts[-1][0] - ts[0][0]) if len(ts) > 1 else 0.0
            qs = {}
            for name, q in self.queues.items():
                try:
                    qs[name] = {"size": q.qsize(), "maxsize": getattr(q, "maxsize", 0)}
                except Exception:  # noqa: BLE001
                    qs[name] = {"size": None}
            return {
                "should_stop": self._should_stop,
                "uptime_s": time.time() - self.start_time,
                "queues": qs,
                "tokens_per_second": (sum(t[2] for t in ts) / span) if span > 0 else 0.0,
                "avg_training_step_s": sum(self.training_times) / len(self.training_times) if self.training_times else 0.0,
                "avg_generation_s": sum(self.generation_times) / len(self.generation_times) if self.generation_times else 0.0,
                "kv_cache_max_concurrency": self.kv_cache_max_concurrency,
            }

    def _start_server(self, port: int) -> None:
        mgr = self

        class H(BaseHTTPRequestHandler):
            def do_GET(self):  # noqa: N802
                if self.path.startswith("/api/status"):
                    body = json.dumps(mgr.status()).encode()
                    ctype = "application/json"
                else:
                    body = (b"<html><body><h3>open_instruct_b200</h3><pre id=s></pre><script>setInterval(()=>fetch('/api/status')"
                            b".then(r=>r.json()).then(j=>document.getElementById('s').textContent=JSON.stringify(j,null,2)),1000)"
                            b"</script></body></html>")
                    ctype = "text/html"
                self.send_response(200)
                self.send_header("Content-Type", ctype)
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def log_message(self, *a):
                pass

        self._server = ThreadingHTTPServer(("127.0.0.1", port), H)
        self.port = self._server.server_address[1]
        threading.Thread(target=self._server.serve_forever, daemon=True).start()

    def shutdown(self) -> None:
        if self._server is not None:
            self._server.shutdown()
            self._server = None
