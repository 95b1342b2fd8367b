"""Visualisation-lab server: loopback HTTP with `/api/status` and `/api/trace`, one
inference worker (requests are serialised by a lock), optional static UI directory
(`summa-llm/src/lab.rs:244-340`)."""
from __future__ import annotations

import json
import os
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from urllib.parse import parse_qs, urlparse

from .generate import SamplingConfig, TextGenerator
from .trace import MAX_TOKENS, TraceGeneration, capture_bundle


DEFAULT_UI = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lab_ui")
_CONTENT_TYPES = {".html": "text/html; charset=utf-8", ".js": "text/javascript; charset=utf-8",
                  ".css": "text/css; charset=utf-8", ".json": "application/json"}


def make_server(model, tokenizer, host="127.0.0.1", port=0, static_dir=DEFAULT_UI, metrics_path=None):
    """`static_dir`: directory of the browser UI (default: the UI shipped in `summa_b200/lab_ui`;
    None serves the API only)."""
    if host not in ("127.0.0.1", "localhost", "::1"):
        raise ValueError("the lab server binds to loopback only")
    lock = threading.Lock()

    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def _json(self, code, obj):
            body = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_GET(self):
            u = urlparse(self.path)
            if u.path == "/api/status":
                return self._json(200, {"model": model.cfg.name, "parameters": model.cfg.estimated_params(),
                                        "max_trace_tokens": MAX_TOKENS, "ready": True})
            if u.path == "/api/trace":
                qs = parse_qs(u.query)
                prompt = qs.get("prompt", [""])[0]
                if not prompt:
                    return self._json(400, {"error": "missing prompt"})
                ids = tokenizer.encode(prompt, False)
                if not ids:
                    return self._json(400, {"error": "empty prompt"})
                try:
                    new = max(0, min(int(qs.get("max_new_tokens", ["8"])[0]), 64))
                    temp = float(qs.get("temperature", ["0"])[0])
                    seed = int(qs.get("seed", ["0"])[0])
                except ValueError:
                    return self._json(400, {"error": "max_new_tokens, temperature and seed must be numbers"})
                with lock:                      # one inference at a time, as the reference's single worker thread
                    cont = (TextGenerator(model, tokenizer).generate_ids(
                        ids, SamplingConfig(max_new_tokens=new, temperature=temp, seed=seed)) if new > 0 else [])
                    try:
                        bundle = capture_bundle(model, tokenizer, prompt, len(ids), ids + cont,
                                                TraceGeneration(new, temp, None, 1.0, seed, True),
                                                metrics_path if (metrics_path and os.path.exists(metrics_path)) else None)
                    except ValueError as e:
                        return self._json(400, {"error": str(e)})
                return self._json(200, bundle)
            if static_dir:
                rel = u.path.lstrip("/") or "model-lab.html"
                full = os.path.realpath(os.path.join(static_dir, rel))
                if full.startswith(os.path.realpath(static_dir) + os.sep) and os.path.isfile(full):
                    data = open(full, "rb").read()
                    self.send_response(200)
                    self.send_header("Content-Type", _CONTENT_TYPES.get(os.path.splitext(full)[1],
                                                                        "application/octet-stream"))
                    self.send_header("Content-Length", str(len(data)))
                    self.end_headers()
                    self.wfile.write(data)
                    return
            self._json(404, {"error": "not found"})

    return ThreadingHTTPServer((host, port), Handler)
