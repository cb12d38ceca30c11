"""Control panel: a small web UI + JSON API that starts and stops named serving profiles.

A profile is a named launch recipe (model, parallelism, port, extra flags, environment) kept in
``profiles.json`` next to this file (or the path in ``$MSGL_PANEL_PROFILES``). The panel can run a
profile in two ways:

* ``process`` (default): ``python -m minisglang_rdna4_b200 ...`` as a child process group, logs
  captured to ``logs/<profile>.log``;
* ``compose``: ``docker compose --profile <name> up -d`` / ``down`` in the directory that holds the
  compose file, which is how the reference's panel drives its deployments
  (control-panel/server.py: compose profiles, optional bearer token, per-profile env defaults).

Standard library only. ``python -m control_panel.panel --port 7070`` serves ``/`` (HTML),
``GET /api/profiles``, ``POST /api/up?name=``, ``POST /api/down?name=``, ``GET /api/log?name=``.
When ``token`` is set in the configuration every ``/api`` call needs ``Authorization: Bearer``.
"""
from __future__ import annotations

import argparse
import html
import json
import os
import shlex
import signal
import subprocess
import sys
import threading
import time
import urllib.parse
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from pathlib import Path
from typing import Callable, Dict, List, Optional

HERE = Path(__file__).resolve().parent
DEFAULT_PROFILES = {
    "token": "",
    "profiles": {
        "qwen3-4b-mxfp4": {"model": "qwen3-4b", "flags": ["--dummy-weight", "--quantization", "mxfp4",
                                                          "--kv-cache-dtype", "fp8"], "tp": 1, "port": 1919},
        "qwen3-4b-mxfp4-tp8": {"model": "qwen3-4b", "flags": ["--dummy-weight", "--quantization", "mxfp4",
                                                              "--kv-cache-dtype", "fp8"], "tp": 8, "port": 1919},
    },
}


def load_config(path: Optional[str] = None) -> dict:
    p = Path(path or os.environ.get("MSGL_PANEL_PROFILES") or (HERE / "profiles.json"))
    if p.exists():
        return json.loads(p.read_text())
    return json.loads(json.dumps(DEFAULT_PROFILES))


def command_for(name: str, prof: dict) -> List[str]:
    """The argv that brings a profile up."""
    if prof.get("mode") == "compose":
        return ["docker", "compose", "--profile", name, "up", "-d"]
    argv = [sys.executable, "-m", "minisglang_rdna4_b200", "--model", str(prof["model"]),
            "--tp-size", str(int(prof.get("tp", 1))), "--port", str(int(prof.get("port", 1919)))]
    if int(prof.get("dp", 1)) > 1:
        argv += ["--dp-size", str(int(prof["dp"]))]
    return argv + [str(f) for f in prof.get("flags", [])]


class Runner:
    """Starts / stops profiles. ``spawn`` is injectable so tests run without docker or a GPU."""

    def __init__(self, config: dict, log_dir: Optional[Path] = None,
                 spawn: Optional[Callable[..., subprocess.Popen]] = None) -> None:
        self.config = config
        self.log_dir = Path(log_dir or (HERE / "logs"))
        self.log_dir.mkdir(parents=True, exist_ok=True)
        self._spawn = spawn or subprocess.Popen
        self._procs: Dict[str, subprocess.Popen] = {}
        self._lock = threading.Lock()

    def profiles(self) -> Dict[str, dict]:
        out = {}
        for name, prof in self.config.get("profiles", {}).items():
            out[name] = dict(prof, state=self.state(name), command=shlex.join(command_for(name, prof)))
        return out

    def state(self, name: str) -> str:
        with self._lock:
            proc = self._procs.get(name)
        if proc is None:
            return "stopped"
        return "running" if proc.poll() is None else f"exited({proc.returncode})"

    def up(self, name: str) -> str:
        prof = self.config.get("profiles", {}).get(name)
        if prof is None:
            raise KeyError(name)
        if self.state(name) == "running":
            return "already running"
        env = dict(os.environ, **{k: str(v) for k, v in prof.get("env", {}).items()})
        log = open(self.log_dir / f"{name}.log", "ab")
        proc = self._spawn(command_for(name, prof), stdout=log, stderr=subprocess.STDOUT, env=env,
                           cwd=prof.get("cwd") or None, start_new_session=True)
        with self._lock:
            self._procs[name] = proc
        return "started"

    def down(self, name: str, grace_s: float = 10.0) -> str:
        prof = self.config.get("profiles", {}).get(name)
        if prof is None:
            raise KeyError(name)
        if prof.get("mode") == "compose":
            self._spawn(["docker", "compose", "--profile", name, "down"], cwd=prof.get("cwd") or None).wait()
        with self._lock:
            proc = self._procs.pop(name, None)
        if proc is None or proc.poll() is not None:
            return "not running"
        try:  # the child leads its own process group: stop exactly that group
            os.killpg(proc.pid, signal.SIGTERM)
        except (ProcessLookupError, PermissionError):
            proc.terminate()
        deadline = time.monotonic() + grace_s
        while proc.poll() is None and time.monotonic() < deadline:
            time.sleep(0.05)
        if proc.poll() is None:
            try:
                os.killpg(proc.pid, signal.SIGKILL)
            except (ProcessLookupError, PermissionError):
                proc.kill()
        return "stopped"

    def log_tail(self, name: str, max_bytes: int = 16384) -> str:
        p = self.log_dir / f"{name}.log"
        if not p.exists():
            return ""
        data = p.read_bytes()
        return data[-max_bytes:].decode("utf-8", "replace")


PAGE = """<!doctype html><meta charset="utf-8"><title>serving profiles</title>
<style>body{font-family:sans-serif;margin:2em}td,th{padding:.3em .8em;text-align:left}code{font-size:85%}</style>
<h1>Serving profiles</h1><table><tr><th>profile</th><th>state</th><th>command</th><th></th></tr>%s</table>
<script>async function act(a,n){await fetch('/api/'+a+'?name='+encodeURIComponent(n),{method:'POST'});location.reload()}</script>"""


def make_handler(runner: Runner):
    token = runner.config.get("token") or ""

    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *args) -> None:  # quiet
            pass

        def _send(self, code: int, body, ctype: str = "application/json") -> None:
            data = body if isinstance(body, bytes) else (json.dumps(body) if ctype.endswith("json") else body).encode()
            self.send_response(code)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def _authorised(self) -> bool:
            return not token or self.headers.get("Authorization", "") == f"Bearer {token}"

        def _route(self, method: str) -> None:
            url = urllib.parse.urlparse(self.path)
            q = urllib.parse.parse_qs(url.query)
            name = (q.get("name") or [""])[0]
            if url.path == "/" and method == "GET":
                rows = ""
                for n, p in runner.profiles().items():
                    en = html.escape(n, quote=True)
                    rows += ("<tr><td>%s</td><td>%s</td><td><code>%s</code></td><td>"
                             "<button onclick='act(&quot;up&quot;,&quot;%s&quot;)'>up</button> "
                             "<button onclick='act(&quot;down&quot;,&quot;%s&quot;)'>down</button></td></tr>"
                             % (en, html.escape(p["state"]), html.escape(p["command"]), en, en))
                return self._send(200, PAGE % rows, "text/html")
            if not url.path.startswith("/api/"):
                return self._send(404, {"error": "not found"})
            if not self._authorised():
                return self._send(401, {"error": "unauthorised"})
            try:
                if url.path == "/api/profiles" and method == "GET":
                    return self._send(200, runner.profiles())
                if url.path == "/api/log" and method == "GET":
                    return self._send(200, {"name": name, "log": runner.log_tail(name)})
                if url.path == "/api/up" and method == "POST":
                    return self._send(200, {"name": name, "result": runner.up(name)})
                if url.path == "/api/down" and method == "POST":
                    return self._send(200, {"name": name, "result": runner.down(name)})
            except KeyError:
                return self._send(404, {"error": f"unknown profile {name!r}"})
            return self._send(405, {"error": "method not allowed"})

        def do_GET(self) -> None:
            self._route("GET")

        def do_POST(self) -> None:
            self._route("POST")

    return Handler


def serve(host: str = "127.0.0.1", port: int = 7070, config_path: Optional[str] = None) -> None:
    runner = Runner(load_config(config_path))
    httpd = ThreadingHTTPServer((host, port), make_handler(runner))
    print(f"control panel on http://{host}:{port}", flush=True)
    try:
        httpd.serve_forever()
    finally:
        for name in list(runner.profiles()):
            runner.down(name)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=7070)
    ap.add_argument("--profiles", default=None)
    a = ap.parse_args()
    serve(a.host, a.port, a.profiles)
