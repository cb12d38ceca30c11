"""Control panel: profile → command mapping, start/stop through an injected spawner, and the
JSON API with bearer-token protection (served on an ephemeral local port)."""
import json
import sys
import threading
import urllib.error
import urllib.request
from http.server import ThreadingHTTPServer

from control_panel.panel import Runner, command_for, make_handler


def test_profile_commands():
    argv = command_for("p", {"model": "qwen3-4b", "tp": 8, "port": 2000, "flags": ["--dummy-weight"]})
    assert argv[1:4] == ["-m", "minisglang_rdna4_b200", "--model"] and "--tp-size" in argv and argv[-1] == "--dummy-weight"
    assert command_for("svc", {"mode": "compose"}) == ["docker", "compose", "--profile", "svc", "up", "-d"]


def test_api_start_stop_and_auth(tmp_path):
    cfg = {"token": "s3cret", "profiles": {"sleepy": {"model": "tiny", "flags": []}}}
    import subprocess

    def spawn(argv, **kw):  # a stand-in process instead of a server launch
        return subprocess.Popen([sys.executable, "-c", "import time; time.sleep(60)"],
                                **{k: v for k, v in kw.items() if k != "cwd"})

    runner = Runner(cfg, log_dir=tmp_path, spawn=spawn)
    httpd = ThreadingHTTPServer(("127.0.0.1", 0), make_handler(runner))
    port = httpd.server_address[1]
    threading.Thread(target=httpd.serve_forever, daemon=True).start()

    def call(path, method="GET", token="s3cret"):
        req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", method=method)
        if token:
            req.add_header("Authorization", f"Bearer {token}")
        with urllib.request.urlopen(req, timeout=10) as r:
            return json.loads(r.read())

    try:
        try:
            call("/api/profiles", token="")
            assert False, "unauthenticated call must be refused"
        except urllib.error.HTTPError as e:
            assert e.code == 401
        assert call("/api/profiles")["sleepy"]["state"] == "stopped"
        assert call("/api/up?name=sleepy", "POST")["result"] == "started"
        assert call("/api/profiles")["sleepy"]["state"] == "running"
        assert call("/api/up?name=sleepy", "POST")["result"] == "already running"
        assert call("/api/down?name=sleepy", "POST")["result"] == "stopped"
        assert call("/api/profiles")["sleepy"]["state"] == "stopped"
        try:
            call("/api/up?name=nope", "POST")
            assert False
        except urllib.error.HTTPError as e:
            assert e.code == 404
    finally:
        runner.down("sleepy")
        httpd.shutdown()
