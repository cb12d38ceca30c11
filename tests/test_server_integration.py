"""Real process tree on CPU: frontend + tokenizer worker + scheduler over ZMQ, tiny random model,
byte tokenizer. Checks a completion, a streamed chat completion, /metrics, and that the server
survives an over-long prompt."""
import json
import os
import signal
import socket
import subprocess
import sys
import time

import pytest
import requests

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture(scope="module")
def server():
    port = _free_port()
    env = dict(os.environ, PYTHONPATH=ROOT, MSGL_LOG_LEVEL="WARNING")
    proc = subprocess.Popen(
        [sys.executable, "-m", "minisglang_rdna4_b200", "--model", "tiny-llama", "--device", "cpu", "--dummy-weight",
         "--port", str(port), "--num-pages", "128", "--max-running-requests", "8", "--max-seq-len-override", "512"],
        env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, start_new_session=True)
    url = f"http://127.0.0.1:{port}"
    deadline = time.time() + 180
    ok = False
    while time.time() < deadline:
        if proc.poll() is not None:
            break
        try:
            if requests.get(url + "/health", timeout=1).status_code == 200:
                ok = True
                break
        except requests.RequestException:
            time.sleep(0.5)
    if not ok:
        out = proc.stdout.read().decode() if proc.poll() is not None else ""
        os.killpg(proc.pid, signal.SIGKILL) if proc.poll() is None else None
        pytest.fail(f"server did not come up: {out[-2000:]}")
    yield url
    os.killpg(proc.pid, signal.SIGTERM)
    try:
        proc.wait(timeout=20)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)


def test_completion_roundtrip(server):
    r = requests.post(server + "/v1/completions", json={"prompt": "hello", "max_tokens": 5, "ignore_eos": True},
                      timeout=120)
    body = r.json()
    assert r.status_code == 200, body
    assert body["usage"]["completion_tokens"] == 5 and body["usage"]["prompt_tokens"] == 5
    assert body["choices"][0]["finish_reason"] == "length"


def test_streaming_chat_and_metrics(server):
    with requests.post(server + "/v1/chat/completions", stream=True, timeout=120,
                       json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "stream": True,
                             "ignore_eos": True, "stream_options": {"include_usage": True}}) as r:
        lines = [ln.decode()[6:] for ln in r.iter_lines() if ln.startswith(b"data: ")]
    assert lines[-1] == "[DONE]"
    usage = [json.loads(x)["usage"] for x in lines[:-1] if "usage" in json.loads(x)]
    assert usage and usage[-1]["completion_tokens"] == 4
    time.sleep(1.5)
    metrics = requests.get(server + "/metrics", timeout=10).text
    assert "minisgl_requests_finished_total" in metrics and "minisgl_generation_tokens_total" in metrics


def test_overlong_prompt_is_an_error_reply_and_server_stays_up(server):
    r = requests.post(server + "/v1/completions", json={"prompt": "x" * 2000, "max_tokens": 2}, timeout=120)
    assert r.status_code == 400
    r = requests.post(server + "/v1/completions", json={"prompt": "ok", "max_tokens": 2, "ignore_eos": True},
                      timeout=120)
    assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 2
