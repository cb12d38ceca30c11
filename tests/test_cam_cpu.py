"""Associative memory: product-key retrieval, edit plane with undo and persistence, and the REST
plane with per-namespace bearer tokens."""
import json

import pytest

from fastapi import FastAPI
from fastapi.testclient import TestClient

from minisglang_rdna4_b200.cam import CamMemory
from minisglang_rdna4_b200.server.cam_api import make_cam_router


def test_store_lookup_undo_persist(tmp_path):
    path = str(tmp_path / "cam.json")
    mem = CamMemory(path)
    mem.remember("Elowen Marsh", "lives in", "Tallinn")
    mem.remember("Project Heron", "is led by", "Dr. Okafor")
    mem.remember("Elowen Marsh", "lives in", "Porto")          # overwrite
    hits = mem.lookup("Where does Elowen Marsh live?")
    assert hits and hits[0][1].object == "Porto"
    assert mem.lookup("the weather on Mars") == []
    assert "Porto" in mem.augment("Where does Elowen Marsh live?") and mem.augment("2 + 2 = ?") == "2 + 2 = ?"
    assert mem.undo() == "undid remember of 'Elowen Marsh'"
    assert mem.lookup("Elowen Marsh home")[0][1].object == "Tallinn"
    assert mem.forget("Project Heron") and not mem.forget("Project Heron")
    assert mem.undo().startswith("undid forget")
    again = CamMemory(path)                                      # persisted across restarts
    assert {f.subject for f in again.facts()} == {"Elowen Marsh", "Project Heron"}


def test_rest_plane_with_namespace_tokens(monkeypatch):
    monkeypatch.setenv("MSGL_CAM_TOKENS", json.dumps({"tok-a": "alpha", "tok-admin": "*"}))
    app = FastAPI()
    app.include_router(make_cam_router(CamMemory()))
    c = TestClient(app)
    a = {"Authorization": "Bearer tok-a", "X-CAM-Namespace": "alpha"}
    assert c.post("/cam/remember", json={"subject": "Kite", "prompt": "colour", "object": "teal"}).status_code == 401
    assert c.post("/cam/remember", json={"subject": "Kite", "prompt": "colour", "object": "teal"}, headers=a).json() == \
        {"stored": True, "replaced": False}
    wrong = {"Authorization": "Bearer tok-a", "X-CAM-Namespace": "beta"}
    assert c.get("/cam/facts", headers=wrong).status_code == 403
    assert c.get("/cam/facts", headers=a).json() == [{"subject": "Kite", "prompt": "colour", "object": "teal"}]
    assert c.post("/cam/ask", json={"prompt": "what colour is the Kite?"}, headers=a).json()["text"] == "teal"
    admin = {"Authorization": "Bearer tok-admin", "X-CAM-Namespace": "beta"}
    c.post("/cam/remember", json={"subject": "Moss", "object": "green"}, headers=admin)
    assert c.get("/cam/namespaces", headers=admin).json() == ["alpha", "beta"]
    assert c.get("/cam/namespaces", headers=a).json() == ["alpha"]
    assert c.delete("/cam/facts/Kite", headers=a).json() == {"deleted": True}
    assert c.post("/cam/undo", headers=a).json()["undone"].startswith("undid forget")
    assert len(c.get("/cam/facts", headers=a).json()) == 1


def test_ambient_read_and_write_hooks_on_the_completion_endpoints(monkeypatch, tmp_path):
    """With the memory mounted, a request can state a fact (``cam_write``) and a later request gets
    it placed in front of its prompt (``cam_read``); both are off unless asked for or enabled by
    the server's environment."""
    from fastapi.testclient import TestClient

    from minisglang_rdna4_b200.config import ServerArgs
    from minisglang_rdna4_b200.message import TokenizeMsg, UserReply
    from minisglang_rdna4_b200.server.api_server import FrontendManager, create_app

    monkeypatch.setenv("MSGL_CAM", "1")
    monkeypatch.setenv("MSGL_CAM_PATH", str(tmp_path / "cam.json"))

    class Fake(FrontendManager):
        def __init__(self, args):
            super().__init__(args)
            self.sent = []

        async def send_one(self, msg):
            self.sent.append(msg)
            if isinstance(msg, TokenizeMsg):
                self.queues[msg.uid].put_nowait(UserReply(msg.uid, "ok", True, "stop", [1], prompt_tokens=3))

    args = ServerArgs(model_path="tiny-llama", served_model_name="tiny")
    mgr = Fake(args)
    c = TestClient(create_app(args, mgr, None))
    ask = {"messages": [{"role": "user", "content": "What is Zephyrina's mother tongue?"}]}
    c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "Zephyrina's mother tongue is Klingon."}]})
    assert c.get("/cam/facts").json() == []                                   # writing is off by default
    c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "Zephyrina's mother tongue is Klingon."}],
                                         "cam_write": True})
    assert c.get("/cam/facts").json() == [{"subject": "Zephyrina's mother tongue", "prompt": "is", "object": "Klingon"}]
    c.post("/v1/chat/completions", json=ask)                                  # read is off by default
    assert mgr.sent[-1].text == ask["messages"]
    c.post("/v1/chat/completions", json={**ask, "cam_read": True})
    sent = mgr.sent[-1].text
    assert sent[0]["role"] == "system" and "Klingon" in sent[0]["content"] and sent[1:] == ask["messages"]
    c.post("/v1/chat/completions", json={**ask, "cam_read": True}, headers={"X-CAM-Namespace": "other"})
    assert mgr.sent[-1].text == ask["messages"]                               # another namespace knows nothing
    monkeypatch.setenv("MSGL_CAM_AUTO", "1")
    c.post("/generate", json={"prompt": "Tell me about Zephyrina's mother tongue", "max_tokens": 4})
    assert "Klingon" in mgr.sent[-1].text and mgr.sent[-1].text.endswith("Tell me about Zephyrina's mother tongue")


def test_client_against_the_rest_plane(monkeypatch):
    """The client's calls, headers and error mapping against the mounted router (an in-process transport
    stands in for the socket)."""
    from minisglang_rdna4_b200.cam import CamClient, CamError

    monkeypatch.setenv("MSGL_CAM_TOKENS", json.dumps({"tok-a": "alpha", "tok-admin": "*"}))
    app = FastAPI()
    app.include_router(make_cam_router(CamMemory()))
    http = TestClient(app)

    def transport(method, path, headers, body):
        r = http.request(method, path, headers=headers, json=body)
        return r.status_code, r.json()

    alpha = CamClient(token="tok-a", namespace="alpha", transport=transport)
    assert alpha.remember("Kite", "teal", prompt="colour") == {"stored": True, "replaced": False}
    assert alpha.ask("what colour is the Kite?")["text"] == "teal"
    assert alpha.facts() == [{"subject": "Kite", "prompt": "colour", "object": "teal"}]
    with pytest.raises(CamError) as err:
        alpha.namespace("beta").facts()
    assert err.value.status == 403
    with pytest.raises(CamError) as err:
        CamClient(namespace="alpha", transport=transport).facts()
    assert err.value.status == 401
    admin = CamClient(token="tok-admin", namespace="beta", transport=transport)
    admin.remember("Moss bank", "green")
    assert admin.namespaces() == ["alpha", "beta"] and alpha.namespaces() == ["alpha"]
    assert admin.forget("Moss bank") is True and admin.facts() == []
    assert admin.undo().startswith("undid forget") and len(admin.facts()) == 1
