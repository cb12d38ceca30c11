"""Associative memory: product-key retrieval, edit plane with undo and persistence, and the REST
plane with per-namespace bearer tokens."""
import json

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
