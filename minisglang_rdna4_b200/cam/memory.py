"""Product-key fact store.

A fact is ``(subject, prompt, object)``: "when the text is about *subject* and asks *prompt*, the
answer is *object*". The reference keeps such facts in a learned product-key memory that is tapped
from the model's hidden states (python/minisgl/cam/memory.py:440). This build keeps the same
*edit plane* (remember / ask / list / delete / undo, namespaces, persistence) over a retrieval
store, and applies a fact at read time by placing it in front of the prompt; it does not tap
hidden states.

Keys are product keys: a text is hashed into two independent sub-key spaces (character-trigram
feature hashing, ``SUB`` buckets each, L2-normalised); a stored fact's score against a query is the
product of the two sub-space cosine similarities, so a lookup touches only the facts that share a
bucket with the query in both halves. Everything is deterministic and dependency-free.
"""
from __future__ import annotations

import json
import math
import os
import threading
import time
import zlib
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Tuple

SUB = 256  # buckets per sub-key space


@dataclass
class Fact:
    subject: str
    prompt: str
    object: str
    created: float = field(default_factory=time.time)


def _subkey(text: str, salt: int) -> Dict[int, float]:
    """Sparse L2-normalised feature vector of the character trigrams of ``text``."""
    t = " " + " ".join(text.lower().split()) + " "
    vec: Dict[int, float] = {}
    for i in range(len(t) - 2):
        h = zlib.crc32(t[i:i + 3].encode("utf-8"), salt) % SUB
        vec[h] = vec.get(h, 0.0) + 1.0
    norm = math.sqrt(sum(v * v for v in vec.values())) or 1.0
    return {k: v / norm for k, v in vec.items()}


def _cos(a: Dict[int, float], b: Dict[int, float]) -> float:
    if len(a) > len(b):
        a, b = b, a
    return sum(v * b.get(k, 0.0) for k, v in a.items())


class CamMemory:
    """Namespaced fact store with an undo log and JSON persistence."""

    def __init__(self, path: Optional[str] = None, max_namespaces: int = 0) -> None:
        self.path = path
        self.max_namespaces = max_namespaces
        self._facts: Dict[str, Dict[str, Fact]] = {}            # namespace -> subject -> fact
        self._keys: Dict[Tuple[str, str], Tuple[Dict[int, float], Dict[int, float]]] = {}
        self._undo: Dict[str, List[Tuple[str, str, Optional[Fact]]]] = {}  # (op, subject, previous)
        self._lock = threading.Lock()
        if path and os.path.exists(path):
            self._load()

    # ---- persistence ----
    def _load(self) -> None:
        with open(self.path) as fh:
            raw = json.load(fh)
        for ns, facts in raw.get("namespaces", {}).items():
            for f in facts:
                self._put(ns, Fact(**f))

    def _save(self) -> None:
        if not self.path:
            return
        tmp = self.path + ".tmp"
        with open(tmp, "w") as fh:
            json.dump({"namespaces": {ns: [asdict(f) for f in facts.values()]
                                      for ns, facts in self._facts.items()}}, fh)
        os.replace(tmp, self.path)

    # ---- internals ----
    def _put(self, ns: str, fact: Fact) -> None:
        self._facts.setdefault(ns, {})[fact.subject] = fact
        text = fact.subject + " " + fact.prompt
        self._keys[(ns, fact.subject)] = (_subkey(text, 1), _subkey(text, 2))

    # ---- edit plane ----
    def namespaces(self) -> List[str]:
        with self._lock:
            return sorted(self._facts)

    def remember(self, subject: str, prompt: str, obj: str, namespace: str = "default") -> Fact:
        subject, obj = subject.strip(), obj.strip()
        if not subject or not obj:
            raise ValueError("subject and object must be non-empty")
        with self._lock:
            if (namespace not in self._facts and self.max_namespaces
                    and len(self._facts) >= self.max_namespaces):
                raise PermissionError("namespace limit reached")
            prev = self._facts.get(namespace, {}).get(subject)
            fact = Fact(subject, prompt.strip(), obj)
            self._put(namespace, fact)
            self._undo.setdefault(namespace, []).append(("remember", subject, prev))
            self._save()
            return fact

    def forget(self, subject: str, namespace: str = "default") -> bool:
        with self._lock:
            prev = self._facts.get(namespace, {}).pop(subject.strip(), None)
            if prev is None:
                return False
            self._keys.pop((namespace, prev.subject), None)
            self._undo.setdefault(namespace, []).append(("forget", prev.subject, prev))
            self._save()
            return True

    def undo(self, namespace: str = "default") -> Optional[str]:
        """Revert the namespace's most recent edit; returns a description or None."""
        with self._lock:
            log = self._undo.get(namespace) or []
            if not log:
                return None
            op, subject, prev = log.pop()
            if prev is None:
                self._facts.get(namespace, {}).pop(subject, None)
                self._keys.pop((namespace, subject), None)
            else:
                self._put(namespace, prev)
            self._save()
            return f"undid {op} of {subject!r}"

    def facts(self, namespace: str = "default") -> List[Fact]:
        with self._lock:
            return list(self._facts.get(namespace, {}).values())

    # ---- read plane ----
    def lookup(self, text: str, namespace: str = "default", top_k: int = 3, threshold: float = 0.12
               ) -> List[Tuple[float, Fact]]:
        qa, qb = _subkey(text, 1), _subkey(text, 2)
        out: List[Tuple[float, Fact]] = []
        with self._lock:
            for subject, fact in self._facts.get(namespace, {}).items():
                ka, kb = self._keys[(namespace, subject)]
                score = _cos(qa, ka) * _cos(qb, kb)
                if fact.subject.lower() in text.lower():
                    score = max(score, 0.5) + 0.5 * score  # an explicit mention always retrieves
                if score >= threshold:
                    out.append((score, fact))
        out.sort(key=lambda p: -p[0])
        return out[:top_k]

    def augment(self, prompt: str, namespace: str = "default", subject: Optional[str] = None) -> str:
        """The prompt with the retrieved facts stated in front of it (unchanged when none apply)."""
        hits = self.lookup(prompt if subject is None else subject + " " + prompt, namespace)
        if not hits:
            return prompt
        lines = [f"{f.subject}: {f.prompt} {f.object}".replace("  ", " ") for _, f in hits]
        return "Known facts:\n" + "\n".join("- " + ln for ln in lines) + "\n\n" + prompt
