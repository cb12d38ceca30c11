"""Baked checkpoints: a rank's weights as they stand after loading, in one flat file
(python/minisgl/weights/bake.py:227, python/minisgl/weights/stage_b.py:378).

Loading a Hugging Face checkpoint is mostly host work per tensor: parse, slice for the
tensor-parallel rank, merge q/k/v and gate/up, stack thousands of expert matrices. The result
does not change between boots. Stage A writes it once, per rank: every persistent tensor of the
model (its state dict as it is between ``load_weights`` and ``post_load``, plus the fp8 expert
stacks the loader parks in ``_raw_fp8``) goes into ``rank<r>.bin`` at a 4096-byte boundary, and
``rank<r>.json`` records name, dtype, shape, offset and a checksum per tensor and a fingerprint
of everything the layout depends on (model config, tensor- / expert-parallel geometry, dtype,
quantisation, the checkpoint files' names, sizes and modification times). Stage B, on a later
boot with the same fingerprint, streams the file through a ring of page-locked chunks (reads on
a small thread pool, ``O_DIRECT`` when the platform allows, each chunk uploaded while the next is
being read) straight into the model's tensors. A missing file or a different fingerprint means
the ordinary loader runs and the bake is written again.

The device-side packing of ``post_load`` (MXFP4 / fp8 expert encodings) still runs after either
path: it is a few kernels, and keeping it out of the file keeps the file independent of kernel
layouts.
"""
from __future__ import annotations

import hashlib
import json
import os
import zlib
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np
import torch

from ..utils import init_logger

logger = init_logger(__name__)

ALIGN = 4096
CHUNK = 64 << 20
FORMAT = 1
_DTYPES = {str(d): d for d in (torch.float32, torch.float16, torch.bfloat16, torch.int8, torch.uint8, torch.int16,
                               torch.int32, torch.int64, torch.bool, torch.float8_e4m3fn, torch.float8_e5m2)}


def _round_up(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def fingerprint(model_config, model_path: Optional[str], dtype, tp_rank: int, tp_size: int, ep: str = "") -> str:
    """Digest of everything the baked layout depends on."""
    h = hashlib.sha256()
    h.update(f"format {FORMAT}|tp {tp_rank}/{tp_size}|ep {ep}|dtype {dtype}|".encode())
    h.update(repr(model_config).encode())
    if model_path and os.path.isdir(model_path):
        for name in sorted(os.listdir(model_path)):
            if name.endswith((".safetensors", ".json")):
                st = os.stat(os.path.join(model_path, name))
                h.update(f"{name}:{st.st_size}:{int(st.st_mtime)}|".encode())
    return h.hexdigest()


def _entries(model) -> Iterator[Tuple[str, object, str, Optional[int]]]:
    """``(name, owner, attribute, tuple index)`` of every tensor that belongs in the file."""
    for name, _tensor, owner, attr in model.named_parameters():
        yield name, owner, attr, None

    def walk(obj, prefix):
        raw = getattr(obj, "_raw_fp8", None)
        if raw is not None:
            for i in range(len(raw)):
                yield f"{prefix}_raw_fp8.{i}", obj, "_raw_fp8", i
        for cname, child in obj._children():
            yield from walk(child, prefix + cname + ".")

    yield from walk(model, "")


def paths(directory: str, rank: int) -> Tuple[str, str]:
    return os.path.join(directory, f"rank{rank}.bin"), os.path.join(directory, f"rank{rank}.json")


def write_bake(model, directory: str, rank: int, print_: str) -> int:
    """Stage A. Returns the bytes written. The index appears last (and atomically), so a crash in
    the middle leaves no bake that a later boot would trust."""
    os.makedirs(directory, exist_ok=True)
    data_path, index_path = paths(directory, rank)
    index: List[Dict] = []
    offset = 0
    with open(data_path + ".tmp", "wb") as fh:
        for name, owner, attr, i in _entries(model):
            t = getattr(owner, attr)
            t = t[i] if i is not None else t
            if t.device.type == "meta":
                raise ValueError(f"{name} has no data to bake")
            raw = t.detach().cpu().contiguous()
            buf = raw.view(torch.uint8).reshape(-1).numpy() if raw.numel() else np.zeros(0, dtype=np.uint8)
            fh.seek(offset)
            fh.write(buf.tobytes())
            index.append({"name": name, "dtype": str(raw.dtype), "shape": list(raw.shape), "offset": offset,
                          "nbytes": int(buf.size), "crc32": zlib.crc32(buf.tobytes()) & 0xFFFFFFFF})
            offset = _round_up(offset + int(buf.size))
        fh.truncate(offset)
    os.replace(data_path + ".tmp", data_path)
    with open(index_path + ".tmp", "w") as fh:
        json.dump({"format": FORMAT, "fingerprint": print_, "bytes": offset, "tensors": index}, fh)
    os.replace(index_path + ".tmp", index_path)
    return offset


def read_index(directory: str, rank: int, print_: str) -> Optional[Dict]:
    data_path, index_path = paths(directory, rank)
    if not (os.path.isfile(data_path) and os.path.isfile(index_path)):
        return None
    try:
        with open(index_path) as fh:
            index = json.load(fh)
    except (OSError, ValueError):
        return None
    if index.get("format") != FORMAT or index.get("fingerprint") != print_:
        return None
    if os.path.getsize(data_path) < int(index.get("bytes", 0)):
        return None
    return index


class _ChunkReader:
    """Positional reads of one file into aligned host chunks, ``depth`` of them in flight."""

    def __init__(self, path: str, pin: bool, depth: int = 3, chunk: int = CHUNK) -> None:
        self.chunk = chunk
        self.direct = False
        self.fd = -1
        if hasattr(os, "O_DIRECT"):
            try:
                self.fd = os.open(path, os.O_RDONLY | os.O_DIRECT)
                self.direct = True
            except OSError:
                self.fd = -1
        if self.fd < 0:
            self.fd = os.open(path, os.O_RDONLY)
        # one slab cut into chunks; an unpinned slab is over-allocated so that the chunks can be aligned
        slab = torch.empty(depth * chunk + ALIGN, dtype=torch.uint8, pin_memory=pin)
        shift = (-slab.data_ptr()) % ALIGN
        self.bufs = [slab[shift + i * chunk: shift + (i + 1) * chunk] for i in range(depth)]
        self.pool = ThreadPoolExecutor(max_workers=depth, thread_name_prefix="bake-read")

    def _read(self, buf: torch.Tensor, offset: int, nbytes: int) -> int:
        want = _round_up(nbytes) if self.direct else nbytes
        view = memoryview(buf.numpy())[:want]
        got = 0
        while got < nbytes:
            n = os.preadv(self.fd, [view[got:]], offset + got)
            if n <= 0:
                break
            got += n
        if got < nbytes:
            raise IOError(f"short read at {offset}: {got} of {nbytes} bytes")
        return nbytes

    def stream(self, spans: List[Tuple[int, int]]):
        """Yield ``(index of the span, host view)`` in order; span i is ``(offset, nbytes)`` with an
        aligned offset and at most one chunk long. The next spans are read while one is consumed."""
        depth = len(self.bufs)
        jobs = {}
        for i in range(min(depth, len(spans))):
            jobs[i] = self.pool.submit(self._read, self.bufs[i % depth], *spans[i])
        for i in range(len(spans)):
            n = jobs.pop(i).result()
            yield i, self.bufs[i % depth][:n]
            nxt = i + depth
            if nxt < len(spans):
                # the consumer is done with this buffer when it asks for the next item
                jobs[nxt] = self.pool.submit(self._read, self.bufs[nxt % depth], *spans[nxt])

    def close(self) -> None:
        self.pool.shutdown(wait=True)
        if self.fd >= 0:
            os.close(self.fd)
            self.fd = -1


def load_bake(model, directory: str, rank: int, print_: str, device, verify: bool = False) -> Optional[int]:
    """Stage B. Fills the model from the rank's file; returns the bytes read, or ``None`` when there
    is no bake for this fingerprint (nothing is touched then). ``verify`` checks every tensor's
    checksum on the host before it is uploaded."""
    index = read_index(directory, rank, print_)
    if index is None:
        return None
    targets = {name: (owner, attr) for name, _t, owner, attr in model.named_parameters()}
    in_file = {e["name"] for e in index["tensors"]}
    missing = [n for n in targets if n not in in_file]
    if missing:
        logger.warning("baked checkpoint lacks %d tensors (%s ...): loading from the checkpoint instead",
                       len(missing), missing[0])
        return None
    modules: Dict[str, object] = {}

    def walk(obj, prefix):
        modules[prefix.rstrip(".")] = obj
        for cname, child in obj._children():
            walk(child, prefix + cname + ".")

    walk(model, "")
    device = torch.device(device)
    cuda = device.type == "cuda"
    reader = _ChunkReader(paths(directory, rank)[0], pin=cuda)
    spans, owners = [], []                       # every tensor in pieces of at most one chunk
    for e in index["tensors"]:
        for done in range(0, e["nbytes"], reader.chunk):
            spans.append((e["offset"] + done, min(reader.chunk, e["nbytes"] - done)))
            owners.append((e, done))
    staged: Dict[str, torch.Tensor] = {e["name"]: torch.empty(e["nbytes"], dtype=torch.uint8, device=device)
                                       for e in index["tensors"]}
    crcs: Dict[str, int] = {}
    try:
        for i, host in reader.stream(spans):
            e, done = owners[i]
            if verify:
                crcs[e["name"]] = zlib.crc32(host.numpy().tobytes(), crcs.get(e["name"], 0))
            staged[e["name"]][done:done + host.numel()].copy_(host, non_blocking=cuda)
            if cuda:
                # the reader refills this chunk as soon as the next one is asked for; later chunks are
                # already being read on the pool's threads while this upload runs
                torch.cuda.current_stream().synchronize()
    finally:
        reader.close()
    if verify:
        for e in index["tensors"]:
            if e["nbytes"] and (crcs.get(e["name"], 0) & 0xFFFFFFFF) != e["crc32"]:
                raise IOError(f"baked tensor {e['name']} fails its checksum")
    parked: Dict[str, Dict[int, torch.Tensor]] = {}
    for e in index["tensors"]:
        name, dtype = e["name"], _DTYPES[e["dtype"]]
        t = staged[name].view(dtype).view(e["shape"]) if e["nbytes"] else torch.empty(e["shape"], dtype=dtype,
                                                                                      device=device)
        if name in targets:
            owner, attr = targets[name]
            cur = getattr(owner, attr)
            if cur.device.type != "meta" and tuple(cur.shape) != tuple(t.shape):
                raise ValueError(f"{name}: baked shape {tuple(t.shape)} != model {tuple(cur.shape)}")
            setattr(owner, attr, t)
        elif "_raw_fp8." in name:                # an fp8 expert stack the loader parks until post_load
            head, _, idx = name.rpartition(".")
            parked.setdefault(head[: -len("_raw_fp8")].rstrip("."), {})[int(idx)] = t
    for owner_name, parts in parked.items():
        owner = modules.get(owner_name)
        if owner is not None:
            owner._raw_fp8 = tuple(parts[k] for k in sorted(parts))
    return int(index["bytes"])
