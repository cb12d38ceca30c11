"""Process launcher (python/minisgl/server/launch.py:16-206): one scheduler process per
(dp_rank, tp_rank), one tokenizer/detokenizer process, a watchdog thread that brings the whole
server down when any child dies, then the HTTP frontend in this process."""
from __future__ import annotations

import dataclasses
import multiprocessing as mp
import os
import signal
import threading
import time
from typing import List

from ..config import ServerArgs
from ..utils import init_logger

logger = init_logger(__name__)


class ServedScheduler:
    """Scheduler + ZMQ I/O. Built lazily inside the child process."""

    @staticmethod
    def build(args: ServerArgs):
        from ..scheduler.io import SchedulerIOMixin
        from ..scheduler.scheduler import Scheduler

        class _Served(SchedulerIOMixin, Scheduler):
            def __init__(self, cfg):
                Scheduler.__init__(self, cfg)
                self.init_io()

        return _Served(args)


def _run_scheduler(args: ServerArgs, ready) -> None:
    init_logger(__name__, suffix=f"dp{args.dp_rank}|tp{args.tp_rank}")
    sched = ServedScheduler.build(args)
    ready.put(f"scheduler dp{args.dp_rank} tp{args.tp_rank} ready")
    try:
        sched.run_forever()
    finally:
        sched.engine.shutdown()


def _run_tokenizer(args: ServerArgs, ready) -> None:
    from ..tokenizer.server import tokenize_worker

    tokenize_worker(args, ready)


def _crash_watchdog(procs: List[mp.Process], poll_s: float = 1.0) -> None:
    """Any dead child takes the server down: a half-alive tensor-parallel group would hang on
    its next collective (python/minisgl/server/launch.py:167-200)."""
    while True:
        time.sleep(poll_s)
        for p in procs:
            if not p.is_alive():
                logger.error("child %s exited with code %s: shutting the server down", p.name, p.exitcode)
                for q in procs:
                    if q.is_alive():
                        q.terminate()
                os.kill(os.getpid(), signal.SIGTERM)
                return


def start_backend(args: ServerArgs) -> List[mp.Process]:
    ctx = mp.get_context("spawn")
    ready = ctx.Queue()
    uniq = f"pid={os.getpid()}"
    args = dataclasses.replace(args, _unique=uniq)
    procs: List[mp.Process] = []
    for dp in range(args.dp_size):
        for tp in range(args.tp_size):
            cfg = dataclasses.replace(args, dp_rank=dp, tp_rank=tp)
            p = ctx.Process(target=_run_scheduler, args=(cfg, ready), name=f"scheduler-dp{dp}-tp{tp}", daemon=True)
            p.start()
            procs.append(p)
    t = ctx.Process(target=_run_tokenizer, args=(args, ready), name="tokenizer", daemon=True)
    t.start()
    procs.append(t)
    for _ in procs:
        logger.info(ready.get(timeout=1800))
    threading.Thread(target=_crash_watchdog, args=(procs,), daemon=True).start()
    return procs


def launch_server(argv=None) -> None:
    import dataclasses as dc

    from .api_server import run_api_server
    from .args import parse_args

    args = parse_args(argv)
    args = dc.replace(args, _unique=f"pid={os.getpid()}")
    if args.shell_mode:
        from .shell import run_shell

        procs = start_backend(args)
        run_shell(args)
        for p in procs:
            p.terminate()
        return
    run_api_server(args, start_backend=lambda: start_backend(args))
