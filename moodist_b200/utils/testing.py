"""Rank-symmetric multi-process test harness.

Every rank runs the same function; a failure (exception) on any rank fails the test on all of them, the
parent collects per-rank tracebacks, and a watchdog kills ranks that outlive the timeout after dumping
their Python stacks — the behaviours of the reference's home-grown runner (``tests/framework.py:248-293``
pass/fail exchange, ``tests/run.py:95-239`` watchdog with stack dump, ``--per-rank-logs``), packaged so
pytest can drive them.  Ports are derived deterministically from a base port and a test id
(``tests/framework.py:65-76``).
"""

from __future__ import annotations

import faulthandler
import multiprocessing as mp
import os
import signal
import socket
import sys
import tempfile
import time
import traceback
from typing import Callable


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(fn, rank, world, port, args, env, result_dir, per_rank_logs):
    os.environ.update({k: str(v) for k, v in env.items()})
    os.environ.update(
        RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port)
    )
    if per_rank_logs:
        log = open(os.path.join(result_dir, f"rank{rank}.log"), "w", buffering=1)
        os.dup2(log.fileno(), 1)
        os.dup2(log.fileno(), 2)
    stack_file = open(os.path.join(result_dir, f"rank{rank}.stacks"), "w")
    faulthandler.register(signal.SIGUSR1, file=stack_file, all_threads=True)
    status = "ok"
    try:
        fn(rank, world, port, *args)
    except BaseException:  # noqa: BLE001 - the parent reports it
        status = traceback.format_exc()
    if status == "ok":
        # os._exit below skips the interpreter's exit hooks; what they would have done for a store that is still
        # alive (kept by an exception's traceback, say) is done here: leave through the coordinated shutdown, so
        # that the answers this rank still owes its peers reach them
        try:
            from .._core import _C

            _C._shutdown_all_stores()
        except Exception:  # noqa: BLE001 - leaving anyway
            pass
    with open(os.path.join(result_dir, f"rank{rank}.status"), "w") as f:
        f.write(status)
    # leave without running destructors of half-torn-down process groups on failure
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0 if status == "ok" else 1)


def run_ranks(
    fn: Callable,
    world: int,
    *args,
    timeout: float = 120.0,
    env: dict | None = None,
    port: int | None = None,
    per_rank_logs: bool = False,
    expect_failure: bool = False,
):
    """Run ``fn(rank, world, port, *args)`` in ``world`` fresh processes; raise if any rank fails.

    With ``expect_failure=True`` returns the list of per-rank status strings instead of raising.
    """
    ctx = mp.get_context("spawn")
    port = port or free_port()
    result_dir = tempfile.mkdtemp(prefix="moodist-test-")
    procs = [
        ctx.Process(target=_worker, args=(fn, r, world, port, args, env or {}, result_dir, per_rank_logs), daemon=True)
        for r in range(world)
    ]
    for p in procs:
        p.start()
    deadline = time.time() + timeout
    timed_out = False
    while any(p.is_alive() for p in procs):
        if time.time() > deadline:
            timed_out = True
            for p in procs:  # stack dump first, then kill (the exact pids we started)
                if p.is_alive():
                    os.kill(p.pid, signal.SIGUSR1)
            time.sleep(0.5)
            for p in procs:
                if p.is_alive():
                    p.kill()
            break
        # one rank failed: give the others a moment to notice, then stop waiting
        if any((not p.is_alive()) and p.exitcode not in (0, None) for p in procs):
            deadline = min(deadline, time.time() + 15)
        time.sleep(0.02)
    for p in procs:
        p.join(5)
    statuses = []
    for r in range(world):
        path = os.path.join(result_dir, f"rank{r}.status")
        if os.path.exists(path):
            statuses.append(open(path).read())
        else:
            stacks = ""
            sp = os.path.join(result_dir, f"rank{r}.stacks")
            if os.path.exists(sp):
                stacks = open(sp).read()
            statuses.append(("timed out" if timed_out else f"died with exit code {procs[r].exitcode}") + "\n" + stacks)
    if expect_failure:
        return statuses
    bad = [(r, s) for r, s in enumerate(statuses) if s != "ok"]
    if bad:
        msg = "\n".join(f"--- rank {r} ---\n{s}" for r, s in bad)
        raise AssertionError(f"{len(bad)} of {world} ranks failed:\n{msg}")
    return statuses


def init_moodist(rank: int, world: int, port: int, device: str = "cpu"):
    """Create the default process group over the moodist backend with torch's TCPStore rendezvous."""
    import torch
    import torch.distributed as dist

    import moodist_b200  # noqa: F401 - registers the backend

    if device == "cuda":
        torch.cuda.set_device(rank % torch.cuda.device_count())
    dist.init_process_group("moodist", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    return dist
