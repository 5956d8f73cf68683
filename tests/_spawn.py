"""Runs a worker script as N rank processes and collects their results."""
from __future__ import annotations

import os
import socket
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def free_port(span: int = 8) -> int:
    """A port p such that p .. p + span - 1 can all be bound right now.  Taken below the range the kernel hands
    out for outgoing connections (32768 and up), so that a rank's own client socket can never sit on a port
    that a worker wants to listen on next (workers use NANO_TEST_PORT + small offsets)."""
    import random

    rng = random.Random(os.getpid() * 7919 + int.from_bytes(os.urandom(4), "little"))
    for _ in range(200):
        base = rng.randrange(15000, 31000, span)
        socks = []
        try:
            for k in range(span):
                s = socket.socket()
                socks.append(s)
                s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
                s.bind(("127.0.0.1", base + k))
            return base
        except OSError:
            continue
        finally:
            for s in socks:
                s.close()
    raise RuntimeError("no free port range found")


def run_ranks(worker: str, nranks: int, args: list[str] | None = None, env: dict | None = None,
              timeout: int = 300) -> list[str]:
    """Starts `nranks` copies of tests/workers/<worker>; returns their outputs; raises on failure."""
    port = free_port()
    master_port = free_port()
    procs = []
    # the ranks compute reference results on the CPU at the same time: share the cores instead of letting
    # every rank start one thread per core
    threads = str(max(1, min(8, (os.cpu_count() or 8) // max(nranks, 1))))
    for r in range(nranks):
        e = dict(os.environ)
        e.setdefault("OMP_NUM_THREADS", threads)
        e.setdefault("MKL_NUM_THREADS", threads)
        e.update({"RANK": str(r), "WORLD_SIZE": str(nranks), "LOCAL_RANK": str(r),
                  "NANO_TEST_PORT": str(port), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(master_port),
                  "PYTHONPATH": str(ROOT) + os.pathsep + e.get("PYTHONPATH", "")})
        e.update(env or {})
        cmd = [sys.executable, str(ROOT / "tests" / "workers" / worker)] + (args or [])
        procs.append(subprocess.Popen(cmd, env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs, failed = [], []
    for r, p in enumerate(procs):
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timeout]"
            failed.append(r)
        outs.append(out)
        if p.returncode != 0 and r not in failed:
            failed.append(r)
    if failed:
        detail = "\n".join(f"--- rank {r} (exit {procs[r].returncode}) ---\n{outs[r][-6000:]}" for r in range(nranks))
        raise AssertionError(f"ranks {failed} failed in {worker}:\n{detail}")
    return outs
