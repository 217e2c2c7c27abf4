"""Launcher: ``python -m mintccl_b200.launch -np 4 script.py [args...]``.

Stands in for ``mpirun -np N python script.py`` of the reference (README.md:26); mpirun is not assumed to
exist.  Starts N processes on this node with RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT set
(the variables ``mintccl_b200.parallel.rendezvous.connect`` reads), forwards their output, and ends all of
them when one fails (by process id, never by name).
"""
from __future__ import annotations

import argparse
import os
import signal
import socket
import subprocess
import sys
import time


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def main() -> int:
    ap = argparse.ArgumentParser(prog="python -m mintccl_b200.launch")
    ap.add_argument("-np", "--nproc", type=int, required=True)
    ap.add_argument("--timeout", type=float, default=0.0, help="seconds; 0 = none")
    ap.add_argument("script")
    ap.add_argument("args", nargs=argparse.REMAINDER)
    a = ap.parse_args()
    port = _free_port()
    procs = []
    for r in range(a.nproc):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(a.nproc), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, a.script, *a.args], env=env))
    t0, rc = time.time(), 0
    try:
        while procs:
            for p in list(procs):
                code = p.poll()
                if code is not None:
                    procs.remove(p)
                    if code != 0:
                        rc = code
                        raise RuntimeError(f"rank process {p.pid} exited with {code}")
            if a.timeout and time.time() - t0 > a.timeout:
                rc = 124
                raise RuntimeError("timeout")
            time.sleep(0.05)
    except (RuntimeError, KeyboardInterrupt) as e:
        print(f"[launch] {e}; stopping the remaining ranks", file=sys.stderr)
        for p in procs:
            p.send_signal(signal.SIGTERM)
        for p in procs:
            try:
                p.wait(10)
            except subprocess.TimeoutExpired:
                p.kill()
        rc = rc or 1
    return rc


if __name__ == "__main__":
    sys.exit(main())
