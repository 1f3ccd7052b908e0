"""Launcher for programs built against baseline/shims/mpi.h: starts N ranks as processes of this machine.

    python baseline/shims/mpirun_local.py -np 4 [--timeout S] [--gpu-per-rank] PROGRAM [ARGS...]

Every rank gets MPISHIM_RANK, MPISHIM_SIZE and MPISHIM_JOB (a name unique to this launch; the ranks meet on abstract
Unix-domain sockets derived from it).  Rank 0 inherits stdout; the other ranks' output goes to stderr with a rank
prefix.  If a rank exits with a non-zero code or the time limit runs out, the remaining ranks are terminated (by the
process ids started here) and that code is returned.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import threading
import time
import uuid


def _die_with_parent() -> None:
    """Child-side hook: a rank is killed if the launcher goes away first (Linux parent-death signal)."""
    import ctypes
    import signal
    try:
        ctypes.CDLL("libc.so.6", use_errno=True).prctl(1, signal.SIGKILL)      # PR_SET_PDEATHSIG
    except OSError:
        pass


def _pump(stream, rank: int) -> None:
    for line in stream:
        sys.stderr.write(f"[rank {rank}] {line}")


def launch(np_: int, cmd, timeout: float = 0.0, env=None, capture_rank0: bool = False):
    """Returns ``(exit_code, rank-0 stdout or None)``."""
    job = uuid.uuid4().hex[:12]
    base = dict(os.environ if env is None else env)
    procs, pumps = [], []
    for r in range(np_):
        e = dict(base, MPISHIM_RANK=str(r), MPISHIM_SIZE=str(np_), MPISHIM_JOB=job)
        if r == 0:
            p = subprocess.Popen(cmd, env=e, stdout=subprocess.PIPE if capture_rank0 else None, text=True, preexec_fn=_die_with_parent)
        else:
            p = subprocess.Popen(cmd, env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, preexec_fn=_die_with_parent)
            t = threading.Thread(target=_pump, args=(p.stdout, r), daemon=True)
            t.start()
            pumps.append(t)
        procs.append(p)
    out0 = []
    if capture_rank0:
        t0 = threading.Thread(target=lambda: out0.append(procs[0].stdout.read()), daemon=True)
        t0.start()
        pumps.append(t0)
    deadline = time.time() + timeout if timeout > 0 else None
    code = 0
    while True:
        states = [p.poll() for p in procs]
        bad = [s for s in states if s not in (None, 0)]
        if bad:
            code = bad[0]
            break
        if all(s == 0 for s in states):
            break
        if deadline is not None and time.time() > deadline:
            code = 124
            break
        time.sleep(0.05)
    for p in procs:
        if p.poll() is None:
            p.terminate()
    for p in procs:
        try:
            p.wait(timeout=10)
        except subprocess.TimeoutExpired:
            p.kill()
    for t in pumps:
        t.join(timeout=5)
    return code, (out0[0] if out0 else None)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("-np", type=int, required=True)
    ap.add_argument("--timeout", type=float, default=0.0)
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = a.cmd[1:] if a.cmd and a.cmd[0] == "--" else a.cmd
    if not cmd:
        ap.error("no program given")
    code, _ = launch(a.np, cmd, a.timeout)
    return code


if __name__ == "__main__":
    sys.exit(main())
