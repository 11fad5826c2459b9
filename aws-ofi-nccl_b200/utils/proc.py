"""Running a multi-process job under a time limit and ending ALL of it when the limit passes.

A launcher such as ``torch.distributed.run`` starts its workers in sessions of their own, so ending
the launcher (or its process group) can leave workers behind, still holding the GPU.  ``run_job``
therefore collects the exact process ids of the launcher's descendants and ends those."""
from __future__ import annotations

import os
import signal
import subprocess
import time


def _descendants(pid: int) -> list[int]:
    """Process ids of every live descendant of `pid` (children first), read from /proc."""
    parents: dict[int, int] = {}
    for name in os.listdir("/proc"):
        if not name.isdigit():
            continue
        try:
            with open(f"/proc/{name}/stat", "rb") as f:
                stat = f.read().decode(errors="replace")
            # pid (comm) state ppid ...; comm may contain spaces and parentheses
            ppid = int(stat[stat.rindex(")") + 2:].split()[1])
        except (OSError, ValueError, IndexError):
            continue
        parents[int(name)] = ppid
    out, frontier = [], [pid]
    while frontier:
        nxt = [p for p, pp in parents.items() if pp in frontier and p not in out]
        out += nxt
        frontier = nxt
    return out


def end_tree(pid: int) -> None:
    """SIGKILL for `pid` and each of its descendants, by exact process id."""
    victims = _descendants(pid) + [pid]
    for p in victims:
        try:
            os.kill(p, signal.SIGKILL)
        except ProcessLookupError:
            pass


def run_job(cmd, env=None, cwd=None, timeout: float = 600.0):
    """Runs `cmd`, returns (returncode, stdout, stderr); returncode is None when the limit passed
    (the launcher and all its descendants have been ended by then)."""
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env, cwd=cwd,
                            start_new_session=True)
    try:
        out, err = proc.communicate(timeout=timeout)
        return proc.returncode, out, err
    except subprocess.TimeoutExpired:
        end_tree(proc.pid)
        deadline = time.time() + 20
        out = err = ""
        try:
            out, err = proc.communicate(timeout=max(1.0, deadline - time.time()))
        except subprocess.TimeoutExpired:
            pass   # a descendant outside the tree still holds the pipes: give up on its output
        return None, out, err
