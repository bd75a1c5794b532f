"""Process-level handle accounting, for leak hunts around repeated IPC opens
(`awex/util/system_util.py:22-85` in the reference): file-descriptor limits and
use, System V and POSIX IPC objects held by this process."""

from __future__ import annotations

import os
import resource
import subprocess
from typing import Dict, Tuple

_SYSV_KINDS = {"msg": "-q", "sem": "-s", "shm": "-m"}


def get_rlimit_nofile() -> Tuple[int, int]:
    return resource.getrlimit(resource.RLIMIT_NOFILE)


def count_open_fds() -> int:
    try:
        return len(os.listdir(f"/proc/{os.getpid()}/fd"))
    except OSError:
        return -1


def count_sysv_ipc() -> Dict[str, int]:
    """Objects whose creator or last-operator pid is this process, per kind
    (``ipcs -p``); -1 where ``ipcs`` is not available."""
    pid = str(os.getpid())
    counts: Dict[str, int] = {}
    for kind, flag in _SYSV_KINDS.items():
        try:
            out = subprocess.check_output(["ipcs", flag, "-p"], text=True, stderr=subprocess.DEVNULL, timeout=10)
        except Exception:
            counts[kind] = -1
            continue
        counts[kind] = sum(1 for line in out.splitlines() if pid in line.split()[1:])
    return counts


def count_posix_ipc() -> Dict[str, int]:
    """POSIX shared memory and message queues seen through open descriptors and
    mappings; event descriptors stand in for semaphores (approximate)."""
    counts = {"shm": 0, "sem": 0, "mq": 0}
    targets = []
    fd_dir = f"/proc/{os.getpid()}/fd"
    try:
        for fd in os.listdir(fd_dir):
            try:
                targets.append(os.readlink(os.path.join(fd_dir, fd)))
            except OSError:
                pass
        with open(f"/proc/{os.getpid()}/maps") as f:
            targets.extend(line.split(None, 5)[5].strip() for line in f if len(line.split(None, 5)) == 6)
    except OSError:
        return counts
    for path in targets:
        if "/dev/shm/" in path:
            counts["shm"] += 1
        elif path.startswith("/dev/mqueue/"):
            counts["mq"] += 1
        elif "anon_inode:[eventfd]" in path:
            counts["sem"] += 1
    return counts


def get_handle_counts() -> Dict[str, int]:
    soft, hard = get_rlimit_nofile()
    sysv = sum(v for v in count_sysv_ipc().values() if v > 0)
    posix = sum(count_posix_ipc().values())
    return {"soft_limit": soft, "hard_limit": hard, "open_fds": count_open_fds(), "sysv_ipc": sysv, "posix_ipc": posix, "total_ipc": sysv + posix}
