"""Cooperative shutdown and readiness signalling (reference: crates/shutdown/src/lib.rs:132-162 —
first SIGINT/SIGTERM asks loops to finish their current step and save, a second one exits
immediately; ``--ready-file`` is written once the service accepts requests)."""
from __future__ import annotations

import os
import signal
import threading
from typing import Callable, List

_flag = threading.Event()
_hooks: List[Callable[[], None]] = []
_installed = False


def requested() -> bool:
    return _flag.is_set()


def request() -> None:
    _flag.set()
    for h in list(_hooks):
        try:
            h()
        except Exception:
            pass


def on_shutdown(fn: Callable[[], None]) -> None:
    _hooks.append(fn)


def wait(timeout=None) -> bool:
    return _flag.wait(timeout)


def reset() -> None:
    _flag.clear()
    _hooks.clear()


def install() -> None:
    """Install the two-stage signal handlers (main thread only; a no-op elsewhere)."""
    global _installed
    if _installed or threading.current_thread() is not threading.main_thread():
        return

    def handler(signum, frame):
        if _flag.is_set():
            os._exit(130)
        request()

    signal.signal(signal.SIGINT, handler)
    signal.signal(signal.SIGTERM, handler)
    _installed = True


def write_ready_file(path: str, body: str = "ready\n") -> None:
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        f.write(body)
    os.replace(tmp, path)
