"""Cross-process GPU lock (``EMMY_GPU_LOCK``), the convention of ``emmy/compiler/backend/gpu_lock.py:50-61``.

When the environment variable names a path, every entry point that puts work on the GPU (``B200Backend.run``,
``benchmark``, the CLI's eager timing) holds an exclusive ``flock`` on that file, so concurrent processes — a parallel
test run, several ``run --bench`` invocations — never interleave kernels on one GPU and timings stay clean. Unset, the
context manager does nothing. Re-entrant within a process (nested ``with gpu_lock():`` blocks do not deadlock).
"""

from __future__ import annotations

import contextlib
import fcntl
import os
import threading
from collections.abc import Iterator
from pathlib import Path

ENV = "EMMY_GPU_LOCK"
_state = threading.local()
_guard = threading.RLock()


@contextlib.contextmanager
def gpu_lock() -> Iterator[None]:
    path = os.environ.get(ENV)
    if not path:
        yield
        return
    depth = getattr(_state, "depth", 0)
    if depth > 0:   # already held by this thread
        _state.depth = depth + 1
        try:
            yield
        finally:
            _state.depth -= 1
        return
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    with _guard, open(path, "a+") as fh:
        fcntl.flock(fh.fileno(), fcntl.LOCK_EX)
        _state.depth = 1
        try:
            yield
        finally:
            _state.depth = 0
            fcntl.flock(fh.fileno(), fcntl.LOCK_UN)
