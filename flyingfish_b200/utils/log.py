"""JSON-lines decision log on stderr (``backend_device``, ``prefill_memory_plan``, ``serve_request`` ...),
the observability channel of the reference (src/backend/cuda/engine.rs:1313, 1580-1583;
src/serve/mod.rs:393-400), with its thread-local verbosity guard (src/backend/mod.rs:168-194)."""
from __future__ import annotations

import contextlib
import json
import sys
import threading
import time

_state = threading.local()


def verbose() -> bool:
    return getattr(_state, "verbose", False)


@contextlib.contextmanager
def with_verbose(flag: bool):
    old = verbose()
    _state.verbose = flag
    try:
        yield
    finally:
        _state.verbose = old


def log_json(event: str, verbose_only: bool = False, **fields) -> None:
    if verbose_only and not verbose():
        return
    rec = {"event": event, "ts": round(time.time(), 3), **fields}
    sys.stderr.write(json.dumps(rec, default=str) + "\n")
    sys.stderr.flush()
