"""One parseable line per (process, rank, path, capture state) saying which paths of the library a process took:

    B200NODES: <path> pid=<pid> rank=<rank> rows=<rows> captured=<0|1>

The counterpart of the reference's branch evidence (qwen36_layer/evidence.py:57-61): not per layer and not per call
(the question is which RANKS took a path and whether it is inside a captured graph); host-side only, written to
stderr, never allowed to break execution.  `seen()` returns the keys recorded so far (tests)."""
from __future__ import annotations

import os
import sys

_seen = set()


def _rank() -> int:
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return int(dist.get_rank())
    except Exception:  # noqa: BLE001
        pass
    return -1


def note(path: str, rows: int) -> None:
    try:
        import torch
        captured = bool(torch.cuda.is_available() and torch.cuda.is_current_stream_capturing())
    except Exception:  # noqa: BLE001
        captured = False
    key = (os.getpid(), _rank(), path, captured)
    if key in _seen:
        return
    _seen.add(key)
    try:
        print(f"B200NODES: {path} pid={key[0]} rank={key[1]} rows={int(rows)} captured={int(captured)}", file=sys.stderr,
              flush=True)
    except Exception:  # noqa: BLE001
        pass


def seen():
    return set(_seen)
