"""Deadline-bounded host waits (reference: src/watchdog.rs:300-332).

Unlike the reference these return an error instead of aborting the process.
"""
from __future__ import annotations

import torch

from ._lib import check, library

#: The reference's per-launch budget (src/watchdog.rs:102).
DEFAULT_BUDGET_MS = 30_000


def wait(stream=None, budget_ms: int = DEFAULT_BUDGET_MS) -> None:
    handle = (stream or torch.cuda.current_stream()).cuda_stream
    check(library().fk_wait_stream(handle, budget_ms))


def wait_event(event: torch.cuda.Event, budget_ms: int = DEFAULT_BUDGET_MS) -> None:
    check(library().fk_wait_event(event.cuda_event, budget_ms))
