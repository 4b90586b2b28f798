"""Deadline-bounded host waits (reference: src/watchdog.rs:300-332).

Unlike the reference these return an error instead of aborting the process.
"""
from __future__ import annotations

import torch

from ._lib import check, library

#: The reference's per-launch budget (src/watchdog.rs:102).
DEFAULT_BUDGET_MS = 30_000
#: The environment variable that overrides it for one process (src/watchdog.rs:106).
BUDGET_VARIABLE = "KITTENS_LAUNCH_BUDGET_MS"


def budget() -> int:
    """The deadline, in milliseconds, of every wait the library makes on its own."""
    return int(library().fk_launch_budget_ms())


def wait(stream=None, budget_ms: int | None = None) -> None:
    handle = (stream or torch.cuda.current_stream()).cuda_stream
    check(library().fk_wait_stream(handle, budget() if budget_ms is None else budget_ms))


def wait_event(event: torch.cuda.Event, budget_ms: int | None = None) -> None:
    check(library().fk_wait_event(event.cuda_event, budget() if budget_ms is None else budget_ms))
