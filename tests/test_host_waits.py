"""Host-side waiting: the launch deadline and the per-device call lock, no GPU needed.

The reference bounds every host wait by a budget read once from the environment
(src/watchdog.rs:102-106, 300-332); this library returns FK_ERR_TIMEOUT where the reference
ends the process.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import sys
import threading
import time

import pytest

from ferro_kittens_b200 import _lib
from ferro_kittens_b200._lib import FK_ERR_INVALID, FK_ERR_TIMEOUT, FK_OK, library

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_a_query_that_never_completes_times_out_with_the_budget_in_the_message():
    start = time.perf_counter()
    code = library().fk_selftest_deadline(120, 0xFFFFFFFF)
    elapsed = time.perf_counter() - start
    assert code == FK_ERR_TIMEOUT
    assert 0.12 <= elapsed < 2.0
    message = _lib.last_error()
    assert "120 ms" in message and "KITTENS_LAUNCH_BUDGET_MS" in message


def test_a_query_that_completes_within_the_budget_returns_ok():
    assert library().fk_selftest_deadline(10_000, 0) == FK_OK
    assert library().fk_selftest_deadline(10_000, 1000) == FK_OK


def test_past_the_spin_window_the_wait_sleeps_between_polls():
    # 50 ms of spinning, then one poll per millisecond: a query that needs a few polls more than the
    # spin can deliver in its window still completes, long before a 5 s budget.
    start = time.perf_counter()
    assert library().fk_selftest_deadline(5_000, 0xFFFFFFFE) in (FK_OK, FK_ERR_TIMEOUT)
    assert time.perf_counter() - start <= 6.0


def _budget_in_a_fresh_process(value):
    env = dict(os.environ)
    env.pop("KITTENS_LAUNCH_BUDGET_MS", None)
    if value is not None:
        env["KITTENS_LAUNCH_BUDGET_MS"] = value
    code = "from ferro_kittens_b200 import watchdog; print(watchdog.budget())"
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    return int(out.stdout.strip().splitlines()[-1])


def test_the_budget_defaults_to_the_references_thirty_seconds():
    assert _budget_in_a_fresh_process(None) == 30_000


@pytest.mark.parametrize("text, expected", [("1500", 1500), ("0", 30_000), ("soon", 30_000), ("", 30_000)])
def test_the_environment_variable_overrides_the_budget_when_it_is_a_positive_number(text, expected):
    assert _budget_in_a_fresh_process(text) == expected


def test_two_threads_on_one_device_serialise_and_two_devices_do_not():
    lib = library()

    def hold(device, out):
        entered, left = ctypes.c_uint64(), ctypes.c_uint64()
        assert lib.fk_selftest_call_guard(device, 150, ctypes.byref(entered), ctypes.byref(left)) == FK_OK
        out.append((entered.value, left.value))

    same = []
    threads = [threading.Thread(target=hold, args=(3, same)) for _ in range(2)]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    (a0, a1), (b0, b1) = sorted(same)
    assert a1 <= b0, "two calls held one device's lock at the same time"

    apart = []
    threads = [threading.Thread(target=hold, args=(device, apart)) for device in (4, 5)]
    start = time.perf_counter()
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    assert time.perf_counter() - start < 0.29, "locks of different devices must not serialise"


def test_the_call_guard_refuses_a_device_it_has_no_lock_for():
    entered, left = ctypes.c_uint64(), ctypes.c_uint64()
    assert library().fk_selftest_call_guard(64, 1, ctypes.byref(entered), ctypes.byref(left)) == FK_ERR_INVALID
    assert library().fk_selftest_call_guard(-1, 1, ctypes.byref(entered), ctypes.byref(left)) == FK_ERR_INVALID
