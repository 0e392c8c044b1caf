"""Retry a callable with exponential backoff inside a wall-clock budget.

Behaviour of the reference helper (`src/kohakumoss_common/retry.py:16`): transient
`OSError`s from checkpoint writes and remote reads are retried until the budget runs out,
then the last error is raised.
"""

from __future__ import annotations

import time
from collections.abc import Callable


def retrying(
    fn: Callable,
    *args,
    budget_s: float = 600.0,
    first_delay_s: float = 0.5,
    max_delay_s: float = 30.0,
    retry_on: tuple[type[BaseException], ...] = (OSError,),
    on_retry: Callable[[int, BaseException, float], None] | None = None,
    sleep: Callable[[float], None] = time.sleep,
    clock: Callable[[], float] = time.monotonic,
    **kwargs,
):
    start = clock()
    delay = first_delay_s
    attempt = 0
    while True:
        attempt += 1
        try:
            return fn(*args, **kwargs)
        except retry_on as err:
            left = budget_s - (clock() - start)
            if left <= 0:
                raise
            wait = min(delay, max_delay_s, left)
            if on_retry is not None:
                on_retry(attempt, err, wait)
            sleep(wait)
            delay *= 2
