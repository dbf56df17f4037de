"""Host-side check of the ticket enumeration behind softmax / layernorm on very long rows.

In the one-launch form a CTA takes a ticket when it starts, and the ticket names its task: the
statistics of one 32 KiB segment of a row, or the application of the row's statistics to one
segment.  An apply task waits for its row's statistics, so progress needs every apply task of a
row to come after ALL statistics tasks of that row in ticket order (tasks with smaller tickets
are held by CTAs that are already running).  The kernel and fdl_debug_split_ticket decode tickets
with the same function; this walks whole enumerations through the C ABI.  No GPU needed.
"""
import ctypes as C

import numpy as np
import pytest

from fast_dl_b200 import capi


def decode_all(rows, segments, lag):
    lib = capi.lib()
    row, seg, apply = C.c_int64(), C.c_int(), C.c_int()
    tasks = []
    for ticket in range(2 * rows * segments):
        status = lib.fdl_debug_split_ticket(rows, segments, lag, ticket, C.byref(row), C.byref(seg), C.byref(apply))
        assert status == 0, (rows, segments, lag, ticket, status)
        tasks.append((row.value, seg.value, apply.value))
    return tasks


@pytest.mark.parametrize("rows,segments,lag", [(1, 1, 1), (1, 5, 1), (2, 3, 1), (2, 3, 2), (7, 4, 3), (7, 4, 7), (40, 17, 9),
                                               (128, 64, 18), (33, 2, 32)])
def test_every_task_once_and_apply_after_the_rows_statistics(rows, segments, lag):
    tasks = decode_all(rows, segments, lag)
    assert len(set(tasks)) == len(tasks) == 2 * rows * segments
    assert set(tasks) == {(r, s, a) for r in range(rows) for s in range(segments) for a in (0, 1)}
    ticket_of = {task: ticket for ticket, task in enumerate(tasks)}
    for r in range(rows):
        last_stats = max(ticket_of[(r, s, 0)] for s in range(segments))
        first_apply = min(ticket_of[(r, s, 1)] for s in range(segments))
        assert last_stats < first_apply
        if r + lag < rows:
            # the distance the launcher asks for: the statistics of `lag` further rows come in between
            assert first_apply > max(ticket_of[(r + lag, s, 0)] for s in range(segments))
    # statistics tasks, and apply tasks, each appear in row-major order
    for kind in (0, 1):
        order = [(r, s) for (r, s, a) in tasks if a == kind]
        assert order == sorted(order)


def test_random_plans():
    rng = np.random.default_rng(5)
    for _ in range(40):
        rows = int(rng.integers(1, 60))
        segments = int(rng.integers(1, 12))
        lag = int(rng.integers(1, rows + 1))
        tasks = decode_all(rows, segments, lag)
        assert len(set(tasks)) == 2 * rows * segments
        ticket_of = {task: ticket for ticket, task in enumerate(tasks)}
        for r in range(rows):
            assert max(ticket_of[(r, s, 0)] for s in range(segments)) < min(ticket_of[(r, s, 1)] for s in range(segments))


def test_arguments_are_checked():
    lib = capi.lib()
    row, seg, apply = C.c_int64(), C.c_int(), C.c_int()
    out = (C.byref(row), C.byref(seg), C.byref(apply))
    assert lib.fdl_debug_split_ticket(4, 4, 2, 2 * 4 * 4, *out) == -1       # ticket past the end
    assert lib.fdl_debug_split_ticket(4, 4, 5, 0, *out) == -1                # lag beyond the rows
    assert lib.fdl_debug_split_ticket(4, 4, 0, 0, *out) == -1
    assert lib.fdl_debug_split_ticket(0, 4, 1, 0, *out) == -1
    assert lib.fdl_debug_split_ticket(4, 4, 2, 0, None, C.byref(seg), C.byref(apply)) == -1
    assert lib.fdl_debug_split_ticket(16384, 4, 2, 0, *out) == -2            # more rows than arrival counters
    assert lib.fdl_debug_split_ticket(16000, 1 << 20, 2, 0, *out) == -2      # more tasks than a grid holds
