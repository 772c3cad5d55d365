"""Host-side tracing of the progress engine.

``enable_profiling(True)`` starts recording one span per engine operation of every live moodist group;
``enable_profiling(False)`` stops and writes ``moodist-trace-cpu-<group>-<rank>.json`` in Chrome trace
format (``"ph": "X"`` events with ``ts``/``dur`` in microseconds), the file name and format of the
reference (``core/cputhread.cc:1008-1078``).  Returns the list of files written.
"""

from __future__ import annotations

from .._core import _C


def _live_groups():
    return _C.live_process_groups()


def enable_profiling(enabled: bool = True, groups=None) -> list[str]:
    """Switch engine tracing on or off for ``groups`` (default: every live moodist group)."""
    paths = []
    for g in groups if groups is not None else _live_groups():
        p = g.enable_profiling(bool(enabled))
        if p and not enabled:
            paths.append(p)
    return paths
