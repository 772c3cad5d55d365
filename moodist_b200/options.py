"""Per-group options, by attribute or as a temporary override.

Option names are the reference's (``py/moodist/options.py:8-113``): ``prefer_kernel_less`` and
``force_kernel_less`` (bool), ``num_chunks``, ``chunk_size`` and ``method`` (int, ``None`` = automatic).
Here ``method`` selects the kernel family (0 = peer load/store kernels, 1 = NVLS multimem kernels, 2 = DMA copies
between one-warp flag kernels).

    pg.options().method = 1
    with pg.options(prefer_kernel_less=True, num_chunks=2):
        ...
"""

from __future__ import annotations

_KINDS = {
    "prefer_kernel_less": "bool",
    "force_kernel_less": "bool",
    "num_chunks": "int",
    "chunk_size": "int",
    "method": "int",
}


def _encode(name: str, value) -> int:
    if name not in _KINDS:
        raise ValueError(f"Unknown option: {name}")
    if _KINDS[name] == "bool":
        return 1 if value else 0
    return -1 if value is None else int(value)


def _decode(name: str, raw: int):
    if _KINDS[name] == "bool":
        return raw != 0
    return None if raw == -1 else raw


class MoodistOptionsContext:
    """Applies overrides on entry, puts the previous values back on exit; yields the group."""

    def __init__(self, pg, overrides: dict):
        self._pg = pg
        self._overrides = overrides
        self._saved: dict = {}

    def __enter__(self):
        for key, value in self._overrides.items():
            self._saved[key] = self._pg._get_option(key)
            self._pg._set_option(key, value)
        return self._pg

    def __exit__(self, exc_type, exc_val, exc_tb):
        for key, value in self._saved.items():
            self._pg._set_option(key, value)
        return False


class MoodistOptions:
    """Attribute view of one group's options; calling it builds a MoodistOptionsContext."""

    def __init__(self, pg):
        object.__setattr__(self, "_pg", pg)

    def __call__(self, **kwargs) -> MoodistOptionsContext:
        return MoodistOptionsContext(self._pg, {k: _encode(k, v) for k, v in kwargs.items()})

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        if name not in _KINDS:
            raise AttributeError(f"Unknown option: {name}")
        return _decode(name, self._pg._get_option(name))

    def __setattr__(self, name: str, value):
        if name not in _KINDS:
            raise AttributeError(f"Unknown option: {name}")
        self._pg._set_option(name, _encode(name, value))


def _options(self, **kwargs):
    opts = MoodistOptions(self)
    return opts(**kwargs) if kwargs else opts


def install(cls) -> None:
    cls.options = _options
