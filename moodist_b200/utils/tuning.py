"""Variant table from measured bus bandwidth.

The collectives have several kernel families per operation (peer loads/stores, NVLS multimem through
NVSwitch, copy-engine DMA) and size thresholds between them.  The thresholds compiled into the library were
measured on one 8 x B200 NVSwitch machine; this module re-derives them from a sweep on the machine at hand:

    torchrun ... benchmarks/collective_sweep.py --impls moodist_p2p,moodist_nvls,moodist_ce,nccl --out sweep.jsonl
    python -m moodist_b200.utils.tuning sweep.jsonl            # prints the table and the settings
    python -m moodist_b200.utils.tuning sweep.jsonl --table variants.json   # adds this world size to the file
    MOODIST_VARIANT_TABLE=variants.json torchrun ...           # groups load their thresholds from it
    eval "$(python -m moodist_b200.utils.tuning sweep.jsonl --export)"   # or: MOODIST_* variables by hand

The table file holds one block of thresholds per world size (``{"8": {"MOODIST_NVLS_AG_MIN_BYTES": 32768,
...}, "2": {...}}``); a CUDA group reads the block of its own size when it is created.  A variable set in
the environment still wins over the table, and the table over the built-in values.
``apply(settings)`` puts the variables into ``os.environ`` (before the process group is created).  The
reference picks its algorithm per call from fixed rules in ``core/processgroup.cc``; it has no measured table.
"""

from __future__ import annotations

import json
import os
import sys
from collections import defaultdict

FAMILIES = {"moodist_p2p": "p2p", "moodist_nvls": "nvls", "moodist_ce": "ce"}


def load_sweep(path: str) -> list[dict]:
    rows = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line.startswith("{"):
                rows.append(json.loads(line))
    return rows


def variant_table(rows: list[dict], dtype: str = "bf16") -> dict[str, list[dict]]:
    """Per operation, per message size: time of every measured family and the fastest one."""
    by = defaultdict(dict)
    for r in rows:
        if r.get("dtype") != dtype or r["impl"] not in FAMILIES:
            continue
        by[(r["op"], r["bytes_per_rank"])][FAMILIES[r["impl"]]] = r["us"]
    table = defaultdict(list)
    for (op, nbytes), times in sorted(by.items()):
        best = min(times, key=times.get)
        table[op].append({"bytes": nbytes, "best": best, "us": times})
    return dict(table)


def _first_size_from_which(entries: list[dict], family: str) -> int:
    """Smallest size such that `family` is the fastest at it and at every larger measured size (-1: none)."""
    start = -1
    for e in entries:
        if e["best"] == family:
            if start < 0:
                start = e["bytes"]
        else:
            start = -1
    return start


def _window(entries: list[dict], family: str) -> tuple[int, int]:
    """Longest run of consecutive sizes at which `family` is fastest, as (first, last) bytes; (-1, -1) if none."""
    best = (-1, -1)
    run = None
    for e in entries + [{"bytes": None, "best": None}]:
        if e["best"] == family:
            run = (run[0], e["bytes"]) if run else (e["bytes"], e["bytes"])
        elif run:
            if best[0] < 0 or (run[1] / run[0]) > (best[1] / best[0]):
                best = run
            run = None
    return best


def settings_from(table: dict[str, list[dict]]) -> dict[str, int]:
    """MOODIST_* thresholds that reproduce the table's choices."""
    out: dict[str, int] = {}
    ag = table.get("ag", [])
    if ag:
        lo, hi = _window(ag, "nvls")
        out["MOODIST_NVLS_AG_MIN_BYTES"] = lo
        out["MOODIST_NVLS_AG_MAX_BYTES"] = hi if lo >= 0 else -1
    rs = table.get("rs_sum", table.get("rs_avg", []))
    if rs:
        out["MOODIST_NVLS_RS_MIN_BYTES"] = _first_size_from_which(rs, "nvls")
    ar = table.get("ar", [])
    if ar:
        out["MOODIST_NVLS_AR_MIN_BYTES"] = _first_size_from_which(ar, "nvls")
    # DMA copies: one threshold per operation (they win for all-gather long before they do for reduce-scatter)
    if ag:
        out["MOODIST_CE_AUTO_BYTES"] = _first_size_from_which(ag, "ce")
    if rs:
        out["MOODIST_CE_AUTO_RS_BYTES"] = _first_size_from_which(rs, "ce")
    return out


def write_table(path: str, world: int, settings: dict[str, int]) -> dict:
    """Merge ``settings`` as the block for ``world`` ranks into the table file at ``path``; returns the table."""
    table = {}
    if os.path.exists(path):
        with open(path) as f:
            table = json.load(f)
    table[str(int(world))] = {k: int(v) for k, v in sorted(settings.items())}
    with open(path, "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
        f.write("\n")
    return table


def apply(settings: dict[str, int]) -> None:
    """Set the variables for this process; call before ``init_process_group``."""
    for k, v in settings.items():
        os.environ[k] = str(int(v))


def format_table(table: dict[str, list[dict]]) -> str:
    lines = []
    for op, entries in table.items():
        lines.append(f"{op}:")
        for e in entries:
            times = "  ".join(f"{k} {v:9.1f} us" for k, v in sorted(e["us"].items()))
            lines.append(f"  {e['bytes']:>11}  best {e['best']:<5} {times}")
    return "\n".join(lines)


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    export = "--export" in argv
    table_path = None
    if "--table" in argv:
        i = argv.index("--table")
        if i + 1 >= len(argv):
            print(__doc__)
            return 2
        table_path = argv[i + 1]
        del argv[i : i + 2]
    paths = [a for a in argv if not a.startswith("--")]
    if len(paths) != 1:
        print(__doc__)
        return 2
    rows = load_sweep(paths[0])
    table = variant_table(rows)
    settings = settings_from(table)
    if table_path:
        worlds = {int(r["world"]) for r in rows if "world" in r}
        if len(worlds) != 1:
            print(f"--table needs a sweep of one world size, this one has {sorted(worlds)}")
            return 2
        write_table(table_path, worlds.pop(), settings)
        print(f"wrote the block for world size {rows[0]['world']} to {table_path}")
    elif export:
        for k, v in settings.items():
            print(f"export {k}={v}")
    else:
        print(format_table(table))
        print()
        for k, v in settings.items():
            print(f"{k}={v}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
