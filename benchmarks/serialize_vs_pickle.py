"""`moodist_b200.serialize` / `deserialize` against `pickle` on nine Python-object workloads (CPU only).

    python benchmarks/serialize_vs_pickle.py [--iters 200] [--json out.json]

For every workload: median / 10th / 90th percentile time of serialize and deserialize, the same for
pickle (protocol 5), the speed-up and the size ratio. The workloads stress what a queue of Python objects
sees: many distinct small objects, heavily shared references, nested containers, long strings, numpy
arrays, and dataclass-like instances (custom ``__reduce__``).  (The reference's counterpart is
``benchmarks/serialize.py``, which prints at run time and commits no numbers.)
"""

from __future__ import annotations

import argparse
import json
import os
import pickle
import statistics
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import moodist_b200 as moodist  # noqa: E402


class Sample:
    """Instance with a dict, as a user-defined message would be."""

    def __init__(self, i):
        self.index = i
        self.name = f"sample-{i}"
        self.weights = [i * 0.5, i * 0.25, -1.0]
        self.tags = ("a", "b", i % 7)


def workloads():
    import numpy as np

    shared = [("key", i) for i in range(64)]
    w = {
        "ints_100k": list(range(100_000)),
        "floats_100k": [i * 0.001 for i in range(100_000)],
        "small_strings_50k": [f"item-{i}" for i in range(50_000)],
        "dict_str_int_50k": {f"k{i}": i for i in range(50_000)},
        "nested_lists": [[j for j in range(20)] for _ in range(5_000)],
        "shared_refs": [shared[i % 64] for i in range(100_000)],
        "tuples_mixed_30k": [(i, str(i), i * 1.5, None, i % 2 == 0) for i in range(30_000)],
        "numpy_arrays": [np.arange(1024, dtype=np.float32) + i for i in range(256)],
        "instances_10k": [Sample(i) for i in range(10_000)],
    }
    return w


def timed(fn, iters, warmup=5):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        t0 = time.perf_counter()
        fn()
        ts.append((time.perf_counter() - t0) * 1e3)
    ts.sort()
    return statistics.median(ts), ts[len(ts) // 10], ts[(len(ts) * 9) // 10]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    rows = []
    print(f"{'workload':<20} {'ser ms (p10-p90)':>24} {'pickle':>9} {'x':>6} {'deser ms (p10-p90)':>24} {'pickle':>9} {'x':>6} {'size':>6}")
    for name, obj in workloads().items():
        blob = moodist.serialize(obj)
        pk = pickle.dumps(obj, protocol=5)
        back = moodist.deserialize(blob)
        if name != "instances_10k" and name != "numpy_arrays":
            assert back == obj, name
        ms, ms10, ms90 = timed(lambda: moodist.serialize(obj), args.iters)
        ps, _, _ = timed(lambda: pickle.dumps(obj, protocol=5), args.iters)
        md, md10, md90 = timed(lambda: moodist.deserialize(blob), args.iters)
        pd, _, _ = timed(lambda: pickle.loads(pk), args.iters)
        size = blob.numel() if hasattr(blob, "numel") else len(blob)
        row = {"workload": name, "ser_ms": ms, "ser_p10": ms10, "ser_p90": ms90, "pickle_ser_ms": ps,
               "deser_ms": md, "deser_p10": md10, "deser_p90": md90, "pickle_deser_ms": pd,
               "ser_speedup": ps / ms, "deser_speedup": pd / md, "size_ratio": size / len(pk)}
        rows.append(row)
        print(f"{name:<20} {ms:8.3f} ({ms10:6.3f}-{ms90:6.3f}) {ps:9.3f} {ps / ms:6.2f} "
              f"{md:8.3f} ({md10:6.3f}-{md90:6.3f}) {pd:9.3f} {pd / md:6.2f} {size / len(pk):6.2f}")
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
