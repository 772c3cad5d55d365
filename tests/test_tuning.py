"""The variant table derived from a (synthetic) sweep reproduces the choices the timings imply."""

import json

from moodist_b200.utils import tuning


def _rows():
    rows = []
    # all-gather: p2p fastest below 32 KiB, nvls from 32 KiB to 2 MiB, ce from 64 MiB up, p2p in between
    for k in range(12, 29):
        n = 1 << k
        base = 10 + n / 500e3
        t = {"moodist_p2p": base, "moodist_nvls": base * (0.8 if (32 << 10) <= n <= (2 << 20) else 1.3),
             "moodist_ce": base * (0.9 if n >= (64 << 20) else 2.0)}
        for impl, us in t.items():
            rows.append({"op": "ag", "impl": impl, "dtype": "bf16", "bytes_per_rank": n, "world": 8, "us": us, "busbw_gbs": 1})
            rows.append({"op": "rs_sum", "impl": impl, "dtype": "bf16", "bytes_per_rank": n, "world": 8,
                         "us": us * (0.95 if impl == "moodist_p2p" else 1.0), "busbw_gbs": 1})
        rows.append({"op": "ag", "impl": "nccl", "dtype": "bf16", "bytes_per_rank": n, "world": 8, "us": 1.0, "busbw_gbs": 1})
    return rows


def test_variant_table_and_settings(tmp_path):
    path = tmp_path / "sweep.jsonl"
    path.write_text("noise line\n" + "\n".join(json.dumps(r) for r in _rows()))
    table = tuning.variant_table(tuning.load_sweep(str(path)))
    assert set(table) == {"ag", "rs_sum"}
    ag = {e["bytes"]: e["best"] for e in table["ag"]}
    assert ag[4096] == "p2p" and ag[1 << 28] == "ce" and "nccl" not in table["ag"][0]["us"]
    s = tuning.settings_from(table)
    lo, hi = s["MOODIST_NVLS_AG_MIN_BYTES"], s["MOODIST_NVLS_AG_MAX_BYTES"]
    assert 0 < lo <= hi and all(ag[b] == "nvls" for b in ag if lo <= b <= hi)
    assert s["MOODIST_NVLS_RS_MIN_BYTES"] == -1  # never fastest up to the largest size
    ce_from = s["MOODIST_CE_AUTO_BYTES"]
    rs = {e["bytes"]: e["best"] for e in table["rs_sum"]}
    assert ce_from > 0 and all(ag[b] == "ce" for b in ag if b >= ce_from)
    rs_from = s["MOODIST_CE_AUTO_RS_BYTES"]
    assert rs_from > 0 and all(rs[b] == "ce" for b in rs if b >= rs_from)
    text = tuning.format_table(table)
    assert "ag:" in text and "best" in text
    assert tuning.main([str(path), "--export"]) == 0


def test_apply_sets_environment(monkeypatch):
    monkeypatch.delenv("MOODIST_CE_AUTO_BYTES", raising=False)
    tuning.apply({"MOODIST_CE_AUTO_BYTES": 1 << 26})
    import os

    assert os.environ["MOODIST_CE_AUTO_BYTES"] == str(1 << 26)


def test_table_file_round_trip_through_the_native_loader(tmp_path):
    """The file `--table` writes is what a CUDA group reads at creation (MOODIST_VARIANT_TABLE)."""
    from moodist_b200._core import _C

    sweep = tmp_path / "sweep.jsonl"
    sweep.write_text("\n".join(json.dumps(r) for r in _rows()))
    path = tmp_path / "variants.json"
    assert tuning.main([str(sweep), "--table", str(path)]) == 0
    tuning.write_table(str(path), 2, {"MOODIST_CE_AUTO_BYTES": 123456, "MOODIST_NVLS_RS_MIN_BYTES": -1})
    want8 = tuning.settings_from(tuning.variant_table(tuning.load_sweep(str(sweep))))
    got8 = _C.load_variant_table(str(path), 8)
    assert got8 == {k: int(v) for k, v in want8.items()}
    assert _C.load_variant_table(str(path), 2) == {"MOODIST_CE_AUTO_BYTES": 123456, "MOODIST_NVLS_RS_MIN_BYTES": -1}
    assert _C.load_variant_table(str(path), 4) == {}
    bad = tmp_path / "bad.json"
    bad.write_text('{"8": ["not", "an", "object"]}')
    assert _C.load_variant_table(str(bad), 8) == {}
    assert _C.load_variant_table(str(tmp_path / "missing.json"), 8) == {}
