"""Performance history in a CSV file, in the manner of the reference's benchmark driver
(benchmark/README.md:84-103: --csv FILE with --generate, --update or --compare).

A record is keyed by (Device, Op, dtype, Shape).  generate: add the record when the key is new; update: replace the
stored record only when the new GPU time is more than 5 % better; compare: report new against stored, change nothing.
The columns follow the reference's report (Op, dtype, Shape, Samples, GPU Time, GlobalMem BW, BWUtil)."""
from __future__ import annotations

import csv
import os
from typing import Dict, Iterable, List, Tuple

COLUMNS = ["Device", "Op", "dtype", "Shape", "Samples", "GPU Time (us)", "GlobalMem BW (GB/s)", "BWUtil (%)"]
KEY = ("Device", "Op", "dtype", "Shape")
UPDATE_THRESHOLD = 0.05


def make_record(device: str, op: str, dtype: str, shape: str, samples: int, gpu_time_us: float, gb_per_s: float,
                peak_gb_per_s: float) -> Dict[str, str]:
    return {"Device": device, "Op": op, "dtype": dtype, "Shape": shape, "Samples": str(int(samples)),
            "GPU Time (us)": f"{gpu_time_us:.3f}", "GlobalMem BW (GB/s)": f"{gb_per_s:.1f}",
            "BWUtil (%)": f"{100.0 * gb_per_s / peak_gb_per_s:.2f}"}


def load(path: str) -> List[Dict[str, str]]:
    if not os.path.exists(path):
        return []
    with open(path, newline="") as fh:
        return [dict(r) for r in csv.DictReader(fh)]


def save(path: str, rows: Iterable[Dict[str, str]]) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w", newline="") as fh:
        w = csv.DictWriter(fh, fieldnames=COLUMNS)
        w.writeheader()
        for r in rows:
            w.writerow({c: r.get(c, "") for c in COLUMNS})


def _key(r: Dict[str, str]) -> Tuple[str, ...]:
    return tuple(r[k] for k in KEY)


def apply(path: str, new: List[Dict[str, str]], mode: str) -> List[Dict[str, object]]:
    """mode: "generate" | "update" | "compare".  Returns one report entry per new record:
    {key, action: added|kept|updated|compared|missing, old_us, new_us, change} (change = new/old - 1, negative = faster)."""
    assert mode in ("generate", "update", "compare")
    rows = load(path)
    index = {_key(r): i for i, r in enumerate(rows)}
    report = []
    dirty = False
    for r in new:
        k = _key(r)
        new_us = float(r["GPU Time (us)"])
        if k not in index:
            if mode == "compare":
                report.append({"key": k, "action": "missing", "old_us": None, "new_us": new_us, "change": None})
                continue
            rows.append(r)
            index[k] = len(rows) - 1
            dirty = True
            report.append({"key": k, "action": "added", "old_us": None, "new_us": new_us, "change": None})
            continue
        old_us = float(rows[index[k]]["GPU Time (us)"])
        change = new_us / old_us - 1.0 if old_us > 0 else None
        if mode == "update" and old_us > 0 and new_us < old_us * (1.0 - UPDATE_THRESHOLD):
            rows[index[k]] = r
            dirty = True
            action = "updated"
        else:
            action = "compared" if mode == "compare" else "kept"
        report.append({"key": k, "action": action, "old_us": old_us, "new_us": new_us, "change": change})
    if dirty:
        save(path, rows)
    return report


def format_report(report: List[Dict[str, object]]) -> str:
    lines = []
    for e in report:
        op = e["key"][1]
        if e["old_us"] is None:
            lines.append(f"{op:28s} {e['action']:9s} new {e['new_us']:.3f} us")
        else:
            lines.append(f"{op:28s} {e['action']:9s} old {e['old_us']:.3f} us  new {e['new_us']:.3f} us  ({100.0 * e['change']:+.1f} %)")
    return "\n".join(lines)
