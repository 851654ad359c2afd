"""Summarise and compare Nsight Compute captures (dev/kernels-gpumode/analyze_ncu.py:32-286).

    ncu -i prof.ncu-rep --page raw --csv > prof.csv
    python -m research_b200.utils.ncu_report prof.csv                 # one table per captured launch
    python -m research_b200.utils.ncu_report before.csv after.csv     # side by side with ratios

Also reads the launch list written by ``ncu --metrics gpu__time_duration.sum --csv --log-file launches.csv``
(one row per launch and metric) and aggregates it per kernel name and grid.
"""

from __future__ import annotations

import csv
import sys
from collections import defaultdict

KEY_METRICS = [
    ("gpu__time_duration.sum", "duration"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "tensor pipe % of active"),
    ("dram__bytes_read.sum", "DRAM read"),
    ("dram__bytes_write.sum", "DRAM write"),
    ("dram__throughput.avg.pct_of_peak_sustained_elapsed", "DRAM % of peak"),
    ("lts__t_sector_hit_rate.pct", "L2 hit %"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "warps active %"),
    ("smsp__issue_active.avg.pct_of_peak_sustained_active", "issue slots busy %"),
    ("launch__registers_per_thread", "registers / thread"),
    ("launch__grid_size", "grid"),
]
STALL_PREFIX = "smsp__pcsamp_warps_issue_stalled_"


def read_raw(path: str) -> list[dict[str, str]]:
    """``--page raw --csv``: header row, a units row, then one row per captured launch."""
    rows = list(csv.reader(open(path, newline="")))
    rows = [r for r in rows if len(r) > 5]
    header, body = rows[0], rows[1:]
    if body and not body[0][0].strip().isdigit():       # units row
        units, body = body[0], body[1:]
    else:
        units = [""] * len(header)
    out = []
    for r in body:
        d = {h: v for h, v in zip(header, r)}
        d["__units__"] = {h: u for h, u in zip(header, units)}  # type: ignore[assignment]
        out.append(d)
    return out


def summarise_launch(d: dict) -> dict[str, str]:
    units = d.get("__units__", {})
    out = {"kernel": d.get("Kernel Name", "?")[:70]}
    for key, label in KEY_METRICS:
        if key in d and d[key] != "":
            out[label] = f"{d[key]} {units.get(key, '')}".strip()
    stalls = {k[len(STALL_PREFIX):]: float(v.replace(",", "")) for k, v in d.items()
              if isinstance(v, str) and k.startswith(STALL_PREFIX) and not k.endswith("_not_issued") and v.replace(",", "").replace(".", "").isdigit()}
    total = sum(stalls.values())
    if total > 0:
        top = sorted(stalls.items(), key=lambda kv: -kv[1])[:4]
        out["top stall reasons"] = ", ".join(f"{k} {100 * v / total:.0f}%" for k, v in top)
    return out


def aggregate_launch_list(path: str) -> list[tuple[str, str, int, float, float]]:
    """Launch-list CSV -> [(kernel, grid, launches, mean us, share %)] sorted by total time."""
    rows = [r for r in csv.reader(open(path, newline="")) if len(r) > 10]
    hdr = rows[0]
    ki, vi, gi, mi = hdr.index("Kernel Name"), hdr.index("Metric Value"), hdr.index("Grid Size"), hdr.index("Metric Name")
    agg: dict[tuple[str, str], list[float]] = defaultdict(list)
    for r in rows[1:]:
        if r[mi] == "gpu__time_duration.sum":
            agg[(r[ki][:60], r[gi])].append(float(r[vi].replace(",", "")))
    total = sum(sum(v) for v in agg.values()) or 1.0
    out = [(k[0], k[1], len(v), sum(v) / len(v) / 1000.0, 100.0 * sum(v) / total) for k, v in agg.items()]
    return sorted(out, key=lambda t: -t[2] * t[3])


def _num(s: str) -> float | None:
    try:
        return float(s.split()[0].replace(",", ""))
    except (ValueError, IndexError):
        return None


def compare(a: dict[str, str], b: dict[str, str]) -> list[str]:
    lines = [f"{'metric':<28}{'before':>22}{'after':>22}{'ratio':>9}"]
    for key in [k for k in a if k in b and k != "kernel"]:
        x, y = _num(a[key]), _num(b[key])
        ratio = f"{y / x:.2f}x" if x and y is not None and x != 0 else ""
        lines.append(f"{key:<28}{a[key]:>22}{b[key]:>22}{ratio:>9}")
    return lines


def main(argv: list[str]) -> int:
    if not argv:
        print(__doc__)
        return 2
    head = "".join(open(argv[0]).readlines()[:60])
    if "Metric Name" in head and "Metric Value" in head and len(argv) == 1:
        for name, grid, n, mean_us, share in aggregate_launch_list(argv[0]):
            print(f"{share:5.1f}%  {n:5d} x {mean_us:9.2f} us  grid {grid:<16} {name}")
        return 0
    reports = [[summarise_launch(d) for d in read_raw(p)] for p in argv[:2]]
    if len(reports) == 1:
        for s in reports[0]:
            print("\n".join(f"{k:<28}{v}" for k, v in s.items()) + "\n")
        return 0
    for a, b in zip(*reports):
        print(a["kernel"])
        print("\n".join(compare(a, b)) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
