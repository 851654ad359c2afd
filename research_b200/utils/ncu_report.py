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


# ------------------------------------------------------------------------------------------- long-format reports
SM_PCT, DRAM_PCT, DURATION = "sm__throughput.avg.pct_of_peak_sustained_elapsed", "dram__throughput.avg.pct_of_peak_sustained_elapsed", "gpu__time_duration.sum"


def load_launches(path: str) -> list[dict]:
    """The ``--csv`` log of a metrics run (one row per launch AND metric) as one dict per launch: ``{"id", "kernel", "grid",
    "block", <metric name>: value ...}``; durations in nanoseconds whatever unit the report used."""
    rows = [r for r in csv.reader(open(path, newline="")) if len(r) > 10]
    if not rows:
        return []
    hdr = rows[0]
    col = {name: hdr.index(name) for name in ("ID", "Kernel Name", "Metric Name", "Metric Value") if name in hdr}
    if len(col) < 4:
        raise ValueError(f"{path} is not a per-metric ncu CSV (columns ID, Kernel Name, Metric Name, Metric Value expected)")
    ui = hdr.index("Metric Unit") if "Metric Unit" in hdr else None
    gi, bi = (hdr.index(n) if n in hdr else None for n in ("Grid Size", "Block Size"))
    to_ns = {"ns": 1.0, "nsecond": 1.0, "us": 1e3, "usecond": 1e3, "ms": 1e6, "msecond": 1e6, "s": 1e9, "second": 1e9}
    out: dict[str, dict] = {}
    for r in rows[1:]:
        d = out.setdefault(r[col["ID"]], {"id": r[col["ID"]], "kernel": r[col["Kernel Name"]], "grid": r[gi] if gi is not None else "",
                                          "block": r[bi] if bi is not None else ""})
        v = _num(r[col["Metric Value"]])
        if v is None:
            continue
        name = r[col["Metric Name"]]
        if name == DURATION and ui is not None:
            v *= to_ns.get(r[ui].strip().lower(), 1.0)
        d[name] = v
    return list(out.values())


def summarize_kernels(launches: list[dict]) -> list[dict]:
    """Per kernel name: launches, total / mean / min / max duration (us), share of the total time, mean SM and DRAM
    throughput (% of peak) where the report has them. Longest total first."""
    groups: dict[str, list[dict]] = defaultdict(list)
    for l in launches:
        groups[l["kernel"]].append(l)
    total = sum(l.get(DURATION, 0.0) for l in launches) or 1.0
    out = []
    for name, ls in groups.items():
        ds = [l.get(DURATION, 0.0) for l in ls]
        mean = (lambda key: (sum(l[key] for l in ls if key in l) / max(sum(1 for l in ls if key in l), 1)) if any(key in l for l in ls) else None)
        out.append({"kernel": name, "launches": len(ls), "total_us": sum(ds) / 1e3, "mean_us": sum(ds) / len(ds) / 1e3, "min_us": min(ds) / 1e3,
                    "max_us": max(ds) / 1e3, "pct_total_time": 100.0 * sum(ds) / total, "sm_pct": mean(SM_PCT), "dram_pct": mean(DRAM_PCT)})
    return sorted(out, key=lambda r: -r["total_us"])


def find_bottlenecks(launches: list[dict], top_n: int = 10, sm_floor: float = 50.0, dram_floor: float = 10.0, min_us: float = 10.0) -> list[dict]:
    """Launches that leave the machine idle, worst first: neither the SMs (below ``sm_floor`` % of peak) nor DRAM (below
    ``dram_floor`` %) is busy and the launch is long enough to matter. Severity = duration x how far below the floor the
    busier of the two sits; such a launch is latency-, occupancy- or launch-bound, and its stall reasons say which."""
    out = []
    for l in launches:
        us = l.get(DURATION, 0.0) / 1e3
        sm, dram = l.get(SM_PCT), l.get(DRAM_PCT)
        if us < min_us or sm is None:
            continue
        if sm < sm_floor and (dram is None or dram < dram_floor):
            kind = "neither compute nor memory busy" if dram is not None else "low SM throughput"
            out.append({"kernel": l["kernel"], "id": l["id"], "grid": l["grid"], "duration_us": us, "sm_pct": sm, "dram_pct": dram, "kind": kind,
                        "severity": us * (sm_floor - sm)})
    return sorted(out, key=lambda r: -r["severity"])[:top_n]


def compare_backends(baseline: list[dict], other: list[dict]) -> dict:
    """Totals of two reports of the same workload (e.g. a library kernel and a hand-written one): time, speed-up, launch
    counts, mean throughputs."""
    def side(ls: list[dict]) -> dict:
        tot = sum(l.get(DURATION, 0.0) for l in ls)
        avg = (lambda key: (sum(l[key] for l in ls if key in l) / max(sum(1 for l in ls if key in l), 1)) if any(key in l for l in ls) else None)
        return {"total_us": tot / 1e3, "launches": len(ls), "avg_sm_pct": avg(SM_PCT), "avg_dram_pct": avg(DRAM_PCT)}

    a, b = side(baseline), side(other)
    return {"baseline": a, "other": b, "speedup": a["total_us"] / b["total_us"] if b["total_us"] > 0 else None}


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
    if "Metric Name" in head and "Metric Value" in head and len(argv) == 2:
        c = compare_backends(load_launches(argv[0]), load_launches(argv[1]))
        for side in ("baseline", "other"):
            r = c[side]
            print(f"{side:<9}{r['total_us']:12.1f} us in {r['launches']} launches" + (f", SM {r['avg_sm_pct']:.0f}%" if r["avg_sm_pct"] is not None else "") +
                  (f", DRAM {r['avg_dram_pct']:.0f}%" if r["avg_dram_pct"] is not None else ""))
        print(f"speed-up {c['speedup']:.2f}x" if c["speedup"] else "no durations to compare")
        return 0
    if "Metric Name" in head and "Metric Value" in head and len(argv) == 1:
        for name, grid, n, mean_us, share in aggregate_launch_list(argv[0]):
            print(f"{share:5.1f}%  {n:5d} x {mean_us:9.2f} us  grid {grid:<16} {name}")
        slow = find_bottlenecks(load_launches(argv[0]))
        if slow:
            print("\nlaunches that keep neither the SMs nor DRAM busy:")
            for b in slow:
                print(f"  {b['duration_us']:9.1f} us  SM {b['sm_pct']:4.0f}%  DRAM {(b['dram_pct'] if b['dram_pct'] is not None else float('nan')):4.0f}%  {b['kernel'][:60]}")
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
