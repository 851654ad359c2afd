"""Terminal monitor for a training run: tails ``metrics.jsonl`` (and optionally log files) and redraws a compact
dashboard with sparklines (rollouts/tui/monitor.py:100-186, without the curses-style panes).

    python -m research_b200.utils.monitor runs/my_run/metrics.jsonl --keys loss mean_reward grad_norm step_s
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

BARS = "▁▂▃▄▅▆▇█"


def sparkline(values: list[float], width: int = 40) -> str:
    vals = [v for v in values[-width:] if v == v]          # drop NaN
    if not vals:
        return ""
    lo, hi = min(vals), max(vals)
    span = hi - lo
    return "".join(BARS[int((v - lo) / span * (len(BARS) - 1))] if span > 0 else BARS[0] for v in vals)


class MetricsTail:
    """Incrementally reads a JSONL file that another process appends to."""

    def __init__(self, path: str | Path):
        self.path, self.pos = Path(path), 0
        self.series: dict[str, list[float]] = {}
        self.last_step = -1
        self.bad_lines = 0

    def poll(self) -> int:
        if not self.path.exists():
            return 0
        n = 0
        with self.path.open() as f:
            f.seek(self.pos)
            while True:
                line = f.readline()
                if not line or not line.endswith("\n"):     # partial last line: read it next time
                    break
                self.pos = f.tell()
                try:
                    rec = json.loads(line)
                except json.JSONDecodeError:
                    self.bad_lines += 1
                    continue
                n += 1
                self.last_step = int(rec.get("step", self.last_step + 1))
                for k, v in rec.items():
                    if isinstance(v, (int, float)) and k != "step":
                        self.series.setdefault(k, []).append(float(v))
        return n

    def render(self, keys: list[str] | None = None, width: int = 40) -> str:
        keys = keys or sorted(self.series)[:12]
        lines = [f"{self.path}  step {self.last_step}  ({sum(len(v) for v in self.series.values())} values)"]
        for k in keys:
            v = self.series.get(k, [])
            if v:
                lines.append(f"{k:<22}{v[-1]:>12.5g}  min {min(v):<10.4g} max {max(v):<10.4g} {sparkline(v, width)}")
            else:
                lines.append(f"{k:<22}{'-':>12}")
        return "\n".join(lines)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("metrics")
    ap.add_argument("--keys", nargs="*", default=None)
    ap.add_argument("--interval", type=float, default=1.0)
    ap.add_argument("--once", action="store_true")
    args = ap.parse_args()
    tail = MetricsTail(args.metrics)
    drawn = 0
    while True:
        tail.poll()
        text = tail.render(args.keys)
        if sys.stdout.isatty() and drawn:
            sys.stdout.write(f"\x1b[{drawn}F\x1b[J")
        print(text, flush=True)
        drawn = text.count("\n") + 1
        if args.once:
            return
        time.sleep(args.interval)


if __name__ == "__main__":
    main()
