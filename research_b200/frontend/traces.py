"""Rollout trace viewer (rollouts/rollouts/tui/traces.py: ``TraceData``, ``StepPicker``): reads a run's
``rollouts.jsonl`` (one record per sample: step, group, reward, lengths and, when the run had a tokenizer, prompt /
response / ground truth), summarises every step and shows single samples.

    python -m research_b200.frontend.traces results/rl/<run>                 # table of steps
    python -m research_b200.frontend.traces results/rl/<run> --step 3        # the step's groups and samples
    python -m research_b200.frontend.traces results/rl/<run> --step 3 --sample 5
"""

from __future__ import annotations

import argparse
import json
import statistics
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from ..utils.monitor import sparkline


@dataclass(frozen=True)
class Trace:
    step: int
    index: int                          # position inside its step
    group: int | None
    reward: float
    tokens: int
    response_length: int
    prompt: str = ""
    response: str = ""
    ground_truth: str = ""
    extra: dict[str, Any] = field(default_factory=dict)


class TraceData:
    def __init__(self, traces: list[Trace]):
        self.traces = traces
        self.by_step: dict[int, list[Trace]] = {}
        for t in traces:
            self.by_step.setdefault(t.step, []).append(t)

    @staticmethod
    def load(run_dir: str | Path) -> "TraceData":
        d = Path(run_dir)
        files = sorted(d.glob("rollouts*.jsonl")) if d.is_dir() else ([d] if d.is_file() else [])
        traces, counters = [], {}
        for f in files:
            for raw in f.read_text(errors="replace").splitlines():
                try:
                    r = json.loads(raw)
                except json.JSONDecodeError:
                    continue
                step = int(r.get("step", 0))
                i = counters.get(step, 0)
                counters[step] = i + 1
                known = {"step", "group", "reward", "tokens", "response_length", "prompt", "response", "ground_truth"}
                traces.append(Trace(step, i, r.get("group"), float(r.get("reward") or 0.0), int(r.get("tokens", 0)), int(r.get("response_length", 0)),
                                    str(r.get("prompt", "")), str(r.get("response", "")), str(r.get("ground_truth", "")),
                                    {k: v for k, v in r.items() if k not in known}))
        return TraceData(traces)

    def steps(self) -> list[int]:
        return sorted(self.by_step)

    def step_summary(self, step: int) -> dict[str, float]:
        ts = self.by_step[step]
        rewards = [t.reward for t in ts]
        groups: dict[Any, list[float]] = {}
        for t in ts:
            groups.setdefault(t.group, []).append(t.reward)
        mixed = sum(1 for g in groups.values() if len(set(g)) > 1)
        return {"samples": len(ts), "mean_reward": statistics.fmean(rewards), "min_reward": min(rewards), "max_reward": max(rewards),
                "mean_response_length": statistics.fmean(t.response_length for t in ts), "groups": len(groups),
                "groups_with_signal": mixed}          # groups whose samples differ in reward: the ones GRPO learns from

    def render_steps(self) -> str:
        rows = ["step  samples  reward(mean/min/max)     resp.len  groups(signal)"]
        means = []
        for s in self.steps():
            m = self.step_summary(s)
            means.append(m["mean_reward"])
            rows.append(f"{s:>4}  {int(m['samples']):>7}  {m['mean_reward']:>6.3f} {m['min_reward']:>6.3f} {m['max_reward']:>6.3f}    "
                        f"{m['mean_response_length']:>8.1f}  {int(m['groups']):>3} ({int(m['groups_with_signal'])})")
        rows.append("mean reward per step  " + sparkline(means, 60))
        return "\n".join(rows)

    def render_step(self, step: int, width: int = 100) -> str:
        rows = [f"step {step}: " + ", ".join(f"{k} {v:.3g}" for k, v in self.step_summary(step).items())]
        for t in sorted(self.by_step[step], key=lambda t: (t.group if t.group is not None else -1, -t.reward)):
            head = f"[{t.index:>3}] group {t.group}  reward {t.reward:6.3f}  {t.response_length:>4} tok  "
            rows.append(head + (t.response.replace("\n", "\\n")[: max(10, width - len(head))] if t.response else ""))
        return "\n".join(rows)

    def render_sample(self, step: int, index: int) -> str:
        t = self.by_step[step][index]
        parts = [f"step {t.step} sample {t.index} group {t.group} reward {t.reward:.4f} ({t.response_length} response tokens of {t.tokens})"]
        if t.prompt:
            parts += ["--- prompt", t.prompt]
        if t.response:
            parts += ["--- response", t.response]
        if t.ground_truth:
            parts += ["--- ground truth", t.ground_truth]
        if t.extra:
            parts += ["--- other fields", json.dumps(t.extra)]
        return "\n".join(parts)


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description="Look at the rollouts of a training run")
    ap.add_argument("run_dir")
    ap.add_argument("--step", type=int, default=None)
    ap.add_argument("--sample", type=int, default=None)
    a = ap.parse_args(argv)
    data = TraceData.load(a.run_dir)
    if not data.traces:
        print(f"no rollouts*.jsonl records under {a.run_dir}")
        return 1
    if a.step is None:
        print(data.render_steps())
    elif a.step not in data.by_step:
        print(f"no step {a.step}; steps: {data.steps()}")
        return 1
    elif a.sample is None:
        print(data.render_step(a.step))
    else:
        print(data.render_sample(a.step, a.sample))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
