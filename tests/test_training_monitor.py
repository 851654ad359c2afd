"""The multi-pane training monitor: parsing, routing, series, keys, rendering, replay of a run directory."""

import io
import json

from research_b200.frontend.training_monitor import TrainingMonitor, main, replay_lines


def _log(logger, msg, level="INFO", **extra):
    return json.dumps({"timestamp": "2025-01-01T12:00:00.000Z", "level": level, "logger": logger, "message": msg, **extra})


def test_routing_series_and_rendering():
    mon = TrainingMonitor()
    mon.feed([_log("research_b200.training.grpo", f"step {i} done", step=i, loss=1.0 / (i + 1), mean_reward=i * 0.1) for i in range(30)])
    mon.feed([_log("research_b200.inference.engine", "scheduled 8 sequences"), _log("other.module", "hello"), "plain text line", "", "{broken json",
              _log("research_b200.training.grpo", "boom", level="ERROR", exception="Traceback...\nValueError: x"),
              json.dumps({"step": 30, "loss": 0.01, "grad_norm": 2.0})])
    by = {p.name: p for p in mon.panes}
    assert len(by["training"].lines) == 30 + 1 + 2 and len(by["engine"].lines) == 1 and len(by["metrics"].lines) == 1
    assert len(by["all"].lines) == 30 + 7 - 1 - 0                       # everything except the empty line
    assert mon.errors == 1 and mon.last_step == 30 and len(mon.series["loss"]) == 31 and list(mon.series["grad_norm"]) == [2.0]
    screen = mon.render(100, 12, color=False)
    assert len(screen) == 12 and "1:training" in screen[0] and "ValueError: x" in "\n".join(screen) and "1 errors" in screen[-2]
    assert "follow" in screen[-2] and "step 30" in screen[-2]
    mon.handle_key("g", 12)
    top = mon.render(100, 12, color=False)
    assert "step 0 done" in top[1] and "paused" in top[-2]
    mon.handle_key("j", 12)
    assert "step 1 done" in mon.render(100, 12, color=False)[1]
    mon.handle_key("G", 12)
    assert "boom" in "\n".join(mon.render(100, 12, color=False))
    mon.handle_key("l", 12)
    assert mon.panes[0].hscroll == 10
    mon.handle_key("h", 12)
    mon.handle_key("3", 12)
    charts = mon.render(100, 12, color=False)
    assert charts[1].startswith("grad_norm") and any(r.startswith("loss") and "▁" in r for r in charts)
    mon.handle_key("j", 12)
    assert mon.render(100, 12, color=False)[1].startswith("loss")
    mon.handle_key("k", 12)
    mon.handle_key("2", 12)
    assert "scheduled 8 sequences" in mon.render(100, 12, color=False)[1]
    colored = mon.render(100, 12)
    assert "\x1b[7m" in colored[0]
    mon.handle_key("q")
    assert not mon.running


def test_replay_directory_and_cli(tmp_path, capsys):
    run = tmp_path / "run"
    run.mkdir()
    (run / "training.log").write_text("\n".join([_log("research_b200.training.grpo", "starting"), "a plain line"]) + "\n")
    (run / "metrics.jsonl").write_text("\n".join(json.dumps({"step": i, "loss": 2.0 - i * 0.5}) for i in range(3)) + "\n")
    (run / "rollouts.jsonl").write_text(json.dumps({"tokens": [1, 2, 3]}) + "\n")
    lines = replay_lines(run)
    assert len(lines) == 5 and lines[0].startswith("{") and '"logger": "metrics"' in lines[-1]
    assert main(["--replay", str(run), "--once"]) == 0
    out = capsys.readouterr().out
    assert "starting" in out and "a plain line" in out and "step 2" in out
    mon = TrainingMonitor()
    mon.run(io.StringIO(_log("training", "from a stream", step=7) + "\n"))          # not a tty: feeds, prints once, returns
    assert "from a stream" in capsys.readouterr().out and mon.last_step == 7


def test_trace_viewer_on_a_real_run(tmp_path, capsys):
    import sys
    from dataclasses import replace
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))
    from examples.rl.reverse_text.base_config import DEFAULT, train
    from research_b200.frontend.traces import TraceData, main as traces_main

    train(replace(DEFAULT, num_steps=2, output_dir=str(tmp_path), batch_size=2, n_samples_per_prompt=2, max_tokens=6, num_minibatches=1),
          num_samples=4, device="cpu")
    run = next(p for p in tmp_path.iterdir() if p.is_dir())
    data = TraceData.load(run)
    assert data.steps() == [0, 1] and len(data.traces) == 8
    t = data.by_step[0][0]
    assert t.prompt and t.ground_truth == t.prompt[::-1] and t.response_length == 6 and "weight_version" in t.extra
    s = data.step_summary(1)
    assert s["samples"] == 4 and s["groups"] == 2 and s["min_reward"] <= s["mean_reward"] <= s["max_reward"]
    assert traces_main([str(run)]) == 0 and "mean reward per step" in capsys.readouterr().out
    assert traces_main([str(run), "--step", "1"]) == 0 and "group" in capsys.readouterr().out
    assert traces_main([str(run), "--step", "1", "--sample", "0"]) == 0
    out = capsys.readouterr().out
    assert "--- prompt" in out and "--- ground truth" in out
    assert traces_main([str(run), "--step", "9"]) == 1 and traces_main([str(tmp_path / "none")]) == 1
    # the monitor's replay skips rollout records but shows the run's metrics
    from research_b200.frontend.training_monitor import TrainingMonitor, replay_lines

    mon = TrainingMonitor()
    mon.feed(replay_lines(run))
    assert "mean_reward" in mon.series and mon.last_step is not None


def test_cli_delegates_to_the_tools(tmp_path, capsys):
    from research_b200.cli import main as cli

    (tmp_path / "rollouts.jsonl").write_text(json.dumps({"step": 0, "reward": 1.0, "group": 0, "tokens": 5, "response_length": 2}) + "\n")
    assert cli(["traces", str(tmp_path)]) == 0 and "mean reward per step" in capsys.readouterr().out
    (tmp_path / "training.log").write_text(_log("training", "hello monitor") + "\n")
    assert cli(["monitor", "--replay", str(tmp_path), "--once"]) == 0 and "hello monitor" in capsys.readouterr().out
    assert cli(["infra", "remote", "exec", "local", "echo via-cli"]) == 0 and "via-cli" in capsys.readouterr().out
    assert cli(["kernel-harness", "--list"]) == 0 and "reference" in capsys.readouterr().out
