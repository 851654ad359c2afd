"""ncu report parsing, the metrics monitor and the phase timer."""

import json

from research_b200.utils.monitor import MetricsTail, sparkline
from research_b200.utils.ncu_report import aggregate_launch_list, compare, read_raw, summarise_launch
from research_b200.utils.timing import PhaseTimer


def test_ncu_raw_and_launch_list(tmp_path):
    raw = tmp_path / "raw.csv"
    raw.write_text('"ID","Kernel Name","gpu__time_duration.sum","sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",'
                   '"launch__grid_size","smsp__pcsamp_warps_issue_stalled_wait","smsp__pcsamp_warps_issue_stalled_barrier",'
                   '"smsp__pcsamp_warps_issue_stalled_wait_not_issued"\n'
                   '"","","us","%","","","",""\n'
                   '"0","k1(int)","74.2","56.2","148","300","100","290"\n'
                   '"1","k1(int)","60.0","70.0","148","100","100","90"\n')
    launches = read_raw(str(raw))
    assert len(launches) == 2
    s0, s1 = summarise_launch(launches[0]), summarise_launch(launches[1])
    assert s0["duration"] == "74.2 us" and s0["top stall reasons"].startswith("wait 75%")
    table = compare(s0, s1)
    assert any("duration" in line and "0.81x" in line for line in table)
    ll = tmp_path / "launches.csv"
    ll.write_text('==PROF== banner\n"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size",'
                  '"Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'
                  + "".join(f'"{i}","1","py","h","gemm","1","7","(192, 1, 1)","(148, 1, 1)","0","10.0","Cmd","gpu__time_duration.sum","ns","{v}"\n'
                            for i, v in enumerate(["10,000", "12,000"]))
                  + '"2","1","py","h","norm","1","7","(64, 1, 1)","(128, 1, 1)","0","10.0","Cmd","gpu__time_duration.sum","ns","2,000"\n')
    agg = aggregate_launch_list(str(ll))
    assert agg[0][0] == "gemm" and agg[0][2] == 2 and abs(agg[0][3] - 11.0) < 1e-6 and abs(agg[0][4] - 91.67) < 0.1


def test_metrics_tail_and_sparkline(tmp_path):
    assert sparkline([1, 2, 3, 4]) == "▁▃▅█" and sparkline([]) == "" and sparkline([5, 5]) == "▁▁"
    p = tmp_path / "metrics.jsonl"
    tail = MetricsTail(p)
    assert tail.poll() == 0
    with p.open("w") as f:
        for i in range(5):
            f.write(json.dumps({"step": i, "loss": 5.0 - i, "tag": "x"}) + "\n")
        f.write('{"step": 5, "loss": 0.')           # partial line, must be left for the next poll
    assert tail.poll() == 5 and tail.last_step == 4 and tail.series["loss"] == [5.0, 4.0, 3.0, 2.0, 1.0]
    with p.open("a") as f:
        f.write('5}\nnot json\n')
    assert tail.poll() == 1 and tail.series["loss"][-1] == 0.5 and tail.bad_lines == 1
    text = tail.render(["loss", "missing"])
    assert "loss" in text and "█" in text and "missing" in text


def test_phase_timer_cpu():
    t = PhaseTimer("cpu")
    with t.phase("a"):
        sum(range(1000))
    with t.phase("a"):
        pass
    with t.phase("b"):
        pass
    s = t.summary()
    assert set(s) == {"a_s", "b_s"} and s["a_s"] >= 0
    t.reset()
    assert t.summary() == {}


def test_grpo_bench_cpu_smoke():
    """The end-to-end GRPO step benchmark runs on the CPU twins and reports every phase."""
    import json
    import subprocess
    import sys

    proc = subprocess.run([sys.executable, "-m", "research_b200.utils.grpo_bench", "--model", "tiny-qwen2", "--prompts", "4",
                           "--samples", "4", "--prompt-len", "16", "--max-tokens", "8", "--steps", "1", "--minibatches", "2",
                           "--device", "cpu"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    row = json.loads([ln for ln in proc.stdout.splitlines() if ln.startswith("{")][-1])
    assert row["bench"] == "grpo_step" and row["samples_per_step"] == 16 and row["rollout_s"] > 0 and row["train_s"] > 0
    assert row["rollout_tokens_per_s"] > 0 and row["sync_s"] >= 0
