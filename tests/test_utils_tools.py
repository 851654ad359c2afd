"""ncu report parsing, the metrics monitor and the phase timer."""

import json
import pytest
import torch

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


def test_print_capture_and_validation(tmp_path):
    import logging

    import pytest

    from research_b200.utils.print_capture import intercept_prints
    from research_b200.utils.validation import (parse_ssh_target, validate_hostname, validate_port, validate_ssh_key_path,
                                                validate_timeout, validate_username)

    records = []

    class H(logging.Handler):
        def emit(self, r):
            records.append((r.levelno, r.getMessage()))

    log = logging.getLogger("capture-test")
    log.setLevel(logging.DEBUG)
    log.addHandler(H())
    import sys
    before = sys.stdout
    with intercept_prints(log, intercept_stderr=True):
        print("hello", end="")
        print(" world")
        print("second line")
        print("oops", file=sys.stderr)
        print("tail without newline", end="")
    assert sys.stdout is before
    assert (logging.INFO, "hello world") in records and (logging.INFO, "second line") in records
    assert (logging.ERROR, "oops") in records and (logging.INFO, "tail without newline") in records
    with pytest.raises(RuntimeError):
        with intercept_prints(log):
            raise RuntimeError("x")
    assert sys.stdout is before

    assert validate_port(22) == 22 and validate_timeout(2.5) == 2.5 and validate_hostname("gpu-1.example.org") == "gpu-1.example.org"
    assert parse_ssh_target("root@10.0.0.5:2222") == ("root", "10.0.0.5", 2222) and parse_ssh_target("me@host")[2] == 22
    for bad in (lambda: validate_port(0), lambda: validate_port(True), lambda: validate_timeout(0), lambda: validate_hostname("a b"),
                lambda: validate_username("1abc"), lambda: parse_ssh_target("nohost"), lambda: validate_ssh_key_path(str(tmp_path / "none"))):
        with pytest.raises(ValueError):
            bad()
    key = tmp_path / "id"
    key.write_text("k")
    key.chmod(0o644)
    with pytest.raises(ValueError):
        validate_ssh_key_path(str(key))
    key.chmod(0o600)
    assert validate_ssh_key_path(str(key)) == str(key)


def test_kernel_harness_checks_times_and_round_trips(tmp_path):
    from research_b200.utils import kernel_harness as kh

    reg = kh.nvfp4_backends()
    assert "reference" in reg and "native" in reg and "library_scaled_mm" in reg and len(reg) == 3
    with pytest.raises(ValueError):
        reg.register("reference", lambda x: x[0])
    with pytest.raises(ValueError):
        reg.register("odd", lambda x: x[0], language="fortran")

    from research_b200.ops import nvfp4

    def fp32_dot(x):                      # a second honest implementation: fp32 accumulation
        a, b, sfa, sfb = x
        av = nvfp4.decode_e2m1(a) * nvfp4.decode_e4m3(sfa).repeat_interleave(16, dim=-1)
        bv = nvfp4.decode_e2m1(b) * nvfp4.decode_e4m3(sfb).repeat_interleave(16, dim=-1)
        return torch.einsum("lmk,lk->lm", av, bv).to(torch.float16)

    def off_by_a_bit(x):
        return fp32_dot(x) + 0.5

    def broken(x):
        raise RuntimeError("no kernel image")

    reg.register("fp32", fp32_dot, "fp32 accumulate", "pytorch")
    reg.register("biased", off_by_a_bit, "wrong on purpose", "pytorch")
    reg.register("broken", broken, "raises", "other")
    lines = []
    res = kh.run_suite(reg, correctness_cases=kh.SMOKE, performance_cases=[kh.GemvCase(128, 256, 1, 7, "p")], iters=3, log=lines.append)
    assert res.get("reference").all_correct and res.get("fp32").all_correct
    assert res.get("native").skipped and not res.get("native").correctness
    assert res.get("biased").correctness_score == 0.0 and "elements differ" in res.get("biased").correctness[0].detail
    assert "RuntimeError" in res.get("broken").correctness[0].detail and not res.get("broken").performance
    assert res.get("reference").performance[0].speedup == pytest.approx(1.0)
    assert res.get("fp32").geomean_speedup > 0 and res.get("fp32").performance[0].gbs > 0
    table = res.table()
    assert "skipped" in table and "2/2" in table and "0/2" in table
    p = tmp_path / "r.json"
    res.to_json(p)
    back = kh.SuiteResults.from_json(p)
    assert back.to_dict() == res.to_dict() and back.get("fp32").avg_speedup == pytest.approx(res.get("fp32").avg_speedup)
    # same seed, same bytes; different seed, different bytes
    a1, a2, a3 = kh.SMOKE[0].generate()[0], kh.SMOKE[0].generate()[0], kh.SMOKE[1].generate()[0]
    assert torch.equal(a1, a2) and a1.shape != a3.shape
    ok, rep = kh.closeness(torch.ones(2, 3), torch.ones(3, 2))
    assert not ok and "shape" in rep
    ok, rep = kh.closeness(torch.tensor([1.0, float("inf")]), torch.tensor([1.0, 2.0]))
    assert not ok and "non-finite" in rep
    assert kh.main(["--tier", "smoke", "--backends", "reference", "--device", "cpu"]) == 0
    assert kh.main(["--list"]) == 0


def test_ncu_long_format_summary_bottlenecks_and_comparison(tmp_path, capsys):
    from research_b200.utils import ncu_report as nr

    hdr = '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"'

    def rows(i, name, grid, dur_us, sm, dram):
        base = f'"{i}","1","python","box","{name}","1","7","(256, 1, 1)","{grid}","0","10.0","Sec",'
        return [base + f'"gpu__time_duration.sum","us","{dur_us}"', base + f'"{nr.SM_PCT}","%","{sm}"', base + f'"{nr.DRAM_PCT}","%","{dram}"']

    a = tmp_path / "a.csv"
    a.write_text("\n".join([hdr] + rows(0, "gemm_kernel", "(148, 1, 1)", "1,200.5", 82, 35) + rows(1, "tiny_norm", "(8, 1, 1)", 45, 6, 3) +
                           rows(2, "gemm_kernel", "(148, 1, 1)", 1100, 80, 33) + rows(3, "copy_kernel", "(592, 1, 1)", 300, 12, 88) + rows(4, "blip", "(1, 1, 1)", 2, 1, 1)) + "\n")
    launches = nr.load_launches(str(a))
    assert len(launches) == 5 and launches[0][nr.DURATION] == 1200.5e3 and launches[0]["grid"] == "(148, 1, 1)"
    summary = nr.summarize_kernels(launches)
    assert [s["kernel"] for s in summary][:2] == ["gemm_kernel", "copy_kernel"] and summary[0]["launches"] == 2 and abs(summary[0]["sm_pct"] - 81) < 1e-9
    assert abs(sum(s["pct_total_time"] for s in summary) - 100) < 1e-6
    slow = nr.find_bottlenecks(launches)
    assert [b["kernel"] for b in slow] == ["tiny_norm"] and slow[0]["kind"].startswith("neither")        # copy is DRAM-bound, blip too short
    b = tmp_path / "b.csv"
    b.write_text("\n".join([hdr] + rows(0, "fused_kernel", "(148, 1, 1)", 1300, 85, 40)) + "\n")
    c = nr.compare_backends(launches, nr.load_launches(str(b)))
    assert abs(c["speedup"] - (1200.5 + 45 + 1100 + 300 + 2) / 1300) < 1e-9 and c["other"]["launches"] == 1
    assert nr.main([str(a), str(b)]) == 0 and "speed-up 2.04x" in capsys.readouterr().out
    assert nr.main([str(a)]) == 0
    out = capsys.readouterr().out
    assert "gemm_kernel" in out and "neither the SMs nor DRAM" in out and "tiny_norm" in out


def test_harness_profile_table_and_ncu_command(tmp_path):
    import torch

    from research_b200.utils.kernel_harness import ncu_command, profile_kernel

    a = torch.randn(64, 64)
    table = profile_kernel(lambda: (a @ a).relu_(), iters=3, trace_path=tmp_path / "trace.json")
    assert "aten::mm" in table or "aten::matmul" in table
    assert (tmp_path / "trace.json").stat().st_size > 100
    cmd = ncu_command(["python", "-m", "research_b200.utils.kernel_harness", "--tier", "smoke"], "gemv", launches=2, skip=4)
    assert cmd[:3] == ["ncu", "--clock-control", "none"] and cmd[cmd.index("-c") + 1] == "2" and cmd[cmd.index("-s") + 1] == "4" and "--set" in cmd
    light = ncu_command(["python", "x.py"], "k", full=False)
    assert light.count("--section") == 2 and "--set" not in light and light[-2:] == ["python", "x.py"]


def test_tracker_writes_runs_and_the_viewer_draws_them(tmp_path):
    """Two runs logged through the Tracker: file layout, auto-incremented steps, non-JSON values coerced, meta closed by
    finish / by an exception; the viewer lists both, tabulates latest values and draws braille charts on a shared scale."""
    import io
    import json

    import pytest
    import torch

    from research_b200.utils.tracker import Tracker, braille_chart, list_runs, load_run, main, render, watch

    t = [1000.0]
    clock = lambda: t[0]                                                        # noqa: E731
    a = Tracker("baseline", config={"lr": 0.1}, dir=tmp_path, run_id="run-a", clock=clock)
    for i in range(50):
        t[0] += 1
        assert a.log({"loss": 3.0 * 0.95**i, "acc": torch.tensor(i / 50), "note": object()}) == i
    assert a.log({"loss": 0.2}, step=100) == 100
    a.log_system({"gpu_util": 0.9})
    a.finish()
    t[0] += 10
    with pytest.raises(RuntimeError):
        with Tracker("variant", config={"lr": 0.3}, dir=tmp_path, run_id="run-b", clock=clock) as b:
            for i in range(20):
                b.log({"loss": 3.0 * 0.8**i})
            raise RuntimeError("boom")
    live = Tracker("live", dir=tmp_path, run_id="run-c", clock=clock)
    live.log({"loss": 1.0})

    meta = json.loads((tmp_path / "run-a" / "meta.json").read_text())
    assert meta["name"] == "baseline" and meta["finished_at"] == t[0] - 10 and meta["status"] == "finished"
    assert json.loads((tmp_path / "run-b" / "meta.json").read_text())["status"] == "failed"
    first = json.loads((tmp_path / "run-a" / "metrics.jsonl").read_text().splitlines()[0])
    assert first["_step"] == 0 and first["acc"] == 0.0 and isinstance(first["note"], str)
    assert json.loads((tmp_path / "run-a" / "system.jsonl").read_text())["gpu_util"] == 0.9

    runs = list_runs(tmp_path)
    assert [r.run_id for r in runs] == ["run-a", "run-b", "run-c"]
    run = load_run(tmp_path / "run-a")
    xs, ys = run.series("loss")
    assert xs[-1] == 100 and ys[-1] == 0.2 and run.metrics() == ["loss", "acc"] and run.latest("nothing") is None
    assert list_runs(tmp_path / "run-a")[0].run_id == "run-a"

    chart = braille_chart([run.series("loss"), runs[1].series("loss")], width=40, height=6)
    assert len(chart) == 8 and chart[0].lstrip().startswith("3") and all(len(row.split("|", 1)[1]) == 40 for row in chart[:6])
    dots = "".join(chart[:6])
    assert sum(0x2800 < ord(c) <= 0x28FF for c in dots) >= 40                   # a connected line, not scattered points
    first_row, last_row = chart[0].split("|", 1)[1], chart[5].split("|", 1)[1]
    assert first_row.strip() and first_row.index(first_row.strip()[0]) < 3      # the decaying loss starts top left ...
    assert last_row.rstrip() and len(last_row.rstrip()) > 30                    # ... and ends bottom right
    assert braille_chart([([], [])]) == ["(no data)"] and len(braille_chart([([0, 1], [2.0, 2.0])], 10, 3)) == 5

    text = render(tmp_path, width=40, height=6)
    assert "run-a" in text and "run-b" in text and "* run-c" in text and "latest:" in text and "\nloss\n" in text and "\nacc\n" in text
    row = next(ln for ln in text.splitlines() if ln.strip().startswith("loss") and "[" not in ln and "|" not in ln)
    assert "0.2" in row and "-" not in row.split()[1:]
    assert "no run has it" in render(tmp_path, metrics=["ghost"]) and "run-b" not in render(tmp_path, run_filter="baseline")
    assert render(tmp_path / "empty") .startswith("no runs")

    out = io.StringIO()
    watch(tmp_path, out=out, iterations=2, sleep=lambda s: live.log({"loss": 0.5}), width=30, height=4)
    assert out.getvalue().count("runs:") == 2                                   # redrawn because a file grew
    out = io.StringIO()
    live.finish()
    watch(tmp_path, out=out, iterations=3, sleep=lambda s: None, width=30, height=4)
    assert out.getvalue().count("runs:") == 1                                   # nothing changed: drawn once
    assert main([str(tmp_path), "--metric", "loss", "--no-colour"]) == 0


def test_tracker_is_a_metrics_sink_and_has_a_command(tmp_path, capsys):
    from research_b200.cli import main
    from research_b200.training.metrics import MetricsLogger
    from research_b200.utils.tracker import Tracker

    t = Tracker("x", dir=tmp_path, run_id="run-x")
    assert isinstance(t, MetricsLogger)
    t.log({"loss": 1.5}, 7)
    t.finish()
    assert main(["track", str(tmp_path), "--no-colour"]) == 0
    assert "run-x" in capsys.readouterr().out
