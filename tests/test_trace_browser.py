"""Hierarchical trace browser and the merged-log runner, driven without a terminal."""

import io
import json
import sys
import threading
import time

from research_b200.frontend.remote_runner import run_training_with_json_logging, tail_file_as_jsonl
from research_b200.frontend.trace_browser import (POP, Browser, GroupPicker, RolloutPicker, StepPicker, TraceData, TraceViewer,
                                                  decode_keys, ingest_line, main)


def _records():
    recs = []
    for step in (0, 1):
        for g in range(3):
            for s in range(4):
                recs.append({"step": step, "group_index": g, "sample_id": f"s{step}_{g}_{s}", "prompt": f"prompt {g}",
                             "response": f"answer {s}\n" + "line\n" * (20 if s == 3 else 1), "reward": float((s + g + step) % 2)})
    recs[0]["messages"] = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "prompt 0"},
                           {"role": "assistant", "content": [{"type": "text", "text": "calling"}]},
                           {"role": "tool", "content": "42"}, {"role": "assistant", "content": "done\n" * 30}]
    return recs


def test_data_model_groups_updates_and_rewards(tmp_path):
    p = tmp_path / "rollouts.jsonl"
    p.write_text("\n".join(json.dumps(r) for r in _records()) + "\nnot json\n")
    data = TraceData.from_jsonl(p)
    assert [s.step for s in data.steps] == [0, 1] and data.steps[0].num_rollouts == 12 and len(data.steps[0].groups) == 3
    g = data.steps[0].groups[1]
    assert (g.min_reward, g.max_reward, g.avg_reward, g.has_signal) == (0.0, 1.0, 0.5, True)
    assert TraceData.from_jsonl(tmp_path).steps[1].avg_reward == data.steps[1].avg_reward     # a run directory works too
    # a record with a known sample id updates in place; without group_index the prompt decides the group
    r = data.add_record({"step": 0, "sample_id": "s0_0_1", "response": "better", "reward": 3.0})
    assert r is data.find_rollout("s0_0_1") and r.reward == 3.0 and data.steps[0].num_rollouts == 12
    a = data.add_record({"step": 5, "prompt": "same text", "response": "x", "reward": 1.0})
    b = data.add_record({"step": 5, "prompt": "same text", "response": "y", "reward": 0.0})
    assert a.group_id == b.group_id and len(data.steps[-1].groups) == 1
    assert [m.role for m in data.find_rollout("s0_0_0").conversation()] == ["system", "user", "assistant", "tool", "assistant"]
    assert data.find_rollout("s0_0_0").conversation()[2].content == "calling"
    assert [m.role for m in data.find_rollout("s0_1_0").conversation()] == ["user", "assistant"]


def test_stream_events_build_a_live_rollout():
    data = TraceData()
    data.handle_stream_event("live1", "text_delta", {"delta": "Hel", "prompt": "say hi", "group_index": 7})
    data.handle_stream_event("live1", "text_delta", {"delta": "lo"})
    data.handle_stream_event("live1", "thinking_end", {"content": "hmm"})
    data.handle_stream_event("live1", "tool_call_end", {"tool_call": {"name": "add", "args": {"v": 1}}})
    data.handle_stream_event("live1", "tool_result", {"content": "2", "is_error": False})
    r = data.find_rollout("live1")
    assert r.is_streaming and r.group_id == 7 and r.response == "Hello"
    assert [m.role for m in r.messages] == ["user", "assistant", "thinking", "assistant", "tool"] and "add(" in r.messages[3].content
    data.handle_stream_event("live1", "done", {"reward": 0.5})
    assert not r.is_streaming and r.reward == 0.5
    assert ingest_line(data, json.dumps({"sample_id": "live2", "event": "text_end", "content": "whole"}))
    assert ingest_line(data, json.dumps({"logger": "rollouts", "message": json.dumps({"step": 2, "reward": 1.0, "response": "r"})}))
    assert not ingest_line(data, "plain text") and data.find_rollout("live2").response == "whole"


def test_browser_navigation_and_folds(tmp_path):
    data = TraceData()
    for r in _records():
        data.add_record(r)
    b = Browser(data, width=80, height=12)
    assert isinstance(b.screen, StepPicker) and "step    0" in b.frame()[1] and b.frame()[1].startswith("> ")
    assert b.feed(decode_keys("j\r")) and isinstance(b.screen, GroupPicker) and b.screen.step.step == 1
    assert b.feed(["G", "enter"]) and isinstance(b.screen, RolloutPicker) and b.screen.group.group_id == 2
    frame = b.frame()
    assert len(frame) == 12 and "sample   0" in frame[1] and frame[-1].endswith("[1/4]")
    b.feed(["j", "j", "j", "l"])
    v = b.screen
    assert isinstance(v, TraceViewer) and v.rollout.sample_id == 3
    assert v.folded == {0: False, 1: True}                      # the 22-line answer starts folded
    text = "\n".join(v.render(80, 40))
    assert "(folded)" in text and "more lines" in text
    b.feed(["j", "z", "a"])
    assert v.folded[1] is False and "more lines" not in "\n".join(v.render(80, 60))
    b.feed(["z", "M"])
    assert all(v.folded.values())
    b.feed(["z", "R", "k", "space"])
    assert v.folded == {0: True, 1: False}
    assert b.feed(["q"]) and isinstance(b.screen, RolloutPicker)
    assert b.feed(["esc", "h"]) and isinstance(b.screen, StepPicker)
    assert b.feed(["q"]) is False and b.stack == []
    # one step only: the browser opens on its groups; the viewer's text export carries every message
    single = TraceData()
    single.add_record(_records()[0])
    sb = Browser(single)
    assert isinstance(sb.screen, GroupPicker)
    sb.feed(["enter", "enter"])
    assert "## tool\n42" in sb.screen.plain_text() and sb.screen.handle_key("q") is POP
    path = sb.screen.open_in_editor()
    assert "be brief" in open(path).read()
    assert decode_keys("\x1b[A\x1b[Bx\x04 ") == ["up", "down", "x", "ctrl-d", "space"]


def test_command_line_frame_and_streaming_viewer(tmp_path, capsys):
    p = tmp_path / "rollouts.jsonl"
    p.write_text("\n".join(json.dumps(r) for r in _records()))
    assert main([str(p), "--keys", "j\r"]) == 0
    out = capsys.readouterr().out
    assert "step 1: groups" in out and "group     0" in out
    assert main([str(tmp_path / "missing.jsonl")]) == 1
    data = TraceData()
    data.handle_stream_event("s", "text_delta", {"delta": "a"})
    v = TraceViewer(data.find_rollout("s"))
    assert v.follow
    for i in range(5):
        data.handle_stream_event("s", "tool_result", {"content": f"result {i}"})
    v.render(60, 8)
    assert v.cursor == len(data.find_rollout("s").messages) - 1             # follows the newest message
    v.handle_key("k")
    assert not v.follow


def test_remote_runner_merges_command_output_and_tailed_files(tmp_path):
    side = tmp_path / "engine.log"
    out = io.StringIO()
    stop = threading.Event()
    counts = []
    t = threading.Thread(target=lambda: counts.append(tail_file_as_jsonl(side, "engine", stop, out, poll_s=0.02)), daemon=True)
    t.start()
    script = (f"import json, sys, time, os\n"
              f"assert os.environ['LOG_JSON'] == 'true'\n"
              f"time.sleep(0.3)\n"
              f"open({str(side)!r}, 'a').write('engine ready\\n' + json.dumps({{'tok_s': 5}}) + '\\n')\n"
              f"print(json.dumps({{'logger': 'metrics', 'loss': 1.5}})); print('plain line'); sys.stdout.flush()\n"
              f"time.sleep(0.4)\n")
    side.write_text("old line that is skipped\n")
    time.sleep(0.3)
    rc = run_training_with_json_logging(f"{sys.executable} -c \"{script}\"", stop, out)
    t.join(timeout=3)
    assert rc == 0 and stop.is_set() and counts == [2]
    recs = [json.loads(line) for line in out.getvalue().splitlines()]
    assert {"logger": "metrics", "loss": 1.5} in recs and {"logger": "training", "message": "plain line"} in recs
    assert {"logger": "engine", "message": "engine ready"} in recs and {"logger": "engine", "tok_s": 5} in recs
    assert not any("old line" in json.dumps(r) for r in recs)
