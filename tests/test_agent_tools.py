"""Pipelines, slicing, export, progress, feedback and transcript import (all offline)."""

import asyncio
import io
import json
import random

from research_b200.agents.agents import run_agent
from research_b200.agents.dtypes import Actor, AgentState, Endpoint, Message, RunConfig, ToolCall, Trajectory
from research_b200.agents.environments import CalculatorEnvironment
from research_b200.agents.export import export_session, handoff_summary
from research_b200.agents.feedback import run_exit_survey, should_survey
from research_b200.agents.import_cc import decode_project_path, encode_project_path, import_transcript, parse_transcript
from research_b200.agents.pipeline import (AgentStage, compact_trajectory, inject_message, reduce_llm_judge,
                                           reduce_majority_vote, reduce_select_best, run_agent_pipeline, run_parallel_agents,
                                           summarize_trajectory)
from research_b200.agents.progress import MultiProgress, format_bar, format_time, tqdm
from research_b200.agents.providers import ScriptedLLM, register_provider
from research_b200.agents.slice import apply_slice, parse_slice_spec, slice_session
from research_b200.agents.store import FileSessionStore


def _state(provider, text="q"):
    return AgentState(Actor(Trajectory((Message("user", text),)), Endpoint(provider=provider)), None, max_turns=3)


def test_trajectory_transforms():
    t = Trajectory(tuple([Message("system", "s")] + [Message("user", f"m{i}") for i in range(10)]))
    c = compact_trajectory(t, keep_last_n=3)
    assert [m.text() for m in c.messages] == ["s", "m7", "m8", "m9"]
    s = summarize_trajectory(t, "did things", keep_last_n=1)
    assert len(s.messages) == 3 and "did things" in s.messages[1].text()
    assert inject_message(t, Message("user", "x"), 1).messages[1].text() == "x"


def test_parallel_agents_and_reducers():
    async def go():
        replies = iter(["4", "5", "4"])
        register_provider("vote-llm", ScriptedLLM(["unused"]))

        async def varied(actor, rc):
            return await ScriptedLLM([next(replies)])(actor, rc)

        register_provider("vote-llm", varied)
        results = await run_parallel_agents([_state("vote-llm") for _ in range(3)], max_concurrent=1)
        assert all(isinstance(r, list) for r in results)
        best = reduce_majority_vote(results)
        assert best[-1].actor.trajectory.messages[-1].text() == "4"
        longest = reduce_select_best(results, lambda r: float(r[-1].actor.trajectory.messages[-1].text()))
        assert longest[-1].actor.trajectory.messages[-1].text() == "5"
        judged = await reduce_llm_judge(results, ScriptedLLM(["Candidate 2 is best"]), Endpoint(provider="mock"))
        assert judged is results[1]

    asyncio.run(go())


def test_pipeline_stages():
    async def go():
        register_provider("stage-a", ScriptedLLM(['<tool_call>{"name": "evaluate", "arguments": {"expression": "6*7"}}</tool_call>', "The answer is 42"]))
        register_provider("stage-b", ScriptedLLM(["Verified: 42"]))
        stages = [AgentStage("solve", Endpoint(provider="stage-a"), CalculatorEnvironment, max_turns=4),
                  AgentStage("verify", Endpoint(provider="stage-b"), None, system_prompt="You verify answers.",
                             transform=lambda t: compact_trajectory(t, keep_last_n=2))]
        traj, chosen = await run_agent_pipeline(stages, Trajectory((Message("user", "what is 6*7?"),)))
        assert traj.messages[0].role == "system" and traj.messages[-1].text() == "Verified: 42"
        assert set(chosen) == {"solve", "verify"}
        assert any(m.role == "tool" and "42" in m.text() for m in chosen["solve"][-1].actor.trajectory.messages)

    asyncio.run(go())


def test_slice_spec_and_apply(tmp_path):
    segs = parse_slice_spec("0:2, compact:2:60%, summarize:60%:-1:'the bug, not style', -1:, inject:'now test, please'")
    assert [s.type for s in segs] == ["range", "compact", "summarize", "range", "inject"]
    assert segs[2].goal == "the bug, not style" and segs[4].content == "now test, please"
    msgs = [Message("user", "start"), Message("assistant", "ok", tool_calls=(ToolCall("c1", "read", {"path": "a"}),)),
            Message("tool", "line\n" * 500, tool_call_id="c1"), Message("assistant", "saw it"), Message("user", "more"),
            Message("assistant", "done"), Message("user", "last")]

    async def go():
        out = await apply_slice(msgs, "0:2, compact:2:3, summarize:3:-1, -1:, inject:'go on'")
        assert [m.role for m in out] == ["user", "assistant", "tool", "user", "user", "user"]
        assert out[2].text().startswith("[read 501 lines") and "Summary of messages 3-5" in out[3].text()
        assert out[-1].text() == "go on" and out[-2].text() == "last"
        store = FileSessionStore(tmp_path)
        sid = await store.create({"provider": "mock", "model": "m"})
        for m in msgs:
            await store.append_message(sid, m)
        child = await slice_session(store, sid, "0:1, -1:")
        sess, cm = await store.get(child)
        assert sess.parent_id == sid and [m.text() for m in cm] == ["start", "last"]
        md = await export_session(store, sid, "md")
        assert "## 2. Tool result" in md and "tool call" in md
        html_text = await export_session(store, sid, "html", str(tmp_path / "s.html"))
        assert html_text.startswith("<!doctype html>") and (tmp_path / "s.html").exists() and "tool call" in html_text
        brief = await handoff_summary(store, sid, goal="finish")
        assert "Files touched" in brief and "- a" in brief and "finish" in brief

    asyncio.run(go())


def test_progress_rendering():
    assert format_time(3725) == "1:02:05" and format_time(65) == "01:05"
    assert format_bar(0.5, 10).startswith("█████") and len(format_bar(0.33, 10)) == 10
    buf = io.StringIO()
    with MultiProgress(stream=buf, min_interval=0.0) as mp:
        mp.add_task("rollouts", total=4)
        mp.update("rollouts", 2, message="step 2")
        mp.finish("rollouts", "done")
    assert "2/4" in buf.getvalue() and "✓" in buf.getvalue()
    buf = io.StringIO()
    bar = tqdm(range(5), desc="it", file=buf, mininterval=0.0)
    bar.set_postfix(loss=0.5)
    assert list(bar) == [0, 1, 2, 3, 4] and "5/5" in buf.getvalue() and "loss=0.5" in buf.getvalue()


def test_feedback(tmp_path):
    assert not should_survey(10, interactive=False)
    assert not should_survey(1, interactive=True, probability=1.0)

    async def go():
        answers = iter(["4", "worked well"])

        async def ask(prompt):
            return next(answers)

        r = await run_exit_survey("s1", ask, 6, "task_completed", probability=1.0, path=tmp_path / "fb.jsonl", rng=random.Random(0))
        assert r.rating == 4 and r.comment == "worked well"
        assert json.loads((tmp_path / "fb.jsonl").read_text())["session_id"] == "s1"

    asyncio.run(go())


def test_transcript_import(tmp_path):
    assert decode_project_path(encode_project_path(tmp_path)) == tmp_path.resolve() or "-" in str(tmp_path)
    events = [
        {"type": "summary", "summary": "x"},
        {"type": "user", "cwd": "/w", "message": {"role": "user", "content": "fix the bug"}},
        {"type": "assistant", "message": {"role": "assistant", "model": "m-1", "content": [
            {"type": "thinking", "thinking": "hm", "signature": "s"}, {"type": "text", "text": "reading"},
            {"type": "tool_use", "id": "tu1", "name": "Read", "input": {"file_path": "a.py"}}]}},
        {"type": "user", "message": {"role": "user", "content": [{"type": "tool_result", "tool_use_id": "tu1", "content": [{"type": "text", "text": "print(1)"}]}]}},
        {"type": "assistant", "message": {"role": "assistant", "content": [{"type": "text", "text": "done"}]}},
    ]
    f = tmp_path / "abc.jsonl"
    f.write_text("\n".join(json.dumps(e) for e in events) + "\nnot json\n")
    msgs, meta = parse_transcript(f)
    assert [m.role for m in msgs] == ["user", "assistant", "tool", "assistant"]
    assert msgs[1].get_tool_calls()[0].name == "Read" and msgs[2].name == "Read" and msgs[2].text() == "print(1)"
    assert meta["model"] == "m-1" and meta["skipped"] == 1

    async def go():
        store = FileSessionStore(tmp_path / "store")
        sid = await import_transcript(store, f)
        sess, got = await store.get(sid)
        assert len(got) == 4 and sess.endpoint["model"] == "m-1"

    asyncio.run(go())
