"""Terminal front ends and the interactive chat loop, driven by scripted input and a scripted model."""

import asyncio
import io
import json

import pytest

from research_b200.agents.dtypes import (Endpoint, StreamDone, TextDelta, ThinkingDelta, ToolCallEnd, ToolResultReceived)
from research_b200.agents.environments import CalculatorEnvironment
from research_b200.agents.providers import ScriptedLLM, register_provider
from research_b200.frontend.terminal import (AnsiFrontend, FenceHighlighter, InteractiveRunner, JsonFrontend, PlainFrontend,
                                             Theme, box, truncate_lines)


def test_box_and_truncate():
    lines = truncate_lines("a\n" * 30 + "x" * 500, 5, 20)
    assert len(lines) == 6 and lines[-1].startswith("…") and all(len(ln) <= 20 for ln in lines[:5])
    b = box("tool: calc", ["1+1", "=2"], 30)
    rows = b.split("\n")
    assert len(rows) == 4 and len({len(r) for r in rows}) == 1 and rows[0].startswith("┌─ tool: calc")


def test_fence_highlighter_streams_in_pieces():
    text = "see:\n```python\nx = 1\ny = 2\n```\nafter\n"
    whole = FenceHighlighter().feed(text)
    h = FenceHighlighter()
    pieces = "".join(h.feed(text[i:i + 3]) for i in range(0, len(text), 3))
    assert whole == pieces
    assert Theme.CODE + "x = 1" in whole and Theme.CODE + "after" not in whole and not h.in_code


def test_ansi_frontend_renders_events():
    out = io.StringIO()
    fe = AnsiFrontend(out=out, inp=io.StringIO("y\n"), width=60, auto_confirm=False)

    async def go():
        await fe.start()
        await fe.handle_event(ThinkingDelta(delta="hmm"))
        await fe.handle_event(TextDelta(delta="The answer"))
        await fe.handle_event(ToolCallEnd(tool_call_id="1", name="evaluate", args={"expression": "2+2"}))
        await fe.handle_event(ToolResultReceived(tool_call_id="1", content="4\n" * 40))
        await fe.handle_event(StreamDone())
        fe.set_status(model="m", turn=2, input_tokens=10, output_tokens=5)
        line = await fe.get_input("> ")
        await fe.stop()
        return line

    assert asyncio.run(go()) == "y"
    s = out.getvalue()
    assert "tool: evaluate" in s and "more lines" in s and "hmm" in s and "turn 2" in s and "10→5 tok" in s
    assert fe._loader_task is None


def test_interactive_runner_with_tools_and_commands(tmp_path):
    register_provider("scripted-chat", ScriptedLLM([
        '<tool_call>{"name": "evaluate", "arguments": {"expression": "6*7"}}</tool_call>', "It is 42.", "Again 42."]))
    out = io.StringIO()
    save = tmp_path / "c.jsonl"
    inp = io.StringIO(f"what is 6*7?\n/status\n/bogus\n/temperature 0.3\n/retry\n/save {save}\n/quit\n")
    fe = PlainFrontend(out=out, inp=inp)
    runner = InteractiveRunner(Endpoint(provider="scripted-chat", model="s"), fe, environment=CalculatorEnvironment(),
                               system_prompt="be brief")
    state = asyncio.run(runner.run())
    s = out.getvalue()
    assert "[tool] evaluate" in s and "[result] current value: 42" in s and "It is 42." in s and "Again 42." in s
    assert "unknown command /bogus" in s and "temperature set to 0.3" in s and runner.endpoint.temperature == 0.3
    roles = [m.role for m in state.actor.trajectory.messages]
    assert roles[0] == "system" and roles.count("user") == 1 and roles[-1] == "assistant"
    saved = [json.loads(ln) for ln in save.read_text().splitlines()]
    assert saved[0]["role"] == "system" and saved[-1]["role"] == "assistant"
    assert fe.status["turn"] == 2


def test_json_frontend_protocol():
    register_provider("scripted-json", ScriptedLLM(["hello there"]))
    out = io.StringIO()
    fe = JsonFrontend(out=out, inp=io.StringIO('{"text": "hi"}\n'))
    runner = InteractiveRunner(Endpoint(provider="scripted-json"), fe, single_turn=True)
    asyncio.run(runner.run())
    events = [json.loads(ln) for ln in out.getvalue().splitlines()]
    kinds = [e["type"] for e in events]
    assert kinds[0] == "start" and kinds[-1] == "stop" and "input_request" in kinds and "text_delta" in kinds and "done" in kinds
    assert next(e for e in events if e["type"] == "text_delta")["delta"] == "hello there"


def test_headless_json_turns_and_interrupted_exchange(tmp_path):
    """Whole turns as JSON lines in both directions; an interrupted exchange ends with an error event and the chat goes on."""
    import asyncio
    import io
    import json

    from research_b200.agents.dtypes import Endpoint, Message, ToolCall
    from research_b200.agents.environments import CalculatorEnvironment
    from research_b200.agents.providers import ScriptedLLM, register_provider
    from research_b200.frontend.terminal import HeadlessJsonFrontend, InteractiveRunner, make_frontend

    holder = {}

    async def model(actor, run_config):
        last = actor.trajectory.messages[-1]
        if last.role == "user" and "slow" in last.text():
            asyncio.get_running_loop().call_later(0.05, lambda: holder["runner"].current_exchange.cancel())   # what SIGINT does
            await asyncio.sleep(30)
        if last.role == "user" and "add" in last.text():
            return await ScriptedLLM([Message("assistant", "Adding.", tool_calls=(ToolCall("t1", "add", {"value": 5}),))])(actor, run_config)
        return await ScriptedLLM(["The result is 5." if last.role == "tool" else "hello"])(actor, run_config)

    register_provider("headless-mock", model)
    inp = io.StringIO('{"type": "user", "text": "add five"}\nplease be slow\n{"type": "user", "text": "/status"}\n{"type": "user", "text": "hi again"}\n/quit\n')
    out = io.StringIO()
    fe = make_frontend("headless", out=out, inp=inp)
    assert isinstance(fe, HeadlessJsonFrontend)
    runner = InteractiveRunner(Endpoint(provider="headless-mock", model="m"), fe, environment=CalculatorEnvironment(), cwd=str(tmp_path), file_commands=[])
    holder["runner"] = runner
    final = asyncio.run(asyncio.wait_for(runner.run(), 20))
    events = [json.loads(line) for line in out.getvalue().splitlines()]
    kinds = [e["type"] for e in events]
    assert events[0] == {"type": "system", "subtype": "init", "session_id": "", "tools": [t.function.name for t in CalculatorEnvironment().get_tools()], "environment": "CalculatorEnvironment"} \
        or events[0]["subtype"] == "init" and "add" in events[0]["tools"]
    first = events[kinds.index("assistant")]
    assert first["message"]["content"] == [{"type": "text", "text": "Adding."}, {"type": "tool_use", "id": "t1", "name": "add", "input": {"value": 5}}]
    result = events[kinds.index("user")]["message"]["content"][0]
    assert result["type"] == "tool_result" and result["tool_use_id"] == "t1" and not result["is_error"] and "5" in result["content"]
    assert {"type": "error", "error": "interrupted"} in events
    texts = [c["text"] for e in events if e["type"] == "assistant" for c in e["message"]["content"] if c["type"] == "text"]
    assert texts[1] == "The result is 5." and any(t.startswith("session") for t in texts) and texts[-1] == "hello"
    assert kinds.count("input_request") == 5 and events[-1]["type"] == "result" and events[-1]["num_turns"] >= 4
    # the interrupted turn left no trace in the conversation except the user's message
    roles = [m.role for m in final.actor.trajectory.messages]
    assert roles == ["user", "assistant", "tool", "assistant", "user", "user", "assistant"] and final.actor.trajectory.messages[-1].text() == "hello"


def test_themes_and_thinking_flag(tmp_path):
    import io

    from research_b200 import cli
    from research_b200.agents.providers import ScriptedLLM, register_provider
    from research_b200.frontend import terminal

    try:
        terminal.apply_theme("none")
        assert terminal.Theme.USER == "" and terminal.Theme.RESET == "" and terminal.box("t", ["x"], 20, terminal.Theme.TOOL).count("\x1b") == 0
        terminal.apply_theme("light")
        assert terminal.Theme.TOOL == "\x1b[35m" and terminal.Theme.RESET == "\x1b[0m"
        with pytest.raises(ValueError):
            terminal.apply_theme("neon")
    finally:
        terminal.apply_theme("dark")
    assert terminal.Theme.TOOL == "\x1b[33m"
    seen = {}

    async def model(actor, run_config):
        seen["extra"] = dict(actor.endpoint.extra_params)
        seen["max_tokens"] = actor.endpoint.max_tokens
        return await ScriptedLLM(["ok"])(actor, run_config)

    register_provider("think-mock", model)
    assert cli.main(["chat", "--provider", "think-mock", "--model", "m", "--no-session", "-q", "-p", "hi", "--thinking", "4096", "--cwd", str(tmp_path)]) == 0
    assert seen["extra"]["thinking"] == {"type": "enabled", "budget_tokens": 4096} and seen["max_tokens"] >= 5120
    with pytest.raises(SystemExit, match="usage"):
        cli.main(["chat", "--provider", "think-mock", "--model", "m", "--no-session", "-q", "-p", "hi", "--thinking", "maybe"])


def test_model_and_temperature_changes_are_recorded_in_the_session(tmp_path):
    """A configuration change between two exchanges lands in the session's change log with the message index it took
    effect at, and a later resume sees the new endpoint."""
    import asyncio
    import io

    from research_b200.agents.dtypes import Endpoint, Message
    from research_b200.agents.store import FileSessionStore
    from research_b200.frontend.terminal import InteractiveRunner, PlainFrontend

    store = FileSessionStore(tmp_path)
    ep = Endpoint("mock", "m1")
    sid = asyncio.run(store.create(ep.to_dict()))
    asyncio.run(store.append_message(sid, Message("user", "hi")))
    agent = InteractiveRunner(ep, PlainFrontend(out=io.StringIO()), session_store=store, session_id=sid)
    assert "m2" in agent._cmd_model("m2")
    agent._cmd_temperature("0.3")
    agent._cmd_temperature("0.3")                               # no change: not recorded twice
    changes = store.config_changes(sid)
    assert [c["what"] for c in changes] == ["endpoint", "endpoint"]
    assert changes[0]["at_message"] == 1 and changes[0]["before"]["model"] == "m1" and changes[0]["after"]["model"] == "m2"
    session, _ = asyncio.run(store.get(sid))
    assert session.endpoint["model"] == "m2" and session.endpoint["temperature"] == 0.3
