"""Agent runtime without a network: scripted model, environments, sessions, evaluation, TI/TO."""

import asyncio
import json
from dataclasses import replace

import pytest

from research_b200.agents import (Actor, AgentState, Endpoint, EvalConfig, FileSessionStore, Message, Metric, RunConfig,
                                  Score, StopReason, ToolCall, Trajectory, evaluate, resume_session, run_agent, run_search)
from research_b200.agents.environments import (BinarySearchEnvironment, CalculatorEnvironment, ComposedEnvironment,
                                               LocalFilesystemEnvironment, MessageParsingREPLEnvironment, REPLEnvironment,
                                               safe_eval)
from research_b200.agents.providers import (NonRetryableError, ProviderError, RateLimiter, ScriptedLLM, async_retry,
                                            classify_http_status, get_provider, parse_tool_calls, register_provider)
from research_b200.training.agent_integration import trajectory_to_sample, trajectory_to_samples


def _state(env, text="compute", max_turns=6, provider="mock"):
    return AgentState(Actor(Trajectory((Message("user", text),)), Endpoint(provider=provider)), env, max_turns=max_turns)


def test_tool_call_parsing():
    text, calls = parse_tool_calls('ok <tool_call>{"name": "add", "arguments": {"value": 3}}</tool_call>')
    assert text == "ok" and calls[0].name == "add" and calls[0].args == {"value": 3}
    _, calls = parse_tool_calls('{"name": "guess", "arguments": {"number": 5}}')
    assert calls[0].name == "guess"
    text, calls = parse_tool_calls("<tool_call>{broken</tool_call>")
    assert calls == [] and "broken" in text
    assert safe_eval("2*(3+4)**2") == 98
    with pytest.raises(ValueError):
        safe_eval("__import__('os')")


def test_agent_loop_with_calculator_and_session_resume(tmp_path):
    llm = ScriptedLLM(['<tool_call>{"name": "add", "arguments": {"value": 5}}</tool_call>',
                       '<tool_call>{"name": "multiply", "arguments": {"value": 3}}</tool_call>',
                       '<tool_call>{"name": "complete_task", "arguments": {}}</tool_call>'])
    register_provider("mock", llm)
    store = FileSessionStore(tmp_path)
    events = []

    async def on_chunk(e):
        events.append(e.type)

    states = asyncio.run(run_agent(_state(CalculatorEnvironment()), RunConfig(session_store=store, on_chunk=on_chunk)))
    final = states[-1]
    assert final.stop == StopReason.TASK_COMPLETED and final.environment.value == 15.0 and final.turn_idx == 3
    assert "tool_result" in events and events[-1] == "done"
    sid = final.session_id
    session, msgs = asyncio.run(store.get(sid))
    assert session.status == "task_completed" and len(msgs) == 7 and msgs[2].role == "tool"
    # resume a session interrupted between an assistant tool call and its result
    sid2 = asyncio.run(store.branch(sid, 2))
    resumed = asyncio.run(resume_session(sid2, store, Endpoint(provider="mock"), CalculatorEnvironment))
    assert [c.name for c in resumed.pending_tool_calls] == ["add"] and resumed.turn_idx == 1
    llm.calls = 1
    st2 = asyncio.run(run_agent(resumed, RunConfig(session_store=store)))[-1]
    assert st2.stop == StopReason.TASK_COMPLETED


def test_stop_reasons_and_tool_errors():
    register_provider("mock", ScriptedLLM(["just text"]))
    assert asyncio.run(run_agent(_state(CalculatorEnvironment())))[-1].stop == StopReason.NO_TOOL_CALLS
    register_provider("mock", ScriptedLLM(['<tool_call>{"name": "divide", "arguments": {"value": 0}}</tool_call>']))
    final = asyncio.run(run_agent(_state(CalculatorEnvironment(), max_turns=2)))[-1]
    assert final.stop == StopReason.MAX_TURNS
    assert any("division by zero" in m.text() for m in final.actor.trajectory.messages if m.role == "tool")
    register_provider("mock", ScriptedLLM(['<tool_call>{"name": "guess", "arguments": {"number": 42}}</tool_call>']))
    assert asyncio.run(run_agent(_state(BinarySearchEnvironment(target=42))))[-1].stop == StopReason.TASK_COMPLETED


def test_environments(tmp_path):
    async def go():
        fs = LocalFilesystemEnvironment(str(tmp_path))
        st = _state(fs)
        r = await fs.exec_tool(ToolCall("1", "write", {"path": "a/b.txt", "content": "hello"}), st, RunConfig())
        assert not r.is_error
        r = await fs.exec_tool(ToolCall("2", "edit", {"path": "a/b.txt", "old": "hello", "new": "bye"}), st, RunConfig())
        assert (tmp_path / "a" / "b.txt").read_text() == "bye"
        r = await fs.exec_tool(ToolCall("3", "read", {"path": "../../etc/passwd"}), st, RunConfig())
        assert r.is_error and "escapes" in r.error
        r = await fs.exec_tool(ToolCall("4", "bash", {"command": "echo hi && ls a"}), st, RunConfig())
        assert "hi" in r.content and "b.txt" in r.content and fs.requires_confirmation(ToolCall("4", "bash", {}))
        repl = REPLEnvironment()
        await repl.exec_tool(ToolCall("5", "python", {"code": "x = 21"}), st, RunConfig())
        r = await repl.exec_tool(ToolCall("6", "python", {"code": "print(x * 2); FINAL(x * 2)"}), st, RunConfig())
        assert "42" in r.content and r.stop_reason == StopReason.TASK_COMPLETED and repl.final_answer == 42
        r = await repl.exec_tool(ToolCall("7", "python", {"code": "1/0"}), st, RunConfig())
        assert r.is_error and "ZeroDivisionError" in r.error
        snap = await repl.serialize()
        assert (await REPLEnvironment.deserialize(json.loads(json.dumps(snap)))).namespace["x"] == 21
        mp = MessageParsingREPLEnvironment()
        assert "3" in mp.run_message("text\n```python\nprint(1+2)\n```")
        comp = ComposedEnvironment([CalculatorEnvironment(), BinarySearchEnvironment()])
        assert len(comp.get_tools()) == 7
        r = await comp.exec_tool(ToolCall("8", "add", {"value": 2}), st, RunConfig())
        assert "2.0" in r.content
        again = await ComposedEnvironment.deserialize(await comp.serialize())
        assert again.envs[0].value == 2.0

    asyncio.run(go())


def test_retry_rate_limit_and_errors():
    calls = {"n": 0}
    slept = []

    async def fake_sleep(s):
        slept.append(s)

    @async_retry(max_attempts=3, base=0.01, sleep=fake_sleep)
    async def flaky():
        calls["n"] += 1
        if calls["n"] < 3:
            raise ProviderError("overloaded", 429)
        return "ok"

    assert asyncio.run(flaky()) == "ok" and calls["n"] == 3 and len(slept) == 2

    @async_retry(max_attempts=3, sleep=fake_sleep)
    async def bad():
        calls["n"] += 1
        raise NonRetryableError("bad request", 400)

    calls["n"] = 0
    with pytest.raises(NonRetryableError):
        asyncio.run(bad())
    assert calls["n"] == 1
    assert isinstance(classify_http_status(503), ProviderError) and not isinstance(classify_http_status(503), NonRetryableError)
    assert isinstance(classify_http_status(401), NonRetryableError)

    async def limited():
        lim = RateLimiter(max_concurrent=2)
        peak = 0

        async def job():
            nonlocal peak
            async with lim:
                peak = max(peak, lim.in_flight)
                await asyncio.sleep(0.01)

        await asyncio.gather(*[job() for _ in range(6)])
        return peak, lim.total

    assert asyncio.run(limited()) == (2, 6)
    with pytest.raises(NonRetryableError):
        get_provider("nope")


def test_evaluate_report(tmp_path):
    register_provider("mock", ScriptedLLM(["4"]))
    cfg = EvalConfig(endpoint=Endpoint(provider="mock"), max_turns=1, output_dir=str(tmp_path), eval_name="arith",
                     score_fn=lambda traj, row: Score((Metric("correct", float(traj.messages[-1].text() == row["answer"]), 1.0),
                                                       Metric("length", len(traj.messages[-1].text()), 0.0))))
    rep = asyncio.run(evaluate([{"id": "a", "prompt": "2+2", "answer": "4"}, {"id": "b", "prompt": "2+3", "answer": "5"}], cfg))
    assert rep.summary["mean_reward"] == 0.5 and rep.summary["mean_length"] == 1.0 and rep.summary["error_rate"] == 0.0
    assert (tmp_path / "arith" / "report.json").exists() and len((tmp_path / "arith" / "samples.jsonl").read_text().splitlines()) == 2
    assert Trajectory.load_jsonl(tmp_path / "arith" / "trajectories.jsonl")[0].messages[0].text() == "2+2"


def test_search():
    async def expand(node):
        return [(node.state + [d], sum(node.state) + d, len(node.state) >= 2) for d in (1, 2, 3)]

    best = asyncio.run(run_search([], expand, beam_width=2, max_depth=5))
    assert best.state == [3, 3, 3] and best.terminal and len(best.path()) == 4


def test_trajectory_to_samples_uses_engine_token_ids():
    from research_b200.agents.dtypes import ChatCompletion, Choice, Logprob, Logprobs

    def comp(prompt, out, lps, v):
        return ChatCompletion("c", "m", (Choice(0, Message("assistant", "x"), "stop",
                                                Logprobs(tuple(Logprob("", l) for l in lps)), tuple(out), tuple(prompt)),),
                              weight_version=v)

    traj = Trajectory((Message("user", "q"), Message("assistant", "x"), Message("tool", "r"), Message("assistant", "y")),
                      (comp([1, 2, 3], [4, 5], [-0.1, -0.2], 7), comp([1, 2, 3, 4, 5, 9, 9], [6], [-0.3], 7)), rewards=1.0)
    s = trajectory_to_sample(traj)
    assert s.tokens == [1, 2, 3, 4, 5, 9, 9, 6] and s.loss_mask == [0, 0, 0, 1, 1, 0, 0, 1]
    assert s.rollout_log_probs == [-0.1, -0.2, -0.3] and s.reward == 1.0 and s.weight_version == 7
    br = trajectory_to_samples(traj, strategy="branching")
    assert len(br) == 2 and br[1].tokens == [1, 2, 3, 4, 5, 9, 9, 6] and br[1].response_length == 1
    t2 = Trajectory.from_dict(json.loads(traj.to_jsonl()))
    assert t2.completions[1].choices[0].token_ids == (6,) and t2.hash() == traj.hash()


def test_evaluate_outcomes_resume_and_files(tmp_path):
    """Three outcomes (success / failed / provider_error), success_rate without the provider errors in its denominator,
    per-sample files with credentials redacted, resume that re-runs only what is missing or hit a provider error."""
    from research_b200.agents.evaluation import (EvalReport, compute_summary_metrics, group_by, load_csv, load_jsonl,
                                                 sanitize_api_keys, simple_evaluate, summarize)

    class Flaky:
        """Answers the prompt with its digits; rows whose prompt says 'down' always raise a provider error."""

        def __init__(self):
            self.calls = []

        async def __call__(self, actor, run_config):
            prompt = actor.trajectory.messages[-1].text()
            self.calls.append(prompt)
            if "down" in prompt:
                raise ProviderError("rate limited", 429)
            return await ScriptedLLM(["".join(c for c in prompt if c.isdigit())])(actor, run_config)

    llm = Flaky()
    register_provider("mock", llm)

    def score(traj, row):
        if row.get("explode"):
            raise ValueError("scorer cannot read this row")
        return Score((Metric("correct", float(traj.messages[-1].text() == row["answer"]), 1.0),))

    rows = [{"id": "a", "prompt": "say 12", "answer": "12", "kind": "easy"}, {"id": "b", "prompt": "say 7", "answer": "8", "kind": "easy"},
            {"id": "c", "prompt": "down 1", "answer": "1", "kind": "hard"}, {"id": "d", "prompt": "say 3", "answer": "3", "explode": True, "kind": "hard"}]
    cfg = EvalConfig(endpoint=Endpoint(provider="mock", api_key="sk-abcdefghijklmnop"), max_turns=1, output_dir=str(tmp_path), eval_name="mix",
                     score_fn=score, n_retries=1, retry_delays=(0.0,))
    seen = []
    rep = asyncio.run(evaluate(rows, cfg, on_sample_done=lambda s, done, total: seen.append((s.sample_id, done, total))))
    by_id = {s.sample_id: s for s in rep.samples}
    assert [by_id[i].status for i in "abcd"] == ["success", "success", "provider_error", "failed"]
    assert by_id["c"].attempts == 2 and by_id["d"].error.startswith("ValueError")
    sm = rep.summary
    assert sm["successful_samples"] == 2 and sm["provider_errors"] == 1 and sm["failed_samples"] == 1
    assert sm["success_rate"] == pytest.approx(2 / 3) and sm["completion_rate"] == 0.5
    assert sm["error_breakdown"] == {"ValueError": 1} and sm["provider_error_breakdown"] == {"mock": 1}
    assert sm["min_correct"] == 0.0 and sm["max_correct"] == 1.0 and sm["std_correct"] == pytest.approx(0.5)
    assert sorted(x[0] for x in seen) == list("abcd") and seen[-1][1:] == (4, 4)
    run = tmp_path / "mix"
    assert sorted(p.name for p in (run / "samples").iterdir()) == ["a.json", "b.json", "c.json", "d.json"]
    assert "sk-abcdefghijklmnop" not in (run / "report.json").read_text()
    assert sanitize_api_keys({"x": [{"api_key": "sk-1"}, "sk-abcdefghijklmnop"], "n": 1}) == {"x": [{"api_key": "***REDACTED***"}, "***REDACTED***"], "n": 1}
    back = EvalReport.load(run)
    assert [s.sample_id for s in back.samples] == list("abcd") and back.samples[0].score.reward == 1.0
    assert back.samples[0].trajectory.messages[-1].text() == "12"
    # resume: only the provider-error sample runs again
    llm.calls.clear()
    rep2 = asyncio.run(evaluate(rows, cfg, resume=True))
    assert llm.calls == ["down 1", "down 1"] and rep2.config["resumed_samples"] == 3
    groups = group_by(rep.samples, key=lambda s: s.input["kind"])
    assert summarize(groups)["easy"]["mean_reward"] == 0.5 and summarize(rep.samples)["n"] == 4
    assert compute_summary_metrics([]) == {"num_samples": 0.0}
    # dataset files
    import json as _json

    (tmp_path / "d.jsonl").write_text("\n".join(_json.dumps(r) for r in rows[:2]) + "\n\n")
    (tmp_path / "d.csv").write_text("id,prompt,answer\nq,say 5,5\n")
    assert [r["id"] for r in load_jsonl(tmp_path / "d.jsonl")] == ["a", "b"] and next(load_csv(tmp_path / "d.csv"))["answer"] == "5"
    cfg2 = EvalConfig(endpoint=Endpoint(provider="mock"), max_turns=1, score_fn=score, eval_name="files")
    assert asyncio.run(simple_evaluate(tmp_path / "d.csv", cfg2)).summary["mean_reward"] == 1.0
    assert asyncio.run(simple_evaluate(tmp_path / "d.jsonl", cfg2)).dataset_path.endswith("d.jsonl")
    with pytest.raises(ValueError):
        asyncio.run(simple_evaluate(tmp_path / "d.txt", cfg2))


def test_filesystem_environment_tools_presets_and_formatting(tmp_path):
    """read windows and notes, edit diff, glob / grep, bash timeout and exit codes, web_fetch through an injected fetcher,
    tool presets, and what the front end prints for a call and its result."""
    import io

    from research_b200.agents.environments.coding import MAX_READ_LINES, format_tool
    from research_b200.frontend.terminal import PlainFrontend
    from research_b200.agents.dtypes import ToolCallEnd, ToolResultReceived

    (tmp_path / "pkg").mkdir()
    (tmp_path / "pkg" / "big.txt").write_text("\n".join(f"line {i}" for i in range(1, 2501)))
    (tmp_path / "pkg" / "wide.txt").write_text("x" * 5000 + "\nshort")
    (tmp_path / "pkg" / "a.py").write_text("import os\n\ndef f():\n    return 1\n")
    (tmp_path / "pkg" / "bin.dat").write_bytes(b"\xff\xfe\x00\x01")

    async def fetch(url):
        return (200, "text/html", "<html><script>x()</script><body><h1>Title</h1><p>Body &amp; more</p></body></html>") if "ok" in url else (404, "", "")

    async def go():
        fs = LocalFilesystemEnvironment(str(tmp_path), bash_timeout=20, fetcher=fetch)
        st, rc = _state(fs), RunConfig()
        call = lambda name, **a: fs.exec_tool(ToolCall("c", name, a), st, rc)                                       # noqa: E731
        r = await call("read", path="pkg/big.txt")
        assert r.content.startswith("line 1\n") and f"line {MAX_READ_LINES}\n" in r.content and f"offset={MAX_READ_LINES + 1}" in r.content
        r = await call("read", path="pkg/big.txt", offset=2400, limit=3)
        assert r.content.startswith("line 2400\nline 2401\nline 2402") and "98 more lines" in r.content
        assert (await call("read", path="pkg/big.txt", offset=2499, limit=50)).content == "line 2499\nline 2500"
        assert "beyond the end" in (await call("read", path="pkg/big.txt", offset=9000)).error
        assert "cut to 2000 characters" in (await call("read", path="pkg/wide.txt")).content
        assert "binary" in (await call("read", path="pkg/bin.dat")).error and "not found" in (await call("read", path="nope")).error
        r = await call("edit", path="pkg/a.py", old="return 1", new="return 2")
        assert "-    return 1" in r.metadata["diff"] and "+    return 2" in r.metadata["diff"]
        assert "found 0" in (await call("edit", path="pkg/a.py", old="return 1", new="x")).error
        assert "identical" in (await call("edit", path="pkg/a.py", old_text="import os", new_text="import os")).error
        assert (await call("write", path="pkg/a.py", content="import sys\n")).metadata["diff"].count("\n-") >= 3
        assert (await call("write", path="new/b.py", content="def g(): pass\n")).metadata == {"created": True}
        assert set((await call("glob", pattern="**/*.py")).content.split()) == {"pkg/a.py", "new/b.py"}
        assert (await call("grep", pattern=r"def \w+", glob="*.py")).content == "new/b.py:1:def g(): pass"
        assert (await call("grep", pattern="line 24..$", path="pkg/big.txt", max_results=2)).content.endswith("(stopped at 2 matches)")
        assert "error" in (await call("grep", pattern="(")).error
        r = await call("bash", command="echo out; echo err >&2; exit 3")
        assert r.is_error and "out" in r.content and "exit code 3" in r.error
        r = await call("bash", command="sleep 30", timeout=0.3)
        assert r.is_error and "timed out after 0.3s" in r.error
        assert (await call("web_fetch", url="https://ok.example/")).content.split() == ["Title", "Body", "&", "more"]
        assert "404" in (await call("web_fetch", url="https://gone.example/")).error and "http" in (await call("web_fetch", url="file:///etc/passwd")).error
        # presets
        ro = LocalFilesystemEnvironment(str(tmp_path), tools="readonly")
        assert [t.function.name for t in ro.get_tools()] == ["read", "list", "glob", "grep"]
        assert "not enabled" in (await ro.exec_tool(ToolCall("c", "write", {"path": "x", "content": ""}), st, rc)).error
        assert [t.function.name for t in LocalFilesystemEnvironment(str(tmp_path), allow_bash=False, tools=["read", "bash"]).get_tools()] == ["read"]
        again = await LocalFilesystemEnvironment.deserialize(await ro.serialize())
        assert again.tools == "readonly" and again.get_status_info()["cwd"].endswith(tmp_path.name)
        with pytest.raises(ValueError):
            LocalFilesystemEnvironment(str(tmp_path), tools="everything")
        # what a front end prints
        out = io.StringIO()
        fe = PlainFrontend(out=out)
        fe.environment = ComposedEnvironment([fs, CalculatorEnvironment()])
        await fe.handle_event(ToolCallEnd(tool_call_id="e1", name="edit", args={"path": "new/b.py", "old": "pass", "new": "return 1"}))
        res = await call("edit", path="new/b.py", old="pass", new="return 1")
        await fe.handle_event(ToolResultReceived(tool_call_id="e1", content=res.content, details=res.metadata))
        await fe.handle_event(ToolCallEnd(tool_call_id="e2", name="add", args={"value": 2}))
        await fe.handle_event(ToolResultReceived(tool_call_id="e2", content="2.0"))
        text = out.getvalue()
        assert "[tool] edit new/b.py" in text and "+def g(): return 1" in text and '[tool] add({"value": 2})' in text and "[result] 2.0" in text

    asyncio.run(go())
    assert format_tool("bash", {"command": "ls"}) == "$ ls" and format_tool("read", {"path": "a", "offset": 5, "limit": 10}) == "read a:5-14"
    from research_b200.agents.dtypes import ToolResult

    long = ToolResult("x", "\n".join(str(i) for i in range(40)))
    assert "(28 more lines)" in format_tool("bash", {"command": "seq"}, long) and "more lines" not in format_tool("bash", {"command": "seq"}, long, expanded=True)
    assert format_tool("read", {"path": "a"}, long).endswith("40 lines")


def test_rlm_environment_code_calls_models_and_sub_agents():
    """`context` lives in the namespace; code running in a worker thread calls llm_query / agent, which run on the event
    loop; a sub-agent works one level deeper on the piece it was given; depth is bounded; state survives serialize()."""
    from research_b200.agents.environments.rlm import MessageParsingRLMEnvironment, RLMEnvironment, _final_call, run_code

    assert run_code("x = 2\nx * 21", {}) == ("42\n", False) and run_code("1/0", {})[1] and "cut" in run_code("print('a' * 50)", {}, 10)[0]
    assert _final_call("so FINAL(f(1) + 'x') done") == "f(1) + 'x'" and _final_call('FINAL("quoted")') == "quoted" and _final_call("```repl\nFINAL(1)\n```") is None
    doc = "\n".join(f"record {i}: value {i * i}" for i in range(200)) + "\nthe secret code is 73519\n"

    async def sub_model(actor, run_config):
        """Plays both the question-answering sub-model and the sub-agent's policy."""
        last = actor.trajectory.messages[-1]
        if actor.tools and last.role == "user":              # a sub-agent's first turn: search its own context
            return await ScriptedLLM([Message("assistant", "", tool_calls=(ToolCall("s1", "repl", {"code": "import re\nre.findall(r'code is (\\d+)', context)[0]"}),))])(actor, run_config)
        if actor.tools:                                      # second turn: answer with what the tool printed
            return await ScriptedLLM([Message("assistant", "", tool_calls=(ToolCall("s2", "final_answer", {"answer": last.text().strip().strip("'")}),))])(actor, run_config)
        return await ScriptedLLM(["LEN=" + str(len(last.text()))])(actor, run_config)

    register_provider("rlm-sub", sub_model)
    env = RLMEnvironment(context=doc, sub_endpoint=Endpoint(provider="rlm-sub"), max_depth=2)
    main = ScriptedLLM([
        Message("assistant", "", tool_calls=(ToolCall("m1", "repl", {"code": "tail = context[-40:]\nn = llm_query('how long? ' + tail)\nprint(n)"}),)),
        Message("assistant", "", tool_calls=(ToolCall("m2", "repl", {"code": "found = agent('find the code', context[-100:])\nprint('FOUND', found)"}),)),
        Message("assistant", "", tool_calls=(ToolCall("m3", "agent", {"task": "find the code"}),)),
        Message("assistant", "", tool_calls=(ToolCall("m4", "final_answer", {"answer": "73519"}),))])
    register_provider("mock", main)
    start = Trajectory((Message("system", env.get_system_prompt()), Message("user", "What is the secret code?")))
    final = asyncio.run(run_agent(AgentState(Actor(start, Endpoint(provider="mock")), env, max_turns=8)))[-1]
    tool_msgs = [m.text() for m in final.actor.trajectory.messages if m.role == "tool"]
    assert final.stop == StopReason.TASK_COMPLETED and final.environment.final_answer == "73519"
    assert tool_msgs[0].strip() == "LEN=50" and tool_msgs[1].strip() == "FOUND 73519" and tool_msgs[2] == "73519"
    assert final.environment.namespace["found"] == "73519" and final.environment.sub_calls == 3     # one query, two sub-agents
    assert "24" in env.get_system_prompt() or str(len(doc)) in env.get_system_prompt().replace(",", "")
    # depth limit: a sub-agent at the last level is refused
    deep = RLMEnvironment(context="x", sub_endpoint=Endpoint(provider="rlm-sub"), max_depth=2, depth=1)
    assert "maximum depth" in asyncio.run(deep._agent("t", None, RunConfig()))
    assert "no sub_endpoint" in asyncio.run(RLMEnvironment(context="x").exec_tool(ToolCall("q", "llm_query", {"prompt": "p"}), None, RunConfig())).error
    # text-only models: fenced blocks run, output returns as a user message, FINAL_VAR ends the episode
    register_provider("mock", ScriptedLLM(["Let me look.\n```repl\nhits = [l for l in context.split('\\n') if 'secret' in l]\nprint(hits[0])\n```",
                                           "```repl\ncode = hits[0].split()[-1]\n```\nFINAL_VAR(code)"]))
    mp = MessageParsingRLMEnvironment(context=doc)
    final = asyncio.run(run_agent(AgentState(Actor(Trajectory((Message("system", mp.get_system_prompt()), Message("user", "code?"))),
                                                   Endpoint(provider="mock")), mp, max_turns=5)))[-1]
    msgs = final.actor.trajectory.messages
    assert final.stop == StopReason.TASK_COMPLETED and final.environment.final_answer == "73519" and final.turn_idx == 2
    assert msgs[3].role == "user" and "the secret code is 73519" in msgs[3].text() and mp.get_tools() == []


def test_preset_files_lineage_lookup_and_environments(tmp_path):
    from research_b200.agents import presets

    assert set(presets.list_presets(presets.PRESET_DIR)) >= {"careful_coder_01_01", "fast_coder_02_01", "explorer_03_01", "scratchpad_04_04"}
    root, fast = presets.load_preset("careful_coder_01_01"), presets.load_preset("fast_coder")
    assert fast.name == "fast_coder" and not fast.thinking and fast.system_prompt.startswith(root.system_prompt) and fast.env == "coding"
    ex = presets.get_preset("explorer")
    env = ex.environment(str(tmp_path))
    assert [t.function.name for t in env.get_tools()] == ["read", "list", "glob", "grep"] and ex.max_turns == 40
    assert presets.get_preset("coding").name == "coding" and "fast_coder_02_01" in str(pytest.raises(KeyError, presets.get_preset, "nope").value)
    # a user's folder: the latest variant of a stem wins; a variant imports the parent beside it; JSON round trip
    (tmp_path / "mine_01_01.py").write_text("from research_b200.agents.presets import AgentPresetConfig\n"
                                            "config = AgentPresetConfig('mine', 'openai/gpt-4o-mini', 'calculator', 'v1')\n")
    (tmp_path / "mine_02_01.py").write_text("from dataclasses import replace\nfrom mine_01_01 import config as parent\n"
                                            "config = replace(parent, system_prompt=parent.system_prompt + ' v2', temperature=0.2)\n")
    (tmp_path / "broken.py").write_text("config = {'name': 'x'}\n")
    latest = presets.load_preset("mine", tmp_path)
    assert latest.system_prompt == "v1 v2" and presets.load_preset("mine_01_01", tmp_path).system_prompt == "v1"
    assert presets.load_preset(str(tmp_path / "mine_02_01.py")).to_cli_args() == {
        "model": "openai/gpt-4o-mini", "env": "calculator", "system_prompt": "v1 v2", "thinking": True, "temperature": 0.2}
    assert type(latest.to_preset().environment(".")).__name__ == "CalculatorEnvironment"
    with pytest.raises(TypeError):
        presets.load_preset(str(tmp_path / "broken.py"))
    with pytest.raises(KeyError):
        presets.AgentPresetConfig("x", "m", "no-such-env", "p").to_preset()
    from dataclasses import replace

    replace(latest, working_dir=tmp_path).save(tmp_path / "saved.json")
    again = presets.load_preset(str(tmp_path / "saved.json"))
    assert again.working_dir == tmp_path and again.temperature == 0.2


def test_tree_search_over_agent_states():
    """Beam search and UCB search on the number-guessing environment with a policy that samples guesses: values are backed
    up, the beam keeps the closest states, branches act on their own copies of the environment."""
    import random

    from research_b200.agents.search import (SearchTree, compose_pruners, make_beam_pruner, make_depth_pruner, make_expand_n_turns,
                                             make_threshold_pruner, make_ucb_selector, run_tree_search, select_all_frontier, select_one_best,
                                             select_one_deepest)

    rng = random.Random(0)

    async def policy(actor, run_config):
        seen = [m.text() for m in actor.trajectory.messages if m.role == "tool"]
        lo, hi = 0, 100
        for m, t in zip([m for m in actor.trajectory.messages if m.role == "assistant"], seen):
            g = m.tool_calls[0].args["number"]
            lo, hi = (max(lo, g + 1), hi) if "higher" in t.lower() else (lo, min(hi, g - 1)) if "lower" in t.lower() else (g, g)
        guess = rng.randint(lo, hi)
        return await ScriptedLLM([Message("assistant", "", tool_calls=(ToolCall(f"g{len(seen)}", "guess", {"number": guess}),))])(actor, run_config)

    register_provider("mock", policy)

    async def value(state):
        if state.stop == StopReason.TASK_COMPLETED:
            return 1.0
        guesses = [m.tool_calls[0].args["number"] for m in state.actor.trajectory.messages if m.role == "assistant" and m.tool_calls]
        return -abs(guesses[-1] - 37) / 100 if guesses else -1.0

    start = _state(BinarySearchEnvironment(target=37, max_guesses=50), max_turns=50)
    tree = asyncio.run(run_tree_search(start, RunConfig(), select_all_frontier, make_expand_n_turns(1, branch_factor=3), value,
                                       compose_pruners(make_beam_pruner(2), make_depth_pruner(12)), max_steps=12))
    best = tree.best_terminal()
    assert best is not None and best.value == 1.0 and best.state.stop == StopReason.TASK_COMPLETED
    path = tree.path_to(best.node_id)
    assert path[0].node_id == "0" and [n.depth for n in path] == list(range(len(path))) and best.node_id.startswith("0.")
    assert any(n.pruned for n in tree.nodes.values()) and tree["0"].visits == len(tree.nodes) - 1
    level1 = [tree[i] for i in tree["0"].children]
    assert len(level1) == 3 and len({id(n.state.environment) for n in level1}) == 3 and start.environment.guesses == 0
    # selectors and pruners on a hand-built tree
    t = SearchTree("root")
    a, b = t.add_child("0", "a", 0.2), t.add_child("0", "b", 0.8)
    c = t.add_child(a.node_id, "c", 0.5)
    t.frontier.remove("0")
    assert select_one_best(t) == [b.node_id] and select_one_deepest(t) == [c.node_id] and t["0"].mean == pytest.approx(0.5)
    ucb = make_ucb_selector(c=0.0)
    assert ucb(t) == [b.node_id]                                        # no exploration: best mean
    t[b.node_id].visits, t[b.node_id].total = 50, 50 * 0.8
    assert make_ucb_selector(c=5.0)(t) != [b.node_id]                   # strong exploration: the rarely visited ones
    make_threshold_pruner(0.4)(t)
    assert t.frontier == [b.node_id, c.node_id] and t[a.node_id].pruned
    # MCTS-style: one node per step, expanded nodes stay selectable
    rng.seed(1)
    tree = asyncio.run(run_tree_search(start, RunConfig(), make_ucb_selector(1.0), make_expand_n_turns(1, 1, keep_expanded=True), value, max_steps=60))
    assert tree.best_node().value == 1.0 and len(tree["0"].children) >= 2


def test_step_hooks_budgets_reminders_and_confirmation_feedback(tmp_path):
    from research_b200.agents.agents import (estimated_tokens, handle_stop_cost_budget, handle_stop_token_budget, inject_turn_warning,
                                             make_confirm_with_feedback, make_tool_reminder)
    from research_b200.agents.dtypes import Cost, Usage

    add = lambda i: Message("assistant", "", tool_calls=(ToolCall(f"c{i}", "add", {"value": 1}),))                 # noqa: E731
    # a warning when two turns are left, exactly once
    register_provider("mock", ScriptedLLM([add(i) for i in range(6)]))
    final = asyncio.run(run_agent(_state(CalculatorEnvironment(), max_turns=4), RunConfig(on_step_start=inject_turn_warning(2))))[-1]
    warns = [i for i, m in enumerate(final.actor.trajectory.messages) if m.role == "user" and "2 turns left" in m.text()]
    assert final.stop == StopReason.MAX_TURNS and len(warns) == 1 and final.turn_idx == 4
    # budgets
    st = _state(CalculatorEnvironment())
    assert estimated_tokens(st) == sum(len(m.text()) for m in st.actor.trajectory.messages) // 4
    assert handle_stop_token_budget(10**6)(st).stop is None and handle_stop_token_budget(1)(replace(st, usage=Usage(5, 5))).stop == StopReason.BUDGET_EXCEEDED
    assert handle_stop_cost_budget(0.5)(replace(st, usage=Usage(cost=Cost(0.3, 0.3)))).stop == StopReason.BUDGET_EXCEEDED
    assert handle_stop_cost_budget(0.5, lambda s: 0.1)(st).stop is None
    # reminders: two in a row, then the episode ends
    register_provider("mock", ScriptedLLM(["thinking...", "still thinking...", "hmm", "never reached"]))
    final = asyncio.run(run_agent(_state(CalculatorEnvironment(), max_turns=10), RunConfig(handle_no_tool=make_tool_reminder(max_reminders=2))))[-1]
    assert final.stop == StopReason.NO_TOOL_CALLS and final.turn_idx == 3
    assert sum(1 for m in final.actor.trajectory.messages if m.metadata.get("reminder")) == 2
    # refusing a call with a reason: refused result, the turn's other call marked not run, then the reason as a user message
    fs = LocalFilesystemEnvironment(str(tmp_path))
    two = Message("assistant", "", tool_calls=(ToolCall("b1", "bash", {"command": "rm -rf build"}), ToolCall("b2", "bash", {"command": "echo hi"})))
    register_provider("mock", ScriptedLLM([two, "understood"]))
    answers = iter(["n", "do not delete build, list it first"])
    said = []
    rc = RunConfig(confirm_tool=make_confirm_with_feedback(lambda prompt: next(answers), said.append))
    final = asyncio.run(run_agent(_state(fs, max_turns=5), rc))[-1]
    roles = [(m.role, m.text()[:40]) for m in final.actor.trajectory.messages[-4:]]
    assert roles[0] == ("tool", "Error: rejected by the user") and roles[1][1].startswith("Error: not run") and roles[2] == ("user", "do not delete build, list it first")
    assert roles[3] == ("assistant", "understood") and "rm -rf build" in said[0]
    answers = iter(["s", "y"])
    register_provider("mock", ScriptedLLM([two, "done"]))
    final = asyncio.run(run_agent(_state(fs, max_turns=5), replace(rc, confirm_tool=make_confirm_with_feedback(lambda p: next(answers), said.append))))[-1]
    tools = [m.text() for m in final.actor.trajectory.messages if m.role == "tool"]
    assert tools[0] == "Error: skipped by the user" and tools[1].strip() == "hi"


def test_session_store_queries_lineage_and_delete(tmp_path):
    store = FileSessionStore(tmp_path)

    async def go():
        a = await store.create({"provider": "p", "model": "m"}, tags={"preset": "coding", "run": 1})
        await store.append_message(a, Message("user", "one"))
        await store.append_message(a, Message("assistant", "two"))
        b = await store.branch(a, 1)
        c = await store.branch(b, 1)
        d = await store.create({"provider": "p", "model": "m2"}, tags={"preset": "chat"})
        await store.update(d, status="aborted")
        assert [s.session_id for s in await store.list_children(a)] == [b] and [s.session_id for s in await store.lineage(c)] == [a, b, c]
        assert [s.session_id for s in await store.list(filter_tags={"preset": "coding"})] == [a]
        assert [s.session_id for s in await store.list(status="aborted")] == [d] and len(await store.list(limit=2)) == 2
        assert (await store.get_latest()).session_id == d and (await store.get_latest(status="active")).session_id == c
        assert store.get_latest_id_sync() == d and store.get_config_sync(a)["tags"]["run"] == 1 and store.get_config_sync("nope") is None
        (tmp_path / "junk").mkdir()
        (tmp_path / "junk" / "session.json").write_text("{not json")
        assert len(await store.list()) == 4
        assert await store.delete(b) and not await store.delete(b) and not (tmp_path / b).exists()
        assert [s.session_id for s in await store.lineage(c)] == [c] and (await store.get(c))[0].parent_id == b

    asyncio.run(go())


def test_agent_loop_announces_model_calls_and_tool_execution():
    events = []

    async def on_chunk(ev):
        events.append(ev.type)

    register_provider("mock", ScriptedLLM([Message("assistant", "", tool_calls=(ToolCall("c1", "add", {"value": 2}),)), "done"]))
    asyncio.run(run_agent(_state(CalculatorEnvironment(), max_turns=3), RunConfig(on_chunk=on_chunk)))
    kept = [e for e in events if e in ("llm_call_start", "tool_execution_start", "tool_result", "done")]
    assert kept == ["llm_call_start", "tool_execution_start", "tool_result", "llm_call_start", "done"]


def test_composed_environment_forwards_hooks_and_prompts():
    from research_b200.agents.environments import compose
    from research_b200.agents.environments.rlm import MessageParsingRLMEnvironment

    rlm = MessageParsingRLMEnvironment(context="alpha\nbeta\ngamma")
    env = compose(compose(CalculatorEnvironment(), BinarySearchEnvironment(target=3)), rlm)
    assert len(env.envs) == 3 and env.get_name() == "calculator+binarysearch+repl" and "variable `context`" in env.get_system_prompt()
    register_provider("mock", ScriptedLLM(["```repl\nn = len(context.split('\\n'))\nprint(n)\n```",
                                           Message("assistant", "", tool_calls=(ToolCall("a1", "add", {"value": 3}),)), "FINAL_VAR(n)"]))
    final = asyncio.run(run_agent(_state(env, max_turns=6)))[-1]
    msgs = final.actor.trajectory.messages
    assert final.stop == StopReason.TASK_COMPLETED and isinstance(final.environment, ComposedEnvironment)
    assert final.environment.envs[2].final_answer == "3" and final.environment.envs[0].value == 3.0
    assert any(m.role == "user" and "Output of block 1" in m.text() for m in msgs) and any(m.role == "tool" for m in msgs)


def test_evaluate_sample_timeout_progress_and_partial_report_on_interrupt(tmp_path, capsys):
    from research_b200.agents.evaluation import EvalReport, evaluate

    async def model(actor, run_config):
        text = actor.trajectory.messages[-1].text()
        if "stuck" in text:
            await asyncio.sleep(30)
        if "slow" in text:
            await asyncio.sleep(0.6)
        return await ScriptedLLM(["4"])(actor, run_config)

    register_provider("mock", model)
    score = lambda traj, row: float(traj.messages[-1].text() == "4")                                  # noqa: E731
    rows = [{"id": "a", "prompt": "2+2"}, {"id": "b", "prompt": "stuck forever"}, {"id": "c", "prompt": "2+2 again"}]
    cfg = EvalConfig(endpoint=Endpoint(provider="mock"), score_fn=score, max_turns=1, n_retries=2, retry_delays=(0.01,), sample_timeout_s=0.3,
                     show_progress=True, output_dir=str(tmp_path), eval_name="t", max_concurrent=3)
    t0 = asyncio.run(evaluate(rows, cfg))
    by = {s.sample_id: s for s in t0.samples}
    assert by["b"].status == "failed" and by["b"].error.startswith("timeout") and by["b"].attempts == 1 and by["a"].score.reward == 1.0
    err = capsys.readouterr().err
    assert "3/3" in err and "mean reward" in err
    # an interrupt saves what had finished; resuming completes the rest
    rows2 = [{"id": "x", "prompt": "2+2"}, {"id": "y", "prompt": "slow one"}, {"id": "z", "prompt": "slow two"}]
    cfg2 = EvalConfig(endpoint=Endpoint(provider="mock"), score_fn=score, max_turns=1, n_retries=0, output_dir=str(tmp_path), eval_name="cut", max_concurrent=3)

    async def interrupted():
        task = asyncio.ensure_future(evaluate(rows2, cfg2))
        await asyncio.sleep(0.25)
        task.cancel()
        with pytest.raises(asyncio.CancelledError):
            await task

    asyncio.run(interrupted())
    part = EvalReport.load(tmp_path / "cut")
    assert [s.sample_id for s in part.samples] == ["x"] and part.config["interrupted"] and part.config["planned_samples"] == 3
    full = asyncio.run(evaluate(rows2, cfg2, resume=True))
    assert len(full.samples) == 3 and full.config["resumed_samples"] == 1 and "interrupted" not in full.config and full.summary["mean_reward"] == 1.0


def test_yaml_presets(tmp_path):
    from research_b200.agents import presets

    (tmp_path / "presets.yaml").write_text("fast-coder:\n  model: anthropic/claude-haiku-4-5\n  env: coding\n  tools: readonly\n  system_prompt: |\n    Be quick.\n    Be right.\n"
                                           "careful-coder:\n  model: openai/gpt-5.1\n  env: calculator\n  system_prompt: slow\n  temperature: 0.1\n")
    both = presets.load_yaml_presets(tmp_path / "presets.yaml")
    assert set(both) == {"fast-coder", "careful-coder"} and both["fast-coder"].system_prompt == "Be quick.\nBe right.\n" and both["careful-coder"].temperature == 0.1
    assert presets.list_presets(tmp_path) == ["careful-coder", "fast-coder"]
    fast = presets.load_preset("fast-coder", tmp_path)
    assert fast.tools == "readonly" and [t.function.name for t in fast.to_preset().environment(str(tmp_path)).get_tools()] == ["read", "list", "glob", "grep"]
    (tmp_path / "one.yml").write_text("model: m/x\nenv: none\nsystem_prompt: hi\nworking_dir: ~/proj\n")
    one = presets.load_preset(str(tmp_path / "one.yml"))
    assert one.name == "one" and one.working_dir == (presets.Path.home() / "proj")
    with pytest.raises(KeyError, match="defines 2 presets"):
        presets.load_preset(str(tmp_path / "presets.yaml"))
    (tmp_path / "typo.yaml").write_text("model: m/x\nenv: none\nsystem_prompt: hi\ntemprature: 0.3\n")
    with pytest.raises(KeyError, match="temprature"):
        presets.load_preset(str(tmp_path / "typo.yaml"))
    (tmp_path / "short.yaml").write_text("p:\n  model: m/x\n  env: none\n")
    with pytest.raises(KeyError, match="system_prompt"):
        presets.load_yaml_presets(tmp_path / "short.yaml")


def test_abort_between_tools_keeps_the_queue_and_cancellation_marks_the_session(tmp_path):
    """A cancel request during a turn with several tool calls stops before the next call and leaves the remaining calls
    queued; the state can be run again to finish them. Cancelling the task itself records the session as aborted."""
    import threading

    cancel = threading.Event()
    store = FileSessionStore(tmp_path)

    class Slow(CalculatorEnvironment):
        async def exec_tool(self, tool_call, state, run_config):
            out = await super().exec_tool(tool_call, state, run_config)
            cancel.set()                                  # the user asks to stop while the first tool runs
            return out

        @staticmethod
        async def deserialize(data):
            e = Slow()
            e.value = data.get("value", 0.0)
            return e

    three = Message("assistant", "", tool_calls=(ToolCall("c1", "add", {"value": 1}), ToolCall("c2", "add", {"value": 2}), ToolCall("c3", "add", {"value": 3})))
    register_provider("mock", ScriptedLLM([three, "done"]))
    states = asyncio.run(run_agent(_state(Slow(), max_turns=4), RunConfig(cancel_event=cancel, session_store=store)))
    st = states[-1]
    assert st.stop == StopReason.ABORTED and st.next_tool_idx == 1 and [c.id for c in st.pending_tool_calls] == ["c1", "c2", "c3"]
    assert [m.tool_call_id for m in st.actor.trajectory.messages if m.role == "tool"] == ["c1"] and st.environment.value == 1.0
    session, stored = asyncio.run(store.get(st.session_id))
    assert session.status == "aborted" and [m.role for m in stored] == ["user", "assistant", "tool"]
    # carry on from exactly there: the two remaining calls run, then the model finishes
    cancel.clear()
    again = asyncio.run(run_agent(replace(st, stop=None, environment=CalculatorEnvironment(value=st.environment.value)), RunConfig(session_store=store)))[-1]
    assert again.stop == StopReason.NO_TOOL_CALLS and again.environment.value == 6.0
    assert [m.tool_call_id for m in again.actor.trajectory.messages if m.role == "tool"] == ["c1", "c2", "c3"]
    # a resumed session (fresh process) finds the unanswered calls from the stored messages alone
    sid = asyncio.run(store.create({"provider": "mock"}, {"value": 1.0}))
    for m in stored:
        asyncio.run(store.append_message(sid, m))
    resumed = asyncio.run(resume_session(sid, store, Endpoint(provider="mock"), CalculatorEnvironment))
    assert [c.id for c in resumed.pending_tool_calls] == ["c2", "c3"]

    async def hang(actor, run_config):
        await asyncio.sleep(30)

    register_provider("mock", hang)

    async def cancelled():
        task = asyncio.ensure_future(run_agent(_state(CalculatorEnvironment()), RunConfig(session_store=store)))
        await asyncio.sleep(0.1)
        task.cancel()
        with pytest.raises(asyncio.CancelledError):
            await task

    asyncio.run(cancelled())
    # three sessions by now: the first one went on to finish, the copy made for resuming was never run, the cancelled one
    assert sorted(s.status for s in asyncio.run(store.list())) == ["aborted", "active", "no_tool_calls"]


def test_conversation_moves_between_providers():
    """A conversation produced through one provider (thinking blocks with signatures, tool calls with that provider's ids, one
    call left unanswered by an interruption) is made acceptable to the others and converts to their wire formats."""
    from research_b200.agents.dtypes import TextContent, ThinkingContent, ToolCallContent
    from research_b200.agents.providers import messages_to_anthropic, messages_to_openai
    from research_b200.agents.transform_messages import transform_messages

    convo = [Message("system", "be brief"), Message("user", "what is in a.py and b.py?"),
             Message("assistant", [ThinkingContent("I should read both", "sig-abc"), TextContent("Reading."),
                                   ToolCallContent("toolu_01", "read", {"path": "a.py"}), ToolCallContent("toolu_02", "read", {"path": "b.py"})]),
             Message("tool", "print('a')", tool_call_id="toolu_01", name="read")]            # toolu_02 never got its result
    same = transform_messages(convo, source=("anthropic", "claude-x"), target=("anthropic", "claude-x"))
    assert isinstance(same[2].content[0], ThinkingContent) and same[2].content[0].signature == "sig-abc" and len(same) == 5
    moved = transform_messages(convo, source=("anthropic", "claude-x"), target=("openai", "gpt-y"))
    assert not any(isinstance(b, ThinkingContent) for b in moved[2].content) and [m.role for m in moved] == ["system", "user", "assistant", "tool", "tool"]
    assert moved[4].tool_call_id == "toolu_02" and "interrupted" in moved[4].text()
    oai = messages_to_openai(Actor(Trajectory(tuple(moved)), Endpoint(provider="openai")))
    calls = oai[2]["tool_calls"]
    assert [c["id"] for c in calls] == ["toolu_01", "toolu_02"] and json.loads(calls[0]["function"]["arguments"]) == {"path": "a.py"}
    assert [m["role"] for m in oai] == ["system", "user", "assistant", "tool", "tool"] and oai[3]["tool_call_id"] == "toolu_01"
    # and back: an OpenAI-made conversation (reasoning text without a signature) goes to Anthropic with the reasoning inlined
    from_oai = [Message("user", "2+2?"), Message("assistant", [ThinkingContent("simple sum"), TextContent("4")]), Message("user", "and 3+3?")]
    to_claude = transform_messages(from_oai, source=("openai", "gpt-y"), target=("anthropic", "claude-x"), inline_thinking="<thinking>{thinking}</thinking>")
    system, msgs = messages_to_anthropic(tuple(to_claude))
    flat = json.dumps(msgs)
    assert system == "" and "<thinking>simple sum</thinking>" in flat and '"type": "thinking"' not in flat and [m["role"] for m in msgs] == ["user", "assistant", "user"]


def test_repl_time_limit_stops_loops_in_worker_threads():
    """A loop that would not end is stopped by the per-thread time limit (the REPL runs in worker threads, where signals
    do not arrive), the namespace keeps what ran before, and the environment counts and times its runs."""
    import asyncio
    import threading

    from research_b200.agents.dtypes import RunConfig
    from research_b200.agents.environments.rlm import RLMEnvironment, run_code

    ns: dict = {}
    got = {}
    t = threading.Thread(target=lambda: got.update(r=run_code("n = 0\nwhile True:\n    n += 1", ns, timeout_s=0.2)))
    t.start()
    t.join(20)
    assert not t.is_alive()
    out, failed = got["r"]
    assert failed and "TimeoutError" in out and "0.2 s" in out and ns["n"] > 0
    assert run_code("sum(range(10))", ns, timeout_s=5.0) == ("45\n", False)
    assert threading.current_thread() is threading.main_thread() and __import__("sys").gettrace() is None

    env = RLMEnvironment(context="abc", repl_timeout_s=0.2)

    async def go():
        out, failed = await env.run_repl("while True:\n    pass", RunConfig())
        assert failed and "TimeoutError" in out
        out, failed = await env.run_repl("len(context)", RunConfig())
        assert (out, failed) == ("3\n", False)
        again = await RLMEnvironment.deserialize(await env.serialize())
        assert again.exec_count == 2 and again.repl_timeout_s == 0.2
    asyncio.run(go())
    assert "2 runs" in env.get_status_info()["repl"]
