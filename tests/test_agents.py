"""Agent runtime without a network: scripted model, environments, sessions, evaluation, TI/TO."""

import asyncio
import json

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
