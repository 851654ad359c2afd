"""Verifiers-style environment adapters: dataset rows, rubric -> Score, environment replies in the agent loop."""

import asyncio
from dataclasses import replace

import pytest

from research_b200.agents.dtypes import Endpoint, Message, Score, ToolCall, Trajectory
from research_b200.agents.integrations import (dataset_rows, evaluate_env, prepare_messages, prime_reward_fn,
                                               split_prompt_completion, to_chat)
from research_b200.agents.providers import ScriptedLLM, register_provider


class _Result:
    def __init__(self, reward, metrics):
        self.reward, self.metrics = reward, metrics


class _Rubric:
    async def score_rollout(self, prompt, completion, answer, state, **_):
        last = next((m["content"] for m in reversed(completion) if m["role"] == "assistant"), "")
        return _Result(1.0 if last.strip() == answer else 0.0, {"turns": state["turn"], "prompt_len": len(prompt)})


class _SingleTurnEnv:
    max_turns = 1
    parser = None
    rubric = _Rubric()
    dataset = [{"question": "2+2?", "answer": "4"}, {"question": "3+3?", "answer": "6"}, {"question": "1+1?", "answer": "2"}]


class _GuessEnv:
    """Higher / lower game: the environment answers every guess until the number is hit."""
    max_turns = 6
    rubric = _Rubric()
    eval_dataset = [{"prompt": [{"role": "system", "content": "guess"}, {"role": "user", "content": "start"}], "answer": "7", "id": "g0"}]

    def is_completed(self, messages, state):
        return messages[-1]["content"].strip() == state["answer"]

    async def env_response(self, messages, state):
        guess = int(messages[-1]["content"])
        return [{"role": "user", "content": "higher" if guess < int(state["answer"]) else "lower"}], {"guesses": state.get("guesses", 0) + 1}


def test_rows_messages_and_chat_conversion():
    assert len(dataset_rows(_SingleTurnEnv())) == 3 and len(dataset_rows(_SingleTurnEnv(), 2)) == 2
    assert dataset_rows(_GuessEnv())[0]["id"] == "g0"
    with pytest.raises(ValueError):
        dataset_rows(object())
    m = prepare_messages({"question": "q"}, "be brief")
    assert [x.role for x in m] == ["system", "user"] and m[1].text() == "q"
    assert [x.role for x in prepare_messages(_GuessEnv.eval_dataset[0])] == ["system", "user"]
    chat = to_chat([Message("assistant", "hi", tool_calls=(ToolCall("c1", "add", {"v": 1}),)), Message("tool", "3", tool_call_id="c1")])
    assert chat[0]["tool_calls"][0]["function"] == {"name": "add", "arguments": {"v": 1}} and chat[1]["tool_call_id"] == "c1"
    traj = Trajectory((Message("system", "be brief"), Message("user", "q"), Message("assistant", "a")))
    prompt, completion = split_prompt_completion(traj, {"question": "q"})
    assert [p["role"] for p in prompt] == ["system", "user"] and completion == [{"role": "assistant", "content": "a"}]


def test_rubric_forms():
    traj = Trajectory((Message("user", "2+2?"), Message("assistant", "4")))
    row = {"question": "2+2?", "answer": "4"}
    s = asyncio.run(prime_reward_fn(_SingleTurnEnv())(traj, row))
    assert isinstance(s, Score) and s.reward == 1.0 and {m.name for m in s.metrics} == {"reward", "turns", "prompt_len"}

    def exact(completion, answer):
        return float(completion[-1]["content"] == answer)

    async def brevity(completion, **kw):
        return 1.0 / len(completion[-1]["content"])

    class FuncRubric:
        reward_funcs = [exact, brevity]
        reward_weights = [1.0, 0.5]

    class E:
        rubric = FuncRubric()

    s = asyncio.run(prime_reward_fn(E())(traj, row))
    assert s.reward == pytest.approx(1.5) and [m.name for m in s.metrics] == ["reward", "exact", "brevity"]

    class NumberRubric:
        def score_rollout(self, completion):
            return 0.25

    class DictRubric:
        def score_rollout(self, **kw):
            return {"reward": 0.5, "metrics": {"x": 2}}

    for rub, want in ((NumberRubric(), 0.25), (DictRubric(), 0.5)):
        env = type("Env", (), {"rubric": rub})()
        assert asyncio.run(prime_reward_fn(env)(traj, row)).reward == want
    with pytest.raises(ValueError):
        prime_reward_fn(object())
    with pytest.raises(ValueError):
        asyncio.run(prime_reward_fn(type("Env", (), {"rubric": object()})())(traj, row))


def test_single_and_multi_turn_evaluation(tmp_path):
    answers = {"2+2?": "4", "3+3?": "6", "1+1?": "3"}                     # the model gets the last one wrong

    async def model(actor, run_config):
        q = next(m.text() for m in actor.trajectory.messages if m.role == "user")
        return await ScriptedLLM([answers[q]])(actor, run_config)

    register_provider("mock", model)
    rep = asyncio.run(evaluate_env(_SingleTurnEnv(), Endpoint(provider="mock"), output_dir=str(tmp_path)))
    assert [s.score.reward for s in rep.samples] == [1.0, 1.0, 0.0] and rep.summary["mean_reward"] == pytest.approx(2 / 3)
    assert any(tmp_path.iterdir())

    class Bisect:                                                           # a model that really plays the game
        async def __call__(self, actor, run_config):
            lo, hi, last = 0, 16, None
            for m in actor.trajectory.messages:
                if m.role == "assistant":
                    last = int(m.text())
                elif last is not None and m.text() == "higher":
                    lo = last + 1
                elif last is not None and m.text() == "lower":
                    hi = last - 1
            return await ScriptedLLM([str((lo + hi) // 2)])(actor, run_config)

    register_provider("mock", Bisect())
    rep = asyncio.run(evaluate_env(_GuessEnv(), Endpoint(provider="mock")))
    s = rep.samples[0]
    assert s.sample_id == "g0" and s.score.reward == 1.0 and s.stop_reason == "task_completed"
    roles = [m.role for m in s.trajectory.messages]
    assert roles[:2] == ["system", "user"] and roles[-1] == "assistant" and roles.count("user") >= 2
    assert s.trajectory.metadata["env_state"]["guesses"] >= 1
    turns = next(m.value for m in s.score.metrics if m.name == "turns")
    assert turns == roles.count("assistant")


def test_rate_limit_stress_run():
    from research_b200.agents.providers import NonRetryableError
    from research_b200.agents.providers.stress import main, simulated_provider, stress

    async def no_sleep(_):
        await asyncio.sleep(0)

    # a tight server quota with an unthrottled client: many calls get a 429 first, all succeed after retries
    rep = asyncio.run(stress(simulated_provider(quota=5, window_s=0.05, latency_s=0.001), requests=40, max_concurrent=16,
                             max_attempts=50, backoff_base=0.01, max_delay=0.05))
    assert rep.succeeded == 40 and rep.failed == 0 and rep.rate_limited_calls > 0 and rep.retries >= rep.rate_limited_calls
    assert rep.peak_in_flight <= 16 and rep.achieved_rps > 0 and rep.percentile(0.95) >= rep.percentile(0.5) > 0
    d = rep.to_dict()
    assert "latencies" not in d and d["p99_s"] >= d["p50_s"] and "40/40 ok" in rep.summary()
    # a client-side rate below the quota never trips it
    calm = asyncio.run(stress(simulated_provider(quota=50, window_s=0.2, latency_s=0.0), requests=20, max_concurrent=4, requests_per_second=200))
    assert calm.succeeded == 20 and calm.rate_limited_calls == 0 and calm.retries == 0 and calm.peak_in_flight <= 4
    # attempts exhausted -> failed; a non-retryable error is not retried

    async def always_429():
        from research_b200.agents.providers import ProviderError
        raise ProviderError("HTTP 429", 429)

    gone = asyncio.run(stress(always_429, requests=3, max_attempts=3, sleep=no_sleep))
    assert gone.failed == 3 and gone.retries == 6 and gone.succeeded == 0

    async def bad_key():
        raise NonRetryableError("HTTP 401", 401)

    auth = asyncio.run(stress(bad_key, requests=4, sleep=no_sleep))
    assert auth.failed == 4 and auth.non_retryable == 4 and auth.retries == 0
    assert main(["--requests", "20", "--concurrency", "4", "--quota", "100", "--latency", "0"]) == 0


def test_stateful_tool_environment_adapter(caplog):
    """A kernel-bench-like environment: one tool that 'tests' submitted code, state that keeps the best result as an
    object, prints that must end up in the log, completion once a submission passes; and the text-only path."""
    import asyncio
    import logging

    from research_b200.agents.agents import run_agent
    from research_b200.agents.dtypes import Actor, AgentState, Endpoint, Message, RunConfig, StopReason, ToolCall, Trajectory
    from research_b200.agents.integrations import StatefulToolEnvironment
    from research_b200.agents.providers import ScriptedLLM, register_provider

    class Result:                                          # not JSON-serialisable on purpose
        def __init__(self, ok):
            self.ok = ok

    class KernelBench:
        oai_tools = [{"type": "function", "function": {"name": "run_code", "description": "compile and test a kernel",
                                                         "parameters": {"type": "object", "properties": {"code": {"type": "string"}}, "required": ["code"]}}}]

        async def env_response(self, messages, state):
            last = messages[-1]
            state = dict(state)
            if last.get("tool_calls"):
                import json

                code = json.loads(last["tool_calls"][0]["function"]["arguments"])["code"]
                ok = "return a + b" in code
                print(f"testing submission {len(state.get('results', [])) + 1}: {'pass' if ok else 'fail'}")
                state["results"] = state.get("results", []) + [Result(ok)]
                return messages + [{"role": "tool", "tool_call_id": last["tool_calls"][0]["id"], "content": "all tests pass" if ok else "wrong output for test 0"}], state
            return [{"role": "user", "content": "Please submit code with the run_code tool."}], state

        def is_completed(self, messages, state):
            return any(r.ok for r in state.get("results", []))

    env = StatefulToolEnvironment(KernelBench(), {"task": "add"})
    assert [t.function.name for t in env.get_tools()] == ["run_code"] and env.get_tools()[0].function.parameters.required == ("code",)
    register_provider("mock", ScriptedLLM(["I think the kernel should add the inputs.",
                                           Message("assistant", "", tool_calls=(ToolCall("k1", "run_code", {"code": "return a - b"}),)),
                                           Message("assistant", "", tool_calls=(ToolCall("k2", "run_code", {"code": "return a + b"}),))]))
    with caplog.at_level(logging.INFO):
        start = AgentState(Actor(Trajectory((Message("user", "write an add kernel"),)), Endpoint(provider="mock")), env, max_turns=6)
        final = asyncio.run(run_agent(start, RunConfig()))[-1]
    msgs = final.actor.trajectory.messages
    assert final.stop == StopReason.TASK_COMPLETED and final.turn_idx == 3
    assert [m.role for m in msgs] == ["user", "assistant", "user", "assistant", "tool", "assistant", "tool"]
    assert "run_code tool" in msgs[2].text() and "wrong output" in msgs[4].text() and msgs[6].text() == "all tests pass"
    kept = final.environment.state["results"]
    assert [r.ok for r in kept] == [False, True] and isinstance(kept[0], Result)             # objects in the state survive the per-call copies
    assert "testing submission 1: fail" in caplog.text and "testing submission 2: pass" in caplog.text
