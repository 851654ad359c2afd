"""Needle in a haystack with a REPL ("recursive language model" pattern of rollouts/examples/eval/rlm/needle_haystack.py):
the long context never enters the prompt. It sits in the REPL namespace as ``context``; the model writes Python to
search it, may call ``llm_query(prompt)`` on slices, and ends with ``FINAL(answer)``. The default model is scripted
(a regex over the context, then a sub-query on the matching line), so the example runs offline."""

import asyncio
import random
import re
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))

from research_b200.agents.dtypes import Endpoint, EvalConfig, Message, Metric, Score, ToolCall  # noqa: E402
from research_b200.agents.environments import REPLEnvironment  # noqa: E402
from research_b200.agents.evaluation import evaluate  # noqa: E402
from research_b200.agents.providers import ScriptedLLM, register_provider  # noqa: E402

FILLER = "The grass is green. The sky is blue. The sun is yellow. Here we go. There and back again."


def make_rows(n: int = 4, lines: int = 2000, seed: int = 0) -> list[dict]:
    rng = random.Random(seed)
    rows = []
    for i in range(n):
        secret = rng.randint(10000, 99999)
        doc = [FILLER] * lines
        doc[rng.randrange(lines)] = f"The special magic number for case {i} is {secret}."
        rows.append({"id": f"needle{i}", "context": "\n".join(doc), "question": f"What is the special magic number for case {i}?", "answer": str(secret)})
    return rows


def sub_model(prompt: str) -> str:
    """What ``llm_query`` calls: here, a reader that extracts the number from a short passage."""
    m = re.search(r"\b(\d{5})\b", prompt)
    return m.group(1) if m else "unknown"


class RLMEnvironment(REPLEnvironment):
    """The agent loop runs every tool call on a copy rebuilt from ``serialize()``; the sub-model hook is not data, so
    it is attached again on the way back."""

    @staticmethod
    async def deserialize(data: dict) -> "RLMEnvironment":
        env = RLMEnvironment(dict(data.get("namespace", {})), llm_query=sub_model)
        env.final_answer = data.get("final_answer")
        return env


def make_env(row: dict) -> RLMEnvironment:
    return RLMEnvironment(namespace={"context": row["context"]}, llm_query=sub_model)


async def scripted_model(actor, run_config):
    code = ("hits = [l for l in context.split('\\n') if 'magic number' in l]\n"
            "print(len(context), len(hits))\n"
            "answer = llm_query('Extract the number: ' + hits[0])\n"
            "print('ANSWER', answer)\n"
            "FINAL(answer)")
    return await ScriptedLLM([Message("assistant", "Searching the context.", tool_calls=(ToolCall("c1", "python", {"code": code}),))])(actor, run_config)


def score_fn(traj, row) -> Score:
    tool_out = "\n".join(m.text() for m in traj.messages if m.role == "tool")
    answers = re.findall(r"^ANSWER (.*)$", tool_out, re.M)
    prompt_chars = sum(len(m.text()) for m in traj.messages if m.role in ("system", "user"))
    return Score((Metric("correct", float(bool(answers) and answers[-1].strip() == row["answer"]), 1.0),
                  Metric("prompt_chars", float(prompt_chars), 0.0)))


def run(rows: list[dict] | None = None, endpoint: Endpoint | None = None):
    rows = rows or make_rows()
    if endpoint is None:
        register_provider("mock", scripted_model)
        endpoint = Endpoint(provider="mock")
    cfg = EvalConfig(endpoint=endpoint, score_fn=score_fn, environment_factory=make_env, max_turns=6, n_retries=0, eval_name="needle_haystack", max_concurrent=1,
                     prepare_messages=lambda r: [Message("system", "A variable `context` holds a long document. Use the python tool to inspect it; "
                                                          "call llm_query(text) for help on short passages; print('ANSWER', value) and finish with FINAL(value)."),
                                                 Message("user", r["question"])])
    return asyncio.run(evaluate(rows, cfg))


if __name__ == "__main__":
    report = run()
    print(report.summary)
