"""Aggregation over a long input with the recursive-language-model environment, in the style of the OOLONG benchmark
(rollouts/examples/eval/rlm/oolong.py): the context is thousands of short user messages, the question asks HOW MANY of
them have some semantic property ("is a complaint"). No single lookup answers it: the input has to be split, every piece
classified by a sub-model (``llm_query`` from inside the REPL), and the counts added up by code.

Offline, both models are stand-ins: the root policy writes the chunk-classify-sum program a capable model writes for this
task, and the sub-model classifies lines by their wording. With real endpoints pass ``endpoint`` / ``sub_endpoint``.
"""

import asyncio
import random
import re
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))

from research_b200.agents.dtypes import Endpoint, EvalConfig, Message, Metric, Score, ToolCall  # noqa: E402
from research_b200.agents.environments.rlm import RLMEnvironment  # noqa: E402
from research_b200.agents.evaluation import evaluate  # noqa: E402
from research_b200.agents.providers import ScriptedLLM, register_provider  # noqa: E402

COMPLAINTS = ["the app crashed again while i was paying", "still waiting for my refund, this is unacceptable", "your support never answers",
              "i was charged twice and nobody cares", "delivery was late for the third time"]
NEUTRAL = ["how do i change my address", "thanks, that solved it", "what are your opening hours", "please send me the invoice",
           "great service today", "can i add a second user", "where can i download the app"]


def make_rows(n: int = 4, lines: int = 600, seed: int = 0) -> list[dict]:
    rng = random.Random(seed)
    rows = []
    for i in range(n):
        msgs, count = [], 0
        for j in range(lines):
            bad = rng.random() < 0.2
            count += bad
            msgs.append(f"[{j:04d}] user{rng.randint(100, 999)}: {rng.choice(COMPLAINTS if bad else NEUTRAL)}")
        rows.append({"id": f"agg-{i}", "context": "\n".join(msgs), "question": "How many of the messages are complaints?", "answer": str(count)})
    return rows


async def sub_model(actor, run_config):
    """Classifies the lines it is shown: answers with the number of complaints among them."""
    text = actor.trajectory.messages[-1].text()
    n = sum(1 for line in text.splitlines() if any(c in line for c in COMPLAINTS))
    return await ScriptedLLM([str(n)])(actor, run_config)


PROGRAM = ("lines = context.split('\\n')\n"
           "total = 0\n"
           "for start in range(0, len(lines), 100):\n"
           "    chunk = '\\n'.join(lines[start:start + 100])\n"
           "    reply = llm_query('Count the complaints among these messages. Answer with a number only.\\n' + chunk)\n"
           "    total += int(reply.strip())\n"
           "print(len(lines), total)")


async def root_policy(actor, run_config):
    tool_msgs = [m for m in actor.trajectory.messages if m.role == "tool"]
    if not tool_msgs:
        return await ScriptedLLM([Message("assistant", "Splitting the input and counting per chunk.", tool_calls=(ToolCall("r1", "repl", {"code": PROGRAM}),))])(actor, run_config)
    total = tool_msgs[-1].text().split()[-1]
    return await ScriptedLLM([Message("assistant", "", tool_calls=(ToolCall("r2", "final_answer", {"answer": total}),))])(actor, run_config)


def score_fn(traj, row) -> Score:
    answer = next((c.args.get("answer") for m in reversed(traj.messages) for c in m.tool_calls if c.name == "final_answer"), None)
    in_prompt = sum(len(m.text()) for m in traj.messages if m.role in ("system", "user"))
    return Score((Metric("correct", float(answer is not None and re.sub(r"\D", "", str(answer)) == row["answer"]), 1.0),
                  Metric("prompt_chars", float(in_prompt), 0.0), Metric("context_chars", float(len(row["context"])), 0.0)))


def run(rows: list[dict] | None = None, endpoint: Endpoint | None = None, sub_endpoint: Endpoint | None = None):
    rows = rows or make_rows()
    if endpoint is None:
        register_provider("rlm-root", root_policy)
        register_provider("rlm-sub", sub_model)
        endpoint, sub_endpoint = Endpoint(provider="rlm-root"), Endpoint(provider="rlm-sub")

    def make_env(row: dict) -> RLMEnvironment:
        return RLMEnvironment(context=row["context"], sub_endpoint=sub_endpoint or endpoint)

    def prepare(row: dict) -> list[Message]:
        return [Message("system", make_env(row).get_system_prompt()), Message("user", row["question"])]

    cfg = EvalConfig(endpoint=endpoint, score_fn=score_fn, environment_factory=make_env, prepare_messages=prepare, max_turns=6, n_retries=0,
                     eval_name="aggregate_records", max_concurrent=2)
    return asyncio.run(evaluate(rows, cfg))


if __name__ == "__main__":
    report = run()
    print(report.summary)
