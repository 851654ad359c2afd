"""Dry run of the browsing evaluation with a scripted searcher-reader (python examples/eval/browsecomp/eval_scripted_01_01.py):
it searches, reads the hits one after another until a page states the fact, and answers from what it read. Swap the endpoint for a real model to run the benchmark proper."""

import re
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))

from examples.eval.browsecomp.base_config import BrowseConfig, run_eval  # noqa: E402
from research_b200.agents.dtypes import Endpoint, Message, ToolCall  # noqa: E402
from research_b200.agents.providers import ScriptedLLM, register_provider  # noqa: E402


async def searcher_reader(actor, run_config):
    msgs = actor.trajectory.messages
    question = next(m.text() for m in msgs if m.role == "user")
    tools = [m.text() for m in msgs if m.role == "tool"]
    n = len(tools)

    def call(name, **args):
        return Message("assistant", "", tool_calls=(ToolCall(f"c{n}", name, args),))

    pattern = r"born in the village of (\w+)" if "born" in question else r"first lit in (\d{4})"
    found = next((m.group(1) for t in tools if (m := re.search(pattern, t))), None)
    fetched = {c.args.get("url") for m in msgs for c in m.tool_calls if c.name == "web_fetch"}
    urls = [u for t in tools for u in re.findall(r"https?://[^\s<]+", t) if u not in fetched]
    if found is not None:
        reply = Message("assistant", f"Explanation: read on the page.\nExact Answer: {found}")
    elif n == 0:
        reply = call("web_search", query=question)
    elif urls:
        reply = call("web_fetch", url=urls[0])
    else:
        reply = Message("assistant", "Explanation: nothing found.\nExact Answer: unknown")
    return await ScriptedLLM([reply])(actor, run_config)


if __name__ == "__main__":
    register_provider("mock", searcher_reader)
    report = run_eval(BrowseConfig(endpoint=Endpoint(provider="mock")))
    for s in report.samples:
        print(s.sample_id, {m.name: m.value for m in s.score.metrics})
    assert report.summary["mean_reward"] == 1.0
