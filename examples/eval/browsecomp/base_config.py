"""Browsing evaluation (rollouts/examples/eval/browsecomp/base_config.py): hard-to-find facts that need a search and
one or two page reads; the grader compares the final answer with the reference answer. ``OfflineWeb`` is a small
in-memory web (pages + a keyword search) so the pipeline runs without a network; with the default ``fetcher`` /
``searcher`` of ``BrowsingEnvironment`` the same code browses the real web."""

from __future__ import annotations

import asyncio
import re
from dataclasses import dataclass
from typing import Any

from research_b200.agents.dtypes import Endpoint, EvalConfig, Message, Metric, Score, Trajectory
from research_b200.agents.environments.interactive import BrowsingEnvironment
from research_b200.agents.evaluation import EvalReport, evaluate

SYSTEM_PROMPT = ("Answer the question. Use web_search to find pages and web_fetch to read them. "
                 "Finish with a line 'Exact Answer: <answer>'.")


class OfflineWeb:
    def __init__(self, pages: dict[str, tuple[str, str]]):
        self.pages = pages                                   # url -> (title, text)

    async def search(self, query: str, k: int) -> list[dict[str, str]]:
        words = set(re.findall(r"\w+", query.lower()))
        scored = sorted(((len(words & set(re.findall(r"\w+", (t + " " + b).lower()))), u, t, b) for u, (t, b) in self.pages.items()), reverse=True)
        return [{"title": t, "url": u, "snippet": b[:30] + "..."} for n, u, t, b in scored[:k] if n > 0]

    async def fetch(self, url: str) -> tuple[int, str, str]:
        if url not in self.pages:
            return 404, "text/plain", "not found"
        title, body = self.pages[url]
        return 200, "text/html", f"<html><head><title>{title}</title></head><body><h1>{title}</h1><p>{body}</p></body></html>"

    def environment(self) -> BrowsingEnvironment:
        return _OfflineBrowsing(self)


def _OfflineBrowsing(web: OfflineWeb) -> BrowsingEnvironment:
    class Env(BrowsingEnvironment):
        @staticmethod
        async def deserialize(data: dict[str, Any]) -> "BrowsingEnvironment":        # keep the in-memory web across tool calls
            return Env(fetcher=web.fetch, searcher=web.search, history=list(data.get("history", [])), max_chars=int(data.get("max_chars", 20_000)))

    return Env(fetcher=web.fetch, searcher=web.search)


DEMO_WEB = OfflineWeb({
    "https://lighthouses.example/skerry": ("Skerry Point lighthouse", "Skerry Point lighthouse was first lit in 1871. Its keeper for 31 years was Marit Olsen."),
    "https://lighthouses.example/list": ("Lighthouses of the north coast", "Skerry Point, Gull Rock and Tern Head are the three lights of the north coast."),
    "https://people.example/olsen": ("Marit Olsen", "Marit Olsen, lighthouse keeper, was born in the village of Askvik."),
})
DEMO_ROWS = [
    {"id": "keeper_birthplace", "question": "In which village was the long-serving keeper of Skerry Point lighthouse born?", "answer": "Askvik"},
    {"id": "first_lit", "question": "In which year was Skerry Point lighthouse first lit?", "answer": "1871"},
]


def extract_answer(text: str) -> str | None:
    m = re.findall(r"Exact Answer:\s*(.+)", text)
    return m[-1].strip().rstrip(".") if m else None


def score_fn(traj: Trajectory, row: dict[str, Any]) -> Score:
    finals = [m.text() for m in traj.messages if m.role == "assistant" and m.text()]
    got = extract_answer(finals[-1]) if finals else None
    pages = sum(1 for m in traj.messages for c in m.tool_calls if c.name == "web_fetch")
    searches = sum(1 for m in traj.messages for c in m.tool_calls if c.name == "web_search")
    correct = float(got is not None and got.lower() == str(row["answer"]).lower())
    return Score((Metric("correct", correct, 1.0), Metric("answered", float(got is not None), 0.0), Metric("pages_read", float(pages), 0.0),
                  Metric("searches", float(searches), 0.0)))


@dataclass(frozen=True)
class BrowseConfig:
    endpoint: Endpoint
    max_turns: int = 8
    max_concurrent: int = 2
    output_dir: str | None = None
    eval_name: str = "browsecomp"


def run_eval(config: BrowseConfig, rows: list[dict[str, Any]] | None = None, web: OfflineWeb | None = DEMO_WEB) -> EvalReport:
    ec = EvalConfig(endpoint=config.endpoint, score_fn=score_fn, max_turns=config.max_turns, max_concurrent=config.max_concurrent, n_retries=0,
                    environment_factory=(lambda row: web.environment()) if web is not None else (lambda row: BrowsingEnvironment()),
                    prepare_messages=lambda row: [Message("system", SYSTEM_PROMPT), Message("user", row["question"])],
                    output_dir=config.output_dir, eval_name=config.eval_name)
    return asyncio.run(evaluate(rows or DEMO_ROWS, ec))
