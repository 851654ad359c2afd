"""Environments that talk to something outside the model: the user, the web, a screenshot grader.

* ``AskUserQuestionEnvironment`` - one tool that puts 1-4 multiple-choice questions to a person
  through an injectable async handler (rollouts/environments/ask_user.py:182).
* ``BrowsingEnvironment`` - ``web_search`` / ``web_fetch`` through injectable callables; the defaults
  use ``urllib`` and fail cleanly where there is no network (rollouts/environments/browsing.py:116).
* ``ScreenSpotEnvironment`` - no tools; a reward that checks whether the predicted click point
  (or the centre of the predicted box) falls inside the ground-truth box
  (rollouts/environments/screenspot.py:14).
"""

from __future__ import annotations

import asyncio
import html
import json
import re
import urllib.parse
import urllib.request
from dataclasses import dataclass, field
from typing import Any, Awaitable, Callable

from ..dtypes import AgentState, RunConfig, Tool, ToolCall, ToolFunction, ToolFunctionParameter, ToolResult

QuestionHandler = Callable[[list[dict[str, Any]]], Awaitable[dict[str, str]]]


async def stdin_question_handler(questions: list[dict[str, Any]]) -> dict[str, str]:
    """Ask on the terminal: a number picks an option, anything else is taken as free text."""
    answers: dict[str, str] = {}
    loop = asyncio.get_running_loop()
    for q in questions:
        lines = [f"[{q.get('header', '?')}] {q['question']}"]
        for i, opt in enumerate(q["options"], 1):
            lines.append(f"  {i}. {opt['label']} - {opt.get('description', '')}")
        lines.append("  (several numbers separated by commas)" if q.get("multiSelect") else "")
        raw = (await loop.run_in_executor(None, input, "\n".join(lines) + "\n> ")).strip()
        picks = []
        for part in raw.split(","):
            part = part.strip()
            if part.isdigit() and 1 <= int(part) <= len(q["options"]):
                picks.append(q["options"][int(part) - 1]["label"])
        answers[q["question"]] = ", ".join(picks) if picks else raw
    return answers


def validate_questions(questions: Any) -> str | None:
    """Return an error message if the tool arguments break the schema, else None."""
    if not isinstance(questions, list) or not 1 <= len(questions) <= 4:
        return "questions must be a list of 1-4 items"
    for q in questions:
        if not isinstance(q, dict) or not isinstance(q.get("question"), str):
            return "every question needs a 'question' string"
        opts = q.get("options")
        if not isinstance(opts, list) or not 2 <= len(opts) <= 4:
            return f"question {q.get('question', '?')!r} needs 2-4 options"
        if any(not isinstance(o, dict) or "label" not in o for o in opts):
            return "every option needs a 'label'"
        if len(str(q.get("header", ""))) > 12:
            return "header is limited to 12 characters"
    return None


@dataclass
class AskUserQuestionEnvironment:
    question_handler: QuestionHandler = stdin_question_handler

    def get_name(self) -> str:
        return "ask_user"

    def get_tools(self) -> list[Tool]:
        option = {"type": "object", "properties": {"label": {"type": "string"}, "description": {"type": "string"}},
                  "required": ["label", "description"]}
        question = {"type": "object",
                    "properties": {"question": {"type": "string"}, "header": {"type": "string", "maxLength": 12},
                                   "options": {"type": "array", "minItems": 2, "maxItems": 4, "items": option},
                                   "multiSelect": {"type": "boolean", "default": False}},
                    "required": ["question", "header", "options", "multiSelect"]}
        return [Tool(ToolFunction(
            "ask_user_question",
            "Ask the user 1-4 multiple-choice questions (2-4 options each; a free-text answer is always possible).",
            ToolFunctionParameter({"questions": {"type": "array", "minItems": 1, "maxItems": 4, "items": question}},
                                  ("questions",))))]

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        return False   # the tool is itself a user interaction

    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        if tool_call.name != "ask_user_question":
            return ToolResult(tool_call.id, is_error=True, error=f"unknown tool {tool_call.name!r}")
        questions = tool_call.args.get("questions")
        err = validate_questions(questions)
        if err:
            return ToolResult(tool_call.id, is_error=True, error=err)
        try:
            answers = await self.question_handler(questions)
        except Exception as e:  # noqa: BLE001 - handler failures go back to the model
            return ToolResult(tool_call.id, is_error=True, error=f"could not ask the user: {e}")
        lines = [f"Q: {q['question']}\nA: {answers.get(q['question'], '(no answer)')}" for q in questions]
        return ToolResult(tool_call.id, content="\n\n".join(lines), metadata={"answers": answers})

    async def serialize(self) -> dict[str, Any]:
        return {"env_kind": "ask_user"}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "AskUserQuestionEnvironment":
        return AskUserQuestionEnvironment()   # the handler is code, not state


# ------------------------------------------------------------------------------------------ browsing
Fetcher = Callable[[str], Awaitable[tuple[int, str, str]]]          # url -> (status, content_type, body)
Searcher = Callable[[str, int], Awaitable[list[dict[str, str]]]]    # query, k -> [{title, url, snippet}]

_TAG = re.compile(r"<(script|style)[^>]*>.*?</\1>|<[^>]+>", re.DOTALL | re.IGNORECASE)


def html_to_text(body: str) -> str:
    text = html.unescape(_TAG.sub(" ", body))
    return re.sub(r"[ \t]*\n\s*", "\n", re.sub(r"[ \t]+", " ", text)).strip()


async def urllib_fetch(url: str) -> tuple[int, str, str]:
    def go() -> tuple[int, str, str]:
        req = urllib.request.Request(url, headers={"User-Agent": "research-b200-agent/1.0"})
        with urllib.request.urlopen(req, timeout=20) as r:  # noqa: S310 - http(s) checked by the caller
            return r.status, r.headers.get("content-type", ""), r.read(2_000_000).decode("utf-8", "replace")

    return await asyncio.get_running_loop().run_in_executor(None, go)


async def duckduckgo_search(query: str, k: int) -> list[dict[str, str]]:
    status, _, body = await urllib_fetch("https://html.duckduckgo.com/html/?q=" + urllib.parse.quote(query))
    if status != 200:
        raise RuntimeError(f"search returned HTTP {status}")
    out = []
    for m in re.finditer(r'class="result__a" href="([^"]+)"[^>]*>(.*?)</a>', body, re.DOTALL):
        out.append({"url": html.unescape(m.group(1)), "title": html_to_text(m.group(2)), "snippet": ""})
        if len(out) >= k:
            break
    return out


@dataclass
class BrowsingEnvironment:
    fetcher: Fetcher = urllib_fetch
    searcher: Searcher = duckduckgo_search
    max_chars: int = 20_000
    history: list[str] = field(default_factory=list)

    def get_name(self) -> str:
        return "browsing"

    def get_status_info(self) -> dict[str, str] | None:
        return {"pages": str(len(self.history))}

    def get_tools(self) -> list[Tool]:
        return [
            Tool(ToolFunction("web_search", "Search the web; returns titles, URLs and snippets.",
                              ToolFunctionParameter({"query": {"type": "string"},
                                                     "max_results": {"type": "integer", "default": 5}}, ("query",)))),
            Tool(ToolFunction("web_fetch", "Fetch a URL and return its text (HTML is reduced to text).",
                              ToolFunctionParameter({"url": {"type": "string"}}, ("url",)))),
        ]

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        return False

    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        try:
            if tool_call.name == "web_search":
                k = max(1, min(int(tool_call.args.get("max_results", 5)), 20))
                hits = await self.searcher(str(tool_call.args["query"]), k)
                if not hits:
                    return ToolResult(tool_call.id, content="no results")
                body = "\n\n".join(f"{i}. {h.get('title', '')}\n   {h.get('url', '')}\n   {h.get('snippet', '')}"
                                   for i, h in enumerate(hits, 1))
                return ToolResult(tool_call.id, content=body, metadata={"results": hits})
            if tool_call.name == "web_fetch":
                url = str(tool_call.args["url"])
                if urllib.parse.urlparse(url).scheme not in ("http", "https"):
                    return ToolResult(tool_call.id, is_error=True, error="only http(s) URLs can be fetched")
                status, ctype, body = await self.fetcher(url)
                if status >= 400:
                    return ToolResult(tool_call.id, is_error=True, error=f"HTTP {status} for {url}")
                text = html_to_text(body) if "html" in ctype or body.lstrip().startswith("<") else body
                self.history.append(url)
                clipped = text[: self.max_chars]
                note = f"\n\n[truncated: {len(text) - self.max_chars} more characters]" if len(text) > self.max_chars else ""
                return ToolResult(tool_call.id, content=clipped + note, metadata={"url": url, "status": status})
            return ToolResult(tool_call.id, is_error=True, error=f"unknown tool {tool_call.name!r}")
        except KeyError as e:
            return ToolResult(tool_call.id, is_error=True, error=f"missing argument {e}")
        except Exception as e:  # noqa: BLE001 - network failures go back to the model
            return ToolResult(tool_call.id, is_error=True, error=f"{type(e).__name__}: {e}")

    async def serialize(self) -> dict[str, Any]:
        return {"env_kind": "browsing", "history": list(self.history), "max_chars": self.max_chars}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "BrowsingEnvironment":
        return BrowsingEnvironment(history=list(data.get("history", [])), max_chars=int(data.get("max_chars", 20_000)))


# ------------------------------------------------------------------------------------------ screenspot
_BOX = re.compile(r"\[\[(\d+\.?\d*),\s*(\d+\.?\d*),\s*(\d+\.?\d*),\s*(\d+\.?\d*)\]\]")
_POINT = re.compile(r"\[\[(\d+\.?\d*),\s*(\d+\.?\d*)\]\]")


class ScreenSpotEnvironment:
    """GUI grounding: the answer is a point ``[[x,y]]`` or a box ``[[x0,y0,x1,y1]]`` in 0-1 coordinates."""

    def get_tools(self) -> list[Tool]:
        return []

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        return False

    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        return ToolResult(tool_call.id, is_error=True, error="this environment has no tools")

    async def serialize(self) -> dict[str, Any]:
        return {"env_kind": "screenspot"}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "ScreenSpotEnvironment":
        return ScreenSpotEnvironment()

    @staticmethod
    def extract_bbox(text: str) -> list[float] | None:
        m = _BOX.search(text)
        return [float(g) for g in m.groups()] if m else None

    @staticmethod
    def extract_point(text: str) -> list[float] | None:
        m = _POINT.search(text)
        return [float(g) for g in m.groups()] if m else None

    @staticmethod
    def compute_reward(response_text: str, gt_bbox: list[int], img_size: list[int]) -> float:
        """1.0 when the predicted click lands inside the ground-truth box (pixels, ``[x1,y1,x2,y2]``)."""
        assert len(gt_bbox) == 4 and len(img_size) == 2
        point = ScreenSpotEnvironment.extract_point(response_text)
        if point is None:
            box = ScreenSpotEnvironment.extract_bbox(response_text)
            if box is None:
                return 0.0
            point = [(box[0] + box[2]) / 2, (box[1] + box[3]) / 2]
        w, h = img_size
        x0, y0, x1, y1 = gt_bbox[0] / w, gt_bbox[1] / h, gt_bbox[2] / w, gt_bbox[3] / h
        return 1.0 if x0 <= point[0] <= x1 and y0 <= point[1] <= y1 else 0.0


def to_json(obj: Any) -> str:
    return json.dumps(obj, ensure_ascii=False)
