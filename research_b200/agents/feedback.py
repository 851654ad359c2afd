"""Exit survey: now and then, ask the person who ran a session how it went and append the answer to
a JSONL file (rollouts/feedback.py:21-229). Input and output are injectable so it is testable and
silent in non-interactive runs."""

from __future__ import annotations

import json
import os
import random
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Awaitable, Callable

AskFn = Callable[[str], Awaitable[str]]


@dataclass
class ExitSurveyResult:
    session_id: str
    rating: int | None = None             # 1-5
    comment: str = ""
    num_turns: int = 0
    stop_reason: str = ""
    timestamp: float = field(default_factory=time.time)


def feedback_path() -> Path:
    base = os.environ.get("RESEARCH_B200_HOME") or os.path.join(os.path.expanduser("~"), ".research_b200")
    return Path(base) / "feedback.jsonl"


def should_survey(num_turns: int, interactive: bool, probability: float = 0.2, min_turns: int = 3, rng: random.Random | None = None) -> bool:
    """Only interactive sessions of some length are surveyed, and only a fraction of those."""
    if not interactive or num_turns < min_turns or os.environ.get("RESEARCH_B200_NO_SURVEY"):
        return False
    return (rng or random).random() < probability


async def collect_exit_survey(session_id: str, ask: AskFn, num_turns: int = 0, stop_reason: str = "") -> ExitSurveyResult | None:
    raw = (await ask("How did this session go? 1 (bad) - 5 (great), Enter to skip: ")).strip()
    if not raw:
        return None
    rating = int(raw[0]) if raw[0].isdigit() and 1 <= int(raw[0]) <= 5 else None
    comment = raw if rating is None else (await ask("Anything to add? (Enter to skip): ")).strip()
    return ExitSurveyResult(session_id, rating, comment, num_turns, stop_reason)


def save_survey_result(result: ExitSurveyResult, path: Path | None = None) -> Path:
    path = path or feedback_path()
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("a") as f:
        f.write(json.dumps(asdict(result)) + "\n")
    return path


async def run_exit_survey(session_id: str, ask: AskFn, num_turns: int, stop_reason: str, interactive: bool = True,
                          probability: float = 0.2, path: Path | None = None, rng: random.Random | None = None) -> ExitSurveyResult | None:
    if not should_survey(num_turns, interactive, probability, rng=rng):
        return None
    result = await collect_exit_survey(session_id, ask, num_turns, stop_reason)
    if result is not None:
        save_survey_result(result, path)
    return result
