"""GEPA on an intent-classification task in the style of banking77 (rollouts/examples/prompt_optimization/banking77_gepa.py):
customer messages, a closed label set, exact-match scoring. The candidate has two components, the system prompt and
the user template, and the optimiser improves them in turn from the feedback the scorer writes.

The task model here is a stand-in with the failure modes a small model shows on this task: without the label list it
invents labels, and without a format instruction it answers in a sentence. Both are fixed by instructions, which is
what the scripted reflection model proposes when it sees the corresponding feedback. Replace ``generate`` / ``reflect``
with provider calls to optimise a real prompt; the data layout (``{"input", "answer"}`` rows) stays.
"""

import asyncio
import random
import re
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from research_b200.agents.prompt_optimization import GEPAConfig, optimize_prompt  # noqa: E402

INTENTS = {
    "card_arrival": ["my new card still has not arrived", "how long until the card gets here", "card was ordered two weeks ago, where is it"],
    "lost_or_stolen_card": ["i lost my card on the train", "someone stole my wallet with the card in it", "my card is missing, block it"],
    "exchange_rate": ["what rate do you use for euros", "is your exchange rate updated on weekends", "how do you calculate the dollar rate"],
    "top_up_failed": ["my top up did not go through", "the money i added is not showing", "top-up was declined twice"],
    "change_pin": ["i want a different pin", "how do i change my pin at an atm", "can i set a new pin in the app"],
    "terminate_account": ["close my account please", "i want to delete my account", "how do i end my membership"],
}
LABELS = sorted(INTENTS)
KEYWORDS = {"card_arrival": ("arriv", "gets here", "ordered", "where is it"), "lost_or_stolen_card": ("lost", "stole", "missing"),
            "exchange_rate": ("rate",), "top_up_failed": ("top up", "top-up", "added"), "change_pin": ("pin",),
            "terminate_account": ("close", "delete", "end my")}


def make_set(n: int, seed: int) -> list[dict]:
    rng = random.Random(seed)
    rows = [{"input": text, "answer": label} for label, texts in INTENTS.items() for text in texts]
    rng.shuffle(rows)
    return rows[:n]


def _guess(text: str) -> str:
    return next((label for label, keys in KEYWORDS.items() if any(k in text.lower() for k in keys)), "other")


async def generate(system: str, user: str) -> str:
    """The stand-in task model. It reads the customer's message from the last line of the user turn."""
    message = user.strip().splitlines()[-1]
    label = _guess(message)
    knows_labels = all(lbl in system + user for lbl in LABELS)
    if not knows_labels:
        label = label.replace("_", " ").replace("lost or stolen card", "card problem").replace("terminate account", "cancellation")
    if "only the label" not in (system + user).lower():
        return f"This looks like a {label} request."
    return label


def score(sample: dict, text: str) -> tuple[float, str]:
    """Exact match scores 1. Partial credit keeps the search informed: the right label inside a sentence (0.5), the right
    idea in the model's own words (0.25)."""
    got, want = text.strip(), sample["answer"]
    if got == want:
        return 1.0, "correct"
    if want in got:
        return 0.5, f"the answer is buried in a sentence ({got!r}); reply with only the label. Expected {want}."
    if got not in LABELS and re.fullmatch(r"[a-z_ ]+", got):
        close = 0.25 if got.replace(" ", "_") == want else 0.0
        return close, f"'{got}' is not one of the allowed labels; the label set was not given to the model. Expected {want}."
    return 0.0, f"wrong or unparseable answer {got!r}: not one of the allowed labels, and reply with only the label. Expected {want}."


async def reflect(prompt: str) -> str:
    """The stand-in reflection model: one fix per round, chosen from the feedback it is shown, written into whichever
    component it was asked to rewrite."""
    current = prompt.split("```")[1].strip() if prompt.count("```") >= 2 else ""
    rewriting_template = "{input}" in current
    if "label set was not given" in prompt or "not one of the allowed labels" in prompt:
        if not all(lbl in current for lbl in LABELS):
            add = "Allowed labels: " + ", ".join(LABELS) + "."
            return f"```\n{add}\n{current}\n```" if rewriting_template else f"```\n{current} {add}\n```"
    if "only the label" in prompt and "only the label" not in current.lower():
        add = "Reply with only the label, exactly as written in the list."
        return f"```\n{add}\n{current}\n```" if rewriting_template else f"```\n{current} {add}\n```"
    return f"```\n{current}\n```"


def run(max_evaluations: int = 200):
    return asyncio.run(optimize_prompt("You classify customer messages for a bank.", "{input}", generate, score, make_set(12, 0), make_set(18, 1),
                                       reflect, GEPAConfig(max_evaluations=max_evaluations, minibatch_size=4, seed=0)))


if __name__ == "__main__":
    result = run()
    print(f"best validation score {result.best_score:.2f}\nsystem: {result.best_candidate['system']!r}\nuser template: {result.best_candidate['user_template']!r}")
