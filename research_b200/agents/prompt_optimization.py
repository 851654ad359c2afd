"""GEPA: reflective prompt evolution with a Pareto front of candidates
(rollouts/prompt_optimization/engine.py:26-274, operations.py:40-253, gepa.py:24-379).

A *candidate* is a dict ``component name -> text`` (e.g. ``{"system": ..., "user_template": ...}``).
One iteration: pick a candidate from the Pareto front (per-validation-sample winners, sampled in
proportion to how many samples they win), evaluate it on a minibatch with traces, ask a reflection
model to rewrite one component given the traces and feedback, re-evaluate on the same minibatch and
keep the child only if the minibatch sum improved; accepted children are scored on the validation
set and update the front. The model calls (task evaluation and reflection) are injected, so the
loop runs against any provider - or against scripted functions in tests.

Also here: the simpler evolutionary variant (elites, tournament selection, sentence-level crossover,
LLM mutation).
"""

from __future__ import annotations

import random
import re
from dataclasses import dataclass, field
from typing import Any, Awaitable, Callable, Protocol, Sequence

Candidate = dict[str, str]


@dataclass
class EvaluationBatch:
    scores: list[float]
    outputs: list[Any] = field(default_factory=list)
    traces: list[dict[str, Any]] | None = None       # per sample: inputs, output, feedback

    def __post_init__(self) -> None:
        assert self.traces is None or len(self.traces) == len(self.scores)


class GEPAAdapter(Protocol):
    async def evaluate(self, batch: Sequence[dict], candidate: Candidate, capture_traces: bool = False) -> EvaluationBatch: ...
    def make_reflective_dataset(self, candidate: Candidate, eval_batch: EvaluationBatch, components: list[str]) -> dict[str, list[dict]]: ...


@dataclass(frozen=True)
class GEPAConfig:
    max_evaluations: int = 500
    minibatch_size: int = 4
    perfect_score: float = 1.0
    seed: int = 0

    def __post_init__(self) -> None:
        assert self.max_evaluations > 0 and self.minibatch_size > 0 and 0.0 <= self.perfect_score <= 1.0


@dataclass
class GEPAState:
    candidates: list[Candidate]
    val_scores: list[dict[int, float]]                # per candidate: validation sample -> score
    pareto_front: dict[int, set[int]] = field(default_factory=dict)   # validation sample -> best candidates
    total_evaluations: int = 0
    iteration: int = 0
    component_cursor: int = 0
    rng: random.Random = field(default_factory=lambda: random.Random(0))

    def next_component(self) -> str:
        names = sorted(self.candidates[0])
        name = names[self.component_cursor % len(names)]
        self.component_cursor += 1
        return name

    def mean_score(self, idx: int) -> float:
        s = self.val_scores[idx]
        return sum(s.values()) / len(s) if s else 0.0

    def best(self) -> int:
        return max(range(len(self.candidates)), key=self.mean_score)


@dataclass(frozen=True)
class GEPAResult:
    best_candidate: Candidate
    best_score: float
    total_evaluations: int
    history: tuple[dict[str, Any], ...]


# ------------------------------------------------------------------------------------------ operations
def dominates(a: dict[int, float], b: dict[int, float]) -> bool:
    keys = set(a) & set(b)
    return bool(keys) and all(a[k] >= b[k] for k in keys) and any(a[k] > b[k] for k in keys)


def update_pareto_front(state: GEPAState, new_idx: int) -> None:
    for sample, score in state.val_scores[new_idx].items():
        holders = state.pareto_front.get(sample, set())
        best = max((state.val_scores[h][sample] for h in holders), default=float("-inf"))
        if score > best:
            state.pareto_front[sample] = {new_idx}
        elif score == best:
            holders.add(new_idx)
            state.pareto_front[sample] = holders


def select_from_pareto_front(state: GEPAState) -> int:
    """Sample a non-dominated candidate with probability proportional to the samples it wins."""
    wins: dict[int, int] = {}
    for holders in state.pareto_front.values():
        for h in holders:
            wins[h] = wins.get(h, 0) + 1
    if not wins:
        return 0
    alive = [c for c in wins if not any(dominates(state.val_scores[o], state.val_scores[c]) for o in wins if o != c)] or list(wins)
    return state.rng.choices(alive, weights=[wins[c] for c in alive], k=1)[0]


def sample_minibatch(n_train: int, state: GEPAState, size: int) -> list[int]:
    return state.rng.sample(range(n_train), min(size, n_train))


def format_reflective_examples(examples: list[dict]) -> str:
    parts = []
    for i, ex in enumerate(examples, 1):
        lines = [f"### Example {i}"]
        for key in ("inputs", "output", "expected", "score", "feedback"):
            if key in ex:
                lines.append(f"{key}: {ex[key]}")
        parts.append("\n".join(lines))
    return "\n\n".join(parts)


def extract_instruction_from_response(response: str) -> str:
    """The new text is the last fenced block if there is one, else the whole reply."""
    blocks = re.findall(r"```(?:[a-zA-Z]*)\n(.*?)```", response, re.DOTALL)
    return (blocks[-1] if blocks else response).strip()


Reflect = Callable[[str], Awaitable[str]]      # prompt -> model reply

REFLECTION_PROMPT = """You are improving one part of a prompt used by another model.

Current text of the part "{component}":
```
{current}
```

Below are examples of how the model behaved with this text, with feedback on each.

{examples}

Write an improved version of the part. Keep what works, fix what the feedback points at, stay
general (do not hard-code the examples). Reply with the new text inside one ``` fenced block."""


async def propose_mutation(candidate: Candidate, component: str, examples: list[dict], reflect: Reflect) -> str:
    reply = await reflect(REFLECTION_PROMPT.format(component=component, current=candidate[component],
                                                   examples=format_reflective_examples(examples)))
    new = extract_instruction_from_response(reply)
    return new or candidate[component]


# ------------------------------------------------------------------------------------------ engine
async def gepa_iteration(state: GEPAState, adapter: GEPAAdapter, trainset: Sequence[dict], reflect: Reflect,
                         config: GEPAConfig) -> Candidate | None:
    parent = state.candidates[select_from_pareto_front(state)]
    batch = [trainset[i] for i in sample_minibatch(len(trainset), state, config.minibatch_size)]
    before = await adapter.evaluate(batch, parent, capture_traces=True)
    state.total_evaluations += len(batch)
    if all(s >= config.perfect_score for s in before.scores):
        return None
    component = state.next_component()
    data = adapter.make_reflective_dataset(parent, before, [component]).get(component)
    if not data:
        return None
    child = {**parent, component: await propose_mutation(parent, component, data, reflect)}
    if child == parent:
        return None
    after = await adapter.evaluate(batch, child, capture_traces=False)
    state.total_evaluations += len(batch)
    return child if sum(after.scores) > sum(before.scores) else None


async def run_gepa(seed_candidate: Candidate, adapter: GEPAAdapter, trainset: Sequence[dict], valset: Sequence[dict],
                   reflect: Reflect, config: GEPAConfig = GEPAConfig()) -> GEPAResult:
    state = GEPAState([dict(seed_candidate)], [], rng=random.Random(config.seed))
    first = await adapter.evaluate(valset, seed_candidate)
    state.total_evaluations += len(valset)
    state.val_scores.append(dict(enumerate(first.scores)))
    update_pareto_front(state, 0)
    history: list[dict[str, Any]] = []
    while state.total_evaluations < config.max_evaluations:
        state.iteration += 1
        spent = state.total_evaluations
        child = await gepa_iteration(state, adapter, trainset, reflect, config)
        accepted = child is not None
        if accepted:
            ev = await adapter.evaluate(valset, child)
            state.total_evaluations += len(valset)
            state.candidates.append(child)
            state.val_scores.append(dict(enumerate(ev.scores)))
            update_pareto_front(state, len(state.candidates) - 1)
        history.append({"iteration": state.iteration, "accepted": accepted, "evaluations": state.total_evaluations,
                        "best_score": state.mean_score(state.best()), "num_candidates": len(state.candidates)})
        if state.total_evaluations == spent:       # nothing was evaluated (all perfect): the budget cannot advance
            break
    b = state.best()
    return GEPAResult(state.candidates[b], state.mean_score(b), state.total_evaluations, tuple(history))


# ------------------------------------------------------------------------------------------ default adapter
@dataclass
class PromptAdapter:
    """Evaluates a ``{"system", "user_template"}`` candidate with ``generate(system, user) -> text`` and
    ``score(sample, text) -> (score, feedback)``."""

    generate: Callable[[str, str], Awaitable[str]]
    score: Callable[[dict, str], tuple[float, str]]

    async def evaluate(self, batch, candidate, capture_traces=False) -> EvaluationBatch:
        scores, outputs, traces = [], [], []
        for sample in batch:
            user = candidate.get("user_template", "{input}").format(**sample)
            text = await self.generate(candidate.get("system", ""), user)
            s, fb = self.score(sample, text)
            scores.append(float(s))
            outputs.append(text)
            traces.append({"inputs": user, "output": text, "expected": sample.get("answer"), "score": s, "feedback": fb})
        return EvaluationBatch(scores, outputs, traces if capture_traces else None)

    def make_reflective_dataset(self, candidate, eval_batch, components) -> dict[str, list[dict]]:
        return {c: list(eval_batch.traces or []) for c in components}


async def optimize_prompt(system: str, user_template: str, generate, score, trainset, valset, reflect,
                          config: GEPAConfig = GEPAConfig()) -> GEPAResult:
    return await run_gepa({"system": system, "user_template": user_template}, PromptAdapter(generate, score), trainset, valset, reflect, config)


# ------------------------------------------------------------------------------------------ evolutionary variant
@dataclass(frozen=True)
class EvolutionaryConfig:
    population_size: int = 8
    generations: int = 5
    elite_fraction: float = 0.25
    tournament_size: int = 3
    crossover_rate: float = 0.5
    seed: int = 0


def select_elites(population: list[Candidate], scores: list[float], fraction: float) -> list[Candidate]:
    k = max(1, int(round(len(population) * fraction)))
    order = sorted(range(len(population)), key=lambda i: scores[i], reverse=True)
    return [population[i] for i in order[:k]]


def tournament_select(population: list[Candidate], scores: list[float], size: int, rng: random.Random) -> Candidate:
    picks = rng.sample(range(len(population)), min(size, len(population)))
    return population[max(picks, key=lambda i: scores[i])]


def crossover_templates(a: str, b: str, rng: random.Random) -> str:
    """Sentence-level uniform crossover."""
    split = lambda t: [s for s in re.split(r"(?<=[.!?])\s+", t.strip()) if s]  # noqa: E731
    sa, sb = split(a), split(b)
    out = [(sa[i] if i < len(sa) and (i >= len(sb) or rng.random() < 0.5) else sb[i]) for i in range(max(len(sa), len(sb)))]
    return " ".join(out)


async def run_evolutionary(seed: Candidate, adapter: GEPAAdapter, dataset: Sequence[dict], reflect: Reflect,
                           config: EvolutionaryConfig = EvolutionaryConfig()) -> GEPAResult:
    rng = random.Random(config.seed)
    population, history, evals = [dict(seed)], [], 0

    async def fitness(c: Candidate) -> tuple[float, EvaluationBatch]:
        ev = await adapter.evaluate(dataset, c, capture_traces=True)
        return sum(ev.scores) / max(len(ev.scores), 1), ev

    scored = [await fitness(seed)]
    evals += len(dataset)
    for gen in range(config.generations):
        scores = [s for s, _ in scored]
        nxt = select_elites(population, scores, config.elite_fraction)
        while len(nxt) < config.population_size:
            parent = tournament_select(population, scores, config.tournament_size, rng)
            child = dict(parent)
            comp = sorted(child)[(gen + len(nxt)) % len(child)]     # every component gets its turn
            if len(population) > 1 and rng.random() < config.crossover_rate:
                other = tournament_select(population, scores, config.tournament_size, rng)
                child[comp] = crossover_templates(parent[comp], other[comp], rng)
            else:
                ev = scored[population.index(parent)][1]
                child[comp] = await propose_mutation(parent, comp, adapter.make_reflective_dataset(parent, ev, [comp])[comp], reflect)
            nxt.append(child)
        population = nxt
        scored = [await fitness(c) for c in population]
        evals += len(dataset) * len(population)
        history.append({"generation": gen + 1, "best_score": max(s for s, _ in scored), "mean_score": sum(s for s, _ in scored) / len(scored)})
    best = max(range(len(population)), key=lambda i: scored[i][0])
    return GEPAResult(population[best], scored[best][0], evals, tuple(history))
