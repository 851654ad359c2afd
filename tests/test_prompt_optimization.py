"""GEPA with scripted task and reflection models."""

import asyncio
import random

from research_b200.agents.prompt_optimization import (EvolutionaryConfig, GEPAConfig, GEPAState, PromptAdapter, crossover_templates,
                                                      dominates, extract_instruction_from_response, optimize_prompt,
                                                      run_evolutionary, select_from_pareto_front, update_pareto_front)


def test_pareto_bookkeeping():
    st = GEPAState([{"p": "a"}, {"p": "b"}, {"p": "c"}], [{0: 1.0, 1: 0.0}, {0: 0.0, 1: 1.0}, {0: 0.0, 1: 0.0}], rng=random.Random(1))
    for i in range(3):
        update_pareto_front(st, i)
    assert st.pareto_front == {0: {0}, 1: {1}}
    assert dominates(st.val_scores[0], st.val_scores[2]) and not dominates(st.val_scores[0], st.val_scores[1])
    assert {select_from_pareto_front(st) for _ in range(30)} == {0, 1}
    assert extract_instruction_from_response("sure\n```\nnew text\n```\nbye") == "new text"
    assert extract_instruction_from_response("just text") == "just text"
    assert crossover_templates("A one. A two.", "B one. B two. B three.", random.Random(0)).count(".") == 3


def _task():
    # the task model answers in upper case only when the system prompt says so
    async def generate(system, user):
        word = user.split(":")[-1].strip()
        return word.upper() if "upper" in system.lower() else word

    def score(sample, text):
        ok = text == sample["answer"]
        return (1.0 if ok else 0.0), ("correct" if ok else f"expected {sample['answer']!r}: the answer must be in upper case")

    data = [{"input": w, "answer": w.upper()} for w in ("alpha", "beta", "gamma", "delta", "eps", "zeta")]
    return generate, score, data


def test_gepa_improves_prompt():
    generate, score, data = _task()
    prompts = []

    async def reflect(prompt):
        prompts.append(prompt)
        return "Improved:\n```\nAnswer with the word in UPPER case.\n```" if "upper case" in prompt else "```\nno idea\n```"

    res = asyncio.run(optimize_prompt("Repeat the word.", "word: {input}", generate, score, data[:4], data[4:], reflect,
                                      GEPAConfig(max_evaluations=60, minibatch_size=2)))
    assert res.best_score == 1.0 and "UPPER" in res.best_candidate["system"]
    assert res.total_evaluations <= 60 + 4 and any(h["accepted"] for h in res.history)
    assert "expected 'ALPHA'" in "".join(prompts) or "expected" in prompts[0]


def test_evolutionary_variant():
    generate, score, data = _task()

    async def reflect(prompt):
        return "```\nAlways answer in upper case.\n```"

    res = asyncio.run(run_evolutionary({"system": "Repeat the word.", "user_template": "word: {input}"}, PromptAdapter(generate, score),
                                       data, reflect, EvolutionaryConfig(population_size=4, generations=3)))
    assert res.best_score == 1.0 and res.history[-1]["best_score"] == 1.0
