"""Bridge from agent runs to training samples (rollouts/training/agent_integration.py:74-700).

``trajectory_to_sample`` builds tokens + loss mask. With stored ``Choice.token_ids`` the sample
uses exactly the tokens the engine produced and consumed (prompt ids of the last completion +
its completion ids, assistant segments masked in, everything else masked out); without them
the conversation is tokenised with the chat template and assistant spans are located by
prefix tokenisation. ``trajectory_to_samples`` with ``strategy="branching"`` emits one sample
per assistant turn (each with its own prompt), ``"interleaved"`` one sample for the episode.
"""

from __future__ import annotations

import asyncio
from typing import Any, Callable

from ..agents.agents import run_agent
from ..agents.dtypes import Actor, AgentState, Endpoint, Message, RunConfig, Trajectory
from .types import Sample, Status


def _content_to_str(content: Any) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    return "".join(getattr(b, "text", "") for b in content)


def _extract_tokens_from_trajectory(traj: Trajectory) -> tuple[list[int], list[float], list[float]] | None:
    """Tokens, loss mask and rollout log-probs from stored engine ids (None if any turn lacks them)."""
    chs = [c.choices[0] for c in traj.completions if c.choices]
    if not chs or any(ch.token_ids is None or ch.prompt_token_ids is None for ch in chs):
        return None
    tokens: list[int] = []
    mask: list[float] = []
    lps: list[float] = []
    for ch in chs:
        prompt = list(ch.prompt_token_ids)
        # the new part of this turn's prompt (tool results, user turns) is context, not trained on
        if len(prompt) >= len(tokens) and prompt[:len(tokens)] == tokens:
            new = prompt[len(tokens):]
        else:  # the engine saw a different prefix (e.g. truncated history): restart from its prompt
            tokens, mask, lps, new = [], [], [], prompt   # the discarded turns' log-probs go with their tokens
        tokens += new
        mask += [0.0] * len(new)
        tokens += list(ch.token_ids)
        mask += [1.0] * len(ch.token_ids)
        lps += [lp.logprob for lp in ch.logprobs.content] if ch.logprobs else [0.0] * len(ch.token_ids)
    return tokens, mask, lps


def _compute_loss_mask(messages: list[Message], tokenizer: Any) -> tuple[list[int], list[float]]:
    """Chat-template tokenisation with assistant spans found by tokenising growing prefixes."""
    dicts = [{"role": m.role, "content": _content_to_str(m.content)} for m in messages]
    tokens: list[int] = []
    mask: list[float] = []
    for i, m in enumerate(dicts):
        upto = list(tokenizer.apply_chat_template(dicts[:i + 1], tokenize=True, add_generation_prompt=False))
        new = upto[len(tokens):] if upto[:len(tokens)] == tokens else upto
        if upto[:len(tokens)] != tokens:
            tokens, mask = [], []
        tokens += new
        mask += [1.0 if m["role"] == "assistant" else 0.0] * len(new)
    return tokens, mask


def trajectory_to_sample(traj: Trajectory, tokenizer: Any = None, reward: float | None = None, **fields: Any) -> Sample:
    got = _extract_tokens_from_trajectory(traj)
    if got is not None:
        tokens, mask, lps = got
    else:
        assert tokenizer is not None, "a tokenizer is required when the trajectory carries no token ids"
        tokens, mask = _compute_loss_mask(list(traj.messages), tokenizer)
        lps = None
    wv = next((c.weight_version for c in reversed(traj.completions) if c.weight_version is not None), 0)
    return Sample(trajectory=traj, tokens=tokens, loss_mask=mask, response_length=int(sum(mask)),
                  rollout_log_probs=lps, reward=traj.rewards if reward is None else reward, status=Status.COMPLETED,
                  weight_version=wv or 0, **fields)


def _branching_trajectory_to_samples(traj: Trajectory, reward: float | None = None, **fields: Any) -> list[Sample]:
    out = []
    for c in traj.completions:
        ch = c.choices[0]
        if ch.token_ids is None or ch.prompt_token_ids is None:
            continue
        p, t = list(ch.prompt_token_ids), list(ch.token_ids)
        out.append(Sample(trajectory=traj, tokens=p + t, loss_mask=[0.0] * len(p) + [1.0] * len(t), response_length=len(t),
                          rollout_log_probs=[lp.logprob for lp in ch.logprobs.content] if ch.logprobs else None,
                          reward=traj.rewards if reward is None else reward, status=Status.COMPLETED,
                          weight_version=c.weight_version or 0, **fields))
    return out


def trajectory_to_samples(traj: Trajectory, tokenizer: Any = None, strategy: str = "interleaved", reward: float | None = None,
                          **fields: Any) -> list[Sample]:
    if strategy == "branching":
        got = _branching_trajectory_to_samples(traj, reward, **fields)
        if got:
            return got
    return [trajectory_to_sample(traj, tokenizer, reward, **fields)]


async def agent_rollout_to_sample(prompt: Any, endpoint: Endpoint, environment_factory: Callable[[], Any] | None,
                                  run_config: RunConfig, max_turns: int = 1, tokenizer: Any = None,
                                  strategy: str = "interleaved") -> list[Sample]:
    msgs = [Message(**m) if isinstance(m, dict) else m for m in prompt] if isinstance(prompt, list) else [Message("user", str(prompt))]
    env = environment_factory() if environment_factory else None
    state = AgentState(Actor(Trajectory(tuple(msgs)), endpoint), env, max_turns=max_turns)
    final = (await run_agent(state, run_config))[-1]
    samples = trajectory_to_samples(final.actor.trajectory, tokenizer or run_config.tokenizer, strategy, prompt=prompt)
    for s in samples:
        s.metadata["stop_reason"] = final.stop.value if final.stop else None
    return samples


async def generate_rollout_batch(prompts: list[Any], endpoint: Endpoint, environment_factory, run_config: RunConfig,
                                 max_turns: int = 1, max_concurrent: int = 32, **kw: Any) -> list[Sample]:
    sem = asyncio.Semaphore(max_concurrent)

    async def one(p):
        async with sem:
            return await agent_rollout_to_sample(p, endpoint, environment_factory, run_config, max_turns, **kw)

    groups = await asyncio.gather(*[one(p) for p in prompts])
    if kw.get("strategy", "interleaved") != "branching":
        return [s for g in groups for s in g[:1]]
    # branching: one sample per assistant turn, all trained on; each remembers which prompt it came from so that the
    # rollout manager gives the whole branch set its prompt's group
    out = []
    for i, g in enumerate(groups):
        for s in g:
            s.metadata["source_prompt"] = i
            out.append(s)
    return out


def make_agent_generate_fn(engine, environment_cls, config, tokenizer):
    """``generate_fn`` for the GRPO driver that runs the agent loop against the native engine."""
    endpoint = Endpoint(provider="native", engine=engine, max_tokens=config.max_tokens, temperature=config.temperature)
    run_config = RunConfig(use_tito=True, tokenizer=tokenizer)

    async def generate(prompts: list[Any], **kw) -> list[Sample]:
        return await generate_rollout_batch(prompts, endpoint, environment_cls, run_config, config.max_turns,
                                            tokenizer=tokenizer, strategy=config.trajectory_strategy)

    return generate
