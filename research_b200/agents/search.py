"""Tree search over agent states: expand, score, select, prune (rollouts/search.py:51-411)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Awaitable, Callable


@dataclass(frozen=True)
class SearchNode:
    state: Any
    score: float = 0.0
    depth: int = 0
    parent: "SearchNode | None" = None
    terminal: bool = False
    metadata: dict[str, Any] = field(default_factory=dict)

    def path(self) -> list["SearchNode"]:
        n, out = self, []
        while n is not None:
            out.append(n)
            n = n.parent
        return out[::-1]


def select_best(frontier: list[SearchNode], k: int) -> list[SearchNode]:
    return sorted(frontier, key=lambda n: n.score, reverse=True)[:k]


def prune(frontier: list[SearchNode], min_score: float | None = None, max_size: int | None = None) -> list[SearchNode]:
    out = [n for n in frontier if min_score is None or n.score >= min_score]
    return select_best(out, max_size) if max_size is not None else out


async def run_search(root: Any, expand: Callable[[SearchNode], Awaitable[list[tuple[Any, float, bool]]]], beam_width: int = 4,
                     max_depth: int = 8, min_score: float | None = None) -> SearchNode:
    """Beam search: ``expand(node)`` returns ``(state, score, terminal)`` children."""
    best = SearchNode(root)
    frontier = [best]
    for depth in range(1, max_depth + 1):
        children: list[SearchNode] = []
        for node in frontier:
            if node.terminal:
                continue
            for st, sc, term in await expand(node):
                children.append(SearchNode(st, sc, depth, node, term))
        if not children:
            break
        frontier = prune(children, min_score, beam_width)
        if not frontier:
            break
        top = frontier[0]
        if top.score > best.score or best.depth == 0:
            best = top
        if all(n.terminal for n in frontier):
            break
    return best
