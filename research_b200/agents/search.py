"""Tree search over agent states: expand, score, select, prune (rollouts/search.py:51-411)."""

from __future__ import annotations

import asyncio
import math
import random
from dataclasses import dataclass, field, replace
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


# ------------------------------------------------------------------------------------------- tree search over agent states
# select -> expand -> prune over a tree of ``AgentState``s (rollouts/search.py:51-461). A step picks frontier nodes
# (``select``), continues each of them for some turns, ``branch_factor`` times independently (``expand``), scores the new
# states (``value_fn``) and trims the frontier (``prune``). Beam search = select everything + beam pruner; best-first =
# select the best; Monte-Carlo tree search = UCB selection (values are backed up along the path, visits counted).
@dataclass
class TreeNode:
    state: Any                                  # AgentState
    node_id: str = "0"                          # path from the root: "0.2.1" is child 1 of child 2 of the root
    parent_id: str | None = None
    depth: int = 0
    value: float | None = None                  # value_fn of this node's state
    visits: int = 0
    total: float = 0.0                          # sum of values backed up through this node
    children: list[str] = field(default_factory=list)
    pruned: bool = False

    @property
    def terminal(self) -> bool:
        return getattr(self.state, "stop", None) is not None

    @property
    def mean(self) -> float:
        return self.total / self.visits if self.visits else (self.value or 0.0)


class SearchTree:
    def __init__(self, root_state: Any):
        self.nodes: dict[str, TreeNode] = {"0": TreeNode(root_state)}
        self.frontier: list[str] = ["0"]

    def __getitem__(self, node_id: str) -> TreeNode:
        return self.nodes[node_id]

    def add_child(self, parent_id: str, state: Any, value: float | None) -> TreeNode:
        parent = self.nodes[parent_id]
        node = TreeNode(state, f"{parent_id}.{len(parent.children)}", parent_id, parent.depth + 1, value)
        parent.children.append(node.node_id)
        self.nodes[node.node_id] = node
        if not node.terminal:
            self.frontier.append(node.node_id)
        if value is not None:                    # back the estimate up to the root
            at: TreeNode | None = node
            while at is not None:
                at.visits += 1
                at.total += value
                at = self.nodes[at.parent_id] if at.parent_id is not None else None
        return node

    def frontier_nodes(self) -> list[TreeNode]:
        return [self.nodes[i] for i in self.frontier]

    def terminal_nodes(self) -> list[TreeNode]:
        return [n for n in self.nodes.values() if n.terminal]

    def best_terminal(self) -> TreeNode | None:
        return max(self.terminal_nodes(), key=lambda n: (n.value if n.value is not None else -math.inf), default=None)

    def best_node(self) -> TreeNode:
        """The best terminal node if any, else the best-valued node reached."""
        return self.best_terminal() or max(self.nodes.values(), key=lambda n: (n.value if n.value is not None else -math.inf, n.depth))

    def path_to(self, node_id: str) -> list[TreeNode]:
        out = []
        at: str | None = node_id
        while at is not None:
            out.append(self.nodes[at])
            at = self.nodes[at].parent_id
        return out[::-1]

    def keep(self, node_ids: list[str]) -> None:
        """Restrict the frontier to ``node_ids``; what leaves it is marked pruned (and stays in the tree for inspection)."""
        kept = set(node_ids)
        for i in self.frontier:
            if i not in kept:
                self.nodes[i].pruned = True
        self.frontier = [i for i in self.frontier if i in kept]


SelectFn = Callable[[SearchTree], list[str]]
PruneFn = Callable[[SearchTree], None]
ValueFn = Callable[[Any], Awaitable[float]]


def _val(n: TreeNode) -> float:
    return n.value if n.value is not None else 0.0


def select_all_frontier(tree: SearchTree) -> list[str]:
    return list(tree.frontier)


def select_one_best(tree: SearchTree) -> list[str]:
    return [max(tree.frontier_nodes(), key=_val).node_id] if tree.frontier else []


def select_one_deepest(tree: SearchTree) -> list[str]:
    return [max(tree.frontier_nodes(), key=lambda n: (n.depth, _val(n))).node_id] if tree.frontier else []


def make_random_selector(seed: int | None = None) -> SelectFn:
    rng = random.Random(seed)
    return lambda tree: [rng.choice(tree.frontier)] if tree.frontier else []


def make_ucb_selector(c: float = 1.414) -> SelectFn:
    """One frontier node by upper confidence bound: mean backed-up value + c * sqrt(ln(N) / n), an unvisited node first."""
    def select(tree: SearchTree) -> list[str]:
        if not tree.frontier:
            return []
        total = sum(n.visits for n in tree.frontier_nodes()) + 1

        def ucb(n: TreeNode) -> float:
            return math.inf if n.visits == 0 else n.mean + c * math.sqrt(math.log(total) / n.visits)

        return [max(tree.frontier_nodes(), key=ucb).node_id]

    return select


def make_beam_pruner(beam_width: int) -> PruneFn:
    return lambda tree: tree.keep([n.node_id for n in sorted(tree.frontier_nodes(), key=_val, reverse=True)[:beam_width]])


def make_threshold_pruner(min_value: float) -> PruneFn:
    return lambda tree: tree.keep([n.node_id for n in tree.frontier_nodes() if n.value is None or n.value >= min_value])


def make_depth_pruner(max_depth: int) -> PruneFn:
    return lambda tree: tree.keep([n.node_id for n in tree.frontier_nodes() if n.depth < max_depth])


def compose_pruners(*pruners: PruneFn) -> PruneFn:
    def prune_all(tree: SearchTree) -> None:
        for p in pruners:
            p(tree)

    return prune_all


async def _fork(state: Any) -> Any:
    env = getattr(state, "environment", None)
    if env is None:
        return state
    return replace(state, environment=await type(env).deserialize(await env.serialize()))


def make_expand_n_turns(n: int = 1, branch_factor: int = 1, parallel: bool = True, keep_expanded: bool = False):
    """An expander: every selected node is continued ``branch_factor`` times, each continuation on its own copy of the
    environment for up to ``n`` agent turns (sampling makes them differ), and each result becomes a child. An expanded
    node leaves the frontier unless ``keep_expanded`` (MCTS revisits nodes)."""
    async def one(state: Any, run_config: Any, value_fn: ValueFn | None) -> tuple[Any, float | None]:
        from .agents import run_agent_step

        state = await _fork(state)
        for _ in range(n):
            state = await run_agent_step(state, run_config)
            if state.stop is not None:
                break
        return state, (await value_fn(state) if value_fn is not None else None)

    async def expand(tree: SearchTree, node_ids: list[str], run_config: Any, value_fn: ValueFn | None = None) -> None:
        jobs = [(i, one(tree[i].state, run_config, value_fn)) for i in node_ids for _ in range(branch_factor)]
        if parallel:
            results = await asyncio.gather(*[j for _, j in jobs])
        else:
            results = [await j for _, j in jobs]
        for (parent_id, _), (state, value) in zip(jobs, results):
            tree.add_child(parent_id, state, value)
        if not keep_expanded:
            tree.frontier = [i for i in tree.frontier if i not in set(node_ids)]

    return expand


async def run_tree_search(initial_state: Any, run_config: Any, select: SelectFn = select_all_frontier, expand=None,
                          value_fn: ValueFn | None = None, prune: PruneFn | None = None, max_steps: int = 100,
                          stop_on_terminal: bool = True) -> SearchTree:
    """select -> expand -> prune until a terminal state appears (``stop_on_terminal``), the frontier empties, or
    ``max_steps`` iterations have run. The whole tree comes back: ``best_node()``, ``path_to(id)``, pruned flags."""
    tree = SearchTree(initial_state)
    expand = expand or make_expand_n_turns()
    for _ in range(max_steps):
        ids = select(tree)
        if not ids:
            break
        await expand(tree, ids, run_config, value_fn)
        if stop_on_terminal and tree.terminal_nodes():
            break
        if prune is not None:
            prune(tree)
        if not tree.frontier:
            break
    return tree
