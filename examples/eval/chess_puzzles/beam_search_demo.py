"""Beam search over chess positions with the environment's value function
(rollouts/examples/eval/chess_puzzles/beam_search_demo.py): states are boards, children are legal moves, the score of a
child is 1 for checkmate and otherwise the material balance mapped to (0, 1); finds a mate in two whose defence is forced (the beam maximises at every level; it is not a minimax)."""

import asyncio
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))

from research_b200.agents.environments.chess_puzzle import Board  # noqa: E402
from research_b200.agents.search import run_search  # noqa: E402

MATE_IN_TWO = "7k/8/5K2/8/8/8/8/6R1 w - - 0 1"      # 1. Kf7 Kh7 (forced) 2. Rh1#


def value(board: Board, white_root: bool) -> float:
    sign = 1 if white_root else -1
    return max(0.01, min(0.99, 0.5 + sign * board.material() / 20.0))


async def expand(node):
    board: Board = node.state
    out = []
    for mv in board.legal_moves():
        nxt = board.copy()
        nxt.push(mv)
        mate = nxt.is_checkmate()
        # after our move the opponent is to move: a checkmate there is a win for the root side at odd depth
        ours = node.depth % 2 == 0
        score = (1.0 if ours else 0.0) if mate else value(nxt, True)
        out.append((nxt, score, mate or not nxt.legal_moves()))
    return out


def run(fen: str = MATE_IN_TWO, beam_width: int = 64, max_depth: int = 3):
    best = asyncio.run(run_search(Board(fen), expand, beam_width=beam_width, max_depth=max_depth))
    return best


if __name__ == "__main__":
    node = run()
    print(f"best line reaches score {node.score:.2f} at depth {node.depth}")
    for n in node.path()[1:]:
        print(n.state.fen())
