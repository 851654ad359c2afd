"""Chess-puzzle evaluation (rollouts/examples/eval/chess_puzzles/run.py): the model sees the board, may try moves with
``make_move`` and must ``submit_answer``; the score is whether the submitted move is the puzzle's solution. The puzzles
below are mates in one; the scripted model (used when no endpoint is given) finds them by trying every legal move."""

import asyncio
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))

from research_b200.agents.dtypes import Endpoint, EvalConfig, Message, Metric, Score, ToolCall  # noqa: E402
from research_b200.agents.environments.chess_puzzle import Board, ChessPuzzleEnvironment  # noqa: E402
from research_b200.agents.evaluation import evaluate  # noqa: E402
from research_b200.agents.providers import ScriptedLLM, register_provider  # noqa: E402

PUZZLES = [
    {"id": "back_rank", "fen": "6k1/5ppp/8/8/8/8/8/R6K w - - 0 1", "solution": ["a1a8"]},
    {"id": "queen_kiss", "fen": "7k/8/5K2/6Q1/8/8/8/8 w - - 0 1", "solution": ["g5g7"]},
    {"id": "rook_ladder", "fen": "k7/8/1R6/8/8/8/8/2R4K w - - 0 1", "solution": ["c1c8", "c1a1"]},
]


def mate_in_one(fen: str) -> str | None:
    board = Board(fen)
    for mv in board.legal_moves():
        nxt = board.copy()
        nxt.push(mv)
        if nxt.is_checkmate():
            return mv.uci()
    return None


def score_fn(traj, row) -> Score:
    submitted = None
    for m in traj.messages:
        for c in m.tool_calls:
            if c.name == "submit_answer":
                submitted = str(c.args.get("move", ""))
    env = ChessPuzzleEnvironment(row["fen"], list(row["solution"]))
    return Score((Metric("solved", float(submitted is not None and env.check_solution(submitted)), 1.0),
                  Metric("submitted", float(submitted is not None), 0.0)))


def prepare(row) -> list[Message]:
    env = ChessPuzzleEnvironment(row["fen"], list(row["solution"]))
    return [Message("system", "Find the best move. Use make_move to explore and submit_answer to finish."), Message("user", env.render())]


async def brute_force_model(actor, run_config):
    """Stand-in model: reads the position from the conversation's puzzle and submits the mating move."""
    fen = actor.trajectory.metadata.get("fen") or next(p["fen"] for p in PUZZLES
                                                         if ChessPuzzleEnvironment(p["fen"], p["solution"]).render() == actor.trajectory.messages[1].text())
    move = mate_in_one(fen) or "a1a1"
    return await ScriptedLLM([Message("assistant", "This mates.", tool_calls=(ToolCall("c1", "submit_answer", {"move": move}),))])(actor, run_config)


def run(endpoint: Endpoint | None = None, output_dir: str | None = None):
    if endpoint is None:
        register_provider("mock", brute_force_model)
        endpoint = Endpoint(provider="mock")
    cfg = EvalConfig(endpoint=endpoint, score_fn=score_fn, prepare_messages=prepare, max_turns=4, n_retries=0, output_dir=output_dir,
                     environment_factory=lambda row: ChessPuzzleEnvironment(row["fen"], list(row["solution"])), eval_name="chess_puzzles")
    return asyncio.run(evaluate(PUZZLES, cfg))


if __name__ == "__main__":
    report = run(output_dir="results/eval")
    for s in report.samples:
        print(s.sample_id, s.score.reward, s.stop_reason)
    print(report.summary)
