"""Dataset loaders of the agent layer: rows in, first trajectory of an agent run out (rollouts/datasets/: calculator
smoke problems, Lichess puzzles, ScreenSpot GUI grounding).

Nothing is downloaded here (there is no network in the environments this package targets): the Lichess loader reads
the puzzle CSV (optionally ``.zst`` / ``.gz`` compressed) from a cache folder the user has filled, and says where to get
it if it is missing.
"""

from __future__ import annotations

import base64
import csv
import gzip
import io
import json
from pathlib import Path
from typing import Any, Iterator

from .dtypes import ImageContent, Message, TextContent, Trajectory

# ------------------------------------------------------------------------------------------- calculator smoke set
CALC_SYSTEM_PROMPT = ("You are a careful math assistant. Use the calculator tools (add, subtract, multiply, divide) for every "
                      "computation, then state the final number.")


def load_calc_smoke(data_path: str | Path) -> list[dict[str, Any]]:
    """``problems.jsonl`` of a folder (or the file itself): one ``{"question", "answer"}`` object per line."""
    p = Path(data_path)
    f = p / "problems.jsonl" if p.is_dir() else p
    if not f.is_file():
        raise FileNotFoundError(f"no calculator problems at {f}")
    rows = [json.loads(line) for line in f.read_text().splitlines() if line.strip()]
    for i, r in enumerate(rows):
        if "question" not in r or "answer" not in r:
            raise ValueError(f"{f}: line {i + 1} needs 'question' and 'answer'")
    if not rows:
        raise ValueError(f"{f} is empty")
    return rows


def builtin_calc_smoke() -> list[dict[str, Any]]:
    """Eight problems that exercise every calculator tool, for dry runs without any file."""
    return [{"question": q, "answer": a} for q, a in (
        ("What is 17 + 25?", 42), ("What is 100 - 37?", 63), ("What is 12 * 12?", 144), ("What is 81 / 9?", 9),
        ("Add 3.5 and 4.25, then multiply the result by 2.", 15.5), ("Subtract 19 from 7.", -12),
        ("What is (8 + 6) * (10 - 7)?", 42), ("Divide 1 by 8, then add 0.875.", 1.0))]


def calc_smoke_to_trajectory(row: dict[str, Any]) -> Trajectory:
    q = row["question"]
    assert isinstance(q, str) and q, "a row needs a non-empty 'question'"
    return Trajectory((Message("system", CALC_SYSTEM_PROMPT), Message("user", q)))


# ------------------------------------------------------------------------------------------- Lichess puzzles
DEFAULT_CACHE_DIR = Path.home() / ".cache" / "research_b200" / "lichess"
PUZZLE_URL = "https://database.lichess.org/lichess_db_puzzle.csv.zst"
TACTICAL_THEMES = ["fork", "pin", "skewer", "discoveredAttack", "doubleCheck", "sacrifice", "deflection", "decoy", "interference",
                   "clearance", "xRayAttack", "zugzwang"]
MATE_THEMES = ["mate", "mateIn1", "mateIn2", "mateIn3", "mateIn4", "mateIn5", "anastasiaMate", "arabianMate", "backRankMate",
               "bodenMate", "doubleBishopMate", "dovetailMate", "hookMate", "smotheredMate"]


def _int(v: str | None) -> int | None:
    return int(v) if v not in (None, "") else None


def parse_puzzle_row(row: dict[str, str]) -> dict[str, Any]:
    """One CSV row. ``FEN`` is the position BEFORE the opponent's last move; ``Moves`` starts with that move, the rest
    is the solution (the solver's and the opponent's moves alternating)."""
    moves = (row.get("Moves") or "").split()
    return {"id": row["PuzzleId"], "fen": row["FEN"], "opponent_move": moves[0] if moves else None, "solution": moves[1:],
            "rating": _int(row.get("Rating")), "rating_deviation": _int(row.get("RatingDeviation")), "popularity": _int(row.get("Popularity")),
            "nb_plays": _int(row.get("NbPlays")), "themes": (row.get("Themes") or "").split(), "game_url": row.get("GameUrl", ""),
            "opening_tags": (row.get("OpeningTags") or "").split()}


def _open_csv(path: Path) -> Iterator[dict[str, str]]:
    if path.suffix == ".gz":
        with gzip.open(path, "rt", newline="") as f:
            yield from csv.DictReader(f)
    elif path.suffix == ".zst":
        try:
            import zstandard
        except ImportError as e:
            raise RuntimeError(f"{path} is zstd-compressed and the zstandard package is not installed: decompress it first "
                               f"(zstd -d {path.name})") from e
        with open(path, "rb") as raw:
            with io.TextIOWrapper(zstandard.ZstdDecompressor().stream_reader(raw), newline="") as f:
                yield from csv.DictReader(f)
    else:
        with open(path, newline="") as f:
            yield from csv.DictReader(f)


def find_puzzle_file(cache_dir: str | Path = DEFAULT_CACHE_DIR) -> Path:
    d = Path(cache_dir)
    for name in ("lichess_db_puzzle.csv", "lichess_db_puzzle.csv.gz", "lichess_db_puzzle.csv.zst"):
        if (d / name).is_file():
            return d / name
    raise FileNotFoundError(f"no Lichess puzzle file in {d}: fetch {PUZZLE_URL} on a machine with network access and put it there")


def load_lichess_puzzles_sync(num_puzzles: int | None = None, min_rating: int | None = None, max_rating: int | None = None,
                              themes: list[str] | None = None, cache_dir: str | Path = DEFAULT_CACHE_DIR,
                              path: str | Path | None = None) -> list[dict[str, Any]]:
    """Puzzles in file order, filtered by rating range and by themes (a puzzle qualifies if it has ANY of them),
    stopping after ``num_puzzles``. The file is streamed, so the multi-million-row database is never held in memory."""
    wanted = set(themes or [])
    out: list[dict[str, Any]] = []
    for row in _open_csv(Path(path) if path is not None else find_puzzle_file(cache_dir)):
        p = parse_puzzle_row(row)
        r = p["rating"]
        if (min_rating is not None and (r is None or r < min_rating)) or (max_rating is not None and (r is None or r > max_rating)):
            continue
        if wanted and not wanted & set(p["themes"]):
            continue
        out.append(p)
        if num_puzzles is not None and len(out) >= num_puzzles:
            break
    return out


async def load_lichess_puzzles(*args: Any, **kw: Any) -> list[dict[str, Any]]:
    """The same from asynchronous code (file reading moved to a worker thread)."""
    import asyncio

    return await asyncio.to_thread(load_lichess_puzzles_sync, *args, **kw)


def get_puzzle_fen_after_opponent_move(puzzle: dict[str, Any]) -> str:
    """The position the solver sees: the stored FEN with the opponent's last move played (this package's own board)."""
    from .environments.chess_puzzle import Board

    board = Board(puzzle["fen"])
    if puzzle.get("opponent_move"):
        move = board.parse_uci(puzzle["opponent_move"])
        assert move is not None, f"puzzle {puzzle.get('id')}: {puzzle['opponent_move']} is not legal in {puzzle['fen']}"
        board.push(move)
    return board.fen()


def puzzle_to_trajectory(puzzle: dict[str, Any]) -> Trajectory:
    fen = get_puzzle_fen_after_opponent_move(puzzle)
    side = "White" if fen.split()[1] == "w" else "Black"
    return Trajectory((Message("system", "You solve chess puzzles. Answer with moves in UCI notation (e2e4, e7e8q)."),
                       Message("user", f"Position (FEN): {fen}\n{side} to move. Find the best move.")))


# ------------------------------------------------------------------------------------------- ScreenSpot
def load_screenspot(data_path: str | Path, annotation_file: str, limit: int | None = None, platforms: list[str] | None = None,
                    applications: list[str] | None = None, ui_types: list[str] | None = None) -> list[dict[str, Any]]:
    """Samples of ``<data_path>/annotations/<annotation_file>`` (a JSON list) filtered by platform / application / UI
    type, each with ``image_path`` under ``<data_path>/images``."""
    root = Path(data_path)
    ann = root / "annotations" / annotation_file
    if not ann.is_file():
        raise FileNotFoundError(f"annotation file not found: {ann}")
    samples = json.loads(ann.read_text())
    if not isinstance(samples, list) or not samples:
        raise ValueError(f"{ann} holds no samples")
    if platforms is not None:
        samples = [s for s in samples if s.get("platform") in platforms]
    if applications:
        samples = [s for s in samples if s.get("application") in applications]
    if ui_types is not None:
        samples = [s for s in samples if s.get("ui_type") in ui_types]
    if limit is not None:
        samples = samples[:limit]
    for s in samples:
        if "img_filename" not in s:
            raise ValueError(f"{ann}: a sample has no 'img_filename'")
        s["image_path"] = str(root / "images" / s["img_filename"])
    return samples


def screenspot_to_trajectory(row: dict[str, Any], inline_image: bool = True) -> Trajectory:
    """Instruction + screenshot. The image travels inline (base64) when the file exists and ``inline_image``; otherwise
    the message only names it (dry runs without the image set)."""
    text = (f"Instruction: {row['instruction']}\nAnswer with the click position as [[x, y]] or the element's box as "
            "[[x0, y0, x1, y1]], in coordinates between 0 and 1.")
    blocks: list[Any] = [TextContent(text)]
    p = Path(row.get("image_path", ""))
    if inline_image and p.is_file():
        mime = "image/jpeg" if p.suffix.lower() in (".jpg", ".jpeg") else "image/png"
        blocks.append(ImageContent(base64.b64encode(p.read_bytes()).decode(), mime))
    else:
        blocks[0] = TextContent(text + f"\n(screenshot: {p.name or 'not available'})")
    return Trajectory((Message("system", "You locate user-interface elements in screenshots."), Message("user", blocks)))
