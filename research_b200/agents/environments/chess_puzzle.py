"""Chess puzzle environment with a self-contained rules engine.

Tools ``make_move`` (play a move on the board) and ``submit_answer`` (final answer, ends the episode)
as in rollouts/environments/chess_puzzle.py:42-377. The reference leans on python-chess and an
optional Stockfish process; neither exists here, so ``Board`` below implements FEN, legal move
generation (castling, en passant, promotion, check / mate / stalemate) and UCI / SAN parsing, and the
optional position value is a material count instead of an engine evaluation.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..dtypes import AgentState, RunConfig, StopReason, Tool, ToolCall, ToolFunction, ToolFunctionParameter, ToolResult

FILES = "abcdefgh"
START_FEN = "rnbqkbnr/pppppppp/8/8/8/8/PPPPPPPP/RNBQKBNR w KQkq - 0 1"
_KNIGHT = [(1, 2), (2, 1), (2, -1), (1, -2), (-1, -2), (-2, -1), (-2, 1), (-1, 2)]
_KING = [(1, 0), (1, 1), (0, 1), (-1, 1), (-1, 0), (-1, -1), (0, -1), (1, -1)]
_ROOK, _BISHOP = _KING[0::2], _KING[1::2]
_VALUE = {"p": 1, "n": 3, "b": 3, "r": 5, "q": 9, "k": 0}


def sq(name: str) -> tuple[int, int]:
    return FILES.index(name[0]), int(name[1]) - 1


def sq_name(f: int, r: int) -> str:
    return f"{FILES[f]}{r + 1}"


@dataclass(frozen=True)
class Move:
    src: tuple[int, int]
    dst: tuple[int, int]
    promo: str = ""

    def uci(self) -> str:
        return sq_name(*self.src) + sq_name(*self.dst) + self.promo


class Board:
    def __init__(self, fen: str = START_FEN):
        parts = fen.split()
        assert len(parts) >= 4, f"bad FEN: {fen!r}"
        self.grid: list[list[str]] = [["" for _ in range(8)] for _ in range(8)]   # grid[file][rank]
        for ri, row in enumerate(parts[0].split("/")):
            f = 0
            for ch in row:
                if ch.isdigit():
                    f += int(ch)
                else:
                    self.grid[f][7 - ri] = ch
                    f += 1
        self.white = parts[1] == "w"
        self.castling = "" if parts[2] == "-" else parts[2]
        self.ep: tuple[int, int] | None = None if parts[3] == "-" else sq(parts[3])
        self.halfmove = int(parts[4]) if len(parts) > 4 else 0
        self.fullmove = int(parts[5]) if len(parts) > 5 else 1

    # ------------------------------------------------------------------ representation
    def fen(self) -> str:
        rows = []
        for r in range(7, -1, -1):
            row, gap = "", 0
            for f in range(8):
                p = self.grid[f][r]
                if p:
                    row += (str(gap) if gap else "") + p
                    gap = 0
                else:
                    gap += 1
            rows.append(row + (str(gap) if gap else ""))
        ep = sq_name(*self.ep) if self.ep else "-"
        return f"{'/'.join(rows)} {'w' if self.white else 'b'} {self.castling or '-'} {ep} {self.halfmove} {self.fullmove}"

    def ascii(self) -> str:
        lines = [f"{r + 1} " + " ".join(self.grid[f][r] or "." for f in range(8)) for r in range(7, -1, -1)]
        return "\n".join(lines + ["  a b c d e f g h"])

    def copy(self) -> "Board":
        b = Board.__new__(Board)
        b.grid = [col[:] for col in self.grid]
        b.white, b.castling, b.ep, b.halfmove, b.fullmove = self.white, self.castling, self.ep, self.halfmove, self.fullmove
        return b

    # ------------------------------------------------------------------ attacks and moves
    @staticmethod
    def _on(f: int, r: int) -> bool:
        return 0 <= f < 8 and 0 <= r < 8

    def _mine(self, p: str, white: bool) -> bool:
        return bool(p) and p.isupper() == white

    def attacked(self, f: int, r: int, by_white: bool) -> bool:
        g = self.grid
        pr = r - 1 if by_white else r + 1     # rank an attacking pawn stands on
        for df in (-1, 1):
            if self._on(f + df, pr) and g[f + df][pr] == ("P" if by_white else "p"):
                return True
        for df, dr in _KNIGHT:
            if self._on(f + df, r + dr) and g[f + df][r + dr] == ("N" if by_white else "n"):
                return True
        for df, dr in _KING:
            if self._on(f + df, r + dr) and g[f + df][r + dr] == ("K" if by_white else "k"):
                return True
        for dirs, pieces in ((_ROOK, "rq"), (_BISHOP, "bq")):
            for df, dr in dirs:
                x, y = f + df, r + dr
                while self._on(x, y):
                    p = g[x][y]
                    if p:
                        if self._mine(p, by_white) and p.lower() in pieces:
                            return True
                        break
                    x, y = x + df, y + dr
        return False

    def king(self, white: bool) -> tuple[int, int] | None:
        k = "K" if white else "k"
        for f in range(8):
            for r in range(8):
                if self.grid[f][r] == k:
                    return f, r
        return None

    def in_check(self, white: bool | None = None) -> bool:
        white = self.white if white is None else white
        k = self.king(white)
        return k is not None and self.attacked(k[0], k[1], not white)

    def _pseudo(self) -> list[Move]:
        g, w, out = self.grid, self.white, []
        for f in range(8):
            for r in range(8):
                p = g[f][r]
                if not self._mine(p, w):
                    continue
                kind = p.lower()
                if kind == "p":
                    d, start, last = (1, 1, 7) if w else (-1, 6, 0)
                    def add(dst):
                        if dst[1] == last:
                            out.extend(Move((f, r), dst, x) for x in "qrbn")
                        else:
                            out.append(Move((f, r), dst))
                    if self._on(f, r + d) and not g[f][r + d]:
                        add((f, r + d))
                        if r == start and not g[f][r + 2 * d]:
                            out.append(Move((f, r), (f, r + 2 * d)))
                    for df in (-1, 1):
                        x, y = f + df, r + d
                        if self._on(x, y) and ((g[x][y] and not self._mine(g[x][y], w)) or self.ep == (x, y)):
                            add((x, y))
                elif kind in "nk":
                    for df, dr in (_KNIGHT if kind == "n" else _KING):
                        x, y = f + df, r + dr
                        if self._on(x, y) and not self._mine(g[x][y], w):
                            out.append(Move((f, r), (x, y)))
                    if kind == "k" and not self.attacked(f, r, not w):
                        rank = 0 if w else 7
                        if (f, r) == (4, rank):
                            if ("K" if w else "k") in self.castling and not g[5][rank] and not g[6][rank] \
                                    and not self.attacked(5, rank, not w):
                                out.append(Move((4, rank), (6, rank)))
                            if ("Q" if w else "q") in self.castling and not g[3][rank] and not g[2][rank] \
                                    and not g[1][rank] and not self.attacked(3, rank, not w):
                                out.append(Move((4, rank), (2, rank)))
                else:
                    dirs = _ROOK if kind == "r" else _BISHOP if kind == "b" else _KING
                    for df, dr in dirs:
                        x, y = f + df, r + dr
                        while self._on(x, y):
                            if self._mine(g[x][y], w):
                                break
                            out.append(Move((f, r), (x, y)))
                            if g[x][y]:
                                break
                            x, y = x + df, y + dr
        return out

    def push(self, m: Move) -> None:
        g, w = self.grid, self.white
        p = g[m.src[0]][m.src[1]]
        capture = bool(g[m.dst[0]][m.dst[1]])
        if p.lower() == "p" and self.ep == m.dst and not capture:   # en passant
            g[m.dst[0]][m.src[1]] = ""
            capture = True
        g[m.src[0]][m.src[1]] = ""
        g[m.dst[0]][m.dst[1]] = (m.promo.upper() if w else m.promo) if m.promo else p
        if p.lower() == "k" and abs(m.dst[0] - m.src[0]) == 2:       # castling: move the rook too
            rank = m.src[1]
            rf, rt = (7, 5) if m.dst[0] == 6 else (0, 3)
            g[rt][rank], g[rf][rank] = g[rf][rank], ""
        self.ep = (m.src[0], (m.src[1] + m.dst[1]) // 2) if p.lower() == "p" and abs(m.dst[1] - m.src[1]) == 2 else None
        lost = ""
        if p == "K": lost += "KQ"
        if p == "k": lost += "kq"
        for corner, flag in (((0, 0), "Q"), ((7, 0), "K"), ((0, 7), "q"), ((7, 7), "k")):
            if m.src == corner or m.dst == corner:
                lost += flag
        self.castling = "".join(c for c in self.castling if c not in lost)
        self.halfmove = 0 if capture or p.lower() == "p" else self.halfmove + 1
        if not w:
            self.fullmove += 1
        self.white = not w

    def legal_moves(self) -> list[Move]:
        out = []
        for m in self._pseudo():
            b = self.copy()
            b.push(m)
            if not b.in_check(self.white):
                out.append(m)
        return out

    def is_checkmate(self) -> bool:
        return self.in_check() and not self.legal_moves()

    def is_stalemate(self) -> bool:
        return not self.in_check() and not self.legal_moves()

    def material(self) -> int:
        """White minus black material in pawns."""
        return sum((_VALUE[p.lower()] if p.isupper() else -_VALUE[p.lower()]) for col in self.grid for p in col if p)

    # ------------------------------------------------------------------ notation
    def parse_uci(self, text: str) -> Move | None:
        t = text.strip().lower()
        if len(t) not in (4, 5) or t[0] not in FILES or t[2] not in FILES or not t[1].isdigit() or not t[3].isdigit():
            return None
        m = Move(sq(t[:2]), sq(t[2:4]), t[4:] if len(t) == 5 else "")
        return m if m in self.legal_moves() else None

    def parse_san(self, text: str) -> Move | None:
        t = text.strip().rstrip("+#!?").replace("x", "").replace("0", "O")
        legal = self.legal_moves()
        if t in ("O-O", "O-O-O"):
            df = 2 if t == "O-O" else -2
            return next((m for m in legal if self.grid[m.src[0]][m.src[1]].lower() == "k" and m.dst[0] - m.src[0] == df), None)
        promo = ""
        if "=" in t:
            t, promo = t.split("=")[0], t.split("=")[1][:1].lower()
        if len(t) < 2 or t[-2] not in FILES or not t[-1].isdigit():
            return None
        dst, kind, hint = sq(t[-2:]), "p", t[:-2]
        if hint and hint[0] in "NBRQK":
            kind, hint = hint[0].lower(), hint[1:]
        cands = [m for m in legal if m.dst == dst and self.grid[m.src[0]][m.src[1]].lower() == kind and m.promo == promo
                 and all((c in FILES and FILES[m.src[0]] == c) or (c.isdigit() and m.src[1] == int(c) - 1) for c in hint)]
        return cands[0] if len(cands) == 1 else None

    def parse(self, text: str) -> Move | None:
        return self.parse_uci(text) or self.parse_san(text)


def _tool(name: str, desc: str, props: dict[str, Any], required: tuple[str, ...]) -> Tool:
    return Tool(ToolFunction(name, desc, ToolFunctionParameter(props, required)))


@dataclass
class ChessPuzzleEnvironment:
    fen: str
    solution: list[str] = field(default_factory=list)      # accepted first moves, UCI or SAN
    moves_made: list[str] = field(default_factory=list)
    submitted_answer: str | None = None
    render_mode: str = "ascii"                              # ascii | fen | both
    board: Board | None = field(default=None, repr=False)

    def __post_init__(self) -> None:
        if self.board is None:
            self.board = Board(self.fen)
            for mv in self.moves_made:
                m = self.board.parse_uci(mv)
                assert m is not None, f"stored move {mv!r} is not legal"
                self.board.push(m)

    def get_tools(self) -> list[Tool]:
        return [
            _tool("make_move", "Play a move on the board (UCI like e2e4, or SAN like Nf3).", {"move": {"type": "string"}}, ("move",)),
            _tool("submit_answer", "Submit the puzzle's solution move; ends the episode.", {"move": {"type": "string"}}, ("move",)),
        ]

    def requires_confirmation(self, tool_call: ToolCall) -> bool:
        return False

    def render(self) -> str:
        side = "White" if self.board.white else "Black"
        parts = []
        if self.render_mode in ("ascii", "both"):
            parts.append(self.board.ascii())
        if self.render_mode in ("fen", "both"):
            parts.append(self.board.fen())
        return "\n".join(parts) + f"\n{side} to move"

    def check_solution(self, move_str: str) -> bool:
        start = Board(self.fen)
        move = start.parse(move_str)
        return move is not None and any(start.parse(s) == move for s in self.solution)

    async def get_value(self) -> float:
        """Position value in [0, 1] for the side that was to move in the puzzle (material only)."""
        sign = 1 if Board(self.fen).white else -1
        return max(0.0, min(1.0, 0.5 + sign * self.board.material() / 20.0))

    async def exec_tool(self, tool_call: ToolCall, state: AgentState, run_config: RunConfig) -> ToolResult:
        move_str = str(tool_call.args.get("move", ""))
        if tool_call.name == "make_move":
            move = self.board.parse(move_str)
            if move is None:
                legal = ", ".join(sorted(m.uci() for m in self.board.legal_moves())[:40])
                return ToolResult(tool_call.id, is_error=True, error=f"illegal or unreadable move {move_str!r}. Legal: {legal}")
            self.board.push(move)
            self.moves_made.append(move.uci())
            note = " Checkmate." if self.board.is_checkmate() else " Stalemate." if self.board.is_stalemate() \
                else " Check." if self.board.in_check() else ""
            return ToolResult(tool_call.id, content=f"Played {move.uci()}.{note}\n{self.render()}")
        if tool_call.name == "submit_answer":
            self.submitted_answer = move_str
            ok = self.check_solution(move_str)
            return ToolResult(tool_call.id, content="Correct." if ok else "Incorrect.", stop_reason=StopReason.TASK_COMPLETED,
                              metadata={"correct": ok})
        return ToolResult(tool_call.id, is_error=True, error=f"unknown tool {tool_call.name!r}")

    async def serialize(self) -> dict[str, Any]:
        return {"env_kind": "chess_puzzle", "fen": self.fen, "solution": list(self.solution), "moves_made": list(self.moves_made),
                "submitted_answer": self.submitted_answer, "render_mode": self.render_mode}

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "ChessPuzzleEnvironment":
        return ChessPuzzleEnvironment(fen=data["fen"], solution=list(data.get("solution", [])),
                                      moves_made=list(data.get("moves_made", [])), submitted_answer=data.get("submitted_answer"),
                                      render_mode=data.get("render_mode", "ascii"))
