"""Terminal widgets as pure state machines (rollouts/frontends/tui/components/{input,question_selector,markdown}.py,
tui/utils.py): each takes decoded key names and returns what to draw, so all of it is testable without a terminal.

* ``parse_keys``: raw terminal input (escape sequences, control bytes, bracketed paste) -> key names;
* ``LineEditor``: the chat prompt: cursor movement by character / word / line, kill and yank, history with the draft kept,
  multi-line input (alt-enter or a trailing backslash), tab completion of slash commands and paths with a ghost hint;
* ``QuestionSelector``: the ask-the-user dialog: one or several questions, single or multiple choice, a free-text
  "other" answer, tab between questions;
* ``render_markdown``: Markdown -> ANSI lines wrapped to a width (headings, emphasis, inline code, fenced code, lists,
  quotes, rules, links, tables);
* ``read_line_raw``: drives a ``LineEditor`` on a real terminal (raw mode, restored on every exit path).
"""

from __future__ import annotations

import os
import re
import unicodedata
from dataclasses import dataclass, field
from typing import Callable, Sequence

RESET, BOLD, DIM, ITALIC, UNDERLINE, REVERSE = "\x1b[0m", "\x1b[1m", "\x1b[2m", "\x1b[3m", "\x1b[4m", "\x1b[7m"
CYAN, GREEN, YELLOW, BLUE, MAGENTA, GREY = "\x1b[36m", "\x1b[32m", "\x1b[33m", "\x1b[34m", "\x1b[35m", "\x1b[90m"
_ANSI = re.compile(r"\x1b\[[0-9;?]*[A-Za-z]")


# ------------------------------------------------------------------------------------------- text measurement
def visible_width(s: str) -> int:
    """Columns ``s`` takes on screen: escape sequences take none, wide (CJK, emoji) characters two, combining marks none."""
    w = 0
    for ch in _ANSI.sub("", s):
        if unicodedata.combining(ch) or ch in "​‍️":
            continue
        w += 2 if unicodedata.east_asian_width(ch) in ("W", "F") else 1
    return w


def wrap_ansi(text: str, width: int) -> list[str]:
    """Word-wrap one paragraph to ``width`` columns, measuring visible width; a word longer than the width is split.
    Styles that are open at a break are closed at the end of the line and reopened on the next."""
    width = max(width, 4)
    lines, cur, cur_w, active = [], "", 0, ""

    def push() -> None:
        nonlocal cur, cur_w
        lines.append(cur.rstrip() + (RESET if active else ""))
        cur, cur_w = active, 0

    for word in re.split(r"( +)", text):
        if not word:
            continue
        codes = _ANSI.findall(word)
        w = visible_width(word)
        if word.isspace():
            if cur_w and cur_w + w <= width:
                cur, cur_w = cur + word, cur_w + w
            continue
        if cur_w and cur_w + w > width:
            push()
        while w > width:                               # split a long word by characters (escape sequences kept whole)
            piece, pw, i = "", 0, 0
            while i < len(word):
                m = _ANSI.match(word, i)
                if m:
                    piece += m.group()
                    i = m.end()
                    continue
                cw = visible_width(word[i])
                if pw + cw > width - cur_w:
                    break
                piece, pw, i = piece + word[i], pw + cw, i + 1
            cur += piece
            push()
            word, w = word[i:], visible_width(word[i:])
        cur, cur_w = cur + word, cur_w + w
        for c in codes:
            active = "" if c == RESET else active + c
    if cur_w or not lines:
        lines.append(cur.rstrip() + (RESET if active else ""))
    return lines


# ------------------------------------------------------------------------------------------- keys
_CSI = {"A": "up", "B": "down", "C": "right", "D": "left", "H": "home", "F": "end", "Z": "shift-tab",
        "1~": "home", "4~": "end", "7~": "home", "8~": "end", "3~": "delete", "5~": "pageup", "6~": "pagedown",
        "1;5C": "ctrl-right", "1;5D": "ctrl-left", "1;3C": "alt-right", "1;3D": "alt-left", "200~": "paste-start", "201~": "paste-end"}
_CTRL = {0: "ctrl-space", 1: "ctrl-a", 2: "ctrl-b", 3: "ctrl-c", 4: "ctrl-d", 5: "ctrl-e", 6: "ctrl-f", 8: "backspace", 9: "tab", 10: "enter",
         11: "ctrl-k", 12: "ctrl-l", 13: "enter", 14: "ctrl-n", 16: "ctrl-p", 18: "ctrl-r", 20: "ctrl-t", 21: "ctrl-u", 23: "ctrl-w", 25: "ctrl-y",
         127: "backspace"}


def parse_keys(data: str) -> list[str]:
    """Key names for raw input: printable characters as themselves, the rest as names (``up``, ``ctrl-a``, ``alt-enter``,
    ``alt-b``, ``paste-start`` ...). Text between bracketed-paste markers comes back as ONE ``paste:<text>`` key, so a
    pasted newline is text and not a submit."""
    keys, i, n = [], 0, len(data)
    while i < n:
        ch = data[i]
        if ch == "\x1b":
            m = re.match(r"\x1b\[([0-9;]*[A-Za-z~])", data[i:])
            if m:
                name = _CSI.get(m.group(1), f"csi:{m.group(1)}")
                i += m.end()
                if name == "paste-start":
                    end = data.find("\x1b[201~", i)
                    end = n if end < 0 else end
                    keys.append("paste:" + data[i:end].replace("\r\n", "\n").replace("\r", "\n"))
                    i = min(end + 6, n)
                    continue
                keys.append(name)
                continue
            if data.startswith("\x1bO", i) and data[i + 2:i + 3] in ("A", "B", "C", "D", "H", "F"):
                keys.append(_CSI[data[i + 2]])
                i += 3
                continue
            if i + 1 < n:
                nxt = data[i + 1]
                keys.append("alt-enter" if nxt in "\r\n" else "alt-backspace" if nxt in "\x7f\x08" else f"alt-{nxt}")
                i += 2
                continue
            keys.append("escape")
            i += 1
        elif ord(ch) in _CTRL:
            keys.append(_CTRL[ord(ch)])
            i += 1
        elif ord(ch) < 32:
            keys.append(f"ctrl-{chr(ord(ch) + 96)}")
            i += 1
        else:
            keys.append(ch)
            i += 1
    return keys


# ------------------------------------------------------------------------------------------- line editor
Completer = Callable[[str], list[str]]        # text before the cursor -> full replacements for the current token, best first


def make_completer(commands: Sequence[str] = (), cwd: str = ".", hints: dict[str, str] | None = None) -> Completer:
    """Completes ``/comm`` at the start of the line to slash commands, and ``@pa`` / ``./pa`` / ``~/pa`` tokens to paths
    under ``cwd`` (directories get a trailing slash)."""
    def complete(before: str) -> list[str]:
        if before.startswith("/") and " " not in before:
            return sorted("/" + c for c in commands if c.startswith(before[1:]))
        token = before.rsplit(" ", 1)[-1]
        lead = "@" if token.startswith("@") else ""
        path = token[len(lead):]
        if not lead and not path.startswith(("./", "../", "~/", "/")):
            return []
        head, _, tail = path.rpartition("/")
        base = os.path.expanduser(head or ("/" if path.startswith("/") else "."))
        base = base if os.path.isabs(base) else os.path.join(cwd, base)
        try:
            names = sorted(os.listdir(base))
        except OSError:
            return []
        prefix = (head + "/") if head or path.startswith("/") else ""
        return [lead + prefix + n + ("/" if os.path.isdir(os.path.join(base, n)) else "") for n in names
                if n.startswith(tail) and (tail.startswith(".") or not n.startswith("."))]

    complete.hints = hints or {}            # type: ignore[attr-defined]
    return complete


def _common_prefix(items: list[str]) -> str:
    return os.path.commonprefix(items) if items else ""


@dataclass
class LineEditor:
    completer: Completer | None = None
    history: list[str] = field(default_factory=list)
    text: str = ""
    cursor: int = 0
    kill_buffer: str = ""
    candidates: list[str] = field(default_factory=list)     # shown under the prompt after an ambiguous tab
    _hist_at: int | None = None
    _draft: str = ""

    # ---- helpers
    def _set(self, text: str, cursor: int | None = None) -> None:
        self.text, self.cursor = text, len(text) if cursor is None else cursor

    def _word_left(self) -> int:
        i = self.cursor
        while i > 0 and not self.text[i - 1].isalnum():
            i -= 1
        while i > 0 and self.text[i - 1].isalnum():
            i -= 1
        return i

    def _word_right(self) -> int:
        i, n = self.cursor, len(self.text)
        while i < n and not self.text[i].isalnum():
            i += 1
        while i < n and self.text[i].isalnum():
            i += 1
        return i

    def _line_bounds(self) -> tuple[int, int]:
        start = self.text.rfind("\n", 0, self.cursor) + 1
        end = self.text.find("\n", self.cursor)
        return start, len(self.text) if end < 0 else end

    def insert(self, s: str) -> None:
        self._set(self.text[:self.cursor] + s + self.text[self.cursor:], self.cursor + len(s))

    def ghost(self) -> str:
        """Dim text to show after the cursor: the rest of the only completion, or a command's argument hint."""
        if self.completer is None or self.cursor != len(self.text) or not self.text or "\n" in self.text:
            return ""
        hints = getattr(self.completer, "hints", {})
        if self.text.startswith("/") and self.text[1:].rstrip() in hints and self.text.endswith(" ") and self.text.count(" ") == 1:
            return hints[self.text[1:].rstrip()]
        c = self.completer(self.text)
        token = self.text if self.text.startswith("/") and " " not in self.text else self.text.rsplit(" ", 1)[-1]
        return c[0][len(token):] if len(c) == 1 and c[0].startswith(token) else ""

    # ---- keys
    def feed(self, key: str) -> str | None:
        """Apply one key. Returns ``"submit"`` (the text is final: read ``.text``, then call ``accept()``), ``"cancel"``
        (ctrl-c on an empty line or escape), ``"eof"`` (ctrl-d on an empty line) or None (keep editing)."""
        t, c = self.text, self.cursor
        if key != "tab":
            self.candidates = []
        if key.startswith("paste:"):
            self.insert(key[6:])
        elif len(key) == 1:
            self.insert(key)
        elif key == "enter":
            if t.endswith("\\") and c == len(t):                    # a trailing backslash continues on the next line
                self._set(t[:-1] + "\n")
            else:
                return "submit"
        elif key in ("alt-enter", "ctrl-j"):
            self.insert("\n")
        elif key == "backspace":
            if c:
                self._set(t[:c - 1] + t[c:], c - 1)
        elif key == "delete":
            self._set(t[:c] + t[c + 1:], c)
        elif key == "ctrl-d":
            if not t:
                return "eof"
            self._set(t[:c] + t[c + 1:], c)
        elif key == "ctrl-c":
            if not t:
                return "cancel"
            self._set("")
        elif key == "escape":
            return "cancel"
        elif key in ("left", "ctrl-b"):
            self.cursor = max(c - 1, 0)
        elif key in ("right", "ctrl-f"):
            if c == len(t) and self.ghost():
                self.insert(self.ghost())                            # right arrow at the end accepts the ghost text
            else:
                self.cursor = min(c + 1, len(t))
        elif key in ("ctrl-left", "alt-left", "alt-b"):
            self.cursor = self._word_left()
        elif key in ("ctrl-right", "alt-right", "alt-f"):
            self.cursor = self._word_right()
        elif key in ("home", "ctrl-a"):
            self.cursor = self._line_bounds()[0]
        elif key in ("end", "ctrl-e"):
            self.cursor = self._line_bounds()[1]
        elif key == "ctrl-k":
            end = self._line_bounds()[1]
            self.kill_buffer = t[c:end]
            self._set(t[:c] + t[end:], c)
        elif key == "ctrl-u":
            start = self._line_bounds()[0]
            self.kill_buffer = t[start:c]
            self._set(t[:start] + t[c:], start)
        elif key in ("ctrl-w", "alt-backspace"):
            start = self._word_left()
            self.kill_buffer = t[start:c]
            self._set(t[:start] + t[c:], start)
        elif key == "alt-d":
            end = self._word_right()
            self.kill_buffer = t[c:end]
            self._set(t[:c] + t[end:], c)
        elif key == "ctrl-y":
            self.insert(self.kill_buffer)
        elif key == "ctrl-t":
            if 0 < c < len(t):
                self._set(t[:c - 1] + t[c] + t[c - 1] + t[c + 1:], c + 1)
        elif key in ("up", "ctrl-p"):
            start, _ = self._line_bounds()
            if start > 0:                                            # inside a multi-line text: move between its lines
                col = c - start
                prev_start = t.rfind("\n", 0, start - 1) + 1
                self.cursor = min(prev_start + col, start - 1)
            elif self.history:
                if self._hist_at is None:
                    self._draft, self._hist_at = t, len(self.history)
                if self._hist_at > 0:
                    self._hist_at -= 1
                    self._set(self.history[self._hist_at])
        elif key in ("down", "ctrl-n"):
            start, end = self._line_bounds()
            if end < len(t):
                col = c - start
                next_end = t.find("\n", end + 1)
                self.cursor = min(end + 1 + col, len(t) if next_end < 0 else next_end)
            elif self._hist_at is not None:
                self._hist_at += 1
                if self._hist_at >= len(self.history):
                    self._hist_at = None
                    self._set(self._draft)
                else:
                    self._set(self.history[self._hist_at])
        elif key == "tab":
            self._complete()
        return None

    def _complete(self) -> None:
        if self.completer is None:
            return
        before = self.text[:self.cursor]
        token = before if before.startswith("/") and " " not in before else before.rsplit(" ", 1)[-1]
        if len(self.candidates) > 1 and (token in self.candidates or self.completer(before) == self.candidates):
            found = self.candidates                                   # tab again: cycle through what was listed
            grow = found[(found.index(token) + 1) % len(found)] if token in found else found[0]
        else:
            found = self.completer(before)
            if not found:
                return
            grow = found[0] if len(found) == 1 else _common_prefix(found)
            if len(found) == 1 and not grow.endswith("/"):
                grow += " "
        if grow and grow != token:
            self._set(before[:len(before) - len(token)] + grow + self.text[self.cursor:], len(before) - len(token) + len(grow))
        self.candidates = found if len(found) > 1 else []

    def accept(self) -> str:
        """Take the submitted text: it joins the history (consecutive duplicates and blanks do not) and the editor clears."""
        text = self.text
        if text.strip() and (not self.history or self.history[-1] != text):
            self.history.append(text)
        self._set("")
        self._hist_at, self._draft, self.candidates = None, "", []
        return text

    def render(self, prompt: str = "> ", width: int = 80) -> tuple[list[str], tuple[int, int]]:
        """Lines to draw and the cursor's (row, column). Continuation lines are indented to the prompt's width; the ghost
        text is dim; completion candidates follow on one more line."""
        pad = " " * visible_width(prompt)
        before = self.text[:self.cursor]
        rows = self.text.split("\n")
        lines = [(prompt if i == 0 else pad) + r for i, r in enumerate(rows)]
        g = self.ghost()
        if g:
            lines[-1] += f"{DIM}{g}{RESET}"
        if self.candidates:
            shown = "  ".join(self.candidates[:12]) + (f"  (+{len(self.candidates) - 12})" if len(self.candidates) > 12 else "")
            lines.append(f"{DIM}{shown[:max(width - 1, 8)]}{RESET}")
        row = before.count("\n")
        col = visible_width(pad) + visible_width(before.rsplit("\n", 1)[-1])
        return lines, (row, col)


# ------------------------------------------------------------------------------------------- question selector
@dataclass
class Question:
    question: str
    options: list[str]
    header: str = ""
    multi_select: bool = False
    descriptions: list[str] = field(default_factory=list)


class QuestionSelector:
    """One or several questions on one screen. Up / down (or j / k) move, space toggles (multi-select) or picks, a digit
    picks that option, the last row "Other" opens a text field (space or enter on it), tab / shift-tab change question,
    enter confirms the current question and moves on; after the last one the dialog is done. Escape cancels everything."""

    OTHER = "Other (type an answer)"

    def __init__(self, questions: Sequence[Question]):
        assert questions, "at least one question"
        self.questions = list(questions)
        self.at = 0                                     # current question
        self.row = [0] * len(self.questions)            # highlighted row per question
        self.picked: list[set[int]] = [set() for _ in self.questions]
        self.other: list[str] = [""] * len(self.questions)
        self.typing = False
        self.done = self.cancelled = False

    def _n_rows(self, q: int) -> int:
        return len(self.questions[q].options) + 1

    def _pick(self, q: int, r: int) -> None:
        if self.questions[q].multi_select:
            self.picked[q] ^= {r}
        else:
            self.picked[q] = {r}

    def feed(self, key: str) -> None:
        q, n = self.at, self._n_rows(self.at)
        if self.typing:
            if key == "enter":
                self.typing = False
                if self.other[q].strip():
                    self.picked[q] = (self.picked[q] | {n - 1}) if self.questions[q].multi_select else {n - 1}
                    if not self.questions[q].multi_select:
                        self._advance()
                else:
                    self.picked[q].discard(n - 1)
            elif key == "escape":
                self.typing = False
            elif key == "backspace":
                self.other[q] = self.other[q][:-1]
            elif key.startswith("paste:"):
                self.other[q] += key[6:].replace("\n", " ")
            elif len(key) == 1:
                self.other[q] += key
            return
        if key in ("up", "k"):
            self.row[q] = (self.row[q] - 1) % n
        elif key in ("down", "j"):
            self.row[q] = (self.row[q] + 1) % n
        elif key in ("tab", "right"):
            self.at = (q + 1) % len(self.questions)
        elif key in ("shift-tab", "left"):
            self.at = (q - 1) % len(self.questions)
        elif key.isdigit() and 1 <= int(key) <= n:
            self.row[q] = int(key) - 1
            self._activate(q)
        elif key == " ":
            self._activate(q)
        elif key == "enter":
            if self.row[q] == n - 1 and not self.other[q].strip():   # on "Other" with nothing typed yet: open the field
                self.typing = True
                return
            if not self.picked[q]:
                self._activate(q)
                if self.questions[q].multi_select:
                    return
            self._advance()
        elif key in ("escape", "ctrl-c"):
            self.cancelled = self.done = True

    def _activate(self, q: int) -> None:
        r = self.row[q]
        if r == self._n_rows(q) - 1:
            self.typing = True
        else:
            self._pick(q, r)

    def _advance(self) -> None:
        unanswered = [i for i in range(len(self.questions)) if not self.picked[i]]
        if not unanswered:
            self.done = True
        else:
            later = [i for i in unanswered if i > self.at]
            self.at = (later or unanswered)[0]

    def answers(self) -> dict[str, str | list[str]] | None:
        """``{question text: answer}`` (a list for multi-select); None when cancelled."""
        if self.cancelled:
            return None
        out: dict[str, str | list[str]] = {}
        for i, q in enumerate(self.questions):
            vals = [self.other[i].strip() if r == len(q.options) else q.options[r] for r in sorted(self.picked[i])]
            out[q.question] = vals if q.multi_select else (vals[0] if vals else "")
        return out

    def render(self, width: int = 80) -> list[str]:
        lines = []
        if len(self.questions) > 1:
            tabs = []
            for i, q in enumerate(self.questions):
                label = f" {'✓' if self.picked[i] else '·'} {q.header or f'Q{i + 1}'} "
                tabs.append(f"{REVERSE}{label}{RESET}" if i == self.at else f"{DIM}{label}{RESET}")
            lines.append("".join(tabs))
        q, i = self.questions[self.at], self.at
        lines += [f"{BOLD}{ln}{RESET}" for ln in wrap_ansi(q.question, width)]
        for r, opt in enumerate(q.options + [self.OTHER]):
            mark = ("[x]" if r in self.picked[i] else "[ ]") if q.multi_select else ("(•)" if r in self.picked[i] else "( )")
            text = opt
            if r == len(q.options) and (self.other[i] or self.typing):
                text = f"Other: {self.other[i]}" + ("▌" if self.typing else "")
            row = f"{'›' if r == self.row[i] else ' '} {r + 1}. {mark} {text}"
            lines.append(f"{CYAN}{row}{RESET}" if r == self.row[i] else row)
            if r < len(q.descriptions) and q.descriptions[r]:
                lines += [f"{DIM}       {d}{RESET}" for d in wrap_ansi(q.descriptions[r], width - 7)]
        hint = "type, enter to confirm, esc to go back" if self.typing else \
            ("↑↓ move · space toggle · enter confirm" if q.multi_select else "↑↓ move · enter or digit pick") + (" · tab next question" if len(self.questions) > 1 else "") + " · esc cancel"
        lines.append(f"{DIM}{hint}{RESET}")
        return lines


# ------------------------------------------------------------------------------------------- markdown
# links first: the escape sequences the other rules insert contain "[", which a link pattern applied later would match
_INLINE = [(re.compile(r"`([^`]+)`"), lambda m: f"{YELLOW}{m.group(1)}{RESET}"),
           (re.compile(r"!?\[([^\]]+)\]\(([^)\s]+)\)"), lambda m: f"{UNDERLINE}{m.group(1)}{RESET}{GREY} ({m.group(2)}){RESET}"),
           (re.compile(r"\*\*\*(.+?)\*\*\*"), lambda m: f"{BOLD}{ITALIC}{m.group(1)}{RESET}"),
           (re.compile(r"\*\*(.+?)\*\*|__(.+?)__"), lambda m: f"{BOLD}{m.group(1) or m.group(2)}{RESET}"),
           (re.compile(r"(?<![\w*])\*(?!\s)(.+?)(?<!\s)\*(?![\w*])|(?<!\w)_(?!\s)(.+?)(?<!\s)_(?!\w)"), lambda m: f"{ITALIC}{m.group(1) or m.group(2)}{RESET}"),
           (re.compile(r"~~(.+?)~~"), lambda m: f"\x1b[9m{m.group(1)}{RESET}")]


def render_inline(text: str) -> str:
    """Emphasis, inline code and links; what is inside back-ticks is left alone."""
    parts = re.split(r"(`[^`]+`)", text)
    for i, p in enumerate(parts):
        if p.startswith("`") and p.endswith("`") and len(p) > 2:
            parts[i] = f"{YELLOW}{p[1:-1]}{RESET}"
        else:
            for rx, fn in _INLINE[1:]:
                p = rx.sub(fn, p)
            parts[i] = p
    return "".join(parts)


def _table(rows: list[list[str]], width: int) -> list[str]:
    cols = max(len(r) for r in rows)
    rows = [r + [""] * (cols - len(r)) for r in rows]
    cells = [[render_inline(c.strip()) for c in r] for r in rows]
    widths = [max(visible_width(r[j]) for r in cells) for j in range(cols)]
    over = sum(widths) + 3 * cols + 1 - width
    while over > 0 and max(widths) > 6:                              # shrink the widest columns until the table fits
        j = widths.index(max(widths))
        widths[j] -= 1
        over -= 1

    def fit(s: str, w: int) -> str:
        if visible_width(s) <= w:
            return s + " " * (w - visible_width(s))
        plain = _ANSI.sub("", s)
        return plain[:max(w - 1, 1)] + "…"

    out = []
    for i, r in enumerate(cells):
        line = "│ " + " │ ".join(fit(c, widths[j]) for j, c in enumerate(r)) + " │"
        out.append(f"{BOLD}{line}{RESET}" if i == 0 else line)
        if i == 0:
            out.append("├─" + "─┼─".join("─" * w for w in widths) + "─┤")
    return out


def render_markdown(text: str, width: int = 80) -> list[str]:
    lines = text.replace("\t", "    ").split("\n")
    out: list[str] = []
    i, n = 0, len(lines)
    while i < n:
        ln = lines[i]
        m = re.match(r"^(\s*)(```|~~~)\s*([\w+-]*)\s*$", ln)
        if m:                                                        # fenced code: verbatim, cut (not wrapped) to the width
            fence, lang = m.group(2), m.group(3)
            out.append(f"{GREY}┌── {lang or 'code'}{RESET}")
            i += 1
            while i < n and not lines[i].strip().startswith(fence):
                code = lines[i]
                out.append(f"{GREY}│{RESET} {GREEN}{code if visible_width(code) <= width - 2 else code[:max(width - 3, 1)] + '…'}{RESET}")
                i += 1
            out.append(f"{GREY}└──{RESET}")
            i += 1
            continue
        if re.match(r"^\s*\|.*\|\s*$", ln) and i + 1 < n and re.match(r"^\s*\|?[\s:|-]+\|[\s:|-]*$", lines[i + 1]) and "-" in lines[i + 1]:
            rows = [[c for c in ln.strip().strip("|").split("|")]]
            i += 2
            while i < n and re.match(r"^\s*\|.*\|\s*$", lines[i]):
                rows.append(lines[i].strip().strip("|").split("|"))
                i += 1
            out += _table(rows, width)
            continue
        m = re.match(r"^(#{1,6})\s+(.*?)\s*#*\s*$", ln)
        if m:
            level, title = len(m.group(1)), render_inline(m.group(2))
            style = BOLD + (UNDERLINE if level == 1 else "") + (CYAN if level <= 2 else "")
            if out and out[-1] != "":
                out.append("")
            out += [f"{style}{w}{RESET}" for w in wrap_ansi(title, width)]
            i += 1
            continue
        if re.match(r"^\s*([-*_])(\s*\1){2,}\s*$", ln):
            out.append(f"{GREY}{'─' * min(width, 60)}{RESET}")
            i += 1
            continue
        m = re.match(r"^(\s*)(>+)\s?(.*)$", ln)
        if m:
            depth = len(m.group(2))
            bar = f"{GREY}{'│ ' * depth}{RESET}"
            out += [bar + f"{ITALIC}{w}{RESET}" for w in wrap_ansi(render_inline(m.group(3)), width - 2 * depth)]
            i += 1
            continue
        m = re.match(r"^(\s*)([-*+]|\d+[.)])\s+(\[[ xX]\]\s+)?(.*)$", ln)
        if m:
            indent = len(m.group(1)) // 2 * 2
            bullet = "•" if not m.group(2)[0].isdigit() else m.group(2)
            if m.group(3):
                bullet = f"{GREEN}☑{RESET}" if "x" in m.group(3).lower() else "☐"
            item = m.group(4)
            while i + 1 < n and lines[i + 1].strip() and re.match(r"^\s{2,}\S", lines[i + 1]) and not re.match(r"^\s*([-*+]|\d+[.)])\s", lines[i + 1]):
                i += 1
                item += " " + lines[i].strip()                       # a lazy continuation line of the same item
            lead = " " * indent + bullet + " "
            wrapped = wrap_ansi(render_inline(item), width - visible_width(lead))
            out += [(lead if k == 0 else " " * visible_width(lead)) + w for k, w in enumerate(wrapped)]
            i += 1
            continue
        if not ln.strip():
            if out and out[-1] != "":
                out.append("")
            i += 1
            continue
        para = ln.strip()
        while i + 1 < n and lines[i + 1].strip() and not re.match(r"^\s*(#{1,6}\s|```|~~~|>|[-*+]\s|\d+[.)]\s|\|)", lines[i + 1]):
            i += 1
            para += " " + lines[i].strip()
        out += wrap_ansi(render_inline(para), width)
        i += 1
    while out and out[-1] == "":
        out.pop()
    return out


# ------------------------------------------------------------------------------------------- a real terminal
def read_line_raw(editor: LineEditor, prompt: str = "> ", fd_in: int = 0, write: Callable[[str], None] | None = None, width: int | None = None) -> str:
    """Run ``editor`` on the terminal behind ``fd_in`` until a line is submitted. Raw mode and bracketed paste are switched
    on for the duration and restored on every way out. Raises ``EOFError`` (ctrl-d on an empty line) or
    ``KeyboardInterrupt`` (ctrl-c on an empty line / escape)."""
    import shutil
    import sys
    import termios
    import tty

    write = write or (lambda s: (sys.stdout.write(s), sys.stdout.flush()) and None)
    width = width or shutil.get_terminal_size((100, 24)).columns
    saved = termios.tcgetattr(fd_in)
    drawn_rows, cursor_row = 0, 0

    def draw() -> None:
        nonlocal drawn_rows, cursor_row
        lines, (row, col) = editor.render(prompt, width)
        up = f"\x1b[{cursor_row}A" if cursor_row else ""
        write(up + "\r\x1b[J" + "\r\n".join(lines))
        back = len(lines) - 1 - row
        write((f"\x1b[{back}A" if back else "") + "\r" + (f"\x1b[{col}C" if col else ""))
        drawn_rows, cursor_row = len(lines), row

    try:
        tty.setraw(fd_in)
        write("\x1b[?2004h")
        draw()
        pending = ""
        while True:
            chunk = os.read(fd_in, 4096).decode("utf-8", "replace")
            if not chunk:
                raise EOFError
            pending += chunk
            if "\x1b[200~" in pending and "\x1b[201~" not in pending:
                continue                                             # wait for the end of a paste before interpreting it
            for key in parse_keys(pending):
                outcome = editor.feed(key)
                if outcome == "submit":
                    editor.candidates = []
                    draw()
                    write("\r\n" * (drawn_rows - cursor_row))
                    return editor.accept()
                if outcome == "eof":
                    raise EOFError
                if outcome == "cancel":
                    raise KeyboardInterrupt
            pending = ""
            draw()
    finally:
        write("\x1b[?2004l")
        termios.tcsetattr(fd_in, termios.TCSADRAIN, saved)


def questions_from_tool_args(questions: list[dict]) -> list[Question]:
    """The ``ask_user_question`` tool's argument format -> ``Question`` objects."""
    return [Question(q["question"], [o["label"] for o in q["options"]], str(q.get("header", "")), bool(q.get("multiSelect")),
                     [str(o.get("description", "")) for o in q["options"]]) for q in questions]


def run_selector(selector: QuestionSelector, keys, draw: Callable[[list[str]], None] | None = None, width: int = 80) -> dict | None:
    """Feed ``keys`` (any iterable of key names) to ``selector`` until it is done; ``draw(lines)`` after every key. Answers
    in the tool's result format: multi-select answers joined with ", ". None when cancelled or the keys ran out."""
    if draw is not None:
        draw(selector.render(width))
    for key in keys:
        selector.feed(key)
        if draw is not None:
            draw(selector.render(width))
        if selector.done:
            break
    if not selector.done or selector.cancelled:
        return None
    return {q: ", ".join(a) if isinstance(a, list) else a for q, a in (selector.answers() or {}).items()}


async def tty_question_handler(questions: list[dict]) -> dict[str, str]:
    """A question handler for ``AskUserQuestionEnvironment`` that shows the dialog on the controlling terminal."""
    import asyncio
    import shutil
    import sys
    import termios
    import tty

    def ask() -> dict[str, str]:
        fd = sys.stdin.fileno()
        saved = termios.tcgetattr(fd)
        rows = 0

        def draw(lines: list[str]) -> None:
            nonlocal rows
            sys.stdout.write((f"\x1b[{rows}A" if rows else "") + "\r\x1b[J" + "\r\n".join(lines) + "\r\n")
            sys.stdout.flush()
            rows = len(lines)

        def keys():
            while True:
                data = os.read(fd, 1024).decode("utf-8", "replace")
                if not data:
                    return
                yield from parse_keys(data)

        try:
            tty.setraw(fd)
            out = run_selector(QuestionSelector(questions_from_tool_args(questions)), keys(), draw, shutil.get_terminal_size((100, 24)).columns)
        finally:
            termios.tcsetattr(fd, termios.TCSADRAIN, saved)
        if out is None:
            raise RuntimeError("the user dismissed the questions")
        return out

    return await asyncio.to_thread(ask)
