"""Hierarchical browser of rollout traces: steps -> prompt groups -> rollouts -> one conversation with folds
(rollouts/rollouts/tui/traces.py:46-1700: ``TraceData``, ``StepPicker``, ``GroupPicker``, ``RolloutPicker``,
``TraceViewer``, ``TraceStreamingViewer``).

    python -m research_b200.frontend.trace_browser results/rl/<run>/rollouts.jsonl
    some_training_command | python -m research_b200.frontend.trace_browser --follow -      # records and stream events

Data model: a record (one JSON object per sample: ``step``, ``group_index`` or ``group``, ``prompt``, ``response``,
``reward``, optional ``messages`` / ``metadata.messages`` and ``status``) becomes a ``Rollout`` inside its ``Group``
inside its ``Step``. A record whose sample id was seen before UPDATES that rollout (a rollout that is still
``streaming`` grows as its records arrive), and ``handle_stream_event`` folds live model events (text / thinking /
tool call / tool result) into the rollout's messages.

Screens are plain objects: ``handle_key(key)`` mutates the state (and may return a child screen or ``POP``),
``render(width, height)`` returns the lines to show. ``Browser`` keeps the screen stack and, on a tty, runs the
raw-mode key loop; without one the same objects are driven by a key list, which is how the tests exercise them.

Keys (vim-like): ``j`` / ``k`` move, ``g`` / ``G`` top / bottom, ``ctrl-d`` / ``ctrl-u`` half page, ``enter`` / ``l`` open,
``q`` / ``h`` / ``esc`` back; in a conversation ``space`` or ``za`` toggles the fold at the cursor, ``zM`` folds all, ``zR``
opens all, ``e`` writes the conversation to a file and opens ``$EDITOR`` on it (interactive runs only).
"""

from __future__ import annotations

import json
import os
import select
import shutil
import subprocess
import sys
import tempfile
import zlib
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Iterable

POP = object()        # returned by handle_key: leave this screen


# ------------------------------------------------------------------------------------------ data model
@dataclass
class TraceMessage:
    role: str                 # user | assistant | tool | system | thinking
    content: str


@dataclass
class Rollout:
    step: int
    group_id: int
    sample_id: int            # position inside its group
    prompt: str
    response: str
    reward: float
    messages: list[TraceMessage] = field(default_factory=list)
    is_streaming: bool = False
    sample_key: str = ""      # the producer's own id of this sample; records with the same key update the rollout
    extra: dict[str, Any] = field(default_factory=dict)

    def conversation(self) -> list[TraceMessage]:
        """The messages to show: the recorded ones, or prompt + response when the record carried none."""
        if self.messages:
            return self.messages
        out = []
        if self.prompt:
            out.append(TraceMessage("user", self.prompt))
        if self.response:
            out.append(TraceMessage("assistant", self.response))
        return out


@dataclass
class Group:
    step: int
    group_id: int
    prompt: str
    rollouts: list[Rollout] = field(default_factory=list)

    def _rewards(self) -> list[float]:
        return [r.reward for r in self.rollouts]

    @property
    def avg_reward(self) -> float:
        rs = self._rewards()
        return sum(rs) / len(rs) if rs else 0.0

    @property
    def max_reward(self) -> float:
        return max(self._rewards(), default=0.0)

    @property
    def min_reward(self) -> float:
        return min(self._rewards(), default=0.0)

    @property
    def has_signal(self) -> bool:
        """Samples of the group differ in reward: the groups a group-relative policy gradient learns from."""
        return len(set(self._rewards())) > 1


@dataclass
class Step:
    step: int
    groups: list[Group] = field(default_factory=list)

    @property
    def num_rollouts(self) -> int:
        return sum(len(g.rollouts) for g in self.groups)

    @property
    def avg_reward(self) -> float:
        rs = [r.reward for g in self.groups for r in g.rollouts]
        return sum(rs) / len(rs) if rs else 0.0


def _group_key(record: dict) -> int:
    g = record.get("group_index", record.get("group"))
    if g is not None:
        return int(g)
    return zlib.crc32(str(record.get("prompt", "")).encode()) % 100000    # stable across processes, unlike hash()


def _messages_of(record: dict) -> list[TraceMessage]:
    raw = record.get("messages") or (record.get("metadata") or {}).get("messages") or []
    out = []
    for m in raw:
        c = m.get("content", "")
        if not isinstance(c, str):
            c = "".join(b.get("text", "") if isinstance(b, dict) else str(b) for b in c) if isinstance(c, list) else str(c)
        out.append(TraceMessage(str(m.get("role", "unknown")), c))
    return out


@dataclass
class TraceData:
    steps: list[Step] = field(default_factory=list)
    _by_key: dict[str, Rollout] = field(default_factory=dict, repr=False)

    @classmethod
    def from_jsonl(cls, path: str | Path) -> "TraceData":
        data = cls()
        p = Path(path)
        files = sorted(p.glob("rollouts*.jsonl")) if p.is_dir() else ([p] if p.exists() else [])
        for f in files:
            for line in f.read_text(errors="replace").splitlines():
                try:
                    rec = json.loads(line)
                except json.JSONDecodeError:
                    continue
                if isinstance(rec, dict):
                    data.add_record(rec)
        return data

    def _step(self, n: int) -> Step:
        for s in self.steps:
            if s.step == n:
                return s
        s = Step(n)
        self.steps.append(s)
        self.steps.sort(key=lambda x: x.step)
        return s

    def _group(self, step: Step, gid: int, prompt: str) -> Group:
        for g in step.groups:
            if g.group_id == gid:
                return g
        g = Group(step.step, gid, prompt)
        step.groups.append(g)
        return g

    def find_rollout(self, sample_key: str) -> Rollout | None:
        return self._by_key.get(sample_key)

    def add_record(self, record: dict) -> Rollout:
        """Add a sample record, or update the rollout that has the same sample id (``sample_id`` / ``id`` field)."""
        key = str(record.get("sample_id", record.get("id", "")))
        step_raw = record.get("step", 0)
        if not isinstance(step_raw, int):            # some producers put the sample's string id in "step"
            key = key or str(step_raw)
            step_raw = 0
        msgs = _messages_of(record)
        streaming = record.get("status") == "streaming"
        if key and key in self._by_key:
            r = self._by_key[key]
            r.response = str(record.get("response", r.response))
            r.reward = float(record.get("reward", r.reward) or 0.0)
            if msgs:
                r.messages = msgs
            r.is_streaming = streaming
            return r
        step = self._step(int(step_raw))
        prompt = str(record.get("prompt", ""))
        group = self._group(step, _group_key(record), prompt)
        known = {"step", "group", "group_index", "prompt", "response", "reward", "messages", "status", "sample_id", "id"}
        r = Rollout(step.step, group.group_id, len(group.rollouts), prompt, str(record.get("response", "")),
                    float(record.get("reward") or 0.0), msgs, streaming, key,
                    {k: v for k, v in record.items() if k not in known and k != "metadata"})
        group.rollouts.append(r)
        if key:
            self._by_key[key] = r
        return r

    def handle_stream_event(self, sample_key: str, event_type: str, event: dict) -> Rollout:
        """Fold one live model event into the rollout ``sample_key`` (created, as streaming, when unknown).
        Text and thinking events carry the whole block so far (``content``) or an increment (``delta``)."""
        r = self._by_key.get(sample_key)
        if r is None:
            r = self.add_record({"sample_id": sample_key, "step": int(event.get("step", 0)), "group_index": event.get("group_index"),
                                 "prompt": event.get("prompt", ""), "status": "streaming"})
            if r.prompt:
                r.messages.append(TraceMessage("user", r.prompt))

        def grow(role: str) -> None:
            last = r.messages[-1] if r.messages and r.messages[-1].role == role and event.get("continues", True) else None
            if last is None or event_type.endswith("_start"):
                last = TraceMessage(role, "")
                r.messages.append(last)
            last.content = event["content"] if "content" in event else last.content + str(event.get("delta", ""))

        if event_type in ("text_delta", "text_end", "text_start"):
            grow("assistant")
            r.response = r.messages[-1].content
        elif event_type in ("thinking_delta", "thinking_end", "thinking_start"):
            grow("thinking")
        elif event_type == "tool_call_end":
            call = event.get("tool_call", event)
            r.messages.append(TraceMessage("assistant", f"[tool call] {call.get('name', '?')}({json.dumps(call.get('args', {}))})"))
        elif event_type == "tool_result":
            r.messages.append(TraceMessage("tool", ("[error] " if event.get("is_error") else "") + str(event.get("content", ""))))
        elif event_type in ("done", "stream_done"):
            r.is_streaming = False
            if "reward" in event:
                r.reward = float(event["reward"])
        return r


# ------------------------------------------------------------------------------------------ screens
def _clip(s: str, width: int) -> str:
    s = s.replace("\n", "\\n").replace("\t", " ")
    return s if len(s) <= width else s[: max(0, width - 1)] + "…"


class ListScreen:
    """A scrolling list with a cursor; subclasses say what the rows are and what opening one means."""

    title = ""
    help = "j/k move  enter open  q back"

    def __init__(self) -> None:
        self.cursor = 0
        self.top = 0

    def rows(self) -> list[str]:
        raise NotImplementedError

    def open(self, index: int):
        return None

    def _move(self, delta: int, height: int) -> None:
        n = len(self.rows())
        self.cursor = max(0, min(n - 1, self.cursor + delta)) if n else 0

    def handle_key(self, key: str, height: int = 24):
        page = max(1, (height - 3) // 2)
        if key in ("j", "down"):
            self._move(1, height)
        elif key in ("k", "up"):
            self._move(-1, height)
        elif key == "g":
            self.cursor = 0
        elif key == "G":
            self.cursor = max(0, len(self.rows()) - 1)
        elif key == "ctrl-d":
            self._move(page, height)
        elif key == "ctrl-u":
            self._move(-page, height)
        elif key in ("enter", "l", "right"):
            return self.open(self.cursor) if self.rows() else None
        elif key in ("q", "h", "esc", "left"):
            return POP
        return None

    def render(self, width: int = 100, height: int = 24) -> list[str]:
        rows = self.rows()
        body = max(1, height - 2)
        if self.cursor < self.top:
            self.top = self.cursor
        if self.cursor >= self.top + body:
            self.top = self.cursor - body + 1
        out = [_clip(self.title, width)]
        for i in range(self.top, min(len(rows), self.top + body)):
            out.append(_clip(("> " if i == self.cursor else "  ") + rows[i], width))
        out += [""] * (height - 1 - len(out))
        out.append(_clip(f"{self.help}   [{self.cursor + 1 if rows else 0}/{len(rows)}]", width))
        return out


def _bar(value: float, lo: float, hi: float, width: int = 10) -> str:
    frac = 0.0 if hi <= lo else (value - lo) / (hi - lo)
    n = max(0, min(width, round(frac * width)))
    return "#" * n + "." * (width - n)


class StepPicker(ListScreen):
    def __init__(self, data: TraceData) -> None:
        super().__init__()
        self.data = data
        self.title = "steps: step, rollouts, groups (with signal), mean reward"

    def rows(self) -> list[str]:
        rs = [s.avg_reward for s in self.data.steps]
        lo, hi = (min(rs), max(rs)) if rs else (0.0, 1.0)
        return [f"step {s.step:>4}  {s.num_rollouts:>5} rollouts  {len(s.groups):>3} groups ({sum(g.has_signal for g in s.groups)})  "
                f"reward {s.avg_reward:7.3f} {_bar(s.avg_reward, lo, hi)}" for s in self.data.steps]

    def open(self, index: int):
        return GroupPicker(self.data.steps[index])


class GroupPicker(ListScreen):
    def __init__(self, step: Step) -> None:
        super().__init__()
        self.step = step
        self.title = f"step {step.step}: groups (samples, reward min / mean / max, * = samples differ)"

    def rows(self) -> list[str]:
        return [f"group {g.group_id:>5} {'*' if g.has_signal else ' '} {len(g.rollouts):>3} samples  "
                f"{g.min_reward:6.3f} / {g.avg_reward:6.3f} / {g.max_reward:6.3f}  {g.prompt}" for g in self.step.groups]

    def open(self, index: int):
        return RolloutPicker(self.step.groups[index])


class RolloutPicker(ListScreen):
    def __init__(self, group: Group) -> None:
        super().__init__()
        self.group = group
        self.title = f"step {group.step} group {group.group_id}: {group.prompt}"

    def rows(self) -> list[str]:
        return [f"sample {r.sample_id:>3}  reward {r.reward:7.3f}{'  (streaming)' if r.is_streaming else ''}  {r.response}"
                for r in self.group.rollouts]

    def open(self, index: int):
        return TraceViewer(self.group.rollouts[index])


class TraceViewer:
    """One conversation, message by message; long messages start folded to their first lines."""

    FOLD_LINES = 3
    help = "j/k scroll  space/za fold  zM/zR all  e editor  q back"

    def __init__(self, rollout: Rollout, fold_over: int = 12) -> None:
        self.rollout = rollout
        self.cursor = 0               # message index
        self.top = 0                  # first rendered line shown
        self.fold_over = fold_over
        self.folded: dict[int, bool] = {}
        self._pending = ""
        self.follow = rollout.is_streaming     # keep the cursor on the newest message while the rollout streams
        self._sync_folds()

    def _sync_folds(self) -> None:
        for i, m in enumerate(self.rollout.conversation()):
            self.folded.setdefault(i, m.content.count("\n") + 1 > self.fold_over)

    def plain_text(self) -> str:
        r = self.rollout
        head = f"# step {r.step} group {r.group_id} sample {r.sample_id} reward {r.reward:.4f}\n"
        return head + "\n".join(f"\n## {m.role}\n{m.content}" for m in r.conversation())

    def open_in_editor(self) -> str:
        """Write the conversation to a temporary markdown file and run ``$EDITOR`` on it (when one is set and this is
        a terminal); returns the file's path."""
        with tempfile.NamedTemporaryFile("w", suffix=".md", prefix="trace_", delete=False) as f:
            f.write(self.plain_text())
            path = f.name
        editor = os.environ.get("EDITOR")
        if editor and sys.stdout.isatty() and shutil.which(editor.split()[0]):
            subprocess.call(editor.split() + [path])
        return path

    def handle_key(self, key: str, height: int = 24):
        n = len(self.rollout.conversation())
        self._sync_folds()
        if self._pending == "z":
            self._pending = ""
            if key == "a":
                self.folded[self.cursor] = not self.folded.get(self.cursor, False)
            elif key == "M":
                self.folded = {i: True for i in range(n)}
            elif key == "R":
                self.folded = {i: False for i in range(n)}
            elif key == "c":
                self.folded[self.cursor] = True
            elif key == "o":
                self.folded[self.cursor] = False
            return None
        if key == "z":
            self._pending = "z"
        elif key in ("j", "down"):
            self.cursor, self.follow = min(max(n - 1, 0), self.cursor + 1), False
        elif key in ("k", "up"):
            self.cursor, self.follow = max(0, self.cursor - 1), False
        elif key == "g":
            self.cursor, self.follow = 0, False
        elif key == "G":
            self.cursor, self.follow = max(n - 1, 0), self.rollout.is_streaming
        elif key in ("space", " "):
            self.folded[self.cursor] = not self.folded.get(self.cursor, False)
        elif key == "e":
            self.open_in_editor()
        elif key in ("q", "h", "esc", "left"):
            return POP
        return None

    def _lines(self, width: int) -> tuple[list[str], list[int]]:
        """All rendered lines and, per message, the index of its first line."""
        out, starts = [], []
        for i, m in enumerate(self.rollout.conversation()):
            starts.append(len(out))
            body = m.content.split("\n")
            folded = self.folded.get(i, False)
            mark = ">" if i == self.cursor else " "
            out.append(_clip(f"{mark} [{m.role}] {len(body)} lines{' (folded)' if folded else ''}", width))
            shown = body[: self.FOLD_LINES] if folded else body
            for ln in shown:
                while len(ln) > width - 4:                 # wrap long lines
                    out.append("    " + ln[: width - 4])
                    ln = ln[width - 4:]
                out.append("    " + ln)
            if folded and len(body) > self.FOLD_LINES:
                out.append(f"    ... {len(body) - self.FOLD_LINES} more lines")
        return out, starts

    def render(self, width: int = 100, height: int = 24) -> list[str]:
        self._sync_folds()
        r = self.rollout
        if self.follow:
            self.cursor = max(0, len(r.conversation()) - 1)
        lines, starts = self._lines(width)
        body = max(1, height - 2)
        if starts:
            first = starts[min(self.cursor, len(starts) - 1)]
            if first < self.top:
                self.top = first
            if first >= self.top + body:
                self.top = first - body + 1
            if self.follow:
                self.top = max(0, len(lines) - body)
        head = f"step {r.step} group {r.group_id} sample {r.sample_id}  reward {r.reward:.4f}{'  STREAMING' if r.is_streaming else ''}"
        out = [_clip(head, width)] + lines[self.top:self.top + body]
        out += [""] * (height - 1 - len(out))
        out.append(_clip(self.help, width))
        return out


# ------------------------------------------------------------------------------------------ driver
_ESCAPES = {"\x1b[A": "up", "\x1b[B": "down", "\x1b[C": "right", "\x1b[D": "left", "\r": "enter", "\n": "enter",
            "\x04": "ctrl-d", "\x15": "ctrl-u", "\x1b": "esc", " ": "space"}


def decode_keys(raw: str) -> list[str]:
    """Terminal bytes -> key names (arrow escape sequences, control keys, printable characters)."""
    keys, i = [], 0
    while i < len(raw):
        if raw.startswith("\x1b[", i) and i + 2 < len(raw) and raw[i:i + 3] in _ESCAPES:
            keys.append(_ESCAPES[raw[i:i + 3]])
            i += 3
            continue
        keys.append(_ESCAPES.get(raw[i], raw[i]))
        i += 1
    return keys


class Browser:
    """Screen stack + key loop. ``feed(keys)`` is the whole logic; ``run`` adds the raw-mode terminal around it."""

    def __init__(self, data: TraceData, width: int = 100, height: int = 24) -> None:
        self.data = data
        self.width, self.height = width, height
        self.stack: list[Any] = [StepPicker(data)]
        # a run with one step (an evaluation, or a live stream) opens on its groups straight away
        if len(data.steps) == 1:
            self.stack.append(GroupPicker(data.steps[0]))

    @property
    def screen(self):
        return self.stack[-1]

    def feed(self, keys: Iterable[str]) -> bool:
        """Apply keys; returns False once the last screen was left."""
        for k in keys:
            res = self.screen.handle_key(k, self.height)
            if res is POP:
                self.stack.pop()
                if not self.stack:
                    return False
            elif res is not None:
                self.stack.append(res)
        return True

    def frame(self) -> list[str]:
        return self.screen.render(self.width, self.height)

    def run(self, follow=None) -> None:
        """Interactive loop on a tty. ``follow``: a text stream of JSON lines (records, or ``{"sample_id", "event",
        ...}`` stream events) merged into the data while browsing."""
        if not sys.stdout.isatty():
            print("\n".join(self.frame()))
            return
        import termios
        import tty as ttymod

        tty = open("/dev/tty", "rb", buffering=0)  # noqa: SIM115 - closed in finally
        restore = termios.tcgetattr(tty.fileno())
        ttymod.setcbreak(tty.fileno())
        try:
            sys.stdout.write("\x1b[?1049h\x1b[?25l")
            alive, eof = True, follow is None
            while alive:
                size = shutil.get_terminal_size((100, 24))
                self.width, self.height = size.columns, size.lines
                sys.stdout.write("\x1b[H" + "\n".join(ln + "\x1b[K" for ln in self.frame()))
                sys.stdout.flush()
                ready = [tty] + ([] if eof else [follow])
                r, _, _ = select.select(ready, [], [], 0.25)
                if not eof and follow in r:
                    line = follow.readline()
                    if not line:
                        eof = True
                    else:
                        ingest_line(self.data, line)
                if tty in r:
                    alive = self.feed(decode_keys(os.read(tty.fileno(), 64).decode(errors="ignore")))
        finally:
            termios.tcsetattr(tty.fileno(), termios.TCSADRAIN, restore)
            tty.close()
            sys.stdout.write("\x1b[?25h\x1b[?1049l")
            sys.stdout.flush()


def ingest_line(data: TraceData, line: str) -> bool:
    """One line of a live stream: a sample record, a stream event (``{"sample_id", "event": type, ...}``), or a
    JSON log line whose ``message`` is itself such an object. Anything else is ignored."""
    try:
        obj = json.loads(line)
    except json.JSONDecodeError:
        return False
    if not isinstance(obj, dict):
        return False
    if "event" in obj and "sample_id" in obj:
        data.handle_stream_event(str(obj["sample_id"]), str(obj["event"]), obj)
        return True
    if "reward" in obj or "response" in obj or "messages" in obj:
        data.add_record(obj)
        return True
    msg = obj.get("message")
    return ingest_line(data, msg) if isinstance(msg, str) and msg.startswith("{") else False


def main(argv: list[str] | None = None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="Browse rollout traces: steps, groups, rollouts, conversations")
    ap.add_argument("path", help="rollouts.jsonl, a run directory, or - with --follow")
    ap.add_argument("--follow", action="store_true", help="also read records / stream events from standard input while browsing")
    ap.add_argument("--keys", default="", help="apply these keys and print the resulting frame (no terminal needed)")
    a = ap.parse_args(argv)
    data = TraceData() if a.path == "-" else TraceData.from_jsonl(a.path)
    if a.path != "-" and not data.steps:
        print(f"no rollout records under {a.path}")
        return 1
    b = Browser(data)
    if a.keys or not sys.stdout.isatty():
        if a.follow:
            for line in sys.stdin:
                ingest_line(data, line)
            b = Browser(data)
        b.feed(decode_keys(a.keys))
        print("\n".join(b.frame()) if b.stack else "")
        return 0
    b.run(sys.stdin if a.follow else None)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
