"""Terminal widgets driven by key names: key decoding, the line editor, the question dialog, Markdown rendering."""

import re

from research_b200.frontend.widgets import (LineEditor, Question, QuestionSelector, make_completer, parse_keys, render_inline, render_markdown,
                                            visible_width, wrap_ansi)

PLAIN = lambda s: re.sub(r"\x1b\[[0-9;?]*[A-Za-z]", "", s)        # noqa: E731


def typed(ed, *keys):
    out = None
    for k in keys:
        for key in (parse_keys(k) if len(k) > 1 and not k.isascii() or k.startswith("\x1b") else [k]) if k.startswith("\x1b") else ([k] if len(k) == 1 or "-" in k or k in NAMES or k.startswith("paste:") else list(k)):
            out = ed.feed(key)
    return out


NAMES = {"enter", "tab", "up", "down", "left", "right", "home", "end", "backspace", "delete", "escape"}


def test_key_decoding():
    assert parse_keys("ab\x1b[A\x1b[1;5D\x7f\r") == ["a", "b", "up", "ctrl-left", "backspace", "enter"]
    assert parse_keys("\x1bOA\x1b\r\x1bb\x01\x1b[3~\x1b[Z") == ["up", "alt-enter", "alt-b", "ctrl-a", "delete", "shift-tab"]
    assert parse_keys("x\x1b[200~two\r\nlines\x1b[201~y") == ["x", "paste:two\nlines", "y"] and parse_keys("\x1b") == ["escape"]
    assert parse_keys("é日") == ["é", "日"] and visible_width("日本\x1b[1mx\x1b[0m") == 5


def test_line_editor_editing_history_and_multiline():
    ed = LineEditor(history=["first", "second"])
    typed(ed, "hello wide world")
    typed(ed, "ctrl-left", "ctrl-left")
    assert ed.text[ed.cursor:] == "wide world"
    typed(ed, "ctrl-k")
    assert ed.text == "hello " and ed.kill_buffer == "wide world"
    typed(ed, "ctrl-y", "home", "alt-d")
    assert ed.text == " wide world" and ed.kill_buffer == "hello"
    typed(ed, "end", "ctrl-w", "ctrl-w")
    assert ed.text == " " and typed(ed, "ctrl-u") is None and ed.text == ""
    # history: up twice, down past the end restores the draft
    typed(ed, "draft")
    typed(ed, "up")
    assert ed.text == "second"
    typed(ed, "up", "up")
    assert ed.text == "first"
    typed(ed, "down", "down")
    assert ed.text == "draft"
    # multi-line: alt-enter, trailing backslash, a paste with a newline; up / down move inside the text
    typed(ed, "ctrl-u", "one")
    typed(ed, "alt-enter")
    typed(ed, "two\\")
    assert typed(ed, "enter") is None and ed.text == "one\ntwo\n"
    typed(ed, "paste:three\nfour")
    assert ed.text == "one\ntwo\nthree\nfour"
    typed(ed, "up")
    assert ed.text[:ed.cursor] == "one\ntwo\nthre"
    lines, (row, col) = ed.render("> ")
    assert [PLAIN(x) for x in lines] == ["> one", "  two", "  three", "  four"] and (row, col) == (2, 6)
    typed(ed, "down")
    assert typed(ed, "enter") == "submit" and ed.accept() == "one\ntwo\nthree\nfour" and ed.text == "" and ed.history[-1].startswith("one\n")
    assert typed(ed, "ctrl-d") == "eof" and typed(ed, "ctrl-c") == "cancel"
    typed(ed, "x")
    assert typed(ed, "ctrl-c") is None and ed.text == "" and typed(ed, "enter") == "submit" and ed.accept() == "" and len(ed.history) == 3
    typed(ed, "ab")
    typed(ed, "left", "ctrl-t")
    assert ed.text == "ba"


def test_completion_of_commands_and_paths(tmp_path):
    (tmp_path / "src").mkdir()
    (tmp_path / "src" / "main.py").write_text("")
    (tmp_path / "src" / "model.py").write_text("")
    (tmp_path / "setup.py").write_text("")
    (tmp_path / ".hidden").write_text("")
    comp = make_completer(["model", "slice", "status", "save"], str(tmp_path), hints={"slice": "[0:5, summarize:5:20]"})
    ed = LineEditor(completer=comp)
    typed(ed, "/mo")
    assert ed.ghost() == "del"
    typed(ed, "tab")
    assert ed.text == "/model " and ed.candidates == []
    typed(ed, "ctrl-u", "/s", "tab")
    assert ed.text == "/s" and ed.candidates == ["/save", "/slice", "/status"]
    typed(ed, "tab")
    assert ed.text == "/save" and "/slice" in PLAIN(ed.render()[0][-1])
    typed(ed, "tab")
    assert ed.text == "/slice"
    typed(ed, " ")
    assert ed.ghost() == "[0:5, summarize:5:20]"
    typed(ed, "ctrl-u", "look at @s", "tab")
    assert ed.text == "look at @s" and ed.candidates == ["@setup.py", "@src/"]
    typed(ed, "r", "tab")
    assert ed.text == "look at @src/"
    typed(ed, "m", "tab")
    assert ed.text == "look at @src/m" and ed.candidates == ["@src/main.py", "@src/model.py"]
    typed(ed, "a")
    assert ed.ghost() == "in.py"
    typed(ed, "right")
    assert ed.text == "look at @src/main.py"
    assert comp("./.h") == ["./.hidden"] and comp("plain words") == [] and comp("@nowhere/x") == []


def test_question_selector_single_multi_and_other():
    qs = QuestionSelector([Question("Which database?", ["Postgres", "SQLite"], header="DB", descriptions=["server", "a file"]),
                           Question("Which features?", ["auth", "search", "export"], header="Features", multi_select=True)])
    shown = [PLAIN(x) for x in qs.render(60)]
    assert "DB" in shown[0] and "Features" in shown[0] and shown[1] == "Which database?" and "› 1. ( ) Postgres" in shown and "       a file" in shown
    for k in ("down", "enter"):                 # pick SQLite: moves on to the second question
        qs.feed(k)
    assert qs.at == 1 and not qs.done
    for k in (" ", "down", "down", " ", "down", "enter"):         # auth, export, then "Other"
        qs.feed(k)
    assert qs.typing
    for k in list("audit log") + ["enter"]:
        qs.feed(k)
    assert not qs.typing and not qs.done and any("[x] Other: audit log" in PLAIN(x) for x in qs.render())
    qs.feed("enter")
    assert qs.done and qs.answers() == {"Which database?": "SQLite", "Which features?": ["auth", "export", "audit log"]}
    # digits pick directly; tab changes question; escape cancels
    one = QuestionSelector([Question("Proceed?", ["yes", "no"])])
    one.feed("2")
    one.feed("enter")
    assert one.done and one.answers() == {"Proceed?": "no"}
    other = QuestionSelector([Question("Name?", ["default"])])
    for k in ["down", "enter", *"zeta", "backspace", "enter"]:
        other.feed(k)
    assert other.done and other.answers() == {"Name?": "zet"}
    gone = QuestionSelector([Question("a", ["x"]), Question("b", ["y"])])
    gone.feed("tab")
    assert gone.at == 1
    gone.feed("escape")
    assert gone.done and gone.answers() is None


def test_markdown_rendering_and_wrapping():
    assert [PLAIN(x) for x in wrap_ansi("aaa bbb ccc ddd", 7)] == ["aaa bbb", "ccc ddd"] and wrap_ansi("x" * 25, 10) == ["x" * 10, "x" * 10, "x" * 5]
    styled = wrap_ansi("\x1b[1mbold words that wrap\x1b[0m", 10)
    assert all(s.endswith("\x1b[0m") for s in styled) and styled[1].startswith("\x1b[1m") and all(visible_width(s) <= 10 for s in styled)
    assert PLAIN(render_inline("a **b** `c*d*` _e_ [f](http://g) 2*3*4 snake_case_name")) == "a b c*d* e f (http://g) 2*3*4 snake_case_name"
    md = """# Title

Some *emphasis* and a paragraph that is long enough to need wrapping at forty columns or so.

- first item
  continues here
- [x] done
1. numbered

> quoted **text**

```python
def f(x):
    return x  # a comment that is much longer than the width of the display area
```

| name | value |
|------|------:|
| alpha | 1 |
| beta | 22 |

---
"""
    out = [PLAIN(x) for x in render_markdown(md, 40)]
    assert out[0] == "Title" and all(visible_width(x) <= 40 for x in out)
    assert "• first item continues here" in out and "☑ done" in out and "1. numbered" in out and "│ quoted text" in out
    assert "┌── python" in out and "│ def f(x):" in out and any(x.endswith("…") and x.startswith("│     return x") for x in out)
    assert "│ name  │ value │" in out and "│ beta  │ 22    │" in out and out[-1].startswith("───")
    assert "\x1b[1m" in render_markdown("# T")[0] and render_markdown("") == []


def test_question_dialog_from_tool_arguments_and_runner_completer(tmp_path):
    import io

    from research_b200.agents.dtypes import Endpoint
    from research_b200.frontend.terminal import AnsiFrontend, InteractiveRunner
    from research_b200.frontend.widgets import questions_from_tool_args, run_selector

    args = [{"question": "Which one?", "header": "Pick", "multiSelect": False, "options": [{"label": "A", "description": "first"}, {"label": "B", "description": "second"}]},
            {"question": "Extras?", "header": "Extras", "multiSelect": True, "options": [{"label": "x", "description": ""}, {"label": "y", "description": ""}]}]
    frames = []
    out = run_selector(QuestionSelector(questions_from_tool_args(args)), ["2", "enter", " ", "down", " ", "enter", "never read"], frames.append)
    assert out == {"Which one?": "B", "Extras?": "x, y"} and len(frames) == 7 and any("second" in PLAIN(x) for x in frames[0])
    assert run_selector(QuestionSelector(questions_from_tool_args(args)), ["escape"]) is None and run_selector(QuestionSelector(questions_from_tool_args(args)), ["1"]) is None
    # the runner hands the ANSI front end a completer that knows built-in and file commands and their hints
    fe = AnsiFrontend(out=io.StringIO(), inp=io.StringIO(""))
    from research_b200.frontend.slash_commands import SlashCommand

    InteractiveRunner(Endpoint(provider="mock"), fe, cwd=str(tmp_path), file_commands=[SlashCommand("review", "r", "<file>", "Review $1", "(user)")])
    assert fe.completer("/re") == ["/retry", "/review"] and fe.completer.hints["review"] == "<file>" and not fe._is_tty()
