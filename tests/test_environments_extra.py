"""Environments beyond the basic set: chess puzzle, git worktree, ask-user, browsing, screenspot."""

import asyncio
import subprocess

from research_b200.agents.dtypes import ToolCall
from research_b200.agents.environments import (AskUserQuestionEnvironment, Board, BrowsingEnvironment,
                                               ChessPuzzleEnvironment, GitWorktreeEnvironment, ScreenSpotEnvironment)


def _call(name, **args):
    return ToolCall(id="c1", name=name, args=args)


def _perft(b, d):
    if d == 0:
        return 1
    n = 0
    for m in b.legal_moves():
        c = b.copy()
        c.push(m)
        n += _perft(c, d - 1)
    return n


def test_chess_rules_perft():
    assert [_perft(Board(), d) for d in (1, 2, 3)] == [20, 400, 8902]
    kiwipete = Board("r3k2r/p1ppqpb1/bn2pnp1/3PN3/1p2P3/2N2Q1p/PPPBBPPP/R3K2R w KQkq - 0 1")
    assert (_perft(kiwipete, 1), _perft(kiwipete, 2)) == (48, 2039)
    ep = Board("8/2p5/3p4/KP5r/1R3p1k/8/4P1P1/8 w - - 0 1")
    assert [_perft(ep, d) for d in (1, 2, 3)] == [14, 191, 2812]
    assert Board().fen() == "rnbqkbnr/pppppppp/8/8/8/8/PPPPPPPP/RNBQKBNR w KQkq - 0 1"


def test_chess_puzzle_environment():
    async def go():
        # back-rank mate in one: Re8#
        env = ChessPuzzleEnvironment(fen="6k1/5ppp/8/8/8/8/8/4R1K1 w - - 0 1", solution=["e1e8"])
        bad = await env.exec_tool(_call("make_move", move="e1e9"), None, None)
        assert bad.is_error and "Legal" in bad.error
        ok = await env.exec_tool(_call("make_move", move="Re8"), None, None)
        assert not ok.is_error and "Checkmate" in ok.content
        snap = await env.serialize()
        env2 = await ChessPuzzleEnvironment.deserialize(snap)
        assert env2.board.fen() == env.board.fen() and env2.moves_made == ["e1e8"]
        res = await env2.exec_tool(_call("submit_answer", move="Re8#"), None, None)
        assert res.metadata["correct"] and res.stop_reason is not None
        wrong = await env2.exec_tool(_call("submit_answer", move="e1e7"), None, None)
        assert not wrong.metadata["correct"]
        assert 0.0 <= await env.get_value() <= 1.0

    asyncio.run(go())


def test_git_worktree_environment(tmp_path):
    async def go():
        (tmp_path / "a.txt").write_text("hello\n")
        env = GitWorktreeEnvironment(working_dir=str(tmp_path))
        await env.on_session_start("s1")
        assert env.worktree_path and (tmp_path / ".rollouts" / "worktrees" / "s1" / "a.txt").exists()
        r = await env.exec_tool(_call("write", path="b.txt", content="new file\n"), None, None)
        assert not r.is_error
        r = await env.exec_tool(_call("edit", path="a.txt", old="hello", new="bye"), None, None)
        assert not r.is_error and env.commit_count == 2
        r = await env.exec_tool(_call("read", path="a.txt"), None, None)
        assert r.content == "bye\n" and env.commit_count == 2
        assert (tmp_path / "a.txt").read_text() == "hello\n"          # the main checkout is untouched
        log = subprocess.run(["git", "log", "--oneline", "rollouts/s1"], cwd=tmp_path, capture_output=True, text=True).stdout
        assert "write: b.txt" in log and "edit: a.txt" in log
        diff = await env.diff_against_base()
        assert "+bye" in diff and "b.txt" in diff
        env2 = await GitWorktreeEnvironment.deserialize(await env.serialize())
        assert env2.worktree_path == env.worktree_path and env2.commit_count == 2
        escape = await env.exec_tool(_call("read", path="../../../a.txt"), None, None)
        assert escape.is_error

    asyncio.run(go())


def test_ask_user_environment():
    async def go():
        seen = []

        async def handler(questions):
            seen.extend(questions)
            return {q["question"]: q["options"][0]["label"] for q in questions}

        env = AskUserQuestionEnvironment(question_handler=handler)
        q = {"question": "Which database?", "header": "DB", "multiSelect": False,
             "options": [{"label": "sqlite", "description": "file"}, {"label": "postgres", "description": "server"}]}
        r = await env.exec_tool(_call("ask_user_question", questions=[q]), None, None)
        assert not r.is_error and "A: sqlite" in r.content and len(seen) == 1
        bad = await env.exec_tool(_call("ask_user_question", questions=[{**q, "options": q["options"][:1]}]), None, None)
        assert bad.is_error and "2-4 options" in bad.error
        assert env.get_tools()[0].function.name == "ask_user_question" and not env.requires_confirmation(_call("x"))

    asyncio.run(go())


def test_browsing_environment_with_fakes():
    async def go():
        async def fetch(url):
            if "missing" in url:
                return 404, "text/html", ""
            return 200, "text/html", "<html><script>x()</script><body><h1>Title</h1><p>Body &amp; more</p></body></html>"

        async def search(query, k):
            return [{"title": f"hit {i} for {query}", "url": f"http://example.test/{i}", "snippet": "s"} for i in range(k)]

        env = BrowsingEnvironment(fetcher=fetch, searcher=search, max_chars=12)
        r = await env.exec_tool(_call("web_search", query="b200", max_results=3), None, None)
        assert r.content.count("http://example.test/") == 3
        r = await env.exec_tool(_call("web_fetch", url="http://example.test/page"), None, None)
        assert r.content.startswith("Title") and "x()" not in r.content and "truncated" in r.content
        assert (await env.exec_tool(_call("web_fetch", url="http://example.test/missing"), None, None)).is_error
        assert (await env.exec_tool(_call("web_fetch", url="file:///etc/passwd"), None, None)).is_error
        env2 = await BrowsingEnvironment.deserialize(await env.serialize())
        assert env2.history == ["http://example.test/page"]

    asyncio.run(go())


def test_screenspot_reward():
    f = ScreenSpotEnvironment.compute_reward
    assert f("click [[0.5, 0.5]]", [400, 300, 600, 500], [1000, 1000]) == 1.0
    assert f("box [[0.1,0.1,0.2,0.2]]", [400, 300, 600, 500], [1000, 1000]) == 0.0
    assert f("box [[0.4,0.3,0.6,0.5]]", [400, 300, 600, 500], [1000, 1000]) == 1.0
    assert f("no coordinates", [0, 0, 10, 10], [100, 100]) == 0.0
