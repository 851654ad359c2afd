"""Fingerprints, run-time system prompts, package paths and the dataset loaders of the agent layer (CPU)."""

import asyncio
import io
import json
import subprocess
from datetime import datetime

import pytest

from research_b200.agents import datasets, fingerprint, paths, prompt
from research_b200.agents.dtypes import Endpoint, EvalConfig, Message, Score, Metric, Tool, ToolFunction, ToolFunctionParameter


def _score(trajectory, row):
    return Score((Metric("ok", 1.0, 1.0),))


def _prep(row):
    return [Message("user", row["q"])]


def _tool(name, description=""):
    return Tool(function=ToolFunction(name=name, description=description, parameters=ToolFunctionParameter(properties={})))


# ------------------------------------------------------------------------------------------- fingerprints
def test_eval_fingerprint_is_stable_ignores_credentials_and_follows_the_config(tmp_path):
    data = tmp_path / "d.jsonl"
    data.write_text('{"q": "1"}\n')
    a = EvalConfig(Endpoint(provider="mock", model="m", api_key="sk-one"), _score, prepare_messages=_prep, max_samples=4)
    b = EvalConfig(Endpoint(provider="mock", model="m", api_key="sk-two"), _score, prepare_messages=_prep, max_samples=4)
    c = EvalConfig(Endpoint(provider="mock", model="m", api_key="sk-one"), _score, prepare_messages=_prep, max_samples=5)
    fa, fb, fc = (fingerprint.fingerprint_eval(x, dataset_path=data, allow_dirty=True, cwd=tmp_path) for x in (a, b, c))
    assert fa["config_hash"] == fb["config_hash"] != fc["config_hash"]
    assert "sk-one" not in json.dumps(fa) and fa["endpoint_summary"] == "mock/m" and fa["git_sha"] == "unknown"
    data.write_text('{"q": "2"}\n')
    assert fingerprint.fingerprint_eval(a, dataset_path=data, allow_dirty=True, cwd=tmp_path)["config_hash"] != fa["config_hash"]
    with pytest.raises(ValueError, match="lambda"):
        fingerprint.fingerprint_eval(EvalConfig(a.endpoint, lambda t, r: None), allow_dirty=True, cwd=tmp_path)


def test_dirty_tree_is_refused_unless_allowed(tmp_path):
    def git(*a):
        subprocess.run(["git", *a], cwd=tmp_path, check=True, capture_output=True)

    git("init", "-q")
    git("config", "user.email", "t@example.com")
    git("config", "user.name", "t")
    (tmp_path / "f").write_text("1")
    git("add", "f")
    git("commit", "-q", "-m", "one")
    sha, dirty = fingerprint.require_clean_git(cwd=tmp_path)
    assert sha != "unknown" and not dirty
    (tmp_path / "f").write_text("2")
    with pytest.raises(RuntimeError, match="uncommitted"):
        fingerprint.require_clean_git(cwd=tmp_path)
    assert fingerprint.require_clean_git(allow_dirty=True, cwd=tmp_path) == (sha, True)
    fp = fingerprint.fingerprint_session("p/m", "coding", ["read", "bash"], "be careful", cwd=tmp_path)
    assert fingerprint.fingerprint_short(fp).endswith(f"@{sha}*") and fp["tools"] == ["bash", "read"]


def test_warn_if_changed_distinguishes_config_from_code():
    base = {"config_hash": "a" * 16, "git_sha": "111", "git_dirty": False}
    out = io.StringIO()
    assert not fingerprint.warn_if_changed(None, base, file=out) and not fingerprint.warn_if_changed(base, dict(base), file=out)
    assert fingerprint.warn_if_changed(base, {**base, "config_hash": "b" * 16}, "run x", file=out) and "configuration changed" in out.getvalue()
    out = io.StringIO()
    assert fingerprint.warn_if_changed(base, {**base, "git_sha": "222"}, file=out) and "111 -> 222" in out.getvalue()
    cmp = fingerprint.compare_fingerprints(base, {**base, "git_sha": "222"})
    assert cmp["same_config"] and not cmp["same_code"]


def test_evaluate_records_its_fingerprint_and_warns_on_resume_after_a_change(tmp_path, capsys):
    from research_b200.agents.evaluation import evaluate
    from research_b200.agents.providers import ScriptedLLM, register_provider

    register_provider("mock", ScriptedLLM(["ok"]))

    rows = [{"id": "a", "q": "hi"}, {"id": "b", "q": "there"}]
    cfg = EvalConfig(Endpoint(provider="mock", model="echo"), _score, prepare_messages=_prep, max_turns=1, output_dir=str(tmp_path),
                     eval_name="run", n_retries=0)
    rep = asyncio.run(evaluate(rows, cfg))
    assert rep.config["fingerprint"]["domain"] == "eval"
    saved = json.loads((tmp_path / "run" / "report.json").read_text())["config"]["fingerprint"]
    assert saved["config_hash"] == rep.config["fingerprint"]["config_hash"]
    capsys.readouterr()
    import dataclasses

    asyncio.run(evaluate(rows, dataclasses.replace(cfg, max_turns=2), resume=True))
    assert "configuration changed" in capsys.readouterr().err
    asyncio.run(evaluate(rows, dataclasses.replace(cfg, max_turns=2), resume=True))
    assert "configuration changed" not in capsys.readouterr().err


# ------------------------------------------------------------------------------------------- paths and prompts
def test_package_paths_point_at_files_that_exist():
    assert (paths.get_package_dir() / "__init__.py").is_file() and paths.get_readme_path().is_file()
    assert paths.get_readme_content().lstrip().startswith("#") and paths.get_version()
    assert paths.get_doc_content("../etc/passwd") is None and paths.get_doc_content("no-such-file.md") is None


def test_system_prompt_follows_the_tool_set_and_the_project_context(tmp_path):
    (tmp_path / "AGENTS.md").write_text("outer advice")
    inner = tmp_path / "pkg" / "sub"
    inner.mkdir(parents=True)
    (inner.parent / "CLAUDE.md").write_text("inner advice")
    (inner.parent / "AGENTS.md").write_text("preferred over the other file of this folder")
    ro = prompt.build_system_prompt("coding", [_tool("read"), _tool("bash"), _tool("lookup", "find a symbol")], cwd=inner,
                                    now=datetime(2025, 1, 2, 3, 4, 5))
    assert "READ-ONLY mode with bash access" in ro and "- lookup: find a symbol" in ro and "- read: read a file" in ro
    assert ro.index("outer advice") < ro.index("preferred over") and "inner advice" not in ro
    assert "2025-01-02 03:04:05" in ro and str(inner) in ro and "research_b200" in ro
    rw = prompt.build_system_prompt("coding", [_tool("read"), _tool("write"), _tool("edit"), _tool("bash")], cwd=inner,
                                    include_self_docs=False, include_project_context=False, env_system_prompt="ENV SAYS")
    assert "READ-ONLY" not in rw and "Read a file before you edit it" in rw and "ENV SAYS" in rw and "advice" not in rw
    assert prompt.build_system_prompt("no-such-env", [], cwd=inner, include_self_docs=False).startswith("You are a helpful assistant.")


# ------------------------------------------------------------------------------------------- datasets
PUZZLES = """PuzzleId,FEN,Moves,Rating,RatingDeviation,Popularity,NbPlays,Themes,GameUrl,OpeningTags
p1,r1bqkbnr/pppp1ppp/2n5/4p3/2B1P3/5Q2/PPPP1PPP/RNB1K1NR b KQkq - 3 3,g8e7 f3f7,600,80,90,1000,mate mateIn1 short,https://lichess.org/x,Italian_Game
p2,4k3/8/8/8/8/8/4P3/4K3 b - - 0 1,e8d8 e2e4 d8c8 e4e5,1500,75,80,200,endgame fork,https://lichess.org/y,
p3,4k3/8/8/8/8/8/4P3/4K3 b - - 0 1,e8d8 e2e3,2400,75,80,200,endgame quietMove,https://lichess.org/z,
"""


def test_lichess_rows_filters_and_the_position_the_solver_sees(tmp_path):
    import gzip

    (tmp_path / "lichess_db_puzzle.csv").write_text(PUZZLES)
    every = datasets.load_lichess_puzzles_sync(cache_dir=tmp_path)
    assert [p["id"] for p in every] == ["p1", "p2", "p3"]
    p1 = every[0]
    assert p1["opponent_move"] == "g8e7" and p1["solution"] == ["f3f7"] and p1["rating"] == 600 and "mateIn1" in p1["themes"]
    assert p1["opening_tags"] == ["Italian_Game"] and every[1]["solution"] == ["e2e4", "d8c8", "e4e5"]
    assert [p["id"] for p in datasets.load_lichess_puzzles_sync(min_rating=1000, max_rating=2000, cache_dir=tmp_path)] == ["p2"]
    assert [p["id"] for p in datasets.load_lichess_puzzles_sync(themes=datasets.MATE_THEMES, cache_dir=tmp_path)] == ["p1"]
    assert [p["id"] for p in datasets.load_lichess_puzzles_sync(themes=["fork", "quietMove"], num_puzzles=1, cache_dir=tmp_path)] == ["p2"]
    fen = datasets.get_puzzle_fen_after_opponent_move(p1)
    assert fen.split()[0] == "r1bqkb1r/ppppnppp/2n5/4p3/2B1P3/5Q2/PPPP1PPP/RNB1K1NR" and fen.split()[1] == "w"
    traj = datasets.puzzle_to_trajectory(p1)
    assert "White to move" in traj.messages[1].text() and fen in traj.messages[1].text()
    # compressed copy, asynchronous entry point, and the message for an empty cache
    gz = tmp_path / "gz"
    gz.mkdir()
    with gzip.open(gz / "lichess_db_puzzle.csv.gz", "wt") as f:
        f.write(PUZZLES)
    assert len(asyncio.run(datasets.load_lichess_puzzles(num_puzzles=2, cache_dir=gz))) == 2
    with pytest.raises(FileNotFoundError, match="lichess_db_puzzle"):
        datasets.load_lichess_puzzles_sync(cache_dir=tmp_path / "empty")


def test_calculator_and_screenspot_loaders(tmp_path):
    with pytest.raises(FileNotFoundError):
        datasets.load_calc_smoke(tmp_path)
    (tmp_path / "problems.jsonl").write_text("\n".join(json.dumps(r) for r in datasets.builtin_calc_smoke()) + "\n")
    rows = datasets.load_calc_smoke(tmp_path)
    assert len(rows) == 8 and rows[0]["answer"] == 42
    t = datasets.calc_smoke_to_trajectory(rows[0])
    assert [m.role for m in t.messages] == ["system", "user"] and t.messages[1].text() == "What is 17 + 25?"
    (tmp_path / "problems.jsonl").write_text('{"question": "x"}\n')
    with pytest.raises(ValueError, match="answer"):
        datasets.load_calc_smoke(tmp_path)

    (tmp_path / "annotations").mkdir()
    (tmp_path / "images").mkdir()
    (tmp_path / "images" / "a.png").write_bytes(b"\x89PNG fake")
    ann = [{"img_filename": "a.png", "instruction": "click save", "bbox": [1, 2, 3, 4], "platform": "web", "application": "shop", "ui_type": "icon"},
           {"img_filename": "b.png", "instruction": "open menu", "bbox": [1, 2, 3, 4], "platform": "desktop", "application": "ide", "ui_type": "text"}]
    (tmp_path / "annotations" / "all.json").write_text(json.dumps(ann))
    assert len(datasets.load_screenspot(tmp_path, "all.json")) == 2
    web = datasets.load_screenspot(tmp_path, "all.json", platforms=["web"])
    assert len(web) == 1 and web[0]["image_path"].endswith("images/a.png")
    assert datasets.load_screenspot(tmp_path, "all.json", ui_types=["text"], limit=5)[0]["application"] == "ide"
    with pytest.raises(FileNotFoundError):
        datasets.load_screenspot(tmp_path, "none.json")
    with_image = datasets.screenspot_to_trajectory(web[0]).messages[1]
    assert len(with_image.content) == 2 and with_image.content[1].mime_type == "image/png" and "click save" in with_image.text()
    named = datasets.screenspot_to_trajectory(datasets.load_screenspot(tmp_path, "all.json", platforms=["desktop"])[0]).messages[1]
    assert len(named.content) == 1 and "b.png" in named.text()


# ------------------------------------------------------------------------------------------- remote machines, run logging
def test_remote_node_is_released_only_if_this_run_created_it():
    import argparse

    from research_b200.agents import remote
    from research_b200.infra.broker import GPUClient, GPUOffer, StaticProvider

    ok = lambda argv, data=None: (0, "ok\n", "")                                   # noqa: E731
    provider = StaticProvider("lab", [GPUOffer("lab", "m1", "B200", 8, 180, 30.0), GPUOffer("lab", "m2", "B200", 1, 180, 4.0)],
                              {"m1": "root@m1", "m2": "root@m2"})
    gc = GPUClient([provider])
    p = argparse.ArgumentParser()
    remote.add_remote_args(p)
    said = []
    # a machine the user named: nothing to release
    client, inst = remote.acquire_from_args(p.parse_args(["--ssh", "root@h:22"]), transport=ok)
    assert inst is None and not remote.release_node(client, inst, out=said.append) and not said
    # provisioned by this run: terminated on release, kept with --keep-alive
    client, inst = remote.acquire_from_args(p.parse_args(["--provision", "--gpu-count", "8"]), gpu_client=gc, transport=ok)
    assert inst.offer.offer_id == "m1" and len(provider.search()) == 1
    assert not remote.release_node(client, inst, keep_alive=True, out=said.append) and "stays up" in said[-1] and "root@m1" in said[-1]
    # an instance that already existed (picked by id) is not this run's to terminate
    again, same = remote.acquire_node(node_id=f"lab:{inst.instance_id}", gpu_client=gc, transport=ok)
    assert same is inst and not remote.release_node(again, same, out=said.append) and len(provider.search()) == 1
    assert remote.release_node(client, inst, out=said.append) and "terminated" in said[-1] and len(provider.search()) == 2
    with pytest.raises(ValueError):
        remote.acquire_node(ssh="a@b", provision=True)
    assert remote.get_broker_credentials({"RUNPOD_API_KEY": "r", "PRIME_API_KEY": "p", "OTHER": "x"}) == {"runpod": "r", "primeintellect": "p"}
    with pytest.raises(RuntimeError, match="credentials"):
        import os
        from unittest import mock

        with mock.patch.dict(os.environ, {}, clear=True):
            remote.acquire_node(provision=True)


def test_run_logging_makes_a_timestamped_folder_with_a_jsonl_log(tmp_path):
    import logging

    from research_b200.utils.logging_config import get_logger, init_run_logging

    root = logging.getLogger()
    before = list(root.handlers), root.level
    try:
        d = init_run_logging("my_eval", tmp_path, logger_levels={"httpx": "DEBUG"}, now=0.0)
        assert d == tmp_path / "my_eval_19700101-000000" and d.is_dir()
        assert logging.getLogger("paramiko").level == logging.WARNING and logging.getLogger("httpx").level == logging.DEBUG
        get_logger("test.run").warning("sample failed", extra={"sample_id": "s7"})
        for h in root.handlers:
            h.flush()
        rows = [json.loads(line) for line in (d / "error_log.jsonl").read_text().splitlines()]
        assert rows[-1]["message"] == "sample failed" and rows[-1]["sample_id"] == "s7" and "results directory" in rows[0]["message"]
    finally:
        for h in list(root.handlers):
            root.removeHandler(h)
            h.close()
        for h in before[0]:
            root.addHandler(h)
        root.setLevel(before[1])
        logging.getLogger("httpx").setLevel(logging.NOTSET)


# ------------------------------------------------------------------------------------------- OAuth log-in
def _oauth(tmp_path, answers, clock):
    from research_b200.agents import oauth

    app = oauth.OAuthApp("lab", "https://auth.example/authorize", "https://auth.example/token", "client-1", "https://auth.example/cb",
                         scopes="inference profile")
    sent = []

    async def transport(url, payload):
        sent.append((url, payload))
        return answers.pop(0)

    return oauth.OAuthClient(app, oauth.TokenStorage(tmp_path / "oauth" / "lab.json"), transport, clock=lambda: clock[0]), sent


def test_oauth_pkce_login_refresh_and_revocation(tmp_path):
    import base64
    import hashlib
    import stat
    from urllib.parse import parse_qs, urlparse

    from research_b200.agents import oauth

    clock = [1000.0]
    client, sent = _oauth(tmp_path, [(200, {"access_token": "at-1", "refresh_token": "rt-1", "expires_in": 3600}),
                                     (200, {"access_token": "at-2", "expires_in": 3600}), (401, "revoked")], clock)
    assert not client.is_logged_in() and asyncio.run(client.get_valid_access_token()) is None
    with pytest.raises(oauth.OAuthError, match="get_authorize_url"):
        asyncio.run(client.exchange_code("abc"))
    q = parse_qs(urlparse(client.get_authorize_url()).query)
    assert q["client_id"] == ["client-1"] and q["code_challenge_method"] == ["S256"] and q["scope"] == ["inference profile"]
    with pytest.raises(oauth.OAuthError, match="state mismatch"):
        asyncio.run(client.exchange_code("abc#someone-elses-state"))
    said = []

    async def ask(prompt):                                       # the user pastes what the page of the printed URL showed
        q.update(parse_qs(urlparse(said[0].split()[-1]).query))
        return f"  the-code#{q['state'][0]}\n"

    asyncio.run(oauth.login(client, ask, said.append))
    url, payload = sent[0]
    assert url.endswith("/token") and payload["grant_type"] == "authorization_code" and payload["code"] == "the-code"
    challenge = base64.urlsafe_b64encode(hashlib.sha256(payload["code_verifier"].encode()).digest()).rstrip(b"=").decode()
    assert q["code_challenge"] == [challenge] and payload["code_verifier"] != q["state"][0]
    path = tmp_path / "oauth" / "lab.json"
    assert stat.S_IMODE(path.stat().st_mode) == 0o600 and "at-1" in path.read_text() and str(path) in said[-1]
    # valid until three minutes before the hour is up; then one refresh that keeps the old refresh token
    clock[0] = 1000.0 + 3600 - 181
    assert asyncio.run(client.get_valid_access_token()) == "at-1" and len(sent) == 1
    clock[0] += 2
    assert asyncio.run(client.get_valid_access_token()) == "at-2" and sent[1][1] == {"grant_type": "refresh_token", "refresh_token": "rt-1", "client_id": "client-1"}
    fresh, _ = _oauth(tmp_path, [], clock)                       # another process reads the same file
    assert fresh.tokens.access_token == "at-2" and fresh.tokens.refresh_token == "rt-1"
    # a refused refresh forgets the log-in
    clock[0] += 4000
    assert asyncio.run(client.get_valid_access_token()) is None and not path.exists() and not client.is_logged_in()


def test_auth_report_and_endpoint_credentials(tmp_path, monkeypatch):
    from research_b200.agents import oauth
    from research_b200.cli import build_parser, _endpoint

    clock = [0.0]
    client, _ = _oauth(tmp_path, [], clock)
    using, lines = oauth.auth_report("hosted", "HOSTED_KEY", client, env={"HOSTED_KEY": "sk-abcdefghijkl"}, now=0.0)
    assert using == "api_key" and "sk-abcde…" in lines[0] and "ghijkl" not in "\n".join(lines)
    assert oauth.auth_report("hosted", "HOSTED_KEY", None, env={})[0] == "none"
    client.storage.save(oauth.OAuthTokens("token-abcdefgh-secret", "rt", 600.0))
    using, lines = oauth.auth_report("hosted", "HOSTED_KEY", client, env={"HOSTED_KEY": "sk-abcdefghijkl"}, now=0.0)
    assert using == "oauth" and "10 more minutes" in lines[1] and "NOT used" in lines[2] and "secret" not in "\n".join(lines)
    # the command line: --oauth NAME reads the application from the environment and the token from the user's folder
    monkeypatch.setattr(oauth, "DEFAULT_DIR", tmp_path / "home")
    for k, v in {"AUTHORIZE_URL": "https://a/x", "TOKEN_URL": "https://a/t", "CLIENT_ID": "c", "REDIRECT_URI": "https://a/cb"}.items():
        monkeypatch.setenv(f"RB_OAUTH_LAB_{k}", v)
    monkeypatch.setenv("HOSTED_KEY", "sk-from-env")
    args = build_parser().parse_args(["chat", "--provider", "anthropic", "--model", "m", "--oauth", "lab", "--api-key-env", "HOSTED_KEY"])
    with pytest.raises(SystemExit, match="not logged in"):
        _endpoint(args)
    import time

    oauth.TokenStorage(tmp_path / "home" / "lab.json").save(oauth.OAuthTokens("at-live", "rt", time.time() + 3600))
    import research_b200.agents.oauth as om

    real = om.OAuthClient

    def client_in_tmp(app, storage=None, **kw):
        return real(app, storage or om.TokenStorage(tmp_path / "home" / f"{app.name}.json"), **kw)

    monkeypatch.setattr(om, "OAuthClient", client_in_tmp)
    ep = _endpoint(args)
    assert ep.oauth_token == "at-live" and ep.api_key == "" and "oauth_token" not in ep.to_dict()
    with pytest.raises(oauth.OAuthError, match="not configured"):
        oauth.OAuthApp.load("other", tmp_path / "home", env={})


def test_read_of_an_image_reaches_the_model_as_an_image_block(tmp_path):
    """An image file read by the coding environment becomes text + image content of the tool message, and both wire
    formats carry it: inside the tool result for Anthropic, as a following user message for chat completions."""
    import asyncio
    import base64

    from research_b200.agents.agents import process_pending_tools
    from research_b200.agents.dtypes import Actor, AgentState, Endpoint, ImageContent, Message, RunConfig, ToolCall, Trajectory
    from research_b200.agents.environments.coding import LocalFilesystemEnvironment
    from research_b200.agents.providers.chat import messages_to_openai
    from research_b200.agents.providers.streaming import messages_to_anthropic

    png = b"\x89PNG\r\n\x1a\n" + b"\0" * 32
    (tmp_path / "shot.png").write_bytes(png)
    env = LocalFilesystemEnvironment(tmp_path)
    call = ToolCall("c1", "read", {"path": "shot.png"})
    actor = Actor(Trajectory((Message("user", "look"), Message("assistant", "", tool_calls=(call,)))), Endpoint("mock", "m"))
    state = AgentState(actor, env, pending_tool_calls=(call,))
    events = []

    async def on_chunk(e):
        events.append(e)

    new = asyncio.run(process_pending_tools(state, RunConfig(on_chunk=on_chunk)))
    tool_msg = new.actor.trajectory.messages[-1]
    assert tool_msg.role == "tool" and isinstance(tool_msg.content, list)
    image = [b for b in tool_msg.content if isinstance(b, ImageContent)][0]
    assert base64.b64decode(image.data) == png and image.mime_type == "image/png"
    assert "shot.png" in tool_msg.text()
    assert all("image" not in getattr(e, "details", {}) for e in events)         # the event stream does not carry the bytes

    _, wire = messages_to_anthropic(new.actor.trajectory.messages)
    result_block = wire[-1]["content"][0]
    assert result_block["type"] == "tool_result" and result_block["content"][-1]["type"] == "image"
    chat = messages_to_openai(new.actor)
    assert chat[-2]["role"] == "tool" and chat[-1]["role"] == "user"
    assert chat[-1]["content"][-1]["image_url"]["url"].startswith("data:image/png;base64,")


def test_diff_lines_are_coloured_and_tabs_expanded():
    from research_b200.agents.environments.coding import _first_lines
    from research_b200.frontend.terminal import Theme, colour_diff_line

    assert colour_diff_line("+new").startswith(Theme.CODE) and colour_diff_line("  -old").startswith(Theme.ERROR)
    assert colour_diff_line(" same") == " same" and colour_diff_line("@@ -1 +1 @@").startswith(Theme.DIM)
    assert "\t" not in _first_lines("a\tb\n\tc", 5)
