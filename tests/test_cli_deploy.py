"""CLI plumbing and deploy helpers, offline."""

import asyncio
import json

import pytest

from research_b200 import cli
from research_b200.agents.dtypes import Message
from research_b200.agents.presets import PRESETS, get_preset
from research_b200.agents.providers import ScriptedLLM, register_provider
from research_b200.agents.store import FileSessionStore
from research_b200.deploy import (ServerConfig, build_command, build_native_command, build_sglang_command, preflight,
                                  wait_until_healthy)


def test_server_commands():
    with pytest.raises(ValueError):
        ServerConfig(tensor_parallel_size=2)
    c = ServerConfig(model="Qwen/Qwen2.5-0.5B", engine="sglang", gpu_ranks=[2, 3], tensor_parallel_size=2, max_model_len=4096,
                     attention_backend="triton")
    cmd = build_sglang_command(c)
    assert "--tp 2" in cmd and "--context-length 4096" in cmd and "--enable-radix-cache" in cmd and "--attention-backend triton" in cmd
    assert "; CUDA_VISIBLE_DEVICES=2,3 python -m sglang.launch_server" in build_command(c)
    assert build_command(ServerConfig(gpu_ranks=[1])).startswith("CUDA_VISIBLE_DEVICES=1 ")
    n = build_native_command(ServerConfig(model="llama-3-8b", gpu_ranks=[0, 1], tensor_parallel_size=2, port=31000))
    assert "torch.distributed.run" in n and "--nproc-per-node 2" in n and "--master-addr 127.0.0.1" in n and "--tp 2" in n
    assert "research_b200.cli serve" in build_native_command(ServerConfig())


def test_preflight_and_health_with_fakes():
    def run(cmd):
        if cmd.startswith("nvidia-smi"):
            return 0, "0, 12\n1, 90000\n"
        if "ss -ltn" in cmd:
            return 0, "taken"
        return 1, "no module"

    problems = preflight(ServerConfig(engine="sglang", gpu_ranks=[1, 2], tensor_parallel_size=2), run)
    assert any("GPU 1 is busy" in p for p in problems) and any("GPU 2 does not exist" in p for p in problems)
    assert any("port" in p for p in problems) and any("sglang" in p for p in problems)
    assert preflight(ServerConfig(), lambda c: (0, "0, 3\n") if c.startswith("nvidia-smi") else (0, "free")) == []
    calls = []
    assert wait_until_healthy("http://x", timeout=5, poll=0.01, probe=lambda u: calls.append(u) or len(calls) >= 3)
    assert not wait_until_healthy("http://x", timeout=5, poll=0.01, probe=lambda u: False, alive=lambda: False)


def test_presets_build_environments(tmp_path):
    for name in PRESETS:
        env = get_preset(name).environment(str(tmp_path))
        assert hasattr(env, "get_tools") and hasattr(env, "exec_tool")
    with pytest.raises(KeyError):
        get_preset("nope")


def test_cli_chat_sessions_eval(tmp_path, capsys):
    register_provider("cli-mock", ScriptedLLM(["hello from the model"]))
    store_dir = str(tmp_path / "sessions")
    assert cli.main(["chat", "--provider", "cli-mock", "--store", store_dir, "-p", "hi"]) == 0
    assert "hello from the model" in capsys.readouterr().out
    sid = asyncio.run(FileSessionStore(store_dir).list())[0].session_id
    assert cli.main(["sessions", "list", "--store", store_dir]) == 0 and sid in capsys.readouterr().out
    assert cli.main(["sessions", "show", sid, "--store", store_dir]) == 0 and "hello from the model" in capsys.readouterr().out
    assert cli.main(["sessions", "slice", sid, "--spec", "0:2", "--store", store_dir]) == 0
    ds = tmp_path / "d.jsonl"
    ds.write_text("\n".join(json.dumps({"prompt": f"q{i}", "answer": "hello"}) for i in range(3)))
    score = tmp_path / "score.py"
    score.write_text("def score(traj, row):\n    return 1.0 if row['answer'] in traj.messages[-1].text() else 0.0\n")
    assert cli.main(["eval", "--provider", "cli-mock", "--dataset", str(ds), "--score-fn", f"{score}:score",
                     "--output-dir", str(tmp_path / "out")]) == 0
    out = capsys.readouterr().out
    assert json.loads(out[out.index("{"):])["mean_reward"] == 1.0
    assert isinstance(cli.load_object("research_b200.agents.dtypes:Message")("user", "x"), Message)


def test_session_frontend(tmp_path):
    from fastapi.testclient import TestClient

    from research_b200.frontend.server import create_app

    store = FileSessionStore(tmp_path)

    async def seed():
        sid = await store.create({"provider": "front-mock", "model": "m"})
        await store.append_message(sid, Message("user", "first <question>"))
        await store.append_message(sid, Message("assistant", "first answer"))
        return sid

    sid = asyncio.run(seed())
    client = TestClient(create_app(store, rollout_override=ScriptedLLM(["second answer"])))
    assert sid in client.get("/").text
    page = client.get(f"/session/{sid}").text
    assert "first answer" in page and "&lt;question&gt;" in page
    assert client.get("/session/nope").status_code == 404
    assert client.get("/api/sessions").json()[0]["id"] == sid
    r = client.post(f"/api/session/{sid}/message", json={"content": "and then?"}).json()
    assert r["content"] == "second answer"
    msgs = client.get(f"/api/session/{sid}").json()["messages"]
    assert [m["role"] for m in msgs] == ["user", "assistant", "user", "assistant"]
    assert client.post(f"/api/session/{sid}/message", json={"content": " "}).status_code == 400


def test_session_doctor_and_chat_flags(tmp_path, capsys):
    """Duplicate / orphaned tool results are found and dropped into a child session, trimming writes another child,
    `chat --continue` resumes the latest session, `--no-session` stores nothing, `--context` reaches the system prompt."""
    from research_b200.agents import ToolCall
    from research_b200.agents import doctor

    store_dir = str(tmp_path / "sessions")
    store = FileSessionStore(store_dir)

    async def build():
        sid = await store.create({"provider": "cli-mock", "model": "m"})
        call = ToolCall("call_1", "add", {"value": 2})
        msgs = [Message("user", "add two"), Message("assistant", "", tool_calls=(call,)),
                Message("tool", "2", tool_call_id="call_1"), Message("tool", "2", tool_call_id="call_1"),
                Message("tool", "lost", tool_call_id="call_gone"), Message("assistant", "done"), Message("user", "x" * 120_000)]
        for m in msgs:
            await store.append_message(sid, m)
        return sid

    sid = asyncio.run(build())
    _, msgs = asyncio.run(store.get(sid))
    kinds = sorted(i.kind for i in doctor.diagnose(msgs))
    assert kinds == ["duplicate_tool_result", "orphaned_tool_result", "oversized_message"]
    assert cli.main(["sessions", "doctor", sid, "--store", store_dir, "--fix"]) == 0
    out = capsys.readouterr().out
    assert "duplicate_tool_result" in out and "created fixed session" in out
    children = [s for s in asyncio.run(store.list()) if s.parent_id == sid]
    assert len(children) == 1 and children[0].tags["doctor"] == "fixed" and children[0].num_messages == 5
    assert [i.kind for i in doctor.diagnose(asyncio.run(store.get(children[0].session_id))[1])] == ["oversized_message"]
    assert cli.main(["sessions", "doctor", sid, "--store", store_dir, "--trim", "1"]) == 0
    trimmed = [s for s in asyncio.run(store.list()) if s.tags.get("doctor") == "trimmed"]
    assert len(trimmed) == 1 and trimmed[0].num_messages == 6
    assert cli.main(["sessions", "doctor", sid, "--store", store_dir, "--trim", "99"]) == 1
    capsys.readouterr()
    assert cli.main(["sessions", "handoff", sid, "--store", store_dir, "--goal", "finish the sum"]) == 0
    assert "finish the sum" in capsys.readouterr().out
    # an unanswered tool call followed by more conversation is reported but not auto-fixed
    broken = [Message("user", "q"), Message("assistant", "", tool_calls=(ToolCall("c9", "add", {}),)), Message("user", "still there?")]
    (issue,) = doctor.diagnose(broken)
    assert issue.kind == "unanswered_tool_call" and not issue.fixable
    assert doctor.format_time_ago(0, now=30) == "just now" and doctor.format_time_ago(0, now=7200) == "2h ago" and doctor.format_time_ago(0, now=3 * 86400) == "3d ago"
    assert cli.parse_model_string("anthropic/claude-x") == ("anthropic", "claude-x")
    with pytest.raises(ValueError):
        cli.parse_model_string("claude-x")

    # chat flags
    class Echo:
        """Replies with the system prompt it was given, so the test can see what reached the model."""

        async def __call__(self, actor, run_config):
            sys_text = " | ".join(m.text() for m in actor.trajectory.messages if m.role == "system")
            return await ScriptedLLM([f"system was: {sys_text}"])(actor, run_config)

    register_provider("cli-mock", Echo())
    ctx = tmp_path / "notes.txt"
    ctx.write_text("the deadline is friday")
    store2 = str(tmp_path / "s2")
    assert cli.main(["chat", "--model", "cli-mock/any", "--store", store2, "-p", "hi", "--system-prompt", "be terse",
                     "--context", "user likes tables", "--context-file", str(ctx), "-q"]) == 0
    out = capsys.readouterr().out
    assert "be terse" in out and "user likes tables" in out and "the deadline is friday" in out
    first = asyncio.run(FileSessionStore(store2).list())
    assert len(first) == 1
    assert cli.main(["chat", "--provider", "cli-mock", "--store", store2, "-p", "again", "--continue"]) == 0
    after = asyncio.run(FileSessionStore(store2).list())
    assert len(after) == 1 and after[0].num_messages > first[0].num_messages
    assert cli.main(["chat", "--provider", "cli-mock", "--store", str(tmp_path / "s3"), "-p", "hi", "--no-session"]) == 0
    assert not (tmp_path / "s3").exists() or not list((tmp_path / "s3").iterdir())

    # the question on standard input, and a fork of the stored conversation from the command line
    import io
    import sys

    monkey_stdin, sys.stdin = sys.stdin, io.StringIO("piped question\n")
    try:
        assert cli.main(["chat", "--provider", "cli-mock", "--store", store2, "-p", "-", "--continue", "--branch", "2"]) == 0
        sys.stdin = io.StringIO("")
        assert cli.main(["chat", "--provider", "cli-mock", "--store", store2, "-p", "-", "--no-session"]) == 2
    finally:
        sys.stdin = monkey_stdin
    sessions = asyncio.run(FileSessionStore(store2).list())
    assert len(sessions) == 2
    fork = next(x for x in sessions if x.parent_id)
    assert fork.branch_point == 2 and fork.tags.get("branch_reason") == "command_line"
    _, fork_msgs = asyncio.run(FileSessionStore(store2).get(fork.session_id))
    assert any(m.role == "user" and m.text() == "piped question" for m in fork_msgs)
    assert cli.main(["chat", "--provider", "cli-mock", "--store", store2, "-p", "x", "--continue", "--branch", "99"]) == 2


def test_bootstrap_model_access_and_endpoint(tmp_path):
    from research_b200.deploy import ServerInfo, check_model_access, generate_bootstrap_command, server_info_to_endpoint

    sg = generate_bootstrap_command(ServerConfig(engine="sglang"))
    assert "uv venv .venv-sglang" in sg and "sglang[all]" in sg and sg.index("uv venv") < sg.index("uv pip install")
    native = generate_bootstrap_command(ServerConfig(), workdir="/srv/my checkout")
    assert native.startswith("cd '/srv/my checkout' && ") and "research_b200.cli build" in native
    assert ".venv-sglang/bin/activate" in build_command(ServerConfig(engine="sglang")) and ".venv-sglang" not in build_command(ServerConfig())
    seen = []

    def hub(status):
        def get(url, headers):
            seen.append((url, headers))
            if status is None:
                raise OSError("no route to host")
            return status
        return get

    assert check_model_access(str(tmp_path)) == (True, None) and check_model_access("qwen2.5-0.5b") == (True, None)       # local dir, preset
    assert "HF_TOKEN is not set" in check_model_access("org/model", env={})[1]
    assert "neither" in check_model_access("just-a-name", env={"HF_TOKEN": "t"})[1]
    assert check_model_access("org/model", env={"HF_TOKEN": "tok"}, get=hub(200)) == (True, None)
    assert seen[0] == ("https://huggingface.co/api/models/org/model", {"Authorization": "Bearer tok"})
    for status, word in ((401, "invalid or expired"), (403, "licence"), (404, "not found"), (500, "HTTP 500")):
        ok, why = check_model_access("org/model", env={"HF_TOKEN": "tok"}, get=hub(status))
        assert not ok and word in why
    ok, why = check_model_access("org/model", env={"HF_TOKEN": "tok"}, get=hub(None))
    assert ok and "could not verify" in why
    ep = server_info_to_endpoint(ServerInfo("http://10.0.0.5:30000", 1, "log", "cmd"), "org/model", engine="sglang", temperature=0.2)
    assert (ep.provider, ep.api_base, ep.model, ep.temperature) == ("sglang", "http://10.0.0.5:30000", "org/model", 0.2)


def test_chat_full_prompt_names_the_tools_and_project_context(tmp_path, capsys):
    from research_b200.agents.providers import register_provider

    seen = {}

    async def model(actor, run_config):
        seen["system"] = actor.trajectory.messages[0].text()
        return await ScriptedLLM(["ok"])(actor, run_config)

    register_provider("prompt-mock", model)
    (tmp_path / "AGENTS.md").write_text("always run the linter")
    assert cli.main(["chat", "--provider", "prompt-mock", "--model", "scripted", "--preset", "explorer", "--cwd", str(tmp_path), "--no-session", "--full-prompt", "-q", "-p", "hi"]) == 0
    s = seen["system"]
    assert s.startswith("You are a careful software engineer") and "- grep: search file contents" in s and "READ-ONLY mode" in s
    assert "always run the linter" in s and str(tmp_path) in s and "Working as an explorer" in s
