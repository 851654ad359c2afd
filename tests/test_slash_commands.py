"""Slash commands of the interactive chat: file commands with arguments, thinking budgets, slicing, environment switch."""

import asyncio
import io

import pytest

from research_b200.agents.dtypes import Endpoint, Message
from research_b200.agents.providers import ScriptedLLM, register_provider
from research_b200.agents.store import FileSessionStore
from research_b200.frontend import slash_commands as sc
from research_b200.frontend.terminal import InteractiveRunner, PlainFrontend


def test_file_commands_front_matter_arguments_and_precedence(tmp_path):
    home, proj = tmp_path / "home", tmp_path / "proj"
    (home / ".research_b200" / "commands" / "git").mkdir(parents=True)
    (proj / ".research_b200" / "commands").mkdir(parents=True)
    (home / ".research_b200" / "commands" / "review.md").write_text("---\ndescription: Review a file\nargument-hint: <file> [focus]\n---\nReview $1 with a focus on $2.\nAll: $@\n")
    (home / ".research_b200" / "commands" / "git" / "pr.md").write_text("# Describe the pull request\nSummarise the diff of $ARGUMENTS.\n")
    (proj / ".research_b200" / "commands" / "review.md").write_text("Project review of $1 ($3).\n")
    cmds = sc.load_file_commands(proj, home)
    by = {c.name: c for c in cmds}
    assert set(by) == {"review", "git:pr"} and by["review"].source == "(project)" and by["git:pr"].description == "Describe the pull request"
    user_only = {c.name: c for c in sc.load_file_commands(tmp_path / "elsewhere", home)}
    assert user_only["review"].arg_hint == "<file> [focus]" and user_only["review"].description == "Review a file"
    assert sc.expand_file_command('/review "my file.py" errors', list(user_only.values())) == "Review my file.py with a focus on errors.\nAll: my file.py errors"
    assert sc.expand_file_command("/review a.py", cmds) == "Project review of a.py ()." and sc.expand_file_command("/nope x", cmds) is None
    assert sc.parse_command_args("""a 'b c' "" d""") == ["a", "b c", "", "d"] and sc.parse_frontmatter("no front matter") == ({}, "no front matter")
    assert sc.find_similar_command("modle", ["model", "env"]) == "model" and sc.find_similar_command("th", ["thinking"]) == "thinking"
    assert sc.get_command_arg_hint("slice", sc.BUILTIN_COMMANDS).startswith("[0:5")


def test_runner_commands_thinking_slice_env_and_file_prompt(tmp_path):
    store = FileSessionStore(tmp_path / "sessions")
    seen = []

    async def model(actor, run_config):
        seen.append(actor)
        return await ScriptedLLM([f"reply {len(seen)}"])(actor, run_config)

    register_provider("slash-mock", model)
    lines = iter(["first question", "second question", "/thinking", "/thinking 8000", "/thinking off", "/thinking 12", "/slice", "/slice 0:1, summarize:1:4",
                  "/env calculator", "/env", "/env nope", "/modle x", "/explain the scheduler", "/commands", "/quit"])
    out = io.StringIO()

    class Scripted(PlainFrontend):
        async def get_input(self, prompt=""):
            return next(lines)

    fe = Scripted(out=out)
    cmds = [sc.SlashCommand("explain", "explain something", "<what>", "Explain $@ in two sentences.", "(project)")]
    runner = InteractiveRunner(Endpoint(provider="slash-mock", model="m"), fe, system_prompt="be brief", session_store=store, cwd=str(tmp_path),
                               file_commands=cmds)
    state = asyncio.run(runner.run())
    text = out.getvalue()
    assert "thinking: off" in text and "thinking on, budget 8000 tokens" in text and "thinking off" in text and "usage: /thinking" in text
    assert "5 messages. usage: /slice" in text and "5 -> 2 messages; now in session" in text
    assert "environment: calculator (tools: add" in text and "unknown environment(s) ['nope']" in text and "did you mean /model?" in text
    assert "explain something  (project)" in text and "/explain <what> " in text and "/slice [0:5" in text
    # the file command reached the model as a user message, on the sliced conversation, with the calculator's tools
    last = seen[-1]
    assert last.trajectory.messages[-1].text() == "Explain the scheduler in two sentences." and "add" in [t.function.name for t in last.tools]
    assert [m.role for m in last.trajectory.messages] == ["system", "user", "user"] and "[Summary of messages 1-3]" in last.trajectory.messages[1].text()
    assert state.actor.trajectory.messages[-1].text() == "reply 3"
    # the slice made a child session that records its origin; the thinking choice and the environment were stored as tags

    async def check():
        sessions = {s.session_id: s for s in await store.list()}
        sliced = next(s for s in sessions.values() if "slice" in s.tags and "env" not in s.tags)
        assert sliced.tags["slice"] == "0:1, summarize:1:4" and sliced.branch_point == 5 and sessions[sliced.parent_id].tags["thinking"] == "off"
        # switching the environment branched once more: the child carries the new tools, its parent stays as it was
        swapped = next(s for s in sessions.values() if s.parent_id == sliced.session_id)
        assert swapped.tags["env"] == "calculator" and swapped.environment is not None and swapped.branch_point == 2
        assert [m.text() for m in (await store.get(swapped.session_id))[1]][-2:] == ["Explain the scheduler in two sentences.", "reply 3"]
        assert len((await store.get(sliced.session_id))[1]) == 2

    asyncio.run(check())
    ep = runner.endpoint
    assert "thinking" not in ep.extra_params and ep.reasoning_effort is None
    sc.handle_thinking(runner, "20000")
    assert sc.thinking_budget(runner.endpoint) == 20000 and runner.endpoint.reasoning_effort == "high" and runner.endpoint.max_tokens >= 21024


def test_session_switch_and_branch(tmp_path):
    store = FileSessionStore(tmp_path / "sessions")

    async def seed():
        sid = await store.create({"provider": "slash-mock", "model": "older-model", "temperature": 0.3})
        for m in (Message("user", "earlier question"), Message("assistant", "earlier answer")):
            await store.append_message(sid, m)
        return sid

    old = asyncio.run(seed())
    seen = []

    async def model(actor, run_config):
        seen.append(actor)
        return await ScriptedLLM([f"reply {len(seen)}"])(actor, run_config)

    register_provider("slash-mock", model)
    lines = iter(["hello", "/session", f"/session {old[:8]}", f"/session {old}", "and now?", "/branch 2", "different follow-up", "/session nope", "/quit"])
    out = io.StringIO()

    class Scripted(PlainFrontend):
        async def get_input(self, prompt=""):
            return next(lines)

    runner = InteractiveRunner(Endpoint(provider="slash-mock", model="m"), Scripted(out=out), session_store=store, cwd=str(tmp_path), file_commands=[])
    asyncio.run(runner.run())
    text = out.getvalue()
    assert f"now in session {old} (2 messages, model older-model)" in text and "0 sessions match 'nope'" in text and old in text.split("now in session")[0]
    assert f"2 sessions match '{old[:8]}'" in text                     # a prefix that two sessions share switches nothing
    # after the switch the model saw the old conversation with the stored model and temperature
    after_switch = seen[1]
    assert [m.text() for m in after_switch.trajectory.messages] == ["earlier question", "earlier answer", "and now?"]
    assert after_switch.endpoint.model == "older-model" and after_switch.endpoint.temperature == 0.3
    # the branch kept two messages, continued in a child session, and left the old session as it was
    assert [m.text() for m in seen[2].trajectory.messages] == ["earlier question", "earlier answer", "different follow-up"]

    async def check():
        sessions = {s.session_id: s for s in await store.list()}
        child = next(s for s in sessions.values() if s.parent_id == old)
        assert child.branch_point == 2 and [m.text() for m in (await store.get(child.session_id))[1]][-2:] == ["different follow-up", "reply 3"]
        assert [m.text() for m in (await store.get(old))[1]] == ["earlier question", "earlier answer", "and now?", "reply 2"]

    asyncio.run(check())


def test_environment_specs_compose_and_cli_env_flag(tmp_path):
    from research_b200 import cli
    from research_b200.agents.presets import environment_from_spec

    env = environment_from_spec("coding+ask_user+calculator", str(tmp_path), "readonly")
    names = [t.function.name for t in env.get_tools()]
    assert names[:4] == ["read", "list", "glob", "grep"] and "ask_user_question" in names and "add" in names and env.get_name() == "coding+ask_user+calculator"
    assert type(environment_from_spec("calculator")).__name__ == "CalculatorEnvironment"
    for bad in ("coding+nope", "", "coding+coding"):
        with pytest.raises(KeyError):
            environment_from_spec(bad, str(tmp_path))
    seen = {}

    async def model(actor, run_config):
        seen["tools"] = [t.function.name for t in actor.tools]
        return await ScriptedLLM(["ok"])(actor, run_config)

    register_provider("env-mock", model)
    assert cli.main(["chat", "--provider", "env-mock", "--model", "m", "--env", "calculator+ask_user", "--no-session", "-q", "-p", "hi", "--cwd", str(tmp_path)]) == 0
    assert "add" in seen["tools"] and "ask_user_question" in seen["tools"]
    with pytest.raises(KeyError):
        cli.main(["chat", "--provider", "env-mock", "--model", "m", "--env", "calculator+typo", "--no-session", "-q", "-p", "hi"])


def test_edit_branches_before_the_message_and_tree_shows_the_family(tmp_path):
    """`/edit` forks the stored conversation just before the reworded message and hands the new wording back to be sent;
    the store can also write the reworded message itself; `/tree` draws parent and children with fork points."""
    import asyncio
    import io

    from research_b200.agents.dtypes import Endpoint, Message
    from research_b200.agents.store import FileSessionStore, format_session_tree
    from research_b200.frontend.slash_commands import handle_edit, handle_tree
    from research_b200.frontend.terminal import InteractiveRunner, PlainFrontend

    async def go():
        store = FileSessionStore(tmp_path)
        ep = Endpoint("mock", "m")
        root = await store.create(ep.to_dict())
        history = [Message("user", "first question"), Message("assistant", "first answer"), Message("user", "secnod question"),
                   Message("assistant", "second answer")]
        for m in history:
            await store.append_message(root, m)
        from research_b200.agents.dtypes import Trajectory

        runner = InteractiveRunner(ep, PlainFrontend(out=io.StringIO()), session_store=store, session_id=root, trajectory=Trajectory(tuple(history)))
        res = await handle_edit(runner, "second question")
        assert res.expanded_text == "second question" and "reworded message 2" in res.message
        child = runner.state.session_id
        assert child != root and [m.text() for m in runner.state.actor.trajectory.messages] == ["first question", "first answer"]
        session, msgs = await store.get(child)
        assert session.parent_id == root and session.branch_point == 2 and session.tags["branch_reason"] == "message_edit" and len(msgs) == 2

        assert "not a user message" in (await handle_edit(runner, "1 nope")).message
        assert "usage" in (await handle_edit(runner, "")).message

        other = await store.branch_with_edit(root, 0, "a different first question")
        _, msgs = await store.get(other)
        assert [m.text() for m in msgs] == ["a different first question"]
        import pytest

        with pytest.raises(ValueError):
            await store.branch_with_edit(root, 1, "cannot reword the model")
        grandchild = await store.branch(child, 1, reason="exploration")

        assert await store.root_of(grandchild) == root
        tree = await store.tree(root)
        assert {c["session"].session_id for c in tree["children"]} == {child, other}
        text = format_session_tree(tree, current=child)
        lines = text.splitlines()
        assert lines[0].startswith(root) and any(child in ln and "@2 (message_edit)" in ln and ln.rstrip().endswith("*") for ln in lines)
        assert any(grandchild in ln and "(exploration)" in ln and ln.startswith(("|   ", "    ")) for ln in lines)
        assert (await handle_tree(runner, "")).message == text
    asyncio.run(go())


def test_sessions_tree_command(tmp_path, capsys):
    import asyncio

    from research_b200.agents.dtypes import Endpoint, Message
    from research_b200.agents.store import FileSessionStore
    from research_b200.cli import main

    store = FileSessionStore(tmp_path)
    root = asyncio.run(store.create(Endpoint("mock", "m").to_dict()))
    asyncio.run(store.append_message(root, Message("user", "q")))
    kid = asyncio.run(store.branch(root, 1))
    assert main(["sessions", "tree", kid, "--store", str(tmp_path)]) == 0
    out = capsys.readouterr().out
    assert out.splitlines()[0].startswith(root) and f"`-- {kid} @1" in out and out.rstrip().endswith("*")
