"""The evaluation dev loop: configs read without being executed, dataset previews, generated configs, child-process runs
that are followed and stopped, results read back; and the same through the HTTP routes."""

import json
import sys
import time

import pytest

from research_b200.frontend.devloop import DevLoop, RunRegistry, describe_config, generate_config, match_score, preview_dataset

MOCK_CONFIG = '''"""Two arithmetic questions against a scripted model."""
from research_b200.agents.dtypes import Message, Trajectory
from research_b200.agents.providers import ScriptedLLM, register_provider
from types import SimpleNamespace

register_provider("devloop-mock", ScriptedLLM(["4", "6"]))
TOOLS = [{"name": "add", "description": "add two numbers", "parameters": {"type": "object"}}]
config = SimpleNamespace(
    experiment_name="arith", provider="devloop-mock", model_name="scripted", api_base="", max_turns=1, max_concurrent=1,
    save_dir="results", show_progress=False, dataset_path="data/arith.jsonl",
    rows=[{"q": "2+2", "a": "4"}, {"q": "3+3", "a": "6"}], environment=None,
    to_trajectory=lambda row: Trajectory((Message("user", row["q"]),)),
    score_fn=lambda traj, row: float(row["a"] in traj.messages[-1].text()))
'''


@pytest.fixture
def project(tmp_path):
    (tmp_path / "configs").mkdir()
    (tmp_path / "data").mkdir()
    (tmp_path / "configs" / "01_arith.py").write_text(MOCK_CONFIG)
    (tmp_path / "configs" / "_private.py").write_text("x = 1\n")
    (tmp_path / "data" / "arith.jsonl").write_text("\n".join(json.dumps({"q": f"{i}+{i}", "a": str(2 * i)}) for i in range(1, 8)) + "\n")
    (tmp_path / "data" / "t.csv").write_text("question,answer\nwhat,42\nwho,me\n")
    (tmp_path / "data" / "w.json").write_text(json.dumps({"version": 1, "data": [1, 2, 3]}))
    return tmp_path


def test_configs_are_described_from_syntax_not_by_running_them(project):
    dev = DevLoop(project)
    assert [c["name"] for c in dev.list_configs()] == ["01_arith"]
    c = dev.load_config("01_arith")
    assert c["doc"].startswith("Two arithmetic") and c["fields"]["config.provider"] == "devloop-mock" and c["fields"]["config.max_turns"] == 1
    assert c["fields"]["config.to_trajectory"].startswith("lambda row") and c["tools"][0]["name"] == "add"
    from research_b200.agents.providers import NonRetryableError, get_provider

    with pytest.raises(NonRetryableError):
        get_provider("devloop-mock")                      # describing the file did not execute its register_provider call
    assert describe_config("class C:\n    lr: float = 3e-4\ndef f(): pass\n") == {
        "doc": "", "fields": {"C.lr": 3e-4}, "functions": ["f"], "classes": ["C"], "tools": []}
    (project / "configs" / "02_broken.py").write_text("def (:\n")
    assert "syntax error at line 1" in dev.load_config("02_broken")["error"]
    for bad in ("../escape", "/etc/passwd", "sub/../../x"):
        with pytest.raises(ValueError):
            dev.load_config(bad)
    with pytest.raises(FileNotFoundError):
        dev.load_config("01_arith.txt")
    assert dev.dataset_preview_for_config("01_arith", n=2)["total_rows"] == 7


def test_dataset_previews(project):
    p = preview_dataset(project / "data" / "arith.jsonl", n=3)
    assert p["total_rows"] == 7 and len(p["rows"]) == 3 and p["fields"] == ["q", "a"]
    assert preview_dataset(project / "data" / "t.csv")["rows"][1] == {"question": "who", "answer": "me"}
    assert preview_dataset(project / "data" / "w.json")["rows"] == [{"value": 1}, {"value": 2}, {"value": 3}]
    dev = DevLoop(project)
    assert {d["path"] for d in dev.list_datasets()} == {"data/arith.jsonl", "data/t.csv", "data/w.json"}
    with pytest.raises(ValueError):
        dev.preview("../outside.jsonl")
    models = dev.list_models()
    assert models and all(isinstance(v, list) and v for v in models.values())


def test_generated_config_loads_and_quotes_every_field(project):
    from research_b200.agents.dtypes import Message, Trajectory
    from research_b200.run_eval import endpoint_from_config, load_config_from_file

    dev = DevLoop(project)
    nasty = 'be brief"""\nimport os; os.system("true")  # \\'
    saved = dev.save_config({"experiment_name": "my eval!", "provider": "openai", "model_name": "gpt-4o-mini", "api_base": "http://x/v1",
                             "dataset_path": str(project / "data" / "t.csv"), "num_samples": 1, "prompt_field": "question",
                             "answer_field": "answer", "system_prompt": nasty, "user_template": "Q: {question}", "max_turns": 2})
    assert saved["name"] == "02_my_eval" and dev.next_config_name("x") == "03_x"
    with pytest.raises(FileExistsError):
        dev.save_config({"source": "config = 1\n"}, name="02_my_eval")
    cfg = load_config_from_file(saved["file"])
    assert cfg.rows == [{"question": "what", "answer": "42"}] and cfg.SYSTEM_PROMPT == nasty and cfg.max_turns == 2
    ep = endpoint_from_config(cfg)
    assert (ep.provider, ep.model, ep.api_base) == ("openai", "gpt-4o-mini", "http://x/v1")
    t = cfg.to_trajectory(cfg.rows[0])
    assert [m.role for m in t.messages] == ["system", "user"] and t.messages[1].text() == "Q: what" and t.metadata == {"answer": "42"}
    assert cfg.score_fn(t.append(Message("assistant", "It is 42.")), cfg.rows[0]) == 1.0
    assert match_score(Trajectory((Message("assistant", "about 1,000.0 items"),)), 1000) == 1.0
    assert match_score(Trajectory((Message("assistant", "no idea"),)), 7) == 0.0
    assert "experiment_name = 'x'" in generate_config({"experiment_name": "x"})


def test_runs_are_followed_killed_and_forgotten():
    reg = RunRegistry()
    run = reg.launch("demo", [sys.executable, "-u", "-c", "import time\nfor i in range(3): print('line', i)\ntime.sleep(0.2)\nraise SystemExit(3)"])
    first = reg.output(run.run_id)
    done = reg.wait(run.run_id, 30)
    assert done.status == "failed" and done.exit_code == 3
    rest = reg.output(run.run_id, first["next"])
    assert first["lines"] + rest["lines"] == ["line 0", "line 1", "line 2"] and rest["done"] and rest["next"] == 3
    assert reg.output(run.run_id, 3)["lines"] == [] and not reg.kill(run.run_id)
    # a run that would go on for a minute, with a child of its own: both end when the group is signalled
    long = reg.launch("long", [sys.executable, "-u", "-c",
                               "import subprocess, sys, time\nsubprocess.Popen([sys.executable, '-c', 'import time; time.sleep(60)'])\n"
                               "print('started', flush=True)\ntime.sleep(60)"])
    deadline = time.monotonic() + 30
    while not reg.output(long.run_id)["lines"] and time.monotonic() < deadline:
        time.sleep(0.05)
    assert not reg.delete(long.run_id) and reg.list()[0]["status"] == "running"
    t0 = time.monotonic()
    assert reg.kill(long.run_id) and time.monotonic() - t0 < 10
    assert reg.wait(long.run_id, 10).status == "killed" and reg.delete(long.run_id) and [r["run_id"] for r in reg.list()] == [run.run_id]


def test_launch_a_config_and_read_its_results_over_http(project):
    from fastapi.testclient import TestClient

    from research_b200.agents.store import FileSessionStore
    from research_b200.frontend.server import create_app

    dev = DevLoop(project)
    client = TestClient(create_app(FileSessionStore(project / "sessions"), devloop=dev))
    assert client.get("/api/dev/configs").json()[0]["name"] == "01_arith" and "EventSource" in client.get("/dev").text
    assert client.get("/api/dev/config/01_arith").json()["fields"]["config.experiment_name"] == "arith"
    assert client.get("/api/dev/config/nope").status_code == 404 and client.get("/api/dev/config/..%2Fx").status_code in (400, 404)
    assert client.get("/api/dev/dataset", params={"path": "data/t.csv", "n": 1}).json()["total_rows"] == 2
    assert "experiment_name = 'web'" in client.post("/api/dev/generate", json={"experiment_name": "web"}).json()["source"]
    assert client.post("/api/dev/generate", json={"experiment_name": "web", "save": True}).json()["name"] == "02_web"
    run = client.post("/api/dev/launch/01_arith").json()
    assert run["status"] == "running" and client.post("/api/dev/launch/nope").status_code == 404
    done = dev.runs.wait(run["run_id"], 180)
    out = "\n".join(dev.runs.output(run["run_id"])["lines"])
    assert done.status == "completed", out
    assert '"mean_reward": 1.0' in out and client.get("/api/dev/runs").json()[0]["exit_code"] == 0
    stream = client.get(f"/api/dev/run/{run['run_id']}/stream").text
    assert "event: done" in stream and '"exit_code": 0' in stream and "mean_reward" in stream
    traces = client.get("/api/dev/traces").json()
    assert len(traces) == 1 and traces[0]["summary"]["completed"] == 2
    trace = client.get(f"/api/dev/trace/{traces[0]['id']}").json()
    assert trace["total"] == 2 and [s["response"] for s in trace["samples"]] == ["4", "6"]
    assert client.delete(f"/api/dev/run/{run['run_id']}").json() == {"deleted": run["run_id"]}
    assert client.delete(f"/api/dev/run/{run['run_id']}").status_code == 409
