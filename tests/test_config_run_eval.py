"""Config protocols / base configs / loader and the config-driven evaluation runner (CPU, scripted model)."""

import asyncio
import json
import textwrap
from dataclasses import dataclass, field
from pathlib import Path

from research_b200.agents.dtypes import Endpoint, Message, Trajectory
from research_b200.agents.providers import ScriptedLLM, register_provider
from research_b200.config import (BaseEnvironmentConfig, BaseEvaluationConfig, BaseModelConfig, BaseOutputConfig,
                                  HasEnvironmentConfig, HasEvaluationConfig, HasModelConfig, HasOutputConfig,
                                  infer_provider_from_model, load_config_from_file, validate_config_protocol)
from research_b200.run_eval import check_api_key, main, run_evaluation


def test_provider_inference_and_model_config(monkeypatch):
    assert infer_provider_from_model("gpt-4o-mini") == "openai"
    assert infer_provider_from_model("claude-sonnet-4-20250514") == "anthropic"
    assert infer_provider_from_model("gemini-2.0-flash") == "google"
    assert infer_provider_from_model("qwen-7b") == "qwen"
    monkeypatch.setenv("ANTHROPIC_API_KEY", "sk-test-1234")
    ep = BaseModelConfig(model_name="claude-sonnet-4", provider="openai", temperature=0.2).to_endpoint()
    assert (ep.provider, ep.api_base, ep.api_key, ep.temperature) == ("anthropic", "https://api.anthropic.com", "sk-test-1234", 0.2)
    local = BaseModelConfig(model_name="tiny", provider="native", api_base="", api_key_env_var="").to_endpoint()
    assert local.provider == "native" and local.api_key == ""


def test_protocols_are_structural():
    @dataclass(frozen=True)
    class Mine:
        env_name: str = "calc"
        output_dir: Path = Path("out")
        experiment_name: str = "x"

        def to_endpoint(self) -> Endpoint:
            return Endpoint(provider="mock")

        def prepare_messages(self, sample_data):
            return [Message("user", sample_data["q"])]

    m = Mine()
    assert isinstance(m, HasModelConfig) and isinstance(m, HasEnvironmentConfig) and isinstance(m, HasOutputConfig)
    assert not isinstance(m, HasEvaluationConfig)
    assert validate_config_protocol(m, HasEvaluationConfig) == ["to_eval_config"]
    assert validate_config_protocol(m, HasModelConfig) == []
    ev = BaseEvaluationConfig(BaseEnvironmentConfig("calc", max_steps=3), num_samples=5, max_turns=10)
    assert isinstance(ev, HasEvaluationConfig)
    cfg = ev.to_eval_config(Endpoint(provider="mock"), None, lambda t, r: 1.0)
    assert cfg.max_turns == 3 and cfg.max_samples == 5 and cfg.prepare_messages({"prompt": "hi"})[0].content == "hi"


def test_output_config_roundtrip_and_loader(tmp_path):
    out = BaseOutputConfig(output_dir=tmp_path / "r", experiment_name="e1", verbose=False)
    out.save_config(out, tmp_path / "cfg" / "out.json")
    back = BaseOutputConfig.load_config(BaseOutputConfig, tmp_path / "cfg" / "out.json")
    assert back == out

    @dataclass(frozen=True)
    class Nested:
        model: BaseModelConfig = field(default_factory=BaseModelConfig)
        fn: object = len

    out.save_config(Nested(), tmp_path / "nested.json")
    data = json.loads((tmp_path / "nested.json").read_text())
    assert data["model"]["model_name"] == "gpt-4o-mini" and data["fn"] == "len"
    (tmp_path / "helper_mod.py").write_text("VALUE = 7\n")
    (tmp_path / "c.py").write_text("import helper_mod\nconfig = {'v': helper_mod.VALUE}\nother = 3\n")
    assert load_config_from_file(tmp_path / "c.py") == {"v": 7}
    assert load_config_from_file(tmp_path / "c.py", "other") == 3


CONFIG = '''
from dataclasses import dataclass, field
from pathlib import Path
from research_b200.agents.dtypes import Message, Trajectory

@dataclass(frozen=True)
class DS:
    dataset_path: Path = Path("data")
    annotation_files: tuple = ("a.json", "b.json")

@dataclass(frozen=True)
class Filters:
    platforms: tuple = ()
    applications: tuple = ()
    ui_types: tuple = ()
    limit: int = 5

def load_dataset(data_path, annotation_file, limit=None, platforms=None, **kw):
    import json
    return json.loads((Path(data_path) / annotation_file).read_text())

class Env:
    def compute_reward(self, text, bbox, img_size):
        return 1.0 if str(bbox[0]) in text else 0.0
    def get_tools(self): return []
    async def serialize(self): return {}

@dataclass(frozen=True)
class Config:
    dataset: DS = field(default_factory=DS)
    filters: Filters = field(default_factory=Filters)
    provider: str = "mock"
    model_name: str = "scripted"
    api_base: str = ""
    temperature: float = 0.0
    max_output_tokens: int = 16
    max_concurrent: int = 2
    max_turns: int = 1
    experiment_name: str = "ground"
    save_jsonl: bool = True
    save_dir: str = "RESULTS"
    show_progress: bool = False
    load_dataset: object = load_dataset
    environment: object = Env
    def to_trajectory(self, row):
        if row.get("boom"):
            raise ValueError("bad row")
        return Trajectory((Message("user", row["q"]),), metadata={"bbox": row["bbox"], "img_size": [10, 10]})

config = Config()
'''


def test_run_evaluation_from_config_file(tmp_path, monkeypatch):
    data = tmp_path / "data"
    data.mkdir()
    (data / "a.json").write_text(json.dumps([{"q": "where is 3", "bbox": [3, 1]}, {"q": "where is 4", "bbox": [4, 1]}, {"q": "x", "bbox": [9, 9], "boom": True}]))
    (data / "b.json").write_text(json.dumps([{"q": "where is 5", "bbox": [5, 1]}, {"q": "6", "bbox": [6, 1]}, {"q": "never", "bbox": [7, 1]}]))
    cfg_path = tmp_path / "eval_cfg.py"
    cfg_path.write_text(CONFIG.replace('"RESULTS"', repr(str(tmp_path / "results"))))
    monkeypatch.chdir(tmp_path)
    register_provider("mock", ScriptedLLM(["the answer is 3"] * 16))
    from research_b200.run_eval import load_config_from_file as load

    config = load(cfg_path, workspace_root=tmp_path)
    assert config.dataset.dataset_path == tmp_path / "data"
    out = asyncio.run(run_evaluation(config, tmp_path / "rd"))
    s = out["summary"]
    assert s["total_samples"] == 5 and s["completed"] == 4 and s["errors"] == 1        # the limit cut row 6, one row raised
    assert out["results"][0]["reward"] == 1.0 and out["results"][1]["reward"] == 0.0
    assert "ValueError" in out["results"][2]["error"] and out["results"][0]["metadata"]["bbox"] == [3, 1]
    lines = (tmp_path / "rd" / "ground_results.jsonl").read_text().strip().splitlines()
    assert len(lines) == 5 and abs(s["mean_reward"] - 0.25) < 1e-9
    # the command line: same config, result file where asked; exit code 2 because one sample failed
    register_provider("mock", ScriptedLLM(["the answer is 3"] * 16))
    rc = main(["--config", str(cfg_path), "--output", str(tmp_path / "final.json"), "--workspace-root", str(tmp_path)])
    assert rc == 2 and json.loads((tmp_path / "final.json").read_text())["summary"]["completed"] == 4


def test_remote_provider_needs_its_key(monkeypatch):
    monkeypatch.delenv("OPENAI_API_KEY", raising=False)
    assert check_api_key("openai") == "OPENAI_API_KEY" and check_api_key("mock") is None
    monkeypatch.setenv("OPENAI_API_KEY", "k")
    assert check_api_key("OpenAI") is None
    _ = textwrap
