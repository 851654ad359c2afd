"""The example scripts run end to end on CPU with the tiny presets and the character tokenizer."""

import sys
from dataclasses import replace
from pathlib import Path
from types import SimpleNamespace

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from research_b200.utils.char_tokenizer import CharTokenizer  # noqa: E402


def test_char_tokenizer_round_trip_and_template():
    tok = CharTokenizer()
    text = "Hello, <b>world</b>!\n\t~"
    ids = tok.encode(text)
    assert tok.decode(ids) == text and len(ids) == len(text) and tok.vocab_size == len(tok) > 100
    assert tok.encode("é")[0] == tok.unk_token_id and tok.encode("x", add_special_tokens=True)[0] == tok.bos_token_id
    msgs = [{"role": "system", "content": "s"}, {"role": "user", "content": "u"}]
    full = tok.apply_chat_template(msgs + [{"role": "assistant", "content": "a"}])
    head = tok.apply_chat_template(msgs, add_generation_prompt=True)
    assert full[:len(head)] == head                                       # prefix-stable
    assert tok.apply_chat_template(msgs, tokenize=False) == "<|system|>s<|eos|><|user|>u<|eos|>"
    assert tok.decode(full, skip_special_tokens=True) == "sua" and tok.eos_token_id in full
    assert tok(["ab", "c"])["input_ids"] == [tok.encode("ab"), tok.encode("c")]
    assert tok.decode([5000, -1]) == "" and tok.convert_ids_to_tokens([2, 99999]) == ["<|eos|>", "<|unk|>"]


def test_score_functions():
    from examples.rl.alphabet_sort.base_config import sort_score_fn
    from examples.rl.gsm8k.base_config import extract_boxed_answer, gsm8k_score_fn, normalize_answer, synthetic_problems, truth_of
    from examples.rl.reverse_text.base_config import make_prompts, make_texts, reverse_text_score_fn

    def sample(text, truth):
        return SimpleNamespace(metadata={"response_text": text}, ground_truth=truth, response_length=0, tokens=[])

    s = reverse_text_score_fn(sample("<think>hm</think><reversed_text> cba </reversed_text><|eos|>junk", "cba"))
    assert s.reward == 1.0 and {m.name: m.value for m in s.metrics}["has_tags"] == 1.0
    assert 0 < reverse_text_score_fn(sample("cbx", "cba")).reward < 1.0
    prompts, truths = make_prompts(make_texts(3, seed=1))
    assert truths[0] == prompts[0][1]["content"][::-1] and make_texts(3, 1) == make_texts(3, 1)
    assert sort_score_fn(sample("<sorted>ada\nbo\ncy</sorted>", ["ada", "bo", "cy"])).reward == pytest.approx(1.0)
    assert sort_score_fn(sample("bo, ada, cy", ["ada", "bo", "cy"])).reward == pytest.approx(0.8 / 3)
    assert extract_boxed_answer(r"so \boxed{1} then \boxed{ 42 }") == "42" and normalize_answer("$1,234.5") == 1234.5
    row = synthetic_problems(1, 0)[0]
    assert gsm8k_score_fn(sample(f"\\boxed{{{int(truth_of(row))}}}", truth_of(row))).reward == pytest.approx(1.0)
    assert gsm8k_score_fn(sample(f"the answer is {int(truth_of(row))}", truth_of(row))).reward == pytest.approx(1.0 / 1.1)
    assert gsm8k_score_fn(sample("no idea", truth_of(row))).reward == 0.0


def test_sft_then_grpo_two_stage(tmp_path):
    from examples.rl.reverse_text.sft_then_grpo import run

    sft_hist, rl_hist = run(sft_steps=6, rl_steps=1, device="cpu", out=str(tmp_path))
    assert sft_hist[-1]["loss"] < sft_hist[0]["loss"] and len(rl_hist) == 1 and 0.0 <= rl_hist[0]["mean_reward"] <= 1.0
    assert (tmp_path / "stage1_sft" / "hf" / "model.safetensors").exists()


@pytest.mark.parametrize("task", ["alphabet_sort", "gsm8k", "calculator"])
def test_rl_examples_take_a_step(tmp_path, task):
    import importlib

    mod = importlib.import_module(f"examples.rl.{task}.base_config")
    cfg = replace(mod.DEFAULT, num_steps=1, output_dir=str(tmp_path), max_tokens=6, batch_size=2, n_samples_per_prompt=2, num_minibatches=1)
    hist = mod.train(cfg, num_samples=4, device="cpu")
    assert len(hist) == 1 and hist[0]["num_samples"] == 4.0 and "mean_reward" in hist[0]


def test_inference_eval_and_prompt_optimization_examples(tmp_path):
    from examples.eval.gsm8k.base_config import GSM8KConfig, run_eval
    from examples.eval.gsm8k.eval_scripted_01_01 import reads_the_numbers
    from examples.inference.base_config import BaseConfig, test_inference as run_inference
    from examples.prompt_optimization.calculator_gepa import run as run_gepa
    from research_b200.agents.dtypes import Endpoint
    from research_b200.agents.providers import register_provider

    res = run_inference(BaseConfig(prompts=("Hello", "Hello there"), max_tokens=5, num_samples_per_prompt=2), device="cpu")
    assert len(res) == 4 and all(r["num_tokens"] == 5 and r["sum_logprob"] < 0 for r in res)
    register_provider("mock", reads_the_numbers)
    rep = run_eval(GSM8KConfig(endpoint=Endpoint(provider="mock"), num_samples=5, output_dir=str(tmp_path)))
    assert rep.summary["mean_reward"] == 1.0 and (tmp_path / "gsm8k" / "report.json").exists()
    best = run_gepa(60)
    assert best.best_score == 1.0 and "only the number" in best.best_candidate["system"].lower()


def test_run_remote_against_this_machine(tmp_path, monkeypatch):
    """``run_remote`` with a local target: push, build step, detached job, streamed log, results fetched."""
    import subprocess

    import examples.common as common

    repo = tmp_path / "repo"
    (repo / "examples").mkdir(parents=True)
    (repo / "research_b200").mkdir()
    (repo / "research_b200" / "__init__.py").write_text("")
    (repo / "research_b200" / "_native.py").write_text("print('built')\n")
    (repo / "examples" / "job.py").write_text("import pathlib\nprint('hello from job')\npathlib.Path('results').mkdir(exist_ok=True)\n"
                                               "pathlib.Path('results/out.txt').write_text('42')\n")
    git = lambda *a: subprocess.run(["git", "-c", "user.name=t", "-c", "user.email=t@t", "-C", str(repo), *a], check=True, capture_output=True)  # noqa: E731
    git("init", "-q", "-b", "main"); git("add", "-A"); git("commit", "-qm", "one")
    monkeypatch.setattr(common, "REPO_ROOT", repo)
    monkeypatch.setenv("HOME", str(tmp_path / "home"))
    (tmp_path / "home").mkdir()
    lines = []
    code = common.run_remote(str(repo / "examples" / "job.py"), ssh="local", out=lines.append)
    assert code == 0 and any("hello from job" in x for x in lines)
    fetched = list((repo / "results").rglob("out.txt"))
    assert fetched and fetched[0].read_text() == "42"


def test_integration_training_single_device_and_two_cpu_ranks(tmp_path):
    import json
    import subprocess

    from examples.integration_training.base_config import Config, OutputSection, RLSection, SFTSection, TargetConfig
    from examples.integration_training.train import launch_command, main

    one = tmp_path / "one.py"
    one.write_text("from examples.integration_training.base_config import *\n"
                   f"config = Config(target=TargetConfig(device='cpu'), sft=SFTSection(num_steps=4, batch_size=4, num_rows=16), "
                   f"rl=RLSection(num_steps=1, batch_size=2, n_samples_per_prompt=2, max_tokens=6, num_prompts=4), "
                   f"output=OutputSection(mode='sft_then_rl', save_dir={str(tmp_path)!r}, experiment_name='one'))\n")
    assert main([str(one)]) == 0
    s = json.loads((tmp_path / "one" / "summary.json").read_text())
    assert s["sft"]["last_loss"] < s["sft"]["first_loss"] and s["rl"]["steps"] == 1 and (tmp_path / "one" / "sft_hf" / "model.safetensors").exists()
    two = tmp_path / "two.py"
    two.write_text("from examples.integration_training.base_config import *\n"
                   f"config = Config(target=TargetConfig(gpu_ranks=(0, 1), train_backend='fsdp', device='cpu', master_port=29533), "
                   f"sft=SFTSection(num_steps=4, batch_size=4, num_rows=16), output=OutputSection(mode='sft', save_dir={str(tmp_path)!r}, experiment_name='two'))\n")
    cmd = launch_command(Config(target=TargetConfig(gpu_ranks=(0, 1))), "train.py", "c.py")
    assert "--nproc-per-node=2" in cmd and "--master-addr=127.0.0.1" in cmd and cmd[-2:] == ["train.py", "c.py"]
    r = subprocess.run([sys.executable, str(ROOT / "examples" / "integration_training" / "train.py"), str(two)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    s2 = json.loads((tmp_path / "two" / "summary.json").read_text())
    assert s2["sft"]["steps"] == 4 and s2["sft"]["last_loss"] < s2["sft"]["first_loss"]


def test_chess_examples():
    from examples.eval.chess_puzzles.beam_search_demo import run as beam
    from examples.eval.chess_puzzles.run import PUZZLES, mate_in_one, run

    assert all(mate_in_one(p["fen"]) in p["solution"] for p in PUZZLES)
    rep = run()
    assert rep.summary["mean_reward"] == 1.0 and all(s.stop_reason == "task_completed" for s in rep.samples)
    node = beam()
    assert node.score == 1.0 and node.depth == 3 and node.state.is_checkmate()


def test_rlm_needle_in_haystack():
    from examples.eval.rlm.needle_haystack import make_rows, run

    rows = make_rows(n=2, lines=300)
    rep = run(rows)
    assert rep.summary["mean_reward"] == 1.0
    chars = [m.value for s in rep.samples for m in s.score.metrics if m.name == "prompt_chars"]
    assert max(chars) < 400 < len(rows[0]["context"])                    # the document never entered the prompt


def test_browsing_eval_on_the_offline_web():
    from examples.eval.browsecomp.base_config import BrowseConfig, extract_answer, run_eval
    from examples.eval.browsecomp.eval_scripted_01_01 import searcher_reader
    from research_b200.agents.dtypes import Endpoint
    from research_b200.agents.providers import register_provider

    assert extract_answer("x\nExact Answer: Askvik.") == "Askvik" and extract_answer("no answer") is None
    register_provider("mock", searcher_reader)
    rep = run_eval(BrowseConfig(endpoint=Endpoint(provider="mock")))
    assert rep.summary["mean_reward"] == 1.0
    by = {s.sample_id: {m.name: m.value for m in s.score.metrics} for s in rep.samples}
    assert all(1 <= m["pages_read"] <= 3 and m["searches"] == 1 and m["answered"] == 1.0 for m in by.values())


def test_intent_gepa_and_rlm_aggregation_examples():
    from examples.eval.rlm.aggregate_records import make_rows, run as run_aggregate
    from examples.prompt_optimization.intent_gepa import LABELS, run as run_intent

    best = run_intent(200)
    assert best.best_score == 1.0 and all(lbl in best.best_candidate["system"] + best.best_candidate["user_template"] for lbl in LABELS)
    assert "only the label" in (best.best_candidate["system"] + best.best_candidate["user_template"]).lower() and "{input}" in best.best_candidate["user_template"]
    rep = run_aggregate(make_rows(3, lines=300, seed=1))
    # every count right, while the prompt the root model saw stayed two orders of magnitude below the input
    assert rep.summary["mean_correct"] == 1.0 and rep.summary["mean_prompt_chars"] * 10 < rep.summary["mean_context_chars"]
