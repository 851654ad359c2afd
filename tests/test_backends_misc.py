"""Functional (torch.func) training backend, backend placeholders, config loader / fingerprint, logging set-up and the
generation comparison helpers."""

import json
import logging
from dataclasses import dataclass, replace

import pytest
import torch

from research_b200.models import get_preset
from research_b200.models.functional import causal_lm_forward
from research_b200.models.weights import init_random_weights
from research_b200.training.backends import (JAXTrainingBackend, NativeTrainingBackend, TorchaxTrainingBackend, TorchFuncTrainingBackend,
                                             TrainingBackend)
from research_b200.training.backends.torch_func import adamw_init, adamw_update, clip_by_global_norm, global_norm
from research_b200.training.types import TrainerConfig


def test_functional_adamw_matches_torch_and_is_pure():
    torch.manual_seed(0)
    p = {"a": torch.randn(5, 3), "b": torch.randn(4)}
    ref = {k: torch.nn.Parameter(v.clone()) for k, v in p.items()}
    opt = torch.optim.AdamW(ref.values(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    state = adamw_init(p)
    cur = p
    for _ in range(4):
        g = {k: torch.randn_like(v) for k, v in p.items()}
        for k in ref:
            ref[k].grad = g[k].clone()
        opt.step()
        before = {k: v.clone() for k, v in cur.items()}
        new, state = adamw_update(cur, g, state, 1e-2, (0.9, 0.95), 1e-8, 0.1)
        assert all(torch.equal(cur[k], before[k]) for k in cur)          # inputs untouched
        cur = new
    assert state.step == 4 and all(torch.allclose(cur[k], ref[k].detach(), atol=1e-6) for k in cur)
    clipped, n = clip_by_global_norm({"x": torch.full((4,), 3.0)}, 1.0)
    assert float(n) == pytest.approx(6.0) and float(global_norm(clipped)) == pytest.approx(1.0, abs=1e-4)


def test_torch_func_backend_tracks_the_native_backend(tmp_path):
    cfg = get_preset("tiny-qwen2")
    w = init_random_weights(cfg, seed=0)
    tc = TrainerConfig(num_minibatches=2, max_grad_norm=1.0)
    a = TorchFuncTrainingBackend(cfg, w, device="cpu", loss_fn="sft", lr=1e-3, weight_decay=0.01, trainer_config=tc, checkpoint_dir=tmp_path)
    b = NativeTrainingBackend(cfg, w, device="cpu", loss_fn="sft", lr=1e-3, weight_decay=0.01, trainer_config=tc)
    assert isinstance(a, TrainingBackend)
    g = torch.Generator().manual_seed(0)
    for _ in range(3):
        ids = torch.randint(0, cfg.vocab_size, (4, 12), generator=g)
        batch = {"input_ids": ids, "labels": ids.clone()}
        ma, mb = a.forward_backward(batch).wait(), b.forward_backward(batch).wait()
        oa, ob = a.optim_step().wait(), b.optim_step().wait()
        assert ma["loss"] == pytest.approx(mb["loss"], rel=1e-4) and oa["grad_norm"] == pytest.approx(ob["grad_norm"], rel=1e-3)
        assert ma["num_tokens"] == mb["num_tokens"] == 4 * 11
    wa, wb = a.get_weights().wait(), b.get_weights().wait()
    assert max(float((wa[k] - wb[k].float()).abs().max()) for k in wa) < 1e-4
    norms = a.per_sample_grad_norms(batch)
    assert norms.shape == (4,) and bool((norms > 0).all())
    path = a.save_checkpoint(metrics={"loss": ma["loss"]})
    fresh = TorchFuncTrainingBackend(cfg, device="cpu", loss_fn="sft", seed=5)
    assert fresh.load_checkpoint(path)["loss"] == pytest.approx(ma["loss"]) and fresh.current_step == 3 and fresh.opt_state.step == 3
    assert all(torch.equal(fresh.params[k], a.params[k]) for k in a.params)
    fresh.load_weights(init_random_weights(cfg, seed=9)).wait()
    assert fresh.weight_version == a.weight_version + 1
    with pytest.raises(AssertionError):
        fresh.optim_step()                                              # nothing accumulated


def test_grpo_loss_through_the_functional_backend():
    cfg = get_preset("tiny-qwen2")
    be = TorchFuncTrainingBackend(cfg, device="cpu", loss_fn="grpo", lr=5e-3, trainer_config=TrainerConfig(max_grad_norm=None))
    ids = torch.randint(0, cfg.vocab_size, (4, 10), generator=torch.Generator().manual_seed(1))
    batch = {"input_ids": ids, "labels": ids.clone(), "advantages": torch.tensor([1.0, -1.0, 0.5, -0.5])}
    first = be.forward_backward(batch).wait()
    be.optim_step().wait()
    second = be.forward_backward(batch).wait()
    assert "entropy" in first and second["pg_loss"] < first["pg_loss"]      # the step raised advantage-weighted log-probs


def test_placeholders_refuse_construction():
    for cls in (JAXTrainingBackend, TorchaxTrainingBackend):
        with pytest.raises(NotImplementedError, match=cls.__name__):
            cls()


@dataclass(frozen=True)
class _Inner:
    lr: float = 1e-4
    fn: object = len


@dataclass(frozen=True)
class _Cfg:
    name: str = "x"
    inner: _Inner = _Inner()
    sizes: tuple = (1, 2)


def test_config_loader_and_fingerprint(tmp_path):
    from research_b200.utils.config_loader import config_to_dict, fingerprint, git_state, load_config_from_file

    f = tmp_path / "exp.py"
    f.write_text("from dataclasses import dataclass, replace\n@dataclass(frozen=True)\nclass C:\n    lr: float = 1e-3\n    steps: int = 5\n"
                 "base = C()\nconfig = replace(base, steps=9)\nother = 3\n")
    cfg = load_config_from_file(f)
    assert cfg.steps == 9 and cfg.lr == 1e-3 and load_config_from_file(f, "other") == 3
    with pytest.raises(AssertionError):
        load_config_from_file(f, "missing")
    with pytest.raises(AssertionError):
        load_config_from_file(tmp_path / "nope.py")
    d = config_to_dict(_Cfg())
    assert d == {"name": "x", "inner": {"lr": 1e-4, "fn": "len"}, "sizes": [1, 2]} and json.dumps(d)
    a, b = fingerprint(_Cfg(), include_git=False), fingerprint(replace(_Cfg(), name="y"), include_git=False)
    assert a["config_hash"] != b["config_hash"] and a == fingerprint(_Cfg(), include_git=False) and "git" not in a
    gs = git_state(tmp_path)                                            # not a repository: empty answers, no exception
    assert set(gs) == {"commit", "dirty"}
    assert "git" in fingerprint(_Cfg(), cwd=tmp_path)


def test_logging_setup_json_file_and_queue(tmp_path, monkeypatch):
    from research_b200.utils.logging_config import ColorFormatter, JSONFormatter, setup_logging

    root = logging.getLogger()
    saved, level = list(root.handlers), root.level
    try:
        monkeypatch.delenv("LOG_LEVEL", raising=False)
        log_file = tmp_path / "logs" / "run.jsonl"
        setup_logging("debug", log_file=log_file, json_console=True)
        log = logging.getLogger("rb.test")
        log.info("step done", extra={"step": 3, "loss": 0.5, "obj": object()})
        try:
            raise ValueError("bad")
        except ValueError:
            log.exception("failed")
        for h in root.handlers:
            h.flush()
        recs = [json.loads(x) for x in log_file.read_text().splitlines()]
        assert recs[0]["message"] == "step done" and recs[0]["step"] == 3 and recs[0]["loss"] == 0.5 and recs[0]["obj"].startswith("<object")
        assert recs[0]["level"] == "INFO" and recs[0]["logger"] == "rb.test" and recs[0]["timestamp"].endswith("Z")
        assert "ValueError: bad" in recs[1]["exception"]
        monkeypatch.setenv("LOG_LEVEL", "warning")
        setup_logging("debug", use_queue=True)
        assert root.level == logging.WARNING and isinstance(root.handlers[0], logging.handlers.QueueHandler)
        root._rb_listener.stop()
        line = ColorFormatter().format(logging.LogRecord("n", logging.ERROR, "", 0, "boom %s", ("x",), None))
        assert "boom x" in line and "\033[31m" in line
        assert json.loads(JSONFormatter().format(logging.LogRecord("n", logging.INFO, "", 0, "m", (), None)))["message"] == "m"
    finally:
        for h in list(root.handlers):
            root.removeHandler(h)
        for h in saved:
            root.addHandler(h)
        root.setLevel(level)


def test_generation_comparison_helpers():
    from research_b200.inference.backends.generate import GenerationOutput
    from research_b200.inference.testing import check_logprobs_close, check_outputs_equal, generate_with_logprobs_forward, topn_at

    cfg = get_preset("tiny-qwen2")
    w = init_random_weights(cfg, seed=0)
    fwd = lambda ids: causal_lm_forward(ids, w, cfg)                                    # noqa: E731
    ref = generate_with_logprobs_forward(fwd, [[1, 2, 3]], max_tokens=5, top_n=4)[0]
    assert len(ref.output_ids) == 5 and len(ref.top_logprobs[0]) == 4 and ref.top_logprobs[0][0][0] == ref.output_ids[0]
    same = check_logprobs_close(ref, ref.output_ids, ref.logprobs)
    assert same.ok and same.exact and same.first_divergence is None
    # diverge at position 2 onto the runner-up: accepted; onto a token outside the top-N: rejected
    runner_up = ref.top_logprobs[2][1][0]
    alt = ref.output_ids[:2] + (runner_up,) + ref.output_ids[3:]
    r = check_logprobs_close(ref, alt, ref.logprobs)
    assert r.ok and not r.exact and r.first_divergence == 2
    outside = next(t for t in range(cfg.vocab_size) if t not in {c for c, _ in ref.top_logprobs[2]})
    bad = check_logprobs_close(ref, ref.output_ids[:2] + (outside,) + ref.output_ids[3:], ref.logprobs)
    assert not bad.ok and "outside" in bad.detail
    off = check_logprobs_close(ref, ref.output_ids, tuple(x - 0.5 for x in ref.logprobs))
    assert not off.ok and off.max_logprob_diff == pytest.approx(0.5, abs=1e-6)
    bare = GenerationOutput(ref.input_ids, ref.output_ids, ref.logprobs)                # no stored candidates: recompute them
    assert check_logprobs_close(bare, alt, ref.logprobs, forward_fn=fwd, top_n=4).ok
    assert not check_logprobs_close(bare, alt, ref.logprobs).ok
    assert topn_at(fwd, [1, 2, 3], 4)[0][0] == ref.output_ids[0]
    assert check_outputs_equal([ref, ref], [ref, GenerationOutput(ref.input_ids, alt, ref.logprobs)]) == [True, False]


def test_http_engine_lifecycle_logs_health_and_crash(tmp_path, caplog):
    """An external inference server as a child process: default command lines, its log lines forwarded to the Python logger,
    readiness by health poll, a start-up crash reported with the tail of its log, shutdown of exactly that child."""
    import asyncio
    import logging
    import socket
    import sys
    import time

    from research_b200.training.weight_sync import SGLangEngine, VLLMEngine

    sg = SGLangEngine("org/model", port=31001, cuda_device_ids=(2, 3), mem_fraction=0.8, extra_args=("--attention-backend", "triton"))
    cmd = sg.default_launch_cmd()
    assert cmd[1:3] == ["-m", "sglang.launch_server"] and cmd[cmd.index("--tp") + 1] == "2" and cmd[-2:] == ["--attention-backend", "triton"]
    assert "--tensor-parallel-size" not in VLLMEngine("m").default_launch_cmd() and "vllm.entrypoints.openai.api_server" in VLLMEngine("m").default_launch_cmd()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = ("import http.server, sys\nprint('loading weights', flush=True)\n"
              "class H(http.server.BaseHTTPRequestHandler):\n"
              "    def do_GET(self):\n        self.send_response(200 if self.path == '/health' else 404); self.end_headers()\n"
              "    def log_message(self, *a): pass\n"
              f"print('server ready', flush=True)\nhttp.server.HTTPServer(('127.0.0.1', {port}), H).serve_forever()\n")
    eng = SGLangEngine("m", port=port, launch_cmd=[sys.executable, "-u", "-c", server], log_path=str(tmp_path / "logs" / "server.log"))

    async def go():
        await eng.launch()
        await eng.wait_until_ready(timeout=30)
        pid = eng._proc.pid
        await asyncio.sleep(0.5)
        await eng.shutdown()
        return pid

    with caplog.at_level(logging.INFO):
        pid = asyncio.run(go())
    assert eng._proc.poll() is not None and pid > 0 and "server ready" in eng.log_tail()
    deadline = time.time() + 5
    while "server ready" not in caplog.text and time.time() < deadline:
        time.sleep(0.1)
    assert "loading weights" in caplog.text and f"sglang:{port}" in caplog.text                # the child's lines reached the logger
    bad = VLLMEngine("m", port=port, launch_cmd=[sys.executable, "-c", "print('CUDA out of memory'); raise SystemExit(3)"], log_path=str(tmp_path / "bad.log"))

    async def crash():
        await bad.launch()
        await bad.wait_until_ready(timeout=20)

    with pytest.raises(RuntimeError, match="exited with code 3") as e:
        asyncio.run(crash())
    assert "CUDA out of memory" in str(e.value)
