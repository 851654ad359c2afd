"""HTTP front end of the native engine, speaking the two token-in / token-out dialects the trainer
and the agent providers already use:

* SGLang style: ``POST /generate {"input_ids", "sampling_params", "return_logprob"}``,
  ``POST /update_weights_from_disk {"model_path"}``, ``POST /flush_cache``, ``GET /health``,
  ``GET /get_server_info``
* vLLM / OpenAI style: ``POST /v1/completions {"prompt": [ids] | "text", "max_tokens", "temperature",
  "logprobs"}``

(the HTTP API phase of rollouts/docs/design/nano_inference.md:716-719; endpoint shapes as consumed by
rollouts/inference/backends/generate.py:66-226 and rollouts/training/weight_sync.py:34-126).

One background thread owns the engine and steps it whenever work is pending (continuous batching
across concurrent HTTP requests); request handlers enqueue prompts and await their futures.
``EngineService`` is usable without HTTP, which is how the tests drive it.
"""

from __future__ import annotations

import asyncio
import threading
import time
from concurrent.futures import Future
from typing import Any

from .types import SamplingParams, TrainingSample


class EngineService:
    """Thread that steps the engine; ``submit`` returns a future resolved with the finished sample."""

    def __init__(self, engine, idle_sleep: float = 0.001):
        self.engine = engine
        self.idle_sleep = idle_sleep
        self._lock = threading.Lock()
        self._pending: list[tuple[list[int], SamplingParams, Future]] = []
        self._futures: dict[int, Future] = {}
        self._paused = threading.Event()
        self._idle = threading.Event()
        self._stop = threading.Event()
        self.steps = 0
        self.thread = threading.Thread(target=self._run, name="engine-service", daemon=True)
        self.thread.start()

    def submit(self, prompt_tokens: list[int], params: SamplingParams) -> Future:
        fut: Future = Future()
        with self._lock:
            self._pending.append((list(prompt_tokens), params, fut))
        return fut

    def _admit(self) -> None:
        with self._lock:
            batch, self._pending = self._pending, []
        for toks, params, fut in batch:
            try:
                self._futures[self.engine.add_request(toks, params)] = fut
            except Exception as e:  # noqa: BLE001 - bad request (too long, empty): report to the caller
                fut.set_exception(e)

    def _run(self) -> None:
        while not self._stop.is_set():
            if self._paused.is_set():
                self._idle.set()
                time.sleep(self.idle_sleep)
                continue
            self._admit()
            if not self.engine.has_pending():
                self._idle.set()
                time.sleep(self.idle_sleep)
                continue
            self._idle.clear()
            try:
                finished = self.engine._step_with_ids()
            except Exception as e:  # noqa: BLE001 - a failed step fails every in-flight request
                for fut in self._futures.values():
                    if not fut.done():
                        fut.set_exception(e)
                self._futures.clear()
                continue
            self.steps += 1
            for sid, sample in finished:
                fut = self._futures.pop(sid, None)
                if fut is not None and not fut.done():
                    fut.set_result(sample)

    def quiesce(self, timeout: float = 300.0) -> None:
        """Stop admitting, wait until nothing is running (needed before a weight update)."""
        deadline = time.monotonic() + timeout
        while self.engine.has_pending() or self._pending:
            if time.monotonic() > deadline:
                raise TimeoutError("engine did not drain in time")
            time.sleep(self.idle_sleep)
        self._paused.set()
        self._idle.clear()
        if not self._idle.wait(timeout):
            raise TimeoutError("engine thread did not pause")

    def resume(self) -> None:
        self._paused.clear()

    def update_weights(self, state_dict: dict) -> int:
        self.quiesce()
        try:
            self.engine.update_weights(state_dict)
            self.engine.flush_cache()
        finally:
            self.resume()
        return self.engine.get_weight_version()

    def flush_cache(self) -> None:
        """Drop the prefix cache once nothing is running."""
        self.quiesce()
        try:
            self.engine.flush_cache()
        finally:
            self.resume()

    def update_weights_from_path(self, path: str, loader=None) -> int:
        """Load a checkpoint (safetensors directory or ``torch.save`` file) and swap it in."""
        return self.update_weights((loader or default_weight_loader)(path))

    def shutdown(self) -> None:
        self._stop.set()
        self.thread.join(timeout=5)


class LockstepEngineService(EngineService):
    """Engine service for a tensor-parallel engine: every rank must see the same requests in the same order
    and step the same number of times. Rank 0 owns the HTTP side; before every step it broadcasts the requests
    admitted since the last one (an object broadcast on a CPU-side group) together with a stop flag, and all
    ranks add them and step together. Ranks other than 0 never resolve futures; they call ``follow()``."""

    def __init__(self, engine, group=None, idle_sleep: float = 0.001, heartbeat_s: float = 5.0):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        # an idle rank 0 still exchanges an empty batch this often, so that followers blocked in the broadcast
        # never run into the group's timeout (which is what detects a dead rank 0)
        self.heartbeat_s = heartbeat_s
        self._last_exchange = time.monotonic()
        self._control: list = []        # (operation, future) queued on rank 0
        self._loader = None
        super().__init__(engine, idle_sleep)

    def _exchange(self, batch, stop: bool, control=None):
        """One broadcast from rank 0: the requests admitted since the last one, the stop flag and at most one
        control operation (``("flush", None)``, ``("load", path)`` or ``("weights", state_dict)``) that every rank
        applies at this point of the common step sequence."""
        payload = [(([t for t, _, _ in batch], [p for _, p, _ in batch]), stop, control)] if self.rank == 0 else [None]
        self.dist.broadcast_object_list(payload, src=0, group=self.group)
        self._last_exchange = time.monotonic()
        return payload[0]

    def _apply_control(self, control) -> None:
        kind, arg = control
        if kind == "flush":
            self.engine.flush_cache()
        elif kind == "load":
            self.engine.update_weights((self._loader or default_weight_loader)(arg))
            self.engine.flush_cache()
        elif kind == "weights":
            self.engine.update_weights(arg)
            self.engine.flush_cache()
        else:
            raise ValueError(f"unknown control operation {kind!r}")

    def _control_op(self, control, timeout: float = 600.0):
        """Queue a control operation on rank 0 and wait until every rank has applied it (between two steps, with
        nothing running)."""
        assert self.rank == 0, "control operations enter through rank 0"
        fut: Future = Future()
        with self._lock:
            self._control.append((control, fut))
        return fut.result(timeout=timeout)

    def flush_cache(self) -> None:
        self._control_op(("flush", None))

    def update_weights(self, state_dict: dict) -> int:
        """Broadcasts the tensors themselves to the followers (pickled); for large models hand every rank a path with
        ``update_weights_from_path`` instead."""
        self._control_op(("weights", state_dict))
        return self.engine.get_weight_version()

    def update_weights_from_path(self, path: str, loader=None) -> int:
        if loader is not None:
            self._loader = loader
        self._control_op(("load", path))
        return self.engine.get_weight_version()

    def _fail_all(self, e: Exception) -> None:
        for fut in self._futures.values():
            if not fut.done():
                fut.set_exception(e)
        self._futures.clear()

    def _run(self) -> None:
        if self.rank != 0:
            return                      # followers run the loop in the caller's thread (see follow)
        while True:
            stop = self._stop.is_set()
            if self._paused.is_set() and not stop:
                # paused (a caller holds the engine): keep the followers' broadcast alive
                self._idle.set()
                if time.monotonic() - self._last_exchange > self.heartbeat_s:
                    self._exchange([], False)
                time.sleep(self.idle_sleep)
                continue
            with self._lock:
                draining = bool(self._control)
                if draining:
                    batch = []          # admissions wait until the control operation has run
                else:
                    batch, self._pending = self._pending, []
            if draining and not self.engine.has_pending() and not stop:
                with self._lock:
                    control, cfut = self._control.pop(0)
                self._exchange([], False, control)
                try:
                    self._apply_control(control)
                    cfut.set_result(True)
                except Exception as e:  # noqa: BLE001 - reported to the caller of the control operation
                    cfut.set_exception(e)
                continue
            if not batch and not self.engine.has_pending() and not stop:
                self._idle.set()
                if time.monotonic() - self._last_exchange > self.heartbeat_s:
                    self._exchange([], False)          # heartbeat: followers see an empty step and wait again
                time.sleep(self.idle_sleep)
                continue
            self._idle.clear()
            self._exchange(batch, stop)
            if stop:
                self._fail_all(RuntimeError("engine service stopped"))
                with self._lock:
                    for _, cfut in self._control:
                        cfut.set_exception(RuntimeError("engine service stopped"))
                    self._control.clear()
                return
            for toks, params, fut in batch:
                try:
                    self._futures[self.engine.add_request(toks, params)] = fut
                except Exception as e:  # noqa: BLE001 - the followers fail the same way and skip it too
                    fut.set_exception(e)
            if self.engine.has_pending():
                try:
                    finished = self.engine._step_with_ids()
                except Exception as e:  # noqa: BLE001 - a failed step fails every in-flight request
                    self._fail_all(e)
                    continue
                for sid, sample in finished:
                    fut = self._futures.pop(sid, None)
                    if fut is not None and not fut.done():
                        fut.set_result(sample)
                self.steps += 1

    def follow(self) -> None:
        """Body of every rank other than 0: mirror rank 0's admissions, steps and control operations until it says stop."""
        assert self.rank != 0
        while True:
            (toks, params), stop, control = self._exchange([], False)
            if stop:
                return
            if control is not None:
                try:
                    self._apply_control(control)
                except Exception:  # noqa: BLE001 - rank 0 fails the same way and reports it
                    pass
                continue
            for t, p in zip(toks, params):
                try:
                    self.engine.add_request(t, p)
                except Exception:  # noqa: BLE001 - rank 0 reports it to the caller
                    pass
            if self.engine.has_pending():
                try:
                    self.engine._step_with_ids()
                except Exception:  # noqa: BLE001 - rank 0 fails the same step and reports it
                    continue
                self.steps += 1

    def shutdown(self) -> None:
        self._stop.set()
        if self.rank == 0:
            self.thread.join(timeout=30)


def _params_from_sglang(sp: dict[str, Any]) -> SamplingParams:
    return SamplingParams(temperature=float(sp.get("temperature", 1.0)), max_tokens=int(sp.get("max_new_tokens", 128)),
                          stop_token_ids=frozenset(sp.get("stop_token_ids") or ()), seed=sp.get("seed"))


def sglang_response(sample: TrainingSample, return_logprob: bool, tokenizer=None) -> dict[str, Any]:
    out: dict[str, Any] = {"output_ids": list(sample.completion_tokens),
                           "text": tokenizer.decode(list(sample.completion_tokens)) if tokenizer else "",
                           "meta_info": {"finish_reason": {"type": sample.finish_reason},
                                         "prompt_tokens": len(sample.prompt_tokens),
                                         "completion_tokens": len(sample.completion_tokens),
                                         "cached_tokens": sample.cached_tokens, "weight_version": sample.weight_version}}
    if return_logprob:
        out["meta_info"]["output_token_logprobs"] = [[lp, tok, None] for lp, tok in zip(sample.logprobs, sample.completion_tokens)]
    return out


def openai_completion_response(sample: TrainingSample, model: str, want_logprobs: bool, tokenizer=None) -> dict[str, Any]:
    choice: dict[str, Any] = {"index": 0, "text": tokenizer.decode(list(sample.completion_tokens)) if tokenizer else "",
                              "token_ids": list(sample.completion_tokens), "finish_reason": sample.finish_reason}
    if want_logprobs:
        choice["logprobs"] = {"token_logprobs": list(sample.logprobs), "tokens": [str(t) for t in sample.completion_tokens]}
    return {"id": f"cmpl-{int(time.time() * 1000)}", "object": "text_completion", "model": model, "choices": [choice],
            "usage": {"prompt_tokens": len(sample.prompt_tokens), "completion_tokens": len(sample.completion_tokens),
                      "total_tokens": len(sample.prompt_tokens) + len(sample.completion_tokens)}}


def create_app(service: EngineService, model_name: str = "native", tokenizer=None, weight_loader=None):
    """FastAPI application over ``service``. ``weight_loader(path) -> state_dict`` serves
    ``/update_weights_from_disk`` (default: safetensors directory or ``torch.load`` file)."""
    from fastapi import FastAPI, HTTPException

    app = FastAPI(title="research_b200 engine")

    async def run(tokens: list[int], params: SamplingParams) -> TrainingSample:
        if not tokens:
            raise HTTPException(400, "empty prompt")
        try:
            return await asyncio.wrap_future(service.submit(tokens, params))
        except (AssertionError, ValueError) as e:
            raise HTTPException(400, str(e)) from e

    def tokens_of(prompt: Any) -> list[int]:
        if isinstance(prompt, list) and all(isinstance(t, int) for t in prompt):
            return prompt
        if isinstance(prompt, str) and tokenizer is not None:
            return list(tokenizer.encode(prompt))
        raise HTTPException(400, "prompt must be a list of token ids (or text when the server has a tokenizer)")

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/get_server_info")
    async def info():
        e = service.engine
        return {"model": model_name, "weight_version": e.get_weight_version(), "running": e.num_running(),
                "waiting": e.num_waiting(), "steps": service.steps, "cache": e.cache_stats()}

    @app.post("/generate")
    async def generate(body: dict):
        ids = body.get("input_ids")
        if ids is None:
            ids = tokens_of(body.get("text"))
        batched = bool(ids) and isinstance(ids[0], list)
        prompts = ids if batched else [ids]
        sp = body.get("sampling_params") or {}
        samples = await asyncio.gather(*(run(p, _params_from_sglang(sp)) for p in prompts))
        outs = [sglang_response(s, bool(body.get("return_logprob")), tokenizer) for s in samples]
        return outs if batched else outs[0]

    @app.post("/v1/completions")
    async def completions(body: dict):
        params = SamplingParams(temperature=float(body.get("temperature", 1.0)), max_tokens=int(body.get("max_tokens", 16)),
                                stop_token_ids=frozenset(body.get("stop_token_ids") or ()), seed=body.get("seed"))
        sample = await run(tokens_of(body.get("prompt")), params)
        return openai_completion_response(sample, body.get("model", model_name), body.get("logprobs") is not None, tokenizer)

    @app.post("/flush_cache")
    async def flush():
        await asyncio.get_running_loop().run_in_executor(None, service.flush_cache)
        return {"success": True}

    @app.post("/update_weights_from_disk")
    async def update(body: dict):
        path = body.get("model_path")
        if not path:
            raise HTTPException(400, "model_path is required")
        try:
            version = await asyncio.get_running_loop().run_in_executor(None, service.update_weights_from_path, path, weight_loader)
        except FileNotFoundError as e:
            raise HTTPException(404, str(e)) from e
        return {"success": True, "message": f"weights loaded from {path}", "weight_version": version}

    return app


def default_weight_loader(path: str) -> dict:
    import os

    import torch

    from ..models.weights import load_safetensors_dir

    if os.path.isdir(path):
        if any(f.endswith(".safetensors") for f in os.listdir(path)):
            return load_safetensors_dir(path)[0]       # (weights, config): the engine keeps its own config
        path = os.path.join(path, "pytorch_model.bin")
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    return torch.load(path, map_location="cpu", weights_only=True)


def serve(engine, host: str = "127.0.0.1", port: int = 30000, model_name: str = "native", tokenizer=None, group=None) -> None:
    """Blocks. With an initialised process group of more than one rank (tensor-parallel engine) rank 0 serves HTTP
    and the other ranks follow its schedule."""
    import torch.distributed as dist
    import uvicorn

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        service = LockstepEngineService(engine, group)
        if service.rank != 0:
            service.follow()
            return
    else:
        service = EngineService(engine)
    try:
        uvicorn.run(create_app(service, model_name, tokenizer), host=host, port=port, log_level="warning")
    finally:
        service.shutdown()
