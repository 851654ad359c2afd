"""Inference engine: continuous batching over a paged KV cache with prefix reuse.

Public API of the reference engine (rollouts/inference/engine.py:23-205): ``generate``,
``generate_text``, ``add_request``, ``step``, ``has_pending``, ``update_weights``,
``get_weight_version``, ``flush_cache``, ``shutdown``. What differs is everything underneath:
the reference re-runs the whole HF model per sequence per token with no KV cache; here a C++
core schedules and builds batches, prompts share cached prefixes through a radix tree or a
hash chain, prefill is one packed varlen pass and decode is one CUDA-graph replay per step.

One step = schedule -> [decode graph] + [prefill pass] -> one device->host copy of the sampled
tokens and log-probabilities -> commit (stop rules, block publication).
"""

from __future__ import annotations

import ctypes
from pathlib import Path

import torch

from .. import _native
from ..models.config import ModelConfig
from ..models.weights import load_safetensors_dir
from ..ops import check_status
from .model_runner import BLOCK, ModelRunner
from .types import EngineConfig, SamplingParams, TrainingSample

_LL, _I, _F, _VP, _ULL = ctypes.c_longlong, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_ulonglong
_CACHE_MODES = {"none": 0, "paged": 1, "radix": 2}


def _core_lib():
    lib = _native.load("rb_engine_core")
    if not getattr(lib, "_rbe_typed", False):
        lib.rbe_create.restype = _VP
        lib.rbe_create.argtypes = [_I] * 6
        lib.rbe_destroy.argtypes = [_VP]
        lib.rbe_add_request.restype = _LL
        lib.rbe_add_request.argtypes = [_VP, _VP, _I, _I, _F, _ULL, _VP, _I, _I]
        for f in ("rbe_num_waiting", "rbe_num_running", "rbe_num_free_blocks", "rbe_num_finished", "rbe_check_invariants"):
            getattr(lib, f).argtypes = [_VP]
        lib.rbe_schedule.argtypes = [_VP, _VP]
        lib.rbe_get_scheduled.argtypes = [_VP, _VP, _VP, _VP]
        lib.rbe_build_batch.argtypes = [_VP, _I] + [_VP] * 6 + [_I, _VP, _VP, _VP, _I, _I]
        lib.rbe_commit.argtypes = [_VP, _I, _VP, _VP, _I]
        lib.rbe_pop_finished.restype = _LL
        lib.rbe_pop_finished.argtypes = [_VP, _VP]
        lib.rbe_read_sequence.argtypes = [_VP, _LL, _VP, _VP, _I]
        lib.rbe_abort.argtypes = [_VP, _LL]
        lib.rbe_flush_cache.argtypes = [_VP]
        lib.rbe_stats.argtypes = [_VP, _VP]
        lib._rbe_typed = True
    return lib


class InferenceEngine:
    def __init__(self, config: EngineConfig, model_config: ModelConfig | None = None,
                 weights: dict[str, torch.Tensor] | None = None, tokenizer=None,
                 device: torch.device | str | None = None, tp=None, ep=None) -> None:
        assert config.block_size == BLOCK, "the KV kernels use 16-token blocks"
        assert config.max_batch_size > 0
        self.config = config
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda" if torch.cuda.is_available() else "cpu")
        if weights is None:
            assert config.model_path, "either weights or EngineConfig.model_path is required"
            weights, loaded_cfg = load_safetensors_dir(config.model_path)
            model_config = model_config or loaded_cfg
        assert model_config is not None
        self.model_config = model_config
        self.tokenizer = tokenizer
        if tokenizer is None and config.model_path and (Path(config.model_path) / "tokenizer.json").exists():
            try:
                from transformers import AutoTokenizer

                self.tokenizer = AutoTokenizer.from_pretrained(config.model_path)
            except Exception:  # tokenizer is optional for token-in/token-out use
                self.tokenizer = None
        self.max_tokens_per_batch = config.max_tokens_per_batch or min(config.max_batch_size * 512, 16384)
        on_gpu = self.device.type == "cuda"
        dtype = torch.bfloat16 if on_gpu else torch.float32
        num_blocks = config.num_kv_blocks or self._size_kv_cache(model_config, tp, ep)
        self.runner = ModelRunner(
            model_config, weights, device=self.device, num_kv_blocks=num_blocks, max_batch=config.max_batch_size,
            max_model_len=config.max_model_len, max_prefill_tokens=self.max_tokens_per_batch + 2 * BLOCK,
            use_cuda_graphs=config.use_cuda_graphs, graph_batch_sizes=config.graph_batch_sizes, tp=tp, ep=ep, dtype=dtype)
        # expert parallel: the engines of all ranks step together (see parallel/ep.py); every rank must then call
        # step() / generate() the same way, and a rank without work of its own runs idle passes
        self.ep = ep if (ep is not None and ep.world > 1) else None
        self.peers_pending = False
        self.idle_passes = 0
        self._lib = _core_lib()
        self._core = self._lib.rbe_create(num_blocks, BLOCK, _CACHE_MODES[config.cache_type], config.max_batch_size,
                                          self.max_tokens_per_batch, config.max_model_len)
        assert self._core, "engine core allocation failed"
        self.num_kv_blocks = num_blocks
        self.weight_version = 0
        self.steps = 0
        self._counts = (_I * 6)()
        self._info = (_I * 5)()
        self._seed_counter = config.seed * 1000003 + 12345
        self.eos_token_id = -1
        if not config.ignore_eos:
            self.eos_token_id = model_config.eos_token_id
            if self.tokenizer is not None and getattr(self.tokenizer, "eos_token_id", None) is not None:
                self.eos_token_id = int(self.tokenizer.eos_token_id)
        if on_gpu and config.use_cuda_graphs:
            self.runner.capture_graphs()
        # timing breakdown of the last step (host perf counters; device time is measured by callers)
        self.last_step_rows = (0, 0)

    # ---------------------------------------------------------------- sizing
    def _size_kv_cache(self, cfg: ModelConfig, tp, ep=None) -> int:
        tp_size = tp.world if tp is not None else 1
        per_block = cfg.num_layers * 2 * (cfg.num_kv_heads // tp_size) * BLOCK * cfg.head_dim * 2
        want_tokens = self.config.max_batch_size * self.config.max_model_len
        want = -(-want_tokens // BLOCK)
        if self.device.type == "cuda":
            free, _total = torch.cuda.mem_get_info(self.device)
            params = cfg.num_params()
            if ep is not None and ep.world > 1 and cfg.is_moe:     # an expert-parallel engine holds its own share of the experts only
                experts = (cfg.num_layers - cfg.first_k_dense_replace) * cfg.num_experts * 3 * cfg.hidden_size * cfg.moe_intermediate_size
                params -= experts - experts // ep.world
            weights_bytes = params * 2 // tp_size
            budget = int(free * self.config.gpu_memory_utilization) - weights_bytes - (4 << 30)
            cap = max(budget // per_block, 64)
            return int(max(64, min(want, cap, (48 << 30) // per_block)))
        return int(min(want, 4096))

    # ---------------------------------------------------------------- high-level API
    def generate(self, prompts: list[list[int]], sampling_params: SamplingParams,
                 num_samples_per_prompt: int = 1) -> list[TrainingSample]:
        """Generate ``num_samples_per_prompt`` completions per prompt; results in request order."""
        assert (len(prompts) > 0 or self.ep is not None) and num_samples_per_prompt > 0
        ids = []
        for prompt in prompts:
            for _ in range(num_samples_per_prompt):
                ids.append(self.add_request(list(prompt), sampling_params))
        done: dict[int, TrainingSample] = {}
        while True:                      # under expert parallelism all ranks leave the loop in the same iteration
            for sid, sample in self._step_with_ids():
                done[sid] = sample
            if not (self.peers_pending if self.ep is not None else self.has_pending()):
                break
        assert len(done) == len(ids)
        return [done[i] for i in ids]

    def generate_text(self, prompts: list[str], sampling_params: SamplingParams,
                      num_samples_per_prompt: int = 1) -> list[TrainingSample]:
        assert self.tokenizer is not None, "generate_text needs a tokenizer"
        toks = [self.tokenizer.encode(p, add_special_tokens=True) for p in prompts]
        return self.generate(toks, sampling_params, num_samples_per_prompt)

    # ---------------------------------------------------------------- mid-level API
    def add_request(self, prompt_tokens: list[int], params: SamplingParams) -> int:
        n = len(prompt_tokens)
        assert n > 0
        toks = (_I * n)(*prompt_tokens)
        stops = sorted(params.stop_token_ids)
        stop_arr = (_I * max(len(stops), 1))(*stops)
        if params.seed is not None:
            seed = params.seed
        else:
            self._seed_counter = (self._seed_counter * 6364136223846793005 + 1442695040888963407) & ((1 << 63) - 1)
            seed = self._seed_counter
        sid = self._lib.rbe_add_request(self._core, toks, n, params.max_tokens, float(params.temperature), seed,
                                        stop_arr, len(stops), self.eos_token_id)
        if sid < 0:
            raise ValueError(f"request of {n} + {params.max_tokens} tokens exceeds max_model_len={self.config.max_model_len}")
        return int(sid)

    def has_pending(self) -> bool:
        return self._lib.rbe_num_waiting(self._core) > 0 or self._lib.rbe_num_running(self._core) > 0

    def num_running(self) -> int:
        return self._lib.rbe_num_running(self._core)

    def num_waiting(self) -> int:
        return self._lib.rbe_num_waiting(self._core)

    def step(self) -> list[TrainingSample]:
        """One scheduling decision + forward pass; returns the sequences that finished."""
        return [s for _, s in self._step_with_ids()]

    def _step_with_ids(self) -> list[tuple[int, TrainingSample]]:
        lib, core, r = self._lib, self._core, self.runner
        mine = self.has_pending()
        if not mine and self.ep is None:
            return []
        n_prefill = n_decode = 0
        if mine:
            lib.rbe_schedule(core, self._counts)
            n_prefill, n_decode = self._counts[0], self._counts[1]
        self.last_step_rows = (n_prefill, n_decode)
        any_decode, any_prefill = n_decode > 0, n_prefill > 0
        if self.ep is not None:
            any_decode, any_prefill, pend = self.ep.agree(n_decode > 0, n_prefill > 0, mine)
            self.peers_pending = bool(pend)
        if mine and n_prefill + n_decode == 0 and self._counts[2] == 0:
            raise RuntimeError("scheduler made no progress: a request does not fit the KV cache")
        if any_decode and n_decode == 0:
            self._idle_pass()
        if any_prefill and n_prefill == 0:
            self._idle_pass()
        if n_prefill + n_decode == 0:
            return []
        mb = r.max_batch
        if n_decode > 0:
            mh = r.meta_host
            base = mh.data_ptr()
            T = lib.rbe_build_batch(
                core, 1, base, base + 4 * mb, base + 8 * mb, r.pf_host.data_ptr() + 4 * r._pf_offsets()["cu_q"],
                base + 12 * mb, r.bt_host.data_ptr(), r.max_blocks_per_seq, base + 16 * mb, base + 20 * mb,
                r.pf_host.data_ptr() + 4 * r._pf_offsets()["sample_rows"], mb, mb)
            assert T == n_decode, T
            max_blocks = self._max_blocks_in(r.meta_host[3 * mb:3 * mb + n_decode])
            r.stage_decode_padding(n_decode)
            r.decode(n_decode, max_blocks)
            self._sync()
            out_i = r.out_host
            fin = lib.rbe_commit(core, 1, out_i.data_ptr(), out_i.data_ptr() + 4 * mb, n_decode)
            assert fin >= 0
        if n_prefill > 0:
            o = r._pf_offsets()
            base = r.pf_host.data_ptr()
            T = lib.rbe_build_batch(
                core, 2, base + 4 * o["tokens"], base + 4 * o["positions"], base + 4 * o["slots"], base + 4 * o["cu_q"],
                base + 4 * o["seq_lens"], r.bt_host.data_ptr(), r.max_blocks_per_seq, base + 4 * o["temps"],
                base + 4 * o["seeds"], base + 4 * o["sample_rows"], r.max_prefill_tokens, mb)
            assert T > 0, f"prefill batch does not fit the staging buffers ({T})"
            cu = r.pf_host[o["cu_q"]:o["cu_q"] + n_prefill + 1]
            max_new = int((cu[1:] - cu[:-1]).max())
            max_blocks = self._max_blocks_in(r.pf_host[o["seq_lens"]:o["seq_lens"] + n_prefill])
            r.prefill(n_prefill, T, max_new, max_blocks, {})
            self._sync()
            out_i = r.out_host
            fin = lib.rbe_commit(core, 2, out_i.data_ptr(), out_i.data_ptr() + 4 * mb, n_prefill)
            assert fin >= 0
        self.steps += 1
        if self.device.type == "cuda" and self.steps % 256 == 0:
            check_status(self.device)
        return self._collect_finished()

    def _idle_pass(self) -> None:
        """A decode pass over padding rows only: it feeds every MoE layer one (tiny) batch, which is what the peers'
        dispatch / combine barriers of this phase wait for. Nothing is read back."""
        r = self.runner
        r.stage_decode_padding(0)
        r.decode(0, 1)
        self._sync()
        self.idle_passes += 1

    def global_pending(self) -> bool:
        """True while this rank, or under expert parallelism any rank (as of the last step), still has work."""
        return self.has_pending() or (self.ep is not None and self.peers_pending)

    @staticmethod
    def _max_blocks_in(seq_lens: torch.Tensor) -> int:
        return int(-(-int(seq_lens.max()) // BLOCK))

    def _sync(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()

    def _collect_finished(self) -> list[tuple[int, TrainingSample]]:
        out = []
        lib, core = self._lib, self._core
        while lib.rbe_num_finished(core) > 0:
            sid = lib.rbe_pop_finished(core, self._info)
            n_prompt, n_total, reason, n_cached = self._info[0], self._info[1], self._info[2], self._info[3]
            toks = (_I * n_total)()
            lps = (_F * max(n_total - n_prompt, 1))()
            lib.rbe_read_sequence(core, sid, toks, lps, 1)
            out.append((int(sid), TrainingSample(
                prompt_tokens=tuple(toks[:n_prompt]), completion_tokens=tuple(toks[n_prompt:n_total]),
                logprobs=tuple(lps[: n_total - n_prompt]), ref_logprobs=None, weight_version=self.weight_version,
                finish_reason="stop" if reason == 1 else "length", cached_tokens=n_cached)))
        return out

    def abort(self, seq_id: int) -> None:
        self._lib.rbe_abort(self._core, seq_id)

    # ---------------------------------------------------------------- weights / cache
    def update_weights(self, state_dict: dict, blocking: bool = True) -> None:
        """Load new weights in place (captured graphs stay valid), bump the version, drop cached prefixes."""
        assert state_dict, "empty state_dict"
        assert not self.has_pending(), "update_weights while requests are in flight"
        self.runner.load_weights(state_dict)
        if blocking:
            self._sync()
        self.weight_version += 1
        self.flush_cache()

    def get_weight_version(self) -> int:
        return self.weight_version

    def flush_cache(self) -> None:
        """Invalidate every cached prefix (KV computed with old weights must not be reused)."""
        self._lib.rbe_flush_cache(self._core)

    def cache_stats(self) -> dict:
        s = (_LL * 5)()
        self._lib.rbe_stats(self._core, s)
        return {"hit_tokens": s[0], "miss_tokens": s[1], "evictions": s[2], "free_blocks": s[3], "evictable_blocks": s[4]}

    def check_invariants(self) -> int:
        return self._lib.rbe_check_invariants(self._core)

    def shutdown(self) -> None:
        core, self._core = getattr(self, "_core", None), None
        if core:
            self._lib.rbe_destroy(core)
        self.runner = None

    def __del__(self) -> None:
        try:
            self.shutdown()
        except Exception:
            pass
