"""Tools for checking a functional (class-free) forward pass against a module-based reference model, e.g. a Hugging
Face ``*ForCausalLM`` (rollouts/tools/functional_extractor: ``debug_toolkit.py:32-511``, ``test_template.py:30-381``,
``verify.py:265-561``).

* ``compare_tensors`` / ``per_position_diff``: how far two tensors are apart, overall and per sequence position.
* ``capture_internals``: forward hooks on the reference model that record every decoder layer's input and output,
  the rotary ``(cos, sin)`` pair and the attention mask the layers received.
* ``DebugSession``: targeted probes (embeddings, rotary tables, masks, whole forward) and ``find_divergence_layer``,
  which feeds each layer of the functional model the REFERENCE's input of that layer, so the first layer whose output
  differs is the one that is wrong, whatever happened before it.
* ``FunctionalModelTestSuite``: the standard battery (sequence lengths, batch sizes, edge cases, padding masks, dtypes).
* ``verify_functional``: one call that loads a reference model, runs the battery and returns a result; with
  ``remote=`` the same check is shipped as a script to another machine (a GPU node) through any object with
  ``exec(command) -> (exit_code, output)`` and ``push(local_dir)`` (``infra.bifrost.BifrostClient`` has both).
"""

from __future__ import annotations

import json
import time
from dataclasses import dataclass, field
from typing import Any, Callable

import torch
from torch import Tensor


# ------------------------------------------------------------------------------------------ comparisons
def compare_tensors(t1: Tensor, t2: Tensor, name: str = "tensor", rtol: float = 1e-5, atol: float = 1e-5) -> dict:
    """Shape / dtype agreement, maximum and mean absolute difference, where the maximum sits, and ``allclose``."""
    out: dict[str, Any] = {"name": name, "shape_match": t1.shape == t2.shape, "dtype_match": t1.dtype == t2.dtype,
                           "t1_shape": tuple(t1.shape), "t2_shape": tuple(t2.shape)}
    if not out["shape_match"]:
        out.update(matches=False, max_diff=float("inf"), mean_diff=float("inf"))
        return out
    a, b = t1.detach().float(), t2.detach().float()
    diff = (a - b).abs()
    flat = int(diff.argmax()) if diff.numel() else 0
    out.update(max_diff=float(diff.max()) if diff.numel() else 0.0, mean_diff=float(diff.mean()) if diff.numel() else 0.0,
               matches=bool(torch.allclose(a, b, rtol=rtol, atol=atol)), max_diff_idx=flat,
               max_diff_pos=tuple(int(i) for i in torch.unravel_index(torch.tensor(flat), diff.shape)) if diff.numel() else ())
    return out


def per_position_diff(t1: Tensor, t2: Tensor, attention_mask: Tensor | None = None) -> list[dict]:
    """Difference per sequence position of ``[batch, seq, ...]`` tensors; padding positions are flagged."""
    assert t1.shape == t2.shape, f"shape mismatch: {tuple(t1.shape)} vs {tuple(t2.shape)}"
    d = (t1.detach().float() - t2.detach().float()).abs().flatten(2) if t1.dim() > 2 else (t1.float() - t2.float()).abs()[..., None]
    out = []
    for pos in range(t1.shape[1]):
        pad = bool((attention_mask[:, pos] == 0).any()) if attention_mask is not None else False
        out.append({"position": pos, "max_diff": float(d[:, pos].max()), "mean_diff": float(d[:, pos].mean()), "is_padding": pad})
    return out


# ------------------------------------------------------------------------------------------ reference internals
@dataclass
class CapturedInternals:
    layer_inputs: dict[int, Tensor] = field(default_factory=dict)
    layer_outputs: dict[int, Tensor] = field(default_factory=dict)
    position_embeddings: tuple[Tensor, Tensor] | None = None
    position_ids: Tensor | None = None
    attention_mask: Tensor | None = None          # what the layers received (4-D additive / boolean mask or None)
    embeddings: Tensor | None = None
    logits: Tensor | None = None


def _decoder_layers(model) -> list:
    inner = getattr(model, "model", model)
    layers = getattr(inner, "layers", None)
    assert layers is not None, "reference model has no .model.layers"
    return list(layers)


def capture_internals(model, input_ids: Tensor, attention_mask: Tensor | None = None) -> CapturedInternals:
    """Run ``model`` once with hooks on its embedding and on every decoder layer."""
    cap = CapturedInternals()
    handles = []

    def pre(idx):
        def hook(module, args, kwargs):
            cap.layer_inputs[idx] = (args[0] if args else kwargs["hidden_states"]).detach()
            if idx == 0:
                pe = kwargs.get("position_embeddings")
                if pe is not None:
                    cap.position_embeddings = (pe[0].detach(), pe[1].detach())
                if kwargs.get("position_ids") is not None:
                    cap.position_ids = kwargs["position_ids"].detach()
                m = kwargs.get("attention_mask")
                cap.attention_mask = m.detach() if isinstance(m, Tensor) else None
        return hook

    def post(idx):
        def hook(module, args, kwargs, output):
            cap.layer_outputs[idx] = (output[0] if isinstance(output, (tuple, list)) else output).detach()
        return hook

    for i, layer in enumerate(_decoder_layers(model)):
        handles.append(layer.register_forward_pre_hook(pre(i), with_kwargs=True))
        handles.append(layer.register_forward_hook(post(i), with_kwargs=True))
    emb = getattr(getattr(model, "model", model), "embed_tokens", None)
    if emb is not None:
        handles.append(emb.register_forward_hook(lambda m, a, o: setattr(cap, "embeddings", o.detach())))
    try:
        with torch.no_grad():
            kw = {"attention_mask": attention_mask} if attention_mask is not None else {}
            out = model(input_ids, **kw)
            cap.logits = (out.logits if hasattr(out, "logits") else out).detach()
    finally:
        for h in handles:
            h.remove()
    return cap


# ------------------------------------------------------------------------------------------ debug session
@dataclass
class DebugSession:
    """``reference_model``: module-based model (called as ``model(input_ids, attention_mask=...)``, ``.logits``);
    ``functional_forward(input_ids, weights, attention_mask=None) -> logits``; ``weights``: the functional model's
    name -> tensor dict."""

    reference_model: Any
    functional_forward: Callable[..., Tensor]
    weights: dict[str, Tensor]
    embed_key: str = "model.embed_tokens.weight"

    def test_embeddings(self, input_ids: Tensor) -> dict:
        cap = capture_internals(self.reference_model, input_ids)
        mine = torch.nn.functional.embedding(input_ids, self.weights[self.embed_key])
        return compare_tensors(cap.embeddings, mine.to(cap.embeddings.dtype), "embeddings", 0.0, 0.0)

    def test_position_embeddings(self, input_ids: Tensor, rope_fn: Callable[[Tensor], tuple[Tensor, Tensor]],
                                 attention_mask: Tensor | None = None) -> dict:
        """``rope_fn(position_ids) -> (cos, sin)`` of the functional model, against what the reference's layers got."""
        cap = capture_internals(self.reference_model, input_ids, attention_mask)
        if cap.position_embeddings is None:
            return {"name": "position_embeddings", "matches": None, "note": "the reference passes no (cos, sin) to its layers"}
        pos = cap.position_ids if cap.position_ids is not None else torch.arange(input_ids.shape[1])[None].expand_as(input_ids)
        cos, sin = rope_fn(pos)
        rc, rs = cap.position_embeddings
        return {"name": "position_embeddings", "cos": compare_tensors(rc, cos.to(rc.dtype), "cos", 1e-5, 1e-5),
                "sin": compare_tensors(rs, sin.to(rs.dtype), "sin", 1e-5, 1e-5), "position_ids": pos[0].tolist(),
                "matches": bool(torch.allclose(rc.float(), cos.float(), atol=1e-5) and torch.allclose(rs.float(), sin.float(), atol=1e-5))}

    def test_attention_mask(self, input_ids: Tensor, attention_mask: Tensor, mask_fn: Callable[[Tensor], Tensor]) -> dict:
        """``mask_fn(attention_mask) -> [B, 1, T, T]`` boolean "may attend" mask of the functional model, against the
        mask the reference's layers received (additive masks count as allowed where finite and >= 0)."""
        cap = capture_internals(self.reference_model, input_ids, attention_mask)
        mine = mask_fn(attention_mask)
        ref = cap.attention_mask
        if ref is None:
            return {"name": "attention_mask", "matches": None, "note": "the reference hands its layers no explicit mask (causal kernel)"}
        allowed = ref if ref.dtype == torch.bool else (ref >= 0)
        same = allowed.expand_as(mine) == mine
        # rows of pure padding attend to nothing useful in either implementation: they do not count
        live_rows = attention_mask.bool()[:, None, :, None].expand_as(mine)
        bad = (~same) & live_rows
        return {"name": "attention_mask", "matches": not bool(bad.any()), "num_mismatches": int(bad.sum()), "ref_shape": tuple(ref.shape)}

    def compare_full_forward(self, input_ids: Tensor, attention_mask: Tensor | None = None, rtol: float = 1e-4, atol: float = 1e-4) -> dict:
        with torch.no_grad():
            kw = {"attention_mask": attention_mask} if attention_mask is not None else {}
            ref = self.reference_model(input_ids, **kw)
            ref = ref.logits if hasattr(ref, "logits") else ref
            mine = self.functional_forward(input_ids, self.weights, **kw)
        res = compare_tensors(ref, mine.to(ref.dtype), "logits", rtol, atol)
        if attention_mask is not None and res["shape_match"]:
            res["per_position"] = per_position_diff(ref, mine, attention_mask)
            live = [p["max_diff"] for p in res["per_position"] if not p["is_padding"]]
            res["max_diff_unpadded"] = max(live) if live else 0.0
        return res

    def find_divergence_layer(self, input_ids: Tensor, attention_mask: Tensor | None = None,
                              layer_forward_fn: Callable[..., Tensor] | None = None, threshold: float = 1e-4) -> dict:
        """``layer_forward_fn(hidden, weights, layer_idx, cos, sin, mask) -> hidden``: one layer of the functional
        model, fed the reference's input of that layer."""
        cap = capture_internals(self.reference_model, input_ids, attention_mask)
        res: dict[str, Any] = {"num_layers": len(cap.layer_outputs), "divergence_layer": None, "per_layer_diff": []}
        cos, sin = cap.position_embeddings if cap.position_embeddings is not None else (None, None)
        for idx in sorted(cap.layer_outputs):
            row: dict[str, Any] = {"layer": idx, "ref_output_shape": tuple(cap.layer_outputs[idx].shape)}
            if layer_forward_fn is not None and idx in cap.layer_inputs:
                with torch.no_grad():
                    mine = layer_forward_fn(cap.layer_inputs[idx], self.weights, idx, cos, sin, cap.attention_mask)
                c = compare_tensors(cap.layer_outputs[idx], mine.to(cap.layer_outputs[idx].dtype), f"layer_{idx}", 0.0, threshold)
                row.update(comparison=c, max_diff=c["max_diff"], matches=c["matches"])
                if not c["matches"] and res["divergence_layer"] is None:
                    res["divergence_layer"] = idx
            res["per_layer_diff"].append(row)
        return res


def format_comparison(c: dict) -> str:
    if not c.get("shape_match", True):
        return f"{c['name']}: SHAPE MISMATCH {c['t1_shape']} vs {c['t2_shape']}"
    return f"{c['name']}: {'ok' if c.get('matches') else 'DIFFERS'}  max {c.get('max_diff', 0):.3e}  mean {c.get('mean_diff', 0):.3e}"


def format_layer_report(res: dict) -> str:
    lines = [f"{res['num_layers']} layers; first divergence: {res['divergence_layer']}"]
    for row in res["per_layer_diff"]:
        if "max_diff" in row:
            lines.append(f"  layer {row['layer']:>3}  max diff {row['max_diff']:.3e}  {'ok' if row['matches'] else '<-- differs'}")
    return "\n".join(lines)


def quick_debug(reference_model, functional_forward, weights, input_ids: Tensor, attention_mask: Tensor | None = None,
                layer_forward_fn=None) -> dict:
    """Whole forward first; the layer hunt only when that differs."""
    s = DebugSession(reference_model, functional_forward, weights)
    out = {"full": s.compare_full_forward(input_ids, attention_mask)}
    if not out["full"]["matches"] and layer_forward_fn is not None:
        out["layers"] = s.find_divergence_layer(input_ids, attention_mask, layer_forward_fn)
    return out


# ------------------------------------------------------------------------------------------ the battery
@dataclass
class CaseResult:
    name: str
    passed: bool
    max_diff: float
    details: str = ""

    def __str__(self) -> str:
        return f"{'PASS' if self.passed else 'FAIL'}  {self.name:<40} max diff {self.max_diff:.3e}  {self.details}"


@dataclass
class SuiteResult:
    model_name: str
    results: list[CaseResult] = field(default_factory=list)
    seconds: float = 0.0

    @property
    def all_passed(self) -> bool:
        return all(r.passed for r in self.results)

    def __str__(self) -> str:
        n = sum(r.passed for r in self.results)
        return "\n".join([f"== {self.model_name}: {n}/{len(self.results)} passed in {self.seconds:.1f}s =="] + [str(r) for r in self.results])

    def to_dict(self) -> dict:
        return {"model": self.model_name, "all_passed": self.all_passed, "seconds": self.seconds,
                "results": [{"name": r.name, "passed": r.passed, "max_diff": r.max_diff, "details": r.details} for r in self.results]}


class FunctionalModelTestSuite:
    """The standard comparisons of a functional forward against its reference model."""

    def __init__(self, model_name: str, reference_model, functional_forward: Callable[..., Tensor], weights: dict[str, Tensor],
                 vocab_size: int, device: str = "cpu", tolerance: float = 1e-4, seed: int = 0):
        self.model_name, self.ref, self.fn, self.weights = model_name, reference_model, functional_forward, weights
        self.vocab, self.device, self.tol = vocab_size, device, tolerance
        self.gen = torch.Generator().manual_seed(seed)
        self.results: list[CaseResult] = []

    def _ids(self, batch: int, seq: int) -> Tensor:
        return torch.randint(0, self.vocab, (batch, seq), generator=self.gen).to(self.device)

    def run_case(self, name: str, input_ids: Tensor, attention_mask: Tensor | None = None, tolerance: float | None = None,
                 weights: dict | None = None, reference=None) -> CaseResult:
        tol = self.tol if tolerance is None else tolerance
        try:
            with torch.no_grad():
                kw = {"attention_mask": attention_mask} if attention_mask is not None else {}
                r = (self.ref if reference is None else reference)(input_ids, **kw)
                r = (r.logits if hasattr(r, "logits") else r).float()
                m = self.fn(input_ids, self.weights if weights is None else weights, **kw).float()
            if attention_mask is not None:          # padding positions carry no meaning in either implementation
                keep = attention_mask.bool()
                r, m = r[keep], m[keep]
            d = float((r - m).abs().max()) if r.numel() else 0.0
            res = CaseResult(name, d <= tol, d, f"tolerance {tol:.1e}")
        except Exception as e:  # noqa: BLE001 - a crashing case is a failed case, the battery goes on
            res = CaseResult(name, False, float("inf"), f"{type(e).__name__}: {e}")
        self.results.append(res)
        return res

    def test_sequence_lengths(self, seq_lengths=(1, 2, 7, 16, 64, 128)) -> None:
        for n in seq_lengths:
            self.run_case(f"seq_len={n}", self._ids(1, n))

    def test_batch_sizes(self, batch_sizes=(1, 2, 4), seq_len: int = 16) -> None:
        for b in batch_sizes:
            self.run_case(f"batch={b}", self._ids(b, seq_len))

    def test_edge_cases(self) -> None:
        self.run_case("all token 0", torch.zeros(1, 8, dtype=torch.long, device=self.device))
        self.run_case("highest token id", torch.full((1, 8), self.vocab - 1, dtype=torch.long, device=self.device))
        self.run_case("repeated token", torch.full((2, 12), min(5, self.vocab - 1), dtype=torch.long, device=self.device))
        self.run_case("ascending ids", (torch.arange(16, device=self.device) % self.vocab)[None])

    def test_attention_masks(self, seq_len: int = 12) -> None:
        ids = self._ids(2, seq_len)
        ones = torch.ones(2, seq_len, dtype=torch.long, device=self.device)
        self.run_case("mask: none padded", ids, ones)
        right = ones.clone()
        right[1, seq_len - 4:] = 0
        self.run_case("mask: right padding", ids, right)
        left = ones.clone()
        left[0, :3] = 0
        self.run_case("mask: left padding", ids, left)

    def test_dtypes(self, dtypes=(("float32", torch.float32, None), ("bfloat16", torch.bfloat16, 0.25))) -> None:
        """Other dtypes run on converted copies of both models; low precision gets a loose, stated tolerance."""
        import copy

        for label, dt, tol in dtypes:
            if dt == torch.float32:
                self.run_case("dtype=float32", self._ids(1, 16))
                continue
            try:
                ref = copy.deepcopy(self.ref).to(dt)
                w = {k: v.to(dt) if v.is_floating_point() else v for k, v in self.weights.items()}
            except Exception as e:  # noqa: BLE001
                self.results.append(CaseResult(f"dtype={label}", False, float("inf"), f"conversion failed: {e}"))
                continue
            self.run_case(f"dtype={label}", self._ids(1, 16), tolerance=tol, weights=w, reference=ref)

    def run_all(self) -> SuiteResult:
        t0 = time.time()
        self.results = []
        self.test_sequence_lengths()
        self.test_batch_sizes()
        self.test_edge_cases()
        self.test_attention_masks()
        self.test_dtypes()
        return SuiteResult(self.model_name, list(self.results), time.time() - t0)


# ------------------------------------------------------------------------------------------ one-call verification
@dataclass
class VerificationResult:
    model_name: str
    passed: bool
    suite: dict
    where: str = "local"
    error: str | None = None


def native_functional_forward(cfg) -> Callable[..., Tensor]:
    """This package's oracle (``models.functional.causal_lm_forward``) in the calling convention of the tools here:
    ``attention_mask [B, T]`` becomes position ids that skip padding (as Hugging Face computes them) and a causal
    mask that also hides padded keys."""
    from .functional import causal_lm_forward

    def forward(input_ids: Tensor, weights: dict, attention_mask: Tensor | None = None) -> Tensor:
        if attention_mask is None:
            return causal_lm_forward(input_ids, weights, cfg)
        am = attention_mask.bool()
        pos = (attention_mask.long().cumsum(-1) - 1).clamp(min=0)
        T = input_ids.shape[1]
        causal = torch.ones(T, T, dtype=torch.bool, device=input_ids.device).tril()
        allowed = causal[None, None] & am[:, None, None, :]
        # a fully masked row (a padding query) would give NaN: let it see itself, its output is ignored anyway
        allowed = allowed | torch.eye(T, dtype=torch.bool, device=input_ids.device)[None, None]
        return causal_lm_forward(input_ids, weights, cfg, positions=pos, attn_mask=allowed)

    return forward


def verify_functional(model_name: str, reference_model=None, functional_forward=None, weights: dict | None = None,
                      vocab_size: int | None = None, tolerance: float = 1e-4, remote=None, remote_python: str = "python",
                      workdir: str = ".") -> VerificationResult:
    """Run the battery for one model. Local: pass the reference model (or a Hugging Face name / path to load), the
    functional forward and its weights (by default this package's oracle on the reference's own ``state_dict``).
    Remote: ``remote`` runs the same call on another machine (``remote.push(local_dir)`` then
    ``remote.exec(command) -> (code, output)``) and the JSON it prints is parsed back."""
    if remote is not None:
        script = build_verification_script(model_name, tolerance)
        if hasattr(remote, "push"):
            remote.push(workdir)
        code, output = remote.exec(f"{remote_python} -c {json.dumps(script)}")
        for line in reversed(str(output).splitlines()):
            if line.startswith("{") and '"all_passed"' in line:
                suite = json.loads(line)
                return VerificationResult(model_name, bool(suite["all_passed"]) and code == 0, suite, "remote")
        return VerificationResult(model_name, False, {}, "remote", f"no result line (exit code {code}): {str(output)[-400:]}")
    if reference_model is None:
        from transformers import AutoModelForCausalLM

        reference_model = AutoModelForCausalLM.from_pretrained(model_name, torch_dtype=torch.float32).eval()
    if weights is None:
        weights = {k: v.detach() for k, v in reference_model.state_dict().items()}
    if functional_forward is None:
        from .config import ModelConfig

        functional_forward = native_functional_forward(ModelConfig.from_hf_dict(reference_model.config.to_dict()))
    vocab = vocab_size or int(reference_model.config.vocab_size)
    suite = FunctionalModelTestSuite(model_name, reference_model, functional_forward, weights, vocab, tolerance=tolerance).run_all()
    return VerificationResult(model_name, suite.all_passed, suite.to_dict())


def build_verification_script(model_name: str, tolerance: float = 1e-4) -> str:
    """Source of the program a remote machine runs: verify ``model_name`` there and print the suite as one JSON line."""
    return ("import json\n"
            "from research_b200.models.verify_tools import verify_functional\n"
            f"r = verify_functional({model_name!r}, tolerance={tolerance!r})\n"
            "print(json.dumps(r.suite))\n")
