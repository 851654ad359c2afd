"""Correctness / speed harness for alternative implementations of one kernel (dev/kernels-gpumode/kernel_utils:
task.py:29-92 case tiers, backends.py:45-138 registry, utils.py:15-279 closeness check + benchmark + comparison,
results.py:13-217 result records, smoke_test.py:59-398 driver).

A *backend* is a callable ``inputs -> tensor``. Every backend is checked against the one registered as ``reference``
on freshly generated inputs (a backend may overwrite its inputs) and timed; the results carry per-case errors and
speedups, render as a table and round-trip through JSON. The NVFP4 block-scaled GEMV ships as the built-in task:
``reference`` is the decode-and-dot formula in PyTorch, ``native`` the sm_100a kernel of ``csrc/quant_sm100.cu``.

    python -m research_b200.utils.kernel_harness --tier smoke --backends reference,native --json out.json
"""

from __future__ import annotations

import argparse
import json
import math
import statistics
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Sequence

import torch

LANGUAGES = ("pytorch", "cuda", "cutlass", "other")


# ---------------------------------------------------------------------------------------------------- cases

@dataclass(frozen=True)
class GemvCase:
    """One NVFP4 GEMV problem: ``a [l, m, k]`` times ``b [l, k]`` -> ``c [l, m]`` (e2m1 data, e4m3 scale per 16)."""
    m: int
    k: int
    l: int
    seed: int
    name: str

    def __post_init__(self) -> None:
        if min(self.m, self.k, self.l) <= 0 or self.k % 16 or self.seed < 0 or not self.name:
            raise ValueError(f"bad case {self}")

    def generate(self, device: str = "cpu") -> tuple[torch.Tensor, ...]:
        """Fresh ``(a, b, sfa, sfb)`` uint8 tensors; the same seed gives the same bytes on every device."""
        from ..ops.nvfp4 import quantize_nvfp4

        g = torch.Generator().manual_seed(self.seed)
        a, sfa = quantize_nvfp4(torch.randn(self.l, self.m, self.k, generator=g))
        b, sfb = quantize_nvfp4(torch.randn(self.l, self.k, generator=g))
        return tuple(t.contiguous().to(device) for t in (a, b, sfa, sfb))

    def bytes_moved(self) -> int:
        return self.l * (self.m * self.k // 2 + self.m * self.k // 16 + self.k // 2 + self.k // 16 + 2 * self.m)

    def describe(self) -> str:
        return f"m={self.m}, k={self.k}, l={self.l}, seed={self.seed}"


SMOKE = [GemvCase(128, 256, 1, 42, "tiny_single"), GemvCase(256, 512, 2, 43, "small_batch")]
CORRECTNESS = [GemvCase(128, 256, 1, 100, "min_size"), GemvCase(256, 512, 4, 101, "medium"),
               GemvCase(512, 1024, 8, 102, "large"), GemvCase(1024, 2048, 16, 103, "xlarge")]
PERFORMANCE = [GemvCase(512, 2048, 32, 200, "perf_medium"), GemvCase(1024, 4096, 64, 201, "perf_large")]
TIERS = {"smoke": SMOKE, "correctness": CORRECTNESS, "performance": PERFORMANCE}
# "published": the two shapes of the reference's profiler traces, checked AND timed (per call; the library backend
# launches once per batch entry, so its time per launch is the call time divided by l)


# ------------------------------------------------------------------------------------------------- backends

@dataclass
class Backend:
    name: str
    fn: Callable[[tuple], torch.Tensor]
    description: str = ""
    language: str = "other"
    needs_cuda: bool = False

    def __call__(self, inputs: tuple) -> torch.Tensor:
        return self.fn(inputs)


class BackendRegistry:
    """Named implementations of one kernel. Names are unique; ``reference`` is the oracle of ``run_suite``."""

    def __init__(self) -> None:
        self._items: dict[str, Backend] = {}

    def register(self, name: str, fn: Callable[[tuple], torch.Tensor], description: str = "", language: str = "other",
                 needs_cuda: bool = False) -> Backend:
        if not name or name in self._items:
            raise ValueError(f"backend name {name!r} is empty or taken")
        if not callable(fn) or language not in LANGUAGES:
            raise ValueError(f"backend {name!r}: fn must be callable and language one of {LANGUAGES}")
        self._items[name] = Backend(name, fn, description, language, needs_cuda)
        return self._items[name]

    def __getitem__(self, name: str) -> Backend:
        if name not in self._items:
            raise KeyError(f"no backend {name!r}; registered: {sorted(self._items)}")
        return self._items[name]

    def __contains__(self, name: str) -> bool:
        return name in self._items

    def __len__(self) -> int:
        return len(self._items)

    def names(self) -> list[str]:
        return list(self._items)

    def listing(self) -> str:
        w = max((len(n) for n in self._items), default=4)
        return "\n".join(f"{b.name:<{w}}  [{b.language}]  {b.description}" for b in self._items.values())


def nvfp4_backends() -> BackendRegistry:
    from ..ops import nvfp4

    reg = BackendRegistry()
    reg.register("reference", lambda x: nvfp4.nvfp4_gemv_reference(*x), "decode to fp64 and dot, rounded to fp16", "pytorch")
    reg.register("native", lambda x: nvfp4.nvfp4_gemv(*x), "sm_100a kernel: cvt.e2m1x2 + HFMA2, one warp per row slice", "cuda",
                 needs_cuda=True)
    reg.register("library_scaled_mm", _LibraryScaledMM(), "torch._scaled_mm block-scaled fp4 GEMM, b padded to 128 columns, one call per batch "
                 "entry (the reference's own baseline, dev/kernels-gpumode/nvfp4/reference_kernel.py:28-55); informational", "pytorch", needs_cuda=True)
    return reg


def blocked_scales(sf: torch.Tensor) -> torch.Tensor:
    """``[rows, cols]`` scale factors (rows % 128 == 0, cols % 4 == 0) in the layout the library's block-scaled GEMM reads:
    tiles of 128 rows x 4 columns, row-tile major; inside a tile the byte of (row r, column c) sits at
    ``(r % 32) * 16 + (r // 32) * 4 + c``."""
    rows, cols = sf.shape
    assert rows % 128 == 0 and cols % 4 == 0, (rows, cols)
    t = sf.reshape(rows // 128, 4, 32, cols // 4, 4)        # (row tile, r // 32, r % 32, column tile, c)
    return t.permute(0, 3, 2, 1, 4).reshape(-1).contiguous()


class _LibraryScaledMM:
    """The GEMV through the library GEMM, as the reference's baseline does it: the vector becomes a 128-column matrix
    (column 0 holds it), scales go into the blocked layout, and every batch entry is one ``torch._scaled_mm`` launch.
    The re-layout is cached per input (it is not part of what is timed)."""

    def __init__(self) -> None:
        self._key = None
        self._prep = None

    def _prepare(self, a, b, sfa, sfb):
        L, M, kb = a.shape
        if M % 128 or (kb // 8) % 4:
            raise ValueError(f"the blocked scale layout needs m % 128 == 0 and k % 64 == 0 (m={M}, k={kb * 2})")
        fp4, f8 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
        prep = []
        for i in range(L):
            b128 = torch.zeros(128, kb, dtype=torch.uint8, device=a.device)
            b128[0] = b[i]
            sb128 = torch.zeros(128, kb // 8, dtype=torch.uint8, device=a.device)
            sb128[0] = sfb[i]
            prep.append((a[i].view(fp4), b128.view(fp4).t(), blocked_scales(sfa[i]).view(f8), blocked_scales(sb128).view(f8)))
        return prep

    def __call__(self, inputs: tuple) -> torch.Tensor:
        a, b, sfa, sfb = inputs
        key = (a.data_ptr(), b.data_ptr(), tuple(a.shape))
        if key != self._key:
            self._prep, self._key = self._prepare(a, b, sfa, sfb), key
        out = torch.empty(a.shape[0], a.shape[1], dtype=torch.float16, device=a.device)
        for i, (ai, bi, sa, sb) in enumerate(self._prep):
            out[i] = torch._scaled_mm(ai, bi, sa, sb, bias=None, out_dtype=torch.float16)[:, 0]
        return out


# --------------------------------------------------------------------------------------------------- checks

def closeness(got: torch.Tensor, want: torch.Tensor, rtol: float = 1e-3, atol: float = 1e-3, max_print: int = 5) -> tuple[bool, str]:
    """``(ok, report)``; the report names shape / non-finite mismatches or the worst offending elements."""
    if got.shape != want.shape:
        return False, f"shape {tuple(got.shape)} != {tuple(want.shape)}"
    g, w = got.detach().double().cpu(), want.detach().double().cpu()
    if not bool(torch.equal(torch.isfinite(g), torch.isfinite(w))):
        return False, "non-finite values differ"
    fin = torch.isfinite(w)
    err = torch.where(fin, (g - w).abs(), torch.zeros_like(w))
    bad = err > atol + rtol * torch.where(fin, w.abs(), torch.zeros_like(w))
    n_bad = int(bad.sum())
    if n_bad == 0:
        return True, f"max abs err {float(err.max()) if err.numel() else 0.0:.3e}"
    idx = torch.nonzero(bad)[:max_print]
    lines = [f"{n_bad} of {w.numel()} elements differ (max abs err {float(err.max()):.3e})"]
    lines += [f"  at {tuple(i.tolist())}: got {float(g[tuple(i)]):.6g}, want {float(w[tuple(i)]):.6g}" for i in idx]
    return False, "\n".join(lines)


def benchmark(fn: Callable[[], Any], device: str = "cpu", warmup: int = 3, iters: int = 20) -> float:
    """Median milliseconds per call: CUDA events with an L2 flush between calls on a GPU, ``perf_counter`` on CPU."""
    if str(device).startswith("cuda"):
        from .timing import time_cuda

        return time_cuda(fn, iters=iters, warmup=warmup, flush=True)["median_ms"]
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        t0 = time.perf_counter()
        fn()
        times.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(times)


# -------------------------------------------------------------------------------------------------- results

def profile_kernel(fn: Callable[[], Any], device: str = "cpu", warmup: int = 2, iters: int = 5, row_limit: int = 12, trace_path: str | Path | None = None) -> str:
    """A ``torch.profiler`` table of what one backend call launches (operators on CPU, kernels with their device time on a
    GPU), optionally with a Chrome trace written to ``trace_path`` (dev/kernels-gpumode/kernel_utils/utils.py:282-352)."""
    from torch.profiler import ProfilerActivity, profile

    for _ in range(warmup):
        fn()
    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if device.startswith("cuda") else [])
    with profile(activities=acts) as prof:
        for _ in range(iters):
            fn()
        if device.startswith("cuda"):
            torch.cuda.synchronize()
    if trace_path is not None:
        prof.export_chrome_trace(str(trace_path))
    key = "cuda_time_total" if device.startswith("cuda") else "cpu_time_total"
    return prof.key_averages().table(sort_by=key, row_limit=row_limit)


def ncu_command(script_argv: Sequence[str], kernel_regex: str, out: str = "prof", launches: int = 3, skip: int = 0, full: bool = True,
                sections: Sequence[str] = ("SpeedOfLight", "MemoryWorkloadAnalysis")) -> list[str]:
    """The Nsight Compute command line for one kernel of a harness run (it is returned, not executed: profiling runs
    where the GPU is). Clocks are left alone, the capture is bounded to ``launches`` launches of the kernels that match."""
    cmd = ["ncu", "--clock-control", "none", "-k", f"regex:{kernel_regex}", "-c", str(launches)]
    if skip:
        cmd += ["-s", str(skip)]
    cmd += ["--set", "full"] if full else [x for s in sections for x in ("--section", s)]
    return cmd + ["-o", out, *script_argv]


@dataclass
class CorrectnessResult:
    case: str
    params: str
    ok: bool
    detail: str = ""


@dataclass
class PerformanceResult:
    case: str
    params: str
    ms: float
    reference_ms: float
    gbs: float = 0.0

    @property
    def speedup(self) -> float:
        return self.reference_ms / self.ms if self.ms > 0 else float("nan")


@dataclass
class BackendResults:
    backend: str
    correctness: list[CorrectnessResult] = field(default_factory=list)
    performance: list[PerformanceResult] = field(default_factory=list)
    skipped: str = ""

    @property
    def correctness_score(self) -> float:
        return sum(c.ok for c in self.correctness) / len(self.correctness) if self.correctness else 0.0

    @property
    def all_correct(self) -> bool:
        return bool(self.correctness) and all(c.ok for c in self.correctness)

    @property
    def avg_speedup(self) -> float:
        s = [p.speedup for p in self.performance if math.isfinite(p.speedup)]
        return statistics.fmean(s) if s else float("nan")

    @property
    def geomean_speedup(self) -> float:
        s = [p.speedup for p in self.performance if math.isfinite(p.speedup) and p.speedup > 0]
        return math.exp(statistics.fmean(math.log(x) for x in s)) if s else float("nan")

    def summary(self) -> str:
        if self.skipped:
            return f"{self.backend}: skipped ({self.skipped})"
        ok = sum(c.ok for c in self.correctness)
        line = f"{self.backend}: {ok}/{len(self.correctness)} correct"
        if self.performance:
            line += f", speedup vs reference avg {self.avg_speedup:.2f}x geomean {self.geomean_speedup:.2f}x"
        return line

    def to_dict(self) -> dict:
        return {"backend": self.backend, "skipped": self.skipped, "correctness": [asdict(c) for c in self.correctness],
                "performance": [asdict(p) for p in self.performance]}

    @classmethod
    def from_dict(cls, d: dict) -> "BackendResults":
        return cls(d["backend"], [CorrectnessResult(**c) for c in d.get("correctness", [])],
                   [PerformanceResult(**p) for p in d.get("performance", [])], d.get("skipped", ""))


@dataclass
class SuiteResults:
    backends: list[BackendResults] = field(default_factory=list)
    device: str = "cpu"

    def get(self, name: str) -> BackendResults | None:
        return next((b for b in self.backends if b.backend == name), None)

    def table(self) -> str:
        rows = [("backend", "correct", "avg speedup", "geomean", "best GB/s")]
        for b in self.backends:
            if b.skipped:
                rows.append((b.backend, "skipped", "-", "-", "-"))
                continue
            best = max((p.gbs for p in b.performance), default=0.0)
            rows.append((b.backend, f"{sum(c.ok for c in b.correctness)}/{len(b.correctness)}",
                         f"{b.avg_speedup:.2f}x" if b.performance else "-", f"{b.geomean_speedup:.2f}x" if b.performance else "-",
                         f"{best:.0f}" if best else "-"))
        w = [max(len(r[i]) for r in rows) for i in range(5)]
        out = ["  ".join(c.ljust(w[i]) for i, c in enumerate(r)) for r in rows]
        out.insert(1, "  ".join("-" * x for x in w))
        return "\n".join(out)

    def to_dict(self) -> dict:
        return {"device": self.device, "backends": [b.to_dict() for b in self.backends]}

    def to_json(self, path: str | Path) -> None:
        Path(path).write_text(json.dumps(self.to_dict(), indent=2))

    @classmethod
    def from_json(cls, path: str | Path) -> "SuiteResults":
        d = json.loads(Path(path).read_text())
        return cls([BackendResults.from_dict(b) for b in d["backends"]], d.get("device", "cpu"))


# --------------------------------------------------------------------------------------------------- driver

def run_suite(registry: BackendRegistry, names: Sequence[str] | None = None, correctness_cases: Sequence[GemvCase] = tuple(SMOKE),
              performance_cases: Sequence[GemvCase] = (), device: str = "cpu", rtol: float = 1e-3, atol: float = 1e-3,
              iters: int = 20, log: Callable[[str], None] | None = None) -> SuiteResults:
    """Check and time the chosen backends against ``registry['reference']``. A backend that raises fails that case
    (the message is kept) instead of ending the run; one that needs CUDA is skipped on a CPU device."""
    say = log or (lambda s: None)
    ref = registry["reference"]
    on_gpu = str(device).startswith("cuda")
    out = SuiteResults(device=str(device))
    ref_ms: dict[str, float] = {}
    for name in names or registry.names():
        be = registry[name]
        res = BackendResults(name)
        out.backends.append(res)
        if be.needs_cuda and not on_gpu:
            res.skipped = "needs a CUDA device"
            say(res.summary())
            continue
        for case in correctness_cases:
            want = ref(case.generate(device))
            try:
                ok, detail = closeness(be(case.generate(device)), want, rtol, atol)
            except Exception as e:  # a broken backend is a result, not a crash of the harness
                ok, detail = False, f"{type(e).__name__}: {e}"
            res.correctness.append(CorrectnessResult(case.name, case.describe(), ok, detail))
            say(f"  {name:<12} {case.name:<14} {'ok  ' if ok else 'FAIL'} {detail.splitlines()[0] if detail else ''}")
        for case in performance_cases:
            if case.name not in ref_ms:
                x = case.generate(device)
                ref_ms[case.name] = benchmark(lambda: ref(x), device, iters=iters)
            if name == "reference":
                ms = ref_ms[case.name]
            else:
                x = case.generate(device)
                try:
                    ms = benchmark(lambda: be(x), device, iters=iters)
                except Exception as e:
                    say(f"  {name:<12} {case.name:<14} benchmark failed: {type(e).__name__}: {e}")
                    continue
            res.performance.append(PerformanceResult(case.name, case.describe(), ms, ref_ms[case.name],
                                                     case.bytes_moved() / (ms * 1e-3) / 1e9 if ms > 0 else 0.0))
            say(f"  {name:<12} {case.name:<14} {ms * 1e3:9.1f} us  {res.performance[-1].speedup:6.2f}x  {res.performance[-1].gbs:7.0f} GB/s")
        say(res.summary())
    return out


def main(argv: Sequence[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--tier", choices=[*TIERS, "all", "published"], default="smoke")
    ap.add_argument("--backends", default="", help="comma-separated names (default: all registered)")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default="", help="write the results here")
    ap.add_argument("--list", action="store_true")
    a = ap.parse_args(argv)
    reg = nvfp4_backends()
    if a.list:
        print(reg.listing())
        return 0
    if a.tier == "all":
        corr, perf = SMOKE + CORRECTNESS, PERFORMANCE
    elif a.tier == "performance":
        corr, perf = SMOKE, PERFORMANCE
    elif a.tier == "published":
        corr, perf = SMOKE, SMOKE
    else:
        corr, perf = TIERS[a.tier], []
    names = [n for n in a.backends.split(",") if n] or None
    res = run_suite(reg, names, corr, perf, a.device, iters=a.iters, log=print)
    print(res.table())
    if a.json:
        res.to_json(a.json)
    # the library backend is a comparison point: an image whose library lacks the fp4 GEMM must not fail the run
    return 0 if all(b.all_correct or b.skipped or b.name.startswith("library_") for b in res.backends) else 1


if __name__ == "__main__":
    raise SystemExit(main())
