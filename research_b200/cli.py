"""Command line: ``python -m research_b200.cli <command>`` (rollouts/cli.py:117-1457, run_eval.py).

    serve     start the native engine behind the HTTP front end
    chat      talk to a model (any provider) with an agent preset; sessions are stored and resumable
    sessions  list / show / export / slice / import stored sessions
    eval      run a JSONL dataset through an agent and score it with a dotted-path score function
    bench     the flagship benchmark (same as the repository's bench.py)
    build     compile the native libraries
"""

from __future__ import annotations

import argparse
import asyncio
import importlib
import json
import os
import sys
from pathlib import Path


def _store(args):
    from .agents.store import FileSessionStore

    return FileSessionStore(args.store or os.path.join(os.path.expanduser("~"), ".research_b200", "sessions"))


def _run_coro(coro):
    """Run a coroutine to completion from synchronous code, also when the caller is itself inside a running loop."""
    try:
        asyncio.get_running_loop()
    except RuntimeError:
        return asyncio.run(coro)
    from concurrent.futures import ThreadPoolExecutor

    with ThreadPoolExecutor(1) as pool:
        return pool.submit(asyncio.run, coro).result()


def _endpoint(args):
    from .agents.dtypes import Endpoint

    provider, model = args.provider, args.model or ""
    if "/" in model:      # --model anthropic/claude-... names the provider too, when the part before the slash is one
        from .agents.providers import NonRetryableError, get_provider

        try:
            get_provider(model.split("/", 1)[0])
            provider, model = parse_model_string(model)
        except NonRetryableError:
            pass          # an organisation prefix of a model name (meta-llama/...), not a provider
    oauth_token, extra = "", {}
    if getattr(args, "oauth", ""):          # a stored subscription log-in takes the place of the API key
        from .agents.oauth import OAuthApp, OAuthClient

        client = OAuthClient(OAuthApp.load(args.oauth))
        oauth_token = _run_coro(client.get_valid_access_token()) or ""
        if not oauth_token:
            raise SystemExit(f"not logged in to {args.oauth!r} (or the log-in was revoked): run `research_b200 auth login {args.oauth}`")
        extra["oauth_app"] = args.oauth
        if client.app.request_headers:
            extra["request_headers"] = dict(client.app.request_headers)
    return Endpoint(provider=provider, model=model, api_base=args.api_base or "",
                    api_key=os.environ.get(args.api_key_env or "", "") if args.api_key_env and not oauth_token else "",
                    oauth_token=oauth_token, max_tokens=args.max_tokens, temperature=args.temperature, extra_params=extra)


def _add_endpoint_args(p: argparse.ArgumentParser) -> None:
    p.add_argument("--provider", default="openai", help="native | sglang | vllm | openai | openai-stream | openai-responses | anthropic | google")
    p.add_argument("--model", default="")
    p.add_argument("--api-base", default="")
    p.add_argument("--api-key-env", default="", help="name of the environment variable that holds the API key")
    p.add_argument("--oauth", default="", help="name of a configured OAuth application whose stored log-in replaces the API key")
    p.add_argument("--max-tokens", type=int, default=1024)
    p.add_argument("--temperature", type=float, default=1.0)


def load_object(path: str):
    """``package.module:attr`` or ``path/to/file.py:attr``."""
    mod_name, _, attr = path.partition(":")
    assert attr, "expected module:attribute"
    if mod_name.endswith(".py"):
        spec = importlib.util.spec_from_file_location(Path(mod_name).stem, mod_name)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    else:
        mod = importlib.import_module(mod_name)
    return getattr(mod, attr)


# ------------------------------------------------------------------------------------------ commands
def cmd_build(args) -> int:
    from . import _native

    for path in _native.build_all(force=args.force):
        print(path)
    return 0


def cmd_serve(args) -> int:
    import torch

    from .inference import EngineConfig, InferenceEngine
    from .inference.server import serve
    from .models import get_preset, init_random_weights
    from .models.weights import load_safetensors_dir

    device = "cuda" if torch.cuda.is_available() else "cpu"
    if os.path.isdir(args.model):
        from .models.config import ModelConfig

        cfg = ModelConfig.from_hf_dict(json.loads((Path(args.model) / "config.json").read_text()))
        weights = load_safetensors_dir(args.model)
        tokenizer = None
        try:
            from transformers import AutoTokenizer

            tokenizer = AutoTokenizer.from_pretrained(args.model)
        except Exception:  # noqa: BLE001 - token-id requests work without a tokenizer
            pass
    else:
        cfg = get_preset(args.model)
        weights = init_random_weights(cfg, seed=0, dtype=torch.bfloat16 if device == "cuda" else torch.float32, device=device)
        tokenizer = None
    ecfg = EngineConfig(cache_type=args.cache, max_batch_size=args.max_batch_size, max_model_len=args.max_model_len,
                        gpu_memory_utilization=args.gpu_memory_utilization, tensor_parallel_size=args.tp)
    tp = group = None
    if args.tp > 1:       # launched with torch.distributed.run: one rank per GPU, rank 0 serves HTTP
        import torch.distributed as dist

        from .parallel.symm import PeerComm
        from .parallel.tp import TensorParallel

        local = int(os.environ.get("LOCAL_RANK", "0"))
        if device == "cuda":
            torch.cuda.set_device(local)
            device = f"cuda:{local}"
        if not dist.is_initialized():
            dist.init_process_group("nccl" if device != "cpu" else "gloo")
        from datetime import timedelta

        # request broadcast travels on a CPU-side group; rank 0 heartbeats every few seconds when idle, so this
        # timeout only fires when a rank is gone
        group = dist.new_group(backend="gloo", timeout=timedelta(seconds=120))
        tp = TensorParallel(PeerComm(device=torch.device(device)), max_rows=ecfg.max_batch_size * 64 + 64, max_cols=max(cfg.hidden_size, 1024))
    engine = InferenceEngine(ecfg, cfg, weights, device=device, tp=tp)
    if tp is None or tp.rank == 0:
        print(f"serving {args.model} on http://{args.host}:{args.port} ({device}, tp={args.tp})", flush=True)
    serve(engine, args.host, args.port, args.model, tokenizer, group=group)
    return 0


async def _chat(args) -> int:
    from .agents.agents import resume_session
    from .agents.presets import PRESETS, AgentPreset, get_preset, list_presets, load_preset
    from .frontend.terminal import InteractiveRunner, make_frontend

    if args.list_presets:
        for p in PRESETS.values():
            print(f"{p.name:<20} {p.description}  (max {p.max_turns} turns)")
        for name in list_presets():
            pc = load_preset(name)
            print(f"{name:<28} {pc.description or pc.env}  [{pc.model}]")
        return 0
    preset = get_preset(args.preset)
    if args.preset not in PRESETS:              # a preset file also names its model; --model / --temperature still win
        pc = load_preset(args.preset)
        if not args.model:
            args.model = pc.model
        if pc.temperature is not None and args.temperature == 1.0:
            args.temperature = pc.temperature
        if args.tools:
            from dataclasses import replace as _replace

            preset = _replace(pc, tools=args.tools).to_preset()
    elif args.tools and args.preset in ("coding", "coding-interactive"):
        from .agents.presets import ENVIRONMENTS

        preset = AgentPreset(preset.name, preset.description, preset.system_prompt, lambda cwd: ENVIRONMENTS[args.preset](cwd, args.tools), preset.max_turns)
    if args.env:
        # --env coding+ask_user: the preset's prompt and turn budget, with these environments instead of the preset's own
        from .agents.presets import environment_from_spec

        environment_from_spec(args.env, args.cwd, args.tools or None)          # fail now on a bad spec
        preset = AgentPreset(preset.name, preset.description, preset.system_prompt, lambda cwd: environment_from_spec(args.env, cwd, args.tools or None),
                             max(preset.max_turns, 30))
    ep = _endpoint(args)
    store = None if args.no_session else _store(args)
    frontend = make_frontend("json" if args.stream_json else ("plain" if args.quiet and args.frontend == "auto" else args.frontend),
                             auto_confirm=args.yes)
    system_prompt = preset.system_prompt
    if args.system_prompt:
        system_prompt = Path(args.system_prompt).read_text() if os.path.isfile(args.system_prompt) else args.system_prompt
    elif args.full_prompt:
        # assembled for this run: the preset's prompt, what the environment says about itself, the tools it really offers
        # and the rules that follow from them, where the program's own documentation is, project context files, time, cwd
        from .agents.prompt import build_system_prompt

        probe = preset.environment(args.cwd)
        tools = probe.get_tools() if probe is not None and hasattr(probe, "get_tools") else []
        own = probe.get_system_prompt() if hasattr(probe, "get_system_prompt") else None
        name = probe.get_name() if hasattr(probe, "get_name") else preset.name
        system_prompt = build_system_prompt(name, tools, Path(args.cwd).resolve(), base_prompt=preset.system_prompt, env_system_prompt=own)
    context = [c for c in (args.context or [])] + [f"# {f}\n{Path(f).read_text()}" for f in (args.context_file or [])]
    if context:
        system_prompt = system_prompt + "\n\n" + "\n\n".join(context)
    trajectory = session_id = None
    if args.prompt == "-":                                   # the question comes on standard input: echo ... | chat -p -
        args.prompt = sys.stdin.read().strip()
        if not args.prompt:
            print("nothing on standard input", file=sys.stderr)
            return 2
    if getattr(args, "continue_session", False) and not args.session and store is not None:
        args.session = await _latest(store) or ""
    if getattr(args, "branch", None) is not None:
        if not args.session or store is None:
            print("--branch needs a stored session (--session ID or --continue)", file=sys.stderr)
            return 2
        _, stored = await store.get(args.session)
        if not 0 < args.branch <= len(stored):
            print(f"--branch: keep between 1 and {len(stored)} messages", file=sys.stderr)
            return 2
        args.session = await store.branch(args.session, args.branch, reason="command_line")
        print(f"branched into session {args.session}", file=sys.stderr)
    if args.session and store is not None:
        state = await resume_session(args.session, store, ep, type(preset.environment(args.cwd)), preset.max_turns)
        env, trajectory, session_id = state.environment, state.actor.trajectory, state.session_id
    else:
        env = preset.environment(args.cwd)
        if hasattr(env, "on_session_start"):
            await env.on_session_start(f"cli-{os.getpid()}")
    tags = None
    if store is not None and session_id is None:
        from .agents.fingerprint import fingerprint_session

        tools = [t.function.name for t in env.get_tools()] if env is not None and hasattr(env, "get_tools") else []
        tags = {"fingerprint": fingerprint_session(f"{ep.provider}/{ep.model}", preset.name, tools, system_prompt, cwd=args.cwd),
                "preset": preset.name}
    if args.debug:
        import logging

        logging.basicConfig(level=logging.DEBUG, stream=sys.stderr, format="%(asctime)s %(levelname)s %(name)s: %(message)s")
    if args.theme != "dark":
        from .frontend.terminal import apply_theme

        apply_theme(args.theme)
    runner = InteractiveRunner(ep, frontend, environment=env, system_prompt=system_prompt, session_store=store,
                               session_id=session_id, max_turns=preset.max_turns, initial_prompt=args.prompt,
                               single_turn=args.prompt is not None, trajectory=trajectory, session_tags=tags, cwd=args.cwd)
    if args.thinking:
        from .frontend.slash_commands import handle_thinking

        note = handle_thinking(runner, args.thinking).message or ""
        if note.startswith("usage"):
            raise SystemExit(f"--thinking {args.thinking}: {note}")
    state = await runner.run()
    if state.session_id and not args.quiet:
        print(f"session: {state.session_id}", file=sys.stderr)
    return 0


def parse_model_string(model: str) -> tuple[str, str]:
    """``provider/model`` -> ``(provider, model)`` (rollouts/cli.py:493-508); a bare model name has no provider part."""
    if "/" not in model:
        raise ValueError(f'expected "provider/model" (e.g. "anthropic/claude-sonnet-4-5"), got {model!r}')
    provider, name = model.split("/", 1)
    return provider, name


def cmd_chat(args) -> int:
    return asyncio.run(_chat(args))


def cmd_auth(args) -> int:
    """``auth login|logout|status NAME``: the subscription log-in of one configured OAuth application."""
    from .agents.oauth import OAuthApp, OAuthClient, OAuthError, auth_report, login

    try:
        client = OAuthClient(OAuthApp.load(args.name))
    except OAuthError as e:
        print(e, file=sys.stderr)
        return 2
    if args.action == "login":
        async def ask(prompt: str) -> str:
            return await asyncio.to_thread(input, prompt)

        try:
            asyncio.run(login(client, ask))
        except OAuthError as e:
            print(f"log-in failed: {e}", file=sys.stderr)
            return 1
        return 0
    if args.action == "logout":
        client.logout()
        print(f"logged out of {args.name}")
        return 0
    using, lines = auth_report(args.provider or args.name, args.api_key_env, client)
    print("\n".join(lines))
    return 0 if using != "none" else 1


async def _sessions(args) -> int:
    from .agents.export import export_session
    from .agents.import_cc import import_transcript
    from .agents.slice import slice_session

    store = _store(args)
    if args.action == "list":
        from .agents.doctor import format_time_ago

        for s in sorted(await store.list(), key=lambda s: s.updated_at, reverse=True)[: args.limit]:
            print(f"{s.session_id}  {s.status:<10} {s.num_messages:>4} msgs  {format_time_ago(s.updated_at):>9}  "
                  f"{s.endpoint.get('provider', '?')}/{s.endpoint.get('model', '?')}")
    elif args.action == "tree":
        from .agents.store import format_session_tree

        sid = args.id or await _latest(store)
        if not sid:
            print("no session found", file=sys.stderr)
            return 1
        print(format_session_tree(await store.tree(await store.root_of(sid)), current=sid))
    elif args.action in ("show", "export"):
        text = await export_session(store, args.id, args.format, args.output)
        if not args.output:
            print(text)
    elif args.action == "slice":
        print(await slice_session(store, args.id, args.spec))
    elif args.action == "import":
        print(await import_transcript(store, Path(args.id)))
    elif args.action == "handoff":
        from .agents.export import handoff_summary

        text = await handoff_summary(store, args.id or await _latest(store), args.goal or None)
        if args.output:
            Path(args.output).write_text(text)
        else:
            print(text)
    elif args.action == "doctor":
        from .agents import doctor

        sid = args.id or await _latest(store)
        if not sid:
            print("no session found", file=sys.stderr)
            return 1
        session, messages = await store.get(sid)
        issues = doctor.diagnose(messages)
        print(doctor.report(doctor.session_stats(session, messages), issues, messages))
        if args.fix:
            new, dropped = await doctor.fix_session(store, sid)
            print(f"\ncreated fixed session {new} (dropped messages {dropped}); resume with: chat --session {new}" if new
                  else "\nnothing auto-fixable; use --trim N for oversized or unanswered messages")
        if args.trim:
            try:
                new = await doctor.trim_session(store, sid, args.trim)
            except ValueError as e:
                print(f"\n{e}", file=sys.stderr)
                return 1
            print(f"\ncreated trimmed session {new} (dropped the last {args.trim} messages); resume with: chat --session {new}")
    return 0


async def _latest(store) -> str | None:
    from .agents.doctor import latest_session_id

    return await latest_session_id(store)


def cmd_sessions(args) -> int:
    return asyncio.run(_sessions(args))


async def _eval(args) -> int:
    from .agents.dtypes import EvalConfig
    from .agents.evaluation import evaluate
    from .agents.presets import get_preset

    rows = [json.loads(line) for line in Path(args.dataset).read_text().splitlines() if line.strip()]
    preset = get_preset(args.preset)
    cfg = EvalConfig(endpoint=_endpoint(args), score_fn=load_object(args.score_fn),
                     environment_factory=(lambda row: preset.environment(args.cwd)) if preset.name != "chat" else None,
                     max_turns=preset.max_turns, max_samples=args.max_samples, max_concurrent=args.max_concurrent,
                     output_dir=args.output_dir, eval_name=args.name)
    report = await evaluate(rows, cfg)
    print(json.dumps(report.summary, indent=2))
    return 0


def cmd_eval(args) -> int:
    return asyncio.run(_eval(args))


def cmd_bench(args) -> int:
    root = Path(__file__).resolve().parent.parent
    os.execv(sys.executable, [sys.executable, str(root / "bench.py")] + args.rest)


_DELEGATES = {   # sub-command -> module whose ``main(argv)`` takes the remaining arguments
    "monitor": "research_b200.frontend.training_monitor", "traces": "research_b200.frontend.traces",
    "pretrain": "research_b200.training.pretrain", "infra": "research_b200.infra.cli",
    "kernel-harness": "research_b200.utils.kernel_harness",
}


def cmd_delegate(args) -> int:
    import importlib

    rest = args.rest[1:] if args.rest[:1] == ["--"] else args.rest
    return int(importlib.import_module(_DELEGATES[args.command]).main(rest) or 0)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="research_b200")
    sub = ap.add_subparsers(dest="command", required=True)
    p = sub.add_parser("build"); p.add_argument("--force", action="store_true"); p.set_defaults(fn=cmd_build)
    p = sub.add_parser("serve")
    p.add_argument("--model", default="qwen2.5-0.5b", help="preset name (random weights) or a checkpoint directory")
    p.add_argument("--host", default="127.0.0.1"); p.add_argument("--port", type=int, default=30000)
    p.add_argument("--cache", default="radix", choices=["paged", "radix", "none"])
    p.add_argument("--max-batch-size", type=int, default=256); p.add_argument("--max-model-len", type=int, default=8192)
    p.add_argument("--gpu-memory-utilization", type=float, default=0.9); p.add_argument("--tp", type=int, default=1)
    p.set_defaults(fn=cmd_serve)
    p = sub.add_parser("chat")
    _add_endpoint_args(p)
    p.add_argument("--preset", default="chat"); p.add_argument("--cwd", default="."); p.add_argument("--store", default="")
    p.add_argument("--session", default="", help="resume this session"); p.add_argument("-p", "--prompt", default=None)
    p.add_argument("-y", "--yes", action="store_true", help="run tools without asking")
    p.add_argument("--frontend", default="auto", choices=["auto", "plain", "json", "headless", "ansi"], help="terminal front end (headless: whole turns as JSON lines, both ways)")
    p.add_argument("-c", "--continue", dest="continue_session", action="store_true", help="resume the most recent session")
    p.add_argument("--no-session", action="store_true", help="do not store this conversation")
    p.add_argument("--branch", type=int, default=None, metavar="N", help="with --session / --continue: fork after the first N messages and continue in the fork")
    p.add_argument("--system-prompt", default="", help="text, or a file holding it, that replaces the preset's system prompt")
    p.add_argument("--full-prompt", action="store_true", help="assemble the system prompt from the preset, the environment's tools, project context files, time and cwd")
    p.add_argument("--context", action="append", help="extra text appended to the system prompt (repeatable)")
    p.add_argument("--context-file", action="append", help="file whose content is appended to the system prompt (repeatable)")
    p.add_argument("--stream-json", action="store_true", help="print every event as one JSON line (for programs)")
    p.add_argument("-q", "--quiet", action="store_true", help="only the model's text")
    p.add_argument("--list-presets", action="store_true")
    p.add_argument("--tools", default="", choices=["", "full", "readonly", "no-write"], help="tool set of a coding preset")
    p.add_argument("--env", default="", metavar="A+B", help="environment(s) to use instead of the preset's, combined with + (coding+ask_user)")
    p.add_argument("--thinking", default="", metavar="on|off|TOKENS", help="extended thinking of the model (a token budget)")
    p.add_argument("--theme", default="dark", choices=["dark", "light", "none"], help="colours of the ANSI front end (none: no colour codes)")
    p.add_argument("--debug", action="store_true", help="log at DEBUG level to stderr")
    p.set_defaults(fn=cmd_chat)
    p = sub.add_parser("auth", help="subscription log-in (OAuth) for a hosted provider")
    p.add_argument("action", choices=["login", "logout", "status"]); p.add_argument("name", help="configured OAuth application")
    p.add_argument("--provider", default=""); p.add_argument("--api-key-env", default="")
    p.set_defaults(fn=cmd_auth)
    p = sub.add_parser("track", help="terminal charts of the runs a utils.tracker.Tracker wrote")
    p.add_argument("rest", nargs=argparse.REMAINDER)
    p.set_defaults(fn=lambda a: __import__("research_b200.utils.tracker", fromlist=["main"]).main(a.rest))
    p = sub.add_parser("sessions")
    p.add_argument("action", choices=["list", "show", "export", "slice", "import", "doctor", "handoff", "tree"]); p.add_argument("id", nargs="?")
    p.add_argument("--fix", action="store_true", help="doctor: write a child session without duplicate / orphaned tool results")
    p.add_argument("--trim", type=int, default=0, help="doctor: write a child session without the last N messages")
    p.add_argument("--goal", default="", help="handoff: what the next session should do")
    p.add_argument("--spec", default=""); p.add_argument("--format", default="md", choices=["md", "html", "ansi"])
    p.add_argument("--output", default=""); p.add_argument("--store", default=""); p.add_argument("--limit", type=int, default=20)
    p.set_defaults(fn=cmd_sessions)
    p = sub.add_parser("eval")
    _add_endpoint_args(p)
    p.add_argument("--dataset", required=True, help="JSONL file, one row per sample")
    p.add_argument("--score-fn", required=True, help="module:function(trajectory, row) -> float | Score")
    p.add_argument("--preset", default="chat"); p.add_argument("--cwd", default=".")
    p.add_argument("--max-samples", type=int, default=None); p.add_argument("--max-concurrent", type=int, default=8)
    p.add_argument("--output-dir", default=None); p.add_argument("--name", default="eval")
    p.set_defaults(fn=cmd_eval)
    p = sub.add_parser("bench"); p.add_argument("rest", nargs=argparse.REMAINDER); p.set_defaults(fn=cmd_bench)
    for name, module in _DELEGATES.items():
        p = sub.add_parser(name, help=f"python -m {module}", add_help=False)
        p.add_argument("rest", nargs=argparse.REMAINDER)
        p.set_defaults(fn=cmd_delegate)
    return ap


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] in _DELEGATES:           # handed over whole: argparse would trip over the tool's own options
        return cmd_delegate(argparse.Namespace(command=argv[0], rest=argv[1:]))
    args = build_parser().parse_args(argv)
    return int(args.fn(args) or 0)


if __name__ == "__main__":
    sys.exit(main())
