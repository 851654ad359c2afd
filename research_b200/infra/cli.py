"""Command line of the infrastructure packages (broker/broker/cli.py, bifrost/bifrost/cli.py, csearch/csearch/cli.py):

    python -m research_b200.infra.cli gpus search --where "gpu_type~B200 gpu_count>=8 price_per_hour<40"
    python -m research_b200.infra.cli gpus create --where "gpu_type~H100" [--provider lambda]
    python -m research_b200.infra.cli gpus terminate --provider lambda --id i-123
    python -m research_b200.infra.cli remote exec   user@host:22 "nvidia-smi"
    python -m research_b200.infra.cli remote push   user@host:22 --repo . --dest ~/work
    python -m research_b200.infra.cli remote run    user@host:22 --name train "python train.py"
    python -m research_b200.infra.cli remote status|logs|stop user@host:22 --name train
    python -m research_b200.infra.cli code index|search|symbols --root . [query]
    python -m research_b200.infra.cli code defs|refs|outline --root . [--backend auto|tree-sitter|ast|scan|ctags] [--snippet] [name]

``gpus`` talks to every provider whose API key is in the environment. The ``--where`` mini-language is a list of
``field OP value`` terms joined by blanks (all must hold); OP is one of ``== != >= <= > <`` or ``~`` (substring).
"""

from __future__ import annotations

import argparse
import json
import os
import re
import sys
from dataclasses import asdict
from pathlib import Path
from typing import Callable, Sequence

from .bifrost import ProcessSpec, RemoteClient
from .broker import Condition, GPUClient, GPUOffer, q
from .csearch import CodeIndex

_TERM = re.compile(r"^(\w+)(==|!=|>=|<=|>|<|~)(.+)$")


def parse_where(text: str) -> Condition | None:
    """``"gpu_type~B200 gpu_count>=8"`` -> a broker ``Condition`` (None for an empty string)."""
    cond: Condition | None = None
    for term in text.split():
        m = _TERM.match(term)
        if not m:
            raise ValueError(f"cannot read condition {term!r} (want field OP value, e.g. gpu_count>=8)")
        name, op, raw = m.groups()
        fld = getattr(q, name)                       # AttributeError names the bad field
        kind = GPUOffer.__dataclass_fields__[name].type
        value: object = raw
        if op != "~":
            if kind in ("int", int):
                value = int(raw)
            elif kind in ("float", float):
                value = float(raw)
            elif kind in ("bool", bool):
                value = raw.lower() in ("1", "true", "yes")
        c = {"==": fld.__eq__, "!=": fld.__ne__, ">=": fld.__ge__, "<=": fld.__le__, ">": fld.__gt__, "<": fld.__lt__,
             "~": fld.contains}[op](value)
        cond = c if cond is None else cond & c
    return cond


def _offer_table(offers: Sequence[GPUOffer]) -> str:
    rows = [("provider", "offer", "gpu", "n", "vram", "$/h", "region", "spot")]
    rows += [(o.provider, o.offer_id, o.gpu_type, str(o.gpu_count), str(o.vram_gb), f"{o.price_per_hour:.2f}", o.region, "spot" if o.spot else "")
             for o in offers]
    w = [max(len(r[i]) for r in rows) for i in range(len(rows[0]))]
    return "\n".join("  ".join(c.ljust(w[i]) for i, c in enumerate(r)).rstrip() for r in rows)


def _gpu_client(a) -> GPUClient:
    if getattr(a, "_client", None) is not None:        # injected by tests and embedding programs
        return a._client
    from .broker_providers import providers_from_env

    provs = providers_from_env()
    if not provs:
        raise SystemExit("no provider API key in the environment (LAMBDA_API_KEY, RUNPOD_API_KEY, VAST_API_KEY, PRIME_API_KEY)")
    return GPUClient(provs, registry=os.path.join(os.path.expanduser("~"), ".research_b200", "instances.json"))


def ssh_command(connection: str, key: str | None = None) -> str:
    host, _, port = connection.partition(":")
    return " ".join(["ssh"] + (["-p", port] if port else []) + (["-i", key] if key else []) + [host])


GPU_QUERY = "nvidia-smi --query-gpu=index,name,memory.used,memory.total,utilization.gpu --format=csv,noheader,nounits"


def instance_info(inst, key: str | None = None, transport=None) -> dict:
    """What is on the machine behind an instance: its GPUs with memory in use and utilisation, free disk, uptime."""
    from .bifrost import RemoteClient, subprocess_transport

    c = RemoteClient(inst.ssh_connection, key=key, transport=transport or subprocess_transport)
    code, out, err = c.exec(GPU_QUERY)
    gpus = []
    for line in out.splitlines() if code == 0 else []:
        f = [x.strip() for x in line.split(",")]
        if len(f) == 5 and f[0].isdigit():
            gpus.append({"index": int(f[0]), "name": f[1], "memory_used_mib": int(f[2]), "memory_total_mib": int(f[3]), "utilization_pct": int(f[4])})
    disk = c.exec("df -h / | tail -1")[1].split()
    return {"instance_id": inst.instance_id, "ssh": inst.ssh_connection, "gpus": gpus, "gpu_error": err.strip()[:200] if code else "",
            "disk_free": disk[3] if len(disk) > 3 else "?", "uptime": c.exec("uptime -p")[1].strip()}


def cmd_gpus(a, out: Callable[[str], None]) -> int:
    gc = _gpu_client(a)
    if a.action == "search":
        offers = gc.search(parse_where(a.where), sort_by=a.sort)[: a.limit]
        out(json.dumps([asdict(o) for o in offers]) if a.json else _offer_table(offers))
        return 0
    if a.action == "create":
        cond = parse_where(a.where)
        if a.provider:
            cond = (q.provider == a.provider) if cond is None else cond & (q.provider == a.provider)
        inst = gc.create(cond)
        out(json.dumps({"provider": inst.provider, "id": inst.instance_id, "status": inst.status, "ssh": inst.ssh_connection,
                        "offer": asdict(inst.offer)}))
        return 0
    if a.action == "list":
        rows = gc.list_instances(refresh=not a.no_refresh)
        if a.json:
            out(json.dumps([{"provider": i.provider, "id": i.instance_id, "status": i.status, "ssh": i.ssh_connection, "gpu": i.offer.gpu_type,
                             "count": i.offer.gpu_count, "price_per_hour": i.offer.price_per_hour} for i in rows]))
        else:
            out("\n".join(f"{i.provider}:{i.instance_id}  {i.status:<10} {i.offer.gpu_count}x{i.offer.gpu_type}  ${i.offer.price_per_hour:.2f}/h  {i.ssh_connection or '-'}"
                          for i in rows) or "no instances")
            if rows:
                out(f"cost so far: ${gc.running_cost():.2f}")
        return 0
    if a.action in ("status", "ssh", "info"):
        inst = gc.get_instance(a.id, refresh=a.action == "status")
        if inst is None:
            out(f"no tracked instance {a.id}")
            return 1
        if a.action == "status":
            out(f"{inst.provider}:{inst.instance_id}: {inst.status}" + (f" ({inst.ssh_connection})" if inst.ssh_connection else ""))
        elif not inst.ssh_connection:
            out(f"{inst.instance_id} has no ssh address yet (status {inst.status})")
            return 1
        elif a.action == "ssh":
            out(ssh_command(inst.ssh_connection, a.key))
        else:
            out(json.dumps(instance_info(inst, a.key, getattr(a, "_transport", None)), indent=1))
        return 0
    if a.action == "cleanup":
        old = gc.older_than(a.older_than)
        if not old:
            out("nothing to clean up")
            return 0
        for i in old:
            out(f"{'terminating' if a.yes else 'would terminate'} {i.provider}:{i.instance_id} ({i.offer.gpu_count}x{i.offer.gpu_type}, ${i.offer.price_per_hour:.2f}/h)")
            if a.yes:
                gc.terminate(i.instance_id)
        if not a.yes:
            out("run again with --yes to terminate them")
        return 0
    ok = gc.terminate(a.id) if a.id in gc.instances else gc.providers[a.provider].terminate(a.id)
    out(f"terminated {a.provider}:{a.id}" if ok else f"{a.provider}:{a.id} was not running")
    return 0 if ok else 1


def cmd_remote(a, out: Callable[[str], None]) -> int:
    c = RemoteClient(a.target, key=a.key)
    if a.action == "exec":
        if a.stream:
            gen = c.exec_stream(a.command)
            while True:
                try:
                    out(next(gen))
                except StopIteration as stop:
                    return int(stop.value or 0)
        code, so, se = c.exec(a.command)
        if so:
            out(so.rstrip("\n"))
        if se:
            print(se.rstrip("\n"), file=sys.stderr)
        return code
    if a.action == "push":
        out(c.push(a.repo, a.dest, a.ref))
        return 0
    if a.action == "run":
        info = c.start_job(ProcessSpec(a.command, cwd=a.cwd, env=dict(kv.split("=", 1) for kv in a.env), name=a.name))
        out(f"{info.name} pid {info.pid} log {info.log_path}")
        if a.wait:
            done = c.wait_job(a.name, timeout=a.timeout)
            out(c.job_logs(a.name, 40).rstrip("\n"))
            return done.exit_code or 0
        return 0
    if a.action == "status":
        i = c.job_status(a.name)
        out(f"{i.name}: {i.status}" + (f" (exit {i.exit_code})" if i.exit_code is not None else "") + (f" pid {i.pid}" if i.pid else ""))
        return 0
    if a.action == "logs":
        out(c.job_logs(a.name, a.tail).rstrip("\n"))
        return 0
    c.stop_job(a.name)
    return 0


def cmd_code(a, out: Callable[[str], None]) -> int:
    root = Path(a.root).resolve()
    if a.action in ("defs", "refs", "outline"):
        from .csearch_symbols import SearchOptions, list_symbols, search_definitions, search_references

        o = SearchOptions(path=root, backend=a.backend, include_snippet=a.snippet, limit=a.limit, exact=not a.fuzzy)
        res = list_symbols(o) if a.action == "outline" else (search_definitions if a.action == "defs" else search_references)(a.query, o)
        for r in res:
            out(r.format_with_snippet() if a.snippet else r.format_compact())
        return 0 if res else 1
    cache = Path(a.index) if a.index else root / ".csearch_index.json"
    if a.action == "index" or not cache.exists():
        ix = CodeIndex(root).build()
        ix.save(cache)
        if a.action == "index":
            out(f"indexed {len(ix.files)} files -> {cache}")
            return 0
    else:
        ix = CodeIndex.load(cache)
        if ix.stale_files():
            ix = CodeIndex(root).build()
            ix.save(cache)
    hits = ix.symbols(a.query or None) if a.action == "symbols" else ix.search(a.query, regex=a.regex, max_hits=a.limit)
    for h in hits:
        out(f"{h.path}:{h.line}: {h.text}")
    return 0 if hits else 1


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="research_b200.infra.cli", description=__doc__.split("\n\n")[0])
    top = ap.add_subparsers(dest="group", required=True)

    g = top.add_parser("gpus").add_subparsers(dest="action", required=True)
    p = g.add_parser("search")
    p.add_argument("--where", default=""); p.add_argument("--sort", default="price_per_hour"); p.add_argument("--limit", type=int, default=20)
    p.add_argument("--json", action="store_true")
    p = g.add_parser("create"); p.add_argument("--where", default=""); p.add_argument("--provider", default="")
    p = g.add_parser("terminate"); p.add_argument("--provider", required=True); p.add_argument("--id", required=True)
    p = g.add_parser("list"); p.add_argument("--json", action="store_true"); p.add_argument("--no-refresh", action="store_true")
    for name in ("status", "ssh", "info"):
        p = g.add_parser(name); p.add_argument("--id", required=True); p.add_argument("--key", default=None)
    p = g.add_parser("cleanup"); p.add_argument("--older-than", type=float, default=0.0, metavar="HOURS"); p.add_argument("--yes", action="store_true")

    r = top.add_parser("remote").add_subparsers(dest="action", required=True)
    for name in ("exec", "push", "run", "status", "logs", "stop"):
        p = r.add_parser(name)
        p.add_argument("target", help="user@host[:port] or 'local'")
        p.add_argument("--key", default=None)
        if name == "exec":
            p.add_argument("command"); p.add_argument("--stream", action="store_true")
        elif name == "push":
            p.add_argument("--repo", default="."); p.add_argument("--dest", required=True); p.add_argument("--ref", default="HEAD")
        elif name == "run":
            p.add_argument("command"); p.add_argument("--name", default="job"); p.add_argument("--cwd", default=None)
            p.add_argument("--env", action="append", default=[], metavar="K=V"); p.add_argument("--wait", action="store_true")
            p.add_argument("--timeout", type=float, default=3600.0)
        else:
            p.add_argument("--name", default="job")
            if name == "logs":
                p.add_argument("--tail", type=int, default=50)

    c = top.add_parser("code").add_subparsers(dest="action", required=True)
    for name in ("index", "search", "symbols"):
        p = c.add_parser(name)
        p.add_argument("query", nargs="?" if name != "search" else None, default="")
        p.add_argument("--root", default="."); p.add_argument("--index", default=""); p.add_argument("--regex", action="store_true")
        p.add_argument("--limit", type=int, default=200)
    for name in ("defs", "refs", "outline"):
        p = c.add_parser(name)
        p.add_argument("query", nargs="?" if name == "outline" else None, default="")
        p.add_argument("--root", default="."); p.add_argument("--backend", default="auto", choices=["auto", "tree-sitter", "ast", "scan", "ctags"])
        p.add_argument("--snippet", action="store_true"); p.add_argument("--fuzzy", action="store_true"); p.add_argument("--limit", type=int, default=200)
    return ap


def main(argv: Sequence[str] | None = None, out: Callable[[str], None] = print, gpu_client: GPUClient | None = None) -> int:
    a = build_parser().parse_args(argv)
    a._client = gpu_client
    return {"gpus": cmd_gpus, "remote": cmd_remote, "code": cmd_code}[a.group](a, out)


if __name__ == "__main__":
    raise SystemExit(main())
