"""GPU inventory queries and provisioning behind one interface (broker/broker/client.py:38-326,
query.py:10-136, api.py:32-638).

Providers implement ``search() -> list[GPUOffer]``, ``create(offer, **kw) -> GPUInstance`` and
``terminate(id)``. ``GPUClient`` merges offers from all providers, filters them with a small
composable query language (``(q.gpu_type == "B200") & (q.price_per_hour < 4)``) and sorts them.
A ``StaticProvider`` (a fixed inventory, e.g. the machines a lab owns) ships here; cloud back ends plug
in through the same three methods.
"""

from __future__ import annotations

import itertools
import operator
from dataclasses import dataclass, field
from typing import Any, Callable, Protocol


@dataclass(frozen=True)
class GPUOffer:
    provider: str
    offer_id: str
    gpu_type: str
    gpu_count: int = 1
    vram_gb: int = 0
    price_per_hour: float = 0.0
    region: str = ""
    interconnect: str = ""        # e.g. "nvlink5"
    spot: bool = False
    extra: dict[str, Any] = field(default_factory=dict)


@dataclass
class GPUInstance:
    provider: str
    instance_id: str
    offer: GPUOffer
    status: str = "running"
    ssh_connection: str | None = None


class Condition:
    def __init__(self, fn: Callable[[GPUOffer], bool], text: str):
        self.fn, self.text = fn, text

    def __call__(self, o: GPUOffer) -> bool:
        return self.fn(o)

    def __and__(self, other: "Condition") -> "Condition":
        return Condition(lambda o: self(o) and other(o), f"({self.text} & {other.text})")

    def __or__(self, other: "Condition") -> "Condition":
        return Condition(lambda o: self(o) or other(o), f"({self.text} | {other.text})")

    def __invert__(self) -> "Condition":
        return Condition(lambda o: not self(o), f"~{self.text}")

    def __repr__(self) -> str:
        return self.text


class Field:
    def __init__(self, name: str):
        self.name = name

    def _cmp(self, op, sym, value) -> Condition:
        return Condition(lambda o: op(getattr(o, self.name), value), f"{self.name} {sym} {value!r}")

    def __eq__(self, v): return self._cmp(operator.eq, "==", v)      # noqa: E704
    def __ne__(self, v): return self._cmp(operator.ne, "!=", v)      # noqa: E704
    def __lt__(self, v): return self._cmp(operator.lt, "<", v)       # noqa: E704
    def __le__(self, v): return self._cmp(operator.le, "<=", v)      # noqa: E704
    def __gt__(self, v): return self._cmp(operator.gt, ">", v)       # noqa: E704
    def __ge__(self, v): return self._cmp(operator.ge, ">=", v)      # noqa: E704

    def isin(self, values) -> Condition:
        vs = set(values)
        return Condition(lambda o: getattr(o, self.name) in vs, f"{self.name} in {sorted(vs)!r}")

    def contains(self, text: str) -> Condition:
        return Condition(lambda o: text.lower() in str(getattr(o, self.name)).lower(), f"{text!r} in {self.name}")

    __hash__ = None  # type: ignore[assignment]


class _Query:
    def __getattr__(self, name: str) -> Field:
        if name not in GPUOffer.__dataclass_fields__:
            raise AttributeError(f"GPUOffer has no field {name!r}")
        return Field(name)


q = _Query()


class Provider(Protocol):
    name: str

    def search(self) -> list[GPUOffer]: ...
    def create(self, offer: GPUOffer, **kw: Any) -> GPUInstance: ...
    def terminate(self, instance_id: str) -> bool: ...


class StaticProvider:
    """A fixed list of machines; ``create`` hands one out, ``terminate`` returns it."""

    def __init__(self, name: str, offers: list[GPUOffer], connections: dict[str, str] | None = None):
        self.name, self._offers, self._conn = name, list(offers), connections or {}
        self._busy: dict[str, str] = {}
        self._ids = itertools.count(1)

    def search(self) -> list[GPUOffer]:
        return [o for o in self._offers if o.offer_id not in self._busy.values()]

    def create(self, offer: GPUOffer, **kw: Any) -> GPUInstance:
        if offer.offer_id in self._busy.values():
            raise RuntimeError(f"{offer.offer_id} is already in use")
        iid = f"{self.name}-{next(self._ids)}"
        self._busy[iid] = offer.offer_id
        return GPUInstance(self.name, iid, offer, "running", self._conn.get(offer.offer_id))

    def terminate(self, instance_id: str) -> bool:
        return self._busy.pop(instance_id, None) is not None


@dataclass
class ProvisionAttempt:
    offer_id: str
    gpu_type: str
    provider: str
    price_per_hour: float
    error: str | None = None                 # None: this attempt produced ``instance``
    error_category: str | None = None        # credentials | unavailable | network | unknown
    instance: GPUInstance | None = None


@dataclass
class ProvisionResult:
    success: bool
    instance: GPUInstance | None = None
    attempts: list[ProvisionAttempt] = field(default_factory=list)
    error_summary: str | None = None
    no_offers_found: bool = False
    all_unavailable: bool = False
    credential_error: bool = False
    network_error: bool = False


def categorize_error(e: BaseException) -> str:
    """HTTP status where the error carries one (401/403 credentials; 404/409/410/422/429/503 capacity), else the
    exception type and a few words providers use for "none left"."""
    status = getattr(e, "status", None)
    text = str(e).lower()
    if status in (401, 403) or "unauthorized" in text or "invalid api key" in text or "forbidden" in text:
        return "credentials"
    if isinstance(e, (TimeoutError, ConnectionError)) or "timed out" in text or "connection" in text or "unreachable" in text:
        return "network"
    if status in (404, 409, 410, 422, 429, 503) or any(w in text for w in ("capacity", "unavailable", "no longer available", "already in use",
                                                                            "sold out", "not enough", "out of stock")):
        return "unavailable"
    return "unknown"


class GPUClient:
    """``registry``: a JSON file that remembers the instances this client created across processes (what a command line
    needs for ``list`` / ``ssh`` / ``cleanup`` after the ``create`` call has exited). Without it, instances live in memory."""

    def __init__(self, providers: list[Provider], registry: str | None = None):
        self.providers = {p.name: p for p in providers}
        self.instances: dict[str, GPUInstance] = {}
        self.created_at: dict[str, float] = {}
        self.registry = registry
        self._load_registry()

    def _load_registry(self) -> None:
        import json
        from pathlib import Path

        if not self.registry or not Path(self.registry).is_file():
            return
        try:
            rows = json.loads(Path(self.registry).read_text())
        except ValueError:
            return
        for r in rows:
            offer = GPUOffer(**r["offer"])
            self.instances[r["instance_id"]] = GPUInstance(r["provider"], r["instance_id"], offer, r.get("status", "unknown"), r.get("ssh_connection"))
            self.created_at[r["instance_id"]] = r.get("created_at", 0.0)

    def _save_registry(self) -> None:
        import json
        import os
        from dataclasses import asdict
        from pathlib import Path

        if not self.registry:
            return
        p = Path(self.registry)
        p.parent.mkdir(parents=True, exist_ok=True)
        rows = [{"provider": i.provider, "instance_id": i.instance_id, "offer": asdict(i.offer), "status": i.status, "ssh_connection": i.ssh_connection,
                 "created_at": self.created_at.get(i.instance_id, 0.0)} for i in self.instances.values()]
        tmp = p.with_suffix(".tmp")
        tmp.write_text(json.dumps(rows, indent=1))
        os.replace(tmp, p)

    def _remember(self, inst: GPUInstance) -> None:
        import time

        self.instances[inst.instance_id] = inst
        self.created_at.setdefault(inst.instance_id, time.time())
        self._save_registry()

    def search(self, where: Condition | None = None, sort_by: str = "price_per_hour", reverse: bool = False) -> list[GPUOffer]:
        offers = [o for p in self.providers.values() for o in p.search()]
        if where is not None:
            offers = [o for o in offers if where(o)]
        return sorted(offers, key=lambda o: getattr(o, sort_by), reverse=reverse)

    def create(self, where: Condition | None = None, **kw: Any) -> GPUInstance:
        """Take the cheapest matching offer; fall through to the next one if a provider refuses."""
        errors = []
        for o in self.search(where):
            try:
                inst = self.providers[o.provider].create(o, **kw)
                self._remember(inst)
                return inst
            except Exception as e:  # noqa: BLE001 - try the next offer
                errors.append(f"{o.provider}/{o.offer_id}: {e}")
        raise RuntimeError("no offer could be provisioned" + (": " + "; ".join(errors) if errors else " (nothing matched)"))

    def provision(self, where: Condition | None = None, max_attempts: int = 3, **kw: Any) -> "ProvisionResult":
        """``create`` with a record of what was tried (broker/broker/api.py:255-527): up to ``max_attempts`` offers,
        cheapest first, each failure sorted into a category so that a caller can tell "change the query" (nothing
        matched), "try another GPU type" (every offer was out of capacity), "fix the API key" and "try again later"
        apart without parsing messages."""
        offers = self.search(where)
        if not offers:
            return ProvisionResult(False, error_summary="no offer matches the query", no_offers_found=True)
        attempts: list[ProvisionAttempt] = []
        for o in offers[:max_attempts]:
            try:
                inst = self.providers[o.provider].create(o, **kw)
            except Exception as e:  # noqa: BLE001 - recorded, next offer
                attempts.append(ProvisionAttempt(o.offer_id, o.gpu_type, o.provider, o.price_per_hour, str(e)[:300], categorize_error(e)))
                continue
            if inst is None:
                attempts.append(ProvisionAttempt(o.offer_id, o.gpu_type, o.provider, o.price_per_hour, "the provider returned no instance", "unavailable"))
                continue
            self._remember(inst)
            attempts.append(ProvisionAttempt(o.offer_id, o.gpu_type, o.provider, o.price_per_hour, instance=inst))
            return ProvisionResult(True, inst, attempts)
        cats = [a.error_category for a in attempts]
        parts = [f"all {len(attempts)} offers tried were out of capacity" if all(c == "unavailable" for c in cats)
                 else f"failed after {len(attempts)} offer(s)"]
        parts += [f"{cats.count(c)} {c} error(s)" for c in ("credentials", "network") if c in cats]
        return ProvisionResult(False, None, attempts, "; ".join(parts), all_unavailable=all(c == "unavailable" for c in cats),
                               credential_error="credentials" in cats, network_error="network" in cats)

    def list_instances(self, refresh: bool = True) -> list[GPUInstance]:
        """Instances this client created, their state re-read from the provider where it offers ``refresh``."""
        out = []
        for iid, inst in list(self.instances.items()):
            fn = getattr(self.providers.get(inst.provider), "refresh", None) if refresh else None
            if fn is not None:
                try:
                    inst = self.instances[iid] = fn(iid)
                    self._save_registry()
                except Exception:  # noqa: BLE001 - keep the last known state
                    pass
            out.append(inst)
        return out

    def get_instance(self, instance_id: str, refresh: bool = True) -> GPUInstance | None:
        return next((i for i in self.list_instances(refresh) if i.instance_id == instance_id), None)

    def terminate(self, instance_id: str) -> bool:
        inst = self.instances.pop(instance_id, None)
        self.created_at.pop(instance_id, None)
        self._save_registry()
        return bool(inst) and inst.provider in self.providers and self.providers[inst.provider].terminate(instance_id)

    def older_than(self, hours: float, now: float | None = None) -> list[GPUInstance]:
        """Instances this client created more than ``hours`` ago (candidates for ``cleanup``: a forgotten instance bills by the hour)."""
        import time

        now = time.time() if now is None else now
        return [i for iid, i in self.instances.items() if now - self.created_at.get(iid, now) >= hours * 3600.0]

    def running_cost(self, now: float | None = None) -> float:
        """What the tracked instances have cost so far at their offers' hourly prices."""
        import time

        now = time.time() if now is None else now
        return sum(i.offer.price_per_hour * max(now - self.created_at.get(iid, now), 0.0) / 3600.0 for iid, i in self.instances.items())

    def terminate_all(self) -> int:
        return sum(self.terminate(i) for i in list(self.instances))
