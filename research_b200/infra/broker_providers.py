"""Cloud back ends of the GPU broker: Lambda, RunPod, Vast.ai and Prime Intellect adapters behind the ``Provider``
protocol of ``infra/broker.py`` (broker/broker/providers/{lambdalabs,runpod,vast,primeintellect}.py).

Every adapter only builds requests and maps replies; the HTTP exchange itself is a ``Transport`` callable
``(method, url, headers, body) -> (status, parsed JSON)``. The default transport uses ``urllib``; tests (and any
offline use) pass a fake. The adapters have only been exercised against scripted transports; the request shapes
follow the providers' public API documentation, as the reference's adapters do.
"""

from __future__ import annotations

import json
import os
import urllib.error
import urllib.request
from typing import Any, Callable

from .broker import GPUInstance, GPUOffer

Transport = Callable[[str, str, dict[str, str], Any], tuple[int, Any]]


class ProviderError(RuntimeError):
    def __init__(self, provider: str, status: int, detail: Any):
        super().__init__(f"{provider}: HTTP {status}: {str(detail)[:300]}")
        self.provider, self.status, self.detail = provider, status, detail


def urllib_transport(method: str, url: str, headers: dict[str, str], body: Any, timeout: float = 30.0) -> tuple[int, Any]:
    data = json.dumps(body).encode() if body is not None else None
    req = urllib.request.Request(url, data=data, method=method, headers={"Content-Type": "application/json", **headers})
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            raw = r.read()
            return r.status, (json.loads(raw) if raw else None)
    except urllib.error.HTTPError as e:
        raw = e.read()
        try:
            return e.code, json.loads(raw)
        except ValueError:
            return e.code, raw.decode(errors="replace")


class _HttpProvider:
    name = "http"
    base_url = ""
    key_env = ""

    def __init__(self, api_key: str | None = None, transport: Transport | None = None):
        self.api_key = api_key or os.environ.get(self.key_env, "")
        self.transport = transport or urllib_transport
        self.instances: dict[str, GPUInstance] = {}

    def _headers(self) -> dict[str, str]:
        return {"Authorization": f"Bearer {self.api_key}"}

    def _call(self, method: str, path: str, body: Any = None) -> Any:
        status, reply = self.transport(method, self.base_url + path, self._headers(), body)
        if not 200 <= status < 300:
            raise ProviderError(self.name, status, reply)
        return reply


def _vram_from_name(name: str) -> int:
    table = {"B200": 180, "H200": 141, "H100": 80, "A100": 80, "A6000": 48, "A10": 24, "4090": 24, "L40": 48, "GH200": 96}
    return next((v for k, v in table.items() if k in name.upper()), 0)


class LambdaProvider(_HttpProvider):
    name, base_url, key_env = "lambda", "https://cloud.lambdalabs.com/api/v1", "LAMBDA_API_KEY"

    def search(self) -> list[GPUOffer]:
        out = []
        for type_name, entry in (self._call("GET", "/instance-types") or {}).get("data", {}).items():
            it = entry.get("instance_type", {})
            specs = it.get("specs", {})
            for region in entry.get("regions_with_capacity_available", []):
                out.append(GPUOffer(self.name, f"{type_name}@{region.get('name', '')}", it.get("description", type_name),
                                    int(specs.get("gpus", 1)), _vram_from_name(it.get("description", type_name)),
                                    it.get("price_cents_per_hour", 0) / 100.0, region.get("name", ""),
                                    extra={"instance_type": type_name}))
        return out

    def create(self, offer: GPUOffer, ssh_key_names: list[str] | None = None, name: str | None = None, **kw: Any) -> GPUInstance:
        body = {"region_name": offer.region, "instance_type_name": offer.extra.get("instance_type", offer.offer_id.split("@")[0]),
                "ssh_key_names": ssh_key_names or [], "quantity": 1}
        if name:
            body["name"] = name
        ids = self._call("POST", "/instance-operations/launch", body)["data"]["instance_ids"]
        inst = GPUInstance(self.name, ids[0], offer, status="booting")
        self.instances[inst.instance_id] = inst
        return inst

    def refresh(self, instance_id: str) -> GPUInstance:
        d = self._call("GET", f"/instances/{instance_id}")["data"]
        inst = self.instances[instance_id]
        inst.status = d.get("status", inst.status)
        if d.get("ip"):
            inst.ssh_connection = f"ubuntu@{d['ip']}:22"
        return inst

    def terminate(self, instance_id: str) -> bool:
        self._call("POST", "/instance-operations/terminate", {"instance_ids": [instance_id]})
        self.instances.pop(instance_id, None)
        return True


class RunPodProvider(_HttpProvider):
    name, base_url, key_env = "runpod", "https://api.runpod.io/graphql", "RUNPOD_API_KEY"

    def _gql(self, query: str, variables: dict[str, Any] | None = None) -> Any:
        reply = self._call("POST", "", {"query": query, "variables": variables or {}})
        if reply.get("errors"):
            raise ProviderError(self.name, 200, reply["errors"])
        return reply["data"]

    def search(self) -> list[GPUOffer]:
        q = "query { gpuTypes { id displayName memoryInGb secureCloud communityCloud lowestPrice(input: {gpuCount: 1}) { minimumBidPrice uninterruptablePrice } } }"
        out = []
        for g in self._gql(q)["gpuTypes"]:
            price = (g.get("lowestPrice") or {})
            if price.get("uninterruptablePrice"):
                out.append(GPUOffer(self.name, g["id"], g.get("displayName", g["id"]), 1, int(g.get("memoryInGb") or 0),
                                    float(price["uninterruptablePrice"]), extra={"secure": bool(g.get("secureCloud"))}))
            if price.get("minimumBidPrice"):
                out.append(GPUOffer(self.name, g["id"] + ":spot", g.get("displayName", g["id"]), 1, int(g.get("memoryInGb") or 0),
                                    float(price["minimumBidPrice"]), spot=True, extra={"secure": bool(g.get("secureCloud"))}))
        return out

    def create(self, offer: GPUOffer, image: str = "runpod/pytorch:latest", disk_gb: int = 50, name: str = "research-b200",
               **kw: Any) -> GPUInstance:
        gpu_id = offer.offer_id.split(":")[0]
        inp = {"gpuTypeId": gpu_id, "gpuCount": offer.gpu_count, "imageName": image, "containerDiskInGb": disk_gb, "name": name,
               "ports": "22/tcp", "startSsh": True, "cloudType": "SECURE" if offer.extra.get("secure") else "COMMUNITY"}
        if offer.spot:
            inp["bidPerGpu"] = offer.price_per_hour
            data = self._gql("mutation($input: PodRentInterruptableInput!) { podRentInterruptable(input: $input) { id desiredStatus } }",
                             {"input": inp})["podRentInterruptable"]
        else:
            data = self._gql("mutation($input: PodFindAndDeployOnDemandInput!) { podFindAndDeployOnDemand(input: $input) { id desiredStatus } }",
                             {"input": inp})["podFindAndDeployOnDemand"]
        inst = GPUInstance(self.name, data["id"], offer, status=str(data.get("desiredStatus", "CREATED")).lower())
        self.instances[inst.instance_id] = inst
        return inst

    def terminate(self, instance_id: str) -> bool:
        self._gql("mutation($input: PodTerminateInput!) { podTerminate(input: $input) }", {"input": {"podId": instance_id}})
        self.instances.pop(instance_id, None)
        return True


class VastProvider(_HttpProvider):
    name, base_url, key_env = "vast", "https://console.vast.ai/api/v0", "VAST_API_KEY"

    def search(self, min_gpus: int = 1) -> list[GPUOffer]:
        query = {"verified": {"eq": True}, "rentable": {"eq": True}, "num_gpus": {"gte": min_gpus}, "order": [["dph_total", "asc"]],
                 "type": "on-demand"}
        reply = self._call("POST", "/bundles/", query) or {}
        return [GPUOffer(self.name, str(o["id"]), o.get("gpu_name", ""), int(o.get("num_gpus", 1)), int(o.get("gpu_ram", 0) // 1024),
                         float(o.get("dph_total", 0.0)), o.get("geolocation", ""), extra={"reliability": o.get("reliability2")})
                for o in reply.get("offers", [])]

    def create(self, offer: GPUOffer, image: str = "pytorch/pytorch:latest", disk_gb: int = 50, **kw: Any) -> GPUInstance:
        reply = self._call("PUT", f"/asks/{offer.offer_id}/", {"client_id": "me", "image": image, "disk": disk_gb, "runtype": "ssh"})
        if not reply.get("success", True):
            raise ProviderError(self.name, 200, reply)
        inst = GPUInstance(self.name, str(reply["new_contract"]), offer, status="loading")
        self.instances[inst.instance_id] = inst
        return inst

    def terminate(self, instance_id: str) -> bool:
        self._call("DELETE", f"/instances/{instance_id}/")
        self.instances.pop(instance_id, None)
        return True


class PrimeIntellectProvider(_HttpProvider):
    name, base_url, key_env = "primeintellect", "https://api.primeintellect.ai/api/v1", "PRIME_API_KEY"

    def search(self) -> list[GPUOffer]:
        reply = self._call("GET", "/availability/") or {}
        out = []
        for gpu_type, entries in reply.items():
            for e in entries if isinstance(entries, list) else []:
                price = (e.get("prices") or {}).get("onDemand") or e.get("price") or 0.0
                out.append(GPUOffer(self.name, str(e.get("cloudId", gpu_type)), gpu_type, int(e.get("gpuCount", 1)),
                                    int(e.get("gpuMemory", 0) or _vram_from_name(gpu_type)), float(price), e.get("dataCenter", ""),
                                    e.get("interconnectType", "") or "", extra={"provider": e.get("provider"), "socket": e.get("socket")}))
        return out

    def create(self, offer: GPUOffer, name: str = "research-b200", image: str = "ubuntu_22_cuda_12", disk_gb: int = 100,
               **kw: Any) -> GPUInstance:
        body = {"pod": {"name": name, "cloudId": offer.offer_id, "gpuType": offer.gpu_type, "socket": offer.extra.get("socket"),
                        "gpuCount": offer.gpu_count, "diskSize": disk_gb, "image": image, "dataCenterId": offer.region or None},
                "provider": {"type": offer.extra.get("provider")}}
        reply = self._call("POST", "/pods/", body)
        inst = GPUInstance(self.name, str(reply["id"]), offer, status=str(reply.get("status", "PROVISIONING")).lower())
        self.instances[inst.instance_id] = inst
        return inst

    def terminate(self, instance_id: str) -> bool:
        self._call("DELETE", f"/pods/{instance_id}")
        self.instances.pop(instance_id, None)
        return True


PROVIDERS = {"lambda": LambdaProvider, "runpod": RunPodProvider, "vast": VastProvider, "primeintellect": PrimeIntellectProvider}


def providers_from_env(transport: Transport | None = None) -> list[_HttpProvider]:
    """One adapter per provider whose API key is set in the environment."""
    return [cls(transport=transport) for cls in PROVIDERS.values() if os.environ.get(cls.key_env)]
