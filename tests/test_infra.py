"""Remote execution, GPU brokering and code search, all on this machine."""

import subprocess

import pytest

from research_b200.infra.bifrost import ProcessSpec, RemoteClient, RemoteError
from research_b200.infra.broker import GPUClient, GPUOffer, StaticProvider, q
from research_b200.infra.csearch import CodeIndex, trigrams


def test_remote_client_local_jobs_and_push(tmp_path):
    c = RemoteClient("local", job_dir=str(tmp_path / "jobs"))
    assert c.exec("echo hi")[1].strip() == "hi"
    with pytest.raises(RemoteError):
        c.exec("exit 3", check=True)
    info = c.start_job(ProcessSpec("echo started; sleep 0.3; echo done; exit 7", name="j1", env={"FOO": "a b"}))
    assert info.pid and info.status == "running"
    done = c.wait_job("j1", timeout=20, poll=0.1)
    assert done.status == "exited" and done.exit_code == 7 and "done" in c.job_logs("j1")
    long = c.start_job(ProcessSpec("sleep 30", name="j2"))
    assert c.job_status("j2").status == "running"
    c.stop_job("j2")
    assert c.wait_job("j2", timeout=10, poll=0.1).status in ("unknown", "exited") and long.pid
    # ssh argv construction goes through the transport
    seen = []
    r = RemoteClient("user@host:2222", key="/k", transport=lambda argv, data=None: (seen.append(argv) or (0, "ok", "")))
    assert r.exec("uptime")[1] == "ok" and seen[0][-2:] == ["user@host", "uptime"] and "-p" in seen[0] and "/k" in seen[0]
    # git bundle push
    repo = tmp_path / "repo"
    repo.mkdir()
    git = lambda *a: subprocess.run(["git", "-c", "user.name=t", "-c", "user.email=t@t", "-C", str(repo), *a], check=True, capture_output=True)  # noqa: E731
    git("init", "-q", "-b", "main")
    (repo / "f.txt").write_text("v1")
    git("add", "-A"); git("commit", "-qm", "one")
    commit = c.push(repo, str(tmp_path / "deploy"), ref="main")
    assert (tmp_path / "deploy" / "f.txt").read_text() == "v1" and len(commit) == 40
    (repo / "f.txt").write_text("v2")
    git("commit", "-qam", "two")
    c.push(repo, str(tmp_path / "deploy"), ref="main")
    assert (tmp_path / "deploy" / "f.txt").read_text() == "v2"


def test_broker_queries_and_provisioning():
    offers = [GPUOffer("lab", "b200-a", "B200", 8, 180, 0.0, "rack1", "nvlink5"), GPUOffer("lab", "h100-a", "H100", 8, 80, 0.0, "rack2", "nvlink4"),
              GPUOffer("cloud", "c1", "B200", 1, 180, 5.5, "us", ""), GPUOffer("cloud", "c2", "A100", 8, 80, 9.0, "eu", "nvlink3", spot=True)]
    lab = StaticProvider("lab", offers[:2], {"b200-a": "ops@b200-a:22"})
    cloud = StaticProvider("cloud", offers[2:])
    client = GPUClient([lab, cloud])
    b200 = client.search((q.gpu_type == "B200") & (q.gpu_count >= 1))
    assert [o.offer_id for o in b200] == ["b200-a", "c1"]
    assert [o.offer_id for o in client.search(q.interconnect.contains("nvlink") & ~(q.spot == True), sort_by="vram_gb", reverse=True)][0] == "b200-a"  # noqa: E712
    assert repr((q.price_per_hour < 6) | q.region.isin(["eu"])) == "(price_per_hour < 6 | region in ['eu'])"
    inst = client.create((q.gpu_type == "B200") & (q.gpu_count == 8))
    assert inst.ssh_connection == "ops@b200-a:22" and [o.offer_id for o in client.search(q.gpu_type == "B200")] == ["c1"]
    with pytest.raises(RuntimeError):
        client.create(q.gpu_type == "TPU")
    with pytest.raises(AttributeError):
        q.nonexistent
    assert client.terminate_all() == 1 and len(client.search(q.gpu_type == "B200")) == 2


def test_code_search(tmp_path):
    (tmp_path / "a.py").write_text("def flash_attention(q, k, v):\n    return q\n\nclass Engine:\n    pass\n")
    (tmp_path / "k.cu").write_text("template <int D>\n__global__ void flash_fwd_kernel(int x) {}\n// tcgen05.mma here\n")
    (tmp_path / ".git").mkdir()
    (tmp_path / ".git" / "x.py").write_text("flash_attention")
    (tmp_path / "bin.dat").write_text("flash_attention")
    ix = CodeIndex(tmp_path).build()
    assert sorted(ix.files) == ["a.py", "k.cu"] and "fla" in trigrams("Flash")
    assert [(h.path, h.line) for h in ix.search("flash_attention")] == [("a.py", 1)]
    assert [h.path for h in ix.search(r"flash_\w+_kernel", regex=True)] == ["k.cu"]
    assert [h.path for h in ix.search("TCGEN05.MMA")] == ["k.cu"] and ix.search("tcgen05.mma", ignore_case=False)
    assert ix._required_literals(r"flash_\w+_kernel") == ["flash_", "_kernel"] and ix._required_literals("a|b") == []
    assert {h.text for h in ix.symbols("Engine")} == {"class Engine"} and any("flash_fwd_kernel" in h.text for h in ix.symbols())
    ix.save(tmp_path / "ix.json")
    ix2 = CodeIndex.load(tmp_path / "ix.json")
    assert ix2.search("Engine")[0].line == 4 and ix2.stale_files() == []


def test_cloud_provider_adapters_with_fake_transport(monkeypatch):
    """Request shapes and reply mapping of the four cloud adapters, against a scripted transport (no network)."""
    import pytest

    from research_b200.infra.broker import GPUClient, q as Q
    from research_b200.infra.broker_providers import (LambdaProvider, PrimeIntellectProvider, ProviderError, RunPodProvider,
                                                      VastProvider, providers_from_env)

    calls = []

    def transport(method, url, headers, body):
        calls.append((method, url, body))
        assert headers["Authorization"] == "Bearer k"
        if url.endswith("/instance-types"):
            return 200, {"data": {"gpu_8x_b200": {"instance_type": {"description": "8x B200 (180 GB)", "price_cents_per_hour": 3992,
                                                                    "specs": {"gpus": 8}},
                                                  "regions_with_capacity_available": [{"name": "us-east-1"}]}}}
        if url.endswith("/instance-operations/launch"):
            return 200, {"data": {"instance_ids": ["i-1"]}}
        if url.endswith("/instances/i-1"):
            return 200, {"data": {"status": "active", "ip": "1.2.3.4"}}
        if url.endswith("/instance-operations/terminate"):
            return 200, {"data": {}}
        if "runpod" in url:
            q = body["query"]
            if "gpuTypes" in q:
                return 200, {"data": {"gpuTypes": [{"id": "NVIDIA B200", "displayName": "B200", "memoryInGb": 180, "secureCloud": True,
                                                    "lowestPrice": {"minimumBidPrice": 3.1, "uninterruptablePrice": 5.9}}]}}
            if "podFindAndDeployOnDemand" in q:
                assert body["variables"]["input"]["gpuTypeId"] == "NVIDIA B200" and body["variables"]["input"]["cloudType"] == "SECURE"
                return 200, {"data": {"podFindAndDeployOnDemand": {"id": "pod-9", "desiredStatus": "RUNNING"}}}
            if "podTerminate" in q:
                return 200, {"data": {"podTerminate": None}}
            return 200, {"errors": [{"message": "bad query"}]}
        if url.endswith("/bundles/"):
            return 200, {"offers": [{"id": 77, "gpu_name": "H100 SXM", "num_gpus": 4, "gpu_ram": 81920, "dph_total": 9.5, "geolocation": "DE"}]}
        if "/asks/77/" in url:
            return 200, {"success": True, "new_contract": 555}
        if "/instances/555/" in url and method == "DELETE":
            return 200, {"success": True}
        if url.endswith("/availability/"):
            return 200, {"B200_180GB": [{"cloudId": "c-1", "gpuCount": 8, "gpuMemory": 180, "prices": {"onDemand": 30.0},
                                         "dataCenter": "dc-7", "interconnectType": "nvlink5", "provider": "px", "socket": "SXM6"}]}
        if url.endswith("/pods/") and method == "POST":
            assert body["pod"]["cloudId"] == "c-1" and body["provider"]["type"] == "px"
            return 200, {"id": "p-3", "status": "PROVISIONING"}
        if "/pods/p-3" in url and method == "DELETE":
            return 200, None
        return 404, {"error": "not found"}

    lam, rp, va, pi = (cls("k", transport) for cls in (LambdaProvider, RunPodProvider, VastProvider, PrimeIntellectProvider))
    client = GPUClient([lam, rp, va, pi])
    offers = client.search(Q.gpu_type.contains("B200"))
    assert {o.provider for o in offers} == {"lambda", "runpod", "primeintellect"} and offers[0].price_per_hour <= offers[-1].price_per_hour
    lo = lam.search()[0]
    assert lo.gpu_count == 8 and lo.vram_gb == 180 and abs(lo.price_per_hour - 39.92) < 1e-9 and lo.region == "us-east-1"
    inst = lam.create(lo, ssh_key_names=["me"])
    assert inst.instance_id == "i-1" and lam.refresh("i-1").ssh_connection == "ubuntu@1.2.3.4:22" and lam.terminate("i-1")
    on_demand = [o for o in rp.search() if not o.spot][0]
    pod = rp.create(on_demand)
    assert pod.instance_id == "pod-9" and pod.status == "running" and rp.terminate("pod-9")
    vo = va.search()[0]
    assert vo.vram_gb == 80 and va.create(vo).instance_id == "555" and va.terminate("555")
    po = pi.search()[0]
    assert po.interconnect == "nvlink5" and pi.create(po).instance_id == "p-3" and pi.terminate("p-3")
    with pytest.raises(ProviderError):
        lam._call("GET", "/nope")
    with pytest.raises(ProviderError):
        rp._gql("query { nonsense }")
    monkeypatch.setenv("VAST_API_KEY", "k")
    for var in ("LAMBDA_API_KEY", "RUNPOD_API_KEY", "PRIME_API_KEY"):
        monkeypatch.delenv(var, raising=False)
    assert [p.name for p in providers_from_env(transport)] == ["vast"]
