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
    c.push(repo, str(tmp_path / "deploy"), ref="main", bootstrap=["cp f.txt copy.txt", "echo built > stamp"])
    assert (tmp_path / "deploy" / "copy.txt").read_text() == "v2" and (tmp_path / "deploy" / "stamp").exists()
    # what is only in the working tree is named, not shipped
    (repo / "f.txt").write_text("v3")
    (repo / "new.txt").write_text("x")
    said = []
    c.push(repo, str(tmp_path / "deploy"), ref="main", warn=said.append)
    assert sorted(c.not_shipped) == ["f.txt", "new.txt"] and "NOT part of this push" in said[0]
    assert (tmp_path / "deploy" / "f.txt").read_text() == "v2" and not (tmp_path / "deploy" / "new.txt").exists()
    # single files on the target: content with quotes and newlines, file mode, atomic replace, removal of files only
    target = str(tmp_path / "fs" / "deep" / "note.txt")
    c.write_file(target, "it's \"quoted\"\n$HOME stays literal\n", mode=0o600)
    assert c.read_file(target) == "it's \"quoted\"\n$HOME stays literal\n" and c.path_exists(target)
    assert oct((tmp_path / "fs" / "deep" / "note.txt").stat().st_mode & 0o777) == "0o600"
    c.write_file(target, b"\x00\x01second")
    assert (tmp_path / "fs" / "deep" / "note.txt").read_bytes() == b"\x00\x01second" and not c.path_exists(target + ".incoming")
    c.ensure_dir(str(tmp_path / "fs" / "made"))
    assert not c.remove_file(str(tmp_path / "fs" / "made")) and (tmp_path / "fs" / "made").is_dir()
    assert c.remove_file(target) and not c.remove_file(target) and not c.path_exists(target)
    with pytest.raises(FileNotFoundError):
        c.read_file(target)
    with pytest.raises(RemoteError):
        c.push(repo, str(tmp_path / "deploy"), ref="main", bootstrap="exit 9")
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


def test_remote_stream_files_server_and_async(tmp_path):
    import asyncio
    import socket

    from research_b200.infra.bifrost import AsyncRemoteClient, ServerInfo

    c = RemoteClient("local", job_dir=str(tmp_path / "jobs"))
    gen = c.exec_stream("echo one; echo two >&2; exit 5")
    lines = []
    try:
        while True:
            lines.append(next(gen))
    except StopIteration as stop:
        assert stop.value == 5
    assert sorted(lines) == ["one", "two"]
    assert c.expand_path("$HOME") and "$" not in c.expand_path("$HOME")

    src = tmp_path / "src"
    (src / "sub").mkdir(parents=True)
    (src / "a.txt").write_text("A")
    (src / "sub" / "b.bin").write_bytes(bytes(range(256)))
    assert c.upload(src, str(tmp_path / "up")) > 0
    assert (tmp_path / "up" / "sub" / "b.bin").read_bytes() == bytes(range(256))
    c.upload(src / "a.txt", str(tmp_path / "single" / "renamed.txt"))
    assert (tmp_path / "single" / "renamed.txt").read_text() == "A"
    assert c.download(str(tmp_path / "up"), tmp_path / "down") == 2 and (tmp_path / "down" / "a.txt").read_text() == "A"
    assert c.download(str(tmp_path / "up" / "sub" / "b.bin"), tmp_path / "one.bin") == 1
    assert (tmp_path / "one.bin").read_bytes() == bytes(range(256))
    with pytest.raises(RemoteError):
        c.download(str(tmp_path / "missing"), tmp_path / "x")
    with pytest.raises(FileNotFoundError):
        c.upload(tmp_path / "nope", "/tmp/x")

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    server = ProcessSpec(f"python3 -m http.server {port} --bind 127.0.0.1", cwd=str(src), name="web")
    info = c.serve(server, port, health_path="/a.txt", timeout=30, poll=0.2)
    try:
        assert isinstance(info, ServerInfo) and info.url == f"http://127.0.0.1:{port}" and c.job_status("web").status == "running"
    finally:
        c.stop_job("web")
    with pytest.raises(RemoteError, match="ended"):
        c.serve(ProcessSpec("echo boom; exit 2", name="dies"), port, timeout=10, poll=0.1)
    r = RemoteClient("u@gpu.example:2200", key="/k")
    argv = r.tunnel_argv(8000, 30000)
    assert argv[0] == "ssh" and "8000:127.0.0.1:30000" in argv and argv[-1] == "u@gpu.example" and "2200" in argv

    async def go():
        ac = AsyncRemoteClient("local", job_dir=str(tmp_path / "jobs"))
        outs = await asyncio.gather(*(ac.exec(f"echo {i}") for i in range(4)))
        streamed = [line async for line in ac.exec_stream("echo x; echo y")]
        return [o[1].strip() for o in outs], streamed

    outs, streamed = asyncio.run(go())
    assert outs == ["0", "1", "2", "3"] and streamed == ["x", "y"]


def test_acquire_node_three_modes():
    from research_b200.infra.bifrost import GPUQuery, acquire_node

    ok = lambda argv, data=None: (0, "ok\n", "")                                   # noqa: E731
    client, inst = acquire_node(ssh="root@h:22", transport=ok)
    assert client.connection == "root@h:22" and inst is None
    offers = [GPUOffer("lab", "m1", "B200", 8, 180, 30.0), GPUOffer("lab", "m2", "B200", 1, 180, 4.0), GPUOffer("lab", "m3", "H100", 8, 80, 16.0)]
    gc = GPUClient([StaticProvider("lab", offers, {"m1": "root@m1", "m2": "root@m2"})])
    client, inst = acquire_node(provision=GPUQuery("B200", count=8, max_price=40.0), gpu_client=gc, transport=ok)
    assert inst.offer.offer_id == "m1" and client.connection == "root@m1"
    again, same = acquire_node(node_id=f"lab:{inst.instance_id}", gpu_client=gc, transport=ok)
    assert same is inst and again.connection == "root@m1"
    with pytest.raises(ValueError):
        acquire_node(ssh="a@b", provision=GPUQuery())
    with pytest.raises(RemoteError):
        acquire_node(node_id="lab:ghost", gpu_client=gc, transport=ok)
    with pytest.raises(RuntimeError):                                                # nothing that large
        acquire_node(provision=GPUQuery("B200", count=16), gpu_client=gc, transport=ok)
    with pytest.raises(TimeoutError):                                                # a machine that never answers
        acquire_node(ssh="root@dead", transport=lambda argv, data=None: (255, "", "refused"), ssh_timeout=0.2, poll=0.05)


def test_infra_cli_gpus_remote_and_code(tmp_path):
    import json

    from research_b200.infra.cli import main, parse_where

    offers = [GPUOffer("lab", "m1", "B200", 8, 180, 30.0, "us"), GPUOffer("lab", "m2", "B200", 1, 180, 4.0, "eu", spot=True),
              GPUOffer("lab", "m3", "H100", 8, 80, 16.0, "us")]
    gc = GPUClient([StaticProvider("lab", offers, {"m1": "root@m1"})])
    cond = parse_where("gpu_type~B200 gpu_count>=8 price_per_hour<40")
    assert [o.offer_id for o in offers if cond(o)] == ["m1"] and parse_where("") is None
    assert [o.offer_id for o in offers if parse_where("spot==true")(o)] == ["m2"]
    with pytest.raises(ValueError):
        parse_where("gpu_count=>8")
    with pytest.raises(AttributeError):
        parse_where("flops>3")
    lines = []
    assert main(["gpus", "search", "--where", "gpu_count>=8"], lines.append, gc) == 0
    assert "m3" in lines[0] and lines[0].index("m3") < lines[0].index("m1") and "m2" not in lines[0]      # cheapest first
    lines.clear()
    assert main(["gpus", "search", "--json", "--limit", "1"], lines.append, gc) == 0 and json.loads(lines[0])[0]["offer_id"] == "m2"
    lines.clear()
    assert main(["gpus", "create", "--where", "gpu_type~B200 gpu_count>=8", "--provider", "lab"], lines.append, gc) == 0
    made = json.loads(lines[0])
    assert made["ssh"] == "root@m1" and made["offer"]["offer_id"] == "m1"
    assert main(["gpus", "terminate", "--provider", "lab", "--id", made["id"]], lines.append, gc) == 0
    assert main(["gpus", "terminate", "--provider", "lab", "--id", made["id"]], lines.append, gc) == 1

    lines.clear()
    assert main(["remote", "exec", "local", "echo hi; exit 4"], lines.append) == 4 and lines == ["hi"]
    lines.clear()
    assert main(["remote", "exec", "local", "--stream", "echo a; echo b"], lines.append) == 0 and lines == ["a", "b"]
    home = tmp_path / "home"
    home.mkdir()
    import os
    old = os.environ.get("HOME")
    os.environ["HOME"] = str(home)                  # jobs are kept under ~/.bifrost/jobs of the target
    try:
        lines.clear()
        assert main(["remote", "run", "local", "--name", "t1", "--env", "X=5", "--wait", "--timeout", "20", "echo val=$X; exit 3"], lines.append) == 3
        assert any("val=5" in x for x in lines)
        lines.clear()
        assert main(["remote", "status", "local", "--name", "t1"], lines.append) == 0 and "exited" in lines[0] and "exit 3" in lines[0]
        assert main(["remote", "logs", "local", "--name", "t1", "--tail", "5"], lines.append) == 0 and "val=5" in lines[-1]
    finally:
        if old is None:
            del os.environ["HOME"]
        else:
            os.environ["HOME"] = old

    proj = tmp_path / "proj"
    proj.mkdir()
    (proj / "mod.py").write_text("def rollout_step(x):\n    return x + 1\n\nclass Sampler:\n    pass\n")
    lines.clear()
    assert main(["code", "index", "--root", str(proj)], lines.append) == 0 and "indexed 1 files" in lines[0]
    lines.clear()
    assert main(["code", "search", "rollout_step", "--root", str(proj)], lines.append) == 0 and lines[0].startswith("mod.py:1:")
    lines.clear()
    assert main(["code", "symbols", "Sampler", "--root", str(proj)], lines.append) == 0 and "mod.py:4" in lines[0]
    assert main(["code", "search", "nothing_like_this", "--root", str(proj)], lines.append) == 1
    (proj / "new.py").write_text("def later():\n    pass\n")                         # an index on disk that predates a file
    lines.clear()
    main(["code", "index", "--root", str(proj)], lines.append)
    assert main(["code", "search", "later", "--root", str(proj)], lines.append) == 0


def test_provision_records_attempts_and_sorts_failures():
    from research_b200.infra.broker import ProvisionResult, categorize_error
    from research_b200.infra.broker_providers import ProviderError

    class Flaky(StaticProvider):
        def __init__(self, name, offers, failures):
            super().__init__(name, offers, {})
            self.failures = dict(failures)

        def create(self, offer, **kw):
            f = self.failures.get(offer.offer_id)
            if isinstance(f, BaseException):
                raise f
            if f == "none":
                return None
            return super().create(offer, **kw)

    offers = [GPUOffer("lab", f"m{i}", "B200", 8, 180, float(i)) for i in range(1, 5)]
    gc = GPUClient([Flaky("lab", offers, {"m1": ProviderError("lab", 503, "no capacity"), "m2": "none"})])
    r = gc.provision(q.gpu_type == "B200")
    assert r.success and r.instance.offer.offer_id == "m3" and [a.error_category for a in r.attempts] == ["unavailable", "unavailable", None]
    assert gc.get_instance(r.instance.instance_id, refresh=False) is r.instance and gc.list_instances() == [r.instance]
    assert gc.provision(q.gpu_type == "H100").no_offers_found
    gc = GPUClient([Flaky("lab", offers, {"m1": ProviderError("lab", 401, "invalid api key"), "m2": TimeoutError("timed out"), "m3": "none"})])
    r = gc.provision(max_attempts=3)
    assert isinstance(r, ProvisionResult) and not r.success and r.credential_error and r.network_error and not r.all_unavailable
    assert "1 credentials error(s)" in r.error_summary and len(r.attempts) == 3
    gc = GPUClient([Flaky("lab", offers, {f"m{i}": RuntimeError("sold out") for i in range(1, 5)})])
    r = gc.provision(max_attempts=2)
    assert r.all_unavailable and "out of capacity" in r.error_summary and len(r.attempts) == 2
    assert categorize_error(ValueError("weird")) == "unknown"


def test_env_injection_bootstrap_detection_worktrees_and_validation(tmp_path):
    from research_b200.infra import bifrost as bf

    c = RemoteClient("local", job_dir=str(tmp_path / "jobs"))
    seen = []
    spy = RemoteClient("local", transport=lambda argv, data=None: (seen.append((argv, data)), bf.subprocess_transport(argv, data))[1])
    code, out, _ = spy.exec_with_env('echo "$API_KEY|$TRICKY"; cd sub 2>/dev/null; pwd', {"API_KEY": "sk-secret", "TRICKY": "a'b \"c\" $HOME"}, cwd=str(tmp_path))
    assert code == 0 and out.splitlines()[0] == "sk-secret|a'b \"c\" $HOME" and out.splitlines()[1] == str(tmp_path)
    argv, data = seen[0]
    assert "sk-secret" not in " ".join(argv) and b"API_KEY=sk-secret" in data                      # the secret is on stdin only
    with pytest.raises(ValueError):
        bf.make_env_payload({"BAD NAME": "x"})
    with pytest.raises(ValueError):
        c.start_job(ProcessSpec("true", name="../escape"))
    with pytest.raises(ValueError):
        c.start_job(ProcessSpec("true", name="ok", env={"1X": "y"}))
    assert bf.validate_job_name(bf.generate_job_name("eval")).startswith("eval-") and bf.validate_working_directory("/srv/run") == "/srv/run"
    for bad in ("", "a/../b", "x\ny"):
        with pytest.raises(ValueError):
            bf.validate_working_directory(bad)
    # dependency bootstrap from the files of a checkout
    have = {"requirements.txt"}
    assert bf.detect_bootstrap(have.__contains__) == "pip install -r requirements.txt"
    have.add("pyproject.toml")
    assert bf.detect_bootstrap(have.__contains__, extra="dev", frozen=True) == "pip install uv && uv sync --frozen --extra dev"
    assert bf.detect_bootstrap(set().__contains__) == ""
    # one worktree per job from one pushed repository
    repo = tmp_path / "repo"
    repo.mkdir()
    git = lambda *a: subprocess.run(["git", "-c", "user.name=t", "-c", "user.email=t@t", "-C", str(repo), *a], check=True, capture_output=True)  # noqa: E731
    git("init", "-q", "-b", "main")
    (repo / "f.txt").write_text("v1")
    (repo / "requirements.txt").write_text("")
    git("add", "-A"); git("commit", "-qm", "one")
    base = str(tmp_path / "remote")
    t1 = c.push_worktree(repo, base, "job-a", ref="main")
    (repo / "f.txt").write_text("v2")
    git("commit", "-qam", "two")
    t2 = c.push_worktree(repo, base, "job-b", ref="main")
    assert (tmp_path / "remote" / "jobs" / "job-a" / "f.txt").read_text() == "v1" and (tmp_path / "remote" / "jobs" / "job-b" / "f.txt").read_text() == "v2"
    assert t1.endswith("jobs/job-a") and t2.endswith("jobs/job-b") and c.detect_bootstrap(t2) == "pip install -r requirements.txt"
    assert c.remove_worktree(base, "job-a") and not (tmp_path / "remote" / "jobs" / "job-a").exists() and (tmp_path / "remote" / "jobs" / "job-b").exists()


def test_instance_registry_and_gpus_commands(tmp_path):
    import json

    from research_b200.infra.cli import instance_info, main, ssh_command

    offers = [GPUOffer("lab", "m1", "B200", 8, 180, 30.0), GPUOffer("lab", "m2", "B200", 1, 180, 4.0)]
    provider = StaticProvider("lab", offers, {"m1": "root@m1:2222", "m2": "root@m2"})
    reg = str(tmp_path / "instances.json")
    gc = GPUClient([provider], registry=reg)
    inst = gc.create(q.gpu_count >= 8)
    # another process (a later command) sees the instance through the registry file
    later = GPUClient([provider], registry=reg)
    assert list(later.instances) == [inst.instance_id] and later.instances[inst.instance_id].offer.gpu_type == "B200"
    later.created_at[inst.instance_id] -= 3 * 3600
    assert [i.instance_id for i in later.older_than(2)] == [inst.instance_id] and later.older_than(5) == [] and abs(later.running_cost() - 90.0) < 0.1
    lines = []
    assert main(["gpus", "list", "--no-refresh"], lines.append, later) == 0 and "8xB200" in lines[0] and "root@m1:2222" in lines[0] and lines[1].startswith("cost so far: $90")
    assert main(["gpus", "ssh", "--id", inst.instance_id, "--key", "/k"], lines.append, later) == 0 and lines[-1] == "ssh -p 2222 -i /k root@m1"
    assert main(["gpus", "status", "--id", inst.instance_id], lines.append, later) == 0 and "running" in lines[-1]
    assert main(["gpus", "status", "--id", "ghost"], lines.append, later) == 1 and ssh_command("u@h") == "ssh u@h"

    def fake(argv, data=None):
        cmd = argv[-1]
        if "nvidia-smi" in cmd:
            return 0, "0, NVIDIA B200, 1024, 183359, 17\n1, NVIDIA B200, 0, 183359, 0\n", ""
        return (0, "/dev/root 2.0T 500G 1.5T 25% /\n", "") if cmd.startswith("df") else (0, "up 3 hours\n", "")

    info = instance_info(later.instances[inst.instance_id], transport=fake)
    assert [g["memory_used_mib"] for g in info["gpus"]] == [1024, 0] and info["disk_free"] == "1.5T" and info["uptime"] == "up 3 hours"
    assert main(["gpus", "cleanup", "--older-than", "2"], lines.append, later) == 0 and lines[-1].startswith("run again with --yes") and later.instances
    assert main(["gpus", "cleanup", "--older-than", "2", "--yes"], lines.append, later) == 0 and not later.instances and len(provider.search()) == 2
    assert json.loads((tmp_path / "instances.json").read_text()) == [] and main(["gpus", "list"], lines.append, later) == 0 and lines[-1] == "no instances"


def _tiny_repo(path):
    import subprocess

    path.mkdir()
    (path / "work.sh").write_text("mkdir -p out && echo result-$TAG > out/result.txt && touch .done\n")
    (path / "fail.sh").write_text("echo broken >&2; touch .failed; sleep 30\n")
    for argv in (["init", "-q"], ["add", "-A"], ["-c", "user.email=a@b", "-c", "user.name=t", "commit", "-q", "-m", "one"]):
        subprocess.run(["git", "-C", str(path), *argv], check=True)
    return path


def test_deploy_experiment_runs_pushes_waits_and_brings_results_back(tmp_path):
    """The whole deployment against this machine as the target: the commit is shipped, the run starts detached with its
    environment, the marker file ends the wait, results come back; a run that writes its failure marker is reported as
    failed at the wait stage with its log, while it is still running."""
    from research_b200.infra.experiment_deploy import DeployJob, deploy_experiment

    repo = _tiny_repo(tmp_path / "repo")
    said = []
    job = DeployJob("demo", "sh work.sh", repo=str(repo), dest=str(tmp_path / "remote"), env={"TAG": "seven"}, bootstrap=None,
                    results=("out", "missing.txt"), local_results=str(tmp_path / "got"), success_marker=".done", poll_s=0.05, timeout_s=20)
    out = deploy_experiment(job, ssh="local", log=said.append)
    assert out.ok and out.stage == "done" and out.commit and out.fetched == {"out": 1}
    assert (tmp_path / "got" / "demo" / "out" / "result.txt").read_text().strip() == "result-seven"
    assert any("no missing.txt" in line for line in said)

    bad = DeployJob("bad", "sh fail.sh", repo=str(repo), dest=str(tmp_path / "remote2"), bootstrap=None, local_results=str(tmp_path / "got"),
                    success_marker=".done", failure_marker=".failed", poll_s=0.05, timeout_s=20)
    out = deploy_experiment(bad, ssh="local", log=said.append)
    assert not out.ok and out.stage == "sync" or out.stage == "wait"
    assert ".failed" in out.error and "broken" in out.log_tail
    assert (tmp_path / "got" / "bad" / "run.log.tail").exists()


def test_deploy_experiment_rents_and_returns_the_machine(tmp_path):
    """With a broker instead of an ssh target the instance is created from the job's query and terminated afterwards,
    also when the run fails; ``keep_running`` leaves it."""
    from dataclasses import replace

    from research_b200.infra.bifrost import GPUQuery
    from research_b200.infra.broker import GPUClient, GPUOffer, StaticProvider
    from research_b200.infra.experiment_deploy import DeployJob, deploy_experiment

    repo = _tiny_repo(tmp_path / "repo")
    offer = GPUOffer("static", "o1", "B200", 1, 180, 3.0)
    provider = StaticProvider("static", [offer], connections={"o1": "local"})
    client = GPUClient([provider])
    job = DeployJob("rent", "sh work.sh", repo=str(repo), dest=str(tmp_path / "r"), bootstrap=None, gpu=GPUQuery("B200", min_vram_gb=100),
                    success_marker=".done", poll_s=0.05, local_results=str(tmp_path / "got"))
    out = deploy_experiment(job, gpu_client=client, log=lambda m: None)
    assert out.ok and out.instance_id and out.terminated and not client.instances
    out = deploy_experiment(replace(job, name="exit1", command="exit 3", success_marker=None), gpu_client=client, log=lambda m: None)
    assert not out.ok and out.exit_code == 3 and out.terminated
    out = deploy_experiment(replace(job, name="keep", keep_running=True), gpu_client=client, log=lambda m: None)
    assert out.ok and not out.terminated and len(client.instances) == 1
    nothing = deploy_experiment(replace(job, gpu=GPUQuery("H100")), gpu_client=client, log=lambda m: None)
    assert not nothing.ok and nothing.stage == "provision"


def test_sweep_launches_one_process_per_config_and_reports_status(tmp_path):
    import time

    from research_b200.infra.experiment_deploy import discover_configs, display_name, format_status, launch_sweep, load_job, main, sweep_status

    repo = _tiny_repo(tmp_path / "repo")
    cfgs = tmp_path / "configs"
    cfgs.mkdir()
    for stem, cmd in (("01_small_model", "sh work.sh"), ("02_big_model", "exit 2"), ("_shared", "")):
        (cfgs / f"{stem}.py").write_text(
            "from research_b200.infra.experiment_deploy import DeployJob\n"
            f"job = DeployJob({stem!r}, {cmd!r}, repo={str(repo)!r}, dest={str(tmp_path / ('remote_' + stem))!r}, bootstrap=None,\n"
            f"                results=('out',), local_results={str(tmp_path / 'got')!r}, poll_s=0.05)\n")
    found = discover_configs(cfgs)
    assert [p.stem for p in found] == ["01_small_model", "02_big_model"] and display_name(found[0]) == "small-model"
    assert [p.stem for p in discover_configs(cfgs, only=["02"])] == ["02_big_model"]
    assert load_job(found[0]).command == "sh work.sh"
    assert main(["sweep", str(cfgs), "--dry-run", "--log-dir", str(tmp_path / "logs")]) == 0 and not (tmp_path / "logs").exists()

    record = launch_sweep(found, tmp_path / "logs", extra_args=["--ssh", "local"], stagger_s=0.0)
    assert len(record["runs"]) == 2 and all("pid" in r for r in record["runs"])
    deadline = time.time() + 120
    while time.time() < deadline:
        rows = sweep_status(tmp_path / "logs")
        if all(r["state"] != "running" for r in rows):
            break
        time.sleep(0.3)
    states = {r["name"]: r["state"] for r in rows}
    assert states == {"small-model": "ok", "big-model": "failed"}, rows
    text = format_status(rows)
    assert "1 ok" in text and "1 failed" in text and "exited with code 2" in text
    assert (tmp_path / "got" / "01_small_model" / "out" / "result.txt").exists()
