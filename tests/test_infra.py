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
