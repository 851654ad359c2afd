"""SSH foundation with a scripted stand-in for paramiko's client (no network)."""

import asyncio
import io
import os
import stat

import pytest

from research_b200.infra.ssh_foundation import (SSHConnectionInfo, UniversalSSHClient, execute_command_streaming,
                                                execute_command_sync, interactive_ssh_argv, secure_temp_ssh_key,
                                                test_ssh_connection as check_connection)


class _Chan:
    def __init__(self, code):
        self.code = code

    def recv_exit_status(self):
        return self.code


class _Out(io.StringIO):
    def __init__(self, text, code=0):
        super().__init__(text)
        self.channel = _Chan(code)


class FakeParamiko:
    instances = []

    def __init__(self, fail=None):
        self.fail, self.connected_with, self.closed, self.commands = fail, None, False, []
        FakeParamiko.instances.append(self)

    def connect(self, **kw):
        if self.fail:
            raise ConnectionRefusedError(self.fail)
        if kw.get("key_filename"):
            st = os.stat(kw["key_filename"])
            kw["_key_mode"] = stat.S_IMODE(st.st_mode)
            kw["_key_text"] = open(kw["key_filename"]).read()
        self.connected_with = kw

    def exec_command(self, command, timeout=None):
        self.commands.append(command)
        if "echo ssh_ok" in command:
            return None, _Out("ssh_ok\n"), _Out("")
        if "fail" in command:
            return None, _Out("", 3), _Out("boom\n", 3)
        return None, _Out("line one\nline two\n", 0), _Out("")

    def close(self):
        self.closed = True


def test_connection_strings():
    a = SSHConnectionInfo.from_string("root@10.0.0.5:2222", key_path="~/.ssh/id")
    assert (a.username, a.hostname, a.port, a.key_path) == ("root", "10.0.0.5", 2222, "~/.ssh/id") and a.connection_string() == "root@10.0.0.5:2222"
    b = SSHConnectionInfo.from_string("ssh -o StrictHostKeyChecking=no -i /k/key -p 40022 ubuntu@gpu.example.com")
    assert (b.username, b.hostname, b.port, b.key_path) == ("ubuntu", "gpu.example.com", 40022, "/k/key")
    assert SSHConnectionInfo.from_string("ssh me@h").port == 22
    for bad in ("nohost", "user@host", "user@host:notaport", "ssh -p x me@h", "ssh -p 22"):
        with pytest.raises(ValueError):
            SSHConnectionInfo.from_string(bad)
    assert interactive_ssh_argv(a)[:3] == ["ssh", "-p", "2222"] and interactive_ssh_argv(a)[-1] == "root@10.0.0.5"


def test_temp_key_is_private_and_removed(tmp_path):
    with secure_temp_ssh_key("-----BEGIN KEY-----\nabc") as p:
        assert stat.S_IMODE(os.stat(p).st_mode) == 0o600 and open(p).read().endswith("abc\n")
    assert not os.path.exists(p)
    with pytest.raises(RuntimeError):
        with secure_temp_ssh_key("k") as p2:
            raise RuntimeError("x")
    assert not os.path.exists(p2)
    key = tmp_path / "id"
    key.write_text("KEYDATA")
    assert SSHConnectionInfo("h", 22, "u", key_path=str(key)).load_key_content() == "KEYDATA"
    assert SSHConnectionInfo("h", 22, "u", key_content="inline").load_key_content() == "inline"
    with pytest.raises(ValueError):
        SSHConnectionInfo("h", 22, "u", key_path=str(tmp_path / "missing")).load_key_content()


def test_client_sync_streaming_and_async():
    info = SSHConnectionInfo("h", 22, "u", key_content="SECRET")
    c = UniversalSSHClient(FakeParamiko)
    assert c.exec_command("ls") == (-1, "", "not connected")
    assert c.connect(info) and c.connected
    fake = FakeParamiko.instances[-1]
    assert fake.connected_with["_key_mode"] == 0o600 and fake.connected_with["_key_text"] == "SECRET\n"
    assert not os.path.exists(fake.connected_with["key_filename"])           # the key file lived only during connect
    assert c.exec_command("ls") == (0, "line one\nline two\n", "")
    assert c.exec_command("please fail") == (3, "", "boom\n")
    items = list(c.exec_command_streaming("tail -f log"))
    assert items == ["line one", "line two", ("exit", 0)] and fake.commands[-1] == "( tail -f log ) 2>&1"
    c.close()
    assert fake.closed and not c.connected
    bad = UniversalSSHClient(lambda: FakeParamiko(fail="refused"))
    assert not bad.connect(info) and "refused" in bad.last_error and not bad.connected

    async def go():
        a = UniversalSSHClient(FakeParamiko)
        assert await a.aconnect(SSHConnectionInfo("h", 22, "u"))
        r = await a.aexec_command("ls")
        await a.aclose()
        return r

    assert asyncio.run(go())[0] == 0
    assert execute_command_sync(info, "ls", client_factory=FakeParamiko)[1].startswith("line one")
    assert execute_command_sync(info, "ls", client_factory=lambda: FakeParamiko(fail="nope"))[0] == -1
    seen = []
    assert execute_command_streaming(info, "run", seen.append, client_factory=FakeParamiko) == 0 and seen == ["line one", "line two"]
    assert check_connection(info, client_factory=FakeParamiko) == (True, "connected to u@h:22")
    ok, msg = check_connection(info, client_factory=lambda: FakeParamiko(fail="down"))
    assert not ok and "sync path failed" in msg
