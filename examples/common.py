"""Shared pieces of the examples: an offline tokenizer, response text of a sample, tag parsing, an LCS-ratio reward,
and ``run_remote`` (rollouts/examples/rl/base_config.py:12-208: provision or reuse a GPU box, push the repository,
start the script as a detached job, stream its log, fetch the results, release the box).

Every example runs offline on the tiny presets (``python examples/rl/reverse_text/grpo_01_01.py``); pass a checkpoint
directory as ``model_name`` and a Hugging Face tokenizer to ``train`` to run the same task on real weights."""

from __future__ import annotations

import re
import sys
import time
from difflib import SequenceMatcher
from pathlib import Path
from typing import Any

REPO_ROOT = Path(__file__).resolve().parents[1]
if str(REPO_ROOT) not in sys.path:            # examples are run as scripts from anywhere
    sys.path.insert(0, str(REPO_ROOT))

from research_b200.utils.char_tokenizer import CharTokenizer  # noqa: E402


def default_tokenizer() -> CharTokenizer:
    return CharTokenizer()


def response_text(sample: Any, tokenizer: Any = None) -> str:
    """The generated part of a training sample as text."""
    text = (getattr(sample, "metadata", None) or {}).get("response_text")
    if text is None and tokenizer is not None and sample.response_length:
        text = tokenizer.decode(list(sample.tokens[-sample.response_length:]), skip_special_tokens=True)
    if text is None:
        text = getattr(sample, "response", "") or ""
    for stop in ("<|eos|>", "<|im_end|>", "<|endoftext|>"):
        text = text.split(stop)[0]
    return text


def parse_tag(text: str, *tags: str) -> str | None:
    for tag in tags:
        m = re.search(rf"<{tag}>\s*(.*?)\s*</{tag}>", text, re.DOTALL)
        if m:
            return m.group(1).strip()
    return None


def strip_thinking(text: str) -> str:
    return re.sub(r"<think>.*?</think>", "", text, flags=re.DOTALL).strip().strip("\"'")


def lcs_ratio(a: str, b: str) -> float:
    return SequenceMatcher(None, a, b).ratio()


def run_remote(script_path: str, ssh: str | None = None, node_id: str | None = None, gpu_type: str = "B200", gpu_count: int = 1,
               keep_alive: bool = False, gpu_client: Any = None, timeout: float = 7200.0, out=print) -> int:
    """Run an example on a remote GPU box and stream its log here. Exactly one of ``ssh`` / ``node_id`` names an
    existing machine; with neither, the cheapest matching offer of ``gpu_client`` (a ``broker.GPUClient``; default:
    the providers whose API keys are in the environment) is provisioned and, unless ``keep_alive``, released at the end."""
    from research_b200.infra.bifrost import GPUQuery, ProcessSpec, acquire_node

    if ssh is None and gpu_client is None:
        from research_b200.infra.broker import GPUClient
        from research_b200.infra.broker_providers import providers_from_env

        gpu_client = GPUClient(providers_from_env())
    provision = None if (ssh or node_id) else GPUQuery(type=gpu_type, count=gpu_count)
    client, instance = acquire_node(ssh=ssh, node_id=node_id, provision=provision, gpu_client=gpu_client)
    run_name = time.strftime("run_%Y%m%d-%H%M%S", time.gmtime())
    rel = Path(script_path).resolve().relative_to(REPO_ROOT)
    try:
        workspace = client.expand_path("~/.bifrost/workspaces/research_b200")
        commit = client.push(REPO_ROOT, workspace, bootstrap="python -m research_b200._native")     # build the kernels there
        out(f"deployed {commit[:12]} to {client.connection}:{workspace}")
        spec = ProcessSpec(f"python {rel}", cwd=workspace, env={"PYTHONUNBUFFERED": "1", "ROLLOUTS_RUN_NAME": run_name}, name=run_name)
        job = client.start_job(spec)
        out(f"started {run_name} (pid {job.pid}, log {job.log_path})")
        code = 1
        for line in client.exec_stream(f"tail -n +1 --pid={job.pid} -f {job.log_path}"):
            out(line)
        code = client.wait_job(run_name, timeout=timeout).exit_code or 0
        client.download(f"{workspace}/results", REPO_ROOT / "results" / run_name)
        return code
    finally:
        if instance is not None and not keep_alive and gpu_client is not None:
            gpu_client.terminate(instance.instance_id)
            out(f"released {instance.provider}:{instance.instance_id}")
