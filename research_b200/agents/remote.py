"""Getting a machine for a remote evaluation or training run, and giving it back (rollouts/remote.py:38-258).

Three ways in, one of which a caller picks: a plain ``user@host:port`` (nothing is provisioned or released), an
instance the broker already tracks (``provider:instance_id``), or a new instance that matches a GPU query. The work is
done by ``infra.bifrost.acquire_node`` and ``infra.broker.GPUClient``; this module adds the command-line flags, the
credential lookup and the release rule (an instance this run created is terminated unless the user asked to keep it; a
machine the user named is never touched).
"""

from __future__ import annotations

import os
from typing import Any

from ..infra.bifrost import GPUQuery, acquire_node as _acquire
from ..infra.broker import GPUClient
from ..infra.broker_providers import PROVIDERS, providers_from_env


def get_broker_credentials(env: dict[str, str] | None = None) -> dict[str, str]:
    """``{provider: api key}`` for every provider whose key is in the environment."""
    env = os.environ if env is None else env
    return {name: env[cls.key_env] for name, cls in PROVIDERS.items() if env.get(cls.key_env)}


def add_remote_args(parser: Any) -> None:
    g = parser.add_argument_group("remote machine (pick one of --ssh / --node-id / --provision)")
    g.add_argument("--ssh", default=None, help="user@host[:port] of a machine that is already up")
    g.add_argument("--node-id", default=None, help="provider:instance_id of an instance the broker tracks")
    g.add_argument("--provision", action="store_true", help="create the cheapest instance that matches --gpu-type / --gpu-count")
    g.add_argument("--gpu-type", default="B200")
    g.add_argument("--gpu-count", type=int, default=1)
    g.add_argument("--max-price", type=float, default=None, help="upper bound in $/h for --provision")
    g.add_argument("--ssh-key", default=None, help="private key file (default: the ssh client's own choice)")
    g.add_argument("--keep-alive", action="store_true", help="do not terminate an instance this run created")


def acquire_node(ssh: str | None = None, node_id: str | None = None, provision: bool = False, gpu_type: str = "B200",
                 gpu_count: int = 1, max_price: float | None = None, ssh_key_path: str | None = None,
                 gpu_client: GPUClient | None = None, **kw: Any):
    """``(client, instance | None)``; ``instance`` is None for a plain ssh target. A broker client is built from the
    environment's credentials when none is passed and one is needed."""
    if sum((ssh is not None, node_id is not None, bool(provision))) != 1:
        raise ValueError("give exactly one of ssh, node_id, provision")
    if ssh is None and gpu_client is None:
        providers = providers_from_env()
        if not providers:
            raise RuntimeError("no provider credentials in the environment: set one of " +
                               ", ".join(cls.key_env for cls in PROVIDERS.values()))
        gpu_client = GPUClient(providers)
    query = GPUQuery(type=gpu_type, count=gpu_count, max_price=max_price) if provision else None
    client, inst = _acquire(ssh=ssh, node_id=node_id, provision=query, gpu_client=gpu_client, key=ssh_key_path, **kw)
    if inst is not None:
        inst_created = bool(provision)
        client._rb_release = (gpu_client, inst.instance_id, inst_created)      # what release_node needs, kept with the client
    return client, inst


def acquire_from_args(args: Any, **kw: Any):
    return acquire_node(ssh=args.ssh, node_id=args.node_id, provision=args.provision, gpu_type=args.gpu_type, gpu_count=args.gpu_count,
                        max_price=args.max_price, ssh_key_path=args.ssh_key, **kw)


def release_node(client: Any, instance: Any, keep_alive: bool = False, out=print) -> bool:
    """Terminate ``instance`` if this run created it and ``keep_alive`` is off. Returns True if it was terminated; says
    how to reach an instance that stays up."""
    if instance is None:
        return False
    gpu_client, iid, created = getattr(client, "_rb_release", (None, getattr(instance, "instance_id", None), False))
    if keep_alive or not created or gpu_client is None:
        out(f"instance {instance.provider}:{iid} stays up" + (f" (ssh {instance.ssh_connection})" if instance.ssh_connection else ""))
        return False
    ok = gpu_client.terminate(iid)
    out(f"instance {instance.provider}:{iid} {'terminated' if ok else 'could NOT be terminated: check the provider console'}")
    return ok
