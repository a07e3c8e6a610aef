"""Single-box launcher: one process per GPU.

``relaunch_under_torchrun`` re-executes the current command under ``torch.distributed.run`` with
``--nproc-per-node N`` (rendezvous on 127.0.0.1); ``spawn`` starts N ranks of a Python callable for
tests and embedding.  This replaces the reference's libp2p discovery + bully election
(``oxidize-core/src/mesh/discovery.rs``, ``election.rs``): inside one NVSwitch box the rank set is
fixed at launch and rank 0 is the leader by construction.
"""
from __future__ import annotations

import os
import socket
import sys
from typing import Callable, Sequence


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def torchrun_command(nproc: int, argv: Sequence[str], module: str = "oxidize_b200.cli.main", port: int = 0):
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
            "127.0.0.1", "--master-port", str(port or free_port()), "-m", module] + list(argv)


def relaunch_under_torchrun(nproc: int) -> None:
    if os.environ.get("OXIDIZE_LAUNCHED"):
        raise SystemExit(f"error: expected WORLD_SIZE={nproc} after relaunch, got {os.environ.get('WORLD_SIZE')}")
    env = dict(os.environ, OXIDIZE_LAUNCHED="1")
    cmd = torchrun_command(nproc, sys.argv[1:])
    os.execvpe(cmd[0], cmd, env)


def follower_loop(llm) -> None:
    from ..engine.server_control import follower_loop as _loop

    _loop(llm)


def _entry(rank: int, world: int, port: int, backend: str, fn: Callable, args: tuple) -> None:
    os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    from .comm import init_distributed

    init_distributed(backend)
    fn(rank, world, *args)


def spawn(fn: Callable, world: int, args: tuple = (), backend: str = None) -> None:
    """Run ``fn(rank, world, *args)`` in ``world`` freshly spawned rank processes."""
    import torch.multiprocessing as mp

    mp.spawn(_entry, args=(world, free_port(), backend, fn, args), nprocs=world, join=True)
