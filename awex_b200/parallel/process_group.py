"""Process groups that span training and inference processes.

The two sides of an exchange are separate jobs with separate default process
groups, so the group that connects them is built from its own TCP store:
transfer rank 0 (the first inference worker) chooses ``(ip, free port)`` and
publishes it as ``master_info`` through the MetaServer
(`awex/reader/nccl_reader.py:80-95`, `awex/util/process_group.py:199-247` in
the reference).  Here the group is a stand-alone c10d backend object (Gloo on
CPU, NCCL on GPUs) that is never registered as anybody's default group, so no
private torch helper is needed.  The fused NVLink data plane does not use a
process group at all; this one carries the CPU transport, bootstrap barriers
and the send/recv baseline.
"""

from __future__ import annotations

from datetime import timedelta
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from awex_b200 import logging

logger = logging.getLogger(__name__)


class ExchangeGroup:
    """Thin wrapper exposing send / recv / barrier on a stand-alone backend."""

    def __init__(self, backend_obj, rank: int, world_size: int, backend: str, store=None):
        self.pg = backend_obj
        self.rank, self.world_size, self.backend = rank, world_size, backend
        self._store = store  # keep the TCP store (and its server) alive

    def send(self, tensor: torch.Tensor, dst: int, tag: int = 0):
        return self.pg.send([tensor], dst, tag)

    def recv(self, tensor: torch.Tensor, src: int, tag: int = 0):
        return self.pg.recv([tensor], src, tag)

    def barrier(self) -> None:
        self.pg.barrier().wait()

    def all_reduce(self, tensor: torch.Tensor, op=dist.ReduceOp.SUM) -> None:
        opts = dist.AllreduceOptions()
        opts.reduceOp = op
        self.pg.allreduce([tensor], opts).wait()

    def destroy(self) -> None:
        self.pg = None
        self._store = None


def _backend_over_store(prefixed, rank: int, world_size: int, backend: str, timeout: timedelta, device, keep_alive, name: str) -> ExchangeGroup:
    if backend == "gloo":
        pg = dist.ProcessGroupGloo(prefixed, rank, world_size, timeout)
    elif backend == "nccl":
        opts = dist.ProcessGroupNCCL.Options()
        opts._timeout = timeout
        pg = dist.ProcessGroupNCCL(prefixed, rank, world_size, opts)
        if device is not None and hasattr(pg, "eager_connect_single_device"):
            pg.eager_connect_single_device(device)
    else:
        raise ValueError(f"unsupported exchange group backend {backend!r}")
    logger.info(f"joined group {name!r}: rank {rank}/{world_size} via {backend}")
    return ExchangeGroup(pg, rank, world_size, backend, keep_alive)


def init_weights_update_group(master_address: str, master_port: int, rank: int, world_size: int,
                              group_name: str = "weights_exchange", backend: Optional[str] = None,
                              timeout_s: float = 1800.0, device: Optional[torch.device] = None) -> ExchangeGroup:
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    timeout = timedelta(seconds=timeout_s)
    store = dist.TCPStore(master_address, int(master_port), world_size, is_master=(rank == 0), timeout=timeout,
                          wait_for_workers=False)
    return _backend_over_store(dist.PrefixStore(group_name, store), rank, world_size, backend, timeout, device, store, group_name)


def init_custom_process_group(backend: Optional[str] = None, init_method: Optional[str] = None, timeout_s: float = 1800.0,
                              world_size: int = -1, rank: int = -1, store=None, group_name: str = "main",
                              device: Optional[torch.device] = None) -> ExchangeGroup:
    """A group beside whatever default group the process already has
    (`awex/util/process_group.py:34-98` in the reference, which reaches into
    torch's private group constructor for this).  Give either a ``store`` or a
    ``tcp://host:port`` ``init_method``; rank 0 hosts the store of the latter."""
    if world_size <= 0 or rank < 0:
        raise ValueError("world_size and rank must be given")
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    timeout = timedelta(seconds=timeout_s)
    if store is None:
        if not init_method or not init_method.startswith("tcp://"):
            raise ValueError("init_custom_process_group needs a store or a tcp://host:port init_method")
        host, _, port = init_method[len("tcp://"):].partition(":")
        store = dist.TCPStore(host, int(port), world_size, is_master=(rank == 0), timeout=timeout, wait_for_workers=False)
    return _backend_over_store(dist.PrefixStore(group_name, store), rank, world_size, backend, timeout, device, store, group_name)


def create_pair_subgroups_from_parent(store, rank: int, pairs: Sequence[Sequence[int]], backend: Optional[str] = None,
                                      timeout_s: float = 1800.0, device: Optional[torch.device] = None) -> dict:
    """Two-rank groups over the parent's store, one per listed pair that
    contains ``rank``; returns ``{(a, b): ExchangeGroup}`` where the group rank
    of ``a`` is 0 (`awex/util/process_group.py:101-196` in the reference)."""
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    timeout = timedelta(seconds=timeout_s)
    out = {}
    for a, b in pairs:
        if a == b:
            raise ValueError(f"a pair needs two different ranks, got ({a}, {b})")
        if rank not in (a, b):
            continue
        name = f"pair_{a}_{b}"
        out[(a, b)] = _backend_over_store(dist.PrefixStore(name, store), 0 if rank == a else 1, 2, backend, timeout, device, store, name)
    return out


def setup_batch_isend_irecv(group: ExchangeGroup, device: torch.device, n_elems: int = 100) -> None:
    """Warm-up and self-check: every rank sends ``n_elems`` floats filled with
    its rank to the next rank and checks what it got from the previous one
    (`awex/util/process_group.py:250-337`)."""
    if group.world_size < 2:
        return
    nxt, prv = (group.rank + 1) % group.world_size, (group.rank - 1) % group.world_size
    out = torch.full((n_elems,), float(group.rank), device=device)
    inp = torch.empty(n_elems, device=device)
    if group.rank % 2 == 0:
        group.send(out, nxt).wait()
        group.recv(inp, prv).wait()
    else:
        group.recv(inp, prv).wait()
        group.send(out, nxt).wait()
    if not torch.all(inp == float(prv)):
        raise RuntimeError(f"exchange group self-check failed on rank {group.rank}: expected {prv}, got {inp[:4].tolist()}")
    group.barrier()
