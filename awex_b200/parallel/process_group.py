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
from typing import List, Optional, Sequence

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


def init_weights_update_group(master_address: str, master_port: int, rank: int, world_size: int,
                              group_name: str = "weights_exchange", backend: Optional[str] = None,
                              timeout_s: float = 1800.0, device: Optional[torch.device] = None) -> ExchangeGroup:
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    timeout = timedelta(seconds=timeout_s)
    store = dist.TCPStore(master_address, int(master_port), world_size, is_master=(rank == 0), timeout=timeout,
                          wait_for_workers=False)
    prefixed = dist.PrefixStore(group_name, store)
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
    logger.info(f"joined exchange group {group_name!r}: rank {rank}/{world_size} via {backend} at {master_address}:{master_port}")
    return ExchangeGroup(pg, rank, world_size, backend, store)


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
