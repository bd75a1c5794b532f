"""Library send/recv transport: the portable data plane for links that peer
stores cannot reach (another node, or a CPU run over gloo).

Where the fused kernel writes straight into a peer's parameters, this path ships
one packed message per (sender, destination) pair with ``torch.distributed``
point-to-point calls.  It keeps the host-side pieces the reference's NCCL
transports are made of (`awex/transfer/nccl_comm.py:53-624`): consistency check
of the train<->inference device maps, the ring-stage schedule of the co-located
exchange with its two-phase colouring, round-robin interleaving across peers,
and a watchdog that reports what was in flight when an exchange stalls.
"""

from __future__ import annotations

import faulthandler
import math
import tempfile
import threading
import time
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from awex_b200 import logging

logger = logging.getLogger(__name__)


# ------------------------------------------------------------------------------------ rank maps
def validate_rank_mappings(train_to_infer: Dict[int, int], infer_to_train: Dict[int, int]) -> None:
    """The two device maps of co-located mode must be inverse bijections."""
    for a, b, fwd, back in ((train_to_infer, infer_to_train, "train", "infer"), (infer_to_train, train_to_infer, "infer", "train")):
        for src, dst in a.items():
            if b.get(dst) != src:
                raise ValueError(f"Inconsistent rank mapping: {fwd}_rank {src} -> {back}_rank {dst} but the inverse map returns {b.get(dst)}")


# ------------------------------------------------------------------------------------ ring stages
def ring_peers(rank: int, stage: int, world: int) -> Tuple[int, int]:
    """At ring stage ``stage`` a rank sends to ``rank + stage`` and receives from
    ``rank - stage`` (mod world); stage 0 is the local copy."""
    return (rank + stage) % world, (rank - stage) % world


def compute_two_phase_partition(rank: int, stage_idx: int, world_size: int) -> int:
    """Colour (0 or 1) of ``rank`` at a ring stage.  The edges ``r -> r+stage``
    split the ranks into ``gcd(world, stage)`` cycles; walking a cycle, colours
    alternate, so on even cycles every edge joins a colour-0 rank (sends first)
    to a colour-1 rank (receives first) and blocking calls cannot deadlock."""
    if stage_idx % world_size == 0:
        return 0
    g = math.gcd(world_size, stage_idx)
    cycle_len, step = world_size // g, stage_idx // g
    position = ((rank // g) * pow(step, -1, cycle_len)) % cycle_len
    return position % 2


def recursive_partition_rounds(rank: int, world: int):
    """Rounds of the recursive-partition ("butterfly") schedule of the reference's
    stream-batch transport (`awex/transfer/nccl_stream_batch.py:261-357`): in
    round k the ranks are cut into partitions of ``world / 2^k``; a rank talks
    to ALL ranks in the other half of its partition, the first half sending
    first.  After ``log2(world)`` rounds every pair has met exactly once.
    Yields ``(peers, send_first)``; ``world`` must be a power of two."""
    if world < 1 or world & (world - 1):
        raise ValueError(f"the recursive-partition schedule needs a power-of-two world, got {world}")
    size = world
    while size >= 2:
        half = size // 2
        base = (rank // size) * size
        first = rank - base < half
        other = range(base + half, base + size) if first else range(base, base + half)
        yield list(other), first
        size = half


def interleave_by_peer(ops: Sequence, peer_of: Callable = lambda op: op.peer) -> list:
    """Round-robin over peers so that consecutive operations target different
    links."""
    lanes: Dict[int, list] = {}
    for op in ops:
        lanes.setdefault(peer_of(op), []).append(op)
    order = sorted(lanes)
    out = []
    depth = max((len(v) for v in lanes.values()), default=0)
    for i in range(depth):
        out.extend(lanes[p][i] for p in order if i < len(lanes[p]))
    return out


# ------------------------------------------------------------------------------------ watchdog
class ExchangeWatchdog:
    """Context manager: if the body has not finished after ``timeout_s``, log
    ``describe()`` and the Python stacks of all threads (the reference shells
    out to py-spy, `nccl_comm.py:299-330`; ``faulthandler`` needs no tool)."""

    def __init__(self, what: str, describe: Callable[[], object] = lambda: None, timeout_s: float = 30.0, sink: Optional[Callable[[str], None]] = None):
        self.what, self.describe, self.timeout_s = what, describe, timeout_s
        self.sink = sink or logger.error
        self.fired = False
        self._done = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def _watch(self):
        if self._done.wait(self.timeout_s):
            return
        self.fired = True
        with tempfile.TemporaryFile(mode="w+") as f:
            faulthandler.dump_traceback(file=f, all_threads=True)
            f.seek(0)
            stacks = f.read()
        self.sink(f"[{self.what}] still running after {self.timeout_s:.1f}s; in flight: {self.describe()}\n{stacks}")

    def __enter__(self):
        self._thread = threading.Thread(target=self._watch, name=f"awex-watchdog-{self.what}", daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._done.set()
        self._thread.join()
        return False


# ------------------------------------------------------------------------------------ send / recv
@dataclass
class P2PRequest:
    """One message: ``send=True`` ships ``tensor`` to ``peer``, else receives
    into it.  ``label`` is what the watchdog prints."""

    send: bool
    tensor: torch.Tensor
    peer: int
    label: str = ""


def summarize_requests(reqs: Iterable[P2PRequest]) -> list:
    return [("send" if r.send else "recv", r.label, str(r.tensor.dtype), list(r.tensor.shape), r.tensor.is_contiguous(), r.peer) for r in reqs]


class PeerStreams:
    """A fixed pool of side streams per device, one picked per peer (peer ``i`` in
    sorted order gets stream ``i mod size``), so that messages to one peer keep
    their order while different peers progress independently; the reference's
    ungrouped send path does the same with 64 streams
    (`awex/transfer/nccl_comm.py:34-50,586-624`).  ``make_stream`` is the stream
    factory (a CUDA stream on the current device by default)."""

    SIZE = 64
    _pools: Dict[Tuple[int, int], list] = {}  # (device, stream factory) -> streams

    def __init__(self, peers: Iterable[int], device_index: int = 0, make_stream: Optional[Callable] = None, size: Optional[int] = None):
        size = size or self.SIZE
        pool = self._pools.setdefault((device_index, id(make_stream)), [])
        wanted = min(size, len(set(peers)))
        make = make_stream or (lambda: torch.cuda.Stream(device=device_index))
        while len(pool) < wanted:
            pool.append(make())
        self.by_peer = {peer: pool[i % size] for i, peer in enumerate(sorted(set(peers)))}

    def used(self) -> list:
        seen, out = set(), []
        for s in self.by_peer.values():
            if id(s) not in seen:
                seen.add(id(s))
                out.append(s)
        return out


def batch_send_recv(requests: Sequence[P2PRequest], group=None, blocking: bool = True, use_group: bool = True,
                    watchdog_s: Optional[float] = 30.0, what: str = "batch_send_recv", use_stream: bool = False) -> list:
    """Issue all requests, interleaved across peers.

    ``use_group=True`` coalesces them in one ``batch_isend_irecv`` (one NCCL
    group call: no ordering constraint between peers).  Otherwise they are posted
    one by one as non-blocking calls in interleaved order, on one side stream
    per peer when ``use_stream`` is set and the tensors are on a GPU (the side
    streams first wait for the caller's stream, and the caller's stream waits
    for them at the end).  Returns the pending ``Work`` handles when
    ``blocking`` is false, else waits for all of them."""
    reqs = interleave_by_peer(list(requests))
    if not reqs:
        return []
    if use_group:
        ops = [dist.P2POp(dist.isend if r.send else dist.irecv, r.tensor, r.peer, group=group) for r in reqs]
        works = dist.batch_isend_irecv(ops)
    elif use_stream and reqs[0].tensor.is_cuda:
        device = reqs[0].tensor.device
        streams = PeerStreams((r.peer for r in reqs), device.index or 0)
        caller = torch.cuda.current_stream(device)
        for s in streams.used():
            s.wait_stream(caller)
        works = []
        for r in reqs:
            with torch.cuda.stream(streams.by_peer[r.peer]):
                works.append((dist.isend if r.send else dist.irecv)(r.tensor, r.peer, group=group))
        for s in streams.used():
            caller.wait_stream(s)
    else:
        works = [(dist.isend if r.send else dist.irecv)(r.tensor, r.peer, group=group) for r in reqs]
    if not blocking:
        return works
    if watchdog_s is None:
        for w in works:
            w.wait()
    else:
        with ExchangeWatchdog(what, lambda: summarize_requests(reqs), watchdog_s):
            for w in works:
                w.wait()
    if any(r.tensor.is_cuda for r in reqs):
        torch.cuda.current_stream().synchronize()
    return []


def two_phase_send_recv(rank: int, stage: int, world: int, sends: Sequence[P2PRequest], recvs: Sequence[P2PRequest], group=None, **kw) -> None:
    """Blocking exchange of one ring stage without a grouped call: colour-0 ranks
    send then receive, colour-1 ranks receive then send."""
    first, second = (sends, recvs) if compute_two_phase_partition(rank, stage, world) == 0 else (recvs, sends)
    batch_send_recv(first, group=group, use_group=False, **kw)
    batch_send_recv(second, group=group, use_group=False, **kw)


# ------------------------------------------------------------------------------------ co-located exchange
def split_by_budget(sizes: Sequence[int], budget: int, max_entries: int = 0) -> List[Tuple[int, int]]:
    """Cut a list of message-entry sizes into consecutive ``[begin, end)`` runs of
    at most ``budget`` bytes each (a single entry larger than the budget gets a
    run of its own) and, with ``max_entries > 0``, at most that many entries.
    ``budget <= 0`` sets no byte bound.  Sender and receiver call
    this on the same sizes, so they agree on the runs without a collective; the
    reference reaches the same agreement with a MIN and a MAX all-reduce
    (`awex/transfer/nccl_stream_batch.py:594-672`)."""
    if not sizes:
        return []
    if budget <= 0 and max_entries <= 0:
        return [(0, len(sizes))]
    runs, begin, acc = [], 0, 0
    for i, n in enumerate(sizes):
        if i > begin and ((budget > 0 and acc + n > budget) or (max_entries > 0 and i - begin >= max_entries)):
            runs.append((begin, i))
            begin, acc = i, 0
        acc += n
    runs.append((begin, len(sizes)))
    return runs


def chunk_budget_from_env() -> int:
    """Bytes of staging one message may take, from ``AWEX_CHUNK_MB`` (0 or unset:
    no bound), the reference's knob for its chunked co-located mode
    (`awex/transfer/nccl_stream_batch.py:115`)."""
    import os

    try:
        return max(0, int(float(os.environ.get("AWEX_CHUNK_MB", "0") or "0") * 1024 * 1024))
    except ValueError:
        return 0


def chunk_entries_from_env() -> int:
    """Entries per run from ``AWEX_CHUNK_OPS`` (0 or unset: no bound), the
    reference's override of its computed step
    (`awex/transfer/nccl_stream_batch.py:612-619`)."""
    import os

    try:
        return max(0, int(os.environ.get("AWEX_CHUNK_OPS", "0").strip() or "0"))
    except ValueError:
        return 0


class NcclColocateTransport:
    """Exchange over ONE communicator whose ranks each hold a training shard and
    an inference shard on the same device (`nccl_comm.py:53-224` in the
    reference).  Messages are the packed per-destination payloads of the lowered
    copy items; the walk over ring stages bounds the staging memory to one
    outgoing and one incoming message at a time, and stage 0 is a local copy.
    ``chunk_bytes`` (default: ``AWEX_CHUNK_MB``) bounds it further: each message
    is cut into runs of entries of at most that many bytes, exchanged one run at
    a time (`awex/transfer/nccl_stream_batch.py:438-805`); ``chunk_entries``
    (default: ``AWEX_CHUNK_OPS``) bounds the entries per run.  ``peak_staging_bytes``
    records the largest amount of staging that was live at once.

    ``items`` are this rank's copy items (destination = inference transfer
    rank), ``local`` its training tensors, ``views`` its inference views,
    ``incoming`` maps a sending transfer rank to the manifest entries it will
    deliver here.
    """

    def __init__(self, transfer_rank: int, world_size: int, group=None, device="cpu", chunk_bytes: Optional[int] = None,
                 chunk_entries: Optional[int] = None):
        self.transfer_rank, self.world_size, self.group = transfer_rank, world_size, group
        self.device = torch.device(device)
        self.chunk_bytes = chunk_budget_from_env() if chunk_bytes is None else int(chunk_bytes)
        self.chunk_entries = chunk_entries_from_env() if chunk_entries is None else int(chunk_entries)
        self.peak_staging_bytes = 0

    def _runs(self, entries: Sequence[tuple]) -> List[Tuple[int, int]]:
        from awex_b200.transfer.cpu_exec import entry_nbytes

        return split_by_budget([entry_nbytes(e) for e in entries], self.chunk_bytes, self.chunk_entries)

    def _exchange_chunked(self, out: Dict[int, list], inc: Dict[int, Sequence[tuple]], local, views, exchange, label: str) -> int:
        """Exchange the messages ``out`` (peer -> items) and ``inc`` (peer ->
        manifest entries) run by run: in step ``k`` every message ships its
        ``k``-th run, so at most one run per message is staged at a time."""
        from awex_b200.transfer.cpu_exec import entry_nbytes, pack_message, unpack_message

        out_runs = {p: self._runs([it.manifest_entry() for it in items]) for p, items in out.items()}
        in_runs = {p: self._runs(entries) for p, entries in inc.items()}
        steps = max([len(r) for r in out_runs.values()] + [len(r) for r in in_runs.values()] + [0])
        moved = 0
        for k in range(steps):
            sends, recvs, landing, live = [], [], [], 0
            for peer in sorted(out):
                if k < len(out_runs[peer]):
                    b, e = out_runs[peer][k]
                    msg = pack_message(out[peer][b:e], local).to(self.device)
                    sends.append(P2PRequest(True, msg, peer, f"{label}.{k}->{peer}"))
                    moved += msg.numel()
                    live += msg.numel()
            for peer in sorted(inc):
                if k < len(in_runs[peer]):
                    b, e = in_runs[peer][k]
                    part = inc[peer][b:e]
                    buf = torch.empty(sum(entry_nbytes(x) for x in part), dtype=torch.uint8, device=self.device)
                    recvs.append(P2PRequest(False, buf, peer, f"{label}.{k}<-{peer}"))
                    landing.append((part, buf))
                    live += buf.numel()
            self.peak_staging_bytes = max(self.peak_staging_bytes, live)
            exchange(sends, recvs, f"{label} run {k}")
            for part, buf in landing:
                unpack_message(part, buf, views)
        return moved

    def update_weights_in_colocate_mode(self, train_to_infer: Dict[int, int], infer_to_train: Dict[int, int], items, local,
                                        views, incoming: Dict[int, Sequence[tuple]], use_group: bool = True,
                                        schedule: str = "ring") -> Dict[str, float]:
        from awex_b200.transfer.cpu_exec import execute_items

        validate_rank_mappings(train_to_infer, infer_to_train)
        me, world = self.transfer_rank, self.world_size
        by_dst: Dict[int, list] = {}
        for it in items:
            by_dst.setdefault(it.dst_rank, []).append(it)
        started = time.time()
        moved = 0
        if schedule == "recursive":
            return self._recursive(by_dst, local, views, incoming, started)
        if schedule != "ring":
            raise ValueError(f"unknown schedule {schedule!r}")
        for stage in range(world):
            to, frm = ring_peers(me, stage, world)
            if stage == 0:
                if me in by_dst:
                    moved += execute_items(by_dst[me], local, {me: views})
                continue
            out = {to: by_dst[to]} if to in by_dst else {}
            inc = {frm: incoming[frm]} if incoming.get(frm) else {}

            def exchange(sends, recvs, what, stage=stage):
                if use_group:
                    batch_send_recv(sends + recvs, group=self.group, what=what)
                else:
                    two_phase_send_recv(me, stage, world, sends, recvs, group=self.group, what=what)

            moved += self._exchange_chunked(out, inc, local, views, exchange, f"colocate stage {stage}")
        return {"seconds": time.time() - started, "bytes": float(moved)}

    def _recursive(self, by_dst, local, views, incoming, started) -> Dict[str, float]:
        """log2(world) rounds of two phases; in each phase all messages of one
        direction between the two halves are in flight together."""
        from awex_b200.transfer.cpu_exec import execute_items

        me = self.transfer_rank
        moved = execute_items(by_dst[me], local, {me: views}) if me in by_dst else 0
        for round_idx, (peers, send_first) in enumerate(recursive_partition_rounds(me, self.world_size)):
            out = {p: by_dst[p] for p in peers if p in by_dst}
            inc = {p: incoming[p] for p in peers if incoming.get(p)}

            def exchange(sends, recvs, what, send_first=send_first):
                for phase_reqs in ((sends, recvs) if send_first else (recvs, sends)):
                    batch_send_recv(phase_reqs, group=self.group, what=what)

            moved += self._exchange_chunked(out, inc, local, views, exchange, f"recursive round {round_idx}")
        return {"seconds": time.time() - started, "bytes": float(moved)}



# ------------------------------------------------------------------------------------ per-operation send / recv
def clone_p2p_send_tensor(tensor: torch.Tensor) -> torch.Tensor:
    """A dense copy fit for a point-to-point send (the source may change after
    the call returns)."""
    return tensor.clone(memory_format=torch.contiguous_format)


class RecvStaging:
    """Point-to-point receives need dense buffers; views that are not dense get a
    staging buffer and are filled when :meth:`finish` copies back
    (`awex/transfer/nccl_stream_batch.py:44-66` in the reference)."""

    def __init__(self):
        self.pairs: list = []

    def prepare(self, view: torch.Tensor) -> torch.Tensor:
        if view.is_contiguous():
            return view
        buffer = torch.empty(tuple(view.shape), dtype=view.dtype, device=view.device)
        self.pairs.append((view, buffer))
        return buffer

    @torch.no_grad()
    def finish(self) -> int:
        n = len(self.pairs)
        for view, buffer in self.pairs:
            view.copy_(buffer)
        self.pairs.clear()
        return n


def _round_robin(per_peer: Dict[int, list]) -> list:
    out, depth = [], max((len(v) for v in per_peer.values()), default=0)
    for i in range(depth):
        out.extend(per_peer[p][i] for p in sorted(per_peer) if i < len(per_peer[p]))
    return out


def build_send_requests(plan, tensors: Dict[str, torch.Tensor], slice_context: Optional[dict] = None) -> list:
    """One send per planned operation, from materialised canonical tensors, in
    round-robin order over the peers: the data path of the reference
    (`awex/transfer/nccl_comm.py:378-445`), kept as the in-repo baseline and for
    links the fused kernel cannot reach.  Strided slices are made dense once per
    (name, slice) through ``slice_context``."""
    from awex_b200.transfer.transfer_plan import slice_tensor

    cache = {} if slice_context is None else slice_context
    per_peer: Dict[int, list] = {}
    for peer, ops in plan.operations.items():
        for op in ops:
            piece = slice_tensor(tensors[op.send_shard_meta.name], op, True, slice_context=cache)
            per_peer.setdefault(peer, []).append(P2PRequest(True, piece, peer, op.send_shard_meta.name))
    return _round_robin(per_peer)


def build_recv_requests(plan, tensors: Dict[str, torch.Tensor], staging: RecvStaging) -> list:
    """The receiving mirror of :func:`build_send_requests` (`nccl_comm.py:448-488`):
    the same operations in the same order, into views of the live parameters or
    staging buffers for strided views."""
    from awex_b200.transfer.transfer_plan import slice_tensor

    per_peer: Dict[int, list] = {}
    for peer, ops in plan.operations.items():
        for op in ops:
            view = slice_tensor(tensors[op.recv_shard_meta.name], op, False)
            per_peer.setdefault(peer, []).append(P2PRequest(False, staging.prepare(view), peer, op.recv_shard_meta.name))
    return _round_robin(per_peer)


@torch.no_grad()
def execute_tensors_to_copy(tensors_to_copy: Sequence[torch.Tensor], copy_ops: Sequence, recv_parameters: Dict[str, torch.Tensor],
                            stage: str = "local copies") -> float:
    """Planned operations whose sender and receiver share this process and
    device: plain device-local copies of each sent piece into the receiving
    view's slice (`awex/transfer/nccl_comm.py:225-241` in the reference).  The
    fused kernel does the same through a local destination pointer; this is the
    library path beside it.  Returns the seconds spent."""
    from awex_b200.transfer.transfer_plan import slice_tensor

    if len(tensors_to_copy) != len(copy_ops):
        raise ValueError(f"{stage}: {len(tensors_to_copy)} tensors for {len(copy_ops)} copy operations")
    started = time.time()
    on_gpu = False
    for piece, op in zip(tensors_to_copy, copy_ops):
        view = slice_tensor(recv_parameters[op.recv_shard_meta.name], op, False)
        view.copy_(piece)
        on_gpu = on_gpu or view.is_cuda
    if on_gpu:
        torch.cuda.current_stream().synchronize()
    took = time.time() - started
    logger.info(f"Finished executing {len(copy_ops)} copy operations for {stage}, took {took:.4f} seconds")
    return took


def execute_p2p_requests(requests: Sequence[P2PRequest], stage: str, group=None, use_group: bool = True,
                         watchdog_s: Optional[float] = 30.0) -> float:
    """Run the requests and return the seconds it took (`nccl_comm.py:333-375`)."""
    started = time.time()
    batch_send_recv(requests, group=group, use_group=use_group, watchdog_s=watchdog_s, what=stage)
    took = time.time() - started
    logger.info(f"Finished executing {len(requests)} p2p operations for {stage}, took {took:.4f} seconds")
    return took
