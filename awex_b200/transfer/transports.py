"""Data planes that execute a compiled send program.

* :class:`PeerStoreSender` / :class:`PeerStoreReceiver` — the B200 path.  The
  receiver publishes an address book of its live parameter views and a pad of
  completion flags; the sender maps them (CUDA IPC, NVLink peer access),
  encodes its copy items into a descriptor table once, and then every update
  is ONE kernel launch per training rank that reads local shards, applies
  layout / dtype / fp8 transforms and stores straight into the peers'
  parameters.  No NCCL call, staging buffer or host synchronisation sits on
  the path; ordering is carried by per-(sender, receiver) epoch flags in
  device memory with bounded waits.
* :class:`GlooSender` / :class:`GlooReceiver` — the same items moved as packed
  byte messages over an exchange group that spans both worlds (gloo on CPUs,
  NCCL on GPUs); used on CPU-only hosts and where peer mapping is impossible
  (several machines).  ``AWEX_CHUNK_MB`` / ``AWEX_CHUNK_OPS`` bound the staging
  of one message run.  :func:`choose_data_plane` picks between the two planes.

What both replace in the reference: per-operation ``isend``/``irecv`` lists
inside one NCCL group, staging copies for strided views and a barrier per step
(`awex/transfer/nccl_comm.py:378-624`, `awex/writer/nccl_writer.py:197-304`,
`awex/reader/nccl_reader.py:329-398`).

Every update between different processes opens with a rendezvous on the host,
through counters of the MetaServer that a waiter sleeps on (no polling): a
receiver announces the update's epoch (``p2p_ready_<dst>``) once its engine is
paused; a sender launches only after all its destinations have announced, takes
the epoch from their announcements, and announces its launch
(``p2p_launched_<src>``); a receiver queues its flag wait only then.  The device
flags therefore only ever bridge launch latencies, and their bounded waits can
stay short however far the two sides' schedules drift apart (the reference blocks
in NCCL receives for as long as it takes, `awex/reader/nccl_reader.py:329-398`).
A receiver whose wait runs out all the same withdraws its announcement before
it reports, so that a late sender cannot write into an engine that has resumed.

A sender and a receiver that are different processes on the SAME GPU (the
reference's co-located deployment) never wait for each other on the device: two
kernels of different processes are time-sliced, and one that spins on a flag the
other has yet to write can starve it.  Such pairs also learn of completion on the
host (``p2p_done_<src>``).  Roles that share one process are ordered by their
stream and skip the rendezvous.

MetaServer keys used here: ``p2p_addr_<infer transfer rank>`` (address book),
``p2p_manifest_<train transfer rank>`` (what that rank writes where, plus the
address of its ready-flag pad), the three counters above, ``master_info``
(exchange group rendezvous).
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import os
import time

import torch

from awex_b200 import logging
from awex_b200.utils import env
from awex_b200.transfer.cpu_exec import entry_nbytes, pack_message, unpack_message
from awex_b200.transfer.lowering import CopyItem, check_exactly_once, manifest_by_destination

logger = logging.getLogger(__name__)

# relative time per byte of a destination in this GPU's own memory (HBM) against one across NVLink
LOCAL_BYTE_COST = 0.25

DONE_PAD = "__done_flags__"
READY_PAD = "__ready_flags__"


def addr_key(infer_transfer_rank: int) -> str:
    return f"p2p_addr_{infer_transfer_rank}"


def manifest_key(train_transfer_rank: int) -> str:
    return f"p2p_manifest_{train_transfer_rank}"


def ready_key(infer_transfer_rank: int) -> str:
    """Counter ``[epoch, address book epoch]``: this receiver may be written now."""
    return f"p2p_ready_{infer_transfer_rank}"


def launched_key(train_transfer_rank: int) -> str:
    """Counter ``[epoch]``: this sender's kernel for the epoch is on its stream."""
    return f"p2p_launched_{train_transfer_rank}"


def done_key(train_transfer_rank: int) -> str:
    """Counter ``[epoch]``: this sender's writes for the epoch are complete (same-GPU pairs)."""
    return f"p2p_done_{train_transfer_rank}"


class CoverageError(RuntimeError):
    pass


class HostHandshakeTimeout(TimeoutError):
    pass


def wait_counters(meta, keys, epoch: int, timeout_s: float):
    try:
        return meta.wait_counters(list(keys), epoch, timeout_s)
    except TimeoutError as exc:
        raise HostHandshakeTimeout(str(exc)) from exc


def shares_gpu(book_or_record, my_uuid: str, me: Tuple[str, int]) -> bool:
    """Another process on this very GPU?"""
    owner = tuple(book_or_record["owner"] if isinstance(book_or_record, dict) else book_or_record.owner)
    uuid = book_or_record["device_uuid"] if isinstance(book_or_record, dict) else book_or_record.device_uuid
    return owner != tuple(me) and owner[0] == me[0] and uuid == my_uuid


def _collect_manifests(meta, infer_world: int, train_world: int, my_rank: int, timeout: float):
    """All training ranks' manifests; returns (senders, per-sender entries, per-sender record)."""
    senders, entries, records = [], [], {}
    for r in range(train_world):
        rec = meta.get_object(manifest_key(infer_world + r), timeout=timeout)
        mine = rec["manifest"].get(my_rank, [])
        if mine:
            senders.append(r)
            entries.append(mine)
            records[r] = rec
    return senders, entries, records


def _check_coverage(entries, views: Dict[str, torch.Tensor], required: Sequence[str], strict: bool, who: str) -> None:
    shapes = {n: (tuple(v.shape), v.dtype) for n, v in views.items()}
    problems = check_exactly_once(entries, shapes, required)
    if problems:
        msg = f"{who}: incoming writes do not tile the parameters exactly once: {problems[:6]}"
        if strict:
            raise CoverageError(msg)
        logger.error(msg)


# ------------------------------------------------------------------------------------ fused NVLink path
class PeerStoreReceiver:
    def __init__(self, meta, views: Dict[str, torch.Tensor], transfer_rank: int, infer_world: int, train_world: int,
                 required: Sequence[str], device, timeout_ms: int = 2000, wait_timeout_s: float = 10000, strict: bool = True,
                 host_wait_timeout_s: Optional[float] = None, may_move: bool = False):
        from awex_b200.ops.fused_transfer import FlagPad
        from awex_b200.parallel.peer_memory import PeerMemoryExporter

        # the engine may re-allocate or re-map its weights between updates (sleep / wake-up): the address book is
        # re-published when they moved and every update starts with a host handshake that names the valid book
        self.may_move = bool(may_move)
        self.meta, self.views, self.rank = meta, views, transfer_rank
        self.infer_world, self.train_world = infer_world, train_world
        self.required, self.device, self.strict = list(required), torch.device(device), strict
        self.timeout_ms, self.wait_timeout_s = timeout_ms, wait_timeout_s
        self.host_wait_timeout_s = wait_timeout_s if host_wait_timeout_s is None else host_wait_timeout_s
        self.host_senders: List[int] = []
        # senders in other processes: every update opens with the host rendezvous
        self.foreign_senders: List[int] = []
        # CUDA events around this side's GPU work of each update, when a list is put here (benchmarks)
        self.gpu_events: Optional[list] = None
        self.done_pad = FlagPad(train_world, self.device)
        self.exporter = PeerMemoryExporter(self.device.index)
        self.waiter = None
        self.poster = None
        # a receiver that replaces an earlier one of the same rank continues its epochs: flags and counters only grow
        earlier = self.meta.get_counter(ready_key(self.rank)) if hasattr(self.meta, "get_counter") else None
        self.epoch_base = int(earlier[0]) if earlier else 0
        self.publish()

    def _named(self):
        return list(self.views.items()) + [(DONE_PAD, self.done_pad.t)]

    def publish(self) -> None:
        book = self.exporter.export(self._named())
        if self.may_move:
            book.may_move = True
        self.meta.put_object(addr_key(self.rank), book)

    def republish_if_moved(self, force: bool = False) -> bool:
        """Publish a new book when a tensor's address changed (or on ``force``: the
        addresses are the same but the memory behind them is new)."""
        if force or self.exporter.changed(self._named()):
            self.publish()
            return True
        return False

    def rebind(self, views: Dict[str, torch.Tensor]) -> None:
        """The same names now live in other tensors (the next ``begin`` publishes them)."""
        missing = [n for n in self.required if n not in views]
        if missing:
            raise KeyError(f"rebound views lack {missing[:5]}")
        self.views = views

    def connect(self) -> None:
        """Learn who writes here, check their manifests, map their ready pads."""
        from awex_b200.ops.fused_transfer import FlagPoster, FlagWaiter
        from awex_b200.parallel.peer_memory import PeerMemoryImporter, _device_uuid, process_identity

        self.senders, entries, records = _collect_manifests(self.meta, self.infer_world, self.train_world, self.rank, self.wait_timeout_s)
        _check_coverage(entries, self.views, self.required, self.strict, f"inference rank {self.rank}")
        self.importer = PeerMemoryImporter()
        my_uuid, me = _device_uuid(self.exporter.device_index), process_identity()
        self.host_senders = [r for r in self.senders if "owner" in records[r] and shares_gpu(records[r], my_uuid, me)]
        device_senders = [r for r in self.senders if r not in self.host_senders]
        self.foreign_senders = [r for r in self.senders if "owner" not in records[r] or tuple(records[r]["owner"]) != tuple(me)]
        self.foreign_device_senders = [r for r in device_senders if r in self.foreign_senders]
        ready_addrs = []
        for r in device_senders:
            pad = self.importer.resolve(records[r]["ready_pad"])[READY_PAD]
            ready_addrs.append(pad.ptr + 8 * self.rank)
        self.poster = FlagPoster(ready_addrs, self.device)
        self.waiter = FlagWaiter(self.done_pad, device_senders, self.device, timeout_ms=self.timeout_ms)
        self.bytes_in = sum(entry_nbytes(e) for es in entries for e in es)
        on_this_gpu = {r for r in self.senders if "owner" in records[r] and
                       (tuple(records[r]["owner"]) == tuple(me) or r in self.host_senders)}
        self.bytes_in_remote = sum(entry_nbytes(e) for r, es in zip(self.senders, entries) if r not in on_this_gpu for e in es)
        logger.info(f"inference rank {self.rank}: {len(self.senders)} senders {self.senders}, {self.bytes_in} bytes per update")

    def begin(self, epoch: int) -> None:
        """Tell every sender that parameters may be overwritten now: device flags
        for the kernels, the ready counter for the hosts that launch them."""
        if self.may_move:
            self.republish_if_moved()
        self.poster.launch(epoch)
        if self.host_senders or self.may_move:
            # work queued on this GPU before the update must not read half-written weights
            torch.cuda.current_stream(self.device).synchronize()
        if self.foreign_senders:
            # the second value is the epoch of the address book that is valid for this update
            self.meta.put_counter(ready_key(self.rank), [epoch, self.exporter.epoch])

    def finish(self, epoch: int, synchronize: bool = True) -> None:
        try:
            self._finish(epoch, synchronize)
        except Exception:
            # whatever went wrong (no sender announced its launch, a flag never came): this side gives the update
            # up, so nobody may write here any more
            self.withdraw(epoch)
            raise

    def _finish(self, epoch: int, synchronize: bool) -> None:
        if self.foreign_device_senders:
            # queue the device wait only once every sender's kernel is on its stream: the wait's
            # deadline then covers a transfer, not the drift between the two sides' schedules
            wait_counters(self.meta, [launched_key(self.infer_world + r) for r in self.foreign_device_senders], epoch, self.host_wait_timeout_s)
        if self.gpu_events is not None:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            self.waiter.launch(epoch)
            stop.record()
            self.gpu_events.append((start, stop))
        else:
            self.waiter.launch(epoch)
        if self.host_senders:
            wait_counters(self.meta, [done_key(self.infer_world + r) for r in self.host_senders], epoch, self.host_wait_timeout_s)
        if synchronize:
            torch.cuda.current_stream(self.device).synchronize()
            self.waiter.status.raise_if_failed()

    def withdraw(self, epoch: int) -> None:
        """Take back the announcement of ``epoch`` (the update failed on this side):
        a sender that has not started yet then finds the destination not ready and
        gives up without writing, instead of writing into an engine that resumed."""
        try:
            self.poster.launch(epoch - 1)
            if self.foreign_senders:
                self.meta.put_counter(ready_key(self.rank), [epoch - 1, self.exporter.epoch])
            torch.cuda.current_stream(self.device).synchronize()
        except Exception as exc:  # the original failure is what the caller must see
            logger.error(f"inference rank {self.rank}: could not withdraw the announcement of epoch {epoch}: {exc!r}")

    def gpu_launches_per_update(self) -> int:
        return (1 if self.poster and self.poster.n else 0) + (1 if self.waiter and self.waiter.n else 0)

    def close(self) -> None:
        if getattr(self, "importer", None) is not None:
            self.importer.close_all()


class PeerStoreSender:
    def __init__(self, meta, items: Sequence[CopyItem], local: Dict[Tuple[str, int], torch.Tensor], train_rank: int,
                 infer_world: int, device, timeout_ms: int = 2000, wait_timeout_s: float = 10000, validate: bool = True,
                 grid: int = 0, host_wait_timeout_s: Optional[float] = None):
        from awex_b200.ops.fused_transfer import FlagPad
        from awex_b200.parallel.peer_memory import PeerMemoryExporter, _device_uuid, process_identity

        self.meta, self.items, self.local = meta, list(items), local
        self.train_rank, self.infer_world = train_rank, infer_world
        self.transfer_rank = infer_world + train_rank
        self.device = torch.device(device)
        self.timeout_ms, self.wait_timeout_s, self.validate, self.grid = timeout_ms, wait_timeout_s, validate, grid
        self.host_wait_timeout_s = wait_timeout_s if host_wait_timeout_s is None else host_wait_timeout_s
        self.host_destinations: List[int] = []
        # destinations whose owner may move its tensors, and the epoch of the book the current table was built from
        self.moving_destinations: List[int] = []
        self._book_epochs: Dict[int, int] = {}
        self.rebuilds = 0
        # destinations owned by other processes (the rendezvous partners) and the last epoch sent
        self.foreign_destinations: List[int] = []
        self.last_epoch = 0
        self.gpu_events: Optional[list] = None  # CUDA events around each kernel launch, when a list is put here
        self.ready_pad = FlagPad(infer_world, self.device)
        self.exporter = PeerMemoryExporter(self.device.index)
        self.manifest = manifest_by_destination(self.items)
        self.destinations = sorted(self.manifest)
        self.meta.put_object(
            manifest_key(self.transfer_rank),
            {"manifest": self.manifest, "ready_pad": self.exporter.export([(READY_PAD, self.ready_pad.t)]),
             "owner": process_identity(), "device_uuid": _device_uuid(self.exporter.device_index)},
        )
        self.program = None

    def connect(self) -> None:
        """Map every destination's address book and encode the descriptor table."""
        from awex_b200.ops.fused_transfer import TransferProgram
        from awex_b200.parallel.peer_memory import PeerMemoryImporter, _device_uuid, process_identity
        from awex_b200.transfer.descriptors import TensorAddr, encode_items, validate_table

        self.importer = PeerMemoryImporter()
        my_uuid, me = _device_uuid(self.exporter.device_index), process_identity()
        dst_addrs, done_flags, remote = {}, [], []
        for d in self.destinations:
            book = self.meta.get_object(addr_key(d), timeout=self.wait_timeout_s)
            addrs = self.importer.resolve(book)
            dst_addrs[d] = addrs
            done_flags.append(addrs[DONE_PAD].ptr + 8 * self.train_rank)
            self._book_epochs[d] = book.epoch
            if getattr(book, "may_move", False) and tuple(book.owner) != me:
                self.moving_destinations.append(d)
            if tuple(book.owner) != me:
                self.foreign_destinations.append(d)
            if shares_gpu(book, my_uuid, me):
                self.host_destinations.append(d)  # same GPU, other process: completion is announced on the host
            elif tuple(book.owner) != me or book.device_uuid != my_uuid:
                # another process, or this process on another GPU (no stream orders the two devices): device flags
                remote.append(d)
        src_addrs = {key: TensorAddr.of(t) for key, t in self.local.items()}
        table, n_tiles, enc = encode_items(self._ordered_items(), src_addrs, dst_addrs)
        if os.environ.get("AWEX_XFER_OUT_BULK", "0") == "1":
            from awex_b200.transfer.descriptors import mark_bulk_output

            mark_bulk_output(table, enc.desc_dst, remote)
        if self.validate:
            dst_spans = [a.byte_span() for book in dst_addrs.values() for n, a in book.items() if n != DONE_PAD]
            problems = validate_table(table, n_tiles, [a.byte_span() for a in src_addrs.values()], dst_spans, check_overlap=False)
            if problems:
                raise ValueError(f"training rank {self.train_rank}: descriptor table rejected: {problems[:6]}")
        # destinations in this very process are ordered by the stream; the others
        # must announce readiness through a flag before they are overwritten.
        # Tiles are dealt to CTAs in round-robin chunks inside one group of CTAs
        # per destination, sized by the destination's bytes (bytes that stay in
        # this GPU's memory cost about a quarter of bytes that cross NVLink): every
        # receiver is fed during the whole kernel, and cheap and expensive tiles
        # are spread over a group's CTAs.  (One group over the whole table puts all
        # CTAs of a sender on one destination at a time; senders that walk equal
        # tables then meet at the same receiver and halve each other's rate:
        # 8B model, 4 senders -> 2 x 2 receivers, 21.7 ms against 12.2 ms.)
        local = [d for d in self.destinations if d not in remote]
        self.program = TransferProgram(
            table, n_tiles, self.device, ready_pad=self.ready_pad, ready_slots=remote, done_flag_addrs=done_flags,
            timeout_ms=self.timeout_ms, grid=self.grid, encoder=enc, interleave=self._interleave(remote),
            desc_group=True if self._group_by_destination() else None, group_cost={d: LOCAL_BYTE_COST for d in local},
        )
        self.bytes_out, self.bytes_in, self.n_desc = enc.bytes_out, enc.bytes_in, int(table.shape[0])
        # bytes that cross NVLink (destinations on other GPUs) and bytes that stay in this GPU's memory
        self.bytes_remote = sum(entry_nbytes(e) for d in remote for e in self.manifest[d])
        self.bytes_local = self.bytes_out - self.bytes_remote
        logger.info(
            f"training rank {self.train_rank}: {len(self.items)} items -> {self.n_desc} descriptors, {n_tiles} tiles, "
            f"{self.bytes_out} bytes to ranks {self.destinations}"
        )

    def _ordered_items(self) -> List[CopyItem]:
        """Items arrive grouped by destination in ascending rank order.  With
        ``AWEX_XFER_DEST_ROTATE=1`` every sender starts its walk at a different
        destination (:meth:`turn_order`), so that senders which work on one
        destination at a time (round-robin chunks over the whole table, i.e.
        together with ``AWEX_XFER_DEST_GROUPS=0``) take turns at each receiver
        instead of meeting there.  With ``AWEX_XFER_DEST_STRIPE_MB=<MiB>`` the items
        are cut into stripes of that size and the destinations' stripes are merged
        in proportion to their bytes (:func:`stripe_by_destination`), and tiles are
        dealt to CTAs in round-robin chunks: every window of the table, hence
        every moment of the kernel, then feeds all receivers at once.  Both are
        experimental and off by default."""
        stripe = self._stripe_bytes()
        if stripe and len(self.destinations) >= 2:
            from awex_b200.transfer.lowering import stripe_by_destination

            return stripe_by_destination(self.items, stripe)
        if os.environ.get("AWEX_XFER_DEST_ROTATE", "0") != "1" or len(self.destinations) < 2:
            return self.items
        position = {d: i for i, d in enumerate(self.turn_order(self.train_rank, {d: sum(entry_nbytes(e) for e in es) for d, es in self.manifest.items()}))}
        return sorted(self.items, key=lambda it: position[it.dst_rank])  # stable: keeps the order inside a destination

    @staticmethod
    def turn_order(train_rank: int, bytes_to: Dict[int, int]) -> List[int]:
        """The order in which a sender that works on one destination at a time
        visits its destinations.  Destinations that take a sizeable share of the
        bytes (a tenth of the largest or more) come first, in ascending order
        rotated by the sender's rank; the small rest follows.  Senders that share
        their large destinations (training TP peers that feed the same inference
        shard of several instances; expert-parallel ranks that feed every
        inference rank) then start at different receivers and take turns."""
        large_from = max(bytes_to.values()) / 10
        large = sorted(d for d, n in bytes_to.items() if n >= large_from)
        small = sorted(d for d in bytes_to if d not in large)
        shift = train_rank % len(large)
        return large[shift:] + large[:shift] + small

    @staticmethod
    def _stripe_bytes() -> int:
        try:
            return max(0, int(float(os.environ.get("AWEX_XFER_DEST_STRIPE_MB", "0") or "0") * 1024 * 1024))
        except ValueError:
            return 0

    @classmethod
    def _interleave(cls, remote) -> bool:
        """Round-robin chunks (default) or, with ``AWEX_XFER_INTERLEAVE=0``, one
        contiguous tile range per CTA."""
        return os.environ.get("AWEX_XFER_INTERLEAVE", "1") != "0"

    @classmethod
    def _group_by_destination(cls) -> bool:
        """One CTA group per destination (default); ``AWEX_XFER_DEST_GROUPS=0`` or a
        striped table order deal the whole table to all CTAs as one group."""
        return os.environ.get("AWEX_XFER_DEST_GROUPS", "1") != "0" and cls._stripe_bytes() == 0

    def _rendezvous(self, epoch: int) -> int:
        """Wait until every destination in another process has announced an update
        newer than the last one sent; returns its epoch.  The announcement also names
        the address book that is valid for the update: when a destination that may
        move names a newer book than the table was built from, everything is unmapped,
        the books are fetched again and the table is rebuilt."""
        if not self.foreign_destinations:
            return epoch
        values = wait_counters(self.meta, [ready_key(d) for d in self.foreign_destinations], self.last_epoch + 1, self.host_wait_timeout_s)
        announced = {d: int(values[ready_key(d)][0]) for d in self.foreign_destinations}
        if len(set(announced.values())) > 1:
            raise RuntimeError(f"training rank {self.train_rank}: destinations announce different update epochs {announced}; "
                               "an update failed on some of them: start the next update on all inference workers")
        agreed = next(iter(announced.values()))
        if agreed != epoch:
            logger.info(f"training rank {self.train_rank}: following the inference side's epoch {agreed} (own count {epoch})")
        stale = any(int(values[ready_key(d)][1]) != self._book_epochs.get(d) for d in self.moving_destinations)
        if stale:
            self._rebuild("destinations moved")
        return agreed

    def _rebuild(self, why: str) -> None:
        """Unmap everything, fetch the address books again and encode a new table
        from the current source and destination addresses."""
        self.importer.close_all()
        self.host_destinations, self.moving_destinations, self.foreign_destinations, self._book_epochs = [], [], [], {}
        self.connect()
        self.rebuilds += 1
        logger.info(f"training rank {self.train_rank}: {why}, table rebuilt ({self.rebuilds} so far)")

    def rebind_sources(self) -> None:
        """The tensors in ``local`` (the dict this sender was given) were replaced:
        the table holds their old addresses and must be encoded again."""
        self._rebuild("training tensors moved")

    def send(self, epoch: Optional[int] = None, synchronize: bool = True) -> int:
        """One update; returns the epoch it carried (the inference side's, when
        destinations live in other processes)."""
        epoch = self._rendezvous(self.last_epoch + 1 if epoch is None else epoch)
        if env.flag("AWEX_P2P_TRACE"):
            per_dst = {d: sum(entry_nbytes(e) for e in es) for d, es in self.manifest.items()}
            logger.info(f"[p2p] train rank {self.train_rank} epoch {epoch}: {self.n_desc} descriptors, {getattr(self.program, 'total_tiles', self.program.n_tiles)} tiles, "
                        f"bytes per destination {per_dst}, host-synchronised {self.host_destinations}")
        if self.gpu_events is not None:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            self.program.launch(epoch)
            stop.record()
            self.gpu_events.append((start, stop))
        else:
            self.program.launch(epoch)
        self.last_epoch = epoch
        if self.foreign_destinations:
            self.meta.put_counter(launched_key(self.transfer_rank), [epoch])
        if synchronize or self.host_destinations:
            torch.cuda.current_stream(self.device).synchronize()
            self.program.check()
        if self.host_destinations:
            self.meta.put_counter(done_key(self.transfer_rank), [epoch])
        return epoch

    def gpu_launches_per_update(self) -> int:
        """The transfer kernel, plus the lean block-fp8 kernel where the table has a part for it."""
        program = getattr(self, "program", None)
        return 1 + (1 if getattr(program, "lean", None) is not None else 0)

    def close(self) -> None:
        if getattr(self, "importer", None) is not None:
            self.importer.close_all()


# ------------------------------------------------------------------------------------ choice of the data plane
DATA_PLANES = ("peer_stores", "messages")


def choose_data_plane(device_type: str, configured: Optional[str] = None) -> str:
    """``peer_stores``: the fused kernel writes through CUDA-IPC mappings; every
    sender and receiver must sit in one NVLink / PCIe peer domain (one machine).
    ``messages``: one packed message per (sender, destination) over a process
    group (NCCL on GPUs, gloo on CPUs); works across machines, as the reference's
    NCCL mode does.  ``AWEX_DATA_PLANE`` overrides ``configured``; the default is
    peer stores on CUDA devices and messages elsewhere.  The inference side
    publishes its choice in ``infer_conf`` and the training side follows it."""
    choice = os.environ.get("AWEX_DATA_PLANE") or configured or ("peer_stores" if device_type == "cuda" else "messages")
    if choice not in DATA_PLANES:
        raise ValueError(f"data plane must be one of {DATA_PLANES}, got {choice!r}")
    if choice == "peer_stores" and device_type != "cuda":
        raise ValueError("the peer_stores data plane needs CUDA devices")
    return choice


# ------------------------------------------------------------------------------------ CPU / portable path
def _join_exchange_group(meta, transfer_rank: int, world: int, wait_timeout_s: float, device, exchange_timeout_s: float = 1800.0):
    from awex_b200.parallel.process_group import init_weights_update_group
    from awex_b200.utils.common import get_free_port, get_ip_address

    if transfer_rank == 0:
        info = (get_ip_address() if device.type == "cuda" else "127.0.0.1", get_free_port())
        meta.put_object("master_info", info)
    else:
        info = meta.get_object("master_info", timeout=wait_timeout_s)
    backend = "nccl" if device.type == "cuda" else "gloo"
    return init_weights_update_group(info[0], info[1], transfer_rank, world, backend=backend, device=device, timeout_s=exchange_timeout_s)


class GlooSender:
    def __init__(self, meta, items, local, train_rank: int, infer_world: int, train_world: int, device="cpu",
                 wait_timeout_s: float = 10000, exchange_timeout_s: float = 1800.0, **_unused):
        self.exchange_timeout_s = exchange_timeout_s
        self.meta, self.items, self.local = meta, list(items), local
        self.train_rank, self.infer_world, self.train_world = train_rank, infer_world, train_world
        self.transfer_rank = infer_world + train_rank
        self.device, self.wait_timeout_s = torch.device(device), wait_timeout_s
        self.manifest = manifest_by_destination(self.items)
        self.destinations = sorted(self.manifest)
        self.by_dst = {d: [it for it in self.items if it.dst_rank == d] for d in self.destinations}
        self.meta.put_object(manifest_key(self.transfer_rank), {"manifest": self.manifest, "ready_pad": None})
        self.bytes_out = sum(entry_nbytes(e) for es in self.manifest.values() for e in es)

    def connect(self) -> None:
        self.group = _join_exchange_group(self.meta, self.transfer_rank, self.infer_world + self.train_world, self.wait_timeout_s, self.device,
                                          self.exchange_timeout_s)
        self.group.barrier()
        env.warn_about_ignored(logger)

    def send(self, epoch: int, synchronize: bool = True) -> None:
        from awex_b200.transfer.nccl_comm import chunk_budget_from_env, chunk_entries_from_env, split_by_budget

        one_by_one = os.environ.get("AWEX_USE_BATCH_SEND_RECV", "1") == "0"
        budget, max_entries = chunk_budget_from_env(), chunk_entries_from_env()
        bounded = budget > 0 or max_entries > 0  # staging bounded to one run at a time (the receiver cuts the same runs)
        works = []
        for d in self.destinations:
            runs = split_by_budget([entry_nbytes(e) for e in self.manifest[d]], budget, max_entries)
            for b, e in runs:
                msg = pack_message(self.by_dst[d][b:e], self.local).to(self.device)
                if env.flag("AWEX_P2P_TRACE"):
                    logger.info(f"[p2p] train rank {self.train_rank} epoch {epoch}: {msg.numel()} bytes in {e - b} items to rank {d}")
                work = self.group.send(msg, d, tag=epoch & 0x7FFF)
                if one_by_one or bounded:
                    work.wait()
                else:
                    works.append((work, msg))
        for w, _keepalive in works:
            w.wait()
        return epoch

    def gpu_launches_per_update(self) -> int:
        return 0

    def rebind_sources(self) -> None:
        """Messages are packed from whatever ``local`` holds when they are sent: nothing to rebuild."""

    def close(self) -> None:
        pass


class GlooReceiver:
    def __init__(self, meta, views, transfer_rank: int, infer_world: int, train_world: int, required, device="cpu",
                 wait_timeout_s: float = 10000, strict: bool = True, exchange_timeout_s: float = 1800.0, **_unused):
        self.exchange_timeout_s = exchange_timeout_s
        self.meta, self.views, self.rank = meta, views, transfer_rank
        self.infer_world, self.train_world = infer_world, train_world
        self.required, self.device, self.strict, self.wait_timeout_s = list(required), torch.device(device), strict, wait_timeout_s
        self.group = None

    # messages land in whatever the views are when they arrive: moved parameters only need fresh views
    may_move = True

    def publish(self) -> None:
        pass

    def republish_if_moved(self, force: bool = False) -> bool:
        return False

    def rebind(self, views: Dict[str, torch.Tensor]) -> None:
        self.views = views

    def connect(self) -> None:
        self.group = _join_exchange_group(self.meta, self.rank, self.infer_world + self.train_world, self.wait_timeout_s, self.device,
                                          self.exchange_timeout_s)
        self.senders, self.entries, _ = _collect_manifests(self.meta, self.infer_world, self.train_world, self.rank, self.wait_timeout_s)
        _check_coverage(self.entries, self.views, self.required, self.strict, f"inference rank {self.rank}")
        self.bytes_in = sum(entry_nbytes(e) for es in self.entries for e in es)
        self.group.barrier()

    def begin(self, epoch: int) -> None:
        pass

    def finish(self, epoch: int, synchronize: bool = True) -> None:
        from awex_b200.transfer.nccl_comm import chunk_budget_from_env, chunk_entries_from_env, split_by_budget

        budget, max_entries = chunk_budget_from_env(), chunk_entries_from_env()
        self.peak_staging_bytes = 0
        for r, entries in zip(self.senders, self.entries):
            sizes = [entry_nbytes(e) for e in entries]
            for b, e in split_by_budget(sizes, budget, max_entries):  # the sender cuts the same runs from the same sizes
                buf = torch.empty(sum(sizes[b:e]), dtype=torch.uint8, device=self.device)
                self.peak_staging_bytes = max(self.peak_staging_bytes, buf.numel())
                self.group.recv(buf, self.infer_world + r, tag=epoch & 0x7FFF).wait()
                unpack_message(entries[b:e], buf, self.views)

    def gpu_launches_per_update(self) -> int:
        return 0

    def close(self) -> None:
        pass
