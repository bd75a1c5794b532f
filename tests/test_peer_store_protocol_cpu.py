"""The host protocol of the peer-store data plane, run on the CPU: real
`PeerStoreSender` / `PeerStoreReceiver`, real MetaServer, real lowering,
descriptor encoding and validation; the device pieces are stand-ins (address
books over host pointers, a "kernel" that runs the descriptor table through the
host interpreter, flag kernels that do nothing).  What is checked: who publishes
what, in which order the sides shake hands, that the table the sender built
moves the right bytes, and what happens when a receiver's parameters move."""

import contextlib
import threading
from types import SimpleNamespace

import pytest
import torch

from awex_b200.parallel import peer_memory
from awex_b200.parallel.peer_memory import AddressBook
from awex_b200.transfer.descriptors import TensorAddr
from awex_b200.transfer.table_interpreter import HostMemory, run_table

ACTING = threading.local()  # which "process" the code under test (of this thread) currently belongs to
GPU_OF = {}  # process -> GPU identity
MEMORY = []  # every tensor a fake kernel may touch


def who():
    return getattr(ACTING, "name", "nobody")


def gpu():
    return getattr(ACTING, "gpu", None) or GPU_OF[who()]


@contextlib.contextmanager
def acting_as(name, on_gpu=None):
    previous, ACTING.name, ACTING.gpu = (who(), getattr(ACTING, "gpu", None)), name, on_gpu
    try:
        yield
    finally:
        ACTING.name, ACTING.gpu = previous


class FakeExporter:
    def __init__(self, device_index=None):
        self.device_index, self.epoch, self._last = 0, 0, {}

    def export(self, named, with_handles=True):
        self.epoch += 1
        book = AddressBook(("box", who()), 0, gpu(), self.epoch)
        for name, t in named:
            lo, hi = TensorAddr.of(t).byte_span()
            book.segments.append((b"", lo, hi - lo))
            book.tensors[name] = (len(book.segments) - 1, t.data_ptr() - lo, tuple(t.shape), tuple(t.stride()), str(t.dtype).replace("torch.", ""))
            self._last[name] = t.data_ptr()
        return book

    def changed(self, named):
        return any(self._last.get(n) != t.data_ptr() for n, t in named if t.numel())


class FakeImporter:
    opened = closed = 0

    def __init__(self):
        FakeImporter.opened += 1

    def resolve(self, book):
        return {n: TensorAddr(book.segments[seg][1] + off, tuple(shape), tuple(strides), getattr(torch, dtype))
                for n, (seg, off, shape, strides, dtype) in book.tensors.items()}

    def close_all(self):
        FakeImporter.closed += 1


class FakeProgram:
    built = 0

    def __init__(self, table, n_tiles, device, ready_pad=None, ready_slots=(), done_flag_addrs=(), timeout_ms=0, grid=0, encoder=None, interleave=True,
                 desc_group=None, group_cost=None):
        from awex_b200.transfer.descriptors import build_cta_plan, plan_tile_order

        FakeProgram.built += 1
        self.table, self.n_tiles, self.encoder = table, n_tiles, encoder
        self.ready_slots, self.interleave, self.launches = list(ready_slots), interleave, []
        self.status = SimpleNamespace(raise_if_failed=lambda: None)
        self.grouped, self.group_cost = desc_group is not None, dict(group_cost or {})
        self.order = None
        if interleave and n_tiles:  # the order in which 16 CTAs would visit the tiles
            plan, index = build_cta_plan(table, n_tiles, min(16, n_tiles), 1, encoder.desc_dst if desc_group is True else desc_group, group_cost)
            self.plan, self.order = plan, plan_tile_order(plan, 1)
            assert sorted(self.order) == list(range(n_tiles)), "the CTA plan must visit every tile exactly once"

    def launch(self, epoch):
        self.launches.append(epoch)
        with DONE:  # what the kernel's first wait does: every peer destination must have announced this epoch
            assert DONE.wait_for(lambda: DONE.ready.get(epoch, 0) >= len(self.ready_slots), timeout=DEVICE_WAIT_S["s"]), f"no ready flags for epoch {epoch}"
        assert run_table(self.table, self.n_tiles, HostMemory(MEMORY), self.encoder.row_offsets, tile_order=self.order) == self.n_tiles
        with DONE:  # what the kernel's last CTA does with the receivers' done flags
            DONE.count[epoch] = DONE.count.get(epoch, 0) + 1
            DONE.notify_all()

    def check(self):
        pass


DONE = threading.Condition()
DONE.count, DONE.ready = {}, {}
DEVICE_WAIT_S = {"s": 30.0}  # how long the stand-in kernels wait for a flag (the real ones: two seconds)


class FakePoster:
    def __init__(self, addrs, device):
        self.n, self.launches = len(addrs), []

    def launch(self, epoch, stream_ptr=None):
        self.launches.append(epoch)
        with DONE:
            DONE.ready[epoch] = DONE.ready.get(epoch, 0) + (1 if self.n else 0)
            DONE.notify_all()


class FakeWaiter:
    """Stands for the kernel that holds the stream until every device sender has raised its flag."""

    def __init__(self, pad, slots, device, timeout_ms=2000):
        self.n, self.launches = len(slots), []
        self.status = SimpleNamespace(raise_if_failed=lambda: None)

    def launch(self, epoch, stream_ptr=None):
        self.launches.append(epoch)
        with DONE:
            assert DONE.wait_for(lambda: DONE.count.get(epoch, 0) >= self.n, timeout=DEVICE_WAIT_S["s"]), f"flags of epoch {epoch} never came"


@pytest.fixture
def fakes(monkeypatch):
    from awex_b200.ops import fused_transfer

    monkeypatch.setattr(peer_memory, "PeerMemoryExporter", FakeExporter)
    monkeypatch.setattr(peer_memory, "PeerMemoryImporter", FakeImporter)
    monkeypatch.setattr(peer_memory, "process_identity", lambda: ("box", who()))
    monkeypatch.setattr(peer_memory, "_device_uuid", lambda index: gpu())
    monkeypatch.setattr(fused_transfer, "TransferProgram", FakeProgram)
    monkeypatch.setattr(fused_transfer, "FlagPoster", FakePoster)
    monkeypatch.setattr(fused_transfer, "FlagWaiter", FakeWaiter)
    DONE.count, DONE.ready = {}, {}
    monkeypatch.setitem(DEVICE_WAIT_S, "s", 30.0)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda device=None: SimpleNamespace(synchronize=lambda: None))
    FakeImporter.opened = FakeImporter.closed = FakeProgram.built = 0
    MEMORY.clear()
    GPU_OF.clear()
    yield


def build_pair(gpus, fp8=False):
    """One training rank (TP1) and one inference rank (TP1) of the tiny model as
    two "processes"; ``gpus`` = (GPU of the trainer, GPU of the server)."""
    from awex_b200.meta.meta_server import MetaServer, MetaServerClient
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout

    GPU_OF.update(train0=gpus[0], infer0=gpus[1])
    job = SimulatedJob(get_arch("tiny-llama"), TrainLayout(tp=1), InferLayout(tp=1, fp8=fp8), dtype=torch.bfloat16 if fp8 else torch.float32)
    items = job.compile_all()[0]
    local = job.local_tensors(0)
    views = job.destination_views()[0]
    MEMORY.extend(list(local.values()) + [p for m in job.infer_models[0] for p in m.parameters()])
    server = MetaServer("127.0.0.1", 0)
    server.start()
    meta = MetaServerClient("127.0.0.1", server.port)
    return job, items, local, views, server, meta


def make_sides(job, items, local, views, meta, **receiver_kw):
    from awex_b200.transfer.transports import PeerStoreReceiver, PeerStoreSender

    required = sorted(n for n in views)
    with acting_as("infer0"):
        receiver = PeerStoreReceiver(meta, views, 0, 1, 1, required, "cpu", wait_timeout_s=20, **receiver_kw)
    with acting_as("train0"):
        sender = PeerStoreSender(meta, items, local, 0, 1, "cpu", wait_timeout_s=20)
    with acting_as("infer0"):
        receiver.connect()
    with acting_as("train0"):
        sender.connect()
    return sender, receiver


def update(sender, receiver, epoch):
    with acting_as("infer0"):
        receiver.begin(epoch)
    with acting_as("train0"):
        sender.send(epoch)
    with acting_as("infer0"):
        receiver.finish(epoch)


@pytest.mark.parametrize("gpus,host_pair", [(("GPU-a", "GPU-a"), True), (("GPU-a", "GPU-b"), False)])
def test_two_processes_exchange_through_books_manifests_and_handshakes(fakes, gpus, host_pair):
    job, items, local, views, server, meta = build_pair(gpus)
    try:
        sender, receiver = make_sides(job, items, local, views, meta)
        assert sender.host_destinations == ([0] if host_pair else []) and receiver.host_senders == ([0] if host_pair else [])
        assert sender.program.ready_slots == ([] if host_pair else [0])  # a peer GPU announces readiness through a device flag
        assert sender.program.interleave and sender.program.grouped  # round-robin chunks inside one CTA group per destination
        assert sender.program.group_cost == ({0: 0.25} if host_pair else {})  # bytes that stay on the GPU are cheap
        assert receiver.bytes_in == sender.bytes_out and sender.bytes_remote == (0 if host_pair else sender.bytes_out)
        update(sender, receiver, 1)
        assert job.mismatches() == [] and sender.program.launches == [1]
        # two processes: the update opened with the rendezvous on the host, whatever GPUs they sit on
        from awex_b200.transfer.transports import done_key, launched_key, ready_key

        assert meta.get_counter(ready_key(0)) == [1, 1] and meta.get_counter(launched_key(1)) == [1]
        assert meta.get_counter(done_key(1)) == ([1] if host_pair else None)  # completion on the host only for a same-GPU pair
        update(sender, receiver, 2)
        assert meta.get_counter(ready_key(0)) == [2, 1] and meta.get_counter(launched_key(1)) == [2]
        assert FakeProgram.built == 1 and FakeImporter.opened == 2  # planned and mapped once, whatever the number of updates
    finally:
        server.stop()


@pytest.mark.parametrize("late", ["sender", "receiver"])
def test_sides_that_reach_the_update_seconds_apart_meet_on_the_host(fakes, late):
    """Trainer and inference side on different GPUs reach an update three seconds
    apart (normal in an RL loop) while the device waits last one second: neither
    kernel is launched before its partner is there, so no device wait runs out,
    and the sender follows the epoch the receiver announces."""
    import time

    job, items, local, views, server, meta = build_pair(("GPU-a", "GPU-b"))
    try:
        sender, receiver = make_sides(job, items, local, views, meta)
        DEVICE_WAIT_S["s"] = 1.0
        failures, order = [], []

        def inference_side(delay):
            try:
                time.sleep(delay)
                with acting_as("infer0"):
                    receiver.begin(5)  # the receiver's own epoch; the sender has counted nothing yet
                    order.append("announced")
                    receiver.finish(5)
            except BaseException as exc:  # noqa: BLE001
                failures.append(exc)

        def training_side(delay):
            try:
                time.sleep(delay)
                with acting_as("train0"):
                    order.append(("sent", sender.send()))
            except BaseException as exc:  # noqa: BLE001
                failures.append(exc)

        threads = [threading.Thread(target=inference_side, args=(3.0 if late == "receiver" else 0.0,)),
                   threading.Thread(target=training_side, args=(3.0 if late == "sender" else 0.0,))]
        started = time.time()
        for t in threads:
            t.start()
        for t in threads:
            t.join(60)
        assert not failures, failures
        assert time.time() - started >= 3.0 and order == ["announced", ("sent", 5)]
        assert sender.program.launches == [5] and sender.last_epoch == 5 and job.mismatches() == []
    finally:
        server.stop()


def test_a_receiver_that_gives_up_withdraws_its_announcement(fakes):
    """The receiver's device wait runs out (its sender never launched a kernel that
    completes): before it reports, it takes its announcement back, on the device
    flags and on the host counter, so that a sender arriving later finds the
    destination not ready."""
    from awex_b200.ops.fused_transfer import TransferError
    from awex_b200.transfer.transports import HostHandshakeTimeout, ready_key

    job, items, local, views, server, meta = build_pair(("GPU-a", "GPU-b"))
    try:
        sender, receiver = make_sides(job, items, local, views, meta)
        sender.host_wait_timeout_s = 0.3

        def failed():
            raise TransferError(3, (0, 0, 0))

        receiver.waiter.status = SimpleNamespace(raise_if_failed=failed)
        receiver.foreign_device_senders = []  # skip the wait for the launch announcement: the device wait is what fails here
        receiver.waiter.launch = lambda epoch, stream_ptr=None: None
        with acting_as("infer0"):
            receiver.begin(1)
            assert meta.get_counter(ready_key(0)) == [1, 1]
            with pytest.raises(TransferError):
                receiver.finish(1)
        assert meta.get_counter(ready_key(0)) == [0, 1] and receiver.poster.launches == [1, 0]
        with acting_as("train0"), pytest.raises(HostHandshakeTimeout):
            sender.send()  # nothing to write into: the announcement is gone
        assert sender.program.launches == []
    finally:
        server.stop()


@pytest.mark.parametrize("gpus", [("GPU-a", "GPU-a"), ("GPU-a", "GPU-b")])
def test_a_receiver_whose_parameters_move_is_followed_by_its_senders(fakes, gpus):
    """An engine that re-allocates its weights between updates (sleep / wake-up):
    the receiver publishes a new address book before it announces the update, the
    announcement names the book's epoch, and a sender that built its table from
    an older book unmaps, fetches and rebuilds before it writes."""
    from awex_b200.transfer.transports import addr_key, ready_key

    job, items, local, views, server, meta = build_pair(gpus)
    try:
        sender, receiver = make_sides(job, items, local, views, meta, may_move=True)
        assert sender.moving_destinations == [0] and meta.get_object(addr_key(0), timeout=5).may_move
        update(sender, receiver, 1)
        assert job.mismatches() == [] and sender.rebuilds == 0
        assert meta.get_counter(ready_key(0)) == [1, 1]  # the announcement carries the epoch of the valid book
        update(sender, receiver, 2)
        assert sender.rebuilds == 0 and FakeProgram.built == 1  # nothing moved: one extra host round trip, nothing else

        # the engine re-allocates every parameter; the old tensors keep their (now stale) contents
        model = job.infer_models[0][0]
        old = dict(model._tensors)
        for name in list(model._tensors):
            model._tensors[name] = torch.zeros_like(old[name])
        MEMORY.extend(model._tensors.values())
        for t in old.values():
            t.fill_(7.0)
        with acting_as("infer0"):
            receiver.rebind(job.destination_views()[0])
        update(sender, receiver, 3)
        assert sender.rebuilds == 1 and FakeProgram.built == 2 and FakeImporter.closed == 1
        assert meta.get_object(addr_key(0), timeout=5).epoch == 2 and meta.get_counter(ready_key(0)) == [3, 2]
        assert job.mismatches() == []                                 # the new tensors hold the weights
        assert all(bool((t == 7.0).all()) for t in old.values())      # and nobody wrote through the stale addresses
        update(sender, receiver, 4)
        assert sender.rebuilds == 1 and sender.program.launches == [3, 4]
        with pytest.raises(KeyError):
            receiver.rebind({})
    finally:
        server.stop()


def test_senders_that_share_their_large_destinations_start_at_different_ones():
    from awex_b200.transfer.transports import PeerStoreSender

    giga = 10**9
    # training TP4 -> two instances of inference TP2: ranks 0, 1 feed shards 0 and 2, ranks 2, 3 feed 1 and 3 (plus crumbs elsewhere)
    tables = {0: {0: 4 * giga, 2: 4 * giga}, 1: {0: 4 * giga, 1: 1000, 2: 4 * giga}, 2: {0: 1000, 1: 4 * giga, 3: 4 * giga}, 3: {1: 4 * giga, 3: 4 * giga}}
    orders = {r: PeerStoreSender.turn_order(r, t) for r, t in tables.items()}
    assert orders == {0: [0, 2], 1: [2, 0, 1], 2: [1, 3, 0], 3: [3, 1]}
    for turn in range(2):  # at every turn each receiver has one writer
        assert sorted(o[turn] for o in orders.values()) == [0, 1, 2, 3]
    # expert-parallel ranks that feed every inference rank: a Latin square
    orders = [PeerStoreSender.turn_order(r, {d: giga for d in range(8)}) for r in range(8)]
    assert all(sorted(o[turn] for o in orders) == list(range(8)) for turn in range(8))


@pytest.mark.parametrize("stripe_mb,turns", [("0", False), ("0.0625", False), ("0", True)])
def test_two_senders_four_receivers_on_six_gpus(fakes, monkeypatch, stripe_mb, turns):
    """Training TP2 -> two engines of inference TP2, every process on a GPU of its
    own: every receiver checks that the senders' manifests tile its views exactly
    once, every sender writes to receivers of both engines; with striping switched on the senders'
    tables are re-ordered and dealt in chunks, and move the same bytes; so do senders that
    take turns at their destinations."""
    from awex_b200.meta.meta_server import MetaServer, MetaServerClient
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout
    from awex_b200.transfer.transports import PeerStoreReceiver, PeerStoreSender

    monkeypatch.setenv("AWEX_XFER_DEST_STRIPE_MB", stripe_mb)
    if turns:
        monkeypatch.setenv("AWEX_XFER_DEST_GROUPS", "0")
        monkeypatch.setenv("AWEX_XFER_DEST_ROTATE", "1")
    job = SimulatedJob(get_arch("tiny-qwen2"), TrainLayout(tp=2), InferLayout(tp=2, num_engines=2), dtype=torch.bfloat16)
    programs = job.compile_all()
    views = job.destination_views()
    GPU_OF.update({f"train{r}": f"GPU-t{r}" for r in programs}, **{f"infer{i}": f"GPU-i{i}" for i in views})
    for r in programs:
        MEMORY.extend(job.local_tensors(r).values())
    MEMORY.extend(p for ms in job.infer_models for m in ms for p in m.parameters())
    server = MetaServer("127.0.0.1", 0)
    server.start()
    meta = MetaServerClient("127.0.0.1", server.port)
    try:
        receivers, senders = {}, {}
        for i, vs in views.items():
            with acting_as(f"infer{i}"):
                receivers[i] = PeerStoreReceiver(meta, vs, i, len(views), len(programs), sorted(n for n in vs if n not in job.aliases), "cpu", wait_timeout_s=20)
        for r, items in programs.items():
            with acting_as(f"train{r}"):
                senders[r] = PeerStoreSender(meta, items, job.local_tensors(r), r, len(views), "cpu", wait_timeout_s=20)
        for i, rx in receivers.items():
            with acting_as(f"infer{i}"):
                rx.connect()
            assert rx.senders and rx.host_senders == []
        for r, tx in senders.items():
            with acting_as(f"train{r}"):
                tx.connect()
            assert len(tx.destinations) >= 2 and tx.program.ready_slots == tx.destinations  # one per engine at least, all on peer GPUs
            assert tx.program.interleave and tx.program.grouped == (stripe_mb == "0" and not turns)
            if tx.program.grouped:  # one group of CTAs per destination, CTAs shared out by bytes
                assert len({(int(e["tile_begin"]), int(e["tile_end"])) for e in tx.program.plan}) == len(tx.destinations)
        if turns:  # the table of each sender opens with another destination
            first = {r: tx.program.encoder.desc_dst[0] for r, tx in senders.items()}
            assert len(set(first.values())) == len(senders), first
        for i, rx in receivers.items():
            with acting_as(f"infer{i}"):
                rx.begin(1)
        for r, tx in senders.items():
            with acting_as(f"train{r}"):
                tx.send(1)
        for i, rx in receivers.items():
            with acting_as(f"infer{i}"):
                rx.finish(1)
        assert job.mismatches() == []
        assert sum(tx.bytes_out for tx in senders.values()) == sum(rx.bytes_in for rx in receivers.values())
        if stripe_mb != "0":
            assert all(tx.program.table.shape[0] > len(programs[r]) for r, tx in senders.items())  # items were cut into stripes
    finally:
        server.stop()


def _drop_expected_head_difference(arch, engine, bad):
    """With ``norm_head`` the served head has unit-norm columns: the raw oracle differs there and only there."""
    return [b for b in bad if b != "lm_head.weight"] if arch.norm_head else bad


@pytest.mark.timeout(120)
@pytest.mark.parametrize("arch_name,validate,moving", [("tiny-llama", 1, False), ("tiny-llama-norm-head", 0, False), ("tiny-llama", 0, True),
                                                     ("tiny-llama-norm-head", 0, "sources")])
def test_public_api_drives_the_peer_store_plane(fakes, monkeypatch, arch_name, validate, moving):
    """`NCCLWeightsWriter` and `WeightsReader` on the peer-store plane (forced
    here; on CPU tensors they would pick messages): metadata exchange, plan,
    lowering, address books, manifests, validated first update with dumps off,
    a second update after the training weights changed."""
    from awex_b200 import NCCLWeightsWriter, WeightsReader
    from awex_b200.meta.meta_server import MetaServer
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticInferenceEngine, SyntheticTrainEngine
    from awex_b200.synthetic.simulate import InferLayout
    from awex_b200.synthetic.topology import infer_rank_infos, train_rank_infos
    from awex_b200.transfer import transports

    monkeypatch.setenv("AWEX_DEVICE_TYPE", "cpu")
    monkeypatch.setattr(transports, "choose_data_plane", lambda device_type, configured=None: "peer_stores")
    # the moving case also shares one GPU between the two processes (host handshake in both directions)
    GPU_OF.update(train0="GPU-a", infer0="GPU-a" if moving is True else "GPU-b", nobody="GPU-x")
    server = MetaServer("127.0.0.1", 0)
    server.start()
    addr = f"127.0.0.1:{server.port}"
    arch = get_arch(arch_name)
    failures = []

    def serve():
        try:
            with acting_as("infer0"):
                engine = SyntheticInferenceEngine(arch, InferLayout(tp=1), infer_rank_infos(tp=1)[0], addr, dtype=torch.float32, device="cpu",
                                                  zero=False,  # holds the step-0 weights, as after loading the same checkpoint
                                                  weights_validation_steps=validate,
                                                  debug_mode_config={"raise_on_validation_fail": True, "parameters_may_move": moving is True})
                MEMORY.extend(engine.model.parameters())
                reader = WeightsReader(engine)
                reader.initialize()
                reader.update_weights(step_id=1)
                failures.extend(("step 1", m) for m in _drop_expected_head_difference(arch, engine, engine.mismatches(step=0)))
                if arch.norm_head:
                    head = dict(engine.model.named_parameters())["lm_head.weight"]
                    norms = head.float().norm(dim=0)
                    assert torch.allclose(norms, torch.ones_like(norms), atol=1e-5), "the head did not arrive with unit-norm columns"
                if moving is True:  # the engine re-allocates all its weights between the updates
                    for name, t in list(engine.model._tensors.items()):
                        engine.model._tensors[name] = torch.zeros_like(t)
                    MEMORY.extend(engine.model._tensors.values())
                reader.update_weights(step_id=2)
                failures.extend(("step 2", m) for m in _drop_expected_head_difference(arch, engine, engine.mismatches(step=2)))
                failures.extend(("validation", v) for v in reader.last_validation_failed)
        except BaseException as exc:
            failures.append(("reader", repr(exc)))
            raise

    thread = threading.Thread(target=serve, daemon=True)
    thread.start()
    try:
        with acting_as("train0"):
            engine = SyntheticTrainEngine(arch, train_rank_infos(tp=1)[0], addr, dtype=torch.float32, device="cpu", comm_backend="nccl",
                                          weights_validation_steps=validate)
            MEMORY.extend(p for chunk in ([engine.model] if not isinstance(engine.model, list) else engine.model) for p in chunk.parameters())
            writer = NCCLWeightsWriter(engine)
            writer.initialize()
            writer.prepare()  # metadata exchange and planning now: sender-side derived buffers exist afterwards
            MEMORY.extend(t for key, t in writer._local.items() if key[0].startswith("__derived__/"))
            assert bool(writer.derived) == arch.norm_head
            writer.write_weights(step_id=1)
            engine.regenerate(step=2)
            if moving == "sources":  # the training framework re-allocates its parameters (same objects, new storage)
                for _name, p in engine.model.named_parameters():
                    p.data = p.data.clone()
                MEMORY.extend(p for _n, p in engine.model.named_parameters())
            writer.write_weights(step_id=2)
            assert type(writer.transport).__name__ == "PeerStoreSender"
            if moving:
                assert writer.transport.rebuilds == 1 and writer.transport.program.launches == [2]  # a new table for the new addresses
                if moving == "sources":
                    assert all(writer._local[key].data_ptr() == p.data_ptr() == writer._encoded_ptrs[key] for key, p in writer._watched)
            else:
                assert writer.transport.rebuilds == 0 and writer.transport.program.launches == [1, 2]
        thread.join(timeout=60)
        assert not thread.is_alive() and failures == []
    finally:
        server.stop()


def test_single_process_emulation_of_all_ranks(fakes):
    """What the smoke test and the one-GPU benchmark do: every rank's program in
    one process on one device, launched in stream order, followed by one waiter."""
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout

    job = SimulatedJob(get_arch("tiny-qwen2"), TrainLayout(tp=2), InferLayout(tp=2, num_engines=2), dtype=torch.bfloat16, device="cpu")
    job.compile_all()
    assert job.check_coverage() == []
    MEMORY.extend(job.source_tensors() + [p for ms in job.infer_models for m in ms for p in m.parameters()])
    programs = job.build_gpu_programs()
    assert len(programs) == 2 and all(p.ready_slots == [] for p in programs.values())  # nobody waits for anybody: stream order
    job.run_gpu(epoch=1)
    job.gpu_status()
    assert job.mismatches() == []


def test_a_receiver_refuses_senders_that_do_not_cover_its_views(fakes):
    """The manifests are checked before anything is mapped or written: a sender
    that lost one item leaves a hole, one that sends an item twice overlaps."""
    from awex_b200.transfer.transports import PeerStoreReceiver, PeerStoreSender

    job, items, local, views, server, meta = build_pair(("GPU-a", "GPU-b"))
    try:
        for broken, word in ((items[:-1], "exactly once.*receives nothing"), (items + items[:1], "exactly once")):
            for key in list(meta.list_keys()):
                meta.delete_if_exists(key)
            with acting_as("infer0"):
                receiver = PeerStoreReceiver(meta, views, 0, 1, 1, sorted(views), "cpu", wait_timeout_s=20)
            with acting_as("train0"):
                PeerStoreSender(meta, broken, local, 0, 1, "cpu", wait_timeout_s=20)
            with acting_as("infer0"), pytest.raises(Exception, match=word):
                receiver.connect()
    finally:
        server.stop()


def test_one_process_with_its_two_roles_on_two_gpus_uses_device_flags(fakes):
    """No stream orders two devices: a destination of the sender's own process on
    another GPU announces readiness through a device flag like any peer; on the
    same GPU the stream order is enough."""
    from awex_b200.transfer.transports import PeerStoreReceiver, PeerStoreSender

    for trainer_gpu, server_gpu, slots in (("GPU-a", "GPU-b", [0]), ("GPU-a", "GPU-a", [])):
        job, items, local, views, server, meta = build_pair((trainer_gpu, server_gpu))
        try:
            with acting_as("both", on_gpu=server_gpu):
                receiver = PeerStoreReceiver(meta, views, 0, 1, 1, sorted(views), "cpu", wait_timeout_s=20)
            with acting_as("both", on_gpu=trainer_gpu):
                sender = PeerStoreSender(meta, items, local, 0, 1, "cpu", wait_timeout_s=20)
            with acting_as("both", on_gpu=server_gpu):
                receiver.connect()
            with acting_as("both", on_gpu=trainer_gpu):
                sender.connect()
            assert sender.host_destinations == [] and receiver.host_senders == []  # one process: no host handshake
            assert sender.program.ready_slots == slots
            with acting_as("both", on_gpu=server_gpu):
                receiver.begin(1)
            with acting_as("both", on_gpu=trainer_gpu):
                sender.send(1)
            with acting_as("both", on_gpu=server_gpu):
                receiver.finish(1)
            assert job.mismatches() == []
        finally:
            server.stop()
            MEMORY.clear()


def test_block_fp8_serving_through_the_peer_store_plane(fakes):
    """bf16 training shards, block-scaled fp8 inference shards: the sender's table
    quantises on the way (weights and scales land in the receiver's tensors)."""
    job, items, local, views, server, meta = build_pair(("GPU-a", "GPU-b"), fp8=True)
    try:
        assert any(it.value_op.kind == "fp8_block" for it in items) and any(n.endswith("_scale_inv") for n in views)
        sender, receiver = make_sides(job, items, local, views, meta)
        update(sender, receiver, 1)
        assert job.mismatches() == []
        assert sender.bytes_out < sender.bytes_in  # one byte per element plus scales leave, two bytes per element are read
    finally:
        server.stop()
