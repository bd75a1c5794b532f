"""Co-located exchange over library send/recv on CPU: four gloo ranks, each
holding one Megatron-layout training shard (TP=2 x PP=2) and one vLLM-layout
inference shard (two engines of TP=2), walk the ring stages and end with
inference weights bit-identical to the layout built from the canonical weights."""

import pytest
import torch
import torch.multiprocessing as mp

WORLD = 4


def _rank_main(rank, port, use_group, schedule, chunk_bytes, result_q):
    import torch.distributed as dist

    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout
    from awex_b200.transfer.lowering import manifest_by_destination
    from awex_b200.transfer.nccl_comm import NcclColocateTransport

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=WORLD)
    job = SimulatedJob(get_arch("tiny-llama"), TrainLayout(tp=2, pp=2), InferLayout(tp=2, num_engines=2), dtype=torch.float32)
    programs = job.compile_all()
    assert not job.check_coverage()
    local = {(n, 0): t for n, t in job.train_models[rank].named_parameters()}
    views = job.destination_views()[rank]
    incoming = {src: manifest_by_destination(items).get(rank, []) for src, items in programs.items()}
    identity = {r: r for r in range(WORLD)}
    transport = NcclColocateTransport(rank, WORLD, chunk_bytes=chunk_bytes)
    stats = transport.update_weights_in_colocate_mode(identity, identity, programs[rank], local, views, incoming, use_group=use_group, schedule=schedule)
    mine = f"engine{rank // 2}/rank{rank % 2}/"
    bad = [m for m in job.mismatches() if m.startswith(mine)]
    result_q.put((rank, bad, stats["bytes"], transport.peak_staging_bytes))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("use_group,schedule,chunk_bytes", [(True, "ring", 0), (False, "ring", 0), (True, "recursive", 0),
                                                            (True, "recursive", 8192), (False, "ring", 8192)])
def test_staged_colocated_exchange(use_group, schedule, chunk_bytes):
    from awex_b200.utils.common import get_free_port

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = get_free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, port, use_group, schedule, chunk_bytes, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == list(range(WORLD))
    for rank, bad, moved, peak in results:
        assert not bad, (rank, bad[:5])
        assert moved > 0
        if chunk_bytes:
            # runs of at most chunk_bytes (or one oversize entry) per message: far below a whole message
            assert 0 < peak < moved / 2, (peak, moved)


def test_split_by_budget_runs():
    from awex_b200.transfer.nccl_comm import split_by_budget

    assert split_by_budget([], 10) == []
    assert split_by_budget([3, 3, 3], 0) == [(0, 3)]
    assert split_by_budget([3, 3, 3, 3], 6) == [(0, 2), (2, 4)]
    assert split_by_budget([3, 30, 3, 3], 6) == [(0, 1), (1, 2), (2, 4)]  # an oversize entry travels alone
    assert split_by_budget([1] * 5, 0, max_entries=2) == [(0, 2), (2, 4), (4, 5)]
    assert split_by_budget([4, 4, 1, 1, 1], 8, max_entries=2) == [(0, 2), (2, 4), (4, 5)]
    sizes = [5, 1, 7, 2, 2, 9, 4]
    runs = split_by_budget(sizes, 8)
    assert runs[0][0] == 0 and runs[-1][1] == len(sizes) and all(a[1] == b[0] for a, b in zip(runs, runs[1:]))
    assert all(sum(sizes[b:e]) <= 8 or e - b == 1 for b, e in runs)


def test_recursive_partition_schedule_meets_every_pair_once():
    from awex_b200.transfer.nccl_comm import recursive_partition_rounds

    for world in (2, 4, 8, 16):
        met = {r: [] for r in range(world)}
        for r in range(world):
            for peers, send_first in recursive_partition_rounds(r, world):
                met[r].extend(peers)
                for p in peers:  # the two sides of a pair agree on who sends first
                    theirs = [sf for ps, sf in recursive_partition_rounds(p, world) if r in ps]
                    assert theirs == [not send_first]
        for r in range(world):
            assert sorted(met[r]) == [p for p in range(world) if p != r]
    with pytest.raises(ValueError):
        list(recursive_partition_rounds(0, 6))
