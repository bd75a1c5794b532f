"""Stand-alone process groups over gloo: a custom group from a tcp:// address,
pair sub-groups over its store, and the send/recv self-check."""

import pytest
import torch
import torch.multiprocessing as mp

WORLD = 4


def _rank_main(rank, port, q):
    from awex_b200.parallel.process_group import (
        create_pair_subgroups_from_parent, init_custom_process_group, setup_batch_isend_irecv,
    )

    try:
        group = init_custom_process_group("gloo", f"tcp://127.0.0.1:{port}", timeout_s=60, world_size=WORLD, rank=rank)
        setup_batch_isend_irecv(group, torch.device("cpu"))
        total = torch.tensor([float(rank)])
        group.all_reduce(total)
        pairs = create_pair_subgroups_from_parent(group._store, rank, [(0, 1), (2, 3)], backend="gloo", timeout_s=60)
        (a, b), pair = next(iter(pairs.items()))
        buf = torch.full((3,), float(rank))
        if rank == a:
            pair.send(buf, 1).wait()
        else:
            pair.recv(buf, 0).wait()
        group.barrier()
        q.put((rank, float(total.item()), list(pairs), buf.tolist()))
    except BaseException as exc:
        q.put((rank, repr(exc), None, None))
        raise


@pytest.mark.timeout(180)
def test_custom_group_and_pair_subgroups():
    from awex_b200.utils.common import get_free_port

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = get_free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, port, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=150) for _ in procs)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    for rank, total, pairs, buf in results:
        assert total == 6.0, (rank, total)
        assert pairs == [(0, 1)] if rank < 2 else pairs == [(2, 3)]
        assert buf == [float(rank - rank % 2)] * 3  # the odd rank received its partner's values


def test_custom_group_argument_checks():
    from awex_b200.parallel.process_group import create_pair_subgroups_from_parent, init_custom_process_group

    with pytest.raises(ValueError):
        init_custom_process_group("gloo", "tcp://127.0.0.1:1")
    with pytest.raises(ValueError):
        init_custom_process_group("gloo", "env://", world_size=2, rank=0)
    with pytest.raises(ValueError):
        create_pair_subgroups_from_parent(None, 0, [(1, 1)], backend="gloo")
