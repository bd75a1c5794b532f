"""The reference-style data path on our own planner, over gloo: two training
ranks (TP=2) materialise their canonical tensors and send one message per
planned operation; one inference rank receives into views of its parameters
(dense staging for strided views).  BASELINE configuration 1 in miniature."""

import pytest
import torch
import torch.multiprocessing as mp

WORLD = 3  # transfer rank 0: inference; 1, 2: training


def _rank_main(rank, port, q):
    import faulthandler

    faulthandler.dump_traceback_later(150, exit=True)  # a rank that is stuck says where, and leaves
    try:
        _rank_body(rank, port, q)
    except BaseException as exc:  # the parent must not wait for a rank that died
        q.put((rank, [f"rank {rank} failed: {exc!r}"], {"op_count": -1}, 0))
        raise


def _rank_body(rank, port, q):
    import torch.distributed as dist

    from awex_b200 import logging
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout
    from awex_b200.transfer.nccl_comm import RecvStaging, build_recv_requests, build_send_requests, execute_p2p_requests
    from awex_b200.transfer.transfer_plan import compute_transfer_plan_stats

    logging.setLevel("WARNING")
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=WORLD)
    train_tp_group = dist.new_group([1, 2], backend="gloo")  # materialising a fused QKV gathers over the training TP group
    job = SimulatedJob(get_arch("tiny-llama"), TrainLayout(tp=2), InferLayout(tp=1), dtype=torch.float32)
    plan = job.builder.build_local_transfer_plan(job.infer_meta, job.train_meta, rank)
    stats = compute_transfer_plan_stats(plan)["total"]
    if rank == 0:
        views = job.destination_views()[0]
        staging = RecvStaging()
        requests = build_recv_requests(plan, views, staging)
        execute_p2p_requests(requests, "receive", use_group=True)
        staged = staging.finish()
        q.put((rank, job.mismatches(), stats, staged))
    else:
        from awex_b200.converter.mcore_converter import set_train_tp_group

        set_train_tp_group(train_tp_group, 2)
        t = rank - 1
        conv = job._train_converter(job.train_ranks[t])
        tensors = {}
        for name, p in job.train_models[t].named_parameters():
            for cname, value in conv.convert_param(name, p, vp_stage=0):
                tensors[cname] = value
        requests = build_send_requests(plan, tensors)
        execute_p2p_requests(requests, "send", use_group=True)
        q.put((rank, [], stats, 0))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(400)
def test_per_operation_send_recv_over_gloo():
    import queue

    from awex_b200.utils.common import get_free_port

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = get_free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, port, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    try:
        results = {r[0]: r[1:] for r in (q.get(timeout=240) for _ in procs)}
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    except queue.Empty:
        pytest.fail("a rank did not report (a stuck rank prints where it stands after 150 s and leaves)")
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
    bad, stats, staged = results[0]
    assert bad == []
    assert stats == {"op_count": 29, "numel": 1705216, "bytes": 6820864}  # the plan of BASELINE configuration 1
    assert results[1][1]["op_count"] + results[2][1]["op_count"] == 29
    assert staged > 0  # column-cut projections arrive through dense staging buffers


def test_recv_staging_and_send_clone():
    from awex_b200.transfer.nccl_comm import RecvStaging, clone_p2p_send_tensor

    base = torch.zeros(4, 4)
    staging = RecvStaging()
    dense = staging.prepare(base[:, 1])
    assert dense.is_contiguous() and dense.data_ptr() != base.data_ptr()
    assert staging.prepare(base[1]) .data_ptr() == base[1].data_ptr()  # dense views are received in place
    dense.copy_(torch.arange(4.0))
    assert staging.finish() == 1 and staging.pairs == []
    assert torch.equal(base[:, 1], torch.arange(4.0)) and not base[:, 0].any()
    view = torch.arange(16.0).reshape(4, 4)[:, 2]
    sent = clone_p2p_send_tensor(view)
    assert sent.is_contiguous() and sent.data_ptr() != view.data_ptr() and torch.equal(sent, view)


def test_planned_operations_inside_one_process_run_as_local_copies():
    """Sender and receiver in one process (the reference's same-GPU operations of
    its co-located mode): every planned operation is a copy of the sent slice into
    the receiving slice."""
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout
    from awex_b200.transfer.nccl_comm import execute_tensors_to_copy
    from awex_b200.transfer.transfer_plan import slice_tensor

    job = SimulatedJob(get_arch("tiny-llama"), TrainLayout(tp=1), InferLayout(tp=2), dtype=torch.float32)
    conv = job._train_converter(job.train_ranks[0])
    tensors = {}
    for name, p in job.train_models[0].named_parameters():
        for cname, value in conv.convert_param(name, p, vp_stage=0):
            tensors[cname] = value
    views = job.destination_views()
    plan = job.builder.build_local_transfer_plan(job.infer_meta, job.train_meta, 2)  # the training rank's plan
    total = 0
    for peer, ops in plan.operations.items():
        pieces = [slice_tensor(tensors[op.send_shard_meta.name], op, True) for op in ops]
        assert execute_tensors_to_copy(pieces, ops, views[peer], stage=f"to {peer}") >= 0
        total += len(ops)
    assert total > 0 and job.mismatches() == []
    with pytest.raises(ValueError, match="copy operations"):
        execute_tensors_to_copy([], next(iter(plan.operations.values()))[:1], views[0])


def test_peer_streams_keep_one_stream_per_peer_within_a_fixed_pool():
    from awex_b200.transfer.nccl_comm import PeerStreams

    made = []

    def make():
        made.append(object())
        return made[-1]

    a = PeerStreams([7, 3, 5, 3], device_index=0, make_stream=make, size=2)
    assert len(made) == 2  # pool bounded by its size, grown only as far as needed
    assert a.by_peer[3] is made[0] and a.by_peer[5] is made[1] and a.by_peer[7] is made[0]  # sorted peers, modulo the pool
    assert a.used() == [made[0], made[1]]
    b = PeerStreams([1], device_index=0, make_stream=make, size=2)
    assert len(made) == 2 and b.by_peer[1] is made[0]  # the pool is shared by later calls
