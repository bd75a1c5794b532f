"""Transfer-plan builder on hand-built shard metadata: key contract, replica
pairing, overlap arithmetic, executing a plan with ``copy_`` on CPU (every
destination element exactly once), determinism, hash and statistics."""

import pytest
import torch

from awex_b200.meta.meta_resolver import assign_global_layout, group_into_replicas
from awex_b200.meta.weight_meta import ParameterMeta, ParameterReplicaMeta, ParameterShardMeta, compute_total_model_size
from awex_b200.sharding.param_sharding import ShardingType
from awex_b200.transfer.transfer_plan import (
    TransferPlan, TransferPlanBuilder, compute_transfer_plan_hash, compute_transfer_plan_stats, normalize_rank_axes, slice_tensor,
)


def shard(name, shape, tp_rank, global_rank, kind=ShardingType.TP_SHARDING, dim=0, n=1, dtype=torch.float32, ep_rank=0, pp_rank=0):
    numel = 1
    for d in shape:
        numel *= d
    return ParameterShardMeta(
        tp_rank=tp_rank, attn_tp_rank=tp_rank, pp_rank=pp_rank, ep_rank=ep_rank, ep_tp_rank=0, global_rank=global_rank,
        world_size=max(n, 1), engine_rank=0, name=name, shape=tuple(shape), numel=numel, dtype=dtype,
        sharding_type=kind, num_shards=n, sharding_dim=dim,
    )


def param(name, shard_shapes, dim=0, first_rank=0, replicas=1, dtype=torch.float32):
    """``replicas`` copies of a tensor cut along ``dim`` into ``shard_shapes``."""
    reps, flat, rank = [], [], first_rank
    for _ in range(replicas):
        one = []
        for i, shape in enumerate(shard_shapes):
            kind = ShardingType.TP_SHARDING if len(shard_shapes) > 1 else ShardingType.NO_SHARDING
            one.append(shard(name, shape, i, rank, kind, dim, len(shard_shapes), dtype))
            rank += 1
        reps.append(one)
        flat.extend(one)
    shape, numel = assign_global_layout(reps)
    return ParameterMeta(name, numel, shape, dtype, flat, [ParameterReplicaMeta(r) for r in reps])


def run_plan(builder, infer_meta, train_meta, truth):
    """Execute every rank's sending plan with copy_ and return destination
    tensors plus per-element write counts."""
    n_inf = builder.infer_world_size
    src = {}
    for p in train_meta:
        for s in p.shards:
            sl = tuple(slice(o, o + e) for o, e in zip(s.global_offset, s.shape))
            src[(p.name, s.global_rank + n_inf)] = truth[p.name][sl].clone()
    dst, hits = {}, {}
    for e in range(builder.num_infer_engines):
        for p in infer_meta:
            for s in p.shards:
                key = (p.name, s.global_rank + e * builder.infer_instance_world_size)
                dst[key] = torch.full(s.shape, float("nan"))
                hits[key] = torch.zeros(s.shape, dtype=torch.int32)
    for t in range(builder.train_world_size):
        plan = builder.build_local_transfer_plan(infer_meta, train_meta, n_inf + t)
        for peer, ops in plan.operations.items():
            for op in ops:
                assert op.send_rank == n_inf + t and op.recv_rank == peer
                piece = slice_tensor(src[(op.send_shard_meta.name, op.send_rank)], op, True)
                assert tuple(piece.shape) == tuple(op.overlap_shape)
                slice_tensor(dst[(op.recv_shard_meta.name, op.recv_rank)], op, False).copy_(piece)
                slice_tensor(hits[(op.recv_shard_meta.name, op.recv_rank)], op, False).add_(1)
    return dst, hits


def check_exact(builder, infer_meta, train_meta, truth):
    dst, hits = run_plan(builder, infer_meta, train_meta, truth)
    for (name, rank), h in hits.items():
        assert bool((h == 1).all()), f"{name} on rank {rank}: elements written {h.unique().tolist()} times"
    n_inf_inst = builder.infer_instance_world_size
    for p in infer_meta:
        for e in range(builder.num_infer_engines):
            for s in p.shards:
                sl = tuple(slice(o, o + n) for o, n in zip(s.global_offset, s.shape))
                assert torch.equal(dst[(p.name, s.global_rank + e * n_inf_inst)], truth[p.name][sl])


# ------------------------------------------------------------------------------------------ end-to-end on CPU
def test_split_merge_and_uneven_resharding_are_exact():
    truth = {"w": torch.arange(8 * 6, dtype=torch.float32).reshape(8, 6)}
    # 1 -> 2 split
    check_exact(TransferPlanBuilder(2, 1), [param("w", [(4, 6), (4, 6)])], [param("w", [(8, 6)])], truth)
    # 2 -> 1 merge
    check_exact(TransferPlanBuilder(1, 2), [param("w", [(8, 6)])], [param("w", [(4, 6), (4, 6)])], truth)
    # 2 -> 2 uneven: 5/3 rows -> 3/5 rows
    check_exact(TransferPlanBuilder(2, 2), [param("w", [(3, 6), (5, 6)])], [param("w", [(5, 6), (3, 6)])], truth)
    # column sharding on one side, row sharding on the other
    check_exact(TransferPlanBuilder(2, 2), [param("w", [(8, 2), (8, 4)], dim=1)], [param("w", [(4, 6), (4, 6)])], truth)


def test_two_inference_engines_and_training_replicas():
    truth = {"w": torch.randn(8, 4), "b": torch.randn(8)}
    infer = [param("w", [(4, 4), (4, 4)]), param("b", [(4,), (4,)])]
    train = [param("w", [(8, 4)], replicas=2), param("b", [(8,)], replicas=2)]
    builder = TransferPlanBuilder(4, 2, num_infer_engines=2)
    check_exact(builder, infer, train, truth)
    # engine 0 is fed by training replica 0, engine 1 by replica 1
    for t, engine_ranks in ((0, {0, 1}), (1, {2, 3})):
        assert set(builder.build_local_transfer_plan(infer, train, 4 + t).operations) == engine_ranks
    spread = TransferPlanBuilder(4, 2, num_infer_engines=2, replica_pairing="spread")
    check_exact(spread, infer, train, truth)


def test_plans_are_deterministic_and_views_agree():
    infer = [param("w", [(3, 6), (5, 6)]), param("v", [(4,), (4,)])]
    train = [param("w", [(5, 6), (3, 6)]), param("v", [(8,)], replicas=2)]
    builder = TransferPlanBuilder(2, 2)
    first = [builder.build_local_transfer_plan(infer, train, r) for r in range(4)]
    again = [TransferPlanBuilder(2, 2).build_local_transfer_plan(infer, train, r) for r in range(4)]
    assert [compute_transfer_plan_hash(p) for p in first] == [compute_transfer_plan_hash(p) for p in again]
    # what a receiver expects from a sender is what that sender plans to send
    for recv in range(2):
        for send, ops in first[recv].operations.items():
            mirror = first[send].operations[recv]
            sig = lambda op: (op.send_shard_meta.name, op.send_offset, op.recv_offset, op.overlap_shape)  # noqa: E731
            assert [sig(o) for o in ops] == [sig(o) for o in mirror]
    for plan in first:
        for ops in plan.operations.values():
            keys = [(o.send_shard_meta.name, o.send_offset, o.recv_offset) for o in ops]
            assert keys == sorted(keys)


# ------------------------------------------------------------------------------------------ contracts
def test_key_contract():
    infer = [param("model.layers.0.w", [(4, 4)]), param("lm_head.weight", [(4, 4)]), param("model.embed_tokens.weight", [(4, 4)])]
    train = [param("model.layers.0.w", [(4, 4)], first_rank=0), param("model.embed_tokens.weight", [(4, 4)])]
    # inference-only lm_head alias of tied embeddings is tolerated ...
    ops = TransferPlanBuilder(1, 1).build_weights_mapping_operations(infer, train)
    assert {o.recv_shard_meta.name for o in ops} == {"model.layers.0.w", "model.embed_tokens.weight"}
    # ... unless the match is strict
    with pytest.raises(ValueError, match="strict=True"):
        TransferPlanBuilder(1, 1, strict_param_key_match=True).build_weights_mapping_operations(infer, train)
    # an unknown inference-only key or a key the inference side lacks always fails
    with pytest.raises(ValueError, match="unsupported_extra_on_infer"):
        TransferPlanBuilder(1, 1).build_weights_mapping_operations(infer + [param("mystery", [(2,)])], train)
    with pytest.raises(ValueError, match="missing_on_infer"):
        TransferPlanBuilder(1, 1).build_weights_mapping_operations(infer, train + [param("train_only", [(2,)])])
    assert TransferPlanBuilder(1, 1).build_weights_mapping_operations([], train) == []
    with pytest.raises(ValueError):
        TransferPlanBuilder(1, 1, num_infer_engines=0)


def test_shard_offset_errors():
    builder = TransferPlanBuilder(1, 1)
    bad = param("w", [(4, 4)])
    bad.replicas[0].shards[0].global_offset = (0,)  # wrong rank
    with pytest.raises(ValueError, match="Dimension mismatch"):
        builder.build_weights_mapping_operations([bad], [param("w", [(4, 4)])])
    empty = param("w", [(4, 4)])
    empty.replicas[0].shards.clear()
    with pytest.raises(ValueError, match="No shards"):
        builder.build_weights_mapping_operations([empty], [param("w", [(4, 4)])])
    none = param("w", [(4, 4)])
    none.replicas.clear()
    with pytest.raises(ValueError, match="No replicas"):
        builder.build_weights_mapping_operations([none], [param("w", [(4, 4)])])


def test_overlap_offsets_are_relative_to_each_shard():
    infer = [param("w", [(3, 6), (5, 6)])]
    train = [param("w", [(5, 6), (3, 6)])]
    plan = TransferPlanBuilder(2, 2).build_local_transfer_plan(infer, train, 1)  # inference rank 1 holds rows 3..7
    got = {(peer, op.send_offset, op.recv_offset, op.overlap_shape) for peer, ops in plan.operations.items() for op in ops}
    assert got == {(2, (3, 0), (0, 0), (2, 6)), (3, (0, 0), (2, 0), (3, 6))}
    for ops in plan.operations.values():
        for op in ops:
            assert op.train_slices == tuple(slice(o, o + n) for o, n in zip(op.send_offset, op.overlap_shape))
            assert op.inf_slices == tuple(slice(o, o + n) for o, n in zip(op.recv_offset, op.overlap_shape))


def test_plan_container_hash_and_stats():
    infer = [param("w", [(4, 6), (4, 6)], dtype=torch.bfloat16)]
    train = [param("w", [(8, 6)], dtype=torch.bfloat16)]
    plan = TransferPlanBuilder(2, 1).build_local_transfer_plan(infer, train, 2)
    assert plan.operations is plan.inter_operations
    legacy = TransferPlan(inter_operations=plan.operations)
    assert legacy.operations is legacy.inter_operations and len(legacy.all_operations()) == 2
    stats = compute_transfer_plan_stats(plan)
    assert stats["total"] == {"op_count": 2, "numel": 48, "bytes": 96}
    assert stats["full_hash"] == compute_transfer_plan_hash(plan) and len(stats["full_hash"]) == 64
    other = TransferPlanBuilder(2, 1).build_local_transfer_plan([param("w", [(2, 6), (6, 6)], dtype=torch.bfloat16)], train, 2)
    assert compute_transfer_plan_hash(other) != stats["full_hash"]
    assert compute_total_model_size(train) == 96


def test_replica_grouping():
    shards = [shard("w", (2, 4), tp, tp + 2 * dp, n=2) for dp in range(2) for tp in range(2)]
    reps = group_into_replicas("w", shards)
    assert [[s.global_rank for s in r] for r in reps] == [[0, 1], [2, 3]]
    shape, numel = assign_global_layout(reps)
    assert shape == (4, 4) and numel == 16
    assert [s.global_offset for s in reps[1]] == [(0, 0), (2, 0)]
    whole = [shard("n", (4,), 0, r, ShardingType.NO_SHARDING) for r in range(3)]
    assert [len(r) for r in group_into_replicas("n", whole)] == [1, 1, 1]
    with pytest.raises(AssertionError, match="Inconsistent number of replicas"):
        group_into_replicas("w", shards[:3])


def test_to_local_parameter_meta_and_engine_copy():
    p = param("w", [(4, 4), (4, 4)], replicas=2)
    local = p.to_local_parameter_meta(3)
    assert [s.global_rank for s in local.shards] == [3] and len(local.replicas) == 1
    assert p.to_local_parameter_meta(9).shards == []
    copy = p.fast_copy_with_engine_rank(5)
    assert {s.engine_rank for s in copy.shards} == {5} and {s.engine_rank for s in p.shards} == {0}
    assert copy.replicas[0].shards[0] is copy.shards[0]


def test_normalize_rank_axes():
    from types import SimpleNamespace

    ri = SimpleNamespace(pp_rank=1, tp_rank=3, tp_size=4, ep_rank=2, ep_size=4, ep_tp_rank=1, ep_tp_size=2, attn_tp_rank=1, attn_tp_size=2)
    attn = normalize_rank_axes("attention", ri)
    assert (attn.tp_rank, attn.tp_size) == (1, 2) and attn.pp_rank == 1
    dense = normalize_rank_axes("dense_other", ri)
    assert (dense.tp_rank, dense.tp_size) == (3, 4)
    assert not hasattr(attn, "cp_rank")  # context-parallel peers are replicas, not an axis
