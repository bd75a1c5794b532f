"""End-to-end plan -> lowering -> execution on CPU for many layouts.

Modelled on the reference's CPU plan simulation
(`awex/tests/test_transfer_plan_cpu_sim.py:94-168`): every destination element
is written exactly once and the assembled inference tensors equal the ground
truth, here for whole synthetic models instead of single tensors.
"""

import pytest
import torch

from awex_b200.synthetic.arch import get_arch
from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout
from awex_b200.transfer.transfer_plan import compute_transfer_plan_hash, compute_transfer_plan_stats

LAYOUTS = [
    ("tiny-llama", TrainLayout(tp=2), InferLayout(tp=1)),
    ("tiny-llama", TrainLayout(tp=1), InferLayout(tp=1)),
    ("tiny-llama", TrainLayout(tp=2), InferLayout(tp=2, num_engines=2)),
    ("tiny-llama", TrainLayout(tp=1, dp=2), InferLayout(tp=2)),
    ("tiny-llama", TrainLayout(tp=2), InferLayout(tp=2, engine_name="sglang")),
    ("tiny-qwen2", TrainLayout(tp=4), InferLayout(tp=2, num_engines=2)),
    ("tiny-qwen2", TrainLayout(tp=2), InferLayout(tp=8)),  # KV heads replicated on the inference side
    ("tiny-qwen2", TrainLayout(tp=1), InferLayout(tp=8)),
    ("tiny-qwen2", TrainLayout(tp=2, pp=2), InferLayout(tp=4)),
    ("tiny-qwen2", TrainLayout(tp=4), InferLayout(tp=4)),
    ("tiny-qwen3-moe", TrainLayout(tp=1, dp=4, ep=4), InferLayout(tp=2, ep=2, num_engines=2)),
    ("tiny-qwen3-moe", TrainLayout(tp=2, dp=2, ep=4), InferLayout(tp=4)),
    ("tiny-qwen3-moe", TrainLayout(tp=1, dp=2, ep=2), InferLayout(tp=2, ep=2, engine_name="sglang")),
    ("tiny-qwen3-moe", TrainLayout(tp=2, dp=2, ep=4), InferLayout(tp=8)),  # split Q/K/V with replicated KV heads
    ("tiny-qwen3-moe", TrainLayout(tp=1, dp=8, ep=8), InferLayout(tp=8)),
    # SGLang DP attention: attention / embeddings cut over attention TP and replicated over attention-DP groups
    ("tiny-qwen2", TrainLayout(tp=2), InferLayout(tp=4, attn_tp=2, engine_name="sglang")),
    ("tiny-qwen2", TrainLayout(tp=4), InferLayout(tp=4, attn_tp=1, engine_name="sglang", dp_lm_head=True)),
    ("tiny-qwen3-moe", TrainLayout(tp=1, dp=2, ep=2), InferLayout(tp=4, ep=4, attn_tp=2, engine_name="sglang")),
    ("tiny-llama", TrainLayout(tp=2, pp=2), InferLayout(tp=2, attn_tp=1, engine_name="sglang", num_engines=2)),
    ("tiny-llama", TrainLayout(tp=2), InferLayout(tp=1, pp=2)),  # pipeline-parallel inference
    ("tiny-qwen2", TrainLayout(tp=2, pp=2), InferLayout(tp=2, pp=2)),
    ("tiny-qwen3-moe", TrainLayout(tp=1, dp=2, ep=2), InferLayout(tp=2, pp=2, num_engines=2)),
]


@pytest.mark.parametrize("arch,train,infer", LAYOUTS, ids=lambda v: v if isinstance(v, str) else v.label())
def test_exchange_is_exact_and_exactly_once(arch, train, infer):
    job = SimulatedJob(get_arch(arch), train, infer, dtype=torch.float32)
    job.compile_all()
    assert job.check_coverage() == []
    assert job.run_cpu() > 0
    assert job.mismatches() == []


def test_golden_numbers_tiny_llama_tp2_to_tp1():
    """Plan of the tiny Llama TP2 -> TP1 exchange: 29 receive operations,
    1 705 216 elements, 6 820 864 bytes in fp32; the same numbers the reference
    planner produces for this model."""
    job = SimulatedJob(get_arch("tiny-llama"), TrainLayout(tp=2), InferLayout(tp=1))
    reader_plan = job.builder.build_local_transfer_plan(job.infer_meta, job.train_meta, 0)
    stats = compute_transfer_plan_stats(reader_plan)
    assert stats["total"] == {"op_count": 29, "numel": 1705216, "bytes": 6820864}
    w1 = job.builder.build_local_transfer_plan(job.infer_meta, job.train_meta, 1)
    w2 = job.builder.build_local_transfer_plan(job.infer_meta, job.train_meta, 2)
    assert [compute_transfer_plan_stats(p)["total"]["op_count"] for p in (w1, w2)] == [17, 12]
    assert [compute_transfer_plan_stats(p)["total"]["numel"] for p in (w1, w2)] == [853248, 851968]
    # determinism: a second build gives the same fingerprint
    again = job.builder.build_local_transfer_plan(job.infer_meta, job.train_meta, 0)
    assert compute_transfer_plan_hash(again) == stats["full_hash"]


def test_no_training_rank_gathers_qkv():
    """With training TP > 1 the regrouped QKV of one rank contains rows of its
    peers; lowering re-homes them so every item reads a local tensor only."""
    job = SimulatedJob(get_arch("tiny-qwen2"), TrainLayout(tp=4), InferLayout(tp=2))
    programs = job.compile_all()
    for rank, items in programs.items():
        local = {n for n, _ in job.train_models[rank].named_parameters()}
        assert all(it.src_param in local for it in items)
        qkv = [it for it in items if "query_key_value" in it.dst_name]
        assert qkv, "every rank owns some QKV rows"


def test_bf16_exchange_bitwise():
    job = SimulatedJob(get_arch("tiny-qwen3-moe"), TrainLayout(tp=1, dp=2, ep=2), InferLayout(tp=2, ep=2), dtype=torch.bfloat16)
    job.compile_all()
    job.run_cpu()
    assert job.mismatches() == []


@pytest.mark.parametrize("arch,train,infer", [
    ("tiny-qwen3-moe", TrainLayout(tp=1, dp=2, ep=2), InferLayout(tp=1, fp8=True)),
    ("tiny-llama", TrainLayout(tp=1), InferLayout(tp=2, fp8=True)),
], ids=lambda v: v if isinstance(v, str) else v.label())
def test_fp8_serving_exchange(arch, train, infer):
    """bf16 training shards -> block-scaled fp8 inference shards: weights and
    scales equal quantising the destination-layout shards directly."""
    job = SimulatedJob(get_arch(arch), train, infer, dtype=torch.bfloat16)
    job.compile_all()
    assert job.check_coverage() == []
    job.run_cpu()
    assert job.mismatches() == []
    assert any(it.src_rows for items in job.programs.values() for it in items) == (arch == "tiny-qwen3-moe")


@pytest.mark.parametrize("train_tp,infer_tp,gathers", [(2, 1, True), (4, 2, True), (4, 1, True), (2, 2, False), (2, 4, False)])
def test_fp8_blocks_that_span_training_ranks_are_gathered_by_their_owner(train_tp, infer_tp, gathers):
    """Fused QKV regrouped for fewer inference ranks than training ranks: a
    quantisation block then mixes rows of several training ranks.  The rank that
    owns the chunk gathers its rows over the training TP group into a buffer and
    quantises from there (the reference gathers every fused QKV, always:
    `awex/converter/mcore_converter.py:1040-1052`); where every block has one
    owner, no gather is planned and each rank sends its own rows."""
    import dataclasses

    arch = dataclasses.replace(get_arch("tiny-qwen2"), head_dim=64, name="tiny-qwen2-hd64")
    job = SimulatedJob(arch, TrainLayout(tp=train_tp), InferLayout(tp=infer_tp, fp8=True), dtype=torch.bfloat16)
    programs = job.compile_all()
    assert job.check_coverage() == []
    qkv = [f"model.layers.{l}.attention.query_key_value_proj.weight" for l in range(arch.num_layers)]
    for rank, items in programs.items():
        derived = sorted(d.key[0] for d in job.derived[rank])
        assert derived == (sorted("__derived__/" + n for n in qkv) if gathers else [])
        assert all(d.gathers for d in job.derived[rank])
        for it in items:
            if it.dst_name in qkv:
                assert it.src_param.startswith("__derived__/") == gathers and it.value_op.kind == "fp8_block"
    job.run_cpu()
    assert job.mismatches() == []


def test_spread_replica_pairing_balances_data_parallel_senders():
    """Dense parameters replicated over four data-parallel training ranks: the
    reference's round-robin lets the first replicas send all of them, the
    least-loaded pairing spreads them; both tile every destination exactly once
    and give bit-identical weights."""
    from awex_b200.transfer.transfer_plan import TransferPlanBuilder

    job = SimulatedJob(get_arch("tiny-qwen3-moe"), TrainLayout(tp=1, dp=4, ep=4), InferLayout(tp=2, ep=2, num_engines=2), dtype=torch.float32)
    spans = {}
    for mode in ("round_robin", "spread"):
        job.builder = TransferPlanBuilder(job.infer_world_size, job.train.world, job.infer.num_engines, replica_pairing=mode)
        programs = job.compile_all()
        assert job.check_coverage() == []
        for models in job.infer_models:
            for m in models:
                for p in m.parameters():
                    p.zero_()
        job.run_cpu()
        assert job.mismatches() == []
        sent = [sum(it.dst_bytes for it in items) for items in programs.values()]
        spans[mode] = max(sent) / min(sent)
    assert spans["round_robin"] > 1.5 and spans["spread"] < 1.05
    with pytest.raises(ValueError):
        TransferPlanBuilder(2, 2, 1, replica_pairing="nearest")


def test_exactly_once_check_finds_gaps_overlaps_and_strays():
    from awex_b200.transfer.lowering import _cover_problems_pairwise, check_exactly_once

    views = {"w": ((8, 6), torch.float32), "s": ((), torch.float32), "w_scale_inv": ((1, 1), torch.float32)}
    entry = lambda name, start, extent, dtype="torch.float32": (name, start, extent, dtype, None, None)  # noqa: E731
    good = [[entry("w", (0, 0), (4, 6)), entry("s", (), ())], [entry("w", (4, 0), (4, 3)), entry("w", (4, 3), (4, 3))]]
    assert check_exactly_once(good, views, ["w", "s"]) == []
    gap = [[entry("w", (0, 0), (4, 6))], [entry("w", (4, 0), (4, 3))]]
    assert any("12 of 48 elements are never written" in p for p in check_exactly_once(gap, views, ["w"]))
    twice = [good[0], good[1] + [entry("w", (3, 2), (2, 2))]]
    assert any("overlaps" in p for p in check_exactly_once(twice, views, ["w"]))
    stray = [[entry("w", (6, 0), (4, 6))]]
    assert any("exceeds" in p for p in check_exactly_once(stray, views, ["w"]))
    assert any("unknown view" in p for p in check_exactly_once([[entry("x", (0,), (1,))]], views, []))
    assert any("dtype" in p for p in check_exactly_once([[entry("w", (0, 0), (8, 6), "torch.bfloat16")]], views, ["w"]))
    assert any("receives nothing" in p for p in check_exactly_once([[entry("s", (), ())]], views, ["w", "s"]))
    with_scale = [[("w", (0, 0), (8, 6), "torch.float32", "w_scale_inv", (0, 0))]]
    assert check_exactly_once(with_scale, views, ["w", "w_scale_inv"]) == []
    # the pairwise fallback agrees
    boxes = [((0, 0), (4, 6), "a"), ((4, 0), (4, 3), "b"), ((4, 3), (4, 3), "c")]
    assert _cover_problems_pairwise("w", (8, 6), boxes) == []
    assert any("overlaps" in p for p in _cover_problems_pairwise("w", (8, 6), boxes + [((3, 2), (2, 2), "d")]))
    assert any("never written" in p for p in _cover_problems_pairwise("w", (8, 6), boxes[:2]))


@pytest.mark.parametrize("arch,train,infer", [
    ("tiny-qwen2", TrainLayout(tp=4, dp=2), InferLayout(tp=2, num_engines=2)),
    ("tiny-qwen2", TrainLayout(tp=4, dp=2), InferLayout(tp=2)),
    ("tiny-llama", TrainLayout(tp=2, dp=3), InferLayout(tp=1, num_engines=2)),
    ("tiny-qwen3-moe", TrainLayout(tp=2, dp=4, ep=4), InferLayout(tp=2, ep=2, num_engines=2)),
], ids=lambda v: v if isinstance(v, str) else v.label())
def test_spread_pairing_agrees_between_a_rank_and_the_plans_it_makes_for_its_peers(arch, train, infer):
    """Rows that a TP peer owns are sent by that peer, which plans them with
    per-parameter calls after its own plan: those calls must choose the same
    training replica as the full pass did."""
    from awex_b200.transfer.transfer_plan import TransferPlanBuilder

    job = SimulatedJob(get_arch(arch), train, infer, dtype=torch.float32)
    builder = TransferPlanBuilder(job.infer_world_size, job.train.world, job.infer.num_engines, replica_pairing="spread")
    job.builder = builder
    seen, clashes = {}, []
    pick = builder._pick_train_replica

    def spy(i, meta):
        k = pick(i, meta)
        if seen.setdefault((meta.name, i), k) != k:
            clashes.append((meta.name, i, seen[(meta.name, i)], k))
        return k

    builder._pick_train_replica = spy
    job.compile_all()
    assert clashes == []
    assert job.check_coverage() == []
    job.run_cpu()
    assert job.mismatches() == []


def test_tied_lm_head_is_an_alias_that_nobody_sends():
    """With tied embeddings the inference worker answers for ``lm_head.weight``
    through the embedding tensor: one memory, two names.  The alias is
    published, the planner leaves it out, and the embedding is written once."""
    import dataclasses

    arch = dataclasses.replace(get_arch("tiny-llama"), tie_embeddings=True)
    job = SimulatedJob(arch, TrainLayout(tp=2, pp=2), InferLayout(tp=2), dtype=torch.float32)
    assert job.aliases == {"lm_head.weight": "model.embed_tokens.weight"}
    assert job.infer_conf["aliased_parameters"] == job.aliases
    programs = job.compile_all()
    assert not any(it.dst_name == "lm_head.weight" for items in programs.values() for it in items)
    assert any(it.dst_name == "model.embed_tokens.weight" for items in programs.values() for it in items)
    assert job.check_coverage() == []
    job.encode_all(validate=True)  # includes the no-two-descriptors-overlap rule
    job.run_cpu()
    assert job.mismatches() == []
    untied = SimulatedJob(get_arch("tiny-llama"), TrainLayout(tp=2), InferLayout(tp=2), dtype=torch.float32)
    assert untied.aliases == {} and any(it.dst_name == "lm_head.weight" for items in untied.compile_all().values() for it in items)


def test_fp8_slices_that_end_inside_a_block_are_refused_with_a_reason():
    """Two training TP ranks feed one inference shard and each holds half of a
    128-row quantisation block: no rank can compute that block's scale."""
    import dataclasses

    arch = dataclasses.replace(get_arch("tiny-qwen3-moe"), num_heads=4, num_kv_heads=4, head_dim=128, hidden=512, num_layers=1,
                               vocab=512, num_experts=4, expert_ffn=128)
    with pytest.raises(NotImplementedError, match="not a whole number of 128-wide quantisation blocks"):
        SimulatedJob(arch, TrainLayout(tp=2), InferLayout(tp=1, fp8=True), dtype=torch.bfloat16)
    aligned = dataclasses.replace(arch, expert_ffn=256)
    job = SimulatedJob(aligned, TrainLayout(tp=2), InferLayout(tp=1, fp8=True), dtype=torch.bfloat16)
    job.compile_all()
    assert job.check_coverage() == []
    job.run_cpu()
    assert job.mismatches() == []


@pytest.mark.parametrize("train_tp,infer_tp", [(1, 2), (2, 1), (2, 4)])
def test_column_normalised_head_is_derived_on_the_sender(train_tp, infer_tp):
    """``norm_head``: the head is published with unit-norm columns, each training
    rank normalising the vocabulary slice it holds (`awex/converter/mcore_converter.py:668-675`
    in the reference).  The reduction needs the whole local tensor, so the sender keeps the
    result in a buffer of its own and sends it with plain copies; a second update
    after the parameters changed must send the new values from the same buffer."""
    import dataclasses

    from awex_b200.synthetic.models import CanonicalWeights

    arch = dataclasses.replace(get_arch("tiny-llama"), norm_head=True, name="tiny-llama-norm-head")
    job = SimulatedJob(arch, TrainLayout(tp=train_tp), InferLayout(tp=infer_tp), dtype=torch.float32)
    programs = job.compile_all()
    assert not job.check_coverage()
    for rank, items in programs.items():
        head = [it for it in items if it.dst_name == "lm_head.weight"]
        assert head and all(it.src_param == "__derived__/lm_head.weight" and it.value_op.kind == "none" for it in head)
        assert [d.key[0] for d in job.derived[rank]] == ["__derived__/lm_head.weight"]

    def expected_shards(scale: float):
        full = CanonicalWeights(arch, torch.float32, "cpu").get("lm_head.weight", (arch.vocab, arch.hidden)) * scale
        normed = torch.cat([torch.nn.functional.normalize(c, dim=0, p=2, eps=1e-7) for c in full.chunk(train_tp, 0)], 0)
        return list(normed.chunk(infer_tp, 0))

    def received():
        return [dict(m.named_parameters())["lm_head.weight"] for m in job.infer_models[0]]

    job.run_cpu()
    assert {m.rsplit("/", 1)[1] for m in job.mismatches()} == {"lm_head.weight"}  # only the head differs from the raw weights
    for got, want in zip(received(), expected_shards(1.0)):
        assert torch.equal(got, want)
    buffers = {r: job.local_tensors(r)[("__derived__/lm_head.weight", 0)].data_ptr() for r in programs}
    # an "optimizer step": rows scaled unevenly, so that the normalised columns change
    ramp = torch.linspace(0.5, 2.0, arch.vocab).unsqueeze(1)
    for r, model in enumerate(job.train_models):
        w = dict(model.named_parameters())["output_layer.weight"]
        n = w.shape[0]
        with torch.no_grad():
            w.mul_(ramp[r * n : (r + 1) * n])
    job.run_cpu()
    full = CanonicalWeights(arch, torch.float32, "cpu").get("lm_head.weight", (arch.vocab, arch.hidden)) * ramp
    normed = torch.cat([torch.nn.functional.normalize(c, dim=0, p=2, eps=1e-7) for c in full.chunk(train_tp, 0)], 0)
    for got, want in zip(received(), normed.chunk(infer_tp, 0)):
        assert torch.equal(got, want)
    assert buffers == {r: job.local_tensors(r)[("__derived__/lm_head.weight", 0)].data_ptr() for r in programs}


def test_block_aligned_head_runs_become_plain_fp8_slabs():
    """De-interleaving Q / K / V for fp8 serving gathers rows of the fused Megatron
    tensor; when every head run is a whole number of quantisation blocks (head size
    128) each run is lowered to a plain slab (fetched with tiled loads by the
    kernel) instead of a row-gather list, and the result is the same."""
    import dataclasses

    from awex_b200.transfer.table_interpreter import HostMemory, run_table

    base = get_arch("tiny-qwen3-moe")
    for head_dim, gathered in ((128, False), (32, True)):
        arch = dataclasses.replace(base, head_dim=head_dim, name=f"tiny-qwen3-moe-hd{head_dim}")
        job = SimulatedJob(arch, TrainLayout(tp=1, dp=2, ep=2), InferLayout(tp=1, fp8=True), dtype=torch.bfloat16)
        programs = job.compile_all()
        assert job.check_coverage() == []
        qkv = [it for items in programs.values() for it in items if ".self_attn." in it.dst_name and it.dst_name.endswith("_proj.weight")
               and "o_proj" not in it.dst_name]
        assert qkv and all(it.value_op.kind == "fp8_block" for it in qkv)
        assert any(it.src_rows for it in qkv) == gathered
        if not gathered:  # one item per head run, each a whole number of blocks
            assert all(it.extent[0] % 128 == 0 and it.dst_start[0] % 128 == 0 for it in qkv)
        encoded = job.encode_all(validate=True)
        mem = HostMemory(job.source_tensors() + [p for ms in job.infer_models for m in ms for p in m.parameters()])
        for table, n_tiles, enc in encoded.values():
            assert run_table(table, n_tiles, mem, enc.row_offsets) == n_tiles
            if not gathered:
                assert len(enc.row_offsets) == 0 and len(enc.tensor_map_descs) > 0  # no gathered rows left; tiled loads everywhere
        assert job.mismatches() == []


def test_local_replica_pairing_keeps_replicated_tensors_on_their_gpu():
    """A TP1 / DP4 / EP4 trainer holds attention, norms and embeddings on every
    rank.  With ``replica_pairing="local"`` and the map of which inference worker
    shares a GPU with which training rank, every inference shard of those tensors
    is written by the training rank on its own GPU; experts still come from
    whoever holds them; the update stays exact and exactly-once."""
    from awex_b200.transfer.transfer_plan import TransferPlanBuilder

    arch = get_arch("tiny-qwen3-moe")
    train, infer = TrainLayout(tp=1, dp=4, ep=4), InferLayout(tp=2, ep=2, num_engines=2)
    colocation = {0: 0, 1: 2, 2: 1, 3: 3}  # worker j of instance 0 on GPU 2j, of instance 1 on GPU 2j+1

    def remote_dense_bytes(pairing, **kw):
        job = SimulatedJob(arch, train, infer, dtype=torch.float32)
        job.builder = TransferPlanBuilder(job.infer_world_size, train.world, infer.num_engines, replica_pairing=pairing,
                                          skip_names=job.builder.skip_names, **kw)
        programs = job.compile_all()
        assert job.check_coverage() == []
        job.run_cpu()
        assert job.mismatches() == []
        dense = [(r, it) for r, items in programs.items() for it in items if ".experts." not in it.dst_name]
        return sum(it.dst_bytes for r, it in dense if colocation[it.dst_rank] != r), sum(it.dst_bytes for _r, it in dense)

    spread_remote, total = remote_dense_bytes("spread")
    local_remote, same_total = remote_dense_bytes("local", colocation=colocation)
    assert same_total == total and spread_remote > 0.5 * total  # least-loaded pairing ignores where things sit
    assert local_remote == 0                                    # every dense shard comes from its own GPU
    with pytest.raises(ValueError):
        TransferPlanBuilder(4, 4, 2, replica_pairing="nearest")
