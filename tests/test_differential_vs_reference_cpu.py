"""Differential tests against the reference package itself (an unmodified copy
under ``baseline/_ref``, with the Megatron stub of ``baseline/stubs`` on the
path): the same inputs through both implementations, results compared with zero
tolerance.  Skipped where the reference copy is not present.

Covered: block-fp8 quantisation, the transfer planner on the benchmark layouts
(same metadata into both planners, operation by operation), and the training-
and serving-side converters of every architecture family on tiny tensors.
Reference counterparts: `awex/tests/test_transfer_plan_cpu_sim.py:94-168`,
`awex/converter/weights_converter.py:42-61`, `awex/models/*.py`."""

import dataclasses
import os
import sys
from types import SimpleNamespace

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
STUBS = os.path.join(ROOT, "baseline", "stubs")

if not os.path.isdir(os.path.join(REF, "awex", "transfer")):
    pytest.skip("no copy of the reference package under baseline/_ref", allow_module_level=True)


@pytest.fixture(scope="module", autouse=True)
def reference_on_the_path():
    """The reference package and the stand-in for Megatron are importable while
    this module's tests run, and only then: processes that later tests spawn
    inherit ``sys.path``, and a ``megatron`` that imports changes what the
    training-side converter takes for its tensor-parallel group."""
    added = [path for path in (STUBS, REF) if path not in sys.path]
    for path in added:
        sys.path.insert(0, path)
    import awex.logging as ref_logging

    ref_logging.setLevel("ERROR")
    yield
    for path in added:
        sys.path.remove(path)
    for name in [n for n in sys.modules if n == "awex" or n.startswith("awex.") or n == "megatron" or n.startswith("megatron.")]:
        del sys.modules[name]


# ---- block fp8 --------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(256, 384), (130, 136), (1, 128), (300, 72)])
@pytest.mark.parametrize("ue8m0", [False, True])
def test_block_fp8_matches_the_reference_function(shape, ue8m0):
    from awex.converter.weights_converter import per_block_cast_to_fp8 as ref_cast

    from awex_b200.converter.weights_converter import per_block_cast_to_fp8 as our_cast

    g = torch.Generator().manual_seed(5)
    x = (torch.randn(shape, generator=g) * 0.05).to(torch.bfloat16)
    x[0, 0] = 3.0
    q_ref, s_ref = ref_cast(x, ue8m0)
    q, s = our_cast(x, ue8m0)
    assert torch.equal(s.reshape(-1), s_ref.float().reshape(-1))
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))


# ---- the planner ------------------------------------------------------------------------------------
def _to_reference(obj, ref_module):
    """Our metadata dataclasses as the reference's, field by field."""
    if isinstance(obj, list):
        return [_to_reference(o, ref_module) for o in obj]
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        ref_cls = getattr(ref_module, type(obj).__name__)
        names = {f.name for f in dataclasses.fields(ref_cls)}
        values = {}
        for f in dataclasses.fields(obj):
            if f.name not in names:
                continue
            v = getattr(obj, f.name)
            if f.name == "sharding_type":
                from awex.sharding.param_sharding import ShardingType as RefShardingType

                v = RefShardingType[v.name]
            values[f.name] = _to_reference(v, ref_module)
        return ref_cls(**values)
    return obj


def _ops_key(plan):
    out = []
    for peer, ops in sorted(plan.operations.items()):
        for op in ops:
            out.append((peer, op.send_rank, op.recv_rank, op.send_shard_meta.name, tuple(op.send_offset), tuple(op.recv_offset),
                        tuple(op.overlap_shape), tuple((s.start, s.stop) for s in op.train_slices),
                        tuple((s.start, s.stop) for s in op.inf_slices)))
    return sorted(out)


LAYOUTS = [
    # the benchmark configurations on tiny models of the same kind: TP2 -> TP1, TP4 -> 2 x TP2, TP2 -> TP2, EP -> 2 x (TP, EP)
    ("tiny-llama", dict(tp=2), dict(tp=1)),
    ("tiny-qwen2", dict(tp=4), dict(tp=2, num_engines=2)),
    ("tiny-qwen2", dict(tp=2), dict(tp=2)),
    ("tiny-qwen3-moe", dict(tp=1, dp=4, ep=4), dict(tp=2, ep=2, num_engines=2)),
    ("tiny-llama", dict(tp=2, pp=2), dict(tp=4)),
]


@pytest.mark.parametrize("arch,train,infer", LAYOUTS)
def test_planner_agrees_with_the_reference_operation_by_operation(arch, train, infer):
    import awex.meta.weight_meta as ref_meta
    from awex.transfer.transfer_plan import TransferPlanBuilder as RefBuilder

    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout
    from awex_b200.transfer.transfer_plan import TransferPlanBuilder

    job = SimulatedJob(get_arch(arch), TrainLayout(**train), InferLayout(**infer), dtype=torch.float32, device="meta")
    infer_world = len(job.infer_ranks) * len(job.infer_ranks[0])
    train_world = len(job.train_ranks)
    ours = TransferPlanBuilder(infer_world, train_world, len(job.infer_ranks), replica_pairing="round_robin",
                               skip_names=job.aliases)
    ref_infer, ref_train = _to_reference(job.infer_meta, ref_meta), _to_reference(job.train_meta, ref_meta)
    if job.aliases:  # second names of one memory are left out of our plan; give the reference the same parameter list
        ref_infer = [m for m in ref_infer if m.name not in job.aliases]
        ref_train = [m for m in ref_train if m.name not in job.aliases]
    theirs = RefBuilder(infer_world, train_world, len(job.infer_ranks), False)
    total = 0
    from awex.transfer.transfer_plan import compute_transfer_plan_hash as ref_hash, compute_transfer_plan_stats as ref_stats

    from awex_b200.transfer.transfer_plan import compute_transfer_plan_hash, compute_transfer_plan_stats

    for rank in range(infer_world + train_world):
        our_plan = ours.build_local_transfer_plan(job.infer_meta, job.train_meta, rank)
        ref_plan = theirs.build_local_transfer_plan(ref_infer, ref_train, rank)
        mine, want = _ops_key(our_plan), _ops_key(ref_plan)
        assert mine == want, f"transfer rank {rank}"
        # the digest both sides log to compare their plans, and the per-peer statistics
        assert compute_transfer_plan_hash(our_plan) == ref_hash(ref_plan), f"plan hash of transfer rank {rank}"
        assert compute_transfer_plan_stats(our_plan) == ref_stats(ref_plan), f"plan statistics of transfer rank {rank}"
        total += len(mine)
    assert total > 0


# ---- converters ---------------------------------------------------------------------------------------
def _rank(module, tp_rank=0, tp_size=1, **kw):
    base = dict(tp_rank=tp_rank, tp_size=tp_size, pp_rank=0, pp_size=1, dp_size=1, dp_rank=0, ep_rank=0, ep_size=1, ep_tp_rank=0,
                ep_tp_size=1, attn_tp_rank=tp_rank, attn_tp_size=tp_size, attn_dp_rank=0, world_size=tp_size, global_rank=tp_rank,
                local_rank=tp_rank, engine_rank=0, is_infer=False)
    base.update(kw)
    return module.RankInfo(**base)


def _both_train_converters(arch, hf, tf, conf, **rank_kw):
    import awex.models.registry as ref_registry
    import awex.sharding.rank_info as ref_rank

    import awex_b200.models.registry as our_registry
    import awex_b200.sharding.rank_info as our_rank

    return (our_registry.get_train_weights_converter("mcore", arch, hf, _rank(our_rank, **rank_kw), dict(conf), tf_config=tf),
            ref_registry.get_train_weights_converter("mcore", arch, hf, _rank(ref_rank, **rank_kw), dict(conf), tf_config=tf))


def _same(ours, theirs, name, tensor):
    got = [(n, t) for n, t in ours.convert_param(name, tensor.clone())]
    want = [(n, t) for n, t in theirs.convert_param(name, tensor.clone())]
    assert [n for n, _ in got] == [n for n, _ in want], name
    for (n, a), (_, b) in zip(got, want):
        assert a.shape == b.shape and a.dtype == b.dtype, n
        assert torch.equal(a.contiguous(), b.contiguous()), n


def _seq(*shape):
    n = 1
    for s in shape:
        n *= s
    return torch.arange(n, dtype=torch.float32).reshape(shape) / 8.0


P = "module.module.decoder.layers.1."


@pytest.mark.parametrize("train_tp,infer_tp", [(1, 1), (2, 1), (2, 4), (1, 2)])
@pytest.mark.parametrize("arch,bias", [("LlamaForCausalLM", False), ("Qwen2ForCausalLM", True)])
def test_dense_decoder_converters_agree(arch, bias, train_tp, infer_tp):
    heads, kv, hd, hidden, ffn = 8, 4, 4, 16, 24
    hf = SimpleNamespace(architectures=[arch], hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=kv, head_dim=hd,
                         num_hidden_layers=2, intermediate_size=ffn, vocab_size=32, tie_word_embeddings=False)
    tf = SimpleNamespace(hidden_size=hidden, num_attention_heads=heads, num_query_groups=kv, kv_channels=hd, num_layers=2,
                         add_qkv_bias=bias)
    conf = {"infer_atten_tp_size": infer_tp, "infer_engine_config": SimpleNamespace(tp_size=infer_tp, ep_size=1)}
    qkv_rows = (heads + 2 * kv) * hd // train_tp
    for tp_rank in range(train_tp):
        ours, theirs = _both_train_converters(arch, hf, tf, conf, tp_rank=tp_rank, tp_size=train_tp)
        cases = {
            "module.module.embedding.word_embeddings.weight": _seq(32 // train_tp, hidden),
            P + "self_attention.linear_qkv.weight": _seq(qkv_rows, hidden),
            P + "self_attention.linear_qkv.layer_norm_weight": _seq(hidden),
            P + "self_attention.linear_proj.weight": _seq(hidden, heads * hd // train_tp),
            P + "mlp.linear_fc1.weight": _seq(2 * ffn // train_tp, hidden),
            P + "mlp.linear_fc1.layer_norm_weight": _seq(hidden),
            P + "mlp.linear_fc2.weight": _seq(hidden, ffn // train_tp),
            "module.module.decoder.final_layernorm.weight": _seq(hidden),
            "module.module.output_layer.weight": _seq(32 // train_tp, hidden),
        }
        if bias:
            cases[P + "self_attention.linear_qkv.bias"] = _seq(qkv_rows)
        for name, tensor in cases.items():
            if train_tp > 1 and "linear_qkv" in name and "layer_norm" not in name:
                # a fused QKV that is regrouped for another TP size needs the peers' shards (a collective in the reference;
                # compared through the single-rank layouts and the planner test instead)
                continue
            _same(ours, theirs, name, tensor)


def test_qwen3_moe_converters_agree_on_attention_experts_and_router():
    heads, kv, hd, hidden, experts, effn = 4, 2, 4, 16, 4, 8
    hf = SimpleNamespace(architectures=["Qwen3MoeForCausalLM"], hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=kv,
                         head_dim=hd, num_hidden_layers=2, num_experts=experts, moe_intermediate_size=effn, vocab_size=32,
                         tie_word_embeddings=False)
    tf = SimpleNamespace(hidden_size=hidden, num_attention_heads=heads, num_query_groups=kv, kv_channels=hd, num_layers=2,
                         num_moe_experts=experts)
    conf = {"infer_atten_tp_size": 1, "infer_engine_config": SimpleNamespace(tp_size=1, ep_size=1)}
    for ep_rank, ep_size in ((0, 1), (1, 2)):
        ours, theirs = _both_train_converters("Qwen3MoeForCausalLM", hf, tf, conf, ep_rank=ep_rank, ep_size=ep_size)
        local = experts // ep_size
        cases = {
            P + "self_attention.linear_qkv.weight": _seq((heads + 2 * kv) * hd, hidden),
            P + "self_attention.q_layernorm.weight": _seq(hd),
            P + "self_attention.k_layernorm.weight": _seq(hd),
            P + "self_attention.linear_proj.weight": _seq(hidden, heads * hd),
            P + "mlp.router.weight": _seq(experts, hidden),
            P + "pre_mlp_layernorm.weight": _seq(hidden),
        }
        for e in range(local):
            cases[P + f"mlp.experts.linear_fc1.weight{e}"] = _seq(2 * effn, hidden) + e
            cases[P + f"mlp.experts.linear_fc2.weight{e}"] = _seq(hidden, effn) + e
        for name, tensor in cases.items():
            _same(ours, theirs, name, tensor)


def test_serving_side_converter_of_a_registered_family_agrees():
    """What an SGLang engine holds for Qwen3-MoE (fused QKV, fused expert stacks),
    under the names both sides publish, whole and on an expert-parallel rank.
    (Architectures the reference does not register get the name-normalising
    converter on every engine here, a stated difference, so a registered family is
    what can be compared.)"""
    import awex.models.registry as ref_registry
    import awex.sharding.rank_info as ref_rank

    import awex_b200.models.registry as our_registry
    import awex_b200.sharding.rank_info as our_rank

    hidden, heads, kv, hd, experts, effn = 16, 4, 2, 4, 4, 8
    hf = SimpleNamespace(architectures=["Qwen3MoeForCausalLM"], hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=kv,
                         head_dim=hd, num_experts=experts, moe_intermediate_size=effn, num_hidden_layers=1, tie_word_embeddings=False)
    for ep_rank, ep in ((0, 1), (1, 2)):
        cfg = SimpleNamespace(tp_size=1, ep_size=ep, device_backend="cuda")
        kw = dict(ep_rank=ep_rank, ep_size=ep, is_infer=True)
        ours = our_registry.get_infer_weights_converter("sglang", "Qwen3MoeForCausalLM", hf, _rank(our_rank, **kw), cfg)
        theirs = ref_registry.get_infer_weights_converter("sglang", "Qwen3MoeForCausalLM", hf, _rank(ref_rank, **kw), cfg)
        local = experts // ep
        cases = {
            "model.embed_tokens.weight": _seq(32, hidden),
            "model.layers.0.self_attn.qkv_proj.weight": _seq((heads + 2 * kv) * hd, hidden),
            "model.layers.0.self_attn.o_proj.weight": _seq(hidden, heads * hd),
            "model.layers.0.self_attn.q_norm.weight": _seq(hd),
            "model.layers.0.self_attn.k_norm.weight": _seq(hd),
            "model.layers.0.input_layernorm.weight": _seq(hidden),
            "model.layers.0.post_attention_layernorm.weight": _seq(hidden),
            "model.layers.0.mlp.gate.weight": _seq(experts, hidden),
            "model.layers.0.mlp.experts.w13_weight": _seq(local, 2 * effn, hidden),
            "model.layers.0.mlp.experts.w2_weight": _seq(local, hidden, effn),
            "model.norm.weight": _seq(hidden),
            "lm_head.weight": _seq(32, hidden),
        }
        for name, tensor in cases.items():
            _same(ours, theirs, name, tensor)


# ---- multimodal, hybrid and MLA families ----------------------------------------------------------------
M = "module.module."


def _both_infer_converters(arch, hf, cfg=None, **rank_kw):
    import awex.models.registry as ref_registry
    import awex.sharding.rank_info as ref_rank

    import awex_b200.models.registry as our_registry
    import awex_b200.sharding.rank_info as our_rank

    cfg = cfg or SimpleNamespace(tp_size=1, ep_size=1, device_backend="cpu")
    rank_kw = dict(is_infer=True, **rank_kw)
    return (our_registry.get_infer_weights_converter("sglang", arch, hf, _rank(our_rank, **rank_kw), cfg),
            ref_registry.get_infer_weights_converter("sglang", arch, hf, _rank(ref_rank, **rank_kw), cfg))


@pytest.mark.parametrize("arch", ["Qwen3VLForConditionalGeneration", "Qwen3VLMoeForConditionalGeneration"])
def test_qwen3_vl_converters_agree_on_decoder_tower_and_experts(arch):
    text = SimpleNamespace(hidden_size=8, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=2,
                           num_experts=4, tie_word_embeddings=False)
    hf = SimpleNamespace(architectures=[arch], text_config=text, vision_config=SimpleNamespace(num_heads=2, hidden_size=4))
    tf = SimpleNamespace(hidden_size=8, num_attention_heads=4, num_query_groups=2, kv_channels=2, num_layers=2)
    for infer_tp in (1, 2):
        conf = {"infer_atten_tp_size": infer_tp, "router_dtype": "fp32", "infer_engine_config": SimpleNamespace(tp_size=infer_tp, ep_size=1)}
        ours, theirs = _both_train_converters(arch, hf, tf, conf)
        cases = {
            M + "language_model.decoder.layers.0.self_attention.linear_qkv.weight": _seq(16, 8),
            M + "language_model.decoder.layers.1.self_attention.linear_proj.weight": _seq(8, 8),
            M + "language_model.embedding.word_embeddings.weight": _seq(4, 8),
            M + "vision_model.decoder.layers.1.self_attention.linear_qkv.weight": _seq(12, 4),
            M + "vision_model.decoder.layers.1.self_attention.linear_qkv.bias": _seq(12),
            M + "vision_model.patch_embed.proj.weight": _seq(8),
            M + "vision_model.decoder.layers.1.mlp.linear_fc1.weight": _seq(8, 4),
            M + "vision_model.merger.linear_fc2.weight": _seq(8, 4),
            M + "vision_model.decoder.deepstack_merger_list.2.patch_norm.weight": _seq(8),
        }
        for name, tensor in cases.items():
            _same(ours, theirs, name, tensor)
    ours, theirs = _both_train_converters(arch, hf, tf, {"infer_atten_tp_size": 1, "infer_engine_config": SimpleNamespace(tp_size=1, ep_size=2)},
                                          ep_rank=1, ep_size=2)
    _same(ours, theirs, M + "language_model.decoder.layers.0.mlp.experts.linear_fc2.weight0", _seq(8, 6))
    ours, theirs = _both_infer_converters(arch, hf)
    for name, tensor in {"model.layers.0.self_attn.qkv_proj.weight": _seq(16, 8), "model.embed_tokens.weight": _seq(4, 8),
                         "visual.patch_embed.proj.weight": _seq(8), "visual.blocks.1.mlp.linear_fc1.weight": _seq(8, 4),
                         "visual.deepstack_merger_list.2.norm.weight": _seq(8)}.items():
        _same(ours, theirs, name, tensor)


def test_qwen3_5_converters_agree_on_gated_attention_and_delta_net():
    text = SimpleNamespace(model_type="qwen3_5_moe_text", architectures=["Qwen3_5MoeForCausalLM"], hidden_size=8, num_hidden_layers=4,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=2, linear_num_key_heads=2, linear_key_head_dim=2,
                           linear_num_value_heads=4, linear_value_head_dim=2, num_experts=4, tie_word_embeddings=False)
    hf = SimpleNamespace(architectures=["Qwen3_5MoeForConditionalGeneration"], text_config=text,
                         vision_config=SimpleNamespace(num_heads=2, hidden_size=4), tie_word_embeddings=False)
    tf = SimpleNamespace(hidden_size=8, num_attention_heads=4, num_query_groups=2, kv_channels=2, num_layers=4)
    for infer_tp in (1, 2):
        conf = {"infer_atten_tp_size": infer_tp, "infer_engine_config": SimpleNamespace(tp_size=infer_tp, ep_size=1)}
        ours, theirs = _both_train_converters(hf.architectures[0], hf, tf, conf)
        cases = {
            M + "language_model.decoder.layers.0.self_attention.linear_qkv.weight": _seq(24, 8),  # [Q, gate, K, V] per KV group
            M + "language_model.decoder.layers.0.self_attention.in_proj.weight": _seq(32, 8),     # Q 4, K 4, V 8, Z 8, B 4, A 4
            M + "language_model.decoder.layers.1.self_attention.linear_proj.weight": _seq(8, 8),
            M + "language_model.embedding.word_embeddings.weight": _seq(4, 8),
        }
        for name, tensor in cases.items():
            _same(ours, theirs, name, tensor)
        for skipped in ("language_model.mtp.layers.0.eh_proj.weight", "mtp.layers.0.mtp_model_layer.mlp.linear_fc1.weight"):
            _same(ours, theirs, M + skipped, _seq(8, 8))  # multi-token-prediction weights are not sent by either
    ours, theirs = _both_infer_converters(hf.architectures[0], hf)
    for name, tensor in {"model.layers.0.qkv_proj.weight": _seq(24, 8), "model.layers.0.linear_attn.A_log": _seq(4),
                         "mtp.norm.weight": _seq(8)}.items():
        _same(ours, theirs, name, tensor)


@pytest.mark.parametrize("tp", [1, 2, 4])
def test_mla_down_projection_packing_agrees(tp):
    from awex.converter.mcore_converter import pack_fused_qkv_a_proj_for_tp as ref_pack

    from awex_b200.converter.mcore_converter import pack_fused_qkv_a_proj_for_tp as our_pack

    q, kv = _seq(8, 3), -_seq(4, 3)
    assert torch.equal(our_pack(q, kv, tp), ref_pack(q, kv, tp))


@pytest.mark.parametrize("arch", ["BailingMoeForCausalLM", "BailingMoeV2ForCausalLM", "BailingMoeV2_5ForCausalLM"])
def test_bailing_families_resolve_to_the_same_kind_of_converters_and_sharding(arch):
    import awex.models.registry as ref_registry

    import awex_b200.models.registry as our_registry

    hf = SimpleNamespace(architectures=[arch], quantization_config={})
    tf = SimpleNamespace(layer_group_size=4)
    ours, theirs = _both_train_converters(arch, hf, tf, {"infer_atten_tp_size": 1})
    assert type(ours).__name__ == type(theirs).__name__
    assert our_registry.get_sharding_strategy(arch).__name__ == ref_registry.get_sharding_strategy(arch).__name__


# ---- the control plane on the wire --------------------------------------------------------------------
def _exercise_meta_client(client, other_client):
    """The calls the exchange makes, written by ``client`` and read back by
    ``other_client`` (and the other way round), both talking to one server."""
    client.put_object("infer_conf", {"tp_size": 2, "names": ["a", "b"], "nested": (1, 2.5, None)})
    assert other_client.get_object("infer_conf") == {"tp_size": 2, "names": ["a", "b"], "nested": (1, 2.5, None)}
    other_client.put_binary("blob/with/slashes", bytes(range(256)) * 40)
    assert client.get_binary("blob/with/slashes") == bytes(range(256)) * 40
    client.put_json("json_key", {"step": 3, "ok": True})
    assert other_client.get_json("json_key") == {"step": 3, "ok": True}
    for member, who in ((0, client), (1, other_client), (1, client)):
        who.add_object_to_set("ready_engines", member)
    assert client.get_set("ready_engines") == {0, 1} == other_client.get_set("ready_engines")
    other_client.wait_set_until_size("ready_engines", 2, timeout=5)
    assert client.has_key("json_key") and other_client.has_key("json_key") and not other_client.has_key("absent")
    assert {"infer_conf", "json_key", "ready_engines"} <= set(client.list_keys()) and set(client.list_keys()) == set(other_client.list_keys())
    ids = [client.allocate_auto_grow_id(), other_client.allocate_auto_grow_id(), client.allocate_auto_grow_id()]
    assert ids == sorted(ids) and len(set(ids)) == 3
    other_client.delete("json_key")
    assert not client.has_key("json_key")
    client.delete_if_exists("json_key")  # absent: no error
    assert other_client.get_object("absent", default_value="fallback") == "fallback"
    assert client.health_check() and other_client.health_check()


def test_both_clients_speak_to_both_servers():
    """The reference's client against this server, this client against the
    reference's server, each mixed with the other client on the same keys: the
    REST routes and the payload encoding are the same."""
    from awex.meta.meta_server import MetaServer as RefServer, MetaServerClient as RefClient

    from awex_b200.meta.meta_server import MetaServer, MetaServerClient
    from awex_b200.utils.common import get_free_port

    ours = MetaServer("127.0.0.1", 0)
    ours.start()
    try:
        _exercise_meta_client(RefClient("127.0.0.1", ours.port), MetaServerClient("127.0.0.1", ours.port))
    finally:
        ours.stop()
    theirs = RefServer("127.0.0.1", get_free_port())
    theirs.start()
    try:
        _exercise_meta_client(MetaServerClient("127.0.0.1", theirs.port), RefClient("127.0.0.1", theirs.port))
    finally:
        theirs.stop()


# ---- the inference-side metadata resolver ---------------------------------------------------------------
def _meta_key(metas):
    """ParameterMeta lists of either implementation as plain comparable data."""
    out = {}
    for p in metas:
        out[p.name] = (
            tuple(p.global_shape), str(p.dtype), p.global_numel,
            tuple(tuple((s.name, tuple(s.shape), tuple(s.global_offset), s.sharding_type.name, s.num_shards, s.sharding_dim,
                         s.tp_rank, s.attn_tp_rank, s.pp_rank, s.ep_rank, s.global_rank, s.world_size, s.engine_rank)
                        for s in replica.shards) for replica in p.replicas),
        )
    return out


class _CannedEngine:
    """An inference engine whose workers answer the metadata task with reports made beforehand."""

    def __init__(self, engine_name, hf_config, config, reports):
        self.engine_name, self.hf_config, self.config, self.reports = engine_name, hf_config, config, reports

    def execute_task_in_model_worker(self, fn, **kwargs):
        return self.reports


def _both_inference_resolvers(arch, infer):
    from awex.meta.infer_meta_resolver import InferParamMetaResolver as RefResolver

    from awex_b200.meta.infer_meta_resolver import InferParamMetaResolver, collect_worker_param_info
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout

    job = SimulatedJob(get_arch(arch), TrainLayout(tp=1), InferLayout(**infer), dtype=torch.bfloat16)
    engine = job.engines[0]
    reports = engine.execute_task_in_model_worker(collect_worker_param_info, engine_name=engine.engine_name,
                                                  infer_engine_config=engine.config, engine_rank=0, convert_params=True)
    for report in reports:  # what an RPC layer hands back; both resolvers restore it to their own class
        report["rank_info"] = dataclasses.asdict(report["rank_info"])
    aliases = set(job.aliases)
    for report in reports:  # second names of one memory are this framework's addition: the reference has no such entry
        report["params_meta"] = [m for m in report["params_meta"] if m["name"] not in aliases]
        report.pop("aliases", None)

    def canned():
        return _CannedEngine(engine.engine_name, engine.hf_config, engine.config, [dict(r) for r in reports])

    ours = InferParamMetaResolver(canned(), convert_params=True, num_engines=job.infer.num_engines, engine_rank=0)
    theirs = RefResolver(canned(), convert_params=True, num_engines=job.infer.num_engines, engine_rank=0)
    return ours, theirs, job


@pytest.mark.parametrize("arch,infer", [
    ("tiny-llama", dict(tp=2)),
    ("tiny-qwen2", dict(tp=2, num_engines=2)),
    ("tiny-qwen3-moe", dict(tp=2, ep=2, engine_name="sglang")),
    ("tiny-llama", dict(tp=4, attn_tp=2, engine_name="sglang")),  # data-parallel attention
])
def test_inference_resolver_builds_the_same_metadata_from_the_same_worker_reports(arch, infer):
    """Per-worker reports (canonical names, local shapes, rank descriptions) of a
    synthetic engine go through the reference's resolver and through this one:
    global shapes, shard offsets, sharding kinds and replicas must agree."""
    ours, theirs, _job = _both_inference_resolvers(arch, infer)
    got, want = _meta_key(ours.get_parameters_meta()), _meta_key(theirs.get_parameters_meta())
    assert set(got) == set(want)
    differing = [name for name in want if got[name] != want[name]]
    assert not differing, (differing[:5], got[differing[0]], want[differing[0]])
    assert (ours.total_numel, ours.total_size, ours.get_model_arch_name()) == (theirs.total_numel, theirs.total_size, theirs.get_model_arch_name())


def test_data_parallel_attention_with_split_projection_names_is_where_the_two_part():
    """Known difference.  The reference recognises attention weights by the
    substring ``attention`` (`awex/sharding/param_sharding.py:289`), so the
    ``self_attn.q_proj`` names of the Qwen3 families fall through to plain tensor
    parallelism over the whole TP group and, under data-parallel attention, get a
    global shape twice too large.  Here they are attention weights: two replicas
    of attention-TP shards and the true global shape."""
    ours, theirs, job = _both_inference_resolvers("tiny-qwen3-moe", dict(tp=4, ep=4, attn_tp=2, engine_name="sglang"))
    name = "model.layers.0.self_attn.q_proj.weight"
    got = {p.name: p for p in ours.get_parameters_meta()}[name]
    want = {p.name: p for p in theirs.get_parameters_meta()}[name]
    true_rows = job.arch.num_heads * job.arch.head_dim
    assert got.global_shape[0] == true_rows and len(got.replicas) == 2 and got.shards[0].sharding_type.name == "DP_TP_SHARDING"
    assert want.global_shape[0] == 2 * true_rows and want.shards[0].sharding_type.name == "TP_SHARDING"
    # everything that is not attention agrees
    a, b = _meta_key(ours.get_parameters_meta()), _meta_key(theirs.get_parameters_meta())
    assert all(a[n] == b[n] for n in a if "self_attn" not in n)


# ---- the training-side metadata resolver (two tensor-parallel ranks over gloo) ----------------------------------
def _train_resolver_rank(rank, world, port, arch, q):
    """One training rank: the reference's resolver and this one on the same
    Megatron-layout shard, with the stand-in for Megatron's parallel state
    (tensor-parallel group = all ranks)."""
    import faulthandler

    faulthandler.dump_traceback_later(200, exit=True)
    try:
        for path in (STUBS, REF):
            if path not in sys.path:
                sys.path.insert(0, path)
        os.environ["AWEX_DEVICE_TYPE"] = "cpu"
        import torch.distributed as dist

        import awex.logging as ref_logging
        from awex.meta.train_meta_resolver import McoreParamMetaResolver as RefResolver

        from awex_b200 import logging as our_logging
        from awex_b200.config import InferenceConfig
        from awex_b200.meta.train_meta_resolver import McoreParamMetaResolver
        from baseline import synth
        from baseline.reference_bench import _TrainEngine

        ref_logging.setLevel("ERROR")
        our_logging.setLevel("ERROR")
        # the reference takes the local rank modulo the number of accelerators, which is zero on a CPU-only
        # machine; tell both sides (in this process only) that the node has eight
        import awex.util.device as ref_device

        import awex_b200.utils.device as our_device

        ref_device.device_count = our_device.device_count = lambda: 8
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        hf_config = synth.hf_config_for(arch)
        model = synth.megatron_module(arch, world, rank, torch.float32, "cpu")
        infer_conf = {"hf_config": hf_config, "engine_name": "vllm", "infer_atten_tp_size": 1, "router_dtype": "bf16",
                      "infer_engine_config": InferenceConfig(tp_size=1, comm_backend="nccl"), "infer_world_size": 1}
        theirs = RefResolver(_TrainEngine(model, hf_config, "unused"), hf_config, dict(infer_conf))
        ours = McoreParamMetaResolver(_TrainEngine(model, hf_config, "unused"), hf_config, dict(infer_conf))
        got, want = _meta_key(ours.get_parameters_meta()), _meta_key(theirs.get_parameters_meta())
        problems = sorted(set(got) ^ set(want)) + [n for n in want if n in got and got[n] != want[n]]
        if (ours.total_numel, ours.total_size) != (theirs.total_numel, theirs.total_size):
            problems.append(f"totals {ours.total_numel, ours.total_size} != {theirs.total_numel, theirs.total_size}")
        if ours.get_pp_stage_layer_id_map() != theirs.get_pp_stage_layer_id_map():
            problems.append("pipeline stage maps differ")
        q.put((rank, problems[:5], len(want)))
        dist.barrier()
        dist.destroy_process_group()
    except BaseException as exc:
        q.put((rank, [f"rank {rank} failed: {exc!r}"], 0))
        raise


@pytest.mark.timeout(400)
@pytest.mark.parametrize("arch", ["tiny-llama", "tiny-qwen2"])
def test_training_resolver_builds_the_same_metadata_on_two_tensor_parallel_ranks(arch):
    import queue

    import torch.multiprocessing as mp

    from awex_b200.utils.common import get_free_port

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = get_free_port()
    procs = [ctx.Process(target=_train_resolver_rank, args=(r, 2, port, arch, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        results = [q.get(timeout=240) for _ in procs]
        for p in procs:
            p.join(timeout=60)
    except queue.Empty:
        pytest.fail("a rank did not report")
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
    for rank, problems, count in results:
        assert problems == [] and count > 0, (rank, problems)


# ---- sharding rules and rank descriptions ---------------------------------------------------------------
SHARDING_NAMES = [
    "model.embed_tokens.weight", "lm_head.weight", "model.norm.weight",
    "model.layers.0.input_layernorm.weight", "model.layers.0.post_attention_layernorm.weight",
    "model.layers.0.attention.query_key_value_proj.weight", "model.layers.0.attention.query_key_value_proj.bias",
    "model.layers.0.attention.dense.weight", "model.layers.0.attention.q_norm.weight",
    "model.layers.3.mlp.gate_proj.weight", "model.layers.3.mlp.up_proj.weight", "model.layers.3.mlp.down_proj.weight",
    "model.layers.3.mlp.gate_up_proj.weight", "model.layers.3.mlp.gate.weight", "model.layers.3.mlp.router.weight",
    "model.layers.3.mlp.gate.expert_bias", "model.layers.3.mlp.experts.7.gate_proj.weight",
    "model.layers.3.mlp.experts.7.down_proj.weight", "model.layers.3.mlp.shared_experts.gate_proj.weight",
    "model.layers.3.mlp.shared_experts.down_proj.weight", "model.layers.1.attention.kv_a_proj_with_mqa.weight",
    "model.layers.1.attention.fused_qkv_a_proj_with_mqa.weight", "model.layers.1.attention.q_a_layernorm.weight",
    "model.layers.1.attention.kv_b_proj.weight", "model.layers.1.attention.g_norm.weight", "model.layers.1.attention.g_proj.weight",
    "model.layers.2.self_attn.o_proj.weight", "model.layers.2.linear_attn.in_proj_qkvz.weight", "model.layers.2.linear_attn.out_proj.weight",
    "model.layers.2.linear_attn.conv1d.weight", "model.layers.2.linear_attn.A_log", "model.layers.2.linear_attn.dt_bias",
    "model.layers.2.linear_attn.norm.weight", "model.visual.blocks.0.attn.qkv.weight", "model.visual.blocks.0.mlp.linear_fc1.weight",
    "model.visual.merger.linear_fc2.weight", "model.visual.patch_embed.proj.weight", "model.language_model.layers.0.mlp.experts.gate_up_proj",
    "model.language_model.layers.0.mlp.experts.down_proj", "something.unrecognised.weight",
]
SHARDING_ARCHS = ["LlamaForCausalLM", "Qwen3MoeForCausalLM", "BailingMoeV2ForCausalLM", "BailingMoeLinearV2ForCausalLM",
                  "Qwen3VLMoeForConditionalGeneration", "Qwen3_5MoeForConditionalGeneration"]


def _rank_kwargs(tp, ep=1, etp=1, attn_tp=None, infer=True):
    attn_tp = attn_tp or tp
    return dict(tp_rank=0, tp_size=tp, pp_rank=0, pp_size=1, dp_size=1, dp_rank=0, ep_rank=0, ep_size=ep, ep_tp_rank=0, ep_tp_size=etp,
                attn_tp_rank=0, attn_tp_size=attn_tp, attn_dp_rank=0, world_size=tp, global_rank=0, local_rank=0, engine_rank=0, is_infer=infer)


@pytest.mark.parametrize("arch", SHARDING_ARCHS)
def test_sharding_rules_agree_name_by_name(arch):
    """(kind, dimension, number of shards) of every kind of parameter name, for
    the training side and both serving engines, over several parallel layouts.
    Names that hold ``self_attn`` are left out under data-parallel attention (the
    known difference above)."""
    import awex.sharding.param_sharding as ref_sharding
    import awex.sharding.rank_info as ref_rank
    from awex.sharding.mcore_sharding import get_mcore_sharding_strategy as ref_mcore

    import awex_b200.sharding.param_sharding as our_sharding
    import awex_b200.sharding.rank_info as our_rank
    from awex_b200.config import InferenceConfig
    from awex_b200.sharding.extractors import get_mcore_sharding_strategy

    layouts = [dict(tp=1), dict(tp=4), dict(tp=4, ep=4), dict(tp=8, ep=4, etp=2), dict(tp=4, ep=2, attn_tp=2)]
    checked = 0
    for layout in layouts:
        kw = _rank_kwargs(**layout)
        dp_attention = kw["attn_tp_size"] != kw["tp_size"]
        config = InferenceConfig(tp_size=kw["tp_size"], ep_size=kw["ep_size"], dp_size=kw["tp_size"] // kw["attn_tp_size"],
                                 enable_dp_attention=dp_attention, enable_dp_lm_head=dp_attention, comm_backend="nccl")
        pairs = [(get_mcore_sharding_strategy(arch, our_rank.RankInfo(**dict(kw, is_infer=False))),
                  ref_mcore(arch, ref_rank.RankInfo(**dict(kw, is_infer=False))))] if not dp_attention else []
        for engine in ("sglang", "vllm"):
            pairs.append((our_sharding.get_sharding_strategy_builder(engine)(arch, config, our_rank.RankInfo(**kw)),
                          ref_sharding.get_sharding_strategy_builder(engine)(arch, config, ref_rank.RankInfo(**kw))))
        for ours, theirs in pairs:
            for name in SHARDING_NAMES:
                if dp_attention and "self_attn" in name:
                    continue
                kind, dim, shards = ours.get_sharding_strategy(name)
                ref_kind, ref_dim, ref_shards = theirs.get_sharding_strategy(name)
                assert (kind.name, dim, shards) == (ref_kind.name, ref_dim, ref_shards), (arch, layout, ours.engine_name, name)
                checked += 1
    assert checked > 300
    for name in SHARDING_NAMES:
        assert our_sharding.get_default_sharding_dim(name) == ref_sharding.get_default_sharding_dim(name), name


def test_rank_descriptions_from_worker_contexts_agree():
    """What a serving worker's context says about its place in the engine, as
    both implementations read it (SGLang and vLLM flavours, expert parallelism
    inside and outside the TP group, context parallelism, data-parallel attention)."""
    from awex.sharding.sglang_sharding import get_sglang_rank_info as ref_sglang
    from awex.sharding.vllm_sharding import get_vllm_rank_info as ref_vllm

    from awex_b200.sharding.extractors import get_sglang_rank_info, get_vllm_rank_info

    def context(tp_rank, tp_size, server_args=None, **extra):
        ctx = dict(tp_rank=tp_rank, tp_size=tp_size, pp_rank=0, pp_size=1, dp_rank=0, dp_size=1, attn_tp_rank=tp_rank,
                   attn_tp_size=tp_size, attn_dp_rank=0, world_size=tp_size, global_rank=tp_rank, local_rank=tp_rank,
                   scheduler=SimpleNamespace(server_args=server_args))
        ctx.update(extra)
        return ctx

    def args(**kw):
        base = dict(dp_size=1, enable_dp_attention=False, ep_size=1)
        base.update(kw)
        return SimpleNamespace(**base)

    sglang_cases = [
        context(3, 8, args()),
        context(5, 8, args(ep_size=4)),                                    # expert TP of two inside each expert group
        context(2, 4, args(ep_size=4)),
        context(1, 4, args(dp_size=2, enable_dp_attention=True), attn_tp_rank=1, attn_tp_size=2, attn_dp_rank=0, dp_size=2),
        context(0, 2, args(context_parallel_size=2, context_parallel_mode="ulysses"), cp_rank=1),
        context(0, 2, args(), cp_size=2, cp_rank=1),                       # mode left to the default of a ring
    ]
    for ctx in sglang_cases:
        assert dataclasses.asdict(get_sglang_rank_info(ctx, 1)) == dataclasses.asdict(ref_sglang(ctx, 1)), ctx
    with pytest.raises(ValueError):
        get_sglang_rank_info(context(0, 2, args(dp_size=2)), 0)
    with pytest.raises(ValueError):
        ref_sglang(context(0, 2, args(dp_size=2)), 0)
    vllm_cases = [
        context(1, 2),
        context(1, 2, ep_size=4, ep_rank=3),
        context(1, 2, ep_size=4, ep_rank=3, ep_tp_size=2, ep_tp_rank=1),
        context(0, 1, ep_size=1, ep_rank=5, ep_tp_size=4, ep_tp_rank=2),      # no expert parallelism: the EP fields are reset
        context(0, 4, dp_size=2, dp_rank=1, cp_size=2, cp_rank=1, cp_mode="ulysses"),
    ]
    for ctx in vllm_cases:
        assert dataclasses.asdict(get_vllm_rank_info(ctx, 2)) == dataclasses.asdict(ref_vllm(ctx, 2)), ctx


# ---- which decoder layers a pipeline stage holds ---------------------------------------------------------------
def _outcome(fn, *args, **kwargs):
    try:
        return ("ok", fn(*args, **kwargs))
    except (ValueError, AssertionError, ZeroDivisionError) as exc:
        return ("error", type(exc).__name__)


def test_pipeline_stage_layer_ids_agree_over_a_grid_of_split_settings():
    """Even and uneven splits, first/last stage sizes, embedding / loss counted as
    layers, virtual stages, explicit layouts: for every (pipeline rank, virtual
    stage) both implementations name the same global layers, and settings one
    refuses the other refuses too."""
    import itertools

    import awex.sharding.rank_info as ref_rank
    from awex.converter.mcore_converter import _process_mcore_pp_name as ref_name, _resolve_pp_stage_global_layer_ids as ref_ids

    import awex_b200.sharding.rank_info as our_rank
    from awex_b200.converter.pp_layout import process_mcore_pp_name, resolve_pp_stage_global_layer_ids

    checked = refused = 0
    grid = itertools.product([8, 12, 14], [1, 2, 4], [None, 2], [None, 1, 3], [None, 2, 3], [False, True], [False, True])
    for layers, pp, vp, first, last, embed, loss in grid:
        tf = SimpleNamespace(num_layers=layers, num_layers_in_first_pipeline_stage=first, num_layers_in_last_pipeline_stage=last,
                             account_for_embedding_in_pipeline_split=embed, account_for_loss_in_pipeline_split=loss,
                             virtual_pipeline_model_parallel_size=vp, pipeline_model_parallel_layout=None)
        hf = SimpleNamespace(num_hidden_layers=layers)
        for pp_rank in range(pp):
            for vp_stage in range(vp or 1):
                kw = dict(_rank_kwargs(tp=1, infer=False), pp_rank=pp_rank, pp_size=pp, world_size=pp, global_rank=pp_rank)
                got = _outcome(resolve_pp_stage_global_layer_ids, our_rank.RankInfo(**kw), hf, tf, vp_stage)
                want = _outcome(ref_ids, ref_rank.RankInfo(**kw), hf, tf, vp_stage)
                assert got[0] == want[0] and (got[0] == "error" or got[1] == want[1]), ((layers, pp, vp, first, last, embed, loss), pp_rank, vp_stage, got, want)
                checked += 1
                refused += got[0] == "error"
    assert checked > 1500 and 0 < refused < checked
    # explicit layouts: a list of stages, each a list of layer kinds ("E" embedding, "t" decoder, "L" loss)
    for layout, pp in (([["embedding", "decoder", "decoder"], ["decoder"], ["decoder", "decoder", "decoder"], ["decoder", "loss"]], 4),
                       ([["embedding", "decoder"], ["decoder", "decoder"], ["decoder", "decoder"], ["decoder", "decoder", "loss"]], 2)):
        tf = SimpleNamespace(num_layers=7, pipeline_model_parallel_layout=layout, virtual_pipeline_model_parallel_size=None)
        hf = SimpleNamespace(num_hidden_layers=7)
        vp_size = len(layout) // pp
        for pp_rank in range(pp):
            for vp_stage in range(vp_size):
                kw = dict(_rank_kwargs(tp=1, infer=False), pp_rank=pp_rank, pp_size=pp, world_size=pp, global_rank=pp_rank)
                got = _outcome(resolve_pp_stage_global_layer_ids, our_rank.RankInfo(**kw), hf, tf, vp_stage)
                want = _outcome(ref_ids, ref_rank.RankInfo(**kw), hf, tf, vp_stage)
                assert got == want and got[0] == "ok", (layout, pp_rank, vp_stage, got, want)
    # renaming a stage-local layer index
    stage_map = {(1, 0): {0: 4, 1: 5}, (1, 1): {0: 12}}
    kw = dict(_rank_kwargs(tp=1, infer=False), pp_rank=1, pp_size=2)
    for name, vp_stage in (("decoder.layers.1.mlp.linear_fc1.weight", 0), ("decoder.layers.0.self_attention.linear_qkv.weight", 1),
                           ("embedding.word_embeddings.weight", 0), ("decoder.layers.7.mlp.linear_fc2.weight", 0)):
        got = _outcome(process_mcore_pp_name, name, our_rank.RankInfo(**kw), None, None, vp_stage, stage_map)
        want = _outcome(ref_name, name, ref_rank.RankInfo(**kw), None, None, vp_stage, stage_map)
        assert got == want, (name, got, want)


# ---- the alignment contract, the configuration schema, packed tensors ---------------------------------------------
def test_metadata_alignment_contract_refuses_the_same_pairs():
    """Training and inference metadata that both implementations accept, and
    seeded mismatches (a missing name, an extra name that is no alias, another
    element count, shape or dtype) that both refuse."""
    import copy

    import awex.meta.weight_meta as ref_meta
    from awex.util.common import check_train_infer_params_meta as ref_check

    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout
    from awex_b200.utils.common import check_train_infer_params_meta

    job = SimulatedJob(get_arch("tiny-llama"), TrainLayout(tp=2), InferLayout(tp=1), dtype=torch.float32, device="meta")

    def verdicts(train, infer, strict=False):
        ours = _outcome(check_train_infer_params_meta, train, infer, raise_exception=True, strict_key_match=strict)[0]
        theirs = _outcome(ref_check, _to_reference(train, ref_meta), _to_reference(infer, ref_meta), raise_exception=True, strict_key_match=strict)[0]
        return ours, theirs

    train, infer = job.train_meta, job.infer_meta
    assert verdicts(train, infer) == ("ok", "ok") and verdicts(train, infer, strict=True) == ("ok", "ok")
    assert verdicts(train, infer[1:]) == ("error", "error")                       # a trained parameter nobody serves
    extra = copy.deepcopy(infer[3])
    extra.name = "model.layers.0.something_else.weight"
    assert verdicts(train, infer + [extra]) == ("error", "error")                 # an extra name that is no alias
    tied = copy.deepcopy(next(m for m in infer if m.name == "model.embed_tokens.weight"))
    tied.name = "lm_head.weight"
    no_head = [m for m in train if m.name != "lm_head.weight"]
    assert verdicts(no_head, infer) == ("ok", "ok")                               # the tied head is an allowed infer-only name
    assert verdicts(no_head, infer, strict=True) == ("error", "error")
    for field, value in (("global_numel", 7), ("global_shape", (3, 5)), ("dtype", torch.float16)):
        changed = copy.deepcopy(infer)
        setattr(changed[2], field, value)
        assert verdicts(train, changed) == ("error", "error"), field


def test_configuration_schema_has_every_field_of_the_reference_with_its_default():
    from awex.config import InferenceConfig as RefConfig

    from awex_b200.config import InferenceConfig

    ours = {f.name: f for f in dataclasses.fields(InferenceConfig)}
    for field in dataclasses.fields(RefConfig):
        assert field.name in ours, field.name
        if field.default is not dataclasses.MISSING:
            assert ours[field.name].default == field.default, field.name
    server_args = SimpleNamespace(tp_size=2, pp_size=1, dp_size=1, ep_size=1, enable_dp_attention=False, nnodes=1, node_rank=0, something_else=1)
    mine = InferenceConfig.from_sgl_server_args(server_args, comm_backend="file")
    theirs = RefConfig.from_sgl_server_args(server_args, comm_backend="file")
    for field in dataclasses.fields(RefConfig):
        assert getattr(mine, field.name) == getattr(theirs, field.name), field.name


def test_packed_tensor_groups_cross_between_the_two_implementations():
    """Tensors packed by dtype by one implementation are taken apart by the
    other: the metadata that travels with the groups means the same."""
    from awex.util.tensor_util import group_tensors_by_shape_and_dtype as ref_group, reconstruct_tensors_from_groups as ref_rebuild

    from awex_b200.utils.tensor_util import group_tensors_by_shape_and_dtype, reconstruct_tensors_from_groups

    g = torch.Generator().manual_seed(3)
    tensors = [torch.randn(4, 6, generator=g), torch.randn(7, generator=g).to(torch.bfloat16), torch.randn(2, 3, 5, generator=g),
               torch.arange(11, dtype=torch.int32), torch.randn(1, 9, generator=g).to(torch.bfloat16), torch.randn(5, 5, generator=g)[:, 1:3]]
    for pack, unpack in ((group_tensors_by_shape_and_dtype, ref_rebuild), (ref_group, reconstruct_tensors_from_groups)):
        for limit in (5 * 1024**3, 64):  # one group per dtype, and groups cut at a small size bound
            groups, metadata = pack(tensors, max_tensor_size=limit)
            back = unpack(groups, metadata)
            assert len(back) == len(tensors)
            for a, b in zip(back, tensors):
                assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)


def test_nan_scans_and_difference_reports_reach_the_same_verdicts():
    from awex.util.tensor_util import check_and_log_nan_values as ref_nan, compare_and_log_tensor_differences as ref_compare

    from awex_b200.utils.tensor_util import check_and_log_nan_values, compare_and_log_tensor_differences

    g = torch.Generator().manual_seed(9)
    base = torch.randn(6, 7, generator=g)
    with_nan = base.clone()
    with_nan[2, 3] = float("nan")
    for tensor in (base, with_nan, torch.full((3,), float("inf")), torch.full((2, 2), float("nan")), torch.zeros(0), base.to(torch.bfloat16)):
        assert check_and_log_nan_values(tensor, "t", " after update") == ref_nan(tensor, "t", " after update")
    near = base + 1e-7
    far = base.clone()
    far[1, 1] += 0.5
    cases = [(base, base.clone(), {}), (base, near, {}), (base, near, dict(exact_match=True)), (base, far, {}), (base, far, dict(atol=1.0)),
             (base, base[:, :3], {}), (base, near, dict(atol=0.0, rtol=0.0)), (base.to(torch.bfloat16), base.to(torch.bfloat16), dict(exact_match=True))]
    for a, b, kw in cases:
        ours, theirs = compare_and_log_tensor_differences(a, b, "t", **kw), ref_compare(a, b, "t", **kw)
        if kw.get("exact_match") and not torch.equal(a, b):
            # Known difference: after a failed bitwise comparison the reference looks for elements outside the
            # tolerances, finds none and reports agreement (`awex/util/tensor_util.py:467-537`); exact means exact here.
            assert (ours, theirs) == (False, True)
            continue
        assert ours == theirs, kw


def test_mbridge_loaders_fill_a_model_with_the_same_values():
    """A bridge that maps Megatron names to one or several checkpoint names
    (fused QKV = q + k + v along the rows, fused gate/up), a critic whose output
    layer stays untouched, a reader that serves tensors by name."""
    from awex.mbridge_loader import load_weights_from_hf_with_mbridge as ref_load

    from awex_b200.mbridge_loader import load_weights_from_hf_with_mbridge

    g = torch.Generator().manual_seed(21)
    checkpoint = {name: torch.randn(shape, generator=g) for name, shape in {
        "q": (8, 6), "k": (4, 6), "v": (4, 6), "gate": (10, 6), "up": (10, 6), "down": (6, 10), "norm": (6,), "head": (12, 6)}.items()}
    hf_names = {"decoder.qkv.weight": ["q", "k", "v"], "decoder.fc1.weight": ["gate", "up"], "decoder.fc2.weight": "down",
                "decoder.norm.weight": "norm", "output_layer.weight": "head"}

    class Bridge:
        def _get_actual_hf_path(self, path):
            return path + "/resolved"

        def _weight_name_mapping_mcore_local_to_global(self, model):
            return {name: name for name in model.state_dict()} | {"decoder.absent.weight": "decoder.absent.weight"}

        def _weight_name_mapping_mcore_to_hf(self, name):
            return hf_names[name]

    def reader(path, name):
        assert path == "ckpt/resolved"
        return checkpoint[name].to(torch.bfloat16)  # the loader casts to the parameter's dtype

    def model():
        m = torch.nn.Module()
        m.register_parameter("placeholder", None)
        for name, shape in {"decoder.qkv.weight": (16, 6), "decoder.fc1.weight": (20, 6), "decoder.fc2.weight": (6, 10),
                            "decoder.norm.weight": (6,), "output_layer.weight": (12, 6)}.items():
            m.register_buffer(name.replace(".", "_"), torch.zeros(shape))
        m.state_dict = lambda: {name: getattr(m, name.replace(".", "_")) for name in hf_names}
        return m

    for critic in (False, True):
        ours, theirs = model(), model()
        load_weights_from_hf_with_mbridge(Bridge(), [ours], "ckpt", reader=reader, is_critic=critic)
        ref_load(Bridge(), [theirs], "ckpt", reader=reader, is_critic=critic)
        for name in hf_names:
            assert torch.equal(ours.state_dict()[name], theirs.state_dict()[name]), (critic, name)
        assert bool(ours.state_dict()["output_layer.weight"].any()) == (not critic)
        assert torch.equal(ours.state_dict()["decoder.qkv.weight"], torch.cat([checkpoint[n] for n in "qkv"]).to(torch.bfloat16).float())


def test_vllm_plugin_request_schema_and_rpc_envelope_agree():
    """The two HTTP request bodies (field names and defaults), what may cross
    vLLM's engine-core RPC (dtypes and devices as strings, tuples as lists) and
    which keyword arguments reach a worker method."""
    pytest.importorskip("vllm")
    import awex.vllm_plugin as ref_plugin

    from awex_b200 import vllm_plugin

    for ours, theirs in ((vllm_plugin.AwexInitRequest, ref_plugin.AwexInitRequest), (vllm_plugin.AwexUpdateRequest, ref_plugin.AwexUpdateRequest)):
        assert list(ours.model_fields) == list(theirs.model_fields)
        for name, field in theirs.model_fields.items():
            assert ours.model_fields[name].default == field.default and ours.model_fields[name].is_required() == field.is_required(), name
    payload = {"dtype": torch.bfloat16, "device": torch.device("cpu"), "shape": (2, 3), "nested": [{"d": torch.float8_e4m3fn, "n": None, "x": 1.5}], "s": "text"}
    assert vllm_plugin.sanitize_for_ipc(payload) == ref_plugin._sanitize_for_ipc(payload)
    # worker methods this framework keeps from the reference's table accept the same keyword arguments
    for method, signature in ref_plugin._AWEX_WORKER_SIGNATURES.items():
        if method not in vllm_plugin.AWEX_WORKER_SIGNATURES:
            continue
        kwargs = {name: 1 for name in signature["required"] + signature["optional"]}
        kwargs["not_for_the_worker"] = 2
        ours = _outcome(vllm_plugin.filter_awex_kwargs, method, dict(kwargs))
        theirs = _outcome(ref_plugin._filter_awex_kwargs, method, dict(kwargs))
        assert ours[0] == theirs[0] == "ok" and set(theirs[1]) <= set(ours[1]) and "not_for_the_worker" not in ours[1], method
        # what this framework requires, the reference requires too (the validation calls take their step as an option here)
        assert set(vllm_plugin.AWEX_WORKER_SIGNATURES[method]["required"]) <= set(signature["required"]), method
        without_required = {name: 1 for name in signature["optional"]}
        if vllm_plugin.AWEX_WORKER_SIGNATURES[method]["required"]:
            assert _outcome(vllm_plugin.filter_awex_kwargs, method, without_required)[0] == "error"
            assert _outcome(ref_plugin._filter_awex_kwargs, method, without_required)[0] == "error"
    assert set(ref_plugin._AWEX_WORKER_METHODS) & set(vllm_plugin.AWEX_WORKER_METHODS)
