"""Train/inference contracts of the multimodal and hybrid families, case by case:
the behaviours the reference pins in `awex/tests/test_qwen3_vl.py`,
`test_qwen3_5.py`, `test_qwen3_moe_sglang_converter.py`, `test_vllm_converter.py`
and `test_model_registry.py`, restated on this package's converters.  Tensors are
tiny and carry recognisable values; comparisons have zero tolerance."""

from types import SimpleNamespace

import pytest
import torch

from awex_b200.meta.meta_resolver import get_num_hidden_layers
from awex_b200.models.registry import get_infer_weights_converter, get_sharding_strategy, get_train_weights_converter
from awex_b200.sharding.param_sharding import ShardingType
from awex_b200.sharding.rank_info import RankInfo

MCORE = "module.module."  # Megatron wraps the model twice (DDP, Float16Module)


def ri(tp_rank=0, tp_size=1, **kw):
    return RankInfo.single(tp_rank=tp_rank, tp_size=tp_size, attn_tp_rank=tp_rank, attn_tp_size=tp_size, global_rank=tp_rank,
                           world_size=tp_size, **kw)


# ---- Qwen3-VL ---------------------------------------------------------------------------------------
def vl_configs(tied=False, arch="Qwen3VLForConditionalGeneration"):
    text = SimpleNamespace(hidden_size=8, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=2,
                           num_experts=4, tie_word_embeddings=tied)
    cfg = SimpleNamespace(architectures=[arch], text_config=text, vision_config=SimpleNamespace(num_heads=2, hidden_size=4))
    tf = SimpleNamespace(hidden_size=8, num_attention_heads=4, num_query_groups=2, kv_channels=2, num_layers=2)
    return cfg, tf


def vl_train(cfg, tf, infer_tp=1, rank=None, **conf):
    conf = {"infer_atten_tp_size": infer_tp, "infer_engine_config": SimpleNamespace(tp_size=infer_tp, ep_size=1), **conf}
    return get_train_weights_converter("mcore", cfg.architectures[0], cfg, rank or ri(), conf, tf_config=tf)


def vl_infer(cfg, rank=None, tp=1, ep=1):
    return get_infer_weights_converter("sglang", cfg.architectures[0], cfg, rank or ri(), SimpleNamespace(tp_size=tp, ep_size=ep, device_backend="cpu"))


@pytest.mark.parametrize("arch", ["Qwen3VLForConditionalGeneration", "Qwen3VLMoeForConditionalGeneration"])
def test_vl_dense_and_moe_share_converters_and_strategy(arch):
    cfg, tf = vl_configs(arch=arch)
    dense_cfg, _ = vl_configs()
    assert type(vl_infer(cfg)) is type(vl_infer(dense_cfg))
    assert get_sharding_strategy(arch) is get_sharding_strategy("Qwen3VLForConditionalGeneration")
    conv = vl_train(cfg, tf)
    assert conv.vl_hf_config is cfg and conv.hf_config is cfg.text_config  # decoder facts come from the text part


def test_decoder_depth_is_read_from_flat_or_composite_configs():
    assert get_num_hidden_layers(SimpleNamespace(num_hidden_layers=12)) == 12
    assert get_num_hidden_layers(SimpleNamespace(text_config=SimpleNamespace(num_hidden_layers=28))) == 28
    assert get_num_hidden_layers({"text_config": {"num_hidden_layers": 48}}) == 48
    with pytest.raises(AttributeError, match="num_hidden_layers"):
        get_num_hidden_layers(SimpleNamespace(vision_config=SimpleNamespace()))


def test_vl_language_qkv_parity():
    cfg, tf = vl_configs()
    meg = torch.arange(16 * 8, dtype=torch.float32).reshape(16, 8)
    sent = vl_train(cfg, tf, router_dtype="fp32").convert_param(MCORE + "language_model.decoder.layers.0.self_attention.linear_qkv.weight", meg)
    served = vl_infer(cfg).convert_param("model.layers.0.self_attn.qkv_proj.weight", torch.cat([t for _, t in sent]))
    names = [f"model.language_model.layers.0.self_attn.{p}_proj.weight" for p in "qkv"]
    assert [n for n, _ in sent] == names == [n for n, _ in served]
    for (_, a), (_, b) in zip(sent, served):
        torch.testing.assert_close(a, b, rtol=0, atol=0)


@pytest.mark.parametrize("kind", ["weight", "bias"])
def test_vl_vision_qkv_is_regrouped_per_inference_rank(kind):
    """Megatron keeps [q_h k_h v_h] per head; the tower on two inference ranks wants [Q_r K_r V_r] per rank."""
    cfg, tf = vl_configs()
    tail = (4,) if kind == "weight" else ()
    q, k, v = ([torch.full((2, *tail), base + h) for h in range(2)] for base in (10.0, 20.0, 30.0))
    meg = torch.cat([torch.cat((q[h], k[h], v[h])) for h in range(2)])
    [(name, packed)] = vl_train(cfg, tf, infer_tp=2).convert_param(MCORE + f"vision_model.decoder.layers.1.self_attention.linear_qkv.{kind}", meg)
    assert name == f"model.visual.blocks.1.attn.qkv.{kind}"
    for r, shard in enumerate(packed.chunk(2)):
        torch.testing.assert_close(shard, torch.cat((q[r], k[r], v[r])), rtol=0, atol=0)


@pytest.mark.parametrize("mcore,sglang,canonical", [
    ("vision_model.patch_embed.proj.weight", "visual.patch_embed.proj.weight", "model.visual.patch_embed.proj.weight"),
    ("vision_model.decoder.layers.1.mlp.linear_fc1.weight", "visual.blocks.1.mlp.linear_fc1.weight", "model.visual.blocks.1.mlp.linear_fc1.weight"),
    ("vision_model.merger.linear_fc2.weight", "visual.merger.linear_fc2.weight", "model.visual.merger.linear_fc2.weight"),
    ("vision_model.decoder.deepstack_merger_list.2.patch_norm.weight", "visual.deepstack_merger_list.2.norm.weight",
     "model.visual.deepstack_merger_list.2.norm.weight"),
])
def test_vl_vision_parameters_meet_under_one_name(mcore, sglang, canonical):
    cfg, tf = vl_configs()
    p = torch.arange(8, dtype=torch.float32)
    [(a_name, a)] = vl_train(cfg, tf).convert_param(MCORE + mcore, p)
    [(b_name, b)] = vl_infer(cfg).convert_param(sglang, p)
    assert a_name == b_name == canonical
    torch.testing.assert_close(a, b, rtol=0, atol=0)


def test_vl_experts_are_numbered_globally_over_expert_parallel_ranks():
    cfg, tf = vl_configs()
    conv = vl_train(cfg, tf, rank=ri(ep_rank=1, ep_size=2))
    out = conv.convert_param(MCORE + "language_model.decoder.layers.0.mlp.experts.linear_fc2.weight0", torch.ones(8, 6))
    assert out[0][0] == "model.language_model.layers.0.mlp.experts.2.down_proj.weight"  # 4 experts over 2 ranks: local 0 of rank 1


def test_vl_tied_embedding_is_published_under_both_names_on_both_sides():
    cfg, tf = vl_configs(tied=True)
    e = torch.arange(32, dtype=torch.float32).reshape(4, 8)
    names = ["model.language_model.embed_tokens.weight", "lm_head.weight"]
    assert [n for n, _ in vl_train(cfg, tf).convert_param(MCORE + "language_model.embedding.word_embeddings.weight", e)] == names
    assert [n for n, _ in vl_infer(cfg).convert_param("model.embed_tokens.weight", e)] == names


def vl_strategy(engine):
    return get_sharding_strategy("Qwen3VLForConditionalGeneration")(
        engine_name=engine, enable_dp_attention=False, enable_dp_lm_head=False, moe_dense_tp_size=2, tp_size=2, ep_size=1, ep_tp_size=1,
        rank_info=ri(tp_size=2), device_backend="cpu")


@pytest.mark.parametrize("name,kind,dim", [
    ("model.visual.patch_embed.proj.weight", ShardingType.NO_SHARDING, 0),
    ("model.visual.blocks.0.attn.qkv.weight", ShardingType.TP_SHARDING, 0),
    ("model.visual.blocks.0.attn.proj.weight", ShardingType.TP_SHARDING, 1),
    ("model.visual.deepstack_merger_list.0.linear_fc1.weight", ShardingType.TP_SHARDING, 0),
    ("model.visual.deepstack_merger_list.0.linear_fc2.weight", ShardingType.TP_SHARDING, 1),
    ("model.visual.deepstack_merger_list.0.linear_fc2.bias", ShardingType.NO_SHARDING, 0),
])
def test_vl_vision_tower_sharding_on_the_serving_side(name, kind, dim):
    assert vl_strategy("sglang").get_sharding_strategy(name) == (kind, dim, 2 if kind is ShardingType.TP_SHARDING else 1)


def test_vl_position_embedding_is_whole_in_training_and_split_in_serving():
    name = "model.visual.pos_embed.weight"
    assert vl_strategy("mcore").get_sharding_strategy(name) == (ShardingType.NO_SHARDING, 0, 1)
    assert vl_strategy("sglang").get_sharding_strategy(name) == (ShardingType.TP_SHARDING, 0, 2)


def test_vl_pipeline_stage_renumbers_decoder_layers_only():
    cfg, tf = vl_configs()
    conv = vl_train(cfg, tf, rank=ri(pp_rank=1, pp_size=2), train_pp_stage_layer_id_map={(1, 0): {0: 1}})
    [(language, _)] = conv.convert_param(MCORE + "language_model.decoder.layers.0.self_attention.linear_proj.weight", torch.ones(8, 8))
    [(vision, _)] = conv.convert_param(MCORE + "vision_model.decoder.layers.0.self_attention.linear_proj.weight", torch.ones(4, 4))
    assert language == "model.language_model.layers.1.self_attn.o_proj.weight"
    assert vision == "model.visual.blocks.0.attn.proj.weight"  # the tower lives on one stage and keeps its numbering


def test_vl_unknown_tower_parameter_is_an_error_not_a_guess():
    cfg, tf = vl_configs()
    with pytest.raises(ValueError, match="[Uu]nknown"):
        vl_train(cfg, tf).convert_param(MCORE + "vision_model.unknown.weight", torch.ones(2))


# ---- Qwen3.5 / Qwen3.6 (gated attention + gated delta-net layers, optional vision tower) ----------------
Q35_ARCHS = ["Qwen3_5ForCausalLM", "Qwen3_5MoeForCausalLM", "Qwen3_5ForConditionalGeneration", "Qwen3_5MoeForConditionalGeneration"]


def q35_configs():
    text = SimpleNamespace(model_type="qwen3_5_moe_text", architectures=["Qwen3_5MoeForCausalLM"], hidden_size=8, num_hidden_layers=4,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=2, linear_num_key_heads=2, linear_key_head_dim=2,
                           linear_num_value_heads=4, linear_value_head_dim=2, num_experts=4, tie_word_embeddings=False)
    vl = SimpleNamespace(architectures=["Qwen3_5MoeForConditionalGeneration"], text_config=text,
                         vision_config=SimpleNamespace(num_heads=2, hidden_size=4), tie_word_embeddings=False)
    tf = SimpleNamespace(hidden_size=8, num_attention_heads=4, num_query_groups=2, kv_channels=2, num_layers=4)
    return text, vl, tf


def q35_train(cfg, tf, rank=None, infer_tp=1, **conf):
    conf = {"infer_atten_tp_size": infer_tp, "infer_engine_config": SimpleNamespace(tp_size=infer_tp, ep_size=1), **conf}
    return get_train_weights_converter("mcore", cfg.architectures[0], cfg, rank or ri(), conf, tf_config=tf)


def q35_infer(cfg, arch=None):
    return get_infer_weights_converter("sglang", arch or cfg.architectures[0], cfg, ri(), SimpleNamespace(tp_size=1, ep_size=1, device_backend="cpu"))


def gated_qkv_rows():
    """Megatron layout per KV group: [Q (2 heads), gate (2 heads), K, V]; values name the part and the group."""
    parts = []
    for group in range(2):
        parts += [torch.full((4, 8), 10.0 + group), torch.full((4, 8), 20.0 + group), torch.full((2, 8), 30.0 + group), torch.full((2, 8), 40.0 + group)]
    return torch.cat(parts)


@pytest.mark.parametrize("arch", Q35_ARCHS)
def test_q35_every_architecture_name_gets_the_same_serving_converter(arch):
    _text, vl, _tf = q35_configs()
    assert type(q35_infer(vl, arch)) is type(q35_infer(vl, Q35_ARCHS[0]))


@pytest.mark.parametrize("arch,root,text_type,hidden,layers,heads,kv,value_heads,experts", [
    ("Qwen3_5ForConditionalGeneration", "qwen3_5", "qwen3_5_text", 5120, 64, 24, 4, 48, None),
    ("Qwen3_5MoeForConditionalGeneration", "qwen3_5_moe", "qwen3_5_moe_text", 2048, 40, 16, 2, 32, 256),
])
def test_q36_release_configs_run_on_the_q35_contract(arch, root, text_type, hidden, layers, heads, kv, value_heads, experts):
    text = SimpleNamespace(model_type=text_type, hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                           num_key_value_heads=kv, head_dim=256, linear_num_key_heads=16, linear_key_head_dim=128,
                           linear_num_value_heads=value_heads, linear_value_head_dim=128, num_experts=experts, tie_word_embeddings=False)
    cfg = SimpleNamespace(architectures=[arch], model_type=root, text_config=text,
                          vision_config=SimpleNamespace(num_heads=16, hidden_size=1152), tie_word_embeddings=False)
    conv = q35_infer(cfg)
    assert conv.model_config is text
    assert conv.convert_param("model.layers.0.linear_attn.A_log", torch.ones(value_heads))[0][0] == "model.layers.0.linear_attn.A_log"
    assert conv.convert_param("mtp.norm.weight", torch.ones(hidden)) == []


def test_q35_gated_qkv_is_grouped_per_inference_rank_and_meets_the_serving_layout():
    _text, vl, tf = q35_configs()
    name = MCORE + "language_model.decoder.layers.0.self_attention.linear_qkv.weight"
    [(canonical, packed)] = q35_train(vl, tf, infer_tp=2).convert_param(name, gated_qkv_rows())
    assert canonical == "model.layers.0.self_attn.qkv_proj.weight"
    for r, shard in enumerate(packed.chunk(2)):
        # per rank: [q_h0 gate_h0 q_h1 gate_h1 | K | V] of its KV group
        assert shard[:, 0].tolist() == [v + r for v in (10, 10, 20, 20, 10, 10, 20, 20, 30, 30, 40, 40)]
    [(_, sent)] = q35_train(vl, tf).convert_param(name, gated_qkv_rows())
    [(served_name, served)] = q35_infer(vl).convert_param("model.layers.0.qkv_proj.weight", sent)
    assert served_name == canonical
    torch.testing.assert_close(sent, served, rtol=0, atol=0)


def test_q35_delta_net_input_projection_is_split_into_the_two_fused_serving_tensors():
    _text, vl, tf = q35_configs()
    # rows: Q 4, K 4, V 8, Z 8, B 4, A 4
    out = q35_train(vl, tf).convert_param(MCORE + "language_model.decoder.layers.0.self_attention.in_proj.weight",
                                          torch.arange(32 * 8, dtype=torch.float32).reshape(32, 8))
    assert [(n, t.shape[0]) for n, t in out] == [("model.layers.0.linear_attn.in_proj_qkvz.weight", 24),
                                                 ("model.layers.0.linear_attn.in_proj_ba.weight", 8)]


@pytest.mark.parametrize("name", ["language_model.mtp.layers.0.eh_proj.weight", "mtp.layers.0.mtp_model_layer.mlp.linear_fc1.weight",
                                  "model.mtp.layers.0.final_layernorm.weight"])
def test_q35_multi_token_prediction_weights_are_not_sent(name):
    _text, vl, tf = q35_configs()
    assert q35_train(vl, tf).convert_param(MCORE + name, torch.ones(8, 8)) == []


@pytest.mark.parametrize("name", ["mtp.fc.weight", "model.mtp.layers.0.norm.weight"])
def test_q35_multi_token_prediction_weights_are_not_expected(name):
    _text, vl, _tf = q35_configs()
    assert q35_infer(vl).convert_param(name, torch.ones(8, 8)) == []


def test_q35_pipeline_stage_renumbers_decoder_layers():
    _text, vl, tf = q35_configs()
    conv = q35_train(vl, tf, rank=ri(pp_rank=1, pp_size=2), train_pp_stage_layer_id_map={(1, 0): {0: 3}})
    out = conv.convert_param(MCORE + "language_model.decoder.layers.0.self_attention.linear_proj.weight", torch.ones(8, 8))
    assert out[0][0] == "model.layers.3.self_attn.o_proj.weight"


def test_q35_text_only_and_wrapped_models_share_the_language_names():
    """The serving engine may expose the wrapped multimodal model or its causal-LM part."""
    text, vl, tf = q35_configs()
    name, p = "model.layers.0.linear_attn.out_proj.weight", torch.ones(8, 8)
    sent = q35_train(vl, tf).convert_param(MCORE + "language_model.decoder.layers.0.self_attention.out_proj.weight", p)
    for got in (sent, q35_infer(vl).convert_param(name, p), q35_infer(text).convert_param(name, p)):
        assert [n for n, _ in got] == [name] and torch.equal(got[0][1], p)


@pytest.mark.parametrize("mcore,canonical", [
    ("vision_model.patch_embed.proj.weight", "model.visual.patch_embed.proj.weight"),
    ("vision_model.patch_embed.proj.bias", "model.visual.patch_embed.proj.bias"),
    ("vision_model.pos_embed.weight", "model.visual.pos_embed.weight"),
    ("vision_model.merger.patch_norm.weight", "model.visual.merger.norm.weight"),
    ("vision_model.merger.patch_norm.bias", "model.visual.merger.norm.bias"),
    ("vision_model.merger.linear_fc1.weight", "model.visual.merger.linear_fc1.weight"),
    ("vision_model.merger.linear_fc1.bias", "model.visual.merger.linear_fc1.bias"),
    ("vision_model.merger.linear_fc2.weight", "model.visual.merger.linear_fc2.weight"),
    ("vision_model.merger.linear_fc2.bias", "model.visual.merger.linear_fc2.bias"),
])
def test_q35_vision_tower_names(mcore, canonical):
    _text, vl, tf = q35_configs()
    p = torch.ones(4)
    [(name, value)] = q35_train(vl, tf).convert_param(MCORE + mcore, p)
    assert name == canonical and torch.equal(value, p)


def test_q35_vision_block_names_meet_the_serving_names():
    _text, vl, tf = q35_configs()
    p = torch.ones(4, 4)
    sent = q35_train(vl, tf).convert_param(MCORE + "vision_model.decoder.layers.2.self_attention.linear_proj.weight", p)
    served = q35_infer(vl).convert_param("visual.blocks.2.attn.proj.weight", p)
    assert sent[0][0] == served[0][0] == "model.visual.blocks.2.attn.proj.weight"


def q35_strategy(tp, ep, dense_tp):
    return get_sharding_strategy("Qwen3_5MoeForCausalLM")(
        engine_name="sglang", enable_dp_attention=False, enable_dp_lm_head=False, moe_dense_tp_size=dense_tp, tp_size=tp, ep_size=ep,
        ep_tp_size=1, rank_info=ri(tp_size=tp, ep_size=ep), device_backend="cpu")


@pytest.mark.parametrize("name,expected", [
    ("model.layers.0.self_attn.qkv_proj.weight", (ShardingType.TP_SHARDING, 0, 2)),
    ("model.layers.0.linear_attn.out_proj.weight", (ShardingType.TP_SHARDING, 1, 2)),
    ("model.layers.0.mlp.experts.0.down_proj.weight", (ShardingType.EP_SHARDING, 1, 2)),
    ("model.layers.0.mlp.shared_expert.down_proj.weight", (ShardingType.TP_SHARDING, 1, 2)),
    ("model.visual.blocks.0.attn.qkv.weight", (ShardingType.TP_SHARDING, 0, 2)),
])
def test_q35_sharding_of_attention_experts_and_tower(name, expected):
    assert q35_strategy(2, 2, 2).get_sharding_strategy(name) == expected


def test_q35_experts_stay_expert_parallel_when_dense_layers_are_not_split():
    assert q35_strategy(1, 2, 1).get_sharding_strategy("model.layers.0.mlp.experts.0.gate_proj.weight") == (ShardingType.EP_SHARDING, 0, 2)


# ---- Qwen3-MoE: what the serving engine holds vs what the trainer sends ------------------------------------
H, NH, NKV, HD, NE, MI = 16, 4, 2, 4, 4, 8


def q3moe_cfg():
    return SimpleNamespace(architectures=["Qwen3MoeForCausalLM"], hidden_size=H, num_attention_heads=NH, num_key_value_heads=NKV,
                           head_dim=HD, num_experts=NE, moe_intermediate_size=MI, num_hidden_layers=1, tie_word_embeddings=False)


def q3moe_serving(tp=1, ep=1, ep_rank=0, engine="sglang"):
    return get_infer_weights_converter(engine, "Qwen3MoeForCausalLM", q3moe_cfg(), ri(0, tp, ep_rank=ep_rank, ep_size=ep),
                                       SimpleNamespace(tp_size=tp, ep_size=ep, device_backend="cuda"))


def serving_params(local_experts=NE):
    """One decoder layer as a serving engine exposes it (fused QKV, fused expert stacks)."""
    return {
        "model.embed_tokens.weight": torch.randn(32, H), "model.layers.0.self_attn.qkv_proj.weight": torch.randn((NH + 2 * NKV) * HD, H),
        "model.layers.0.self_attn.o_proj.weight": torch.randn(H, NH * HD), "model.layers.0.self_attn.q_norm.weight": torch.randn(HD),
        "model.layers.0.self_attn.k_norm.weight": torch.randn(HD), "model.layers.0.input_layernorm.weight": torch.randn(H),
        "model.layers.0.post_attention_layernorm.weight": torch.randn(H), "model.layers.0.mlp.gate.weight": torch.randn(NE, H),
        "model.layers.0.mlp.experts.w13_weight": torch.randn(local_experts, 2 * MI, H),
        "model.layers.0.mlp.experts.w2_weight": torch.randn(local_experts, H, MI), "model.norm.weight": torch.randn(H),
        "lm_head.weight": torch.randn(32, H),
    }


def training_params(local_experts=NE):
    """The same layer as Megatron holds it on one rank (interleaved QKV, grouped-GEMM experts)."""
    p = "decoder.layers.0."
    out = {
        "embedding.word_embeddings.weight": (32, H), p + "self_attention.linear_qkv.weight": ((NH + 2 * NKV) * HD, H),
        p + "self_attention.linear_proj.weight": (H, NH * HD), p + "self_attention.q_layernorm.weight": (HD,),
        p + "self_attention.k_layernorm.weight": (HD,), p + "self_attention.linear_qkv.layer_norm_weight": (H,),
        p + "pre_mlp_layernorm.weight": (H,), p + "mlp.router.weight": (NE, H), "decoder.final_layernorm.weight": (H,),
        "output_layer.weight": (32, H),
    }
    for e in range(local_experts):
        out[p + f"mlp.experts.linear_fc1.weight{e}"] = (2 * MI, H)
        out[p + f"mlp.experts.linear_fc2.weight{e}"] = (H, MI)
    return out


def canonical_names(expert_ids):
    names = {"model.embed_tokens.weight", "model.norm.weight", "lm_head.weight", "model.layers.0.mlp.gate.weight",
             "model.layers.0.input_layernorm.weight", "model.layers.0.post_attention_layernorm.weight"}
    names |= {f"model.layers.0.self_attn.{p}.weight" for p in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")}
    names |= {f"model.layers.0.mlp.experts.{e}.{p}_proj.weight" for e in expert_ids for p in ("gate", "up", "down")}
    return names


@pytest.mark.parametrize("ep,ep_rank", [(1, 0), (2, 1)])
def test_q3moe_both_sides_publish_one_name_set_with_global_expert_ids(ep, ep_rank):
    local = NE // ep
    experts = range(ep_rank * local, (ep_rank + 1) * local)
    serving = q3moe_serving(ep=ep, ep_rank=ep_rank)
    served = {n for name, p in serving_params(local).items() for n, _ in serving.convert_param(name, p)}
    assert served == canonical_names(experts)
    conf = {"infer_atten_tp_size": 1, "router_dtype": "fp32", "infer_engine_config": SimpleNamespace(tp_size=1, ep_size=ep)}
    tf = SimpleNamespace(hidden_size=H, num_attention_heads=NH, num_query_groups=NKV, kv_channels=HD, num_layers=1, num_moe_experts=NE)
    trainer = get_train_weights_converter("mcore", "Qwen3MoeForCausalLM", q3moe_cfg(), ri(ep_rank=ep_rank, ep_size=ep), conf, tf_config=tf)
    sent = {s.name for name, shape in training_params(local).items() for s in trainer.plan_param(name, shape, torch.bfloat16)}
    assert sent == served


def test_q3moe_vllm_reuses_the_registered_serving_converter():
    """One canonical contract per architecture whatever the serving engine (the
    reference falls back to a generic vLLM converter whose names do not meet the trainer's)."""
    assert type(q3moe_serving(engine="vllm")) is type(q3moe_serving(engine="sglang"))


def test_q3moe_fused_qkv_is_split_by_head_counts_or_refused():
    q, k, v = torch.randn(NH * HD, H), torch.randn(NKV * HD, H), torch.randn(NKV * HD, H)
    out = dict(q3moe_serving().convert_param("model.layers.0.self_attn.qkv_proj.weight", torch.cat([q, k, v])))
    assert torch.equal(out["model.layers.0.self_attn.q_proj.weight"], q)
    assert torch.equal(out["model.layers.0.self_attn.k_proj.weight"], k) and torch.equal(out["model.layers.0.self_attn.v_proj.weight"], v)
    with pytest.raises(ValueError, match="not divisible"):
        q3moe_serving().convert_param("model.layers.0.self_attn.qkv_proj.weight", torch.randn((NH + 2 * NKV) * HD + 1, H))


def test_q3moe_expert_stacks_are_exposed_as_views_per_expert():
    w13, w2 = torch.randn(NE, 2 * MI, H), torch.randn(NE, H, MI)
    gate_up = dict(q3moe_serving().convert_param("model.layers.0.mlp.experts.w13_weight", w13))
    down = dict(q3moe_serving().convert_param("model.layers.0.mlp.experts.w2_weight", w2))
    for e in range(NE):
        gate, up = gate_up[f"model.layers.0.mlp.experts.{e}.gate_proj.weight"], gate_up[f"model.layers.0.mlp.experts.{e}.up_proj.weight"]
        assert torch.equal(gate, w13[e, :MI]) and torch.equal(up, w13[e, MI:]) and torch.equal(down[f"model.layers.0.mlp.experts.{e}.down_proj.weight"], w2[e])
        # views, not copies: received data lands in the engine's own buffers
        assert gate.data_ptr() == w13[e].data_ptr() and up.data_ptr() == w13[e, MI:].data_ptr()


# ---- generic vLLM names, Bailing registry entries, MLA packing -------------------------------------------
@pytest.mark.parametrize("name,canonical", [
    ("model.layers.0.self_attn.qkv_proj.weight", "model.layers.0.attention.query_key_value_proj.weight"),
    ("model.layers.0.self_attn.qkv.weight", "model.layers.0.attention.query_key_value_proj.weight"),  # GLM-4V spelling
    ("model.layers.0.self_attn.o_proj.weight", "model.layers.0.attention.dense.weight"),
    ("model.layers.0.self_attn.proj.weight", "model.layers.0.attention.dense.weight"),  # GLM-4V spelling
])
def test_generic_vllm_attention_names(name, canonical):
    from awex_b200.config import InferenceConfig
    from awex_b200.converter.vllm_converter import VLLMToHFWeightConverter

    conv = VLLMToHFWeightConverter(SimpleNamespace(num_attention_heads=8, num_key_value_heads=8), InferenceConfig(tp_size=1, ep_size=1), ri())
    w = torch.zeros(12, 12)
    [(got, value)] = conv.convert_param(name, w)
    assert got == canonical and value is w


@pytest.mark.parametrize("arch,tf", [("BailingMoeForCausalLM", SimpleNamespace()), ("BailingMoeV2_5ForCausalLM", SimpleNamespace(layer_group_size=4))])
def test_bailing_train_converters_keep_the_transformer_config(arch, tf):
    cfg = SimpleNamespace(architectures=[arch], quantization_config={})
    conv = get_train_weights_converter("mcore", arch, cfg, ri(), {"infer_atten_tp_size": 1}, tf_config=tf)
    assert conv.tf_config is tf


def test_bailing_linear_sharding_knows_the_mla_exceptions():
    strategy = get_sharding_strategy("BailingMoeV2_5ForCausalLM")(
        engine_name="sglang", enable_dp_attention=False, enable_dp_lm_head=False, moe_dense_tp_size=2, tp_size=2, ep_size=1, ep_tp_size=1,
        rank_info=ri(tp_size=2))
    assert strategy.get_sharding_strategy("model.layers.0.attention.g_norm.weight") == (ShardingType.TP_SHARDING, 0, 2)
    assert strategy.get_sharding_strategy("model.layers.0.attention.kv_a_proj_with_mqa.weight") == (ShardingType.NO_SHARDING, 0, 1)


def mla_q_kv():
    return torch.arange(24, dtype=torch.float32).reshape(8, 3), -torch.arange(12, dtype=torch.float32).reshape(4, 3)


@pytest.mark.parametrize("tp", [1, 2, 4])
def test_mla_down_projections_are_packed_so_that_every_rank_slice_is_its_own_pair(tp):
    from awex_b200.converter.mcore_converter import pack_fused_qkv_a_proj_for_tp

    q, kv = mla_q_kv()
    packed = pack_fused_qkv_a_proj_for_tp(q, kv, tp)
    assert packed.shape == (12, 3)
    for r, shard in enumerate(packed.chunk(tp)):
        assert torch.equal(shard, torch.cat([q.chunk(tp)[r], kv.chunk(tp)[r]]))
    assert torch.equal(packed, torch.cat([q, kv])) == (tp == 1)  # beyond one rank the plain concatenation would corrupt attention
    # order preserving and invertible
    assert torch.equal(torch.cat([s[: 8 // tp] for s in packed.chunk(tp)]), q)
    assert torch.equal(torch.cat([s[8 // tp:] for s in packed.chunk(tp)]), kv)


@pytest.mark.parametrize("bad", ["tp0", "q_rows", "kv_rows", "columns", "one_dim"])
def test_mla_packing_refuses_shapes_it_cannot_split(bad):
    from awex_b200.converter.mcore_converter import pack_fused_qkv_a_proj_for_tp

    q, kv = mla_q_kv()
    tp = 0 if bad == "tp0" else 4
    q = torch.zeros(7, 3) if bad == "q_rows" else torch.zeros(8) if bad == "one_dim" else q
    kv = torch.zeros(3, 3) if bad == "kv_rows" else torch.zeros(4, 4) if bad == "columns" else kv
    with pytest.raises(ValueError):
        pack_fused_qkv_a_proj_for_tp(q, kv, tp)
