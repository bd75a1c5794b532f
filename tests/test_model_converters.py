"""Converter contracts of the registered architectures: names, layouts and
train/infer parity with zero tolerance, on synthetic tensors whose rows carry
their own identity."""

from types import SimpleNamespace

import pytest
import torch

from awex_b200.converter.mcore_converter import pack_fused_qkv_a_proj_for_tp
from awex_b200.models.registry import ModelRegistry, get_infer_weights_converter, get_sharding_strategy, get_train_weights_converter
from awex_b200.sharding.param_sharding import ShardingStrategy, ShardingType
from awex_b200.sharding.rank_info import RankInfo

ARCHS = [
    "BailingMoeForCausalLM", "BailingMoeV2ForCausalLM", "BailingMoeLinearForCausalLM", "BailingMoeV2_5ForCausalLM",
    "BailingMoeV2_5ForCausalLMNextN", "Qwen3ForCausalLM", "Qwen3MoeForCausalLM", "Qwen3VLForConditionalGeneration",
    "Qwen3VLMoeForConditionalGeneration", "Qwen3_5ForCausalLM", "Qwen3_5MoeForCausalLM",
    "Qwen3_5ForConditionalGeneration", "Qwen3_5MoeForConditionalGeneration",
]


def ri(tp_rank=0, tp_size=1, **kw):
    return RankInfo.single(tp_rank=tp_rank, tp_size=tp_size, attn_tp_rank=tp_rank, attn_tp_size=tp_size, global_rank=tp_rank,
                           world_size=tp_size, **kw)


def rows_tensor(n, cols=3, base=0):
    """[n, cols] tensor whose row i holds base + i in every column."""
    return (torch.arange(n, dtype=torch.float32) + base).unsqueeze(1).repeat(1, cols)


def test_registry_lists_thirteen_architectures_and_defaults():
    assert sorted(ModelRegistry.get_registered_models()) == sorted(ARCHS)
    assert get_sharding_strategy("LlamaForCausalLM") is ShardingStrategy
    conv = get_infer_weights_converter("vllm", "LlamaForCausalLM", SimpleNamespace(num_attention_heads=4, num_key_value_heads=2),
                                       ri(), SimpleNamespace(tp_size=1, ep_size=1))
    out = conv.convert_param("model.layers.0.self_attn.qkv_proj.weight", torch.zeros(8, 2))
    assert [n for n, _ in out] == ["model.layers.0.attention.query_key_value_proj.weight"]


def qwen35_cfg():
    return SimpleNamespace(architectures=["Qwen3_5ForCausalLM"], num_attention_heads=4, num_key_value_heads=2, head_dim=2,
                           hidden_size=8, num_hidden_layers=2, linear_num_key_heads=2, linear_key_head_dim=2,
                           linear_num_value_heads=4, linear_value_head_dim=2, num_experts=4)


def train_conv(arch, cfg, rank_info, infer_tp, tf=None):
    tf = tf or SimpleNamespace(hidden_size=cfg.hidden_size, num_attention_heads=cfg.num_attention_heads,
                               num_query_groups=cfg.num_key_value_heads, kv_channels=getattr(cfg, "head_dim", None), num_layers=2)
    conf = {"infer_atten_tp_size": infer_tp, "router_dtype": "fp32", "infer_engine_config": SimpleNamespace(tp_size=infer_tp, ep_size=1)}
    return get_train_weights_converter("mcore", arch, cfg, rank_info, conf, tf_config=tf)


def test_qwen35_gated_qkv_is_q_with_gate_then_k_then_v_per_infer_rank():
    cfg = qwen35_cfg()  # 2 KV groups, 2 query heads per group, head_dim 2
    hd, qpg = 2, 2
    # label rows: kind*100 + head*10 + r ; kinds: q=1 gate=2 k=3 v=4
    def head_rows(kind, head):
        return torch.tensor([[kind * 100 + head * 10 + r] for r in range(hd)], dtype=torch.float32)
    groups = []
    for g in range(2):
        q = torch.cat([head_rows(1, g * qpg + h) for h in range(qpg)])
        gate = torch.cat([head_rows(2, g * qpg + h) for h in range(qpg)])
        groups.append(torch.cat([q, gate, head_rows(3, g), head_rows(4, g)]))
    megatron = torch.cat(groups)
    conv = train_conv("Qwen3_5ForCausalLM", cfg, ri(), infer_tp=2)
    (name, fused), = conv.convert_param("decoder.layers.0.self_attention.linear_qkv.weight", megatron)
    assert name == "model.layers.0.self_attn.qkv_proj.weight"
    want = []
    for r in range(2):  # inference rank r: its 2 query heads (each followed by its gate), KV head r
        for head in (2 * r, 2 * r + 1):
            want += [head_rows(1, head), head_rows(2, head)]
        want += [head_rows(3, r), head_rows(4, r)]
    assert torch.equal(fused, torch.cat(want))
    # KV heads are repeated when the inference TP exceeds their number
    conv4 = train_conv("Qwen3_5ForCausalLM", cfg, ri(), infer_tp=4)
    (_, fused4), = conv4.convert_param("decoder.layers.0.self_attention.linear_qkv.weight", megatron)
    per_rank = fused4.view(4, -1)
    assert per_rank[0, -4:].tolist() == per_rank[1, -4:].tolist() == [300.0, 301.0, 400.0, 401.0]


def test_qwen35_gdn_input_and_conv_follow_inference_rank_order():
    cfg = qwen35_cfg()
    qk, val, vh = 4, 8, 4
    cats = [rows_tensor(n, 1, base=1000 * (i + 1)) for i, n in enumerate((qk, qk, val, val, vh, vh))]
    train_tp = 2
    full = torch.cat([torch.cat([c.chunk(train_tp)[r] for c in cats]) for r in range(train_tp)])
    from awex_b200.models.qwen3_5 import _Qwen3_5Layout

    qkvz, ba = _Qwen3_5Layout.pack_gdn_input(full, cfg, train_tp, 2)
    for r in range(2):
        assert torch.equal(qkvz.chunk(2)[r], torch.cat([c.chunk(2)[r] for c in cats[:4]]))
        assert torch.equal(ba.chunk(2)[r], torch.cat([c.chunk(2)[r] for c in cats[4:]]))
    conv_cats = cats[:3]
    conv_full = torch.cat([torch.cat([c.chunk(train_tp)[r] for c in conv_cats]) for r in range(train_tp)])
    packed = _Qwen3_5Layout.pack_gdn_conv(conv_full, cfg, train_tp, 4)
    for r in range(4):
        assert torch.equal(packed.chunk(4)[r], torch.cat([c.chunk(4)[r] for c in conv_cats]))


def test_qwen35_names_values_and_frozen_mtp():
    cfg = qwen35_cfg()
    conv = train_conv("Qwen3_5MoeForCausalLM", cfg, ri(), infer_tp=1)
    w = torch.full((4,), 0.5)
    assert conv.convert_param("language_model.mtp.layers.0.x.weight", w) == []
    (n, t), = conv.convert_param("language_model.decoder.layers.1.self_attention.out_norm.weight", w)
    assert n == "model.layers.1.linear_attn.norm.weight" and torch.equal(t, w + 1.0)
    (n, _), = conv.convert_param("decoder.layers.1.self_attention.A_log", w)
    assert n == "model.layers.1.linear_attn.A_log"
    names = [n for n, _ in conv.convert_param("decoder.layers.0.mlp.shared_experts.linear_fc1.weight", torch.zeros(8, 8))]
    assert names == ["model.layers.0.mlp.shared_expert.gate_proj.weight", "model.layers.0.mlp.shared_expert.up_proj.weight"]
    infer = get_infer_weights_converter("sglang", "Qwen3_5MoeForCausalLM", cfg, ri(), SimpleNamespace(tp_size=1, ep_size=1))
    assert infer.convert_param("mtp.fc.weight", w) == []
    assert infer.convert_param("model.language_model.layers.0.qkv_proj.weight", torch.zeros(12, 8))[0][0] == "model.layers.0.self_attn.qkv_proj.weight"
    assert infer.convert_param("model.layers.0.mlp.shared_experts.down_proj.weight", torch.zeros(8, 8))[0][0] == "model.layers.0.mlp.shared_expert.down_proj.weight"
    strat = get_sharding_strategy("Qwen3_5MoeForCausalLM")("sglang", False, False, None, 2, 2, 1, ri(tp_size=2))
    assert strat.get_sharding_strategy("model.layers.0.linear_attn.out_proj.weight") == (ShardingType.TP_SHARDING, 1, 2)
    assert strat.get_sharding_strategy("model.layers.0.linear_attn.norm.weight")[0] == ShardingType.NO_SHARDING


def test_qwen3_gqa_split_matches_inference_split():
    cfg = SimpleNamespace(architectures=["Qwen3ForCausalLM"], num_attention_heads=8, num_key_value_heads=4, head_dim=2, hidden_size=16,
                          num_hidden_layers=1)
    hd, qpg = 2, 2
    q, k, v = rows_tensor(16, 2, 100), rows_tensor(8, 2, 200), rows_tensor(8, 2, 300)
    for tp in (1, 2):
        trained, served = {}, {}
        for r in range(tp):
            groups = range(r * 4 // tp, (r + 1) * 4 // tp)
            meg = torch.cat([torch.cat([q[g * qpg * hd:(g + 1) * qpg * hd], k[g * hd:(g + 1) * hd], v[g * hd:(g + 1) * hd]]) for g in groups])
            for n, t in train_conv("Qwen3ForCausalLM", cfg, ri(r, tp), infer_tp=tp).convert_param("decoder.layers.0.self_attention.linear_qkv.weight", meg):
                trained.setdefault(n, []).append(t)
            fused = torch.cat([q.chunk(tp)[r], k.chunk(tp)[r], v.chunk(tp)[r]])
            infer = get_infer_weights_converter("sglang", "Qwen3ForCausalLM", cfg, ri(r, tp), SimpleNamespace(tp_size=tp, ep_size=1))
            for n, t in infer.convert_param("model.layers.0.self_attn.qkv_proj.weight", fused):
                served.setdefault(n, []).append(t)
        assert sorted(trained) == sorted(served) == [f"model.layers.0.self_attn.{p}_proj.weight" for p in "kqv"]
        for n in trained:
            torch.testing.assert_close(torch.cat(trained[n]), torch.cat(served[n]), rtol=0, atol=0)


def test_mla_fused_a_proj_chunks_are_q_then_kv():
    q, kv = rows_tensor(8, 2, 0), rows_tensor(4, 2, 100)
    packed = pack_fused_qkv_a_proj_for_tp(q, kv, 4)
    for i, chunk in enumerate(packed.chunk(4)):
        assert torch.equal(chunk, torch.cat([q.chunk(4)[i], kv.chunk(4)[i]]))
    with pytest.raises(ValueError):
        pack_fused_qkv_a_proj_for_tp(q, kv, 3)
    with pytest.raises(ValueError):
        pack_fused_qkv_a_proj_for_tp(q, rows_tensor(4, 3), 2)


def test_qwen3_vl_namespaces_and_vision_qkv():
    text = SimpleNamespace(num_attention_heads=4, num_key_value_heads=2, head_dim=2, hidden_size=8, num_hidden_layers=1,
                           tie_word_embeddings=True)
    cfg = SimpleNamespace(architectures=["Qwen3VLForConditionalGeneration"], text_config=text,
                          vision_config=SimpleNamespace(num_heads=2, hidden_size=4), num_hidden_layers=1)
    conv = train_conv("Qwen3VLForConditionalGeneration", cfg, ri(), infer_tp=2,
                      tf=SimpleNamespace(hidden_size=8, num_attention_heads=4, num_query_groups=2, kv_channels=2, num_layers=1))
    emb = torch.zeros(10, 8)
    assert [n for n, _ in conv.convert_param("language_model.embedding.word_embeddings.weight", emb)] == [
        "model.language_model.embed_tokens.weight", "lm_head.weight"]
    assert conv.convert_param("vision_model.merger.patch_norm.weight", torch.zeros(4))[0][0] == "model.visual.merger.norm.weight"
    assert conv.convert_param("vision_model.decoder.deepstack_merger_list.1.linear_fc2.weight", torch.zeros(4, 4))[0][0] == \
        "model.visual.deepstack_merger_list.1.linear_fc2.weight"
    # vision MHA with 2 heads of size 2, Megatron order [q0 k0 v0 q1 k1 v1] -> per inference rank [Q_r K_r V_r]
    meg = rows_tensor(12, 1)
    (n, t), = conv.convert_param("vision_model.decoder.layers.3.self_attention.linear_qkv.weight", meg)
    assert n == "model.visual.blocks.3.attn.qkv.weight"
    assert t.view(-1).tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11]  # one head per group and per rank: identity here
    with pytest.raises(ValueError):
        conv.convert_param("audio_model.x", emb)
    strat = get_sharding_strategy("Qwen3VLForConditionalGeneration")("sglang", False, False, None, 2, 1, 1, ri(tp_size=2))
    assert strat.get_sharding_strategy("model.visual.blocks.0.attn.proj.weight") == (ShardingType.TP_SHARDING, 1, 2)
    assert strat.get_sharding_strategy("model.visual.blocks.0.attn.proj.bias")[0] == ShardingType.NO_SHARDING
    assert strat.get_sharding_strategy("model.visual.pos_embed.weight")[0] == ShardingType.TP_SHARDING
    mc = get_sharding_strategy("Qwen3VLForConditionalGeneration")("mcore", False, False, None, 2, 1, 1, ri(tp_size=2))
    assert mc.get_sharding_strategy("model.visual.pos_embed.weight")[0] == ShardingType.NO_SHARDING


def test_bailing_fp8_keys_and_power_of_two_scales():
    cfg = SimpleNamespace(architectures=["BailingMoeForCausalLM"], num_attention_heads=4, num_key_value_heads=4, hidden_size=256,
                          num_hidden_layers=1, num_experts=2, quantization_config={"quant_method": "fp8"})
    conv = train_conv("BailingMoeForCausalLM", cfg, ri(), infer_tp=1,
                      tf=SimpleNamespace(hidden_size=256, num_attention_heads=4, num_query_groups=4, kv_channels=64, num_layers=1))
    def ops(name, shape):
        return {s.name: s.value_op for s in conv.plan_param(name, shape, torch.bfloat16)}
    dense = ops("decoder.layers.0.self_attention.linear_proj.weight", (256, 256))
    assert dense["model.layers.0.attention.dense.weight"].kind == "fp8_block" and dense["model.layers.0.attention.dense.weight"].ue8m0
    assert "model.layers.0.attention.dense.weight_scale_inv" in dense
    expert = ops("decoder.layers.0.mlp.experts.local_experts.1.linear_fc1.weight", (256, 256))
    assert expert["model.layers.0.mlp.experts.1.gate_proj.weight"].ue8m0
    down = ops("decoder.layers.0.mlp.experts.local_experts.1.linear_fc2.weight", (256, 128))
    assert down["model.layers.0.mlp.experts.1.down_proj.weight"].kind == "fp8_block" and not down["model.layers.0.mlp.experts.1.down_proj.weight"].ue8m0
    mlp = ops("decoder.layers.0.mlp.linear_fc1.weight", (256, 256))
    assert mlp["model.layers.0.mlp.gate_proj.weight"].kind == "fp8_block" and not mlp["model.layers.0.mlp.gate_proj.weight"].ue8m0
    norm = ops("decoder.layers.0.self_attention.linear_qkv.layer_norm_weight", (256,))
    assert norm["model.layers.0.input_layernorm.weight"].kind == "none"
    # materialised form equals quantising the converted tensor
    from awex_b200.converter.weights_converter import per_block_cast_to_fp8
    w = torch.randn(256, 256).to(torch.bfloat16)
    got = dict(conv.convert_param("decoder.layers.0.self_attention.linear_proj.weight", w))
    q, s = per_block_cast_to_fp8(w, True)
    assert torch.equal(got["model.layers.0.attention.dense.weight"].view(torch.uint8), q.view(torch.uint8))
    assert torch.equal(got["model.layers.0.attention.dense.weight_scale_inv"], s)


def test_bailing_linear_serves_lm_head_in_fp32_and_quantises_routed_experts_only():
    cfg = SimpleNamespace(architectures=["BailingMoeV2ForCausalLM"], num_attention_heads=4, num_key_value_heads=4, hidden_size=256,
                          num_hidden_layers=4, num_experts=2, layer_group_size=4, quantization_config={"quant_method": "fp8"}, q_lora_rank=None)
    conv = train_conv("BailingMoeV2ForCausalLM", cfg, ri(), infer_tp=1,
                      tf=SimpleNamespace(hidden_size=256, num_attention_heads=4, num_query_groups=4, kv_channels=64, num_layers=4))
    (spec,) = conv.plan_param("output_layer.weight", (100, 256), torch.bfloat16)
    assert spec.dtype == torch.float32
    shared = {s.name: s.value_op.kind for s in conv.plan_param("decoder.layers.0.mlp.shared_experts.linear_fc1.weight", (256, 256), torch.bfloat16)}
    assert set(shared.values()) == {"none"}
    routed = {s.name: s.value_op for s in conv.plan_param("decoder.layers.0.mlp.experts.local_experts.0.linear_fc1.weight", (256, 256), torch.bfloat16)}
    assert routed["model.layers.0.mlp.experts.0.up_proj.weight"].kind == "fp8_block" and not routed["model.layers.0.mlp.experts.0.up_proj.weight"].ue8m0
    # layer 0 of a group of 4 is Lightning attention, layer 3 is MLA
    assert conv.plan_param("decoder.layers.0.self_attention.linear_gate.weight", (256, 256), torch.bfloat16)[0].name == "model.layers.0.attention.g_proj.weight"
    assert conv.plan_param("decoder.layers.3.self_attention.linear_kv_up_proj.weight", (256, 64), torch.bfloat16)[0].name == "model.layers.3.attention.kv_b_proj.weight"
    assert conv.plan_param("decoder.layers.0.self_attention.pre_gate_norm.te_norm.weight", (256,), torch.bfloat16) == []
    strat = get_sharding_strategy("BailingMoeV2ForCausalLM")("sglang", False, False, None, 2, 1, 1, ri(tp_size=2))
    assert strat.get_sharding_strategy("model.layers.3.attention.q_a_proj.weight")[0] == ShardingType.NO_SHARDING
    assert strat.get_sharding_strategy("model.layers.0.attention.g_norm.weight") == (ShardingType.TP_SHARDING, 0, 2)


def test_a_registered_training_tp_group_wins_over_an_importable_megatron(monkeypatch):
    """A host program that registers its training TP group gets that group, even
    where a ``megatron`` package imports and answers something else."""
    import sys
    from types import ModuleType

    from awex_b200.converter import mcore_converter as mc

    state = ModuleType("megatron.core.parallel_state")
    state.get_tensor_model_parallel_group = lambda: "megatron-group"
    state.get_tensor_model_parallel_world_size = lambda: 4
    core = ModuleType("megatron.core")
    core.parallel_state = state
    top = ModuleType("megatron")
    top.core = core
    for name, module in (("megatron", top), ("megatron.core", core), ("megatron.core.parallel_state", state)):
        monkeypatch.setitem(sys.modules, name, module)
    monkeypatch.setitem(mc._TRAIN_TP_GROUP, "group", None)
    monkeypatch.setitem(mc._TRAIN_TP_GROUP, "size", 1)
    assert mc._train_tp_group() == ("megatron-group", 4)  # nothing registered: Megatron's
    mc.set_train_tp_group("registered", 2)
    assert mc._train_tp_group() == ("registered", 2)
    monkeypatch.delitem(sys.modules, "megatron.core.parallel_state")
    monkeypatch.delitem(sys.modules, "megatron.core")
    monkeypatch.delitem(sys.modules, "megatron")
    monkeypatch.setitem(mc._TRAIN_TP_GROUP, "group", None)
    monkeypatch.setitem(mc._TRAIN_TP_GROUP, "size", 1)
    assert mc._train_tp_group() == (None, 1)  # neither: a single rank
