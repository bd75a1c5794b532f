"""Sharding rules, rank-info extraction from engine contexts, and the vLLM name
normalisation: both ends of an exchange must classify every name identically."""

from types import SimpleNamespace

import pytest
import torch

from awex_b200.sharding.param_sharding import LinearMLAShardingMixin, ShardingStrategy, ShardingType, get_default_sharding_dim
from awex_b200.sharding.rank_info import RankInfo


def rank_info(tp=4, tp_rank=0, attn_tp=None, ep=1, etp=1, cp=1, infer=True):
    attn_tp = tp if attn_tp is None else attn_tp
    return RankInfo(tp_rank=tp_rank, tp_size=tp, pp_rank=0, pp_size=1, dp_size=1, dp_rank=0, ep_rank=0, ep_size=ep, ep_tp_rank=0,
                    ep_tp_size=etp, attn_tp_rank=tp_rank % attn_tp, attn_tp_size=attn_tp, attn_dp_rank=0, world_size=tp * cp,
                    global_rank=tp_rank, local_rank=tp_rank, engine_rank=0, is_infer=infer, cp_rank=0, cp_size=cp,
                    cp_mode="ring" if cp > 1 else "none")


def strategy(ri, engine="sglang", dp_attention=False, dp_lm_head=False, cls=ShardingStrategy):
    return cls(engine, dp_attention, dp_lm_head, None, ri.tp_size, ri.ep_size, ri.ep_tp_size, ri)


def test_default_shard_dimensions():
    for name, dim in [("model.layers.0.self_attn.o_proj.weight", 1), ("model.layers.0.attention.dense.weight", 1),
                      ("model.layers.0.mlp.down_proj.weight", 1), ("model.layers.0.mlp.experts.w2_weight", 1),
                      ("model.layers.0.mlp.down_proj.weight_scale_inv", 1), ("model.layers.0.self_attn.q_proj.weight", 0),
                      ("model.layers.0.mlp.gate_up_proj.weight", 0), ("lm_head.weight", 0), ("model.embed_tokens.weight", 0),
                      ("something.unknown", 0), ("model.layers.0.mlp.down_proj.bias", 0)]:
        assert get_default_sharding_dim(name) == dim, name


def test_name_routing_with_tensor_parallelism():
    s = strategy(rank_info(tp=4))
    for name, want in [
        ("model.layers.0.input_layernorm.weight", (ShardingType.NO_SHARDING, 0, 1)),
        ("model.embed_tokens.weight", (ShardingType.TP_SHARDING, 0, 4)),
        ("lm_head.weight", (ShardingType.TP_SHARDING, 0, 4)),
        ("model.layers.0.attention.dense.weight", (ShardingType.TP_SHARDING, 1, 4)),
        ("model.layers.0.mlp.gate_proj.weight", (ShardingType.TP_SHARDING, 0, 4)),
        ("model.layers.0.mlp.down_proj.weight", (ShardingType.TP_SHARDING, 1, 4)),
        ("model.layers.0.mlp.gate.weight", (ShardingType.NO_SHARDING, 0, 1)),
        ("model.layers.0.mlp.experts.3.down_proj.weight", (ShardingType.TP_SHARDING, 1, 4)),  # no EP: experts are TP-cut
        ("model.layers.0.mlp.gate.expert_bias", (ShardingType.NO_SHARDING, 0, 1)),
    ]:
        assert s.get_sharding_strategy(name) == want, name
    whole = strategy(rank_info(tp=1))
    assert whole.get_sharding_strategy("model.layers.0.mlp.down_proj.weight") == (ShardingType.NO_SHARDING, 1, 1)


def test_expert_parallel_and_dp_attention_variants():
    ep = strategy(rank_info(tp=4, ep=4))
    assert ep.get_sharding_strategy("model.layers.0.mlp.experts.3.gate_proj.weight") == (ShardingType.EP_SHARDING, 0, 4)
    ep_tp = strategy(rank_info(tp=4, ep=2, etp=2))
    assert ep_tp.get_sharding_strategy("model.layers.0.mlp.experts.3.down_proj.weight") == (ShardingType.EP_TP_SHARDING, 1, 2)
    # shared experts: TP-cut on the training side, treated like experts by inference engines
    assert strategy(rank_info(tp=4, ep=4), engine="mcore").get_sharding_strategy("model.layers.0.mlp.shared_experts.up_proj.weight") == \
        (ShardingType.TP_SHARDING, 0, 4)
    assert ep.get_sharding_strategy("model.layers.0.mlp.shared_experts.up_proj.weight") == (ShardingType.EP_SHARDING, 0, 4)
    dp = strategy(rank_info(tp=4, attn_tp=2), dp_attention=True, dp_lm_head=True)
    assert dp.get_sharding_strategy("model.layers.0.attention.dense.weight") == (ShardingType.DP_TP_SHARDING, 1, 2)
    assert dp.get_sharding_strategy("model.embed_tokens.weight") == (ShardingType.DP_TP_SHARDING, 0, 2)
    assert dp.get_sharding_strategy("lm_head.weight") == (ShardingType.DP_TP_SHARDING, 0, 2)
    assert dp.get_sharding_strategy("model.layers.0.mlp.down_proj.weight") == (ShardingType.TP_SHARDING, 1, 4)


def test_mla_mixin_and_bailing_attention_under_context_parallelism():
    from awex_b200.models.ling_linear import BailingLinearMoeShardingStrategy

    class Mla(LinearMLAShardingMixin, ShardingStrategy):
        pass

    s = strategy(rank_info(tp=4), cls=Mla)
    assert s.get_sharding_strategy("model.layers.0.attention.q_a_proj.weight")[0] == ShardingType.NO_SHARDING
    assert s.get_sharding_strategy("model.layers.0.attention.kv_a_layernorm.weight")[0] == ShardingType.NO_SHARDING
    assert s.get_sharding_strategy("model.layers.0.attention.g_norm.weight") == (ShardingType.TP_SHARDING, 0, 4)
    assert s.get_sharding_strategy("model.layers.0.attention.q_b_proj.weight") == (ShardingType.TP_SHARDING, 0, 4)
    # training side: fused QKV is TP-cut with attention TP 4 whatever the CP size; with attention TP 1 (pure context
    # parallelism) it is whole on every rank, and the planner cuts it for the inference shards
    name = "model.layers.0.attention.query_key_value.weight"
    for cp in (1, 8):
        healthy = strategy(rank_info(tp=4, cp=cp, infer=False), engine="mcore", cls=BailingLinearMoeShardingStrategy)
        assert healthy.get_sharding_strategy(name) == (ShardingType.TP_SHARDING, 0, 4)
        pure_cp = strategy(rank_info(tp=1, cp=cp, infer=False), engine="mcore", cls=BailingLinearMoeShardingStrategy)
        assert pure_cp.get_sharding_strategy(name) == (ShardingType.NO_SHARDING, 0, 1)


def test_rank_info_from_engine_contexts(monkeypatch):
    from awex_b200.sharding.extractors import get_sglang_rank_info, get_vllm_rank_info

    base = dict(tp_rank=5, tp_size=8, pp_rank=0, pp_size=1, dp_rank=0, dp_size=1, attn_tp_rank=5, attn_tp_size=8, attn_dp_rank=0,
                world_size=8, global_rank=5, local_rank=5)
    args = SimpleNamespace(dp_size=1, enable_dp_attention=False, ep_size=4)
    sgl = get_sglang_rank_info({**base, "scheduler": SimpleNamespace(server_args=args)}, engine_rank=2)
    assert (sgl.ep_size, sgl.ep_tp_size, sgl.ep_rank, sgl.ep_tp_rank) == (4, 2, 2, 1)  # expert TP nests inside TP
    assert sgl.engine_rank == 2 and sgl.is_infer and (sgl.cp_size, sgl.cp_mode) == (1, "none")
    args.dp_size = 2
    with pytest.raises(ValueError):
        get_sglang_rank_info({**base, "scheduler": SimpleNamespace(server_args=args)}, 0)
    vllm = get_vllm_rank_info({**base, "ep_size": 8, "ep_rank": 5, "cp_size": 2, "cp_rank": 1, "cp_mode": "ring"}, 0)
    assert (vllm.ep_size, vllm.ep_rank, vllm.ep_tp_size) == (8, 5, 1) and (vllm.cp_size, vllm.cp_rank, vllm.cp_mode) == (2, 1, "ring")
    plain = get_vllm_rank_info(base, 1)
    assert (plain.ep_size, plain.ep_rank, plain.cp_size, plain.engine_rank) == (1, 0, 1, 1)


def test_vllm_names_are_normalised_to_the_canonical_contract():
    from awex_b200.config import InferenceConfig
    from awex_b200.converter.vllm_converter import VLLMToHFWeightConverter

    hf = SimpleNamespace(num_attention_heads=8, num_key_value_heads=4, hidden_size=64, num_hidden_layers=1)
    conv = VLLMToHFWeightConverter(hf, InferenceConfig(tp_size=1, ep_size=1), rank_info(tp=1))
    t = torch.zeros(4, 4)
    assert [n for n, _ in conv.convert_param("model.layers.0.self_attn.qkv_proj.weight", t)] == ["model.layers.0.attention.query_key_value_proj.weight"]
    assert [n for n, _ in conv.convert_param("model.layers.0.self_attn.o_proj.weight", t)] == ["model.layers.0.attention.dense.weight"]
    assert [n for n, _ in conv.convert_param("model.layers.0.self_attn.q_norm.weight", t[0])] == ["model.layers.0.attention.query_layernorm.weight"]
    assert [n for n, _ in conv.convert_param("model.layers.0.self_attn.o_proj.weight_scale_inv", t)] == ["model.layers.0.attention.dense.weight_scale_inv"]
    halves = conv.convert_param("model.layers.0.mlp.gate_up_proj.weight", torch.arange(8.0).reshape(4, 2))
    assert [n for n, _ in halves] == ["model.layers.0.mlp.gate_proj.weight", "model.layers.0.mlp.up_proj.weight"]
    assert torch.equal(halves[1][1], torch.arange(4.0, 8.0).reshape(2, 2))
