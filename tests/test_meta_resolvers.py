"""Metadata resolvers: inference-side shard / replica construction from canned
per-worker reports, canonical rank-0 selection with internal data parallelism,
the tied-embedding alias, PP / VPP layer renumbering, and what the control
reader publishes to the training side."""

from types import SimpleNamespace

import pytest
import torch

from awex_b200.config import InferenceConfig
from awex_b200.sharding.rank_info import RankInfo


def rank(tp_rank=0, tp_size=1, global_rank=None, dp_rank=0, dp_size=1, pp_rank=0, pp_size=1, ep_rank=0, ep_size=1, engine_rank=0, infer=True):
    g = tp_rank if global_rank is None else global_rank
    return RankInfo(tp_rank=tp_rank, tp_size=tp_size, pp_rank=pp_rank, pp_size=pp_size, dp_size=dp_size, dp_rank=dp_rank,
                    ep_rank=ep_rank, ep_size=ep_size, ep_tp_rank=0, ep_tp_size=1, attn_tp_rank=tp_rank, attn_tp_size=tp_size,
                    attn_dp_rank=0, world_size=tp_size * pp_size * dp_size, global_rank=g, local_rank=g, engine_rank=engine_rank,
                    is_infer=infer)


def raw(name, shape, dtype="torch.bfloat16"):
    numel = 1
    for d in shape:
        numel *= d
    return {"name": name, "shape": tuple(shape), "numel": numel, "dtype": dtype}


class CannedEngine:
    """Inference engine whose workers answer the metadata task with canned data."""

    engine_name = "sglang"

    def __init__(self, reports, tp=2):
        self.hf_config = SimpleNamespace(num_hidden_layers=2, architectures=["LlamaForCausalLM"], tie_word_embeddings=False)
        self.config = InferenceConfig(tp_size=tp, pp_size=1, dp_size=1, ep_size=1)
        self.reports, self.calls = reports, []

    def execute_task_in_model_worker(self, fn, **kwargs):
        self.calls.append((getattr(fn, "__name__", str(fn)), kwargs))
        return self.reports


def tp2_reports():
    names = [("model.embed_tokens.weight", (8, 4)), ("model.layers.0.self_attn.o_proj.weight", (4, 2)),
             ("model.layers.0.input_layernorm.weight", (4,)), ("model.layers.0.mlp.down_proj.weight", (4, 6))]
    return [{"rank_info": rank(r, 2), "model_arch_name": "LlamaForCausalLM", "params_meta": [raw(n, s) for n, s in names]} for r in range(2)]


# ------------------------------------------------------------------------------------------ inference side
def test_infer_resolver_builds_shards_replicas_and_offsets():
    from awex_b200.meta.infer_meta_resolver import InferParamMetaResolver
    from awex_b200.sharding.param_sharding import ShardingType

    engine = CannedEngine(tp2_reports())
    resolver = InferParamMetaResolver(engine, convert_params=True)
    assert engine.calls[0][1]["convert_params"] is True and engine.calls[0][1]["engine_name"] == "sglang"
    meta = {p.name: p for p in resolver.get_parameters_meta()}
    embed = meta["model.embed_tokens.weight"]
    assert embed.global_shape == (16, 4) and embed.dtype == torch.bfloat16
    assert [s.global_offset for s in embed.replicas[0].shards] == [(0, 0), (8, 0)]
    o_proj = meta["model.layers.0.self_attn.o_proj.weight"]  # row-parallel: split along the input dimension
    assert o_proj.global_shape == (4, 4) and [s.global_offset for s in o_proj.replicas[0].shards] == [(0, 0), (0, 2)]
    norm = meta["model.layers.0.input_layernorm.weight"]  # not sharded: one replica per holder
    assert norm.global_shape == (4,) and len(norm.replicas) == 2 and norm.shards[0].sharding_type == ShardingType.NO_SHARDING
    assert resolver.get_model_arch_name() == "LlamaForCausalLM"
    assert resolver.total_numel == 16 * 4 + 16 + 4 + 4 * 12 and resolver.total_size == 2 * resolver.total_numel


def test_rank_infos_that_arrive_as_dicts_are_restored():
    import dataclasses

    from awex_b200.meta.infer_meta_resolver import InferParamMetaResolver

    reports = tp2_reports()
    for r in reports:
        r["rank_info"] = dataclasses.asdict(r["rank_info"])  # what a msgpack RPC layer hands back
    resolver = InferParamMetaResolver(CannedEngine(reports))
    assert isinstance(resolver.rank0_info, RankInfo) and resolver.rank0_info.tp_size == 2


def test_canonical_rank0_with_internal_data_parallel_cores():
    from awex_b200.meta.infer_meta_resolver import InferParamMetaResolver

    pick = InferParamMetaResolver._select_canonical_rank0_meta
    core1 = {"rank_info": rank(0, 1, global_rank=0, dp_rank=1, dp_size=2), "tag": "dp1"}
    core0 = {"rank_info": rank(0, 1, global_rank=0, dp_rank=0, dp_size=2), "tag": "dp0"}
    assert pick([core1, core0])["tag"] == "dp0"
    assert pick([{"rank_info": rank(1, 2, global_rank=3), "tag": "b"}, {"rank_info": rank(0, 2, global_rank=2), "tag": "a"}])["tag"] == "a"
    with pytest.raises(ValueError):
        pick([])


def test_tied_embeddings_publish_an_lm_head_alias():
    from awex_b200.meta.infer_meta_resolver import collect_worker_param_info
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.models import build_vllm_model, vllm_model_context
    from awex_b200.synthetic.topology import infer_rank_infos

    import dataclasses

    arch = dataclasses.replace(get_arch("tiny-llama"), tie_embeddings=True)
    ri = infer_rank_infos(tp=1)[0]
    model = build_vllm_model(arch, ri, torch.float32, "cpu")
    assert "lm_head.weight" not in dict(model.named_parameters())
    cfg = InferenceConfig(tp_size=1, pp_size=1, dp_size=1, ep_size=1)
    info = collect_worker_param_info("vllm", cfg, convert_params=True, model=model, model_context=vllm_model_context(ri, infer_engine_config=cfg))
    names = {p["name"]: p for p in info["params_meta"]}
    assert "lm_head.weight" in names and names["lm_head.weight"]["shape"] == names["model.embed_tokens.weight"]["shape"]
    untied = build_vllm_model(get_arch("tiny-llama"), ri, torch.float32, "cpu")
    info = collect_worker_param_info("vllm", cfg, convert_params=True, model=untied, model_context=vllm_model_context(ri, infer_engine_config=cfg))
    assert [p["name"] for p in info["params_meta"]].count("lm_head.weight") == 1


# ------------------------------------------------------------------------------------------ pipeline stages
def _stage_report(pp_rank, pp_size, vp_stage, local_ids):
    return {"rank_info": rank(0, 1, global_rank=pp_rank, pp_rank=pp_rank, pp_size=pp_size, infer=False),
            "params_meta": [dict(raw(f"decoder.layers.{i}.mlp.linear_fc2.weight", (2, 2)), vp_stage=vp_stage) for i in local_ids]
            + [dict(raw("decoder.final_layernorm.weight", (2,)), vp_stage=vp_stage)]}


def test_pp_and_vpp_layer_renumbering():
    from awex_b200.converter.pp_layout import normalize_pp_stage_layer_id_map, process_mcore_pp_name
    from awex_b200.meta.train_meta_resolver import build_pp_stage_layer_id_map, canonicalize_pp_layer_names

    # two pipeline ranks x two virtual stages, two layers each: virtual stage outermost
    reports = [_stage_report(0, 2, 0, [0, 1]), _stage_report(1, 2, 0, [0, 1]), _stage_report(0, 2, 1, [0, 1]), _stage_report(1, 2, 1, [0, 1])]
    stage_map = build_pp_stage_layer_id_map(reports)
    assert stage_map == {(0, 0): {0: 0, 1: 1}, (1, 0): {0: 2, 1: 3}, (0, 1): {0: 4, 1: 5}, (1, 1): {0: 6, 1: 7}}
    canonicalize_pp_layer_names(reports, stage_map)
    assert [p["name"] for p in reports[3]["params_meta"]][:2] == [f"decoder.layers.{i}.mlp.linear_fc2.weight" for i in (6, 7)]
    assert reports[3]["params_meta"][2]["name"] == "decoder.final_layernorm.weight"
    # one-based local ids keep their order
    assert build_pp_stage_layer_id_map([_stage_report(0, 2, 0, [1, 2]), _stage_report(1, 2, 0, [1, 2])]) == {(0, 0): {1: 0, 2: 1}, (1, 0): {1: 2, 2: 3}}
    assert build_pp_stage_layer_id_map([{"rank_info": rank(infer=False), "params_meta": [raw("embedding.weight", (2, 2))]}]) == {}
    with pytest.raises(ValueError, match="no entry"):
        canonicalize_pp_layer_names([_stage_report(1, 2, 0, [5])], {(1, 0): {0: 2}})
    # the converter applies the same map by (pp_rank, vp_stage)
    wire = normalize_pp_stage_layer_id_map({"1:1": {"0": 6, "1": 7}, (0, 0): {0: 0}})
    assert wire == {(1, 1): {0: 6, 1: 7}, (0, 0): {0: 0}}
    ri = SimpleNamespace(pp_rank=1, pp_size=2)
    assert process_mcore_pp_name("decoder.layers.1.self_attention.linear_qkv.weight", ri, vp_stage=1, pp_stage_layer_id_map=wire) == \
        "decoder.layers.7.self_attention.linear_qkv.weight"
    assert process_mcore_pp_name("embedding.word_embeddings.weight", ri, pp_stage_layer_id_map=wire) == "embedding.word_embeddings.weight"
    assert process_mcore_pp_name("decoder.layers.1.x", ri, pp_stage_layer_id_map=None) == "decoder.layers.1.x"
    with pytest.raises(ValueError, match="Missing pp stage layer map"):
        process_mcore_pp_name("decoder.layers.0.x", ri, vp_stage=0, pp_stage_layer_id_map=wire)
    with pytest.raises(ValueError, match="Local layer id missing"):
        process_mcore_pp_name("decoder.layers.9.x", ri, vp_stage=1, pp_stage_layer_id_map=wire)
    for bad in ({"1-1": {}}, {3: {}}, {"1:0": [1]}):
        with pytest.raises(ValueError):
            normalize_pp_stage_layer_id_map(bad)


def test_stage_layer_ids_from_the_transformer_config():
    from awex_b200.converter.pp_layout import resolve_pp_stage_global_layer_ids

    hf = SimpleNamespace(num_hidden_layers=8)
    even = lambda pp, vp=None: resolve_pp_stage_global_layer_ids(SimpleNamespace(pp_rank=pp, pp_size=2), hf, {}, vp)  # noqa: E731
    assert even(0) == [0, 1, 2, 3] and even(1) == [4, 5, 6, 7]
    vpp = {"virtual_pipeline_model_parallel_size": 2}
    stage = lambda pp, vp: resolve_pp_stage_global_layer_ids(SimpleNamespace(pp_rank=pp, pp_size=2), hf, vpp, vp)  # noqa: E731
    assert [stage(0, 0), stage(1, 0), stage(0, 1), stage(1, 1)] == [[0, 1], [2, 3], [4, 5], [6, 7]]
    with pytest.raises(ValueError):
        resolve_pp_stage_global_layer_ids(SimpleNamespace(pp_rank=2, pp_size=2), hf, {})
    with pytest.raises(ValueError):
        stage(0, 2)


# ------------------------------------------------------------------------------------------ control reader
def test_control_reader_publishes_engine_name_and_layout_facts():
    """What the training side needs to pick its converter travels as
    ``infer_conf``: engine flavour, attention TP size, world size; rank 0 also
    publishes the inference metadata, and the workers receive both sides' metadata."""
    import copy
    import pickle

    from awex_b200.reader.weights_reader import WeightsReader

    published = {}

    class FakeMeta:
        def put_object(self, key, value):
            published[key] = value

        def get_object(self, key, timeout=0, default_value=None):
            if key == "training_params_meta":  # a training side with the same layout
                return copy.deepcopy(published["infer_params_meta"])
            return published.get(key, default_value)

    engine = CannedEngine(tp2_reports())
    engine.config = InferenceConfig(tp_size=2, pp_size=1, dp_size=1, ep_size=1, comm_backend="nccl", meta_server_addr="127.0.0.1:9")
    engine.num_engines, engine.engine_rank = 1, 0
    reader = WeightsReader(engine)
    reader.meta_server_client = FakeMeta()
    reader._initialize()
    conf = published["infer_conf"]
    assert conf["engine_name"] == "sglang" and conf["infer_atten_tp_size"] == 2 and conf["infer_world_size"] == 2
    assert conf["expected_pp_ranks"] == [0] and conf["fp8_block_quant"] is False
    assert {p.name for p in published["infer_params_meta"]} == {p["name"] for p in tp2_reports()[0]["params_meta"]}
    name, kwargs = engine.calls[-1]
    assert name == "_init_in_tp_worker" and kwargs["weights_comm_backend"] == "nccl" and kwargs["num_engines"] == 1
    assert pickle.loads(kwargs["infer_conf_bytes"])["engine_name"] == "sglang"
    assert len(pickle.loads(kwargs["training_params_meta_bytes"])) == 4


def test_uneven_pipeline_splits_and_explicit_layouts():
    from awex_b200.converter.pp_layout import resolve_pp_stage_global_layer_ids, stage_counts_from_layout, stage_counts_from_split_config

    assert stage_counts_from_split_config(10, 4, {"num_layers_in_first_pipeline_stage": 2, "num_layers_in_last_pipeline_stage": 2}) == [[2], [3], [3], [2]]
    assert stage_counts_from_split_config(7, 2, {"num_layers_in_first_pipeline_stage": 3}) == [[3], [4]]
    # the embedding and the loss each count as a layer when the split is made, then give their slot back
    assert stage_counts_from_split_config(6, 4, {"account_for_embedding_in_pipeline_split": True, "account_for_loss_in_pipeline_split": True}) == [[1], [2], [2], [1]]
    assert stage_counts_from_split_config(8, 2, {"virtual_pipeline_model_parallel_size": 2}) == [[2, 2], [2, 2]]
    for bad in ({"num_layers_in_first_pipeline_stage": 2, "account_for_loss_in_pipeline_split": True}, {"num_layers_in_first_pipeline_stage": 0},
                {"num_layers_in_first_pipeline_stage": 9, "num_layers_in_last_pipeline_stage": 9}, {"virtual_pipeline_model_parallel_size": 3}):
        with pytest.raises(ValueError):
            stage_counts_from_split_config(8, 2, bad)
    with pytest.raises(ValueError):
        stage_counts_from_split_config(7, 2, {})
    flat = [["embedding", "decoder"], ["decoder", "decoder"], ["decoder"], ["decoder", "loss"]]  # stage = vp * pp + pp_rank
    assert stage_counts_from_layout(flat, 2) == [[1, 1], [2, 1]]
    nested = [[["embedding", "decoder"], ["decoder"]], [["decoder", "decoder"], ["decoder", "loss"]]]
    assert stage_counts_from_layout(nested, 2) == [[1, 1], [2, 1]]
    for bad, pp in (([], 2), ("decoder", 2), ([["decoder"]] * 3, 2), ([[["decoder"]], [["decoder"], ["decoder"]]], 2)):
        with pytest.raises(ValueError):
            stage_counts_from_layout(bad, pp)
    hf = SimpleNamespace(num_hidden_layers=5)
    ids = lambda pp, vp: resolve_pp_stage_global_layer_ids(SimpleNamespace(pp_rank=pp, pp_size=2), hf, {"pipeline_model_parallel_layout": flat}, vp)  # noqa: E731
    assert [ids(0, 0), ids(1, 0), ids(0, 1), ids(1, 1)] == [[0], [1, 2], [3], [4]]
    with pytest.raises(ValueError, match="do not match num_hidden_layers"):
        resolve_pp_stage_global_layer_ids(SimpleNamespace(pp_rank=0, pp_size=2), SimpleNamespace(num_hidden_layers=6), {"pipeline_model_parallel_layout": flat}, 0)


# ---- shard / replica construction from canned worker reports (the reference's mocked cases) ----------------
def _worker_rank(tp_rank, tp_size, dp_size, attn_tp_rank, attn_tp_size, attn_dp_rank, world, global_rank):
    return RankInfo(tp_rank=tp_rank, tp_size=tp_size, pp_rank=0, pp_size=1, dp_size=dp_size, dp_rank=0, ep_rank=0, ep_size=1,
                    ep_tp_rank=0, ep_tp_size=1, attn_tp_rank=attn_tp_rank, attn_tp_size=attn_tp_size, attn_dp_rank=attn_dp_rank,
                    world_size=world, global_rank=global_rank, local_rank=global_rank, engine_rank=0, is_infer=True)


class _ReportingEngine:
    engine_name = "sglang"

    def __init__(self, tp, dp, dp_attention, names, ranks):
        self.config = InferenceConfig(tp_size=tp, pp_size=1, dp_size=dp, ep_size=1, enable_dp_attention=dp_attention, moe_dense_tp_size=1)
        self.hf_config = SimpleNamespace(num_hidden_layers=4, architectures=["Dummy"], tie_word_embeddings=False)
        self.reports = [{"rank_info": _worker_rank(*r), "model_arch_name": "Dummy",
                         "params_meta": [raw(n, s, "torch.float32") for n, s in names]} for r in ranks]

    def execute_task_in_model_worker(self, fn, **kwargs):
        return self.reports


@pytest.mark.parametrize("tp,dp,dp_attention,names,ranks,kind,shards,replicas,offsets", [
    (1, 1, False, [("embed_tokens.weight", (8, 8)), ("mlp.weight", (8, 8)), ("attention.weight", (8, 8))],
     [(0, 1, 1, 0, 1, 0, 1, 0)], "NO_SHARDING", 1, 1, [(0, 0)]),
    (2, 1, False, [("mlp.weight", (4, 8)), ("attention.weight", (4, 8))],
     [(0, 2, 1, 0, 1, 0, 2, 0), (1, 2, 1, 0, 1, 0, 2, 1)], "TP_SHARDING", 2, 1, [(0, 0), (4, 0)]),
    # DP attention: sharded over the attention-TP ranks, one replica per attention-DP rank
    (2, 2, True, [("attention.weight", (2, 8))],
     [(0, 2, 2, 0, 2, 0, 4, 0), (1, 2, 2, 1, 2, 0, 4, 1), (0, 2, 2, 0, 2, 1, 4, 2), (1, 2, 2, 1, 2, 1, 4, 3)],
     "DP_TP_SHARDING", 4, 2, [(0, 0), (2, 0), (0, 0), (2, 0)]),
])
def test_shards_replicas_and_offsets_from_worker_reports(tp, dp, dp_attention, names, ranks, kind, shards, replicas, offsets):
    from awex_b200.meta.infer_meta_resolver import InferParamMetaResolver

    resolver = InferParamMetaResolver(_ReportingEngine(tp, dp, dp_attention, names, ranks))
    params = resolver.get_parameters_meta()
    assert [p.name for p in params] == [n for n, _ in names]
    for p in params:
        assert {s.sharding_type.name for s in p.shards} == {kind}
        assert len(p.shards) == shards and len(p.replicas) == replicas and p.dtype == torch.float32
        assert [tuple(s.global_offset) for s in p.shards] == offsets
        for rep in p.replicas:
            assert sum(s.numel for s in rep.shards) == p.global_numel  # every replica is a whole copy
            assert sorted(s.tp_rank for s in rep.shards) == sorted({r[0] for r in ranks})
        shard = p.shards[0]
        assert (shard.cp_rank, shard.cp_size, shard.cp_mode) == (0, 1, "none")  # context-parallel fields stay at their defaults


def test_ranks_that_disagree_on_the_number_of_replicas_are_refused():
    from awex_b200.meta.infer_meta_resolver import InferParamMetaResolver

    ranks = [(0, 2, 1, 0, 1, 0, 2, 0), (0, 2, 1, 0, 1, 0, 2, 1), (1, 2, 1, 0, 1, 0, 2, 2)]  # two holders of TP shard 0, one of shard 1
    with pytest.raises(AssertionError, match="Inconsistent number of replicas"):
        InferParamMetaResolver(_ReportingEngine(2, 1, False, [("mlp.weight", (4, 8))], ranks))
