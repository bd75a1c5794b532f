"""Rank coordinates for synthetic jobs.

Training ranks follow Megatron's order (TP fastest, then DP, then PP); the
expert grid re-uses the ``tp * dp`` ranks of a pipeline stage as
``expert_tp`` (fastest) x ``ep`` x expert-DP.  Inference ranks follow vLLM:
TP inside an instance, experts either TP-sliced (``ep == 1``) or distributed
whole over the instance's ranks (``ep == tp``, expert TP 1); the SGLang flavour
nests expert TP inside TP (``ep_tp = tp // ep``).
"""

from __future__ import annotations

from typing import List

from awex_b200.sharding.rank_info import RankInfo


def train_rank_infos(tp: int = 1, pp: int = 1, dp: int = 1, ep: int = 1, etp: int = 1, gpus_per_node: int = 8) -> List[RankInfo]:
    world = tp * pp * dp
    if ep == 1:
        etp = tp  # Megatron's default: without expert parallelism the experts are cut over the TP group
    assert (tp * dp) % (ep * etp) == 0, "expert grid must tile the tp*dp ranks of a stage"
    out = []
    for rank in range(world):
        tp_rank = rank % tp
        dp_rank = (rank // tp) % dp
        pp_rank = rank // (tp * dp)
        in_stage = dp_rank * tp + tp_rank
        out.append(
            RankInfo(
                tp_rank=tp_rank, tp_size=tp, pp_rank=pp_rank, pp_size=pp, dp_size=dp, dp_rank=dp_rank,
                ep_rank=(in_stage // etp) % ep, ep_size=ep, ep_tp_rank=in_stage % etp, ep_tp_size=etp,
                attn_tp_rank=tp_rank, attn_tp_size=tp, attn_dp_rank=dp_rank, world_size=world,
                global_rank=rank, local_rank=rank % gpus_per_node, engine_rank=0, is_infer=False,
            )
        )
    return out


def infer_rank_infos(tp: int = 1, ep: int = 1, engine_rank: int = 0, pp: int = 1, flavour: str = "vllm",
                     first_local_rank: int = 0, attn_tp: int = 0) -> List[RankInfo]:
    """Ranks of ONE inference instance (``global_rank`` is instance-local).
    ``attn_tp`` (SGLang's DP attention): attention, embeddings and, optionally,
    the head are cut over ``attn_tp`` ranks and replicated over ``tp / attn_tp``
    attention-DP groups; everything else is cut over ``tp``."""
    world = tp * pp
    attn_tp = attn_tp or tp
    assert tp % attn_tp == 0, "attention TP must divide TP"
    out = []
    for rank in range(world):
        tp_rank, pp_rank = rank % tp, rank // tp
        if ep > 1:
            ep_tp = tp // ep if flavour == "sglang" else 1
            ep_rank = tp_rank // ep_tp if flavour == "sglang" else tp_rank % ep
            ep_tp_rank = tp_rank % ep_tp if flavour == "sglang" else 0
        else:
            ep_tp, ep_rank, ep_tp_rank = 1, 0, 0
        out.append(
            RankInfo(
                tp_rank=tp_rank, tp_size=tp, pp_rank=pp_rank, pp_size=pp, dp_size=1, dp_rank=0,
                ep_rank=ep_rank, ep_size=ep, ep_tp_rank=ep_tp_rank, ep_tp_size=ep_tp,
                attn_tp_rank=tp_rank % attn_tp, attn_tp_size=attn_tp, attn_dp_rank=tp_rank // attn_tp, world_size=world,
                global_rank=rank, local_rank=first_local_rank + rank, engine_rank=engine_rank, is_infer=True,
            )
        )
    return out
