from awex_b200.sharding.param_sharding import (  # noqa: F401
    LinearMLAShardingMixin,
    ShardingStrategy,
    ShardingType,
    get_default_sharding_dim,
    get_rank_info_extractor,
    get_sharding_strategy_builder,
)
from awex_b200.sharding.rank_info import RankInfo  # noqa: F401
