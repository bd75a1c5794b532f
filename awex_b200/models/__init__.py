from awex_b200.models.registry import (  # noqa: F401
    ModelRegistry,
    get_infer_weights_converter,
    get_sharding_strategy,
    get_train_weights_converter,
)
