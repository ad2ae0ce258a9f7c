from .sharded import (  # noqa: F401
    combine_amax,
    plan_row_shards,
    sharded_dynamic_scaled_quant,
    sharded_global_amax,
    sharded_quantize_nvfp4,
)
