from .scaled_quant import (  # noqa: F401
    dynamic_scaled_quant,
    eager_dynamic_scaled_quant,
    eager_scaled_quant,
    dynamic_scaled_quant_transpose,
    dynamic_scaled_quant_with_scale,
    rowwise_scaled_quant,
    scaled_quant,
    scaled_quant_transpose,
)
from .delayed_scaling import DelayedScaling, combine_amaxes  # noqa: F401
from .producer_quant import (  # noqa: F401
    rms_norm_quantize_mxfp8,
    rms_norm_rowwise_quant,
    swiglu_quantize_mxfp8,
    swiglu_rowwise_quant,
)
