from .quantize import quantize_mxfp8  # noqa: F401
from .to_blocked import ceil_div, to_blocked  # noqa: F401
