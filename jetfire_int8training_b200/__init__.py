"""B200 (sm_100a) implementation of the Jetfire INT8 data-flow hot path.

Sub-packages mirror the reference's operator layer so a caller written against it keeps working:
    from jetfire_int8training_b200.Nonlinear import int8_quantize, int8_gelu_forward, ...
    from jetfire_int8training_b200.Linear import int8_linear_forward, int8_linear_backward
`jetfire_int8training_b200.compat.install()` additionally registers them under the reference's own top-level module
names (`Nonlinear`, `Linear`, `BlockQuantizeCUDA`).
"""
from . import rng  # noqa: F401
from . import Nonlinear  # noqa: F401
from . import Linear  # noqa: F401

__all__ = ["Nonlinear", "Linear", "rng"]
