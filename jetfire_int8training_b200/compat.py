"""Register the package's operator modules under the reference's top-level import names, so code written as
`from Nonlinear import int8_quantize` / `from Linear import int8_linear_forward` / `import BlockQuantizeCUDA`
(INT8_GPT2/qmodel.py:18-22, Jetfire/Linear/linear_fwd.py:2) picks up the sm_100a kernels."""
import sys


def install():
    from . import BlockQuantizeCUDA, Linear, Nonlinear
    sys.modules.setdefault("Nonlinear", Nonlinear)
    sys.modules.setdefault("Linear", Linear)
    sys.modules.setdefault("BlockQuantizeCUDA", BlockQuantizeCUDA)
