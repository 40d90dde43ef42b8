"""tmq_b200: TMQ's soft-staircase QAT and packed-ternary inference on B200 (sm_100a) CUDA kernels.

`from tmq_b200 import *` yields the same names as `from tmq import *` of the reference project.  The API module
(and with it the CUDA library) is loaded on first use, so that `python -m tmq_b200.build` can run before the
library exists."""
import importlib

__all__ = ["CUDA_EXT_AVAILABLE", "NATIVE_EXT_AVAILABLE", "Conv2d", "ConvTranspose2d", "Linear", "QuantizationControl",
           "QuantizationScheduleBuilder", "QuantMode", "SoftStep", "SoftStepDerivative", "TensorType", "TMQLayer",
           "compressed_state_dict", "expand_compact_layers", "load_compressed_state_dict", "prepare_compressed_load",
           "quantize_model", "quantize_weights", "fwd_softstep", "bwd_softstep", "fwd_softstep_derivative",
           "bwd_softstep_derivative", "compactify_ternary", "expand_ternary", "compress_ternary", "decompress_ternary"]


def __getattr__(name):
    if name in __all__:
        return getattr(importlib.import_module(".tmq", __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
