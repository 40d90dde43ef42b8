"""tmq_b200: TMQ's soft-staircase QAT and packed-ternary inference on B200 (sm_100a) CUDA kernels.

`from tmq_b200 import *` yields the same names as `from tmq import *` of the reference project."""
from .tmq import *  # noqa: F401,F403
from .tmq import (CUDA_EXT_AVAILABLE, NATIVE_EXT_AVAILABLE, Conv2d, ConvTranspose2d, Linear, QuantizationControl,  # noqa: F401
                  QuantizationScheduleBuilder, QuantMode, SoftStep, SoftStepDerivative, TensorType, TMQLayer,
                  compressed_state_dict, expand_compact_layers, load_compressed_state_dict, prepare_compressed_load,
                  quantize_model, quantize_weights)
