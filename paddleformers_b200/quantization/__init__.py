from .checkpoint_dequant import dequant_fp8_block, dequant_mxfp4  # noqa: F401
from .fp8 import FP8Linear, convert_linears_to_fp8, quant_act_1x128, quant_weight_128x128  # noqa: F401
from .weight_only import QuantizationLinear, quantize_model  # noqa: F401
