"""Counterpart of the reference's RTN_quantization/ directory: same module and function names."""
from .per_tensor_channel_group import (W8A8Linear, quantize_activation_codes,  # noqa: F401
                                       quantize_activation_per_group_absmax_token_dim,
                                       quantize_activation_per_tensor_absmax,
                                       quantize_activation_per_token_absmax, quantize_weight_codes,
                                       quantize_weight_per_channel_absmax,
                                       quantize_weight_per_group_absmax_input_features,
                                       quantize_weight_per_tensor_absmax)
from .Smooth import smooth_ln_fcs  # noqa: F401
from .utils import replace_linear_with_target_and_quantize, smooth_sam  # noqa: F401
from .calibration import get_act_scales_sam  # noqa: F401
