"""mxfp4 -- B200-native (sm_100a) implementation of the MoizMXFP4 public API."""
from .quantizer import MXFP4Quantizer
from .modules import MXLinear
from .utils import quantize_model_mxfp4, get_model_size_mb
from .kernel_dispatcher import quant_matmul, print_architecture_info
from .gemm import quant_matmul_host

__version__ = "0.1.0"
__all__ = [
    "MXFP4Quantizer",
    "MXLinear",
    "quantize_model_mxfp4",
    "get_model_size_mb",
    "quant_matmul",
    "quant_matmul_host",
    "print_architecture_info",
]
