from .model_utils import quantize_model_mxfp4, get_model_size_mb

__all__ = ["quantize_model_mxfp4", "get_model_size_mb"]
