"""MXLinear -- drop-in for the reference's src/mxfp4/modules.py:16-156.

Same constructor, attributes, buffers and state_dict keys.  What changes is the arithmetic of the
quantised forward: the reference re-materialises the whole float32 weight on every call and hands it
to F.linear; here the packed weight goes straight to the block-scaled FP4 tensor-core GEMM.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .quantizer import MXFP4Quantizer


class MXLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, block_size: int = 32):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.block_size = block_size
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()
        self._init_quant_state(block_size)

    def _init_quant_state(self, block_size):
        self.quantizer = MXFP4Quantizer(block_size=block_size)
        self.is_quantized = False
        self.simulate_quantization = False
        # buffers so that packed weights travel in state_dict (modules.py:51-52)
        self.register_buffer("packed_weight", None)
        self.register_buffer("weight_scales", None)

    @classmethod
    def from_linear(cls, linear: nn.Linear, block_size: int = 32) -> "MXLinear":
        """Wrap an existing nn.Linear without allocating or initialising a second weight."""
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self.in_features = linear.in_features
        self.out_features = linear.out_features
        self.block_size = block_size
        self.weight = nn.Parameter(linear.weight.data, requires_grad=False)
        if linear.bias is not None:
            self.bias = nn.Parameter(linear.bias.data, requires_grad=linear.bias.requires_grad)
        else:
            self.register_parameter("bias", None)
        self._init_quant_state(block_size)
        return self

    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        if self.bias is not None:
            fan_in, _ = nn.init._calculate_fan_in_and_fan_out(self.weight)
            bound = 1 / (fan_in ** 0.5) if fan_in > 0 else 0
            nn.init.uniform_(self.bias, -bound, bound)

    def quantize(self, device=None):
        """Pack .weight into MXFP4 buffers and delete it (modules.py:61-88)."""
        if self.is_quantized:
            return
        if self.weight is None:
            raise ValueError("No weights to quantize.")
        if device:
            self.to(device)
        with torch.no_grad():
            packed, scales = self.quantizer.quantize(self.weight)
            self.packed_weight = packed
            self.weight_scales = scales
            del self.weight
            self.register_parameter("weight", None)
            self.is_quantized = True

    def dequantize(self):
        """Restore a float32 .weight from the packed buffers (modules.py:90-112)."""
        if not self.is_quantized:
            return
        with torch.no_grad():
            w = self.quantizer.dequantize(self.packed_weight, self.weight_scales)
            w = w.view(self.out_features, -1)[:, : self.in_features].contiguous()
            self.weight = nn.Parameter(w)
            self.packed_weight = None
            self.weight_scales = None
            self.is_quantized = False

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self.is_quantized:
            from .gemm import mxlinear_forward
            return mxlinear_forward(input, self.packed_weight, self.weight_scales, self.bias, self.in_features)
        if self.simulate_quantization:
            # fake quantisation: quantise -> dequantise -> dense forward (modules.py:144-150), the first two as one kernel
            from . import _capi
            w_fake = _capi.fake_quantize(self.weight.detach(), self.block_size, self.quantizer.scale_format)
            w_fake = w_fake.view(self.out_features, -1)[:, : self.in_features].to(input.dtype)
            return F.linear(input, w_fake, self.bias)
        return F.linear(input, self.weight, self.bias)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"block_size={self.block_size}, quantized={self.is_quantized}")
