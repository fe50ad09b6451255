"""MXFP4Quantizer -- same class, arguments and results as the reference's
src/mxfp4/quantizer.py:3-198, computed by the sm_100a CUDA kernels behind the C ABI.

Numerics kept exactly (they differ from OCP/hardware E2M1 on purpose, because the reference does):
the 8 magnitudes are {0.5, 0.75, 1, 1.5, 2, 3, 4, 6} (no zero), ties round to the smaller magnitude,
codes are taken against s = amax/6 while the stored E8M0 byte is round(log2 s)+127, the even element
of each pair sits in the high nibble, and dequantize returns float32 of the padded width.
"""
import torch

from . import _capi


class MXFP4Quantizer:
    def __init__(self, block_size: int = 32, scale_format: str = "e8m0"):
        """
        Args:
            block_size: elements per quantisation block (default 32)
            scale_format: "e8m0" (uint8 power-of-two scales) or "bf16"
        """
        self.block_size = block_size
        self.scale_format = scale_format
        if scale_format not in ["e8m0", "bf16"]:
            raise ValueError(f"scale_format must be 'e8m0' or 'bf16', got {scale_format}")
        self.E2M1_VALUES = torch.tensor([0.5, 0.75, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=torch.float32)

    # -- small helpers of the reference's public surface (quantizer.py:35-69); plain tensor algebra --
    def _to_e8m0(self, bf16_scale: torch.Tensor) -> torch.Tensor:
        exponent = torch.round(torch.log2(torch.clamp(bf16_scale, min=1e-10))) + 127
        return torch.clamp(exponent, 0, 255).to(torch.uint8)

    def _from_e8m0(self, e8m0_scale: torch.Tensor) -> torch.Tensor:
        return torch.pow(2.0, e8m0_scale.to(torch.float32) - 127)

    def _pad_tensor(self, tensor: torch.Tensor):
        last_dim = tensor.shape[-1]
        if last_dim % self.block_size != 0:
            pad_len = self.block_size - (last_dim % self.block_size)
            return torch.nn.functional.pad(tensor, (0, pad_len)), pad_len
        return tensor, 0

    def quantize(self, tensor: torch.Tensor):
        """Returns (packed uint8 [..., Kpad/2], scales uint8-or-bf16 [..., Kpad/block_size]) on the
        input's device (quantizer.py:71-141).  Padding to a multiple of block_size happens inside
        the kernel; no padded copy of the input is made."""
        return _capi.quantize(tensor, self.block_size, self.scale_format)

    def dequantize(self, packed_data: torch.Tensor, scales: torch.Tensor, output_shape=None):
        """Returns float32 [..., Kpad] (quantizer.py:143-198).  `output_shape` is accepted and ignored,
        as in the reference."""
        return _capi.dequantize(packed_data, scales, self.block_size, torch.float32)
