"""The single compute backend of this package: hand-written sm_100a CUDA behind libmxfp4_b200.so.

The reference (src/mxfp4/backends.py) detects the GPU architecture and chooses among a third-party
QuTLASS backend, a Triton backend and a dequantise-then-matmul fallback.  Here that selection
collapses to one backend.  The names the reference exports are kept so that callers keep working:
`detect_architecture`, `MXFP4Backend`, `get_backend`, `print_backend_info`.
"""
from typing import Optional

import torch

from . import _capi

BACKEND_NAME = "sm100a"


def detect_architecture():
    """Returns (backend_name, info) like src/mxfp4/backends.py:34-131.  The backend name is always
    "sm100a"; `info["supported"]` tells whether the current device can run it."""
    info = {"backend": BACKEND_NAME, "architecture": "blackwell", "native_fp4": True}
    if not torch.cuda.is_available():
        info.update(device="none", major=0, minor=0, supported=False, reason="CUDA not available")
        return BACKEND_NAME, info
    major, minor = torch.cuda.get_device_capability()
    info.update(device=torch.cuda.get_device_name(), major=major, minor=minor, compute_capability=f"sm_{major}{minor}",
                supported=(major == 10), reason="" if major == 10 else "kernels are compiled for sm_100a only")
    return BACKEND_NAME, info


class MXFP4Backend:
    """Interface of a backend (src/mxfp4/backends.py:134-148)."""

    def quantize(self, tensor: torch.Tensor, block_size: int = 32):
        raise NotImplementedError

    def dequantize(self, packed: torch.Tensor, scales: torch.Tensor, shape: tuple):
        raise NotImplementedError

    def matmul(self, input: torch.Tensor, packed_weight: torch.Tensor, weight_scales: torch.Tensor,
               bias: Optional[torch.Tensor] = None):
        raise NotImplementedError


class B200Backend(MXFP4Backend):
    """quantize / dequantize / matmul on the sm_100a kernels."""

    def __init__(self):
        _capi.load()

    def quantize(self, tensor: torch.Tensor, block_size: int = 32):
        return _capi.quantize(tensor, block_size, "e8m0")

    def dequantize(self, packed: torch.Tensor, scales: torch.Tensor, shape: tuple = None):
        return _capi.dequantize(packed, scales, 32, torch.float32)

    def matmul(self, input: torch.Tensor, packed_weight: torch.Tensor, weight_scales: torch.Tensor,
               bias: Optional[torch.Tensor] = None):
        """[M,K] bf16 x packed [N,K/2] -> [M,N] bf16 on the block-scaled FP4 tensor cores
        (same contract as the reference backends' matmul, src/mxfp4/backends.py:191-312)."""
        from .gemm import quant_matmul_2d
        return quant_matmul_2d(input, packed_weight, weight_scales, bias)


_backend = None


def get_backend(backend: Optional[str] = "auto") -> MXFP4Backend:
    """src/mxfp4/backends.py:315-343.  Only one backend exists; "auto" and its own name select it."""
    global _backend
    if backend not in ("auto", BACKEND_NAME, "b200"):
        raise ValueError(f"Unknown backend: {backend} (this build has the single backend '{BACKEND_NAME}')")
    if _backend is None:
        _backend = B200Backend()
    return _backend


def print_backend_info():
    name, info = detect_architecture()
    print("=" * 80)
    print("MXFP4 backend")
    print("=" * 80)
    print(f"Device:   {info.get('device')}")
    if info.get("compute_capability"):
        print(f"Compute:  {info['compute_capability']}")
    print(f"Backend:  {name} (tcgen05 block-scaled FP4 tensor cores, hand-written CUDA)")
    if not info["supported"]:
        print(f"NOT SUPPORTED on this device: {info['reason']}")
    print("=" * 80)
