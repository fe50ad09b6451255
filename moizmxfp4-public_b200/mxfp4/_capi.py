"""ctypes binding of libmxfp4_b200.so -- the only compute backend of this package.

There is no CPU implementation and no alternative GPU path: if the shared library is missing or a
tensor is not on a CUDA device, the call raises.  Build the library with
``python moizmxfp4-public_b200/build.py``.
"""
import contextlib
import ctypes
import os

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_lib", "libmxfp4_b200.so")
_lib = None

DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
SF = {"e8m0": 0, "bf16": 1}
GEMM_EXACT, GEMM_FAST = 0, 1
GEMM_CHAINED, GEMM_KEEP_PARTIALS = 1, 2
ACT_RMSNORM, ACT_SILU_MUL, ACT_SUM3, ACT_IDENTITY = 1, 2, 3, 4


class ActFusedArgs(ctypes.Structure):
    """struct mxfp4_act_fused_args of include/mxfp4_b200.h"""
    _fields_ = [("op", ctypes.c_int), ("in_bf16", ctypes.c_void_p), ("in_f32", ctypes.c_void_p), ("splits", ctypes.c_int),
                ("split_stride", ctypes.c_int64), ("ld_in", ctypes.c_int64), ("peer_blocks", ctypes.POINTER(ctypes.c_void_p)),
                ("world", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_void_p), ("peer_wait_done", ctypes.c_int),
                ("status_dev", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p), ("ld_res", ctypes.c_int64),
                ("hidden_out", ctypes.c_void_p), ("ld_hid", ctypes.c_int64), ("eps", ctypes.c_float), ("M", ctypes.c_int64),
                ("K", ctypes.c_int64), ("packed", ctypes.c_void_p), ("sf", ctypes.c_void_p), ("gamma", ctypes.c_void_p),
                ("peer_results", ctypes.POINTER(ctypes.c_void_p)), ("owner_count", ctypes.c_void_p)]


class MXFP4BackendError(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def lib_path() -> str:
    return _LIB_PATH


def load():
    """Load the shared library once; raise loudly if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"mxfp4: CUDA backend library not found at {_LIB_PATH}. Build it with "
            "`python moizmxfp4-public_b200/build.py` (needs nvcc). This package has no CPU or Triton fallback.")
    L = ctypes.CDLL(_LIB_PATH)
    i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
    L.mxfp4_version.restype = ci
    L.mxfp4_last_error.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    L.mxfp4_last_error.restype = None
    L.mxfp4_device_info.argtypes = [ctypes.POINTER(ci)] * 3
    L.mxfp4_quantize.argtypes = [vp, ci, i64, i64, i64, ci, ci, vp, vp, vp]
    L.mxfp4_dequantize.argtypes = [vp, vp, ci, i64, i64, ci, vp, ci, vp]
    L.mxfp4_fake_quantize.argtypes = [vp, ci, i64, i64, i64, ci, ci, vp, vp]
    for name in ("mxfp4_device_info", "mxfp4_quantize", "mxfp4_dequantize", "mxfp4_fake_quantize"):
        getattr(L, name).restype = ci
    L.mxfp4_act_scales_bytes.argtypes = [i64, i64]
    L.mxfp4_act_scales_bytes.restype = i64
    L.mxfp4_prepared_scales_bytes.argtypes = [i64, i64]
    L.mxfp4_prepared_scales_bytes.restype = i64
    L.mxfp4_act_quantize.argtypes = [vp, i64, i64, i64, vp, vp, vp]
    L.mxfp4_act_quantize.restype = ci
    L.mxfp4_prepare_weight_scales.argtypes = [vp, i64, i64, vp, vp]
    L.mxfp4_prepare_weight_scales.restype = ci
    L.mxfp4_gemm_workspace_bytes.argtypes = [i64, i64, i64, ci]
    L.mxfp4_gemm_workspace_bytes.restype = i64
    L.mxfp4_gemm.argtypes = [vp, i64, vp, vp, vp, vp, i64, i64, i64, i64, ci, vp, i64, vp]
    L.mxfp4_gemm.restype = ci
    L.mxfp4_gemm_prequantized.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, ci, vp, i64, vp, vp]
    L.mxfp4_gemm_noalloc.argtypes = [vp, i64, vp, vp, vp, vp, i64, i64, i64, i64, ci, vp, vp]
    L.mxfp4_gemm_noalloc.restype = ci
    L.mxfp4_gemm_splitk_bytes.argtypes = [i64, i64, i64]
    L.mxfp4_gemm_splitk_bytes.restype = i64
    L.mxfp4_gemm_prequantized.restype = ci
    L.mxfp4_gemm_prequantized_ex.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, ci, vp, i64, vp, ci, vp]
    L.mxfp4_gemm_prequantized_ex.restype = ci
    L.mxfp4_gemm_w4a16.argtypes = [vp, i64, vp, vp, ci, ci, vp, vp, i64, i64, i64, i64, vp, vp]
    L.mxfp4_gemm_w4a16.restype = ci
    L.mxfp4_gemm_plan.argtypes = [i64, i64, i64, ci, ctypes.POINTER(ci), ctypes.POINTER(ci)]
    L.mxfp4_gemm_plan.restype = ci
    L.mxfp4_act_fused_result_row_bytes.argtypes = [i64]
    L.mxfp4_act_fused_result_row_bytes.restype = i64
    L.mxfp4_act_fused.argtypes = [ctypes.POINTER(ActFusedArgs), vp]
    L.mxfp4_act_fused.restype = ci
    L.mxfp4_peer_block_bytes.argtypes = [i64, i64]
    L.mxfp4_peer_block_bytes.restype = i64
    L.mxfp4_peer_partial_offset.argtypes = []
    L.mxfp4_peer_partial_offset.restype = i64
    L.mxfp4_peer_allreduce.argtypes = [ctypes.POINTER(vp), ci, ci, vp, vp, vp, i64, i64, i64, i64, vp, vp]
    L.mxfp4_peer_allreduce.restype = ci
    _lib = L
    return L


def last_error() -> str:
    buf = ctypes.create_string_buffer(512)
    load().mxfp4_last_error(buf, 512)
    return buf.value.decode("utf-8", "replace")


def check(rc: int, what: str):
    if rc != 0:
        raise MXFP4BackendError(f"{what} failed (status {rc}): {last_error()}")


def require_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise RuntimeError(f"mxfp4: {what} needs a CUDA tensor (got device '{t.device}'); "
                           "the sm_100a backend is the only backend and there is no CPU fallback")


_NULL_CTX = contextlib.nullcontext()


def on_device(device):
    """Context that makes `device` current; free when it already is (the common case)."""
    if torch.cuda.current_device() == device.index:
        return _NULL_CTX
    return torch.cuda.device(device)


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def device_info():
    maj, mnr, sms = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    check(load().mxfp4_device_info(ctypes.byref(maj), ctypes.byref(mnr), ctypes.byref(sms)), "mxfp4_device_info")
    return maj.value, mnr.value, sms.value


# ---------------------------------------------------------------------------------------------
# Tensor-level wrappers.  Each one validates on the host, allocates outputs with torch, and
# enqueues on torch's current stream of the tensor's device.
# ---------------------------------------------------------------------------------------------
def quantize(x: torch.Tensor, block_size: int, scale_format: str):
    require_cuda(x, "MXFP4Quantizer.quantize")
    L = load()
    if x.dtype not in DT:
        x = x.float()                      # the reference upcasts everything with .float()
    if x.dim() == 0:
        raise RuntimeError("mxfp4: cannot quantize a 0-d tensor")
    cols = x.shape[-1]
    lead = tuple(x.shape[:-1])
    if x.dim() == 2 and x.stride(1) == 1 and x.stride(0) >= cols and x.numel() > 0:
        ld = x.stride(0)                   # row-strided views go straight to the kernel
    else:
        x = x.contiguous()
        ld = cols
    rows = 1
    for d in lead:
        rows *= d
    nblk = (cols + block_size - 1) // block_size
    packed = torch.empty(lead + (nblk * block_size // 2,), dtype=torch.uint8, device=x.device)
    scales = torch.empty(lead + (nblk,), dtype=torch.uint8 if scale_format == "e8m0" else torch.bfloat16, device=x.device)
    with on_device(x.device):
        check(L.mxfp4_quantize(x.data_ptr(), DT[x.dtype], rows, cols, ld, block_size, SF[scale_format],
                               packed.data_ptr(), scales.data_ptr(), stream_ptr(x.device)), "mxfp4_quantize")
    return packed, scales


def dequantize(packed: torch.Tensor, scales: torch.Tensor, block_size: int, out_dtype=torch.float32):
    require_cuda(packed, "MXFP4Quantizer.dequantize")
    L = load()
    if packed.dtype != torch.uint8:
        raise TypeError("mxfp4: packed data must be uint8")
    if scales.dtype == torch.uint8:
        fmt = "e8m0"
    else:
        fmt = "bf16"
        if scales.dtype != torch.bfloat16:
            # the reference applies scales.float(); only bf16 is produced by its quantiser, other float
            # scales are rounded here if they are not already bf16 values
            s16 = scales.to(torch.bfloat16)
            if not torch.equal(s16.float(), scales.float()):
                raise MXFP4BackendError("mxfp4: float scales must be representable in bfloat16")
            scales = s16
    packed = packed.contiguous()
    scales = scales.to(packed.device).contiguous()
    cols_pad = packed.shape[-1] * 2
    rows = packed.numel() // packed.shape[-1] if packed.shape[-1] else 0
    if scales.numel() * block_size != rows * cols_pad:
        raise RuntimeError(f"mxfp4: shape mismatch: {scales.numel()} scales x block {block_size} != {rows * cols_pad} elements")
    out = torch.empty(tuple(packed.shape[:-1]) + (cols_pad,), dtype=out_dtype, device=packed.device)
    with on_device(packed.device):
        check(L.mxfp4_dequantize(packed.data_ptr(), scales.data_ptr(), SF[fmt], rows, cols_pad, block_size,
                                 out.data_ptr(), DT[out_dtype], stream_ptr(packed.device)), "mxfp4_dequantize")
    return out


def fake_quantize(x: torch.Tensor, block_size: int, scale_format: str) -> torch.Tensor:
    """dequantize(quantize(x)) in one kernel: float32 [..., Kpad] (MXLinear.simulate_quantization)."""
    require_cuda(x, "fake_quantize")
    L = load()
    if x.dtype not in DT:
        x = x.float()
    x = x.contiguous()
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    nblk = (cols + block_size - 1) // block_size
    out = torch.empty(tuple(x.shape[:-1]) + (nblk * block_size,), dtype=torch.float32, device=x.device)
    with on_device(x.device):
        check(L.mxfp4_fake_quantize(x.data_ptr(), DT[x.dtype], rows, cols, cols, block_size, SF[scale_format], out.data_ptr(),
                                    stream_ptr(x.device)), "mxfp4_fake_quantize")
    return out
