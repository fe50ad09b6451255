"""ctypes front end of the CPU oracle (oracle/mxfp4_oracle.c).

TEST INFRASTRUCTURE ONLY.  The oracle is the checker for the CUDA path and the timed CPU baseline of
the benchmark; the shipped package never imports this module.  Each function takes and returns
torch CPU tensors so that parity tests read like the reference's own tests
(MXFP4Quantizer.quantize / dequantize, src/mxfp4/quantizer.py:71-198; FallbackBackend.matmul,
src/mxfp4/backends.py:295-312).

`build()` compiles the C file with gcc (OpenMP) into oracle/_build/libmxfp4_oracle.so.  When a
checkout of the reference is present the same call also refreshes nothing else: the reference is pure
Python, it has no C sources to compile into oracle/_ref, so the restatement is pinned through the
golden fixtures under tests/golden instead.
"""
import ctypes
import os
import subprocess

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "mxfp4_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libmxfp4_oracle.so")

_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
_SF = {"e8m0": 0, "bf16": 1}
_lib = None


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-shared", "-fPIC",
               "-o", LIB, SRC, "-lm"]
        subprocess.run(cmd, check=True)
    return LIB


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(LIB)
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.mxfp4_oracle_quantize.argtypes = [vp, ci, i64, i64, ci, ci, vp, vp]
        L.mxfp4_oracle_dequantize.argtypes = [vp, vp, ci, i64, i64, ci, vp]
        L.mxfp4_oracle_act_quantize.argtypes = [vp, i64, i64, vp, vp]
        L.mxfp4_oracle_act_dequantize.argtypes = [vp, vp, i64, i64, vp]
        L.mxfp4_oracle_matmul_nt.argtypes = [vp, vp, vp, i64, i64, i64, vp]
        for f in (L.mxfp4_oracle_quantize, L.mxfp4_oracle_dequantize, L.mxfp4_oracle_act_quantize,
                  L.mxfp4_oracle_act_dequantize, L.mxfp4_oracle_matmul_nt, L.mxfp4_oracle_num_threads):
            f.restype = ci
        _lib = L
    return _lib


def num_threads() -> int:
    return int(lib().mxfp4_oracle_num_threads())


def _check(rc, what):
    if rc != 0:
        raise ValueError(f"oracle {what} rejected its arguments (rc={rc})")


def quantize(x: torch.Tensor, block_size: int = 32, scale_format: str = "e8m0"):
    """MXFP4Quantizer(block_size, scale_format).quantize(x) on a CPU tensor."""
    assert x.device.type == "cpu"
    if x.dtype not in _DT:
        x = x.float()
    x = x.contiguous()
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    nblk = (cols + block_size - 1) // block_size
    lead = tuple(x.shape[:-1])
    packed = torch.empty(lead + (nblk * block_size // 2,), dtype=torch.uint8)
    scales = torch.empty(lead + (nblk,), dtype=torch.uint8 if scale_format == "e8m0" else torch.bfloat16)
    _check(lib().mxfp4_oracle_quantize(x.data_ptr(), _DT[x.dtype], rows, cols, block_size, _SF[scale_format],
                                       packed.data_ptr(), scales.data_ptr()), "quantize")
    return packed, scales


def dequantize(packed: torch.Tensor, scales: torch.Tensor, block_size: int = 32) -> torch.Tensor:
    """MXFP4Quantizer(block_size).dequantize(packed, scales): float32, padded width."""
    assert packed.device.type == "cpu" and packed.dtype == torch.uint8
    packed = packed.contiguous()
    fmt = "e8m0" if scales.dtype == torch.uint8 else "bf16"
    if fmt == "bf16" and scales.dtype != torch.bfloat16:
        raise TypeError("oracle dequantize takes uint8 or bfloat16 scales")
    scales = scales.contiguous()
    cols_pad = packed.shape[-1] * 2
    rows = packed.numel() // packed.shape[-1] if packed.shape[-1] else 0
    out = torch.empty(tuple(packed.shape[:-1]) + (cols_pad,), dtype=torch.float32)
    _check(lib().mxfp4_oracle_dequantize(packed.data_ptr(), scales.data_ptr(), _SF[fmt], rows, cols_pad,
                                         block_size, out.data_ptr()), "dequantize")
    return out


def act_quantize(x: torch.Tensor):
    """Activation quantiser of the GEMM: bf16 [M,K] -> (packed u8 [M,K/2], e8m0 u8 [M,K/32])."""
    assert x.dtype == torch.bfloat16 and x.dim() == 2
    x = x.contiguous()
    M, K = x.shape
    packed = torch.empty(M, K // 2, dtype=torch.uint8)
    scales = torch.empty(M, K // 32, dtype=torch.uint8)
    _check(lib().mxfp4_oracle_act_quantize(x.data_ptr(), M, K, packed.data_ptr(), scales.data_ptr()), "act_quantize")
    return packed, scales


def act_dequantize(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    M, K2 = packed.shape
    out = torch.empty(M, K2 * 2, dtype=torch.float32)
    _check(lib().mxfp4_oracle_act_dequantize(packed.contiguous().data_ptr(), scales.contiguous().data_ptr(),
                                             M, K2 * 2, out.data_ptr()), "act_dequantize")
    return out


def matmul_nt_f64acc(a: torch.Tensor, w: torch.Tensor, bias=None) -> torch.Tensor:
    """a[M,K] . w[N,K]^T (+bias) with double accumulation; small shapes only (naive loops)."""
    a = a.float().contiguous()
    w = w.float().contiguous()
    b = None if bias is None else bias.float().contiguous()
    M, K = a.shape
    N = w.shape[0]
    out = torch.empty(M, N, dtype=torch.float32)
    _check(lib().mxfp4_oracle_matmul_nt(a.data_ptr(), w.data_ptr(), None if b is None else b.data_ptr(),
                                        M, N, K, out.data_ptr()), "matmul")
    return out


def matmul_w4a16(x: torch.Tensor, packed_w: torch.Tensor, w_scales: torch.Tensor, bias=None, block_size: int = 32) -> torch.Tensor:
    """FallbackBackend.matmul (src/mxfp4/backends.py:295-312): dequantise the weight, cast it to the
    input dtype, torch.matmul, add the bias in the output dtype."""
    wd = dequantize(packed_w, w_scales, block_size)
    out = torch.matmul(x, wd.T.to(x.dtype))
    if bias is not None:
        out += bias
    return out


def act_fake_quantize(x: torch.Tensor, block_size: int = 32) -> torch.Tensor:
    """bf16 activations as the GEMM sees them: quantised by its own MXFP4 quantiser and decoded again, float32.
    For block-16 weights the GEMM quantises every 16 elements as a group of their own (padded with zeros to the
    32 elements the tensor cores scale together); 32- and 64-element weight blocks use 32-element groups."""
    M, K = x.shape
    if block_size == 16:
        xs = torch.nn.functional.pad(x.reshape(M, K // 16, 16), (0, 16)).reshape(M, 2 * K).contiguous()
        ap, asc = act_quantize(xs)
        return act_dequantize(ap, asc).reshape(M, K // 16, 32)[:, :, :16].reshape(M, K).contiguous()
    ap, asc = act_quantize(x)
    return act_dequantize(ap, asc)


def matmul_operand_matched(x: torch.Tensor, packed_w: torch.Tensor, w_scales: torch.Tensor, bias=None, block_size: int = 32,
                           rows=None) -> torch.Tensor:
    """The gated GEMM oracle: float32 product of the operands the tensor cores actually see --
    activations after the GEMM's own MXFP4 quantiser, weights exactly as the reference dequantises
    them -- plus the bias, left in float32.  `rows` (an index tensor) restricts the product to a sample of the
    activation rows, for shapes whose full product would take the CPU too long."""
    a = act_fake_quantize(x.contiguous(), block_size)
    if rows is not None:
        a = a[rows]
    wd = dequantize(packed_w, w_scales, block_size)
    out = torch.matmul(a, wd.T)
    if bias is not None:
        out = out + bias.float()
    return out
