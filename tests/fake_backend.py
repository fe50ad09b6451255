"""Test-only stand-in for the CUDA backend: routes the package's compute entry points to the CPU oracle
so that host-side logic (module surgery, sharding, state_dict flow) can be exercised without a GPU.
The shipped package never imports this file."""
import torch

from oracle import oracle


def _quantize(x, block_size, scale_format):
    return oracle.quantize(x.detach().cpu(), block_size, scale_format)


def _dequantize(packed, scales, block_size, out_dtype=torch.float32):
    return oracle.dequantize(packed, scales, block_size).to(out_dtype)


def _fake_quantize(x, block_size, scale_format):
    p, sc = oracle.quantize(x.detach().cpu(), block_size, scale_format)
    return oracle.dequantize(p, sc, block_size)


def _matmul(x, packed, scales, bias=None, out=None, reuse_act=False):
    y = oracle.matmul_operand_matched(x.detach().to(torch.bfloat16), packed, scales, None).to(torch.bfloat16)
    if bias is not None:
        y = (y.float() + bias.detach().float()).to(torch.bfloat16)
    return y.to(x.dtype)


def _forward(x, packed, scales, bias, in_features, reuse_act=False):
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    k_pad = packed.shape[-1] * 2
    if x2.shape[-1] != k_pad:
        x2 = torch.nn.functional.pad(x2, (0, k_pad - x2.shape[-1]))
    return _matmul(x2, packed, scales, bias).reshape(*lead, packed.shape[0])


def install(monkeypatch=None):
    from mxfp4 import _capi, gemm
    pairs = [(_capi, "quantize", _quantize), (_capi, "dequantize", _dequantize), (_capi, "fake_quantize", _fake_quantize),
             (gemm, "quant_matmul_2d", _matmul), (gemm, "mxlinear_forward", _forward)]
    for mod, name, fn in pairs:
        if monkeypatch is not None:
            monkeypatch.setattr(mod, name, fn)
        else:
            setattr(mod, name, fn)
