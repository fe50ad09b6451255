"""Parity of the CUDA quantiser / dequantiser with the CPU oracle and the reference's golden vectors.

Everything here is bit-exact.  Calls go through the package's public API, which binds the C ABI with
ctypes (tests/test_capi_symbols.py checks the exported symbols; tests/test_zz_no_alloc.py and tests/test_gemm_gpu.py call
C entry points directly).
"""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, load_quant_cases, to_bits, weight
from oracle import oracle

pytestmark = pytest.mark.gpu
CASES = load_quant_cases()


def same_bits(a, b):
    return a.shape == b.shape and a.dtype == b.dtype and np.array_equal(to_bits(a), to_bits(b))


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_golden_quantize_dequantize(case):
    from mxfp4.quantizer import MXFP4Quantizer
    q = MXFP4Quantizer(block_size=case["block"], scale_format=case["fmt"])
    packed, scales = q.quantize(case["x"].cuda())
    assert packed.is_cuda and scales.is_cuda
    assert same_bits(packed.cpu(), case["packed"]), "codes differ from the reference"
    assert same_bits(scales.cpu(), case["scales"]), "scales differ from the reference"
    rec = q.dequantize(packed, scales)
    assert rec.dtype == torch.float32
    assert same_bits(rec.cpu(), case["rec"]), "dequantised values differ from the reference"


def _sha(t):
    return hashlib.sha256(np.ascontiguousarray(to_bits(t)).tobytes()).hexdigest()


@pytest.mark.parametrize("tag,N,K,seed,outl", [("c1_4096x4096_seed0_outliers", 4096, 4096, 0, True),
                                               ("c2_4096x4096_seed1", 4096, 4096, 1, False),
                                               ("c2_11008x4096_seed1", 11008, 4096, 1, False)])
def test_fullsize_matches_oracle_and_reference_digest(tag, N, K, seed, outl):
    from mxfp4.quantizer import MXFP4Quantizer
    q = MXFP4Quantizer(32, "e8m0")
    w = weight(N, K, seed, outl)
    packed, scales = q.quantize(w.cuda())
    rec = q.dequantize(packed, scales)
    op, os_ = oracle.quantize(w)
    assert torch.equal(packed.cpu(), op) and torch.equal(scales.cpu(), os_)
    assert same_bits(rec.cpu(), oracle.dequantize(op, os_))
    with open(os.path.join(GOLDEN, "fullsize_digests.json")) as f:
        dig = json.load(f)[tag]
    if _sha(w) == dig["x"]:        # same inputs as when the reference produced the digests
        assert _sha(packed.cpu()) == dig["packed"] and _sha(scales.cpu()) == dig["scales"] and _sha(rec.cpu()) == dig["rec"]


def test_streaming_kernel_adversarial_blocks():
    """Every decision boundary of the rounding rule, for many block maxima and magnitudes (bf16, block 32)."""
    from mxfp4.quantizer import MXFP4Quantizer
    g = torch.Generator().manual_seed(5)
    am = torch.randint(0x0100, 0x7F00, (40000,), generator=g).to(torch.int16).view(torch.bfloat16).float()
    mids = torch.tensor([0.625, 0.875, 1.25, 1.75, 2.5, 3.5, 5.0])
    blk = torch.zeros(40000, 32)
    blk[:, 0] = am
    s = am / 6.0
    for k in range(7):
        t = mids[k] * s
        blk[:, 1 + 3 * k] = t
        blk[:, 2 + 3 * k] = torch.nextafter(t.to(torch.bfloat16).float(), torch.tensor(3e38))
        blk[:, 3 + 3 * k] = -t
    blk[:, 22:] = torch.randn(40000, 10, generator=g) * s[:, None]
    x = blk.to(torch.bfloat16)
    r = (torch.randn(40000, 32, generator=g) * torch.exp2(torch.randint(-40, 30, (40000, 1), generator=g).float())).to(torch.bfloat16)
    x = torch.cat([x, r]).view(-1, 64)             # two blocks per row
    q = MXFP4Quantizer(32, "e8m0")
    packed, scales = q.quantize(x.cuda())
    op, os_ = oracle.quantize(x)
    assert torch.equal(packed.cpu(), op) and torch.equal(scales.cpu(), os_)
    assert same_bits(q.dequantize(packed, scales).cpu(), oracle.dequantize(op, os_))
    qb = MXFP4Quantizer(32, "bf16")
    packed, scales = qb.quantize(x.cuda())
    op, os_ = oracle.quantize(x, 32, "bf16")
    assert torch.equal(packed.cpu(), op) and same_bits(scales.cpu(), os_)
    finite = torch.isfinite(os_.float()).all(-1)
    assert same_bits(qb.dequantize(packed, scales).cpu()[finite], oracle.dequantize(op, os_)[finite])


def test_every_scale_byte_dequantises_exactly():
    from mxfp4.quantizer import MXFP4Quantizer
    q = MXFP4Quantizer(32, "e8m0")
    packed = torch.randint(0, 256, (256, 64), dtype=torch.uint8, generator=torch.Generator().manual_seed(1))
    scales = torch.arange(256, dtype=torch.int32).to(torch.uint8).view(256, 1).repeat(1, 4).contiguous()
    rec = q.dequantize(packed.cuda(), scales.cuda())
    assert same_bits(rec.cpu(), oracle.dequantize(packed, scales))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape,block", [((7, 33), 32), ((3, 5, 100), 32), ((10, 64), 16), ((10, 256), 64), ((1, 32), 32), ((129,), 32)])
def test_general_kernel_shapes(dtype, shape, block):
    from mxfp4.quantizer import MXFP4Quantizer
    g = torch.Generator().manual_seed(hash((str(dtype), shape, block)) % 1000)
    x = (torch.randn(*shape, generator=g) * 0.3).to(dtype)
    for fmt in ("e8m0", "bf16"):
        q = MXFP4Quantizer(block, fmt)
        packed, scales = q.quantize(x.cuda())
        op, os_ = oracle.quantize(x, block, fmt)
        assert same_bits(packed.cpu(), op) and same_bits(scales.cpu(), os_)
        assert same_bits(q.dequantize(packed, scales).cpu(), oracle.dequantize(op, os_, block))


def test_row_strided_and_noncontiguous_inputs():
    from mxfp4.quantizer import MXFP4Quantizer
    q = MXFP4Quantizer(32, "e8m0")
    g = torch.Generator().manual_seed(9)
    base = torch.randn(64, 256, generator=g).to(torch.bfloat16)
    view = base.cuda()[:, 32:160]                 # row-strided view, 64-byte offset
    packed, scales = q.quantize(view)
    op, os_ = oracle.quantize(base[:, 32:160].contiguous())
    assert torch.equal(packed.cpu(), op) and torch.equal(scales.cpu(), os_)
    t = base.cuda().t()                           # genuinely non-contiguous
    packed, scales = q.quantize(t)
    op, os_ = oracle.quantize(base.t().contiguous())
    assert torch.equal(packed.cpu(), op) and torch.equal(scales.cpu(), os_)


def test_empty_inputs_and_errors():
    from mxfp4.quantizer import MXFP4Quantizer
    q = MXFP4Quantizer(32, "e8m0")
    packed, scales = q.quantize(torch.empty(0, 64, dtype=torch.bfloat16, device="cuda"))
    assert packed.shape == (0, 32) and scales.shape == (0, 2)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        q.quantize(torch.zeros(4, 32))             # no CPU fallback
    with pytest.raises(ValueError):
        MXFP4Quantizer(32, "fp8")


def test_roundtrip_properties_fullsize():
    """Size-independent properties at benchmark size: idempotence and sign/zero handling."""
    from mxfp4.quantizer import MXFP4Quantizer
    q = MXFP4Quantizer(32, "bf16")                 # bf16 scales: quantise(dequantise(q)) reproduces the codes
    w = weight(4096, 4096, 0, True).cuda()
    p1, s1 = q.quantize(w)
    rec = q.dequantize(p1, s1)
    p2, s2 = q.quantize(rec)
    assert torch.equal(p1, p2)
    neg = q.quantize(-w)[0]
    assert torch.equal(neg ^ 0x88, p1)             # negating the input flips exactly the two sign bits


def test_every_positive_bf16_and_fp16_block_maximum_gives_the_reference_scale_byte():
    """All 32 639 positive finite bf16 values and all 31 743 positive finite fp16 values as a block's maximum: the CUDA
    quantiser's E8M0 byte equals the byte the reference produced (tests/golden/scale_exhaustive.npz), through the
    streaming kernel (bf16, contiguous) and the general kernel (fp16; bf16 with a row stride)."""
    from mxfp4.quantizer import MXFP4Quantizer
    z = np.load(os.path.join(GOLDEN, "scale_exhaustive.npz"))
    q = MXFP4Quantizer(32, "e8m0")
    v = torch.arange(1, 0x7F80, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    blk = torch.zeros(v.numel(), 32, dtype=torch.bfloat16)
    blk[:, 5] = v
    _, sc = q.quantize(blk.cuda())
    assert np.array_equal(sc.cpu().numpy().reshape(-1), z["bf16_scale"])
    wide = torch.zeros(v.numel(), 64, dtype=torch.bfloat16)
    wide[:, 5] = v
    _, sc = q.quantize(wide.cuda()[:, :32])             # strided rows: the general kernel
    assert np.array_equal(sc.cpu().numpy().reshape(-1), z["bf16_scale"])
    vh = torch.arange(1, 0x7C00, dtype=torch.int32).to(torch.int16).view(torch.float16)
    blk = torch.zeros(vh.numel(), 32, dtype=torch.float16)
    blk[:, 11] = vh
    _, sc = q.quantize(blk.cuda())
    assert np.array_equal(sc.cpu().numpy().reshape(-1), z["f16_scale"])


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_fake_quantize_equals_quantize_then_dequantize(case):
    """mxfp4_fake_quantize (MXLinear.simulate_quantization) against the reference's recorded dequantize(quantize(x))."""
    from mxfp4 import _capi
    out = _capi.fake_quantize(case["x"].cuda(), case["block"], case["fmt"])
    assert out.dtype == torch.float32
    assert same_bits(out.cpu(), case["rec"]), "fake-quantised values differ from the reference"


def test_simulate_quantization_forward():
    """The QAT-style forward of an unquantised MXLinear: weights fake-quantised, dense forward (modules.py:144-150)."""
    from mxfp4 import MXLinear
    torch.manual_seed(3)
    layer = MXLinear(96, 40, bias=True).cuda()
    layer.simulate_quantization = True
    x = torch.randn(5, 96, device="cuda")
    y = layer(x)
    p, s = oracle.quantize(layer.weight.detach().cpu())
    w = oracle.dequantize(p, s)[:, :96]
    ref = torch.nn.functional.linear(x.cpu(), w, layer.bias.detach().cpu())
    assert torch.allclose(y.cpu(), ref, rtol=1e-4, atol=1e-5)
