"""Pins the CPU oracle (oracle/mxfp4_oracle.c) to outputs of the reference itself.

The fixtures under tests/golden were produced by tests/golden/make_golden.py, which runs the
reference's MXFP4Quantizer / FallbackBackend on CPU.  Everything here is bit-exact except the
matmul, whose summation order inside the BLAS is not specified.
"""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, load_matmul_cases, load_quant_cases, to_bits, weight
from oracle import oracle

CASES = load_quant_cases()


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_quantize_matches_reference(case):
    packed, scales = oracle.quantize(case["x"], case["block"], case["fmt"])
    assert packed.shape == case["packed"].shape and scales.shape == case["scales"].shape
    assert scales.dtype == case["scales"].dtype
    assert np.array_equal(to_bits(packed), to_bits(case["packed"]))
    assert np.array_equal(to_bits(scales), to_bits(case["scales"]))


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_dequantize_matches_reference(case):
    rec = oracle.dequantize(case["packed"], case["scales"], case["block"])
    assert rec.dtype == torch.float32 and rec.shape == case["rec"].shape
    assert np.array_equal(to_bits(rec), to_bits(case["rec"]))


def test_known_answer_vectors():
    """tests/test_quantizer.py:66-81 and :130-148 of the reference: [0.5,1,2,6]*8 -> byte 127, exact."""
    for sgn in (1.0, -1.0):
        data = torch.tensor([0.5, 1.0, 2.0, 6.0] * 8) * sgn
        packed, scales = oracle.quantize(data)
        assert scales.item() == 127
        assert torch.equal(oracle.dequantize(packed, scales), data)
        want = [(0 << 4 | 2), (4 << 4 | 7)] if sgn > 0 else [(8 << 4 | 10), (12 << 4 | 15)]
        assert packed.tolist() == want * 8


def test_scale_byte_exhaustive_bf16_and_f16():
    z = np.load(os.path.join(GOLDEN, "scale_exhaustive.npz"))
    v = torch.arange(1, 0x7F80, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    blk = torch.zeros(v.numel(), 32, dtype=torch.bfloat16)
    blk[:, 5] = v
    _, sc = oracle.quantize(blk)
    assert np.array_equal(sc.numpy().reshape(-1), z["bf16_scale"])
    # closed form on the bf16 bit pattern: E - 3 + [m7 >= 8], floor 98 from the 1e-8 clamp
    b = torch.arange(1, 0x7F80, dtype=torch.int32)
    closed = torch.clamp((b >> 7) - 3 + ((b & 0x7F) >= 8).int(), 98, 255)
    assert np.array_equal(closed.numpy().astype(np.uint8), z["bf16_scale"])
    vh = torch.arange(1, 0x7C00, dtype=torch.int32).to(torch.int16).view(torch.float16)
    blk = torch.zeros(vh.numel(), 32, dtype=torch.float16)
    blk[:, 11] = vh
    _, sc = oracle.quantize(blk)
    assert np.array_equal(sc.numpy().reshape(-1), z["f16_scale"])


def test_from_e8m0_all_bytes():
    z = np.load(os.path.join(GOLDEN, "from_e8m0.npz"))
    packed = torch.full((256, 16), 0x22, dtype=torch.uint8)          # code 2 = 1.0 everywhere
    rec = oracle.dequantize(packed, torch.arange(256, dtype=torch.int32).to(torch.uint8).view(256, 1))
    assert np.array_equal(to_bits(rec[:, 0]), z["values"])


def _sha(t):
    return hashlib.sha256(np.ascontiguousarray(to_bits(t)).tobytes()).hexdigest()


@pytest.mark.parametrize("tag,N,K,seed,outl", [("c1_4096x4096_seed0_outliers", 4096, 4096, 0, True),
                                               ("c2_11008x4096_seed1", 11008, 4096, 1, False)])
def test_fullsize_digests(tag, N, K, seed, outl):
    """Full-size benchmark matrices: the oracle reproduces the reference's outputs byte for byte."""
    with open(os.path.join(GOLDEN, "fullsize_digests.json")) as f:
        dig = json.load(f)[tag]
    w = weight(N, K, seed, outl)
    if _sha(w) != dig["x"]:
        pytest.skip("torch's CPU generator produced different inputs on this build")
    packed, scales = oracle.quantize(w)
    assert _sha(packed) == dig["packed"] and _sha(scales) == dig["scales"]
    assert _sha(oracle.dequantize(packed, scales)) == dig["rec"]
    assert int(scales.min()) == dig["scale_min"] and int(scales.max()) == dig["scale_max"]


MM = load_matmul_cases()


@pytest.mark.parametrize("case", MM, ids=[f"M{c['M']}N{c['N']}K{c['K']}" for c in MM])
def test_w4a16_matmul_matches_reference(case):
    """FallbackBackend.matmul: same operands, so only BLAS summation order may differ (<= 1 bf16 ulp)."""
    p, s = oracle.quantize(case["w"])
    assert torch.equal(p, case["packed"]) and torch.equal(s, case["scales"])
    y = oracle.matmul_w4a16(case["x"], p, s, case["bias"])
    assert y.dtype == torch.bfloat16
    ref = case["y"].float()
    err = (y.float() - ref).norm() / ref.norm()
    assert err < 2e-3, err
    # and the double-accumulated C matmul agrees with it to bf16 rounding
    wd = oracle.dequantize(p, s)
    y64 = oracle.matmul_nt_f64acc(case["x"].float(), wd, case["bias"])
    assert ((y64 - ref).norm() / ref.norm()) < 4e-3


def test_act_quantizer_definition():
    """The GEMM's activation quantiser: power-of-two scale 2^ceil(log2(amax/6)), RNE onto hardware E2M1."""
    x = torch.tensor([[6.0, 5.0, 3.5, 2.5, 1.75, 1.25, 0.75, 0.25, 0.26, 0.0, -0.0, -6.0, -0.5, 1.0, 1.5, 2.0] * 2,
                      [3.0, -3.0, 1.5, 0.1] * 8, [0.0] * 32, [7.0, 1.0, -1.0, 0.4] * 8], dtype=torch.bfloat16)
    p, s = oracle.act_quantize(x)
    assert s.view(-1).tolist() == [127, 126, 0, 128]
    d = oracle.act_dequantize(p, s)
    assert d[0].tolist()[:16] == [6.0, 4.0, 4.0, 2.0, 2.0, 1.0, 1.0, 0.0, 0.5, 0.0, -0.0, -6.0, -0.5, 1.0, 1.5, 2.0]
    assert d[1].tolist()[:4] == [3.0, -3.0, 1.5, 0.0]
    assert d[2].abs().max() == 0
    assert d[3].tolist()[:4] == [8.0, 1.0, -1.0, 0.0]        # scale 2: 7/2 = 3.5 ties to the even code 4.0
    g = torch.Generator().manual_seed(3)
    xr = torch.randn(64, 256, generator=g).to(torch.bfloat16)
    pr, sr = oracle.act_quantize(xr)
    dr = oracle.act_dequantize(pr, sr)
    rel = (dr - xr.float()).norm() / xr.float().norm()
    assert 0.05 < rel < 0.2
