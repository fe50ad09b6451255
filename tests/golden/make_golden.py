#!/usr/bin/env python
"""Regenerate the golden fixtures in this folder by running the reference's own CPU code.

Usage (only where a checkout of the reference is available):

    python tests/golden/make_golden.py --reference /path/to/MoizMXFP4-public

The script imports the reference package from ``<reference>/src`` and records, for seeded and
hand-built inputs, exactly what ``MXFP4Quantizer.quantize`` / ``.dequantize``
(src/mxfp4/quantizer.py:71-198) and ``FallbackBackend.matmul`` (src/mxfp4/backends.py:295-312) return
on CPU tensors.  Floating-point tensors are stored as raw bit patterns (uint16 for bf16/fp16, uint32
for fp32) so that the fixtures are bit-exact and independent of numpy's dtype support.

Files written:
  quant_cases.npz        small quantise/dequantise cases (all dtypes, block sizes, scale formats,
                         ragged K, N-D, adversarial blocks, the reference tests' known-answer vectors)
  scale_exhaustive.npz   scale byte for every positive finite bf16 and fp16 value used as block maximum
  from_e8m0.npz          _from_e8m0 for all 256 bytes
  matmul_cases.npz       FallbackBackend.matmul (W4A16 dequantise-then-matmul) on small shapes
  model_cases.npz        quantize_model_mxfp4 on a small seeded model (state_dict before and after, forward
                         outputs for 2-D/3-D inputs) and MXLinear.forward for block sizes 16/32/64, ragged
                         in_features, float32 / float16 / bfloat16 inputs
  fullsize_digests.json  sha256 of inputs and outputs for the full-size benchmark matrices
"""
import argparse
import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    """Raw bit pattern of a tensor as an unsigned numpy array of the same shape."""
    t = t.detach().contiguous().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype == torch.float32:
        return t.view(torch.int32).numpy().view(np.uint32).copy()
    if t.dtype == torch.uint8:
        return t.numpy().copy()
    raise TypeError(t.dtype)


def weight(N, K, seed, outliers):
    """Benchmark weight generator: N(0, 0.02) with optionally 0.1 % of entries scaled x50."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.02
    if outliers:
        idx = torch.randperm(N * K, generator=g)[: int(0.001 * N * K)]
        w.view(-1)[idx] *= 50
    return w.to(torch.bfloat16)


def act(M, K, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, K, generator=g).to(torch.bfloat16)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def adversarial_blocks_bf16():
    """Blocks built to sit on every decision boundary of the reference's rounding."""
    rows = []
    mids = [0.625, 0.875, 1.25, 1.75, 2.5, 3.5, 5.0]
    levels = [0.5, 0.75, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    # maximum 6.0 -> scale 1.0: midpoints and levels land exactly, both signs
    r = [6.0] + mids + [-m for m in mids] + levels + [-l for l in levels] + [0.0]
    rows.append(r[:32])
    # same pattern scaled by powers of two and by awkward maxima
    for mx in [6.0 * 2 ** -9, 6.0 * 2 ** 7, 3.0, 1.0, 0.02, 0.0123, 7.5, 1e-3, 100.0, 2.0 ** -20]:
        s = mx / 6.0
        rows.append(([mx] + [m * s for m in mids] + [-m * s for m in mids] + [l * s for l in levels]
                     + [-l * s for l in levels] + [0.0])[:32])
    rows.append([0.0] * 32)                       # all-zero block (scale clamps to 1e-8/6)
    rows.append([-0.0] * 32)                      # negative zeros: sign bit must stay clear
    rows.append([0.0, -0.0] * 15 + [1.0, -1.0])
    rows.append([0.37] * 32)                      # all equal
    rows.append([-0.37] * 32)
    rows.append([0.001] * 31 + [5.0])             # single outlier
    rows.append([1e-6, 1e-7, 1e-8] * 10 + [0.0, 0.0])
    rows.append([1e6, 2e6, 3e6, 6e6] * 8)
    rows.append([1.0, 1e6] * 16)
    rows.append([1.0, -1.0, 2.0, -2.0, 3.0, -3.0, 4.0, -4.0] * 4)
    rows.append([2.0 ** -126, -(2.0 ** -126), 2.0 ** -130, 2.0 ** -133] * 8)   # bf16 subnormals
    rows.append([3.0e38, -3.0e38, 1.0e38, 1.0] * 8)                            # near bf16 max
    rows.append([2.0 ** 20, -(2.0 ** -133), 2.0 ** -133, -(2.0 ** -120)] * 8)  # quotient underflow
    rows.append([2.0 ** 17 * 6, -(2.0 ** -133), 2.0 ** -132, -(2.0 ** -131)] * 8)
    return torch.tensor(rows, dtype=torch.float32).to(torch.bfloat16)


class SmallModel(torch.nn.Module):
    """The model of the reference's tests/test_utils.py:8-20 (fc1, act, fc2, head), one level deeper."""

    def __init__(self):
        super().__init__()
        self.body = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 96, bias=False))
        self.head = torch.nn.Linear(96, 10)

    def forward(self, x):
        return self.head(self.body(x))


def model_cases(args):
    """quantize_model_mxfp4 (src/mxfp4/utils/model_utils.py:8-73) and MXLinear.forward (src/mxfp4/modules.py:114-140)
    as the reference computes them on CPU tensors."""
    from mxfp4 import MXLinear, quantize_model_mxfp4
    out, names = {}, []
    torch.manual_seed(2024)
    model = SmallModel()
    for k, v in model.state_dict().items():
        out[f"model_init_{k}"] = bits(v)
    x2 = torch.randn(5, 64, generator=torch.Generator().manual_seed(1))
    x3 = torch.randn(2, 3, 64, generator=torch.Generator().manual_seed(2))
    quantize_model_mxfp4(model, exclude_layers=["head"], verbose=False)
    for k, v in model.state_dict().items():
        out[f"model_q_{k}"] = bits(v)
    out["model_q_keys"] = np.array(list(model.state_dict().keys()))
    with torch.no_grad():
        out["model_x2"], out["model_y2"] = bits(x2), bits(model(x2))
        out["model_x3"], out["model_y3"] = bits(x3), bits(model(x3))
    # single layers: (in, out, bias, block, input dtype, leading shape).  in_features is a multiple of the block: the
    # reference's forward cannot view a padded weight as [out, in] (modules.py:132) for anything else.
    for i, (fin, fout, bias, block, dt, lead) in enumerate([(128, 64, True, 32, "float32", (8,)), (64, 48, True, 32, "bfloat16", (2, 3)),
                                                            (256, 32, False, 32, "float16", (4,)), (64, 40, True, 16, "float32", (6,)),
                                                            (128, 24, True, 64, "bfloat16", (3, 2)), (96, 16, True, 16, "bfloat16", (5,))]):
        torch.manual_seed(100 + i)
        layer = MXLinear(fin, fout, bias=bias, block_size=block)
        w0 = layer.weight.data.clone()
        tdt = getattr(torch, dt)
        x = torch.randn(*lead, fin, generator=torch.Generator().manual_seed(200 + i)).to(tdt)
        layer.quantize()
        if dt != "float32":
            layer = layer.to(tdt)          # as model.to(bfloat16) does: the bias follows the activations' dtype
        with torch.no_grad():
            y = layer(x)
        assert y.dtype == tdt
        names.append(json.dumps(dict(fin=fin, fout=fout, bias=bias, block=block, dtype=dt, lead=list(lead))))
        out[f"l{i}_w"] = bits(w0)
        if bias:
            out[f"l{i}_b"] = bits(layer.bias.data.float())
        out[f"l{i}_packed"] = bits(layer.packed_weight)
        out[f"l{i}_scales"] = bits(layer.weight_scales)
        out[f"l{i}_x"] = bits(x)
        out[f"l{i}_y"] = bits(y)
    out["layer_meta"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "model_cases.npz"), **out)
    print(f"model_cases.npz: model + {len(names)} layers")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path to a checkout of moizyousufi/MoizMXFP4-public")
    ap.add_argument("--skip-fullsize", action="store_true")
    ap.add_argument("--only-model", action="store_true", help="write model_cases.npz only")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    from mxfp4.quantizer import MXFP4Quantizer           # noqa: E402
    from mxfp4.backends import get_backend               # noqa: E402

    torch.set_num_threads(os.cpu_count())
    meta = {"torch": torch.__version__}
    model_cases(args)
    if args.only_model:
        return

    # ---------------------------------------------------------------- quantise / dequantise cases
    cases = []

    def add(name, x, block=32, fmt="e8m0"):
        q = MXFP4Quantizer(block_size=block, scale_format=fmt)
        packed, scales = q.quantize(x)
        rec = q.dequantize(packed, scales)
        assert rec.dtype == torch.float32
        cases.append(dict(name=name, x=x, block=block, fmt=fmt, packed=packed, scales=scales, rec=rec))

    g = torch.Generator().manual_seed(1234)
    add("known_answer_pos", torch.tensor([0.5, 1.0, 2.0, 6.0] * 8))              # tests/test_quantizer.py:66
    add("known_answer_neg", torch.tensor([-0.5, -1.0, -2.0, -6.0] * 8))          # tests/test_quantizer.py:130
    add("zeros_128", torch.zeros(128))                                             # tests/test_quantizer.py:150
    add("mixed_signs", torch.tensor([1.0, -1.0, 2.0, -2.0, 3.0, -3.0, 4.0, -4.0] * 4))
    add("tiny_values", torch.tensor([1e-6, 1e-7, 1e-8] * 10 + [0.0]))              # ragged: 31 elements
    add("large_values", torch.tensor([1e6, 2e6, 3e6, 6e6] * 8))
    add("multi_magnitude", torch.tensor([1.0, 1e6] * 16))
    add("adversarial_bf16", adversarial_blocks_bf16())
    add("adversarial_bf16_bf16scale", adversarial_blocks_bf16(), fmt="bf16")
    add("bf16_weightlike_64x256", weight(64, 256, 7, True))
    add("bf16_randn_33x96", torch.randn(33, 96, generator=g).to(torch.bfloat16))
    add("bf16_ragged_5x100", torch.randn(5, 100, generator=g).to(torch.bfloat16))
    add("bf16_ragged_7x33", (torch.randn(7, 33, generator=g) * 3).to(torch.bfloat16))
    add("bf16_nd_2x3x4x64", torch.randn(2, 3, 4, 64, generator=g).to(torch.bfloat16))
    add("bf16_1d_33", torch.randn(33, generator=g).to(torch.bfloat16))
    add("bf16_block16", torch.randn(10, 64, generator=g).to(torch.bfloat16), block=16)
    add("bf16_block64", torch.randn(10, 256, generator=g).to(torch.bfloat16), block=64)
    add("bf16_block64_ragged", torch.randn(3, 100, generator=g).to(torch.bfloat16), block=64)
    add("bf16_bf16scale", weight(16, 128, 9, True), fmt="bf16")
    add("f32_randn_128x128_seed42", torch.randn(128, 128, generator=torch.Generator().manual_seed(42)))
    add("f32_randn_10x64", torch.randn(10, 64, generator=g))
    add("f32_ragged_9x70", torch.randn(9, 70, generator=g) * 0.02)
    add("f32_block16", torch.randn(10, 64, generator=g), block=16)
    add("f32_block64", torch.randn(10, 256, generator=g), block=64)
    add("f32_bf16scale", torch.randn(8, 96, generator=g), fmt="bf16")
    add("f16_randn_12x128", torch.randn(12, 128, generator=g).to(torch.float16))
    add("f16_ragged_4x50", (torch.randn(4, 50, generator=g) * 0.1).to(torch.float16))
    add("f16_bf16scale", torch.randn(4, 64, generator=g).to(torch.float16), fmt="bf16")

    out = {}
    names = []
    for i, c in enumerate(cases):
        names.append(json.dumps(dict(name=c["name"], block=c["block"], fmt=c["fmt"],
                                     dtype=str(c["x"].dtype).replace("torch.", ""),
                                     shape=list(c["x"].shape))))
        out[f"c{i}_x"] = bits(c["x"])
        out[f"c{i}_packed"] = bits(c["packed"])
        out[f"c{i}_scales"] = bits(c["scales"])
        out[f"c{i}_rec"] = bits(c["rec"])
    out["meta"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "quant_cases.npz"), **out)
    print(f"quant_cases.npz: {len(cases)} cases")

    # ---------------------------------------------------------------- exhaustive scale bytes
    q = MXFP4Quantizer(32, "e8m0")
    b16 = torch.arange(1, 0x7F80, dtype=torch.int32).to(torch.int16)          # every positive finite bf16
    v = b16.view(torch.bfloat16)
    blk = torch.zeros(v.numel(), 32, dtype=torch.bfloat16)
    blk[:, 5] = v
    _, sc_bf16 = q.quantize(blk)
    h16 = torch.arange(1, 0x7C00, dtype=torch.int32).to(torch.int16)          # every positive finite fp16
    vh = h16.view(torch.float16)
    blk = torch.zeros(vh.numel(), 32, dtype=torch.float16)
    blk[:, 11] = vh
    _, sc_f16 = q.quantize(blk)
    np.savez_compressed(os.path.join(HERE, "scale_exhaustive.npz"),
                        bf16_scale=bits(sc_bf16).reshape(-1), f16_scale=bits(sc_f16).reshape(-1))
    np.savez_compressed(os.path.join(HERE, "from_e8m0.npz"),
                        values=bits(q._from_e8m0(torch.arange(256, dtype=torch.int32).to(torch.uint8))))
    print("scale_exhaustive.npz, from_e8m0.npz")

    # ---------------------------------------------------------------- W4A16 matmul (FallbackBackend)
    fb = get_backend("fallback")
    mm = {}
    mnames = []
    for i, (M, N, K, with_bias, seed) in enumerate([(16, 64, 128, False, 11), (128, 128, 128, True, 12),
                                                    (1, 96, 256, True, 13), (33, 48, 64, False, 14)]):
        w = weight(N, K, seed, True)
        x = act(M, K, 1000 + seed)
        packed, scales = q.quantize(w)
        bias = (torch.randn(N, generator=torch.Generator().manual_seed(seed)) * 0.1).to(torch.bfloat16) \
            if with_bias else None
        y = fb.matmul(x, packed, scales, None if bias is None else bias.clone())
        assert y.dtype == torch.bfloat16
        mnames.append(json.dumps(dict(M=M, N=N, K=K, bias=with_bias, seed=seed)))
        mm[f"m{i}_x"] = bits(x)
        mm[f"m{i}_w"] = bits(w)
        mm[f"m{i}_packed"] = bits(packed)
        mm[f"m{i}_scales"] = bits(scales)
        if bias is not None:
            mm[f"m{i}_bias"] = bits(bias)
        mm[f"m{i}_y"] = bits(y)
    mm["meta"] = np.array(mnames)
    np.savez_compressed(os.path.join(HERE, "matmul_cases.npz"), **mm)
    print("matmul_cases.npz")

    # ---------------------------------------------------------------- full-size digests
    if not args.skip_fullsize:
        dig = {}
        for tag, (N, K, seed, outl) in {"c1_4096x4096_seed0_outliers": (4096, 4096, 0, True),
                                        "c2_4096x4096_seed1": (4096, 4096, 1, False),
                                        "c2_11008x4096_seed1": (11008, 4096, 1, False)}.items():
            w = weight(N, K, seed, outl)
            ps, ss, rs = [], [], []
            for r0 in range(0, N, 1024):       # row chunks bound the reference's 8x fp32 temporary
                p, s = q.quantize(w[r0:r0 + 1024])
                ps.append(p); ss.append(s); rs.append(q.dequantize(p, s))
            packed, scales, rec = torch.cat(ps), torch.cat(ss), torch.cat(rs)
            dig[tag] = dict(x=sha(bits(w)), packed=sha(bits(packed)), scales=sha(bits(scales)),
                            rec=sha(bits(rec)), scale_min=int(scales.min()), scale_max=int(scales.max()))
            print(tag, dig[tag])
        dig["_meta"] = meta
        with open(os.path.join(HERE, "fullsize_digests.json"), "w") as f:
            json.dump(dig, f, indent=1)


if __name__ == "__main__":
    main()
