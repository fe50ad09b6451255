"""MXLinear.forward, quantize_model_mxfp4 and the MXLinear block stack on the GPU, against the CPU oracle and against
what the reference itself returned on CPU tensors (tests/golden/model_cases.npz).

The reference's forward (src/mxfp4/modules.py:114-140) takes N-D input, returns the input's dtype, adds the bias in
that dtype and honours block_size; its tests are tests/test_modules.py:41-78 and tests/test_utils.py:22-67.
Gate: relative Frobenius error <= 1e-2 against the operand-matched oracle (activations as the GEMM's own MXFP4
quantiser leaves them, weights exactly as the reference dequantises them); against the reference's recorded outputs
(bf16/float32 activations, no activation quantisation) only the intrinsic FP4 activation error (~0.12) is left.
"""
import pytest
import torch
import torch.nn as nn

from conftest import SmallModel, act, load_model_cases, weight
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-2
MODEL, LAYERS = load_model_cases()


def rel_fro(y, ref):
    return ((y - ref).norm() / ref.norm()).item()


def oracle_forward(x, packed, scales, bias, block, k_in):
    """MXLinear.forward restated on the oracle: flatten, pad to the packed width, bf16 activations, operand-matched
    product rounded to bf16 (the GEMM's output type), bias added as the product's epilogue (bf16 inputs) or in the
    input's dtype (everything else), leading dimensions restored."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    k_pad = packed.shape[-1] * 2
    if k_pad != x2.shape[-1]:
        x2 = torch.nn.functional.pad(x2, (0, k_pad - x2.shape[-1]))
    y = oracle.matmul_operand_matched(x2.to(torch.bfloat16), packed, scales, None, block).to(torch.bfloat16)
    if bias is not None:
        if x.dtype == torch.bfloat16:
            y = (y.float() + bias.to(torch.bfloat16).float()).to(torch.bfloat16)
        else:
            y = y.to(x.dtype) + bias.to(x.dtype)
    return y.to(x.dtype).reshape(*lead, packed.shape[0])


@pytest.mark.parametrize("case", LAYERS, ids=[f"in{c['fin']}_out{c['fout']}_b{c['block']}_{c['dtype']}" for c in LAYERS])
def test_mxlinear_forward_against_oracle_and_reference_fixture(case):
    from mxfp4 import MXLinear, gemm
    layer = MXLinear(case["fin"], case["fout"], bias=case["bias"], block_size=case["block"])
    layer.weight.data = case["w"].clone()
    if case["bias"]:
        layer.bias.data = case["b"].clone()              # float32, as MXLinear creates it
    layer = layer.cuda()
    layer.quantize()
    assert layer.weight is None and layer.is_quantized
    assert torch.equal(layer.packed_weight.cpu(), case["packed"]) and torch.equal(layer.weight_scales.cpu(), case["scales"])
    x = case["x"]
    with torch.no_grad():
        y = layer(x.cuda())
    gemm.check_status()
    assert y.dtype == x.dtype and y.shape == tuple(case["lead"]) + (case["fout"],)
    want = oracle_forward(x, case["packed"], case["scales"], case["b"], case["block"], case["fin"])
    err = rel_fro(y.float().cpu(), want.float())
    lit = rel_fro(y.float().cpu(), case["y"].float())
    print(f"block {case['block']} {case['dtype']}: rel_fro operand-matched {err:.3e}, vs the reference's forward {lit:.3e}")
    assert err <= TOL
    assert lit < 0.25


@pytest.mark.parametrize("fin,block", [(100, 32), (33, 32), (40, 16), (100, 64)])
def test_mxlinear_forward_ragged_in_features(fin, block):
    """in_features that is not a multiple of the block: the quantiser pads the weight rows, the forward pads the
    activations with zeros (the reference's own forward cannot run this case: its view to [out, in] fails)."""
    from mxfp4 import MXLinear, gemm
    torch.manual_seed(fin)
    layer = MXLinear(fin, 72, bias=True, block_size=block)
    w0, b0 = layer.weight.data.clone(), layer.bias.data.clone()
    layer = layer.cuda()
    layer.quantize()
    op, os_ = oracle.quantize(w0, block)
    assert torch.equal(layer.packed_weight.cpu(), op) and torch.equal(layer.weight_scales.cpu(), os_)
    x = torch.randn(3, 7, fin, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    with torch.no_grad():
        y = layer(x.cuda())
    gemm.check_status()
    want = oracle_forward(x, op, os_, b0, block, fin)
    assert y.shape == (3, 7, 72) and y.dtype == torch.bfloat16
    assert rel_fro(y.float().cpu(), want.float()) <= TOL
    layer.dequantize()
    assert layer.weight.shape == (72, fin) and layer.weight.dtype == torch.float32
    assert torch.equal(layer.weight.cpu(), oracle.dequantize(op, os_, block)[:, :fin])


def test_mis_shaped_scales_raise():
    """A scale tensor that does not belong to the packed weight must be refused on the host, before any kernel reads it."""
    from mxfp4 import _capi, quant_matmul
    op, os_ = oracle.quantize(weight(64, 256, 1, False))
    x = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    for bad in (os_[:32], os_[:, :5], os_.view(-1), torch.zeros(64, 256 // 8, dtype=torch.uint8), torch.zeros(64, 1, dtype=torch.uint8)):
        with pytest.raises(_capi.MXFP4BackendError):
            quant_matmul(x, op.cuda(), bad.cuda())


def test_quantize_model_state_dict_equals_reference_fixture(capsys):
    """quantize_model_mxfp4 on the seeded model: same keys, same bytes in every packed weight, scale and bias as the
    reference's own call produced (src/mxfp4/utils/model_utils.py:8-73), head excluded; forward against the oracle
    evaluated layer by layer and against the reference's recorded outputs."""
    from mxfp4 import MXLinear, gemm, get_model_size_mb, quantize_model_mxfp4
    model = SmallModel()
    model.load_state_dict(MODEL["init"])
    model = model.cuda()
    before = get_model_size_mb(model)
    out = quantize_model_mxfp4(model, exclude_layers=["head"])
    assert out is model and "Quantized 2 Linear layers." in capsys.readouterr().out
    assert isinstance(model.body[0], MXLinear) and isinstance(model.body[2], MXLinear) and isinstance(model.head, nn.Linear)
    assert get_model_size_mb(model) < before
    sd = model.state_dict()
    assert list(sd.keys()) == MODEL["keys"]
    for k in MODEL["keys"]:
        assert sd[k].dtype == MODEL["q"][k].dtype and torch.equal(sd[k].cpu(), MODEL["q"][k]), k
    for x, y_ref in ((MODEL["x2"], MODEL["y2"]), (MODEL["x3"], MODEL["y3"])):
        with torch.no_grad():
            y = model(x.cuda())
        gemm.check_status()
        assert y.shape == y_ref.shape and y.dtype == torch.float32
        q = MODEL["q"]
        h = oracle_forward(x, q["body.0.packed_weight"], q["body.0.weight_scales"], q["body.0.bias"], 32, 64)
        h = oracle_forward(torch.relu(h), q["body.2.packed_weight"], q["body.2.weight_scales"], None, 32, 128)
        want = torch.nn.functional.linear(h, q["head.weight"], q["head.bias"])
        assert rel_fro(y.cpu(), want) <= TOL
        assert rel_fro(y.cpu(), y_ref) < 0.25
    # the reference's load flow (tests/test_modules.py:80-112): quantize() a fresh layer, then load the packed state
    fresh = SmallModel().cuda()
    quantize_model_mxfp4(fresh, exclude_layers=["head"], verbose=False)
    fresh.load_state_dict({k: v.cuda() for k, v in MODEL["q"].items()})
    with torch.no_grad():
        assert torch.equal(fresh(MODEL["x2"].cuda()), model(MODEL["x2"].cuda()))


def test_block_stack_against_layer_by_layer_oracle():
    """Two layers of the Llama-shaped MXLinear block stack at M = 128: the GPU stack against the same arithmetic on the
    CPU with every GEMM replaced by the operand-matched oracle (bf16 between the operations, as on the GPU)."""
    from mxfp4 import gemm
    from mxfp4.parallel import MXBlockStack
    hidden, inter, n_layers, M = 512, 1536, 2, 128
    x = act(M, hidden, 11)
    stack = MXBlockStack.build(n_layers=n_layers, hidden=hidden, inter=inter, device="cuda", seed=3)
    with torch.no_grad():
        y = stack(x.cuda())
    gemm.check_status()

    def lin(h, n, k, seed):
        w = (torch.randn(n, k, generator=torch.Generator().manual_seed(seed)) * 0.02).to(torch.bfloat16)
        p, s = oracle.quantize(w)
        return oracle.matmul_operand_matched(h, p, s).to(torch.bfloat16)

    def norm(h):
        return torch.nn.functional.rms_norm(h.float(), (h.shape[-1],), eps=1e-6).to(torch.bfloat16)

    h = x
    for li in range(n_layers):
        s0 = 3 + li * 7
        t = norm(h)
        a = lin(t, hidden, hidden, s0) + lin(t, hidden, hidden, s0 + 1) + lin(t, hidden, hidden, s0 + 2)
        h = h + lin(a, hidden, hidden, s0 + 3)
        t = norm(h)
        g = torch.nn.functional.silu(lin(t, inter, hidden, s0 + 4)) * lin(t, inter, hidden, s0 + 5)
        h = h + lin(g, hidden, inter, s0 + 6)
    err = rel_fro(y.float().cpu(), h.float())
    print(f"2-layer stack, M={M}: rel_fro vs layer-by-layer oracle {err:.3e}")
    assert torch.isfinite(y.float()).all() and err <= TOL
