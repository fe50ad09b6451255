"""Host-side behaviour of the reference's API surface, run on CPU with the oracle standing in for the
CUDA backend (tests/fake_backend.py).  Mirrors the reference's tests/test_modules.py and tests/test_utils.py."""
import pytest
import torch
import torch.nn as nn

import fake_backend


@pytest.fixture(autouse=True)
def oracle_backend(monkeypatch):
    fake_backend.install(monkeypatch)


def test_public_names():
    import mxfp4
    for name in ["MXFP4Quantizer", "MXLinear", "quantize_model_mxfp4", "get_model_size_mb", "quant_matmul", "print_architecture_info"]:
        assert hasattr(mxfp4, name)
    q = mxfp4.MXFP4Quantizer()
    assert q.block_size == 32 and q.scale_format == "e8m0" and len(q.E2M1_VALUES) == 8
    with pytest.raises(ValueError):
        mxfp4.MXFP4Quantizer(scale_format="int8")
    x = torch.randn(33)
    padded, pad_len = q._pad_tensor(x)
    assert padded.shape[0] == 64 and pad_len == 31
    assert q._to_e8m0(torch.tensor([1.0, 0.5, 3.0])).tolist() == [127, 126, 129]
    assert q._from_e8m0(torch.tensor([127, 128], dtype=torch.uint8)).tolist() == [1.0, 2.0]


def test_no_cpu_fallback_in_the_product():
    """Without the test stand-in, CPU tensors are refused."""
    from mxfp4 import _capi
    import importlib
    real = importlib.reload(_capi)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        real.quantize(torch.zeros(4, 32), 32, "e8m0")


def test_mxlinear_quantize_and_state_dict_flow():
    from mxfp4 import MXLinear
    layer = MXLinear(64, 64)
    assert layer.weight.shape == (64, 64) and not layer.is_quantized
    layer.quantize()
    assert layer.is_quantized and layer.weight is None
    assert layer.packed_weight.numel() == 2048 and layer.packed_weight.dtype == torch.uint8
    assert layer.weight_scales.shape == (64, 2)
    layer.quantize()                                   # second call is a no-op
    sd = layer.state_dict()
    assert "packed_weight" in sd and "weight_scales" in sd and "weight" not in sd
    new = MXLinear(64, 64)
    new.quantize()
    new.load_state_dict(sd)
    assert torch.equal(new.packed_weight, layer.packed_weight)
    x = torch.randn(3, 5, 64)
    y = layer(x)
    assert y.shape == (3, 5, 64) and y.dtype == x.dtype
    layer.dequantize()
    assert not layer.is_quantized and layer.weight.shape == (64, 64) and layer.weight.dtype == torch.float32
    empty = MXLinear(32, 32)
    empty.quantize()
    empty.is_quantized = False
    with pytest.raises(ValueError, match="No weights to quantize"):
        empty.quantize()
    assert "quantized=" in repr(layer)


def test_forward_close_to_dense():
    from mxfp4 import MXLinear
    torch.manual_seed(0)
    layer = MXLinear(128, 64)
    x = torch.randn(8, 128)
    ref = layer(x)
    layer.quantize()
    out = layer(x)
    assert (out - ref).abs().mean() < 0.5               # the reference's own CPU forward tolerance


class SimpleModel(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(64, 128)
        self.act = nn.ReLU()
        self.fc2 = nn.Linear(128, 64)
        self.head = nn.Linear(64, 10)

    def forward(self, x):
        return self.head(self.fc2(self.act(self.fc1(x))))


def test_quantize_model_and_size(capsys):
    from mxfp4 import MXLinear, get_model_size_mb, quantize_model_mxfp4
    model = SimpleModel()
    before = get_model_size_mb(model)
    out = quantize_model_mxfp4(model, exclude_layers=["head"])
    assert out is model
    assert isinstance(model.fc1, MXLinear) and isinstance(model.fc2, MXLinear) and isinstance(model.head, nn.Linear)
    assert model.fc1.is_quantized and model.fc1.bias is not None
    assert "Quantized 2 Linear layers." in capsys.readouterr().out
    assert get_model_size_mb(model) < before
    assert model(torch.randn(5, 64)).shape == (5, 10)


def test_dispatcher_without_cuda_raises():
    from mxfp4.kernel_dispatcher import KernelDispatcher, get_dispatcher
    d = get_dispatcher()
    assert isinstance(d, KernelDispatcher) and d is KernelDispatcher()
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="No backend loaded"):
            d.quant_matmul(torch.zeros(1, 32), torch.zeros(1, 16, dtype=torch.uint8), torch.zeros(1, 1, dtype=torch.uint8))
    from mxfp4.backends import get_backend
    with pytest.raises(ValueError):
        get_backend("triton")


def test_quantize_model_state_dict_equals_reference_fixture_on_cpu():
    """Module surgery of quantize_model_mxfp4 with the oracle as the quantiser: keys, dtypes and bytes of the state_dict
    equal what the reference's own call recorded (tests/golden/model_cases.npz)."""
    from conftest import SmallModel, load_model_cases
    from mxfp4 import quantize_model_mxfp4
    fixture, _ = load_model_cases()
    model = SmallModel()
    model.load_state_dict(fixture["init"])
    quantize_model_mxfp4(model, exclude_layers=["head"], verbose=False)
    sd = model.state_dict()
    assert list(sd.keys()) == fixture["keys"]
    for k in fixture["keys"]:
        assert sd[k].dtype == fixture["q"][k].dtype and torch.equal(sd[k], fixture["q"][k]), k


def test_scale_shape_validation_and_block16_spreading():
    """Host-side checks in front of the GEMM: a scale tensor must be [N, K/16|32|64]; block-16 operands are spread
    so that every 16-element block becomes half of a 32-element tensor-core block."""
    import importlib
    from mxfp4 import _capi, gemm
    gemm = importlib.reload(gemm)          # the real functions, not the oracle stand-ins
    N, K = 8, 128
    for cols, want in ((8, 16), (4, 32), (2, 64)):
        assert gemm.scale_block_size(torch.zeros(N, cols, dtype=torch.uint8), N, K) == want
    for bad in (torch.zeros(N, 3, dtype=torch.uint8), torch.zeros(N - 1, 4, dtype=torch.uint8), torch.zeros(N * 4, dtype=torch.uint8),
                torch.zeros(N, 1, dtype=torch.uint8), torch.zeros(N, 16, dtype=torch.uint8), torch.zeros(N, 0, dtype=torch.uint8)):
        with pytest.raises(_capi.MXFP4BackendError):
            gemm.scale_block_size(bad, N, K)
    x = torch.arange(2 * 32, dtype=torch.float32).view(2, 32).to(torch.bfloat16)
    xs = gemm.spread_block16(x)
    assert xs.shape == (2, 64)
    assert torch.equal(xs[:, :16], x[:, :16]) and torch.equal(xs[:, 32:48], x[:, 16:]) and float(xs[:, 16:32].abs().max()) == 0
