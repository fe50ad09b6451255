"""Shared test plumbing: import paths, the `gpu` marker, fixture loaders."""
import json
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "moizmxfp4-public_b200")
for p in (ROOT, PKG_DIR):
    if p not in sys.path:
        sys.path.insert(0, p)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


_NP2T = {"bfloat16": (np.uint16, torch.bfloat16), "float16": (np.uint16, torch.float16),
         "float32": (np.uint32, torch.float32), "uint8": (np.uint8, torch.uint8)}


def from_bits(a: np.ndarray, dtype: str) -> torch.Tensor:
    """Rebuild a torch tensor from the raw bit pattern stored in a fixture."""
    npdt, tdt = _NP2T[dtype]
    a = np.ascontiguousarray(a.astype(npdt, copy=False))
    if dtype == "uint8":
        return torch.from_numpy(a.copy())
    signed = {np.uint16: np.int16, np.uint32: np.int32}[npdt]
    return torch.from_numpy(a.view(signed).copy()).view(tdt)


def to_bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float32:
        return t.view(torch.int32).numpy().view(np.uint32)
    return t.numpy()


def load_quant_cases():
    z = np.load(os.path.join(GOLDEN, "quant_cases.npz"))
    cases = []
    for i, m in enumerate(z["meta"]):
        m = json.loads(str(m))
        sdt = "uint8" if m["fmt"] == "e8m0" else "bfloat16"
        cases.append(dict(m, x=from_bits(z[f"c{i}_x"], m["dtype"]), packed=from_bits(z[f"c{i}_packed"], "uint8"),
                          scales=from_bits(z[f"c{i}_scales"], sdt), rec=from_bits(z[f"c{i}_rec"], "float32")))
    return cases


def load_matmul_cases():
    z = np.load(os.path.join(GOLDEN, "matmul_cases.npz"))
    cases = []
    for i, m in enumerate(z["meta"]):
        m = json.loads(str(m))
        c = dict(m, x=from_bits(z[f"m{i}_x"], "bfloat16"), w=from_bits(z[f"m{i}_w"], "bfloat16"),
                 packed=from_bits(z[f"m{i}_packed"], "uint8"), scales=from_bits(z[f"m{i}_scales"], "uint8"),
                 y=from_bits(z[f"m{i}_y"], "bfloat16"),
                 bias=from_bits(z[f"m{i}_bias"], "bfloat16") if m["bias"] else None)
        cases.append(c)
    return cases


def weight(N, K, seed, outliers):
    """Benchmark weight generator (same as tests/golden/make_golden.py)."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.02
    if outliers:
        idx = torch.randperm(N * K, generator=g)[: int(0.001 * N * K)]
        w.view(-1)[idx] *= 50
    return w.to(torch.bfloat16)


def act(M, K, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, K, generator=g).to(torch.bfloat16)


class SmallModel(torch.nn.Module):
    """Same architecture as the model tests/golden/make_golden.py quantises with the reference."""

    def __init__(self):
        super().__init__()
        self.body = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 96, bias=False))
        self.head = torch.nn.Linear(96, 10)

    def forward(self, x):
        return self.head(self.body(x))


_DT_OF_KEY = {"packed_weight": "uint8", "weight_scales": "uint8"}


def load_model_cases():
    """model_cases.npz: the reference's quantize_model_mxfp4 / MXLinear.forward on CPU tensors."""
    z = np.load(os.path.join(GOLDEN, "model_cases.npz"))
    init = {k[len("model_init_"):]: from_bits(z[k], "float32") for k in z.files if k.startswith("model_init_")}
    keys = [str(k) for k in z["model_q_keys"]]
    q = {k: from_bits(z[f"model_q_{k}"], _DT_OF_KEY.get(k.rsplit(".", 1)[-1], "float32")) for k in keys}
    model = dict(init=init, keys=keys, q=q, x2=from_bits(z["model_x2"], "float32"), y2=from_bits(z["model_y2"], "float32"),
                 x3=from_bits(z["model_x3"], "float32"), y3=from_bits(z["model_y3"], "float32"))
    layers = []
    for i, m in enumerate(z["layer_meta"]):
        m = json.loads(str(m))
        layers.append(dict(m, w=from_bits(z[f"l{i}_w"], "float32"), b=from_bits(z[f"l{i}_b"], "float32") if m["bias"] else None,
                           packed=from_bits(z[f"l{i}_packed"], "uint8"), scales=from_bits(z[f"l{i}_scales"], "uint8"),
                           x=from_bits(z[f"l{i}_x"], m["dtype"]), y=from_bits(z[f"l{i}_y"], m["dtype"])))
    return model, layers
