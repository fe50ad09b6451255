"""The allocation-free GEMM entry point (mxfp4_gemm_noalloc) against the regular one (mxfp4_gemm).

Some hosts of the library cannot call cudaMalloc when they need a matmul (their own pool owns the GPU, or they
sit on a latency-critical path), so that entry point keeps its scratch in a fixed array inside the library.
Both entry points run the same kernels on the same operands, so their outputs must be identical; two calls in
a row check that what the first call left in the shared scratch does not leak into the second.
This file sorts last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes

import pytest
import torch

from conftest import act, weight

pytestmark = pytest.mark.gpu


def _run_both(L, gemm, x, packed, scales, bias):
    from mxfp4 import _capi
    M, K = x.shape
    N = packed.shape[0]
    prep = gemm.prepared_scales(scales, N, K)
    dev = x.device
    sp = torch.cuda.current_stream(dev).cuda_stream
    ws = torch.zeros(L.mxfp4_gemm_workspace_bytes(M, N, K, 0), dtype=torch.uint8, device=dev)
    ref = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    bptr = None if bias is None else bias.data_ptr()
    _capi.check(L.mxfp4_gemm(x.data_ptr(), K, packed.data_ptr(), prep.data_ptr(), bptr, ref.data_ptr(), N, M, N, K, 0,
                             ws.data_ptr(), ws.numel(), sp), "mxfp4_gemm")
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    _capi.check(L.mxfp4_gemm_noalloc(x.data_ptr(), K, packed.data_ptr(), prep.data_ptr(), bptr, out.data_ptr(), N, M, N, K, 0,
                                     status.data_ptr(), sp), "mxfp4_gemm_noalloc")
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(ws[:4].view(torch.int32).item()) == 0
    return out, ref


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    from mxfp4 import _capi, gemm
    from mxfp4.quantizer import MXFP4Quantizer
    L = _capi.load()
    q = MXFP4Quantizer(32, "e8m0")
    # first call: a split-K decode shape; second call: a smaller, different problem that reuses the scratch
    for (M, N, K, seed, with_bias) in [(48, 4096, 4096, 1, True), (128, 1376, 1024, 2, False)]:
        packed, scales = q.quantize(weight(N, K, seed, True).cuda())
        x = act(M, K, 10 + seed).cuda()
        bias = (torch.randn(N, generator=torch.Generator().manual_seed(seed)) * 0.1).to(torch.bfloat16).cuda() if with_bias else None
        out, ref = _run_both(L, gemm, x, packed, scales, bias)
        assert not torch.isnan(out.float()).any()
        assert torch.equal(out, ref), f"max diff {(out.float() - ref.float()).abs().max().item()}"


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from mxfp4 import _capi
    L = _capi.load()
    one = torch.zeros(64, dtype=torch.uint8, device="cuda")
    rc = L.mxfp4_gemm_noalloc(one.data_ptr(), 8192, one.data_ptr(), one.data_ptr(), None, one.data_ptr(), 4096, 8192, 4096, 8192, 0, None, None)
    assert rc == -7                                    # MXFP4_E_WORKSPACE, before anything is launched
    assert "16777216" in _capi.last_error()
