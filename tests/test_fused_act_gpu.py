"""mxfp4_act_fused -- the single kernel between two GEMMs of a block (gather of the previous result, residual + RMS norm /
silu*mul / q+k+v, activation quantiser) -- against the same steps as separate PyTorch operations followed by the oracle's
activation quantiser, and the fused MXLinear block stack against the unfused one.

Bit-exact where the arithmetic is the same operations in the same order (adds, roundings, the quantiser itself); where a
float32 reduction order or a transcendental differs from PyTorch's (the mean of squares, exp) values may differ in the last
bf16 bit before the quantiser, so those comparisons allow a small fraction of differing codes."""
import ctypes

import pytest
import torch

from conftest import act
from oracle import oracle
from test_gemm_gpu import unblock

pytestmark = pytest.mark.gpu


def run_fused(op, M, K, *, in_bf16=None, in_f32=None, residual=None, bias=None, hidden=False, quantize=True, eps=1e-6, peer=None):
    from mxfp4 import _capi
    L = _capi.load()
    dev = torch.device("cuda", 0)
    a = _capi.ActFusedArgs()
    a.op, a.M, a.K, a.eps = op, M, K, eps
    if in_bf16 is not None:
        a.in_bf16, a.ld_in = in_bf16.data_ptr(), in_bf16.stride(0)
    if in_f32 is not None:
        a.in_f32, a.splits, a.split_stride, a.ld_in = in_f32.data_ptr(), in_f32.shape[0], in_f32.stride(0), in_f32.stride(1)
    if peer is not None:
        arr, world, rank, epoch, status, ld, done = peer
        a.peer_blocks, a.world, a.rank, a.epoch, a.status_dev, a.ld_in, a.peer_wait_done = arr, world, rank, epoch.data_ptr(), status.data_ptr(), ld, done
    if residual is not None:
        a.residual, a.ld_res = residual.data_ptr(), residual.stride(0)
    hid = torch.full((M, K), 7.0, dtype=torch.bfloat16, device=dev) if hidden else None
    if hid is not None:
        a.hidden_out, a.ld_hid = hid.data_ptr(), K
    if bias is not None:
        a.bias = bias.data_ptr()
    packed = sf = None
    if quantize:
        packed = torch.empty(M, K // 2, dtype=torch.uint8, device=dev)
        sf = torch.full((L.mxfp4_act_scales_bytes(M, K),), 255, dtype=torch.uint8, device=dev)
        a.packed, a.sf = packed.data_ptr(), sf.data_ptr()
    _capi.check(L.mxfp4_act_fused(ctypes.byref(a), None), "mxfp4_act_fused")
    torch.cuda.synchronize()
    return packed, sf, hid


def codes_close(packed, sf, x_ref, M, K, exact):
    """Compares with the oracle's quantisation of the bf16 reference activations."""
    op, os_ = oracle.act_quantize(x_ref.cpu())
    got_s = unblock(sf, M, K)
    if exact:
        assert torch.equal(packed.cpu(), op) and torch.equal(got_s, os_)
        return
    same = (packed.cpu() == op).float().mean().item()
    assert same > 0.995, f"only {same:.4f} of the code bytes agree"
    ref = oracle.act_dequantize(op, os_)
    got = oracle.act_dequantize(packed.cpu(), got_s)
    assert ((got - ref).norm() / ref.norm()).item() < 1e-2


@pytest.mark.parametrize("M,K", [(1, 32), (5, 4096), (128, 4096), (130, 1376), (3, 11008), (2, 16384), (2, 32768)])
def test_sum3_and_silu_mul(M, K):
    from mxfp4 import _capi
    x = act(M, 3 * K, 21 + M).cuda()
    packed, sf, _ = run_fused(_capi.ACT_SUM3, M, K, in_bf16=x)
    ref = (x[:, :K] + x[:, K:2 * K]) + x[:, 2 * K:]
    codes_close(packed, sf, ref, M, K, exact=True)
    mask = torch.ones(sf.numel(), dtype=torch.bool)
    assert int(sf.max()) < 255                                       # every scale byte, padding included, was written
    packed, sf, _ = run_fused(_capi.ACT_SILU_MUL, M, K, in_bf16=x[:, :2 * K])
    ref = torch.nn.functional.silu(x[:, :K]) * x[:, K:2 * K]
    codes_close(packed, sf, ref, M, K, exact=False)


@pytest.mark.parametrize("M,K,splits", [(7, 512, 0), (128, 4096, 0), (128, 4096, 4), (33, 1024, 3), (2, 11008, 2)])
def test_rmsnorm_with_residual_bias_and_split_k_partials(M, K, splits):
    from mxfp4 import _capi
    g = torch.Generator().manual_seed(M + K)
    res = act(M, K, 5).cuda()
    bias = (torch.randn(K, generator=g) * 0.1).to(torch.bfloat16).cuda()
    if splits:
        part = torch.randn(splits, M, K, generator=g).cuda()
        value = part[0].clone()
        for s in range(1, splits):
            value = value + part[s]                                  # fixed order, float32
        value = value.to(torch.bfloat16)
        packed, sf, hid = run_fused(_capi.ACT_RMSNORM, M, K, in_f32=part, residual=res, bias=bias, hidden=True)
    else:
        value = act(M, K, 6).cuda()
        packed, sf, hid = run_fused(_capi.ACT_RMSNORM, M, K, in_bf16=value, residual=res, bias=bias, hidden=True)
    h_ref = res + (value + bias)                                     # bf16 roundings after each add, as PyTorch makes them
    assert torch.equal(hid, h_ref)
    x_ref = torch.nn.functional.rms_norm(h_ref, (K,), eps=1e-6)
    codes_close(packed, sf, x_ref, M, K, exact=False)
    # hidden only (the last step of a stack), and no input at all (the first): hidden = residual
    _, _, hid2 = run_fused(_capi.ACT_RMSNORM, M, K, in_bf16=value.contiguous(), residual=res, hidden=True, quantize=False)
    assert torch.equal(hid2, res + value)
    packed, sf, hid3 = run_fused(_capi.ACT_RMSNORM, M, K, residual=res, hidden=True)
    assert torch.equal(hid3, res)
    codes_close(packed, sf, torch.nn.functional.rms_norm(res, (K,), eps=1e-6), M, K, exact=False)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_rmsnorm_over_peer_blocks_is_the_all_reduce(monkeypatch, world):
    """All 'ranks' emulated by buffers of one GPU (rank 0 runs, the others are data whose flags are set by hand, as their
    launches would set them): value = bf16(float32 sum of the partials in rank order).  Then a call whose peers never
    arrive: bounded wait, status MXFP4_E_TIMEOUT, NaN in hidden_out, context still usable."""
    from mxfp4 import _capi
    L = _capi.load()
    dev = torch.device("cuda", 0)
    M, K = 96, 512
    off = L.mxfp4_peer_partial_offset()
    blocks = [torch.zeros(L.mxfp4_peer_block_bytes(M, K), dtype=torch.uint8, device=dev) for _ in range(world)]
    parts = [act(M, K, 70 + r).to(dev) for r in range(world)]
    for b, p_ in zip(blocks, parts):
        b[off:off + M * K * 2].view(torch.bfloat16).view(M, K).copy_(p_)
    arr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in blocks])
    epoch = torch.zeros(2, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    res = act(M, K, 9).to(dev)
    flags0 = blocks[0][:off].view(torch.int32)
    for r in range(1, world):
        flags0[r] = 1
    monkeypatch.setenv("MXFP4_PEER_WAIT_MS", "200")
    peer = (ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p)), world, 0, epoch, status, K, 0)
    packed, sf, hid = run_fused(_capi.ACT_RMSNORM, M, K, residual=res, hidden=True, peer=peer)
    acc = torch.zeros(M, K, dtype=torch.float32, device=dev)
    for p_ in parts:
        acc = acc + p_.float()
    h_ref = res + acc.to(torch.bfloat16)
    assert int(status.item()) == 0 and int(epoch[0].item()) == 1 and int(epoch[1].item()) == 0
    assert torch.equal(hid, h_ref)
    codes_close(packed, sf, torch.nn.functional.rms_norm(h_ref, (K,), eps=1e-6), M, K, exact=False)
    for r in range(1, world):                                    # rank 0 published ready = 1 and done = 1 in every peer's block
        fl = blocks[r][:off].view(torch.int32)
        assert int(fl[0].item()) == 1 and int(fl[8].item()) == 1
    if world != 2:
        return
    packed, sf, hid = run_fused(_capi.ACT_RMSNORM, M, K, residual=res, hidden=True, peer=peer)      # call 2: nobody arrives
    assert int(status.item()) == -6
    assert bool(torch.isnan(hid.float()).all()) and int(packed.max()) == 0
    assert torch.equal(torch.ones(4, device=dev) * 2, torch.full((4,), 2.0, device=dev))


def test_two_shot_peer_sum_with_emulated_ranks(monkeypatch):
    """Two-shot mode on one GPU: rank 0 reduces, normalises and quantises the rows it owns and leaves them in its result
    block; the rows the other 'ranks' own are copied from their result blocks (filled by hand here, their flags set as
    their launches would set them)."""
    from mxfp4 import _capi
    L = _capi.load()
    dev = torch.device("cuda", 0)
    world, M, K = 4, 90, 512
    rows_per = -(-M // world)                                   # 23: ranks own 23, 23, 23, 21 rows
    off = L.mxfp4_peer_partial_offset()
    rb = L.mxfp4_act_fused_result_row_bytes(K)
    assert rb == K * 2 + K // 2 + 16
    blocks = [torch.zeros(L.mxfp4_peer_block_bytes(M, K), dtype=torch.uint8, device=dev) for _ in range(world)]
    results = [torch.zeros(rows_per * rb, dtype=torch.uint8, device=dev) for _ in range(world)]
    parts = [act(M, K, 50 + r).to(dev) for r in range(world)]
    for b, p_ in zip(blocks, parts):
        b[off:off + M * K * 2].view(torch.bfloat16).view(M, K).copy_(p_)
    # what the other ranks "computed" for their rows: recognisable hidden values, codes and scales
    fake_h = act(M, K, 99).to(dev)
    fake_codes = torch.randint(0, 256, (M, K // 2), generator=torch.Generator().manual_seed(5), dtype=torch.uint8).to(dev)
    fake_sc = torch.randint(100, 140, (M, K // 32), generator=torch.Generator().manual_seed(6), dtype=torch.uint8).to(dev)
    for r in range(1, world):
        for m in range(r * rows_per, min(M, (r + 1) * rows_per)):
            row = results[r][(m - r * rows_per) * rb:(m - r * rows_per + 1) * rb]
            row[:K * 2].copy_(fake_h[m].view(torch.uint8))
            row[K * 2:K * 2 + K // 2].copy_(fake_codes[m])
            row[K * 2 + K // 2:K * 2 + K // 2 + K // 32].copy_(fake_sc[m])
    flags0 = blocks[0][:off].view(torch.int32)
    for r in range(1, world):
        flags0[r] = 1          # ready
        flags0[8 + r] = 1      # the rank's rows are in its result block
    arr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in blocks])
    rarr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in results])
    epoch = torch.zeros(2, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    count = torch.zeros(1, dtype=torch.int32, device=dev)
    res = act(M, K, 9).to(dev)
    a = _capi.ActFusedArgs()
    a.op, a.M, a.K, a.eps = _capi.ACT_RMSNORM, M, K, 1e-6
    a.peer_blocks, a.world, a.rank = ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p)), world, 0
    a.epoch, a.status_dev, a.ld_in = epoch.data_ptr(), status.data_ptr(), K
    a.peer_results, a.owner_count = ctypes.cast(rarr, ctypes.POINTER(ctypes.c_void_p)), count.data_ptr()
    a.residual, a.ld_res = res.data_ptr(), K
    hid = torch.zeros(M, K, dtype=torch.bfloat16, device=dev)
    packed = torch.zeros(M, K // 2, dtype=torch.uint8, device=dev)
    sf = torch.full((L.mxfp4_act_scales_bytes(M, K),), 255, dtype=torch.uint8, device=dev)
    a.hidden_out, a.ld_hid, a.packed, a.sf = hid.data_ptr(), K, packed.data_ptr(), sf.data_ptr()
    monkeypatch.setenv("MXFP4_PEER_WAIT_MS", "500")
    _capi.check(L.mxfp4_act_fused(ctypes.byref(a), None), "mxfp4_act_fused")
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(epoch[0].item()) == 1 and int(count.item()) == 0
    own = slice(0, rows_per)
    acc = torch.zeros(M, K, dtype=torch.float32, device=dev)
    for p_ in parts:
        acc = acc + p_.float()
    h_ref = res + acc.to(torch.bfloat16)
    assert torch.equal(hid[own], h_ref[own])                                        # first shot: this rank's rows
    assert torch.equal(hid[rows_per:], fake_h[rows_per:])                           # second shot: fetched rows
    assert torch.equal(packed[rows_per:], fake_codes[rows_per:])
    sc = unblock(sf, M, K)
    assert torch.equal(sc[rows_per:], fake_sc[rows_per:].cpu())
    op, os_ = oracle.act_quantize(torch.nn.functional.rms_norm(h_ref[own], (K,), eps=1e-6).cpu())
    assert (packed[own].cpu() == op).float().mean().item() > 0.995 and (sc[own] == os_).float().mean().item() > 0.995
    # this rank's result block holds exactly what it wrote locally, and the peers were told
    mine = results[0].view(rows_per, rb)
    assert torch.equal(mine[:, :K * 2].contiguous().view(torch.bfloat16).view(rows_per, K), hid[own])
    assert torch.equal(mine[:, K * 2:K * 2 + K // 2], packed[own])
    assert torch.equal(mine[:, K * 2 + K // 2:K * 2 + K // 2 + K // 32].cpu(), sc[own])
    for r in range(1, world):
        fl = blocks[r][:off].view(torch.int32)
        assert int(fl[0].item()) == 1 and int(fl[8].item()) == 1


def test_argument_checks():
    from mxfp4 import _capi
    L = _capi.load()
    x = torch.zeros(4, 96, dtype=torch.bfloat16, device="cuda")
    a = _capi.ActFusedArgs()
    a.op, a.M, a.K = _capi.ACT_SUM3, 4, 32
    assert L.mxfp4_act_fused(ctypes.byref(a), None) == -1                       # no input
    a.in_bf16, a.ld_in = x.data_ptr(), 64
    assert L.mxfp4_act_fused(ctypes.byref(a), None) == -2                       # ld_in < 3 K
    a.ld_in, a.K = 96, 40
    assert L.mxfp4_act_fused(ctypes.byref(a), None) == -2                       # K not a multiple of 32
    a.K, a.op = 32, 9
    assert L.mxfp4_act_fused(ctypes.byref(a), None) == -1
    a.op, a.K = _capi.ACT_RMSNORM, 65536
    assert L.mxfp4_act_fused(ctypes.byref(a), None) == -4                       # a row no longer fits in registers


@pytest.mark.parametrize("M", [16, 128, 300])
def test_fused_block_stack_matches_unfused(M):
    """Eight launches per layer against the same arithmetic as separate operations and layer calls."""
    from mxfp4 import gemm
    from mxfp4.parallel import MXBlockStack
    x = act(M, 512, 11).cuda()
    stack = MXBlockStack.build(n_layers=3, hidden=512, inter=1536, device="cuda", seed=5)
    with torch.no_grad():
        a = stack(x, fused=True)
        b = stack(x, fused=False)
        a2 = stack(x, fused=True)
    gemm.check_status()
    stack._chain.check_status()
    assert torch.equal(a, a2)
    err = ((a.float() - b.float()).norm() / b.float().norm()).item()
    print(f"M={M}: fused vs unfused stack rel_fro {err:.3e}")
    assert torch.isfinite(a.float()).all() and err < 1e-2
