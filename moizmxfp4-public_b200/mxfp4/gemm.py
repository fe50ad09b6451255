"""Host side of quant_matmul / MXLinear.forward: operand preparation caches, workspace, launch.

The arithmetic is entirely in libmxfp4_b200.so (mxfp4_act_quantize + the tcgen05 GEMM kernel).  This
module only keeps, per weight, the scale bytes re-tiled for the tensor cores (a cache rebuilt on
demand, never part of a checkpoint) and, per device and stream, a workspace for the quantised
activations.
"""
import os
import threading
import weakref
from collections import OrderedDict
from typing import Optional

import torch

from . import _capi

_MODES = {"exact": _capi.GEMM_EXACT, "fast": _capi.GEMM_FAST}
_mode = _MODES[os.environ.get("MXFP4_GEMM_MODE", "exact")]
_lock = threading.RLock()
_prepared = OrderedDict()        # id(scale tensor) -> (weakref, version, (N, K, ptr), prepared scale tensor)
_PREPARED_MAX = 4096
_workspaces = {}                 # (device index, stream) -> uint8 tensor
_last_act = {}                   # (device index, stream) -> (activation pointer, M, K, workspace pointer) of the last quantisation


def _align(v, a):
    return (v + a - 1) // a * a


def set_gemm_mode(mode: str):
    """"exact" (default): weights decode exactly as the reference dequantises them, two MMAs per K step.
    "fast": single pass with hardware E2M1 decoding of the weight codes; faster, not parity."""
    global _mode
    _mode = _MODES[mode]


def get_gemm_mode() -> str:
    return "exact" if _mode == _capi.GEMM_EXACT else "fast"


def prepared_scales(weight_scales: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """Tensor-core layout of a weight's E8M0 scales.

    Cached per live tensor OBJECT (a weak reference guards against a recycled address) and per version
    counter (an in-place update such as load_state_dict invalidates the entry).  A module's buffer hits
    the cache on every forward; a temporary tensor simply pays one small re-tiling kernel."""
    key = id(weight_scales)
    with _lock:
        hit = _prepared.get(key)
        if hit is not None:
            ref, version, shape, prepared = hit
            if ref() is weight_scales and version == weight_scales._version and shape == (N, K, weight_scales.data_ptr()):
                _prepared.move_to_end(key)
                return prepared
            del _prepared[key]
    L = _capi.load()
    ws = weight_scales.contiguous()
    out = torch.empty(L.mxfp4_prepared_scales_bytes(N, K), dtype=torch.uint8, device=ws.device)
    with _capi.on_device(ws.device):
        _capi.check(L.mxfp4_prepare_weight_scales(ws.data_ptr(), N, K, out.data_ptr(), _capi.stream_ptr(ws.device)),
                    "mxfp4_prepare_weight_scales")

    def _drop(_ref, key=key):
        with _lock:
            ent = _prepared.get(key)
            if ent is not None and ent[0] is _ref:
                del _prepared[key]

    with _lock:
        _prepared[key] = (weakref.ref(weight_scales, _drop), weight_scales._version, (N, K, weight_scales.data_ptr()), out)
        while len(_prepared) > _PREPARED_MAX:
            _prepared.popitem(last=False)
    return out


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)   # zeroed: the status word starts clear
        _workspaces[key] = ws
        _last_act.pop(key, None)
    return ws


def check_status(device=None):
    """Synchronises and raises if a GEMM kernel on `device` reported a bounded wait that ran out."""
    for (idx, _), ws in list(_workspaces.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        code = int(ws[:4].view(torch.int32).item())
        if code != 0:
            ws[:4].zero_()
            raise _capi.MXFP4BackendError(f"mxfp4 GEMM kernel reported status {code} (a device-side wait timed out)")


def act_quantize(x: torch.Tensor):
    """bf16 [M, K] -> (packed u8 [M, K/2], blocked E8M0 scales u8 [bytes]); the GEMM's own activation format."""
    _capi.require_cuda(x, "act_quantize")
    L = _capi.load()
    assert x.dim() == 2 and x.dtype == torch.bfloat16
    x = x.contiguous()
    M, K = x.shape
    packed = torch.empty(M, K // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(L.mxfp4_act_scales_bytes(M, K), dtype=torch.uint8, device=x.device)
    with _capi.on_device(x.device):
        _capi.check(L.mxfp4_act_quantize(x.data_ptr(), M, K, K, packed.data_ptr(), sf.data_ptr(), _capi.stream_ptr(x.device)),
                    "mxfp4_act_quantize")
    return packed, sf


def quant_matmul_2d(input: torch.Tensor, packed_weight: torch.Tensor, weight_scales: torch.Tensor,
                    bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, reuse_act: bool = False) -> torch.Tensor:
    """[M,K] x packed [N,K/2] (+bias) -> [M,N]; argument contract of the reference's quant_matmul
    (src/mxfp4/fused_kernels.py:160-207: 2-D tensors, K_packed*2 == K)."""
    assert input.dim() == 2, "Input must be 2D [M, K]"
    assert packed_weight.dim() == 2, "Packed weight must be 2D [N, K//2]"
    M, K = input.shape
    N, K_packed = packed_weight.shape
    assert K_packed * 2 == K, f"Weight K dimension mismatch: {K_packed * 2} vs {K}"
    _capi.require_cuda(input, "quant_matmul")
    _capi.require_cuda(packed_weight, "quant_matmul")
    if packed_weight.dtype != torch.uint8:
        raise TypeError("mxfp4: packed_weight must be uint8")
    if weight_scales.dtype != torch.uint8:
        return _matmul_bf16_scales(input, packed_weight, weight_scales, bias)
    if K % 32 != 0:
        raise _capi.MXFP4BackendError(f"mxfp4: K={K} must be a multiple of 32 (pad activations to the packed weight's width)")
    in_dtype = input.dtype
    x = input if in_dtype == torch.bfloat16 else input.to(torch.bfloat16)
    if x.stride(1) != 1 or (x.stride(0) * 2) % 32 != 0 or x.data_ptr() % 32 != 0:
        x = x.contiguous()
    L = _capi.load()
    dev = x.device
    pw = packed_weight.contiguous()
    sfw = prepared_scales(weight_scales, N, K)
    b = None
    if bias is not None:
        b = bias.to(device=dev, dtype=torch.bfloat16).contiguous()
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    if M == 0 or N == 0:
        return out.to(in_dtype)
    nbytes = L.mxfp4_gemm_workspace_bytes(M, N, K, _mode)
    ws = _workspace(dev, nbytes)
    ws_key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    a_off = 4096
    sf_off = a_off + _align(M * (K // 2), 256)
    part_off = sf_off + _align(L.mxfp4_act_scales_bytes(M, K), 256)
    last = _last_act.get(ws_key)
    reuse = reuse_act and last == (x.data_ptr(), M, K, ws.data_ptr())
    with _capi.on_device(dev):
        if reuse:
            # the caller vouches that the previous GEMM on this stream quantised these same activations (q/k/v and
            # gate/up share their input); the workspace still holds their MXFP4 form
            _capi.check(L.mxfp4_gemm_prequantized(ws.data_ptr() + a_off, ws.data_ptr() + sf_off, pw.data_ptr(), sfw.data_ptr(),
                                                  None if b is None else b.data_ptr(), out.data_ptr(), out.stride(0), M, N, K, _mode,
                                                  ws.data_ptr() + part_off, ws.numel() - part_off, ws.data_ptr(), _capi.stream_ptr(dev)),
                        "mxfp4_gemm_prequantized")
        else:
            _capi.check(L.mxfp4_gemm(x.data_ptr(), x.stride(0), pw.data_ptr(), sfw.data_ptr(), None if b is None else b.data_ptr(),
                                     out.data_ptr(), out.stride(0), M, N, K, _mode, ws.data_ptr(), ws.numel(), _capi.stream_ptr(dev)),
                        "mxfp4_gemm")
            _last_act[ws_key] = (x.data_ptr(), M, K, ws.data_ptr())
    return out if in_dtype == torch.bfloat16 else out.to(in_dtype)


class _HostPipe:
    """Per-device staging for quant_matmul_host: three streams (host->device, GEMM, device->host) and a ring of
    device chunk buffers, each with the events that say when it may be overwritten."""

    def __init__(self, dev, depth=3):
        self.dev, self.depth = dev, depth
        self.s_in, self.s_mm, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.slots = []            # dicts: x, y, ev_in, ev_mm, ev_out, used
        self.shape = None

    def ring(self, rows, K, N):
        if self.shape != (rows, K, N):
            for s in (self.s_in, self.s_mm, self.s_out):
                s.synchronize()
            self.slots = [dict(x=torch.empty(rows, K, dtype=torch.bfloat16, device=self.dev),
                               y=torch.empty(rows, N, dtype=torch.bfloat16, device=self.dev),
                               ev_in=torch.cuda.Event(), ev_mm=torch.cuda.Event(), ev_out=torch.cuda.Event(), used=False)
                          for _ in range(self.depth)]
            self.shape = (rows, K, N)
        return self.slots


_host_pipes = {}                 # device index -> _HostPipe


def quant_matmul_host(input: torch.Tensor, packed_weight: torch.Tensor, weight_scales: torch.Tensor,
                      bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                      chunk_rows: int = 1024) -> torch.Tensor:
    """quant_matmul for activations that live in HOST memory: [M,K] (pinned for full overlap) x device-resident packed
    weight -> [M,N] bf16 in host memory (`out`, pinned; allocated when None).

    The rows are cut into chunks; the host->device copy of chunk i+1, the GEMM of chunk i and the device->host copy of
    chunk i-1 run on three streams, so the PCIe link is busy in both directions while the tensor cores work.  Rows are
    independent and no chunk is small enough to be K-split unless M itself is, so the result equals quant_matmul's on
    the same rows bit for bit.  The call returns after enqueueing; the current stream waits for the last device->host
    copy, so synchronise it (or the device) before reading `out` on the host."""
    assert input.dim() == 2 and packed_weight.dim() == 2
    if input.is_cuda:
        raise ValueError("quant_matmul_host takes host activations; use quant_matmul for device tensors")
    _capi.require_cuda(packed_weight, "quant_matmul_host")
    dev = packed_weight.device
    M, K = input.shape
    N = packed_weight.shape[0]
    in_dtype = input.dtype
    x = input if in_dtype == torch.bfloat16 else input.to(torch.bfloat16)
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
    if out.dtype != torch.bfloat16 or out.shape != (M, N) or out.is_cuda:
        raise ValueError("quant_matmul_host: out must be a host bf16 tensor of shape [M, N]")
    if M == 0 or N == 0:
        return out if in_dtype == torch.bfloat16 else out.to(in_dtype)
    n_chunks = -(-M // max(int(chunk_rows), 129))
    rows = _align(-(-M // n_chunks), 128)
    with _lock:
        pipe = _host_pipes.get(dev.index)
        if pipe is None:
            pipe = _host_pipes[dev.index] = _HostPipe(dev)
        slots = pipe.ring(rows, K, N)
        cur = torch.cuda.current_stream(dev)
        pipe.s_mm.wait_stream(cur)                       # the weight (and bias) may have been produced on the caller's stream
        for c, r0 in enumerate(range(0, M, rows)):
            n = min(rows, M - r0)
            sl = slots[c % pipe.depth]
            if sl["used"]:
                pipe.s_in.wait_event(sl["ev_mm"])        # the GEMM that read this x buffer has finished
            with torch.cuda.stream(pipe.s_in):
                sl["x"][:n].copy_(x[r0:r0 + n], non_blocking=True)
                sl["ev_in"].record(pipe.s_in)
            pipe.s_mm.wait_event(sl["ev_in"])
            if sl["used"]:
                pipe.s_mm.wait_event(sl["ev_out"])       # the copy that read this y buffer has finished
            with torch.cuda.stream(pipe.s_mm):
                quant_matmul_2d(sl["x"][:n], packed_weight, weight_scales, bias, out=sl["y"][:n])
                sl["ev_mm"].record(pipe.s_mm)
            pipe.s_out.wait_event(sl["ev_mm"])
            with torch.cuda.stream(pipe.s_out):
                out[r0:r0 + n].copy_(sl["y"][:n], non_blocking=True)
                sl["ev_out"].record(pipe.s_out)
            sl["used"] = True
        cur.wait_stream(pipe.s_out)
    return out if in_dtype == torch.bfloat16 else out.to(in_dtype)


def _matmul_bf16_scales(input, packed_weight, weight_scales, bias):
    """scale_format="bf16" weights have no power-of-two scales, so they cannot feed the block-scaled
    tensor-core path; they take the reference's own formulation (dequantise, cast, dense matmul,
    src/mxfp4/backends.py:295-312) with this package's dequantiser."""
    w = _capi.dequantize(packed_weight, weight_scales, 32, torch.float32).to(input.dtype)
    out = torch.matmul(input, w.T)
    if bias is not None:
        out += bias
    return out


def mxlinear_forward(input: torch.Tensor, packed_weight: torch.Tensor, weight_scales: torch.Tensor,
                     bias: Optional[torch.Tensor], in_features: int, reuse_act: bool = False) -> torch.Tensor:
    """MXLinear.forward for a quantised layer: any leading dimensions, output in the input's dtype."""
    lead = input.shape[:-1]
    x = input.reshape(-1, input.shape[-1])
    k_pad = packed_weight.shape[-1] * 2
    if x.shape[-1] != k_pad:
        # the quantiser padded the weight rows to a multiple of the block; padded weight columns meet zeros
        x = torch.nn.functional.pad(x, (0, k_pad - x.shape[-1]))
    y = quant_matmul_2d(x, packed_weight, weight_scales, bias, reuse_act=reuse_act)
    return y.reshape(*lead, packed_weight.shape[0])
