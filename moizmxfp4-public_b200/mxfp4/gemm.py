"""Host side of quant_matmul / MXLinear.forward: operand preparation caches, workspace, launch.

The arithmetic is entirely in libmxfp4_b200.so (mxfp4_act_quantize + the tcgen05 GEMM kernel).  This
module only keeps, per weight, the scale bytes re-tiled for the tensor cores (a cache rebuilt on
demand, never part of a checkpoint) and, per device and stream, a workspace for the quantised
activations.
"""
import ctypes
import os
import threading
import weakref
from collections import OrderedDict
from typing import Optional

import torch

from . import _capi

_MODES = {"exact": _capi.GEMM_EXACT, "fast": _capi.GEMM_FAST, "w4a16": -1}
_mode = _MODES[os.environ.get("MXFP4_GEMM_MODE", "exact")]
_lock = threading.RLock()
_PREPARED_MAX = 4096
_derived = OrderedDict()         # (id(tensor), tag) -> (weakref, version, ptr, derived tensor, event, ids of streams ordered behind it)
_workspaces = {}                 # (device index, stream) -> uint8 tensor
_last_act = {}                   # (device index, stream) -> (activation pointer, M, K, workspace pointer) of the last quantisation


def _align(v, a):
    return (v + a - 1) // a * a


def set_gemm_mode(mode: str):
    """"exact" (default): FP4 tensor cores, weights decode exactly as the reference dequantises them (two MMAs per K
    step), activations quantised to MXFP4.
    "fast": single pass with hardware E2M1 decoding of the weight codes; faster, not parity.
    "w4a16": the reference's literal arithmetic (bf16 activations left as they are, weights decoded to bf16 inside the
    kernel, bf16 tensor cores): within bf16 rounding of FallbackBackend.matmul, at a quarter of the FP4 rate."""
    global _mode
    _mode = _MODES[mode]


def get_gemm_mode() -> str:
    return {_capi.GEMM_EXACT: "exact", _capi.GEMM_FAST: "fast"}.get(_mode, "w4a16")


def _cached(src: torch.Tensor, tag, build):
    """Per live tensor OBJECT (a weak reference guards against a recycled address) and version counter (an in-place
    update such as load_state_dict invalidates the entry): the tensor `build()` derives from `src`, made once, on the
    stream that was current at first use.  The first reader on any other stream waits for that work through an event
    (and tells the caching allocator about the new user); after that the stream's own order covers it.  A stream under
    CUDA graph capture cannot wait for an event recorded outside the capture, so run a layer once on the capturing
    stream before capturing it (any warm-up call does)."""
    key = (id(src), tag)
    dev = src.device
    with _lock:
        hit = _derived.get(key)
        if hit is not None:
            ref, version, ptr, out, ev, synced = hit
            if ref() is src and version == src._version and ptr == src.data_ptr():
                _derived.move_to_end(key)
                cur = torch.cuda.current_stream(dev)
                if cur.cuda_stream not in synced:
                    if torch.cuda.is_current_stream_capturing():
                        raise _capi.MXFP4BackendError(
                            "mxfp4: a prepared weight tensor is first used on this stream inside a CUDA graph capture; "
                            "call the layer once on the capturing stream before the capture")
                    cur.wait_event(ev)
                    out.record_stream(cur)
                    synced.add(cur.cuda_stream)
                return out
            del _derived[key]
    out = build()
    ev = torch.cuda.Event()
    cur = torch.cuda.current_stream(dev)
    ev.record(cur)

    def _drop(_ref, key=key):
        with _lock:
            ent = _derived.get(key)
            if ent is not None and ent[0] is _ref:
                del _derived[key]

    with _lock:
        _derived[key] = (weakref.ref(src, _drop), src._version, src.data_ptr(), out, ev, {cur.cuda_stream})
        while len(_derived) > _PREPARED_MAX:
            _derived.popitem(last=False)
    return out


def bias_bf16(bias: Optional[torch.Tensor], device) -> Optional[torch.Tensor]:
    """The bias as a contiguous bf16 tensor on `device`: the tensor itself when it already is one, else a copy made
    once per parameter version (MXLinear's default bias is float32; casting it on every call cost a launch)."""
    if bias is None:
        return None
    if bias.dtype == torch.bfloat16 and bias.device == device and bias.is_contiguous():
        return bias
    if bias.device != device:
        return bias.detach().to(device=device, dtype=torch.bfloat16).contiguous()
    return _cached(bias, "bias_bf16", lambda: bias.detach().to(torch.bfloat16).contiguous())


def scale_block_size(weight_scales: torch.Tensor, N: int, K: int) -> int:
    """Block size a scale tensor implies for a packed weight [N, K/2]; raises on anything but [N, K/16|32|64].

    A mis-shaped scale tensor would otherwise be read past its end (or mis-indexed) by the re-tiling kernel."""
    if weight_scales.dim() != 2 or weight_scales.shape[0] != N or weight_scales.shape[1] == 0 or K % weight_scales.shape[1]:
        raise _capi.MXFP4BackendError(
            f"mxfp4: weight_scales of shape {tuple(weight_scales.shape)} do not match a packed weight [{N}, {K // 2}] "
            f"(expected [{N}, {K}/block] with block 16, 32 or 64)")
    block = K // weight_scales.shape[1]
    if block not in (16, 32, 64):
        raise _capi.MXFP4BackendError(
            f"mxfp4: weight_scales of shape {tuple(weight_scales.shape)} imply block size {block}; the tensor-core path "
            "takes 16, 32 or 64 (MXFP4_E_UNSUPPORTED)")
    return block


def prepared_scales(weight_scales: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """Tensor-core layout of a weight's E8M0 scales [N, K/32] (or [N, K/64]: the tensor cores scale per 32 elements, so
    every byte of a 64-element block is simply used for both of its halves).

    Cached per live tensor object and version; a module's buffer hits the cache on every forward, a temporary tensor
    simply pays one small re-tiling kernel."""
    block = scale_block_size(weight_scales, N, K)
    if block == 16:
        raise _capi.MXFP4BackendError("mxfp4: block-16 scales are expanded by expand_block16() before they are prepared")

    def build():
        L = _capi.load()
        ws = weight_scales.contiguous()
        if block == 64:
            ws = ws.repeat_interleave(2, dim=1).contiguous()
        out = torch.empty(L.mxfp4_prepared_scales_bytes(N, K), dtype=torch.uint8, device=ws.device)
        with _capi.on_device(ws.device):
            _capi.check(L.mxfp4_prepare_weight_scales(ws.data_ptr(), N, K, out.data_ptr(), _capi.stream_ptr(ws.device)),
                        "mxfp4_prepare_weight_scales")
        return out
    return _cached(weight_scales, ("prepared", N, K), build)


def expand_block16(packed_weight: torch.Tensor) -> torch.Tensor:
    """Block-16 weights on 32-element tensor-core blocks: every 16-element block (8 bytes) becomes the first half of a
    32-element block whose second half is padding, so that the [N, K/16] scales apply unchanged as [N, 2K/32].  The
    activations are spread the same way with zeros in the padding (spread_block16), which removes the padded weight
    codes from every dot product.  Costs twice the K extent; block 16 is a side path.  Cached per weight."""
    def build():
        N, kb = packed_weight.shape
        return torch.nn.functional.pad(packed_weight.reshape(N, kb // 8, 8), (0, 8)).reshape(N, kb * 2).contiguous()
    return _cached(packed_weight, "block16", build)


def spread_block16(x: torch.Tensor) -> torch.Tensor:
    M, K = x.shape
    return torch.nn.functional.pad(x.reshape(M, K // 16, 16), (0, 16)).reshape(M, 2 * K)


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
    for idx, st in list(_w4a16_status.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        code = int(st.item())
        if code != 0:
            st.zero_()
            raise _capi.MXFP4BackendError(f"mxfp4 W4A16 GEMM kernel reported status {code} (a device-side wait timed out)")


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
    block = scale_block_size(weight_scales, N, K)
    if weight_scales.dtype != torch.uint8 or _mode == -1:
        return matmul_w4a16(input, packed_weight, weight_scales, bias, block, out=out)
    in_dtype = input.dtype
    x = input if in_dtype == torch.bfloat16 else input.to(torch.bfloat16)
    if block == 16:
        # twice the K extent: [block of 16 | 16 zeros] against [8 code bytes | 8 padding bytes], scales unchanged
        y = quant_matmul_2d(spread_block16(x), expand_block16(packed_weight.contiguous()), weight_scales.view(N, -1), bias, out=out)
        return y if in_dtype == torch.bfloat16 else y.to(in_dtype)
    if K % 32 != 0:
        raise _capi.MXFP4BackendError(f"mxfp4: K={K} must be a multiple of 32 (pad activations to the packed weight's width)")
    if x.stride(1) != 1 or (x.stride(0) * 2) % 32 != 0 or x.data_ptr() % 32 != 0:
        x = x.contiguous()
    L = _capi.load()
    dev = x.device
    pw = packed_weight.contiguous()
    sfw = prepared_scales(weight_scales, N, K)
    b = bias_bf16(bias, dev)
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


class FusedChain:
    """Workspace and launches of a chain  fused activation step -> GEMM -> fused activation step -> ...  on one device
    and stream (mxfp4_act_fused + mxfp4_gemm_prequantized_ex): the activations between two GEMMs exist only in MXFP4
    form, a K-split's partial sums are summed by the step that consumes them, and every launch is chained to the one
    in front.  Buffers grow on demand, so run a chain once eagerly before capturing it in a CUDA graph."""

    def __init__(self, device):
        self.dev = device
        self.L = _capi.load()
        self.ctrl = torch.zeros(1024, dtype=torch.int32, device=device)      # 4 KB control block: status word
        self.a_packed = self.a_sf = self.out = None
        self.src = None                                                       # what the last GEMM left for the next step

    def _grow(self, name, nbytes):
        t = getattr(self, name)
        if t is None or t.numel() < nbytes:
            if torch.cuda.is_current_stream_capturing():
                raise _capi.MXFP4BackendError("mxfp4: run the chain once before capturing it (its buffers are allocated on first use)")
            setattr(self, name, torch.empty(_align(nbytes, 256), dtype=torch.uint8, device=self.dev))
        return getattr(self, name)

    def feed(self, x: torch.Tensor):
        """Makes a bf16 matrix [M, K] (row pitch = stride(0)) the input of the next act() -- e.g. an attention output."""
        assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.stride(1) == 1
        self.src = ("bf16", x, x.stride(0))

    def act(self, op, M, K, *, residual=None, hidden_out=None, bias=None, gamma=None, eps=1e-6, peer=None, quantize=True):
        """One mxfp4_act_fused launch on what the previous gemm() left (or on nothing: the first step of a stack)."""
        a = _capi.ActFusedArgs()
        a.op, a.M, a.K, a.eps = op, M, K, eps
        keep = []
        if peer is not None:
            a.peer_blocks, a.world, a.rank = ctypes.cast(peer.blocks, ctypes.POINTER(ctypes.c_void_p)), peer.world, peer.rank
            a.epoch, a.status_dev, a.peer_wait_done = peer.epoch.data_ptr(), peer.status.data_ptr(), 0 if peer.interleaved else 1
            a.ld_in = peer.N
            if getattr(peer, "results", None) is not None and M >= peer.world and M * peer.N * 2 >= getattr(peer, "two_shot_min_bytes", 0):
                a.peer_results = ctypes.cast(peer.results, ctypes.POINTER(ctypes.c_void_p))
                a.owner_count = peer.owner_count.data_ptr()
        elif self.src is not None:
            kind = self.src[0]
            if kind == "bf16":
                a.in_bf16, a.ld_in = self.src[1].data_ptr(), self.src[2]
            else:
                _, t, splits, stride, ld = self.src
                a.in_f32, a.splits, a.split_stride, a.ld_in = t.data_ptr(), splits, stride, ld
            a.status_dev = self.ctrl.data_ptr()
        if residual is not None:
            a.residual, a.ld_res = residual.data_ptr(), residual.stride(0)
        if hidden_out is not None:
            a.hidden_out, a.ld_hid = hidden_out.data_ptr(), hidden_out.stride(0)
        if bias is not None:
            b = bias_bf16(bias, self.dev)
            keep.append(b)
            a.bias = b.data_ptr()
        if gamma is not None:
            g = bias_bf16(gamma, self.dev)
            keep.append(g)
            a.gamma = g.data_ptr()
        if quantize:
            pk = self._grow("a_packed", M * (K // 2))
            sf = self._grow("a_sf", self.L.mxfp4_act_scales_bytes(M, K))
            a.packed, a.sf = pk.data_ptr(), sf.data_ptr()
        with _capi.on_device(self.dev):
            _capi.check(self.L.mxfp4_act_fused(ctypes.byref(a), _capi.stream_ptr(self.dev)), "mxfp4_act_fused")
        self.src = None
        self.act_shape = (M, K)

    def gemm(self, packed_weight, weight_scales, out=None):
        """GEMM of the activations the last act() produced with a packed weight [N, K/2].  Without `out` the result
        stays in the chain's own buffer in whatever form is cheapest (bf16, or the partial sums of a K-split) for the
        next act(); with `out` (bf16 [M, N], e.g. a peer-visible partial buffer) it is a finished bf16 matrix."""
        if _mode < 0:
            raise _capi.MXFP4BackendError("mxfp4: fused chains run on the FP4 tensor cores (MXFP4 activations); "
                                          "the W4A16 mode has no activation quantiser to fuse -- set_gemm_mode('exact')")
        M, K = self.act_shape
        N = packed_weight.shape[0]
        assert packed_weight.shape[1] * 2 == K, "activation width does not match the weight"
        sfw = prepared_scales(weight_scales, N, K)
        ks, pairs = ctypes.c_int(0), ctypes.c_int(0)
        _capi.check(self.L.mxfp4_gemm_plan(M, N, K, _mode, ctypes.byref(ks), ctypes.byref(pairs)), "mxfp4_gemm_plan")
        ksplit = ks.value
        flags = _capi.GEMM_CHAINED
        need = max(M * N * 2, ksplit * M * N * 4 if ksplit > 1 else 0)
        if out is None:
            buf = self._grow("out", need)
            dst, ldo = buf.data_ptr(), N
            flags |= _capi.GEMM_KEEP_PARTIALS
            split_ptr, split_bytes = (buf.data_ptr(), ksplit * M * N * 4) if ksplit > 1 else (None, 0)
            self.src = ("f32", buf, ksplit, M * N, N) if ksplit > 1 else ("bf16", buf, N)
        else:
            dst, ldo = out.data_ptr(), out.stride(0)
            buf = self._grow("out", ksplit * M * N * 4) if ksplit > 1 else None
            split_ptr, split_bytes = (buf.data_ptr(), ksplit * M * N * 4) if ksplit > 1 else (None, 0)
            self.src = ("bf16", out, out.stride(0))
        with _capi.on_device(self.dev):
            _capi.check(self.L.mxfp4_gemm_prequantized_ex(self.a_packed.data_ptr(), self.a_sf.data_ptr(), packed_weight.data_ptr(), sfw.data_ptr(),
                                                          None, dst, ldo, M, N, K, _mode, split_ptr, split_bytes, self.ctrl.data_ptr(), flags,
                                                          _capi.stream_ptr(self.dev)), "mxfp4_gemm_prequantized_ex")
        return N

    def check_status(self):
        code = int(self.ctrl[0].item())
        if code != 0:
            self.ctrl[0] = 0
            raise _capi.MXFP4BackendError(f"mxfp4 fused chain reported status {code} (a device-side wait timed out)")


_w4a16_status = {}               # device index -> int32 status word of the W4A16 kernel


def matmul_w4a16(input, packed_weight, weight_scales, bias=None, block=32, out=None):
    """W4A16 GEMM (mxfp4_gemm_w4a16): bf16 activations as they are, weights decoded to bf16 inside the kernel.  The path of
    scale_format="bf16" weights (no power-of-two scales, so no block-scaled FP4 MMA) and of set_gemm_mode("w4a16");
    the arithmetic of the reference's FallbackBackend.matmul (src/mxfp4/backends.py:295-312)."""
    L = _capi.load()
    M, K = input.shape
    N = packed_weight.shape[0]
    dev = input.device
    if weight_scales.dtype == torch.uint8:
        fmt = _capi.SF["e8m0"]
    else:
        fmt = _capi.SF["bf16"]
        if weight_scales.dtype != torch.bfloat16:
            weight_scales = weight_scales.to(torch.bfloat16)
    in_dtype = input.dtype
    x = input if in_dtype == torch.bfloat16 else input.to(torch.bfloat16)
    if x.stride(1) != 1 or (x.stride(0) * 2) % 16 != 0 or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    if K % 32 != 0:
        raise _capi.MXFP4BackendError(f"mxfp4: K={K} must be a multiple of 32 (pad activations to the packed weight's width)")
    pw, sw = packed_weight.contiguous(), weight_scales.contiguous()
    b = bias_bf16(bias, dev)
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    if M == 0 or N == 0:
        return out.to(in_dtype)
    st = _w4a16_status.get(dev.index)
    if st is None:
        st = _w4a16_status[dev.index] = torch.zeros(1, dtype=torch.int32, device=dev)
    with _capi.on_device(dev):
        _capi.check(L.mxfp4_gemm_w4a16(x.data_ptr(), x.stride(0), pw.data_ptr(), sw.data_ptr(), fmt, block, None if b is None else b.data_ptr(),
                                       out.data_ptr(), out.stride(0), M, N, K, st.data_ptr(), _capi.stream_ptr(dev)), "mxfp4_gemm_w4a16")
    return out if in_dtype == torch.bfloat16 else out.to(in_dtype)


def mxlinear_forward(input: torch.Tensor, packed_weight: torch.Tensor, weight_scales: torch.Tensor,
                     bias: Optional[torch.Tensor], in_features: int, reuse_act: bool = False) -> torch.Tensor:
    """MXLinear.forward for a quantised layer: any leading dimensions, output in the input's dtype."""
    lead = input.shape[:-1]
    x = input.reshape(-1, input.shape[-1])
    k_pad = packed_weight.shape[-1] * 2
    if x.shape[-1] != k_pad:
        # the quantiser padded the weight rows to a multiple of the block; padded weight columns meet zeros
        x = torch.nn.functional.pad(x, (0, k_pad - x.shape[-1]))
    if bias is not None and x.dtype != torch.bfloat16:
        # the reference adds the bias in the input's dtype (F.linear, src/mxfp4/modules.py:140); only bf16 inputs get
        # it from the GEMM epilogue
        y = quant_matmul_2d(x, packed_weight, weight_scales, None, reuse_act=reuse_act)
        y = y + bias.to(device=y.device, dtype=y.dtype)
    else:
        y = quant_matmul_2d(x, packed_weight, weight_scales, bias, reuse_act=reuse_act)
    return y.reshape(*lead, packed_weight.shape[0])
