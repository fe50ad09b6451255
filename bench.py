#!/usr/bin/env python
"""Benchmark of the MXFP4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemm|quantize|stack|decode] [--impl ours|reference]

One JSON line on stdout (rank 0).  Workloads:

  gemm      (default) one step = quant_matmul of bf16 activations [8192, 4096] with an MXFP4 weight [11008, 4096]
            (Llama-2-7B gate/up projection shape of the GEMM sweep): activation quantiser + tcgen05 GEMM; metric =
            TFLOP/s counted as 2*M*N*K.  The same load runs for a second before the timed region so that the K timed
            steps are taken at the clock the power governor settles on; the SM clock is sampled throughout.  After the
            timed region a seeded sample of rows of the last output is compared with the CPU oracle ("parity").
            The line also carries, under "extra", the other parts of the metric: quantise and dequantise GB/s
            (4096 x 4096 with eight rotating buffers, and one Llama-2-7B decoder layer) and the 32-layer MXLinear block
            stack (128-token decode step, 2048-token prefill) tensor-parallel over the N ranks, row-parallel sums inside
            the timed region.
  quantize  one step = MXFP4Quantizer.quantize of the 7 weight matrices of one Llama-2-7B decoder layer.
  stack     the block stack alone.
  decode    HF-shaped Llama-2-7B: quantize_model_mxfp4 + greedy decode (one GPU).

Multi-GPU (gemm): every rank runs the same per-GPU GEMM on its own data (weak scaling, no data-path collective: GEMM
tiles are independent); `value` is the sum over ranks of work divided by the slowest rank's device time.  The block
stack under "extra" is the tensor-parallel part: strong scaling, one process per GPU, sums over peer memory.

`--impl reference` times the CPU port of the reference's own path (dequantise the whole weight, cast, matmul) on this
box's host cores, on the same shape.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "moizmxfp4-public_b200"))

if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":     # keep NCCL's version banner off stdout: one JSON line only
    os.environ["NCCL_DEBUG"] = "WARN"

import torch  # noqa: E402

QUANT_BYTES_PER_ELEM = 2.0 + 0.5 + 1.0 / 32.0
DEQUANT_BYTES_PER_ELEM = 0.5 + 1.0 / 32.0 + 4.0
LAYER_SHAPES = [(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)]
GEMM_M, GEMM_N, GEMM_K = 8192, 11008, 4096


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.stop = index, [], threading.Event()
        self.thread = threading.Thread(target=self.run, daemon=True)

    def run(self):
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self.stop.wait(0.1)

    def __enter__(self):
        self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.thread.join(timeout=6)

    def summary(self):
        mhz = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        reasons = set()
        for s in self.samples:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


def weight(N, K, seed, outliers=False):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.02
    if outliers:
        idx = torch.randperm(N * K, generator=g)[: int(0.001 * N * K)]
        w.view(-1)[idx] *= 50
    return w.to(torch.bfloat16)


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def max_over_ranks(ms, world, device):
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


# ------------------------------------------------------------------------------------------------
# quantize workload
# ------------------------------------------------------------------------------------------------
def run_quantize(args, rank, world, local):
    from mxfp4.quantizer import MXFP4Quantizer
    from mxfp4 import _capi
    dev = torch.device("cuda", local)
    q = MXFP4Quantizer(32, "e8m0")
    host = [weight(n, k, 100 * rank + i).pin_memory() for i, (n, k) in enumerate(LAYER_SHAPES)]
    devw = [h.to(dev) for h in host]
    elems = sum(n * k for n, k in LAYER_SHAPES)
    launches = 0

    def step():
        out = [q.quantize(w) for w in devw]
        return out

    for _ in range(args.warmup):
        step()
    # seven launches of 7-29 us each are launch-bound from Python: replay the layer from a CUDA graph
    graphed = False
    run = step
    try:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            graph_out = step()
        run, graphed = g.replay, True
    except Exception as e:
        sys.stderr.write(f"CUDA graph capture failed ({e}); timing eager launches\n")
        torch.cuda.synchronize()
    for _ in range(3):
        run()
    barrier(world)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    with ClockSampler(local) as cs:
        ev[0].record()
        for _ in range(args.steps):
            run()
            launches += len(devw)
        ev[1].record()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[1])
        if ms < 300:   # keep the GPU busy long enough for a few clock samples
            t_end = time.time() + 0.5
            while time.time() < t_end:
                run()
            torch.cuda.synchronize()
    ms = max_over_ranks(ms, world, dev)
    barrier(world)
    ms_per_step = ms / args.steps
    value = world * elems * QUANT_BYTES_PER_ELEM / (ms_per_step * 1e-3) / 1e9

    # per-launch time of the dominant kernel (the largest matrix), events on the launching stream
    big = devw[4]
    reps = 20
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    others = [devw[5], devw[6], devw[0], devw[1]]
    torch.cuda.synchronize()
    tot = 0.0
    for i in range(reps):
        q.quantize(others[i % 4])                # evicts `big` from L2 between timed launches (4 x >= 33 MB)
        q.quantize(others[(i + 1) % 4])
        e0.record()
        q.quantize(big)
        e1.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e1)
    k_ms = tot / reps
    k_bytes = big.numel() * QUANT_BYTES_PER_ELEM
    pk = peaks()
    roof = {"bound": "hbm", "kernel": "quantize_bf16_b32_kernel [11008x4096]", "achieved": k_bytes / (k_ms * 1e-3) / 1e9,
            "peak": pk["hbm_gbs"], "unit": "GB/s", "peak_source": pk["source"], "traffic": None}
    # DRAM traffic per launch: one ncu capture of this kernel on a 16384x8192 tensor read+wrote 324.08 MB for 339.74 MB of
    # algorithmic bytes (the rest of the output was still in L2); traffic is proportional to the element count
    roof["traffic"] = 324.08 / 339.74 * elems * QUANT_BYTES_PER_ELEM / len(LAYER_SHAPES)
    if graphed:
        # all launches of a step are this one kernel: mean launch duration over the timed region = step time / 7
        roof.update({"kernel": "quantize_bf16_b32_kernel (mean over the 7 launches of a step, timed region)",
                     "achieved": elems * QUANT_BYTES_PER_ELEM / (ms_per_step * 1e-3) / 1e9,
                     "single_launch_11008x4096_gbs": k_bytes / (k_ms * 1e-3) / 1e9})
    roof["frac"] = roof["achieved"] / roof["peak"]

    # end to end through the public API with host buffers
    e2e_ms = None
    outs_host = [(torch.empty(n, k // 2, dtype=torch.uint8).pin_memory(), torch.empty(n, k // 32, dtype=torch.uint8).pin_memory())
                 for n, k in LAYER_SHAPES]
    stage = [torch.empty_like(w) for w in devw]

    def e2e_step():
        for h, d, (hp, hs) in zip(host, stage, outs_host):
            d.copy_(h, non_blocking=True)
            p, s = q.quantize(d)
            hp.copy_(p, non_blocking=True)
            hs.copy_(s, non_blocking=True)
    for _ in range(2):
        e2e_step()
    barrier(world)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), world, dev) / args.steps
    barrier(world)
    h2d = elems * 2
    d2h = elems // 2 + elems // 32
    res = {"metric": "mxfp4_quantize_hbm_gbs", "value": value, "unit": "GB/s", "ms_per_step": ms_per_step,
           "config": {"workload": "quantize: one Llama-2-7B decoder layer (4x4096x4096, 2x11008x4096, 1x4096x11008 bf16), block 32, e8m0",
                      "elements_per_step": elems, "l2": "inputs (405 MB per step) larger than L2", "cuda_graph": graphed},
           "dtype": "bf16->fp4(e2m1-like codes)+e8m0", "roofline": roof, "gpu_launches": launches,
           "e2e": {"value": world * elems * QUANT_BYTES_PER_ELEM / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                   "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
           "clocks": cs.summary()}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        res["cpu_baseline"] = cpu_quantize_baseline()
    return res


def cpu_quantize_baseline(budget_s=12.0):
    from oracle import oracle
    w = weight(4096, 4096, 0, True)
    oracle.quantize(w[:64])
    n, t0 = 0, time.time()
    while True:
        oracle.quantize(w)
        n += 1
        if time.time() - t0 > budget_s or n >= 20:
            break
    dt = (time.time() - t0) / n
    return {"value": w.numel() * QUANT_BYTES_PER_ELEM / dt / 1e9, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": f"{n} x quantize of one 4096x4096 bf16 matrix (C restatement of the reference quantiser, OpenMP)"}


# ------------------------------------------------------------------------------------------------
# gemm workload
# ------------------------------------------------------------------------------------------------
def cpu_gemm_baseline(steps=3, rows=None):
    """The reference's own formulation of the path (FallbackBackend.matmul, src/mxfp4/backends.py:295-312:
    dequantise the whole weight, cast to the activations' dtype, torch.matmul) on the host cores, on the benchmark
    shape: every step dequantises the whole [N, K] weight and multiplies all M activation rows.  The dequantiser is the
    C restatement of the reference's PyTorch code (the reference runs ~15 separate torch ops there); the matmul is
    torch's CPU bf16 matmul, as in the reference."""
    from oracle import oracle
    rows = GEMM_M if rows is None else rows
    torch.set_num_threads(os.cpu_count())
    w = weight(GEMM_N, GEMM_K, 1)
    p, s = oracle.quantize(w)
    x = torch.randn(rows, GEMM_K, generator=torch.Generator().manual_seed(1000)).to(torch.bfloat16)
    oracle.matmul_w4a16(x[:8], p, s)
    t0 = time.time()
    for _ in range(steps):
        oracle.matmul_w4a16(x, p, s)
    dt = (time.time() - t0) / steps
    return {"value": 2.0 * rows * GEMM_N * GEMM_K / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{steps} x dequantise-then-matmul of all {rows} activation rows against the full [{GEMM_N},{GEMM_K}] weight "
                      "(C dequantiser in place of the reference's PyTorch ops + torch CPU bf16 matmul, all host threads)",
            "ms_per_step": dt * 1e3}


def gemm_parity(x_host, packed, scales, y_dev, n_rows=256):
    """Checks what the benchmark timed: a seeded sample of rows of the last output against the CPU oracle.
    rel_fro_operand_matched is the gated figure (activations as the GEMM's own quantiser leaves them, weights exactly as
    the reference dequantises them, float32 product); rel_fro_w4a16 is the distance to the reference's literal
    dequantise-then-matmul on unquantised bf16 activations, i.e. the intrinsic FP4 activation error."""
    from oracle import oracle
    M = x_host.shape[0]
    g = torch.Generator().manual_seed(7)
    rows = torch.cat([torch.tensor([0, M - 1]), torch.randperm(M, generator=g)[:max(n_rows - 2, 0)]]).unique()
    y = y_dev[rows.to(y_dev.device)].float().cpu()
    p, s = packed.cpu(), scales.cpu()
    ref = oracle.matmul_operand_matched(x_host, p, s, rows=rows)
    lit = oracle.matmul_w4a16(x_host[rows], p, s).float()
    return {"rows_checked": int(rows.numel()), "rel_fro_operand_matched": ((y - ref).norm() / ref.norm()).item(),
            "max_abs": (y - ref).abs().max().item(), "rel_fro_w4a16": ((y - lit).norm() / lit.norm()).item(), "tolerance": 1e-2}


def run_gemm(args, rank, world, local):
    import mxfp4
    from mxfp4 import _capi, gemm
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    L = _capi.load()
    M, N, K = GEMM_M, GEMM_N, GEMM_K
    q = mxfp4.MXFP4Quantizer(32, "e8m0")
    packed, scales = q.quantize(weight(N, K, 1 + rank).to(dev))
    nbuf = 2                                            # two activation/output sets: 2 x (67 + 180) MB, far beyond L2
    host_x = [torch.randn(M, K, generator=torch.Generator().manual_seed(1000 + M + i)).to(torch.bfloat16).pin_memory() for i in range(nbuf)]
    xs = [h.to(dev) for h in host_x]
    outs = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(nbuf)]
    flops = 2.0 * M * N * K
    settle_s = 0.0 if args.gemm_shape else args.settle

    def step(i):
        gemm.quant_matmul_2d(xs[i % nbuf], packed, scales, None, out=outs[i % nbuf])   # the public quant_matmul path

    def hold(seconds, fn):
        # keeps the same load on the GPU (in bursts the host can keep ahead of) for `seconds`
        t_end = time.time() + seconds
        i = 0
        while time.time() < t_end:
            for _ in range(50):
                fn(i); i += 1
            torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    gemm.check_status()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as cs:
        hold(settle_s, step)                       # untimed: the governor settles on its sustained clock under this load
        barrier(world)
        e0.record()
        for i in range(args.steps):
            step(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        hold(min(settle_s, 0.4), step)             # the load stays up while the last clock samples are taken
    ms = max_over_ranks(ms, world, dev)
    gemm.check_status()
    parity = None
    if rank == 0 and not args.no_parity:
        parity = gemm_parity(host_x[(args.steps - 1) % nbuf], packed, scales, outs[(args.steps - 1) % nbuf])
    barrier(world)
    ms_per_step = ms / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12

    # dominant kernel alone: the tcgen05 GEMM on pre-quantised activations, events on the launching stream, under the same
    # sustained load (the settle loop runs this very kernel first)
    aq = [gemm.act_quantize(x) for x in xs]
    prep = gemm.prepared_scales(scales, N, K)
    st = torch.zeros(1024, dtype=torch.int32, device=dev)      # 4 KB control block (status word + reserved)
    sp = torch.cuda.current_stream(dev).cuda_stream
    mode = _capi.GEMM_EXACT if gemm.get_gemm_mode() == "exact" else _capi.GEMM_FAST
    reps = max(args.steps, 50)

    def kern(i):
        j = i % nbuf
        rc = L.mxfp4_gemm_prequantized(aq[j][0].data_ptr(), aq[j][1].data_ptr(), packed.data_ptr(), prep.data_ptr(), None, outs[j].data_ptr(),
                                       N, M, N, K, mode, None, 0, st.data_ptr(), sp)
        assert rc == 0, _capi.last_error()
    with ClockSampler(local) as cs_k:
        hold(settle_s, kern)
        torch.cuda.synchronize()
        e0.record()
        for i in range(reps):
            kern(i)
        e1.record()
        torch.cuda.synchronize()
        k_ms = e0.elapsed_time(e1) / reps
        hold(min(settle_s, 0.3), kern)
    assert int(st[0].item()) == 0, "GEMM kernel reported a timed-out wait"
    # the other kernel of a step: the activation quantiser, timed the same way
    e0.record()
    for i in range(reps):
        gemm.act_quantize(xs[i % nbuf])
    e1.record()
    torch.cuda.synchronize()
    aq_ms = e0.elapsed_time(e1) / reps
    pk = peaks()
    # The kernel is timed inside a seconds-long loop under the power cap, so the matching denominator is the SUSTAINED
    # cuBLAS bf16 figure (x 4 as the FP4 proxy: the peaks file has no FP4 entry); the fraction of the burst proxy is given too.
    sustained = settle_s >= 0.5
    fp4_peak = 4.0 * (pk["bf16_tflops_sustained"] if sustained else pk["bf16_tflops"])
    pair = gemm.get_gemm_mode() == "exact" and os.environ.get("MXFP4_GEMM_PAIR", "1") != "0" and M >= 768
    ck = cs_k.summary()
    roof = {"bound": "tensor", "kernel": (f"gemm_mxf4_pair_kernel<256> [{M}x{N}x{K}]" if pair else f"gemm_mxf4_kernel [{M}x{N}x{K}]") + f", {gemm.get_gemm_mode()} mode",
            "achieved": flops / (k_ms * 1e-3) / 1e12, "peak": fp4_peak, "unit": "TFLOP/s",
            "peak_source": (f"4 x {pk['source']} bf16 cuBLAS {'sustained' if sustained else 'burst'} figure "
                            f"({pk['bf16_tflops_sustained'] if sustained else pk['bf16_tflops']} TFLOP/s): MEASURED_PEAKS.json has no FP4 entry; "
                            + ("the kernel is timed in a sustained loop under the power cap" if sustained else "the kernel is timed in a short burst")),
            "frac_of_burst_proxy": flops / (k_ms * 1e-3) / 1e12 / (4.0 * pk["bf16_tflops"]), "frac_of_nominal_9000": flops / (k_ms * 1e-3) / 1e12 / 9000.0,
            "traffic": GEMM_TRAFFIC_BYTES if (M, N, K) == (8192, 11008, 4096) else None, "kernel_ms": k_ms, "launches_timed": reps,
            "act_quantize_ms": aq_ms, "sm_mhz_median": ck["sm_mhz"],
            "kernel_ms_x_sm_mhz": (k_ms * ck["sm_mhz"]) if ck["sm_mhz"] else None,
            "exact_mode_ceiling": "two MMAs per K step (reference codebook): at most 0.5 of the FP4 peak in 2*M*N*K FLOPs"}
    roof["frac"] = roof["achieved"] / roof["peak"]

    # end to end through the public API with host buffers: H2D of the activations, quant_matmul, D2H of the result
    # (quant_matmul_host: row chunks; the copy in, the GEMM and the copy out of neighbouring chunks overlap on three streams)
    host_out = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()

    def e2e_step(i):
        mxfp4.quant_matmul_host(host_x[i % nbuf], packed, scales, out=host_out)
    for i in range(2):
        e2e_step(i)
    barrier(world)
    e0.record()
    for i in range(args.steps):
        e2e_step(i)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), world, dev) / args.steps
    barrier(world)
    res = {"metric": "mxfp4_gemm_tflops", "value": value, "unit": "TFLOP/s", "per_gpu_tflops": value / world,
           "ms_per_step": ms_per_step,
           "config": {"workload": f"quant_matmul: bf16 activations [{M},{K}] x MXFP4 weight [{N},{K}] (Llama-2-7B gate/up shape of the GEMM sweep), "
                                  f"bf16 out, fp32 accumulate, {gemm.get_gemm_mode()} mode; step = activation quantiser + GEMM",
                      "M": M, "N": N, "K": K, "l2": f"two activation/output sets of {(M * K + M * N) * 2 / 1e6:.0f} MB rotate" + ("; each step touches more than L2" if (M * K + M * N) * 2 > 126e6 else ""),
                      "settle_s": settle_s, "timing": f"{settle_s:.1f} s of the same load, untimed, directly before the {args.steps} timed steps; clocks sampled over both"},
           "dtype": "fp4 (e2m1) x fp4 with e8m0 block scales, fp32 accumulate", "roofline": roof, "gpu_launches": 2 * args.steps,
           "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2,
                   "ms_per_step": e2e_ms},
           "clocks": cs.summary()}
    if parity is not None:
        res["parity"] = parity
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        res["cpu_baseline"] = cpu_gemm_baseline()
    return res


# ------------------------------------------------------------------------------------------------
# the other parts of the metric, reported under "extra" of the default line
# ------------------------------------------------------------------------------------------------
def _graph_or_eager(fn, dev):
    """fn() replayed from a CUDA graph when capture works (launch-bound sequences), else fn itself."""
    try:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            keep = fn()
        g._keep = keep
        return g.replay, True
    except Exception as e:
        sys.stderr.write(f"CUDA graph capture failed ({e}); timing eager launches\n")
        torch.cuda.synchronize()
        return fn, False


def _timed_loop(run, local, min_s=0.5, batch=20):
    """Device time per call of run(): untimed settle of min_s, then batches until min_s of timed work; clocks sampled."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as cs:
        t_end = time.time() + min_s
        while time.time() < t_end:
            for _ in range(batch):
                run()
            torch.cuda.synchronize()
        n, tot = 0, 0.0
        while tot < min_s * 1e3 and n < 100000:
            e0.record()
            for _ in range(batch):
                run()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
            n += batch
    return tot / n, n, cs.summary()


def extra_quantize_dequantize(local):
    """Quantise and dequantise GB/s: one 4096 x 4096 bf16 weight per launch with eight distinct buffers rotating (268 MB of
    inputs, beyond L2), and the seven matrices of one Llama-2-7B decoder layer (405 MB).  Algorithmic bytes per element:
    quantise 2 + 0.5 + 1/32 = 2.53125, dequantise to float32 0.5 + 1/32 + 4 = 4.53125."""
    from mxfp4.quantizer import MXFP4Quantizer
    dev = torch.device("cuda", local)
    q = MXFP4Quantizer(32, "e8m0")
    pk = peaks()
    out = {}
    sets = {"4096x4096_x8_rotating": [weight(4096, 4096, i, outliers=(i == 0)).to(dev) for i in range(8)],
            "llama7b_layer": [weight(n, k, 50 + i).to(dev) for i, (n, k) in enumerate(LAYER_SHAPES)]}
    for name, ws in sets.items():
        elems = sum(w.numel() for w in ws)
        run, graphed = _graph_or_eager(lambda: [q.quantize(w) for w in ws], dev)
        ms, n, clk = _timed_loop(run, local)
        gbs = elems * QUANT_BYTES_PER_ELEM / (ms * 1e-3) / 1e9
        out.setdefault("quantize", {})[name] = {
            "value": gbs, "unit": "GB/s", "ms_per_pass": ms, "launches_per_pass": len(ws), "passes_timed": n, "cuda_graph": graphed,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                         "bytes_per_element": QUANT_BYTES_PER_ELEM, "peak_source": pk["source"]}, "clocks": clk}
        qs = [q.quantize(w) for w in ws]
        run, graphed = _graph_or_eager(lambda: [q.dequantize(p, s) for p, s in qs], dev)
        ms, n, clk = _timed_loop(run, local)
        gbs = elems * DEQUANT_BYTES_PER_ELEM / (ms * 1e-3) / 1e9
        out.setdefault("dequantize", {})[name] = {
            "value": gbs, "unit": "GB/s", "ms_per_pass": ms, "launches_per_pass": len(ws), "passes_timed": n, "cuda_graph": graphed,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                         "bytes_per_element": DEQUANT_BYTES_PER_ELEM, "peak_source": pk["source"]}, "clocks": clk}
        del run, qs
    return out


def extra_tp_stack(rank, world, local, n_layers=32):
    """The 32-layer Llama-2-7B-shaped MXLinear block stack, column/row tensor-parallel over the ranks (strong scaling): a
    128-token decode step and a 2048-token prefill, each replayed from a CUDA graph; the row-parallel sums run inside the
    timed region.  Device time, max over ranks."""
    from mxfp4 import gemm
    from mxfp4.parallel import MXBlockStack
    dev = torch.device("cuda", local)
    stack = MXBlockStack.build(n_layers=n_layers, device=dev, init="cuda")
    w_elems = n_layers * (4 * 4096 * 4096 + 3 * 11008 * 4096)
    pk = peaks()
    out = {"parallelism": f"tp{world}", "scaling": "strong", "layers": n_layers,
           "launches_per_layer": 8,
           "collective": "none" if world == 1 else "64 row-parallel sums of [M, 4096] bf16 per step over NVLink peer memory, inside mxfp4_act_fused "
                                                   "(the kernel that also adds the residual, normalises and quantises the next GEMM's activations)"}
    for name, M in (("decode_M128", 128), ("prefill_M2048", 2048)):
        x = torch.randn(M, 4096, generator=torch.Generator().manual_seed(M)).to(torch.bfloat16).to(dev)
        with torch.no_grad():
            for _ in range(3):
                y = stack(x)
            gemm.check_status()
            run, graphed = _graph_or_eager(lambda: stack(x), dev)
            for _ in range(3):
                run()
            barrier(world)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            steps = 100 if M <= 128 else 20
            with ClockSampler(local) as cs:
                for _ in range(steps // 2):                 # untimed: same load while the clock settles
                    run()
                barrier(world)
                e0.record()
                for _ in range(steps):
                    run()
                e1.record()
                torch.cuda.synchronize()
            ms = max_over_ranks(e0.elapsed_time(e1), world, dev) / steps
            gemm.check_status()
            y = stack(x)
            same = True
            if world > 1:
                import torch.distributed as dist
                ys = [torch.empty_like(y) for _ in range(world)]
                dist.all_gather(ys, y.contiguous())
                same = all(torch.equal(ys[0], t) for t in ys)
            barrier(world)
        rec = {"ms_per_step": ms, "tokens_per_s": M / (ms * 1e-3), "steps_timed": steps, "cuda_graph": graphed,
               "finite": bool(torch.isfinite(y.float()).all().item()), "all_ranks_bit_identical": same, "clocks": cs.summary()}
        if M <= 128:
            gbs = w_elems * (0.5 + 1 / 32) / world / (ms * 1e-3) / 1e9
            rec["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                               "what": "packed weights + scales of this rank's shards streamed once per step"}
        else:
            tf = 2.0 * M * w_elems / world / (ms * 1e-3) / 1e12
            rec["roofline"] = {"bound": "tensor", "achieved": tf, "peak": 4.0 * pk["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / (4.0 * pk["bf16_tflops"]),
                               "what": "2*M*N*K of this rank's shards"}
        out[name] = rec
        del run
    return out


def run_gemm_sweep(args, local):
    """Kernel-only times over a grid of shapes: mxfp4_gemm_prequantized in the FP4 modes, mxfp4_gemm_w4a16 in w4a16 mode
    (current MXFP4_GEMM_MODE / MXFP4_GEMM_PAIR settings)."""
    import mxfp4
    from mxfp4 import _capi, gemm
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    L = _capi.load()
    ms_part, nk_part = args.sweep.split(":")
    q = mxfp4.MXFP4Quantizer(32, "e8m0")
    mode = _capi.GEMM_EXACT if gemm.get_gemm_mode() == "exact" else _capi.GEMM_FAST
    rows = []
    for nk in nk_part.split(","):
        N, K = (int(v) for v in nk.lower().split("x"))
        packed, scales = q.quantize(weight(N, K, 3).to(dev))
        prep = gemm.prepared_scales(scales, N, K)
        for M in (int(v) for v in ms_part.split(",")):
            x = torch.randn(M, K, generator=torch.Generator().manual_seed(11)).to(torch.bfloat16).to(dev)
            aq = gemm.act_quantize(x)
            out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            nsp = L.mxfp4_gemm_splitk_bytes(M, N, K)
            spl = torch.empty(max(nsp, 16), dtype=torch.uint8, device=dev)
            st = torch.zeros(1024, dtype=torch.int32, device=dev)
            sp = torch.cuda.current_stream(dev).cuda_stream

            def kern():
                if gemm.get_gemm_mode() == "w4a16":
                    gemm.matmul_w4a16(x, packed, scales, None, 32, out=out)
                    return
                rc = L.mxfp4_gemm_prequantized(aq[0].data_ptr(), aq[1].data_ptr(), packed.data_ptr(), prep.data_ptr(), None, out.data_ptr(),
                                               N, M, N, K, mode, spl.data_ptr(), nsp, st.data_ptr(), sp)
                assert rc == 0, _capi.last_error()
            for _ in range(3):
                kern()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                kern()
            e1.record()
            torch.cuda.synchronize()
            assert int(st[0].item()) == 0, "GEMM kernel reported a timed-out wait"
            gemm.check_status()
            us = e0.elapsed_time(e1) / 10 * 1e3
            rows.append({"M": M, "N": N, "K": K, "kernel_us": round(us, 1), "tflops": round(2.0 * M * N * K / us / 1e6, 0)})
    return {"sweep": rows, "mode": gemm.get_gemm_mode(), "pair": os.environ.get("MXFP4_GEMM_PAIR", "default")}


# ------------------------------------------------------------------------------------------------
# stack workload: 32-layer Llama-2-7B-shaped MXLinear block stack, tensor-parallel over the ranks
# ------------------------------------------------------------------------------------------------
def run_stack(args, rank, world, local):
    from mxfp4 import gemm
    from mxfp4.parallel import MXBlockStack
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    stack = MXBlockStack.build(n_layers=32, device=dev, init="cuda")   # sharded over the default process group when world > 1
    out = {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cs_sum = None
    for name, M, steps in (("decode_M128", 128, args.steps), ("prefill_M2048", 2048, max(2, args.steps // 4))):
        x = torch.randn(M, 4096, generator=torch.Generator().manual_seed(M)).to(torch.bfloat16).to(dev)
        with torch.no_grad():
            for _ in range(args.warmup):
                stack(x)
            gemm.check_status()
            # the step is launch-bound from Python (224 small GEMMs): capture it once into a CUDA graph and replay it
            graphed = False
            try:
                side = torch.cuda.Stream(dev)
                side.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(side):
                    stack(x)                                   # allocates the side stream's GEMM workspace before capture
                torch.cuda.current_stream(dev).wait_stream(side)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    y = stack(x)
                run = g.replay
                graphed = True
            except Exception as e:                             # keep measuring eagerly if capture is not possible
                sys.stderr.write(f"CUDA graph capture failed ({e}); timing eager launches\n")
                torch.cuda.synchronize()
                run = lambda: stack(x)
            for _ in range(3):
                run()
            barrier(world)
            with ClockSampler(local) as cs:
                e0.record()
                for _ in range(steps):
                    r = run()
                    if not graphed:
                        y = r
                e1.record()
                torch.cuda.synchronize()
            ms = max_over_ranks(e0.elapsed_time(e1), world, dev) / steps
            gemm.check_status()
            barrier(world)
        out[name] = {"ms_per_step": ms, "tokens_per_s": M / (ms * 1e-3), "finite": bool(torch.isfinite(y.float()).all().item()), "cuda_graph": graphed}
        cs_sum = cs.summary()
    w_elems = 32 * (4 * 4096 * 4096 + 3 * 11008 * 4096)
    dec = out["decode_M128"]
    res = {"metric": "mxlinear_stack_decode_tokens_per_s", "value": dec["tokens_per_s"], "unit": "tokens/s", "ms_per_step": dec["ms_per_step"],
           "config": {"workload": "32 x (q,k,v,o 4096x4096; gate,up 11008x4096; down 4096x11008) MXLinear block stack, 128-token decode step; "
                                  "also a 2048-token prefill; column/row tensor-parallel over the ranks (2 NCCL all-reduces per layer)",
                      "parallelism": f"tp{world}", "l2": "3.44 GB of packed weights per step, larger than L2"},
           "dtype": "fp4 x fp4, e8m0 block scales, fp32 accumulate", "stack": out, "gpu_launches": 32 * 7 * 2 * args.steps,
           "roofline": {"bound": "hbm", "kernel": "whole decode step (weights streamed once)", "achieved": w_elems * (0.5 + 1 / 32) / world / (dec["ms_per_step"] * 1e-3) / 1e9,
                        "peak": peaks()["hbm_gbs"], "unit": "GB/s", "traffic": None},
           "clocks": cs_sum, "scaling_note": "strong"}
    res["roofline"]["frac"] = res["roofline"]["achieved"] / res["roofline"]["peak"]
    return res


# ------------------------------------------------------------------------------------------------
# decode workload: random-init Llama-2-7B architecture, quantize_model_mxfp4, greedy decode (one GPU)
# ------------------------------------------------------------------------------------------------
def run_decode(args, rank, world, local):
    """Config 4: random-init Llama-2-7B architecture (Hugging Face LlamaForCausalLM), quantize_model_mxfp4, greedy decode of
    128 new tokens at batch 128 from 512-token uniform-random prompts, tensor-parallel over the ranks.  The linear layers
    run as this library's fused chains (mxfp4.llama.LlamaMXDecoder); attention is torch's scaled_dot_product_attention on
    a preallocated KV cache; a decode step is replayed from a CUDA graph.  MXFP4_DECODE_HF=1 times Hugging Face's own
    generate loop on the quantised model instead (one GPU)."""
    import mxfp4
    from mxfp4 import gemm
    from transformers import LlamaConfig, LlamaForCausalLM
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    layers = int(os.environ.get("MXFP4_DECODE_LAYERS", "32"))
    cfg = LlamaConfig(hidden_size=4096, intermediate_size=11008, num_hidden_layers=layers, num_attention_heads=32, num_key_value_heads=32,
                      vocab_size=32000, max_position_embeddings=4096, torch_dtype=torch.bfloat16)
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    n_lin = sum(m.weight.numel() for m in model.modules() if isinstance(m, torch.nn.Linear))
    torch.cuda.synchronize()
    t0 = time.time()
    mxfp4.quantize_model_mxfp4(model, verbose=False)
    torch.cuda.synchronize()
    t_quant = time.time() - t0
    batch, prompt, new = 128, 512, 128
    ids = torch.randint(0, 32000, (batch, prompt), generator=torch.Generator().manual_seed(4)).to(dev)
    hf = os.environ.get("MXFP4_DECODE_HF", "0") == "1" and world == 1
    with torch.no_grad():
        if hf:
            model.generate(ids[:2, :16], max_new_tokens=4, do_sample=False)        # warm-up of kernels and caches
            torch.cuda.synchronize()
            with ClockSampler(local) as cs:
                t0 = time.time()
                model(ids[:, :prompt])                                              # prefill alone, to separate it from decode
                torch.cuda.synchronize()
                t_prefill = time.time() - t0
                t0 = time.time()
                out = model.generate(ids, max_new_tokens=new, min_new_tokens=new, do_sample=False)
                torch.cuda.synchronize()
                t_gen = time.time() - t0
            t_dec = max(t_gen - t_prefill, 1e-9)
            n_new = int(out.shape[1] - prompt)
            how = "Hugging Face generate loop and attention, growing KV cache"
        else:
            from mxfp4.llama import LlamaMXDecoder

            def note(msg):
                if os.environ.get("MXFP4_BENCH_TRACE"):
                    sys.stderr.write(f"[rank {rank}] {time.strftime('%H:%M:%S')} decode: {msg}\n"); sys.stderr.flush()
            dec = LlamaMXDecoder(model, batch, prompt + new)
            del model
            torch.cuda.empty_cache()
            barrier(world)
            note("first prefill (buffers, peer set-up)")
            dec.prefill(ids)
            torch.cuda.synchronize()
            barrier(world)
            note("timed prefill")
            t0 = time.time()
            dec.prefill(ids)
            torch.cuda.synchronize()
            barrier(world)
            t_prefill = time.time() - t0
            note("graph capture")
            dec.decode(2)                                                            # captures the batch-128 step
            torch.cuda.synchronize()
            dec.prefill(ids)
            barrier(world)
            note("timed decode")
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with ClockSampler(local) as cs:
                e0.record()
                toks = dec.decode(new)
                e1.record()
                torch.cuda.synchronize()
            note("done")
            t_dec = max_over_ranks(e0.elapsed_time(e1), world, dev) * 1e-3
            t_gen = t_dec + t_prefill
            n_new = int(toks.shape[1])
            dec.chain.check_status()
            how = ("fused MXFP4 chains for the linear layers (8 launches + attention per layer), torch scaled_dot_product_attention on a "
                   "preallocated KV cache, decode step replayed from a CUDA graph")
    gemm.check_status()
    steps = max(n_new - 1, 1) if not hf else n_new
    return {"metric": "llama7b_shape_decode_tokens_per_s", "value": batch * steps / t_dec, "unit": "tokens/s", "ms_per_step": t_dec / steps * 1e3,
            "config": {"workload": f"random-init Llama-2-7B architecture ({layers} layers), quantize_model_mxfp4 (225 Linear incl. lm_head), "
                                   "greedy decode of 128 new tokens at batch 128 from 512-token random prompts; " + how,
                       "parallelism": f"tp{world}"},
            "dtype": "fp4 x fp4 linear layers, bf16 elsewhere", "generate_s": t_gen, "prefill_s": t_prefill, "new_tokens": n_new,
            "quantize_model": {"seconds": t_quant, "linear_elements": n_lin, "gbs": n_lin * QUANT_BYTES_PER_ELEM / t_quant / 1e9},
            "gpu_launches": None, "clocks": cs.summary(), "scaling_note": "strong"}


def extra_w4a16(local):
    """The same GEMM shape in W4A16 mode (bf16 activations untouched, weights decoded to bf16 inside the kernel, bf16
    tensor cores): the reference's literal arithmetic.  Roofline against the measured cuBLAS bf16 rate."""
    import mxfp4
    from mxfp4 import gemm
    from oracle import oracle
    dev = torch.device("cuda", local)
    M, N, K = GEMM_M, GEMM_N, GEMM_K
    packed, scales = mxfp4.MXFP4Quantizer(32, "e8m0").quantize(weight(N, K, 1).to(dev))
    hx = [torch.randn(M, K, generator=torch.Generator().manual_seed(1000 + M + i)).to(torch.bfloat16) for i in range(2)]
    xs = [h.to(dev) for h in hx]
    outs = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    i = [0]

    def run():
        gemm.matmul_w4a16(xs[i[0] % 2], packed, scales, None, 32, out=outs[i[0] % 2])
        i[0] += 1
    ms, n, clk = _timed_loop(run, local, min_s=0.5, batch=10)
    gemm.check_status()
    j = (i[0] - 1) % 2
    rows = torch.cat([torch.tensor([0, M - 1]), torch.randperm(M, generator=torch.Generator().manual_seed(7))[:254]]).unique()
    ref = oracle.matmul_w4a16(hx[j][rows], packed.cpu(), scales.cpu()).float()
    y = outs[j][rows.to(dev)].float().cpu()
    pk = peaks()
    tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
    return {"value": tf, "unit": "TFLOP/s", "ms_per_launch": ms, "launches_timed": n, "kernel": f"gemm_w4a16_kernel<256, 1> [{M}x{N}x{K}]",
            "parity": {"rows_checked": int(rows.numel()), "rel_fro_w4a16": ((y - ref).norm() / ref.norm()).item(), "max_abs": (y - ref).abs().max().item(),
                       "tolerance": 1e-2, "oracle": "the reference's literal dequantise-then-matmul (FallbackBackend.matmul)"},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": tf / pk["bf16_tflops_sustained"],
                         "peak_source": f"{pk['source']} cuBLAS bf16 sustained"}, "clocks": clk}


def extra_llama_decode(args, rank, world, local):
    """Config 4 as a sub-record of the default line: Llama-2-7B-shape greedy decode, tensor-parallel over the ranks."""
    r = run_decode(args, rank, world, local)
    return {"value": r["value"], "unit": r["unit"], "ms_per_step": r["ms_per_step"], "parallelism": r["config"]["parallelism"], "scaling": "strong",
            "workload": r["config"]["workload"], "prefill_s": r["prefill_s"], "new_tokens": r["new_tokens"], "quantize_model": r["quantize_model"],
            "clocks": r["clocks"]}


# DRAM traffic of one GEMM launch of the bench shape: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture
# (two launches: 46.2 / 46.3 MB read, 141.6 / 138.1 MB written)
GEMM_TRAFFIC_BYTES = 46.25e6 + 139.85e6


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--settle", type=float, default=1.0, help="seconds of the same load run untimed directly before the timed steps")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the timed output")
    ap.add_argument("--no-extras", action="store_true", help="gemm workload: skip the quantise / dequantise / block-stack sub-records")
    ap.add_argument("--workload", default=os.environ.get("MXFP4_BENCH_WORKLOAD", "gemm"), choices=["quantize", "gemm", "stack", "decode"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gemm-shape", default=None, metavar="MxNxK",
                    help="gemm workload on another shape (profiling captures on a small case); the default is the bench shape")
    ap.add_argument("--sweep", default=None, metavar="M,M,..:NxK,NxK,..",
                    help="gemm workload: time only the GEMM kernel (10 launches after 3 warm-ups) for every M x (N,K) and print one JSON line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        rank = int(os.environ.get("RANK", "0"))
        if rank != 0:
            return
        if args.workload == "gemm":
            base = cpu_gemm_baseline(steps=max(1, min(args.steps, 5)))     # the steps are capped, not the rows: same shape as our arm
            metric, unit, cfg = "mxfp4_gemm_tflops", "TFLOP/s", (f"quant_matmul: bf16 activations [{GEMM_M},{GEMM_K}] x MXFP4 weight [{GEMM_N},{GEMM_K}] "
                                                                 "(Llama-2-7B gate/up shape of the GEMM sweep); " + base["sample"])
        else:
            base = cpu_quantize_baseline(budget_s=max(5.0, 2.0 * args.steps))
            metric, unit, cfg = "mxfp4_quantize_hbm_gbs", "GB/s", "quantize (bounded sample: one 4096x4096 matrix per step)"
        out = {"impl": "reference", "metric": metric, "value": base["value"], "unit": unit, "n_gpus": args.gpus,
               "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
               "dtype": "bf16 x bf16 (dequantised weight), CPU", "data": "synthetic",
               "config": {"workload": cfg, "M": GEMM_M, "N": GEMM_N, "K": GEMM_K},
               "ms_per_step": base.get("ms_per_step"), "steps_timed": max(1, min(args.steps, 5)) if args.workload == "gemm" else None,
               "port_note": "the reference is pure Python (PyTorch CPU ops); this arm runs its formulation with the dequantiser restated in C "
                            "(faster than the reference's own ~15 torch ops) and the same torch CPU matmul",
               "cpu_baseline": base, "e2e": {"value": base["value"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(out))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product has no CPU path); use --impl reference for the CPU baseline")
    rank, world, local = dist_setup(args.gpus)
    if args.gemm_shape:
        g = globals()
        g["GEMM_M"], g["GEMM_N"], g["GEMM_K"] = (int(v) for v in args.gemm_shape.lower().split("x"))
    if args.sweep:
        if rank == 0:
            print(json.dumps(run_gemm_sweep(args, local)))
        return
    res = {"gemm": run_gemm, "quantize": run_quantize, "stack": run_stack, "decode": run_decode}[args.workload](args, rank, world, local)
    if args.workload == "gemm" and not args.no_extras and not args.gemm_shape:
        extra = {}
        for name, fn in (("quantize_dequantize", (lambda: extra_quantize_dequantize(local)) if world == 1 else None),
                         ("w4a16_gemm", (lambda: extra_w4a16(local)) if world == 1 else None),
                         ("tp_stack", lambda: extra_tp_stack(rank, world, local)),
                         ("llama_decode", lambda: extra_llama_decode(args, rank, world, local))):
            if fn is None:
                continue
            try:
                torch.cuda.empty_cache()
                if os.environ.get("MXFP4_BENCH_TRACE"):
                    sys.stderr.write(f"[rank {rank}] {time.strftime('%H:%M:%S')} extra: {name}\n"); sys.stderr.flush()
                r = fn()
                if name == "quantize_dequantize":
                    extra.update(r)
                else:
                    extra[name] = r
            except Exception as e:            # a sub-record must not take the main line down; it says what happened
                if world > 1:
                    raise                     # ranks must not diverge
                extra[name] = {"error": f"{type(e).__name__}: {e}"}
        res["extra"] = extra
    res.update({"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "data": "synthetic"})
    if "scaling_note" in res:
        res["scaling"] = res.pop("scaling_note")
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
