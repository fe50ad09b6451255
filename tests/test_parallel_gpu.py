"""Tensor-parallel MXLinear layers on real GPUs (2, 4 and 8 ranks; a case is skipped when the box has fewer devices):
each rank is a child process with its own GPU; the row-parallel sum runs as this library's kernels over peer memory
(mxfp4_peer_allreduce for single layers, mxfp4_act_fused inside the block stack), NCCL being the comparison.  Column-parallel shards must be bit-identical to
the matching slice of the unsharded output; the row-parallel sum is compared within the GEMM tolerance."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        import conftest
        from mxfp4 import MXLinear, gemm
        from mxfp4.parallel import ColumnParallelMXLinear, MXBlockStack, RowParallelMXLinear
        dev = torch.device("cuda", rank)
        up = MXLinear(4096, 11008, bias=False)
        down = MXLinear(11008, 4096, bias=True)
        up.weight.data = conftest.weight(11008, 4096, 1, True).float()
        down.weight.data = conftest.weight(4096, 11008, 2, True).float()
        up.to(dev); down.to(dev)
        up.quantize(); down.quantize()
        x = conftest.act(128, 4096, 5).to(dev)
        h_full = up(x)
        full = down(torch.relu(h_full))
        cp = ColumnParallelMXLinear.from_mxlinear(up)
        rp = RowParallelMXLinear.from_mxlinear(down)
        h = cp(x)
        n = 11008 // world
        ok_col = torch.equal(h, h_full[:, rank * n:(rank + 1) * n])
        y = rp(torch.relu(h))
        err = ((y.float() - full.float()).norm() / full.float().norm()).item()
        # The row-parallel sum ran as this library's kernel over peer memory.  With two ranks NCCL's bf16 all-reduce rounds
        # the same float32 sum once, so the two paths must agree bit for bit; the second and third call use the next call
        # numbers of the device-side epoch, the larger M re-makes the peer buffer, and a CUDA graph replays the launch.
        ok_peer = getattr(rp, "_peer", None) is not None and not rp._peer.disabled
        if ok_peer:
            hin = torch.relu(h)
            y2 = rp(hin)
            rp._peer.disabled = True
            y_nccl = rp(hin)
            rp._peer.disabled = False
            ok_peer = torch.equal(y, y2) and (world != 2 or torch.equal(y, y_nccl))
            big = torch.relu(cp(conftest.act(640, 4096, 6).to(dev)))
            yb = rp(big)
            rp._peer.disabled = True
            yb_nccl = rp(big)
            rp._peer.disabled = False
            ok_peer = ok_peer and (world != 2 or torch.equal(yb, yb_nccl))
            g = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                rp(hin)
                torch.cuda.synchronize()
                with torch.cuda.graph(g, stream=side):
                    yg = rp(hin)
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            ok_peer = ok_peer and torch.equal(yg, y)
            rp._peer.check_status()
        xin = conftest.act(16, 4096, 9).to(dev)
        stack = MXBlockStack.build(n_layers=2, device=dev)
        out = stack(xin)
        unfused = MXBlockStack.build(n_layers=2, device=dev, fuse=False)(xin)
        # the fused layers may pick another K-split, i.e. another float32 summation order: equal up to bf16 rounding
        assert ((out.float() - unfused.float()).norm() / unfused.float().norm()).item() < 2e-3
        gemm.check_status()
        # the other mode of the fused peer sum (one-shot: every rank reads all partials; two-shot: every rank reduces its
        # own rows and fetches the others' results) computes every row with the same arithmetic: same bits
        default_two_shot = stack.layers[0]["o"]._peer.two_shot
        os.environ["MXFP4_TP_TWO_SHOT"] = "0" if default_two_shot else "1"
        try:
            other = MXBlockStack.build(n_layers=2, device=dev)
            out_other = other(xin)
            assert other.layers[0]["o"]._peer.two_shot != default_two_shot
        finally:
            os.environ.pop("MXFP4_TP_TWO_SHOT")
        assert torch.equal(out, out_other)
        fin = bool(torch.isfinite(out.float()).all().item())
        ref = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(ref, out)
        same = all(torch.equal(ref[0], r) for r in ref)           # every rank ends with the same replicated activations
        # the Llama decoder under tensor parallelism against the same decoder on one rank (a one-rank group per process)
        from transformers import LlamaConfig, LlamaForCausalLM
        from mxfp4 import quantize_model_mxfp4
        from mxfp4.llama import LlamaMXDecoder
        solo = None
        for r in range(world):
            g = dist.new_group([r])
            if r == rank:
                solo = g
        heads = max(4, world)
        cfg = LlamaConfig(hidden_size=32 * heads, intermediate_size=64 * world, num_hidden_layers=2, num_attention_heads=heads,
                          num_key_value_heads=heads, vocab_size=96, max_position_embeddings=64, tie_word_embeddings=False)
        torch.manual_seed(0)
        model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval().to(dev)
        quantize_model_mxfp4(model, verbose=False)
        ids = torch.randint(0, cfg.vocab_size, (5, 7), generator=torch.Generator().manual_seed(2)).to(dev)
        with torch.no_grad():
            ref = LlamaMXDecoder(model, 5, 16, group=solo)._forward(ids, 7).float()
            tp = LlamaMXDecoder(model, 5, 16)
            lg = tp._forward(ids, 7).float()
            # sharding rounds every rank's partial products to bf16 before they are summed and the next FP4 activation
            # quantiser turns last-bit differences into code flips: on this tiny random model that is 10-15 % of the logits'
            # norm (an error in the sharding itself would give ~100 %)
            err_dec = ((lg - ref).norm() / ref.norm()).item()
            tp.prefill(ids)
            toks = tp.decode(4)
            tl = [torch.empty_like(toks) for _ in range(world)]
            dist.all_gather(tl, toks)
            same_toks = all(torch.equal(tl[0], t) for t in tl)
            tp.chain.check_status()
        q.put((rank, ok_col and ok_peer and err < 1e-2 and fin and same and err_dec < 0.25 and same_toks, (err, err_dec)))
    except Exception as e:                     # report instead of leaving the parent to time out
        q.put((rank, False, repr(e)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_layers_real_ranks(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 200 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok, _ in res), res
