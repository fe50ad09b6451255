"""mxfp4.llama.LlamaMXDecoder on a tiny Hugging-Face-shaped Llama: the fused chains (norm weights, residuals, silu*mul, q|k|v
and gate|up as one GEMM each) plus an own KV cache against the model's own forward on the same quantised layers."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def tiny_llama(seed=0, kv_heads=2):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=kv_heads,
                      vocab_size=160, max_position_embeddings=64, tie_word_embeddings=False)
    torch.manual_seed(seed)
    return LlamaForCausalLM(cfg).to(torch.bfloat16).eval().cuda()


@pytest.mark.parametrize("kv_heads", [4, 2])
def test_decoder_matches_the_models_own_forward(kv_heads):
    from mxfp4 import gemm, quantize_model_mxfp4
    from mxfp4.llama import LlamaMXDecoder
    model = tiny_llama(kv_heads=kv_heads)
    with torch.no_grad():
        for p in model.parameters():                      # norm weights away from 1 so that their handling is visible
            if p.dim() == 1:
                p.mul_(torch.rand_like(p.float()).to(p.dtype) + 0.5)
    quantize_model_mxfp4(model, verbose=False)
    B, T, new = 6, 9, 5
    ids = torch.randint(0, 160, (B, T), generator=torch.Generator().manual_seed(1)).cuda()
    dec = LlamaMXDecoder(model, max_batch=B + 2, max_len=T + new + 1)      # a cache larger than the batch
    with torch.no_grad():
        want = model(ids).logits[:, -1].float()
        got = dec._forward(ids, T).float()
        err = ((got - want).norm() / want.norm()).item()
        print(f"prefill logits, kv_heads={kv_heads}: rel_fro vs the model's forward {err:.3e}")
        assert err < 5e-2
        first = dec.prefill(ids, chunk=4)                 # two chunks
        assert torch.equal(first, got.argmax(-1))         # same arithmetic per row, whatever the chunking
        eager = dec.decode(new, use_graph=False)
        dec.prefill(ids, chunk=4)
        graphed = dec.decode(new, use_graph=True)
        assert torch.equal(eager, graphed)
        # teacher-forced check of the decode steps: the model's logits on prompt + generated tokens at the positions the
        # decoder predicted from
        full = torch.cat([ids, eager[:, :-1]], 1)
        ref = model(full).logits[:, T - 1:].float()       # [B, new, vocab]: predictions for tokens T .. T+new-1
        dec.prefill(ids, chunk=B)
        for j in range(1, new):
            lg = dec._forward(eager[:, j - 1:j], 1).float()
            dec.pos.add_(1)
            e = ((lg - ref[:, j]).norm() / ref[:, j].norm()).item()
            assert e < 5e-2, (j, e)
    gemm.check_status()
    dec.chain.check_status()
