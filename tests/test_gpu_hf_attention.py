"""Stock HF forward / generate with the paged TurboQuant cache plugged in as the attention function:
decode steps run on the packed pages (fused kernel), and must agree with the same cache used the
compatible way (dense K/V de-quantized from the pages + SDPA)."""

import pytest
import torch

from conftest import rel_l2
from leankv_b200.combined import optimize_model, reset_optimizations

pytestmark = pytest.mark.gpu


def _model():
    from transformers import MistralConfig, MistralForCausalLM

    torch.manual_seed(0)
    cfg = MistralConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                        num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                        max_position_embeddings=256, rope_theta=1e6, tie_word_embeddings=False)
    return MistralForCausalLM(cfg).half().to("cuda:0").eval()


def _steps(model, cache, ids, forced):
    logits = []
    with torch.no_grad():
        out = model(ids, past_key_values=cache, use_cache=True)
        logits.append(out.logits[:, -1].float().cpu())
        for tok in forced:
            out = model(tok.reshape(-1, 1).to(ids.device), past_key_values=cache, use_cache=True)
            logits.append(out.logits[:, -1].float().cpu())
    return logits


def test_fused_decode_matches_dense_route_and_generate_runs(capsys):
    model = _model()
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 512, (2, 37), generator=g).to("cuda:0")       # two sequences, ragged page fill
    forced = [torch.randint(0, 512, (2,), generator=g) for _ in range(20)]  # crosses a page boundary (37 -> 57)

    _, dense_cache = optimize_model(model, use_paged_cache=True, max_pages=64)
    want = _steps(model, dense_cache, ids, forced)

    _, cache = optimize_model(model, use_paged_cache=True, max_pages=64, fused_attention=True)
    assert cache.fused_decode and model.config._attn_implementation == "leankv_paged"
    got = _steps(model, cache, ids, forced)
    assert cache.kernel_status() == 0
    errs = [rel_l2(a, b) for a, b in zip(got, want)]
    print("fused vs dense-route logits rel-L2:", [f"{e:.1e}" for e in errs])
    assert errs[0] < 1e-6                     # the prompt pass is the same code either way
    assert max(errs) < 1e-2                   # fp16 K_hat/V_hat + SDPA vs fp32 accumulation on the codes
    # same pages either way: the appended codes do not depend on which attention ran
    assert torch.equal(cache.kv_data[0][int(cache._block_table[0, 0])],
                       dense_cache.kv_data[0][int(dense_cache._block_table[0, 0])])

    # stock generate() on a fresh cache
    reset_optimizations(model)
    _, cache2 = optimize_model(model, use_paged_cache=True, max_pages=64, fused_attention=True)
    out = model.generate(ids[:1], past_key_values=cache2, max_new_tokens=12, do_sample=False,
                         pad_token_id=0)
    assert out.shape == (1, 37 + 12)
    assert cache2.get_seq_length() == 37 + 11
    reset_optimizations(model)
    assert model.config._attn_implementation != "leankv_paged"


def test_fused_prefill_runs_prompt_chunks_on_the_packed_pages():
    """With ``fused_prefill`` a prompt pass only appends and attends on the packed pages: logits of the
    prompt, of a second chunk fed on top of it, and of decode steps after both, against the dense route."""
    model = _model()
    g = torch.Generator().manual_seed(6)
    ids = torch.randint(0, 512, (2, 45), generator=g).to("cuda:0")
    more = torch.randint(0, 512, (2, 21), generator=g).to("cuda:0")       # a second chunk: starts mid-page
    forced = [torch.randint(0, 512, (2,), generator=g) for _ in range(4)]

    def run(cache):
        with torch.no_grad():
            a = model(ids, past_key_values=cache, use_cache=True).logits.float().cpu()
            b = model(more, past_key_values=cache, use_cache=True).logits.float().cpu()
        return [a, b] + _steps_only(model, cache, forced)

    def _steps_only(model, cache, forced):
        outs = []
        with torch.no_grad():
            for tok in forced:
                outs.append(model(tok.reshape(-1, 1).to("cuda:0"), past_key_values=cache,
                                  use_cache=True).logits[:, -1].float().cpu())
        return outs

    _, dense_cache = optimize_model(model, use_paged_cache=True, max_pages=64)
    want = run(dense_cache)
    reset_optimizations(model)
    _, cache = optimize_model(model, use_paged_cache=True, max_pages=64, fused_attention=True, fused_prefill=True)
    assert cache.fused_prefill
    got = run(cache)
    assert cache.kernel_status() == 0
    errs = [rel_l2(a, b) for a, b in zip(got, want)]
    print("fused prefill vs dense-route logits rel-L2:", [f"{e:.1e}" for e in errs])
    assert max(errs) < 1e-2
    assert cache.get_seq_length() == 45 + 21 + 4
    reset_optimizations(model)
    assert not cache.fused_prefill
