"""The HF attention-interface plug-in, on CPU with a stand-in cache built from the oracle.

The stand-in keeps the de-quantized K/V the oracle produces and implements ``decode_attention``
with plain fp32 math, so the test checks the plumbing (registration, routing of one-token steps,
placeholder K/V, restore) and not a kernel: stock ``generate`` must produce the same tokens with and
without the plug-in.
"""

import pytest
import torch

from leankv_b200.turboquant import hf_attention
from oracle import turboquant as otq


class StandInCache:
    """Duck-typed like PagedKVCache: quantize on update (oracle), dense K/V kept per layer."""

    is_compileable = False
    layer_type = None

    def __init__(self, num_layers, head_dim=128, seed=42):
        from leankv_b200.turboquant.codebook import get_codebook_tensors
        from leankv_b200.turboquant.rotation import generate_rotation_matrix

        self.layers = [None] * num_layers
        cents, bounds = get_codebook_tensors(head_dim, 3, "cpu")
        self.cents, self.bounds = cents.float(), bounds[1:-1].float()
        self.Pi = [(generate_rotation_matrix(head_dim, "cpu", torch.float32, seed + 2 * i),
                    generate_rotation_matrix(head_dim, "cpu", torch.float32, seed + 2 * i + 1))
                   for i in range(num_layers)]
        self.head_dim = head_dim
        self.fused_decode = False
        self.decode_calls = 0
        self.dense_returns = 0
        self._seen = 0

    def update(self, k, v, layer_idx, cache_kwargs=None):
        if layer_idx == 0:
            self._seen += k.shape[2]
        outs = []
        for which, x in enumerate((k, v)):
            packed, norms, _, _ = otq.quantize(x.float(), self.Pi[layer_idx][which], self.bounds, 3)
            deq = otq.dequantize(packed, norms, self.Pi[layer_idx][which], self.cents, 3, self.head_dim).to(x.dtype)
            prev = self.layers[layer_idx][which] if self.layers[layer_idx] is not None else None
            outs.append(deq if prev is None else torch.cat([prev, deq], dim=2))
        self.layers[layer_idx] = outs
        if self.fused_decode and k.shape[2] == 1:
            return k, v
        self.dense_returns += 1
        return outs[0], outs[1]

    def decode_attention(self, layer_idx, q):
        self.decode_calls += 1
        K, V = self.layers[layer_idx]
        rep = q.shape[1] // K.shape[1]
        Kf, Vf = K.float().repeat_interleave(rep, dim=1), V.float().repeat_interleave(rep, dim=1)
        s = torch.einsum("bhd,bhtd->bht", q.float(), Kf) / self.head_dim ** 0.5
        return torch.einsum("bht,bhtd->bhd", torch.softmax(s, dim=-1), Vf).to(q.dtype)

    def get_seq_length(self, layer_idx=0):
        return self._seen

    def get_mask_sizes(self, query_length, layer_idx=0):
        return self._seen + (query_length.shape[0] if hasattr(query_length, "shape") else query_length), 0

    def get_max_cache_shape(self, *a, **k):
        return -1


def _model():
    from transformers import MistralConfig, MistralForCausalLM

    torch.manual_seed(0)
    cfg = MistralConfig(vocab_size=128, hidden_size=256, intermediate_size=256, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=128,
                        tie_word_embeddings=False)
    return MistralForCausalLM(cfg).eval()


def _decode(model, cache, ids, n_new):
    toks, logits = [], []
    with torch.no_grad():
        out = model(ids, past_key_values=cache, use_cache=True)
        for _ in range(n_new):
            logits.append(out.logits[0, -1])
            toks.append(int(out.logits[0, -1].argmax()))
            out = model(torch.tensor([[toks[-1]]]), past_key_values=cache, use_cache=True)
    return toks, torch.stack(logits)


def test_plugin_routes_decode_steps_and_restores():
    model = _model()
    ids = torch.randint(0, 128, (1, 9), generator=torch.Generator().manual_seed(1))
    prev = model.config._attn_implementation

    plain = StandInCache(2)
    want_toks, want_logits = _decode(model, plain, ids, 6)
    assert plain.decode_calls == 0

    fused = StandInCache(2)
    hf_attention.enable_paged_attention(model, fused)
    assert model.config._attn_implementation == hf_attention.ATTN_NAME and fused.fused_decode
    got_toks, got_logits = _decode(model, fused, ids, 6)
    assert fused.decode_calls == 2 * 6                 # every layer of every one-token step
    assert fused.dense_returns == 2                    # only the prompt pass saw dense K/V
    assert got_toks == want_toks
    assert torch.allclose(got_logits, want_logits, atol=2e-4, rtol=1e-4)

    hf_attention.disable_paged_attention(model)
    assert model.config._attn_implementation == prev and not fused.fused_decode
    assert not hasattr(model.model.layers[0].self_attn, "_leankv_paged_cache")
    again_toks, _ = _decode(model, StandInCache(2), ids, 6)
    assert again_toks == want_toks


def test_other_scale_is_refused():
    q = torch.zeros(1, 4, 1, 128)

    class M:
        layer_idx = 0
        _leankv_paged_cache = StandInCache(1)

    M._leankv_paged_cache.fused_decode = True
    with pytest.raises(RuntimeError):
        hf_attention.paged_attention_forward(M(), q, q, q, None, scaling=0.5)


def test_mask_that_hides_cached_positions_is_refused():
    """A padded batch or a sliding window would be ignored by the fused kernel: refuse instead."""
    q = torch.zeros(2, 4, 1, 128)

    class M:
        layer_idx = 0
        _leankv_paged_cache = StandInCache(1)

    M._leankv_paged_cache.fused_decode = True
    hidden = torch.ones(2, 1, 1, 5, dtype=torch.bool)
    hidden[1, 0, 0, 0] = False
    with pytest.raises(RuntimeError, match="attention mask"):
        hf_attention.paged_attention_forward(M(), q, q, q, hidden)
    additive = torch.zeros(2, 1, 1, 5)
    additive[0, 0, 0, 2] = float("-inf")
    with pytest.raises(RuntimeError, match="attention mask"):
        hf_attention.paged_attention_forward(M(), q, q, q, additive)
    assert not hf_attention._masks_something(torch.ones(2, 1, 1, 5, dtype=torch.bool))
    assert not hf_attention._masks_something(torch.zeros(2, 1, 1, 5))


def test_plain_causal_mask_detection():
    """The prefill kernel applies the causal mask only; anything that hides more must be told apart."""
    from leankv_b200.turboquant.hf_attention import _is_plain_causal

    t_q, t_kv = 5, 12
    i = torch.arange(t_q).unsqueeze(1)
    j = torch.arange(t_kv).unsqueeze(0)
    causal = (j <= t_kv - t_q + i).reshape(1, 1, t_q, t_kv)
    assert _is_plain_causal(causal, t_q)
    additive = torch.zeros(1, 1, t_q, t_kv).masked_fill(~causal, float("-inf"))
    assert _is_plain_causal(additive, t_q)
    padded = causal.clone()
    padded[..., 0] = False                                   # a left-padded position
    assert not _is_plain_causal(padded, t_q)
    window = causal & (j > t_kv - t_q + i - 4).reshape(1, 1, t_q, t_kv)
    assert not _is_plain_causal(window, t_q)
