"""HuggingFace attention-interface plug-in for the paged TurboQuant cache.

HF attention layers call ``past_key_values.update(k, v, layer)`` and hand whatever comes back to
the function registered under ``config._attn_implementation``. The reference cache honours that
contract by de-quantizing the whole history on every call (``leankv/turboquant/cache.py:102-127,
169-189``). With this plug-in a stock ``model.generate(..., past_key_values=cache)`` keeps working
but decode steps (one query token) never see dense K/V: ``update`` only appends to the packed
pages and the registered function answers from ``cache.decode_attention`` (the fused kernel).
Prompt passes (more than one query token) take the dense route through SDPA unless
``fused_prefill=True``: then they too only append, and their causal attention runs on the packed pages
(``cache.prefill_attention``).

    cache = PagedKVCache(num_layers=..., num_kv_heads=..., num_q_heads=..., device="cuda")
    enable_paged_attention(model, cache)
    model.generate(ids, past_key_values=cache, max_new_tokens=64)
    disable_paged_attention(model)
"""

from __future__ import annotations

import torch

ATTN_NAME = "leankv_paged"


def _sdpa(module, query, key, value, attention_mask, **kwargs):
    from transformers.integrations.sdpa_attention import sdpa_attention_forward

    return sdpa_attention_forward(module, query, key, value, attention_mask, **kwargs)


def paged_attention_forward(module, query, key, value, attention_mask, dropout: float = 0.0,
                            scaling=None, **kwargs):
    """Signature of an HF attention function. ``query`` is ``[B, Hq, T_q, D]``; returns
    ``([B, T_q, Hq, D], None)``."""
    cache = getattr(module, "_leankv_paged_cache", None)
    if cache is not None and query.shape[2] == 1 and getattr(cache, "fused_decode", False):
        d = query.shape[-1]
        if scaling is not None and abs(float(scaling) * d ** 0.5 - 1.0) > 1e-6:
            raise RuntimeError("the paged decode kernel uses scale = head_dim ** -0.5")
        if attention_mask is not None and getattr(module, "layer_idx", 0) == 0 and _masks_something(attention_mask):
            # The fused kernel attends to every cached token of a sequence. A mask that hides cached
            # positions (left-padded prompts of unequal length in one batch, a sliding window) would be
            # ignored silently, so it is refused; checked once per step, on the first layer.
            raise RuntimeError(
                "the paged decode kernel cannot apply an attention mask that hides cached positions "
                "(padded batches of unequal prompt length, sliding-window attention): run such inputs "
                "with disable_paged_attention(model), which takes the dense SDPA route")
        out = cache.decode_attention(module.layer_idx, query[:, :, 0, :])        # [B, Hq, D]
        return out.unsqueeze(1), None
    if cache is not None and query.shape[2] > 1 and getattr(cache, "fused_decode", False) and \
            getattr(cache, "fused_prefill", False):
        d = query.shape[-1]
        if scaling is not None and abs(float(scaling) * d ** 0.5 - 1.0) > 1e-6:
            raise RuntimeError("the paged prefill kernel uses scale = head_dim ** -0.5")
        if attention_mask is not None and getattr(module, "layer_idx", 0) == 0 and \
                not _is_plain_causal(attention_mask, query.shape[2]):
            raise RuntimeError(
                "the paged prefill kernel applies the causal mask only: a mask that hides more (padded prompts "
                "of unequal length, sliding-window attention) needs enable_paged_attention(model, cache, "
                "fused_prefill=False), which sends prompt passes through the dense route")
        out = cache.prefill_attention(module.layer_idx, query)                   # [B, Hq, T, D]
        return out.transpose(1, 2), None
    return _sdpa(module, query, key, value, attention_mask, dropout=dropout, scaling=scaling, **kwargs)


def _is_plain_causal(mask: torch.Tensor, t_q: int) -> bool:
    """True if ``mask`` ([B, 1, T_q, T_kv], boolean with False = hidden or additive with negative = hidden)
    shows query i exactly the keys 0 .. T_kv - T_q + i."""
    vis = mask if mask.dtype == torch.bool else mask >= 0
    t_kv = vis.shape[-1]
    i = torch.arange(t_q, device=vis.device).unsqueeze(1)
    j = torch.arange(t_kv, device=vis.device).unsqueeze(0)
    return bool((vis == (j <= t_kv - t_q + i)).all())


def _masks_something(mask: torch.Tensor) -> bool:
    """True if a boolean (False = hidden) or additive (negative = hidden) mask hides any position."""
    if mask.dtype == torch.bool:
        return not bool(mask.all())
    return bool((mask < 0).any())


def register() -> None:
    """Register the attention function (and an SDPA-style mask builder) under ``ATTN_NAME``."""
    from transformers import AttentionInterface
    from transformers.masking_utils import AttentionMaskInterface, sdpa_mask

    AttentionInterface.register(ATTN_NAME, paged_attention_forward)
    AttentionMaskInterface.register(ATTN_NAME, sdpa_mask)


def _attention_modules(model):
    inner = getattr(model, "model", model)
    return [layer.self_attn for layer in inner.layers]


def enable_paged_attention(model, cache, fused_prefill: bool = False) -> None:
    """Route ``model``'s decode-step attention through ``cache.decode_attention`` and, with
    ``fused_prefill``, its prompt passes through ``cache.prefill_attention`` (causal masks only)."""
    register()
    for attn in _attention_modules(model):
        attn._leankv_paged_cache = cache
    model._leankv_prev_attn = model.config._attn_implementation
    model.config._attn_implementation = ATTN_NAME
    cache.fused_decode = True
    cache.fused_prefill = bool(fused_prefill)


def disable_paged_attention(model) -> None:
    for attn in _attention_modules(model):
        cache = getattr(attn, "_leankv_paged_cache", None)
        if cache is not None:
            cache.fused_decode = False
            cache.fused_prefill = False
            del attn._leankv_paged_cache
    prev = getattr(model, "_leankv_prev_attn", None)
    if prev is not None:
        model.config._attn_implementation = prev
        del model._leankv_prev_attn
