"""One-call set-up of TEAL + TurboQuant on a HuggingFace model (API of ``leankv/combined.py``).

    model, tokenizer = load_model("mistralai/Mistral-7B-v0.3")
    model, cache = optimize_model(model, teal_thresholds_path="thresholds.json", turboquant_bits=3)
    output = model.generate(**inputs, past_key_values=cache)
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .teal.patching import apply_teal, remove_teal
from .turboquant.cache import TurboQuantCache
from .turboquant.paged_cache import PagedKVCache

HAS_PAGED = True   # the paged cache here has no optional dependency


@dataclass
class TEALConfig:
    sparsity: Optional[float] = None
    thresholds_path: Optional[str] = None


@dataclass
class TurboQuantConfig:
    bits: int = 3
    head_dim: int = 128
    num_layers: int = 32


def load_model(model_name: str, dtype=torch.float16, device_map="cuda"):
    """Load a HuggingFace causal LM and its tokenizer (``combined.py:45-54``)."""
    from transformers import AutoModelForCausalLM, AutoTokenizer

    print(f"Loading {model_name}...")
    model = AutoModelForCausalLM.from_pretrained(model_name, torch_dtype=dtype, device_map=device_map)
    tokenizer = AutoTokenizer.from_pretrained(model_name)
    tokenizer.pad_token = tokenizer.pad_token or tokenizer.eos_token
    print(f"Model loaded. Device: {model.device}")
    return model, tokenizer


def optimize_model(model, teal_sparsity: Optional[float] = None,
                   teal_thresholds_path: Optional[str] = None,
                   turboquant_bits: Optional[int] = None, use_paged_cache: bool = False,
                   page_size: int = 16, max_pages: int = 2048, use_triton: bool = False,
                   fused_attention: bool = False, fused_prefill: bool = False):
    """Apply TEAL and/or build a TurboQuant cache; returns ``(model, cache)``.

    ``use_triton`` (an addition: the reference's ``optimize_model`` cannot select its kernel
    path, ``combined.py:83-87``) forwards to ``apply_teal`` and selects the CUDA sparse GEMV.
    ``fused_attention`` (an addition, paged cache only) registers the HF attention function of
    ``turboquant/hf_attention.py`` so that decode steps of ``model.generate`` run on the packed pages;
    with ``fused_prefill`` prompt passes do too (causal masks only).
    """
    if teal_sparsity is not None or teal_thresholds_path is not None:
        apply_teal(model, sparsity=teal_sparsity, thresholds_path=teal_thresholds_path,
                   use_triton=use_triton)
        label = teal_thresholds_path or f"{teal_sparsity:.0%}"
        print(f"[LeanKV] TEAL enabled (sparsity={label})")

    cfg = model.config
    head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
    num_layers = cfg.num_hidden_layers
    num_q_heads = cfg.num_attention_heads
    num_kv_heads = getattr(cfg, "num_key_value_heads", num_q_heads)

    cache = None
    if use_paged_cache:
        cache = PagedKVCache(num_layers=num_layers, num_kv_heads=num_kv_heads, num_q_heads=num_q_heads,
                             head_dim=head_dim, page_size=page_size, max_pages=max_pages,
                             device=model.device, dtype=torch.float16,
                             bits=turboquant_bits if turboquant_bits is not None else 3)
        print(f"[LeanKV] PagedKVCache enabled (pages={max_pages}, page_size={page_size}, "
              f"pool={cache.get_total_pool_mb():.0f} MB)")
        if fused_attention:
            from .turboquant.hf_attention import enable_paged_attention

            enable_paged_attention(model, cache, fused_prefill=fused_prefill)
            print("[LeanKV] decode attention runs on the packed pages")
    elif turboquant_bits is not None:
        cache = TurboQuantCache(bits=turboquant_bits, head_dim=head_dim, num_layers=num_layers,
                                device=model.device, dtype=torch.float16)
        print(f"[LeanKV] TurboQuant enabled (bits={turboquant_bits}, head_dim={head_dim})")
    return model, cache


def reset_optimizations(model):
    """Remove the TEAL hooks (and the paged attention function, if installed) from ``model``."""
    from .turboquant.hf_attention import disable_paged_attention

    remove_teal(model)
    disable_paged_attention(model)
    print("[LeanKV] All optimizations removed.")
