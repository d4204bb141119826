"""Install TEAL activation sparsity on a HuggingFace decoder (API of ``leankv/teal/patching.py``).

Two modes, as in the reference:

* hook mode (``use_triton=False``): a forward pre-hook zeroes sub-threshold inputs of the
  seven projections of every block; the matmul stays dense (correctness only);
* kernel mode (``use_triton=True``; the keyword keeps the reference's name): each
  projection's weight is re-laid out once and its ``forward`` is replaced so that
  single-token decode calls run the sm_100a sparse GEMV. Prefill and batched calls use the
  dense matmul, exactly as ``patching.py:178-180`` does. With ``fuse_mlp=True`` (an
  addition) the MLP's gate/up pair runs as one fused SwiGLU kernel.
"""

from __future__ import annotations

import json
import os
from typing import Optional

import torch
import torch.nn as nn

from .sparse_fns import SparsifyFn, compute_threshold_for_sparsity

try:
    from .kernels.sparse_gemv import (batched_sparse_gemm, prepare_weight_for_sparse_gemv,
                                      sparse_gemv, sparse_swiglu)
    from .. import _native

    # Name kept from the reference: True when the compiled sparse kernels are present.
    HAS_TRITON = os.path.exists(_native.LIB_PATH)
except ImportError:   # pragma: no cover
    HAS_TRITON = False

PROJ_NAMES = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
ATTN_PROJS = {"q_proj", "k_proj", "v_proj", "o_proj"}
MLP_PROJS = {"gate_proj", "up_proj", "down_proj"}


def _get_layers(model):
    """Decoder blocks of a Llama/Mistral-style HF model."""
    inner = getattr(model, "model", None)
    if inner is not None and hasattr(inner, "layers"):
        return inner.layers
    raise ValueError(
        f"Cannot find transformer layers in model of type {type(model)}. "
        "Expected model.model.layers attribute.")


def _get_projection(layer, proj_name: str) -> nn.Linear:
    parent = layer.self_attn if proj_name in ATTN_PROJS else layer.mlp
    return getattr(parent, proj_name)


def _resolve_threshold(model, proj, layer_idx, proj_name, sparsity, thresholds, calibration_data):
    if thresholds is not None:
        return thresholds.get(layer_idx, {}).get(proj_name, 0.0)
    if sparsity is not None and sparsity > 0:
        if calibration_data is not None:
            with torch.no_grad():
                acts = _collect_input_activations(model, proj, calibration_data)
                return compute_threshold_for_sparsity(acts, sparsity)
        # uncalibrated rule of the reference (patching.py:117-118)
        return sparsity * 0.1
    return 0.0


def apply_teal(model, sparsity: Optional[float] = None, thresholds: Optional[dict] = None,
               thresholds_path: Optional[str] = None,
               calibration_data: Optional[list[torch.Tensor]] = None, use_triton: bool = False,
               fuse_mlp: bool = False):
    """Apply TEAL to ``model``; exactly one of sparsity / thresholds / thresholds_path.

    ``thresholds`` maps ``{layer_idx: {proj_name: t}}``; the JSON form has string layer
    keys (``greedy_opt.py:183-199``). Returns ``{(layer_idx, proj_name): SparsifyFn}``.
    """
    if sum(a is not None for a in (sparsity, thresholds, thresholds_path)) != 1:
        raise ValueError("Exactly one of sparsity, thresholds, or thresholds_path must be provided.")
    if use_triton and not HAS_TRITON:
        raise RuntimeError(
            "the CUDA sparse GEMV library is not built (python -m leankv_b200.build); "
            "leankv_b200 does not fall back to hooks silently")
    if thresholds_path is not None:
        with open(thresholds_path, "r") as f:
            thresholds = {int(k): v for k, v in json.load(f).items()}

    sparsifiers, hooks = {}, []
    for layer_idx, layer in enumerate(_get_layers(model)):
        layer_t = {}
        for proj_name in PROJ_NAMES:
            proj = _get_projection(layer, proj_name)
            t = _resolve_threshold(model, proj, layer_idx, proj_name, sparsity, thresholds,
                                   calibration_data)
            layer_t[proj_name] = t
            sf = SparsifyFn(threshold=t, enabled=(t > 0))
            sparsifiers[(layer_idx, proj_name)] = sf
            if use_triton and t > 0:
                _patch_linear_with_triton(proj, t, sparsity or 0.4)
            else:
                hooks.append(proj.register_forward_pre_hook(_make_hook(sf)))
        if use_triton and fuse_mlp and layer_t["gate_proj"] > 0 and layer_t["up_proj"] > 0:
            _patch_mlp_fused(layer.mlp, layer_t["gate_proj"], layer_t["up_proj"])

    if not hasattr(model, "_teal_hooks"):
        model._teal_hooks = []
    model._teal_hooks.extend(hooks)
    model._teal_sparsifiers = sparsifiers
    if use_triton:
        print("[TEAL] Using CUDA sparse GEMV kernels (sm_100a)")
    else:
        print("[TEAL] Using hook-based sparsification (correctness only)")
    return sparsifiers


def _make_hook(sf: SparsifyFn):
    def hook_fn(module, args):
        return (sf(args[0]),) + args[1:]

    return hook_fn


def _is_single_token(x: torch.Tensor) -> bool:
    return x.shape[-2] == 1 and (x.shape[0] if x.dim() == 3 else 1) == 1


def _patch_linear_with_triton(linear: nn.Linear, threshold: float, sparsity: float):
    """Swap ``linear.forward`` for the sparse GEMV on single-token calls (``patching.py:152-183``)."""
    with torch.no_grad():
        linear.weight.data = prepare_weight_for_sparse_gemv(linear.weight.data)
    sparsity_bin = int(sparsity * 10)

    def sparse_forward(x):
        if _is_single_token(x):
            out = sparse_gemv(x.reshape(1, 1, x.shape[-1]), linear.weight, threshold, sparsity_bin)
            out = out.reshape(x.shape[:-1] + (linear.weight.shape[0],))
            return out if linear.bias is None else out + linear.bias
        return torch.nn.functional.linear(x, linear.weight, linear.bias)

    linear.forward = sparse_forward
    linear._teal_patched = True


# Alias under the name that says what it does here.
_patch_linear_with_cuda = _patch_linear_with_triton


def _patch_mlp_fused(mlp, t_gate: float, t_up: float):
    """Run gate_proj/up_proj/act as one fused kernel on single-token calls (no reference counterpart)."""
    gate, up, down = mlp.gate_proj, mlp.up_proj, mlp.down_proj
    if gate.bias is not None or up.bias is not None:
        return
    dense_forward = mlp.forward

    def fused_forward(x):
        if _is_single_token(x) and x.dtype == torch.float16:
            h = sparse_swiglu(x.reshape(1, 1, x.shape[-1]), gate.weight, up.weight, t_gate, t_up)
            return down(h.reshape(x.shape[:-1] + (gate.weight.shape[0],)))
        return dense_forward(x)

    mlp.forward = fused_forward
    mlp._teal_fused = True


def remove_teal(model):
    """Remove the TEAL hooks (patched forwards stay, as in ``patching.py:186-193``)."""
    for handle in getattr(model, "_teal_hooks", []):
        handle.remove()
    if hasattr(model, "_teal_hooks"):
        model._teal_hooks.clear()
    if hasattr(model, "_teal_sparsifiers"):
        del model._teal_sparsifiers


def get_sparsity_report(model) -> dict:
    """Last observed sparsity per ``(layer_idx, proj_name)`` (hook mode only)."""
    return {key: sf.last_sparsity for key, sf in getattr(model, "_teal_sparsifiers", {}).items()}


def print_sparsity_report(model):
    report = get_sparsity_report(model)
    if not report:
        print("No TEAL sparsifiers found on model.")
        return
    by_layer: dict[int, dict[str, float]] = {}
    for (layer_idx, proj_name), s in report.items():
        by_layer.setdefault(layer_idx, {})[proj_name] = s
    print(f"{'Layer':<8}" + "".join(f"{p:<12}" for p in PROJ_NAMES) + f"{'Avg':<8}")
    print("-" * (8 + 12 * len(PROJ_NAMES) + 8))
    for layer_idx in sorted(by_layer):
        vals = [by_layer[layer_idx].get(p, 0.0) for p in PROJ_NAMES]
        print(f"{layer_idx:<8}" + "".join(f"{v:>10.1%}  " for v in vals)
              + f"{sum(vals) / len(vals):>6.1%}")


def _collect_input_activations(model, target_module, data_samples):
    """Inputs seen by ``target_module`` over (at most 10 of) ``data_samples``."""
    seen = []
    handle = target_module.register_forward_pre_hook(
        lambda module, args: seen.append(args[0].detach().cpu()))
    try:
        with torch.no_grad():
            for sample in data_samples[:10]:
                model(sample.to(model.device))
    finally:
        handle.remove()
    return torch.cat(seen, dim=0)
