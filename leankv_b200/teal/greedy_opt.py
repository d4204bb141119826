"""Threshold files in the reference's on-disk format.

The reference's calibration (``scripts/calibrate.py:81-82`` via ``leankv/teal/greedy_opt.py:183-199``)
writes ``thresholds_s{NN}.json``: ``{"<layer>": {"q_proj": t, ..., "down_proj": t}, ...}`` with the
layer index as a *string* key and 0.0 meaning "leave this projection dense". Only the file round-trip
lives here, so that thresholds calibrated by a real reference run drop into ``apply_teal`` or
``DecodeEngine.set_thresholds``; the greedy allocator itself is outside the decode hot path.
"""

from __future__ import annotations

import json
import os


def save_thresholds(thresholds: dict, path: str) -> None:
    """``{layer:int -> {proj:str -> float}}`` to JSON (layer keys become strings)."""
    folder = os.path.dirname(path)
    if folder:
        os.makedirs(folder, exist_ok=True)
    out = {str(int(layer)): {str(p): float(t) for p, t in projs.items()} for layer, projs in thresholds.items()}
    with open(path, "w") as f:
        json.dump(out, f, indent=2)
    print(f"[TEAL] Saved thresholds to {path}")


def load_thresholds(path: str) -> dict:
    """Inverse of ``save_thresholds``: layer keys back to ``int``."""
    with open(path) as f:
        raw = json.load(f)
    return {int(layer): dict(projs) for layer, projs in raw.items()}
